// Flash attention forward for sm_100a (non-causal, head_dim 64 or 128, bf16 in / bf16 out, fp32
// softmax state), token-major tensors [B, L, H, Dh] so that the QKV projection's output and the
// output projection's input need no transposes.
//
// One CTA per (128-query tile, head, batch), two CTAs resident per SM so that one CTA's softmax
// overlaps the other's tensor-core work:
//   warp 0     TMA loads: Q once, then one K tile and one V tile (128 keys) per iteration
//   warp 1     tcgen05.mma issue:  S = Q K^T  (smem x smem -> TMEM, fp32)
//                                  O += P V   (P read from TMEM as packed bf16, V from smem as an
//                                              MN-major operand, accumulator O in TMEM)
//   warps 2-9  softmax: two threads per query row (warps w and w + 4 share 32 rows and take 64 of
//              the tile's 128 keys each) read S from TMEM, keep the running max / partial sum in
//              registers, write P back over S in TMEM as packed bf16, rescale their half of O in
//              TMEM only when the running max moved by more than 2^8 (lazy rescale), and write
//              O / l and the log-sum-exp at the end.
// Key masks (MASK variant): an additive per-(batch, key) bias in log2 units, 0 for a visible key
// and -1e30 for a masked or padded one, is added to the scaled scores before the running maximum
// is taken; a masked probability is then exactly zero and a fully masked tile is wiped by the next
// rescale. This is the text-padding mask of cached-embedding batches ([B, 1, 1, T],
// crates/training/src/flux/data_loader.rs:254-264, masked attention path of
// crates/training/src/flux/runtime.rs:943-961) and the 77-key cross-attention of the SDXL blocks
// (crates/training/src/sdxl/runtime.rs:146-246), whose single key tile is mostly padding.
// The reference reaches attention through an external flame-core SDPA or a chunked online-softmax
// composition of bmm + elementwise ops (crates/training/src/sdxl/runtime.rs:2814-3025,
// crates/training/src/flux/runtime.rs:707-745); the softmax recurrence is the same.
#include <cstdlib>

#include "ptx.cuh"
#include "tma_host.h"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

struct FaParams {
  int B, H, Lq, Lk;
  float scale_log2;  // softmax scale * log2(e)
  bf16* out;         // [B, Lq, H, DH]; consecutive tokens are out_ld elements apart
  long long out_ld;  // >= H * DH (larger when the output is a column block of a wider matrix)
  float* lse;        // [B, H, Lq] natural-log log-sum-exp (may be null)
  int* err;
  const float* kbias;  // MASK variant: [B, Lkb] additive key bias in log2 units (-1e30 = masked),
                       // followed by one int per (batch, 128-key tile): 1 = the tile has a non-zero bias
  int Lkb;             // row length of kbias: ceil(Lk / 128) * 128
};

constexpr int BQ = 128, BKV = 128;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

ERI_DEBUG_BOUNDS_DEFINE(fa)

template <int DH, int POLY, bool MASK>
__global__ void __launch_bounds__(320, 2)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const FaParams p) {
  constexpr int CHUNKS = DH / 64;
  constexpr int TILE_BYTES = 128 * 128 * CHUNKS;  // 128 rows x DH bf16
  constexpr int CHUNK_BYTES = 128 * 128;          // 128 rows x 64 bf16
  constexpr int TMEM_COLS = 256;                  // S/P: 128 columns, O: DH columns
  constexpr uint32_t S_COL = 0, O_COL = 128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;
  uint8_t* sV = sK + TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + TILE_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* o_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  float* xchg = reinterpret_cast<float*>(bars + 16);  // [4][128] row max / row sum exchange

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BQ, h = blockIdx.y, b = blockIdx.z;
  const int nkv = (p.Lk + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 8);
    mbar_init(o_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(q_full, TILE_BYTES);
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c)
        tma_load_3d(sQ + c * CHUNK_BYTES, &tmQ, q_full, h * DH + c * 64, q0, b);
      for (int j = 0; j < nkv; ++j) {
        const uint32_t par = (uint32_t)(j & 1);
        if (!mbar_wait(k_empty, par ^ 1)) { atomicExch(p.err, 11); break; }
        mbar_expect_tx(k_full, TILE_BYTES);
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_3d(sK + c * CHUNK_BYTES, &tmK, k_full, h * DH + c * 64, j * BKV, b);
        if (!mbar_wait(v_empty, par ^ 1)) { atomicExch(p.err, 12); break; }
        mbar_expect_tx(v_full, TILE_BYTES);
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_3d(sV + c * CHUNK_BYTES, &tmV, v_full, h * DH + c * 64, j * BKV, b);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc_s = umma_idesc_bf16(BQ, BKV, 0, 0);
      const uint32_t idesc_o = umma_idesc_bf16(BQ, DH, 0, 1);  // B (V) is MN-major
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(p.err, 13);
      for (int j = 0; j < nkv && ok; ++j) {
        const uint32_t par = (uint32_t)(j & 1);
        if (!mbar_wait(k_full, par)) { atomicExch(p.err, 14); break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          const uint64_t dq = umma_desc_kmajor(aQ + c * CHUNK_BYTES, 128);
          const uint64_t dk = umma_desc_kmajor(aK + c * CHUNK_BYTES, 128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(tmem_base + S_COL, dq + kk * 2, dk + kk * 2, idesc_s, (c | kk) != 0);
        }
        umma_commit(s_full);
        umma_commit(k_empty);
        if (!mbar_wait(p_full, par)) { atomicExch(p.err, 15); break; }
        if (!mbar_wait(v_full, par)) { atomicExch(p.err, 16); break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint64_t dv = umma_desc_mn128(aV + kk * 2048, CHUNK_BYTES);
          umma_bf16_ts(tmem_base + O_COL, tmem_base + S_COL + (kk >> 2) * 64 + (kk & 3) * 8, dv, idesc_o,
                       (j | kk) != 0);
        }
        umma_commit(o_done);
        umma_commit(v_empty);
      }
    }
  } else {
    // Eight softmax warps: warps w and w + 4 own the same 32 query rows (TMEM lanes) and split
    // the 128 key columns of every tile in halves, so each scheduler has two softmax warps of this
    // CTA to interleave (four with the second resident CTA). The row maximum and, at the end, the
    // row sum are exchanged through shared memory.
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r_in = qd * 32 + lane;
    const int row = q0 + r_in;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    const uint32_t s_col = S_COL + half * 64;        // this warp's 64 score columns
    float* s_mx = xchg;                               // [2][128]
    float* s_l = xchg + 256;                          // [2][128]
    float m_used = -INFINITY, l = 0.f;                // l: partial row sum over this warp's columns
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      const uint32_t par = (uint32_t)(j & 1);
      if (ok && !mbar_wait(s_full, par)) {
        if (lane == 0) atomicExch(p.err, 17);
        ok = false;
      }
      if (!ok) {
        // a warp that gave up still meets its partners at the block barrier and on p_full, so that
        // no other warp is left waiting without a limit
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (lane == 0) mbar_arrive(p_full);
        continue;
      }
      tc_fence_after();
      const int kv_left = p.Lk - j * BKV - half * 64;  // valid key columns in this warp's half
      // MASK: a tile without any biased key runs the unmasked paths (the flags sit behind the rows)
      const bool use_bias =
          MASK && reinterpret_cast<const int*>(p.kbias + (size_t)p.B * p.Lkb)[b * (p.Lkb / BKV) + j] != 0;
      const bool full_half = !use_bias && kv_left >= 64;
      // MASK: this half's 64 bias values (every lane reads the same addresses: one transaction each)
      const float4* kb4 = MASK ? reinterpret_cast<const float4*>(p.kbias + (size_t)b * p.Lkb + j * BKV + half * 64)
                               : nullptr;
      float mx = -INFINITY;
      if (use_bias) {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(lane_addr + s_col + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i4 = 0; i4 < 8; ++i4) {
            const float4 kb = __ldg(kb4 + c * 8 + i4);
            mx = fmaxf(mx, fmaf(__uint_as_float(r[4 * i4]), p.scale_log2, kb.x));
            mx = fmaxf(mx, fmaf(__uint_as_float(r[4 * i4 + 1]), p.scale_log2, kb.y));
            mx = fmaxf(mx, fmaf(__uint_as_float(r[4 * i4 + 2]), p.scale_log2, kb.z));
            mx = fmaxf(mx, fmaf(__uint_as_float(r[4 * i4 + 3]), p.scale_log2, kb.w));
          }
        }
      } else if (full_half) {
        uint32_t r[32], r2[32];
        tmem_ld32(lane_addr + s_col, r);
        tmem_ld32(lane_addr + s_col + 32, r2);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          mx = fmax3(mx, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
          mx = fmax3(mx, __uint_as_float(r2[i]), __uint_as_float(r2[i + 1]));
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(lane_addr + s_col + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < kv_left) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
      }
      s_mx[half * 128 + r_in] = mx;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      mx = fmaxf(mx, s_mx[(half ^ 1) * 128 + r_in]);
      const float m_new = use_bias ? mx : mx * p.scale_log2;   // biased tile: the bias went in before the maximum
      if (j == 0) {
        m_used = m_new;
      } else {
        const bool need = (m_new - m_used) > kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // s_full of this tile was committed after PV of the previous tile, so O is complete.
          // Both warps of a row pair take the same decision; each rescales its half of O.
          const float m_t = need ? m_new : m_used;
          const float alpha = exp2f(m_used - m_t);
#pragma unroll 1
          for (int c = 0; c < DH / 64; ++c) {
            uint32_t r[32];
            const uint32_t oc = O_COL + half * (DH / 2) + c * 32;
            tmem_ld32(lane_addr + oc, r);
            tmem_ld_wait();
            uint32_t a0[16], a1[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              a0[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              a1[i] = __float_as_uint(__uint_as_float(r[16 + i]) * alpha);
            }
            tmem_st16(lane_addr + oc, a0);
            tmem_st16(lane_addr + oc + 16, a1);
          }
          tmem_st_wait();
          l *= alpha;
          m_used = m_t;
        }
      }
      // s_mx needs no second barrier: the next tile's s_full cannot complete before all eight warps
      // have arrived on p_full, i.e. after both warps of a pair have read the other's maximum
      float lsum = 0.f;
      if (full_half) {
        // Hot path: packed fp32 pairs (one fma / add per two scores), 2^x split between the
        // special-function unit and a polynomial on the FMA pipe (POLY of every 16 pairs), the
        // row sum taken from the unrounded fp32 values.
        const f32x2 sc2 = f2_pack(p.scale_log2, p.scale_log2);
        const f32x2 nm2 = f2_pack(-m_used, -m_used);
        f32x2 acc2 = f2_pack(0.f, 0.f);
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(lane_addr + s_col + c * 32, r);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            f32x2 v = f2_fma(f2_pack_bits(r[2 * i], r[2 * i + 1]), sc2, nm2);
            if (i < 16 - POLY) {
              float lo, hi;
              f2_unpack(v, lo, hi);
              v = f2_pack(ex2_mufu(lo), ex2_mufu(hi));
            } else {
              v = MASK ? ex2_poly2_z(v) : ex2_poly2(v);
            }
            acc2 = f2_add(acc2, v);
            pk[i] = f2_to_bf162(v);
          }
          // packed P of this half starts at the half's own first column
          tmem_st16(lane_addr + s_col + c * 16, pk);
        }
        float a_lo, a_hi;
        f2_unpack(acc2, a_lo, a_hi);
        lsum = a_lo + a_hi;
      } else if (use_bias) {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(lane_addr + s_col + c * 32, r);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int i4 = 0; i4 < 8; ++i4) {
            const float4 kb = __ldg(kb4 + c * 8 + i4);
            // a masked score is about -1e30: its 2^x is exactly zero whatever the running maximum
            const float p0 = ex2_mufu(fmaf(__uint_as_float(r[4 * i4]), p.scale_log2, kb.x) - m_used);
            const float p1 = ex2_mufu(fmaf(__uint_as_float(r[4 * i4 + 1]), p.scale_log2, kb.y) - m_used);
            const float p2 = ex2_mufu(fmaf(__uint_as_float(r[4 * i4 + 2]), p.scale_log2, kb.z) - m_used);
            const float p3 = ex2_mufu(fmaf(__uint_as_float(r[4 * i4 + 3]), p.scale_log2, kb.w) - m_used);
            lsum += (p0 + p1) + (p2 + p3);
            pk[2 * i4] = pack_bf162(p0, p1);
            pk[2 * i4 + 1] = pack_bf162(p2, p3);
          }
          tmem_st16(lane_addr + s_col + c * 16, pk);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(lane_addr + s_col + c * 32, r);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float p0 = exp2f(fmaf(__uint_as_float(r[2 * i]), p.scale_log2, -m_used));
            float p1 = exp2f(fmaf(__uint_as_float(r[2 * i + 1]), p.scale_log2, -m_used));
            if (c * 32 + 2 * i >= kv_left) p0 = 0.f;
            if (c * 32 + 2 * i + 1 >= kv_left) p1 = 0.f;
            lsum += p0 + p1;
            pk[i] = pack_bf162(p0, p1);
          }
          tmem_st16(lane_addr + s_col + c * 16, pk);
        }
      }
      l += lsum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok) {
      if (!mbar_wait(o_done, (uint32_t)((nkv - 1) & 1))) {
        if (lane == 0) atomicExch(p.err, 18);
        ok = false;
      }
    }
    // total row sum = the two halves' partial sums (exchanged even after an error so that the
    // barrier is always reached by all eight warps)
    s_l[half * 128 + r_in] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    l += s_l[(half ^ 1) * 128 + r_in];
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      bf16* orow = p.out + ((size_t)b * p.Lq + row) * p.out_ld + h * DH + half * (DH / 2);
#pragma unroll 1
      for (int c = 0; c < DH / 64; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_addr + O_COL + half * (DH / 2) + c * 32, r);
        tmem_ld_wait();
        if (row < p.Lq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]) * inv_l;
            if (ERI_DBG_RANGE(p.out, (((size_t)p.B * p.Lq - 1) * p.out_ld + (size_t)p.H * DH) * 2, orow + c * 32 + g * 8, 16, 51))
              *reinterpret_cast<bf16x8*>(orow + c * 32 + g * 8) = pack8(v);
          }
        }
      }
      if (half == 0 && p.lse && row < p.Lq)
        p.lse[((size_t)b * p.H + h) * p.Lq + row] = (m_used + log2f(l)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

int* g_fa_err[64] = {nullptr};   // one error word per device

template <int DH, int POLY, bool MASK>
int launch_fwd(const CUtensorMap& q, const CUtensorMap& k, const CUtensorMap& v, const FaParams& p,
               int dev, cudaStream_t st) {
  constexpr int SMEM = 3 * 128 * 128 * (DH / 64) + 1024 + 128 + 2048;
  static bool configured[64] = {};
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fa_fwd_kernel<DH, POLY, MASK>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    configured[dev] = true;
  }
  dim3 grid((p.Lq + BQ - 1) / BQ, p.H, p.B);
  fa_fwd_kernel<DH, POLY, MASK><<<grid, 320, SMEM, st>>>(q, k, v, p);
  return (int)cudaGetLastError();
}

// Pairs (of every 16) whose 2^x runs on the FMA pipe instead of the special-function unit.
// ERI_B200_FA_POLY = 0, 4 or 8 selects the variant (read once).
int poly_pairs() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("ERI_B200_FA_POLY");
    v = e ? atoi(e) : 4;
    if (v != 0 && v != 4 && v != 8) v = 4;
  }
  return v;
}

int make_qkv_map(CUtensorMap* m, const void* ptr, int B, int L, int H, int DH) {
  uint64_t dims[3] = {(uint64_t)H * DH, (uint64_t)L, (uint64_t)B};
  uint64_t strides[2] = {(uint64_t)H * DH * 2, (uint64_t)L * H * DH * 2};
  uint32_t box[3] = {64, 128, 1};
  return make_tensor_map(m, ptr, 3, dims, strides, box, 128);
}

int fwd_entry(const void* q, const void* k, const void* v, void* out, float* lse, const float* kbias,
              int B, int H, int Lq, int Lk, int DH, float scale, void* stream, long long out_ld = 0) {
  if (DH != 64 && DH != 128) return -1;
  if (out_ld == 0) out_ld = (long long)H * DH;
  // rows are written as 16-byte words
  if (out_ld < (long long)H * DH || out_ld % 8 || (((uintptr_t)out) & 15)) return -7;
  // Fewer than 128 keys (one mostly empty tile) need the key bias to blank the padding; queries are
  // tiled by 128 rows and a short last tile is simply not written back.
  if (Lq < 1 || Lk < 1 || (Lk < 128 && !kbias)) return -2;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -3;
  if (!g_fa_err[dev]) {
    if (cudaMalloc(&g_fa_err[dev], sizeof(int)) != cudaSuccess) return -3;
    cudaMemset(g_fa_err[dev], 0, sizeof(int));
  }
  CUtensorMap tq, tk, tv;
  if (make_qkv_map(&tq, q, B, Lq, H, DH) || make_qkv_map(&tk, k, B, Lk, H, DH) ||
      make_qkv_map(&tv, v, B, Lk, H, DH))
    return -4;
  FaParams p;
  p.B = B; p.H = H; p.Lq = Lq; p.Lk = Lk;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.out = (bf16*)out; p.out_ld = out_ld; p.lse = lse; p.err = g_fa_err[dev];
  p.kbias = kbias; p.Lkb = (Lk + BKV - 1) / BKV * BKV;
  cudaStream_t st = (cudaStream_t)stream;
  if (kbias) {
    if (((uintptr_t)kbias) & 15) return -6;
    // the unbiased tiles of a masked call run the packed path, the biased tiles the scalar one; all
    // exponentials on the special-function unit (the zero-flushing polynomial measured 272 against 269 us)
    return DH == 128 ? launch_fwd<128, 0, true>(tq, tk, tv, p, dev, st)
                     : launch_fwd<64, 0, true>(tq, tk, tv, p, dev, st);
  }
  const int poly = poly_pairs();
  if (DH == 128) {
    if (poly == 0) return launch_fwd<128, 0, false>(tq, tk, tv, p, dev, st);
    if (poly == 8) return launch_fwd<128, 8, false>(tq, tk, tv, p, dev, st);
    return launch_fwd<128, 4, false>(tq, tk, tv, p, dev, st);
  }
  if (poly == 0) return launch_fwd<64, 0, false>(tq, tk, tv, p, dev, st);
  if (poly == 8) return launch_fwd<64, 8, false>(tq, tk, tv, p, dev, st);
  return launch_fwd<64, 4, false>(tq, tk, tv, p, dev, st);
}

}  // namespace

extern "C" {

int eri_fa_check_error() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || !g_fa_err[dev]) return 0;
  int h = 0;
  cudaMemcpy(&h, g_fa_err[dev], sizeof(int), cudaMemcpyDeviceToHost);
  if (h) cudaMemset(g_fa_err[dev], 0, sizeof(int));
  return h;
}

// q [B, Lq, H, DH], k/v [B, Lk, H, DH], out [B, Lq, H, DH] (all contiguous bf16), lse [B, H, Lq].
int eri_flash_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B,
                       int H, int Lq, int Lk, int DH, float scale, void* stream) {
  return fwd_entry(q, k, v, out, lse, nullptr, B, H, Lq, Lk, DH, scale, stream);
}

// The same with the output's token stride given: out_ld elements between consecutive tokens (a
// multiple of 8, at least H * DH), batches Lq * out_ld apart. Lets the attention write a column block
// of a wider matrix (the attention half of a single-stream block's second linear's input) in place.
int eri_flash_attn_fwd_ld(const void* q, const void* k, const void* v, void* out, float* lse, int B,
                          int H, int Lq, int Lk, int DH, float scale, long long out_ld, void* stream) {
  return fwd_entry(q, k, v, out, lse, nullptr, B, H, Lq, Lk, DH, scale, stream, out_ld);
}

// The same with an additive key bias: kbias [B, ceil(Lk/128)*128] fp32 in log2 units (the caller
// multiplies a natural-log bias by log2(e)); -1e30 marks a masked key and every column at or beyond
// Lk. Any Lk >= 1 is accepted.
int eri_flash_attn_fwd_masked(const void* q, const void* k, const void* v, void* out, float* lse,
                              const float* kbias, int B, int H, int Lq, int Lk, int DH, float scale,
                              void* stream) {
  if (!kbias) return -6;
  return fwd_entry(q, k, v, out, lse, kbias, B, H, Lq, Lk, DH, scale, stream);
}

}  // extern "C"

ERI_DEBUG_BOUNDS_EXPORT(fa)
