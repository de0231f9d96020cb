// Flash attention forward on CTA pairs (cta_group::2), head_dim 128, no mask.
//
// The one-CTA kernel (flash_attn.cu) feeds S = Q K^T with BOTH operands from shared memory: 64 KB
// per 128 x 128 x 128 product in 512 tensor cycles is the full 128 B/clk of an SM's shared memory,
// so the tensor pipe runs without any slack and measures 58 % active. Here two CTAs on one TPC
// process 256 query rows together: each keeps its own 128 rows of Q (and of S, P, O in its own
// tensor memory) but stages only HALF of every K tile (64 keys) and half of every V tile (64 of the
// 128 head columns); tcgen05.mma.cta_group::2 reads the two halves from both CTAs. Shared-memory
// traffic per product drops to 48 KB (Q K^T) and 16 KB (P V, P from tensor memory), and each K / V
// tile crosses L2 -> shared memory once per 256 queries instead of once per 128.
//
// Roles per CTA: warp 0 TMA producer (both CTAs; completion bytes of both land on the LEADER's
// barriers), warp 1 MMA issuer (leader only; every commit goes to the barriers of both CTAs),
// warps 2-9 softmax exactly as in the one-CTA kernel (two threads per query row, lazy rescale,
// packed fp32 pairs, part of the exponentials as a polynomial on the FMA pipe). K and V are
// double-buffered. No multicast load is used: every CTA loads its own halves.
//
// The reference reaches attention through an external SDPA or a chunked online-softmax
// composition of bmm + elementwise ops (crates/training/src/sdxl/runtime.rs:2814-3025,
// crates/training/src/flux/runtime.rs:707-745); the softmax recurrence is the same.
#include <cstdlib>

#include "ptx.cuh"
#include "tma_host.h"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

struct Fa2Params {
  int B, H, Lq, Lk;
  float scale_log2;
  bf16* out;     // [B, Lq, H, 128]
  float* lse;    // [B, H, Lq]
  int* err;
};

constexpr int DH = 128, BQ = 128, BKV = 128, NST = 2;
constexpr int Q_BYTES = BQ * DH * 2;          // this CTA's 128 query rows: two 64-column chunks
constexpr int KH_BYTES = (BKV / 2) * DH * 2;  // half a K tile: 64 keys x 128, two 64-column chunks
constexpr int VH_BYTES = BKV * (DH / 2) * 2;  // half a V tile: 128 keys x 64 head columns
constexpr int Q_CHUNK = BQ * 128, K_CHUNK = (BKV / 2) * 128;
constexpr float kRescaleThreshold = 8.0f;
constexpr uint32_t S_COL = 0, O_COL = 128, TMEM_COLS = 256;

template <int POLY>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(320, 2)
fa_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const Fa2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Q_BYTES;              // NST stages
  uint8_t* sV = sK + NST * KH_BYTES;       // NST stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NST * VH_BYTES);
  uint64_t* q_full = bars + 0;             // leader: Q of both CTAs
  uint64_t* k_full = bars + 1;             // [NST] leader: both halves of a K tile
  uint64_t* k_empty = bars + 3;            // [NST] per CTA
  uint64_t* v_full = bars + 5;             // [NST] leader
  uint64_t* v_empty = bars + 7;            // [NST] per CTA
  uint64_t* s_full = bars + 9;             // per CTA
  uint64_t* p_full = bars + 10;            // leader: 16 softmax warps (8 per CTA)
  uint64_t* o_done = bars + 11;            // per CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  float* xchg = reinterpret_cast<float*>(bars + 16);  // [4][128] row max / row sum exchange

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int q0 = (int)(blockIdx.x >> 1) * (2 * BQ) + (int)rank * BQ, h = blockIdx.y, b = blockIdx.z;
  const int nkv = (p.Lk + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < NST; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 16);
    mbar_init(o_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // both CTAs' barriers exist before any remote use
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // The pair MMA addresses the accumulators of BOTH CTAs with the leader's tensor-memory address:
  // the two allocations must sit at the same columns. Both CTAs compare (symmetric, so both take
  // the same decision); on a mismatch the launch records code 19 and does no work.
  uint32_t peer_base;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(peer_base) : "r"(map_to_cta(smem_u32(tmem_slot), rank ^ 1)));
  const bool tm_ok = peer_base == tmem_base;
  if (!tm_ok && threadIdx.x == 0) atomicExch(p.err, 19);

  if (!tm_ok) {
    // fall through to the common exit
  } else if (warp == 0) {
    if (elect_one()) {
      // every load credits the LEADER's barrier; only the leader announces the byte count
      if (leader) mbar_expect_tx(q_full, 2 * Q_BYTES);
      const uint32_t qb = map_to_cta(smem_u32(q_full), 0);
#pragma unroll
      for (int c = 0; c < 2; ++c) tma_load_3d_pair(sQ + c * Q_CHUNK, &tmQ, qb, h * DH + c * 64, q0, b);
      for (int j = 0; j < nkv; ++j) {
        const int s = j % NST;
        const uint32_t par = (uint32_t)((j / NST) & 1);
        if (!mbar_wait(&k_empty[s], par ^ 1)) { atomicExch(p.err, 11); break; }
        if (leader) mbar_expect_tx(&k_full[s], 2 * KH_BYTES);
        const uint32_t kb = map_to_cta(smem_u32(&k_full[s]), 0);
#pragma unroll
        for (int c = 0; c < 2; ++c)
          tma_load_3d_pair(sK + s * KH_BYTES + c * K_CHUNK, &tmK, kb, h * DH + c * 64,
                           j * BKV + (int)rank * (BKV / 2), b);
        if (!mbar_wait(&v_empty[s], par ^ 1)) { atomicExch(p.err, 12); break; }
        if (leader) mbar_expect_tx(&v_full[s], 2 * VH_BYTES);
        tma_load_3d_pair(sV + s * VH_BYTES, &tmV, map_to_cta(smem_u32(&v_full[s]), 0),
                         h * DH + (int)rank * 64, j * BKV, b);
      }
    }
  } else if (warp == 1) {
    if (leader && elect_one()) {
      const uint32_t idesc_s = umma_idesc_bf16(2 * BQ, BKV, 0, 0);
      const uint32_t idesc_o = umma_idesc_bf16(2 * BQ, DH, 0, 1);  // B (V) is MN-major
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
      auto commit_both = [&](uint64_t* bar) {
        const uint32_t a = smem_u32(bar);
        umma2_commit_addr(a);
        umma2_commit_addr(map_to_cta(a, 1));
      };
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(p.err, 13);
      for (int j = 0; j < nkv && ok; ++j) {
        const int s = j % NST;
        const uint32_t par = (uint32_t)((j / NST) & 1);
        if (!mbar_wait(&k_full[s], par)) { atomicExch(p.err, 14); break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const uint64_t dq = umma_desc_kmajor(aQ + c * Q_CHUNK, 128);
          const uint64_t dk = umma_desc_kmajor(aK + s * KH_BYTES + c * K_CHUNK, 128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma2_bf16(tmem_base + S_COL, dq + kk * 2, dk + kk * 2, idesc_s, (c | kk) != 0);
        }
        commit_both(s_full);
        commit_both(&k_empty[s]);
        if (!mbar_wait(p_full, (uint32_t)(j & 1))) { atomicExch(p.err, 15); break; }
        if (!mbar_wait(&v_full[s], par)) { atomicExch(p.err, 16); break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          // this CTA's half of V: one 64-column slab, 16 key rows per step
          const uint64_t dv = umma_desc_mn128(aV + s * VH_BYTES + kk * 2048, VH_BYTES);
          umma2_bf16_ts(tmem_base + O_COL, tmem_base + S_COL + (kk >> 2) * 64 + (kk & 3) * 8, dv, idesc_o,
                        (j | kk) != 0);
        }
        commit_both(o_done);
        commit_both(&v_empty[s]);
      }
    }
  } else {
    // Eight softmax warps per CTA, as in the one-CTA kernel: warps w and w + 4 own the same 32
    // query rows and split the 128 key columns of every tile in halves.
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r_in = qd * 32 + lane;
    const int row = q0 + r_in;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    const uint32_t s_col = S_COL + half * 64;
    const uint32_t p_full_leader = map_to_cta(smem_u32(p_full), 0);
    float* s_mx = xchg;
    float* s_l = xchg + 256;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      const uint32_t par = (uint32_t)(j & 1);
      if (ok && !mbar_wait(s_full, par)) {
        if (lane == 0) atomicExch(p.err, 17);
        ok = false;
      }
      if (!ok) {
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (lane == 0) mbar_arrive_cluster(p_full_leader);
        continue;
      }
      tc_fence_after();
      const int kv_left = p.Lk - j * BKV - half * 64;
      const bool full_half = kv_left >= 64;
      float mx = -INFINITY;
      if (full_half) {
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
      const float m_new = mx * p.scale_log2;
      if (j == 0) {
        m_used = m_new;
      } else {
        const bool need = (m_new - m_used) > kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // s_full of this tile was committed after PV of the previous tile, so O is complete
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
      float lsum = 0.f;
      if (full_half) {
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
              v = ex2_poly2(v);
            }
            acc2 = f2_add(acc2, v);
            pk[i] = f2_to_bf162(v);
          }
          tmem_st16(lane_addr + s_col + c * 16, pk);
        }
        float a_lo, a_hi;
        f2_unpack(acc2, a_lo, a_hi);
        lsum = a_lo + a_hi;
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
      if (lane == 0) mbar_arrive_cluster(p_full_leader);
    }
    if (ok) {
      if (!mbar_wait(o_done, (uint32_t)((nkv - 1) & 1))) {
        if (lane == 0) atomicExch(p.err, 18);
        ok = false;
      }
    }
    s_l[half * 128 + r_in] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    l += s_l[(half ^ 1) * 128 + r_in];
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      bf16* orow = p.out + (((size_t)b * p.Lq + row) * p.H + h) * DH + half * (DH / 2);
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
  cluster_sync_all();   // the peer may still read this CTA's shared memory / signal its barriers
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

int* g_fa2_err[64] = {nullptr};

int make_map(CUtensorMap* m, const void* ptr, int B, int L, int H, int rows) {
  uint64_t dims[3] = {(uint64_t)H * DH, (uint64_t)L, (uint64_t)B};
  uint64_t strides[2] = {(uint64_t)H * DH * 2, (uint64_t)L * H * DH * 2};
  uint32_t box[3] = {64, (uint32_t)rows, 1};
  return make_tensor_map(m, ptr, 3, dims, strides, box, 128);
}

template <int POLY>
int launch(const CUtensorMap& q, const CUtensorMap& k, const CUtensorMap& v, const Fa2Params& p, int dev,
           cudaStream_t st) {
  constexpr int SMEM = Q_BYTES + NST * (KH_BYTES + VH_BYTES) + 1024 + 128 + 2048;
  static bool configured[64] = {};
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(fa_fwd2_kernel<POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) !=
        cudaSuccess)
      return -5;
    configured[dev] = true;
  }
  dim3 grid(2 * ((p.Lq + 2 * BQ - 1) / (2 * BQ)), p.H, p.B);
  fa_fwd2_kernel<POLY><<<grid, 320, SMEM, st>>>(q, k, v, p);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

int eri_fa2_check_error() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || !g_fa2_err[dev]) return 0;
  int h = 0;
  cudaMemcpy(&h, g_fa2_err[dev], sizeof(int), cudaMemcpyDeviceToHost);
  if (h) cudaMemset(g_fa2_err[dev], 0, sizeof(int));
  return h;
}

// q [B, Lq, H, 128], k/v [B, Lk, H, 128], out like q (contiguous bf16), lse [B, H, Lq].
// Returns -100 for shapes this kernel does not take (the caller uses the one-CTA kernel).
int eri_flash_attn_fwd_pair(const void* q, const void* k, const void* v, void* out, float* lse, int B,
                            int H, int Lq, int Lk, int head_dim, float scale, int poly, void* stream) {
  if (head_dim != DH || Lq < 2 * BQ || Lk < BKV) return -100;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -3;
  if (!g_fa2_err[dev]) {
    if (cudaMalloc(&g_fa2_err[dev], sizeof(int)) != cudaSuccess) return -3;
    cudaMemset(g_fa2_err[dev], 0, sizeof(int));
  }
  CUtensorMap tq, tk, tv;
  if (make_map(&tq, q, B, Lq, H, BQ) || make_map(&tk, k, B, Lk, H, BKV / 2) || make_map(&tv, v, B, Lk, H, BKV))
    return -4;
  Fa2Params p;
  p.B = B; p.H = H; p.Lq = Lq; p.Lk = Lk;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.out = (bf16*)out; p.lse = lse; p.err = g_fa2_err[dev];
  cudaStream_t st = (cudaStream_t)stream;
  if (poly == 0) return launch<0>(tq, tk, tv, p, dev, st);
  if (poly == 8) return launch<8>(tq, tk, tv, p, dev, st);
  return launch<4>(tq, tk, tv, p, dev, st);
}

}  // extern "C"
