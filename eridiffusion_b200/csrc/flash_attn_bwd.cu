// Flash attention backward for sm_100a (non-causal, head_dim 64 / 128, token-major [B, L, H, Dh]).
//
// Three launches, no atomics, deterministic:
//   prep   delta[b,h,q] = sum_d O * dO, and the log-sum-exp converted to log2 units, both written
//          to buffers padded to a multiple of 128 queries (padding: lse = +inf, so P = 0 there)
//   dkdv   one CTA per 128-key tile, loop over 128-query tiles:
//              S^T  = K Q^T,  dP^T = V dO^T            (smem x smem -> TMEM, keys on TMEM lanes)
//              P^T  = exp2(S^T c - lse2[q]),  dS^T = P^T * (dP^T - delta[q])   (one thread per key)
//              dV  += P^T dO,  dK += dS^T Q            (A operand read from TMEM as packed bf16,
//                                                       dO / Q tiles re-read as MN-major B operands)
//   dq     one CTA per 128-query tile, loop over 128-key tiles:
//              S = Q K^T, dP = dO V^T, dS = P * (dP - delta), dQ += dS K
// Recomputing S and dP in the dq pass costs two extra MMAs per tile pair and removes the global
// fp32 dQ accumulation (atomics or reduce-adds) that a single-pass backward needs.
// The reference's only attention gradient is a recompute through tensor ops
// (crates/core/src/autograd_ops.rs:10-75, attention_backward_recompute).
#include <cstdlib>

#include "ptx.cuh"
#include "tma_host.h"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

struct FaBwdParams {
  int B, H, Lq, Lk, Lp;  // Lp: padded query length of lse2 / delta
  float scale, scale_log2;
  const float* lse2;     // [B, H, Lp]
  const float* delta;    // [B, H, Lp]
  const bf16* q;         // [B, Lq, H, DH] (read directly by the dQ kernel's operand staging)
  const bf16* dout;      // [B, Lq, H, DH]
  long long* trace;      // optional timeline buffer (CTA 0 only), see eri_fa_bwd_set_trace
  int trace_cap;         // entries per recorder
  bf16* dq;              // [B, Lq, H, DH]
  bf16* dk;              // [B, Lk, H, DH]
  bf16* dv;
  int* err;
  const float* kbias;    // MASK variants: [B, Lkb] additive key bias in log2 units (-1e30 = masked),
                         // followed by one int per (batch, 128-key tile): 1 = the tile has a non-zero bias
  int Lkb;               // ceil(Lk / 128) * 128
};

constexpr int T = 128;  // tile edge (queries and keys)

__global__ void fa_bwd_prep_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dout,
                                   const float* __restrict__ lse, float* __restrict__ lse2,
                                   float* __restrict__ delta, int B, int H, int Lq, int Lp, int DH,
                                   long long o_ld) {
  // 16 lanes per (b, h, l) row, one 16-byte load of O and of dO per lane per 128 columns
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long rowid = gid >> 4;
  const int sub = threadIdx.x & 15;
  const long long total = (long long)B * H * Lp;
  if (rowid >= total) return;
  const int l = (int)(rowid % Lp), h = (int)((rowid / Lp) % H), b = (int)(rowid / ((long long)Lp * H));
  float acc = 0.f;
  if (l < Lq) {
    const size_t base = (((size_t)b * Lq + l) * H + h) * DH;
    const size_t obase = ((size_t)b * Lq + l) * o_ld + (size_t)h * DH;   // O may be a column block
    for (int d = sub * 8; d < DH; d += 128) {
      float a[8], g[8];
      unpack8(*reinterpret_cast<const bf16x8*>(o + obase + d), a);
      unpack8(*reinterpret_cast<const bf16x8*>(dout + base + d), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(a[j], g[j], acc);
    }
  }
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (sub == 0) {
    if (l < Lq) {
      delta[rowid] = acc;
      lse2[rowid] = lse[((size_t)b * H + h) * Lq + l] * 1.4426950408889634f;
    } else {
      lse2[rowid] = INFINITY;
      delta[rowid] = 0.f;
    }
  }
}

// Timeline recorder for performance work: when a trace buffer is set, the MMA-issuing thread and
// lane 0 of the first softmax warp of CTA (0,0,0) store (clock64 << 8 | event code) at each
// pipeline hand-off. `rec` selects the recorder's half of the buffer.
__device__ __forceinline__ void trace_ev(const FaBwdParams& p, int rec, int& n, int code) {
  if (p.trace && n < p.trace_cap && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) {
    p.trace[rec * p.trace_cap + n] = (clock64() << 8) | (long long)code;
    ++n;
  }
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ------------------------------------------------------------------------------------- dK, dV
template <int DH, int POLY, bool MASK>
__global__ void __launch_bounds__(576, 1)
fa_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const FaBwdParams p) {
  constexpr int CHUNKS = DH / 64;
  constexpr int CHUNK_BYTES = T * 128;
  constexpr int TILE_BYTES = CHUNK_BYTES * CHUNKS;
  constexpr uint32_t S_COL = 0, DP_COL = 128, DV_COL = 256, DK_COL = 384;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;        // 2 stages
  uint8_t* sDO = sQ + 2 * TILE_BYTES;   // 2 stages
  float* s_lse = reinterpret_cast<float*>(sDO + 2 * TILE_BYTES);  // [2][128]
  float* s_delta = s_lse + 2 * T;                                 // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_delta + 2 * T);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;   // [2]
  uint64_t* qdo_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* dp_full = bars + 6;
  uint64_t* p_ready = bars + 7;    // 16 softmax warps wrote P^T
  uint64_t* ds_ready = bars + 8;   // 16 softmax warps wrote dS^T
  uint64_t* acc_done = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * T, h = blockIdx.y, b = blockIdx.z;
  const int nq = (p.Lq + T - 1) / T;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_ready, 16);
    mbar_init(ds_ready, 16);
    mbar_init(acc_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(kv_full, 2 * TILE_BYTES);
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        tma_load_3d(sK + c * CHUNK_BYTES, &tmK, kv_full, h * DH + c * 64, k0, b);
        tma_load_3d(sV + c * CHUNK_BYTES, &tmV, kv_full, h * DH + c * 64, k0, b);
      }
      for (int i = 0; i < nq; ++i) {
        const int s = i & 1;
        const uint32_t par = (uint32_t)((i >> 1) & 1);
        if (!mbar_wait(&qdo_empty[s], par ^ 1)) { atomicExch(p.err, 21); break; }
        mbar_expect_tx(&qdo_full[s], 2 * TILE_BYTES);
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          tma_load_3d(sQ + s * TILE_BYTES + c * CHUNK_BYTES, &tmQ, &qdo_full[s], h * DH + c * 64,
                      i * T, b);
          tma_load_3d(sDO + s * TILE_BYTES + c * CHUNK_BYTES, &tmDO, &qdo_full[s],
                      h * DH + c * 64, i * T, b);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      // Phase pipeline, every MMA 128 x 128 x 16:
      //   S_i | dP_i | dV_i | S_{i+1} | dK_i | dP_{i+1} | dV_{i+1} | S_{i+2} | dK_{i+1} | ...
      // The softmax warps turn S_i into P_i while dP_i runs, and P_i, dP_i into dS_i while
      // dV_i and S_{i+1} run, so the tensor pipe never waits for them in steady state.
      const uint32_t idesc_s = umma_idesc_bf16(T, T, 0, 0);
      const uint32_t idesc_g = umma_idesc_bf16(T, DH, 0, 1);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV);
      const uint32_t aQ0 = smem_u32(sQ), aDO0 = smem_u32(sDO);
      auto issue_s = [&](int st) {
        const uint32_t aQ = aQ0 + st * TILE_BYTES;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          const uint64_t da = umma_desc_kmajor(aK + c * CHUNK_BYTES, 128);
          const uint64_t db = umma_desc_kmajor(aQ + c * CHUNK_BYTES, 128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(tmem_base + S_COL, da + kk * 2, db + kk * 2, idesc_s, (c | kk) != 0);
        }
        umma_commit(s_full);
      };
      auto issue_dp = [&](int st) {
        const uint32_t aDO = aDO0 + st * TILE_BYTES;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          const uint64_t da = umma_desc_kmajor(aV + c * CHUNK_BYTES, 128);
          const uint64_t db = umma_desc_kmajor(aDO + c * CHUNK_BYTES, 128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(tmem_base + DP_COL, da + kk * 2, db + kk * 2, idesc_s, (c | kk) != 0);
        }
        umma_commit(dp_full);
      };
      // A operand from TMEM: the packed bf16 of query chunk kk/2 sits in that chunk's first columns
      auto issue_acc = [&](uint32_t acc_col, uint32_t a_col, uint32_t b_smem, bool first) {
#pragma unroll
        for (int kk = 0; kk < T / 16; ++kk) {
          const uint64_t db = umma_desc_mn128(b_smem + kk * 2048, CHUNK_BYTES);
          umma_bf16_ts(tmem_base + acc_col, tmem_base + a_col + (kk >> 1) * 32 + (kk & 1) * 8, db,
                       idesc_g, !first || kk != 0);
        }
      };
      int tn = 0;
      trace_ev(p, 0, tn, 0);
      bool ok = mbar_wait(kv_full, 0);
      if (!ok) atomicExch(p.err, 22);
      if (ok && !mbar_wait(&qdo_full[0], 0)) { atomicExch(p.err, 23); ok = false; }
      trace_ev(p, 0, tn, 1);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        issue_dp(0);
      }
      for (int i = 0; i < nq && ok; ++i) {
        const int s = i & 1;
        const uint32_t par = (uint32_t)(i & 1);
        const bool more = i + 1 < nq;
        if (!mbar_wait(p_ready, par)) { atomicExch(p.err, 24); ok = false; break; }
        trace_ev(p, 0, tn, 2);
        tc_fence_after();
        issue_acc(DV_COL, S_COL, aDO0 + s * TILE_BYTES, i == 0);
        trace_ev(p, 0, tn, 3);
        if (more) {
          if (!mbar_wait(&qdo_full[s ^ 1], (uint32_t)(((i + 1) >> 1) & 1))) {
            atomicExch(p.err, 23);
            ok = false;
            break;
          }
          trace_ev(p, 0, tn, 4);
          tc_fence_after();
          issue_s(s ^ 1);
          trace_ev(p, 0, tn, 5);
        }
        if (!mbar_wait(ds_ready, par)) { atomicExch(p.err, 27); ok = false; break; }
        trace_ev(p, 0, tn, 6);
        tc_fence_after();
        issue_acc(DK_COL, DP_COL, aQ0 + s * TILE_BYTES, i == 0);
        umma_commit(&qdo_empty[s]);
        trace_ev(p, 0, tn, 7);
        if (more) issue_dp(s ^ 1);
        trace_ev(p, 0, tn, 8);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    // Sixteen softmax warps: warp (qd, c) owns TMEM lanes [32 qd, 32 qd + 32) (keys) and the
    // 32-query chunk c of every tile. Phase 1 (after S^T): P^T = exp2(S^T c - lse2), written back
    // over the chunk's first 16 columns as packed bf16 and kept in registers as fp32. Phase 2
    // (after dP^T): dS^T = P^T * (dP^T - delta), written the same way over dP^T.
    const int qd = warp & 3;
    const int ew = warp - 2;
    const int c = ew >> 2;
    const int sub = c;                                // epilogue column chunk
    const int tid = threadIdx.x - 64;                 // 0..511
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    const size_t stat_base = ((size_t)b * p.H + h) * p.Lp;
    const f32x2 sc2 = f2_pack(p.scale_log2, p.scale_log2);
    // MASK: this thread's key (its TMEM lane) carries one bias value for every query of the tile
    float kb = 0.f;
    if constexpr (MASK) kb = p.kbias[(size_t)b * p.Lkb + k0 + qd * 32 + lane];
    const f32x2 kb2 = f2_pack(kb, kb);
    bool ok = true;
    int tn = 0;
    const int rec = (ew == 0 && lane == 0) ? 1 : -1;
    // Row statistics of the query tile: -lse2 (so one packed fma gives s * c - lse2) and delta,
    // staged through shared memory one tile ahead: the global load for tile i + 1 is issued at
    // the top of tile i and stored at its end, so its latency never sits in the loop.
    const float* stat_src = tid < T ? p.lse2 + stat_base + tid : p.delta + stat_base + tid - T;
    float* stat_dst = tid < T ? s_lse + tid : s_delta + tid - T;
    const float stat_sign = tid < T ? -1.f : 1.f;
    if (tid < 2 * T) stat_dst[0] = stat_sign * stat_src[0];
    for (int i = 0; i < nq; ++i) {
      const int s = i & 1;
      float stat_next = 0.f;
      if (tid < 2 * T && i + 1 < nq) stat_next = stat_sign * stat_src[(size_t)(i + 1) * T];
      named_bar_sync(1, 512);
      const float4* ls4 = reinterpret_cast<const float4*>(s_lse + s * T) + c * 8;
      const float4* dl4 = reinterpret_cast<const float4*>(s_delta + s * T) + c * 8;
      if (rec > 0) trace_ev(p, rec, tn, 10);
      if (!mbar_wait(s_full, (uint32_t)(i & 1))) {
        if (lane == 0) atomicExch(p.err, 25);
        ok = false;
        break;
      }
      if (rec > 0) trace_ev(p, rec, tn, 11);
      tc_fence_after();
      f32x2 pr[16];
      {
        uint32_t r[32];
        tmem_ld32(lane_addr + S_COL + c * 32, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int x4 = 0; x4 < 8; ++x4) {
          const float4 nl = ls4[x4];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int x = 2 * x4 + hh;
            const f32x2 nl2 = hh ? f2_pack(nl.z, nl.w) : f2_pack(nl.x, nl.y);
            f32x2 v = f2_fma(f2_pack_bits(r[2 * x], r[2 * x + 1]), sc2, nl2);
            if constexpr (MASK) v = f2_add(v, kb2);
            if (x < 16 - POLY) {
              float lo, hi;
              f2_unpack(v, lo, hi);
              v = f2_pack(ex2_mufu(lo), ex2_mufu(hi));
            } else {
              v = MASK ? ex2_poly2_z(v) : ex2_poly2(v);
            }
            pr[x] = v;
            pk[x] = f2_to_bf162(v);
          }
        }
        tmem_st16(lane_addr + S_COL + c * 32, pk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready);
      }
      if (rec > 0) trace_ev(p, rec, tn, 13);
      if (!mbar_wait(dp_full, (uint32_t)(i & 1))) {
        if (lane == 0) atomicExch(p.err, 28);
        ok = false;
        break;
      }
      if (rec > 0) trace_ev(p, rec, tn, 14);
      tc_fence_after();
      {
        uint32_t g[32];
        tmem_ld32(lane_addr + DP_COL + c * 32, g);
        tmem_ld_wait();
        uint32_t dk_[16];
#pragma unroll
        for (int x4 = 0; x4 < 8; ++x4) {
          const float4 dl = dl4[x4];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int x = 2 * x4 + hh;
            const f32x2 dl2 = hh ? f2_pack(dl.z, dl.w) : f2_pack(dl.x, dl.y);
            dk_[x] = f2_to_bf162(f2_mul(pr[x], f2_sub(f2_pack_bits(g[2 * x], g[2 * x + 1]), dl2)));
          }
        }
        tmem_st16(lane_addr + DP_COL + c * 32, dk_);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_ready);
        if (rec > 0) trace_ev(p, rec, tn, 17);
      }
      if (tid < 2 * T && i + 1 < nq) stat_dst[(s ^ 1) * T] = stat_next;
    }
    if (ok && !mbar_wait(acc_done, 0)) {
      if (lane == 0) atomicExch(p.err, 26);
      ok = false;
    }
    if (ok) {
      tc_fence_after();
      const int kv = k0 + qd * 32 + lane;
      const size_t obase = (((size_t)b * p.Lk + kv) * p.H + h) * DH;
#pragma unroll 1
      for (int c = sub; c < DH / 32; c += 4) {
        uint32_t rv[32], rk[32];
        tmem_ld32(lane_addr + DV_COL + c * 32, rv);
        tmem_ld32(lane_addr + DK_COL + c * 32, rk);
        tmem_ld_wait();
        if (kv < p.Lk) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float a[8], bb[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              a[x] = __uint_as_float(rv[g * 8 + x]);
              bb[x] = __uint_as_float(rk[g * 8 + x]) * p.scale;
            }
            *reinterpret_cast<bf16x8*>(p.dv + obase + c * 32 + g * 8) = pack8(a);
            *reinterpret_cast<bf16x8*>(p.dk + obase + c * 32 + g * 8) = pack8(bb);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------- dQ
template <int DH, int POLY, bool MASK>
__global__ void __launch_bounds__(576, 1)
fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const FaBwdParams p) {
  constexpr int CHUNKS = DH / 64;
  constexpr int CHUNK_BYTES = T * 128;
  constexpr int TILE_BYTES = CHUNK_BYTES * CHUNKS;
  // TMEM: S, dP and the dQ accumulator (fp32, 128 columns each), Q as a packed-bf16 A operand
  // (64 columns, staged once) and dS as a packed-bf16 A operand (64 columns). dS has its own
  // columns so that the next dP does not have to wait for dQ to consume dS out of the dP region.
  constexpr uint32_t S_COL = 0, DP_COL = 128, DQ_COL = 256, QA_COL = 384, DS_COL = 448;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  // Three K/V stages: a 64 KB tile pair takes ~1500 cycles to arrive, about one tile period, so
  // the load of tile j + 2 has to start while tile j is still being consumed.
  constexpr int NST = 3;
  uint8_t* sK = smem;                    // NST stages
  uint8_t* sV = sK + NST * TILE_BYTES;   // NST stages
  uint8_t* sDO = sV + NST * TILE_BYTES;  // this CTA's dO tile (A operand of dP, loaded once)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDO + TILE_BYTES);
  uint64_t* qa_ready = bars + 0;  // Q / dO staged in TMEM by the 16 softmax warps
  uint64_t* kv_full = bars + 1;   // [NST]
  uint64_t* kv_empty = bars + 4;  // [NST]
  uint64_t* s_full = bars + 7;
  uint64_t* dp_full = bars + 8;
  uint64_t* s_read = bars + 9;     // 16 softmax warps hold S in registers
  uint64_t* ds_ready = bars + 10;  // 16 softmax warps wrote dS
  uint64_t* acc_done = bars + 11;
  uint64_t* do_full = bars + 12;
  uint64_t* dp_read = bars + 13;   // 16 softmax warps hold dP in registers
  uint64_t* dq_done = bars + 14;   // dQ_j finished reading dS_j
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * T, h = blockIdx.y, b = blockIdx.z;
  const int nkv = (p.Lk + T - 1) / T;

  if (threadIdx.x == 0) {
    mbar_init(qa_ready, 16);
    for (int s = 0; s < NST; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(s_read, 16);
    mbar_init(ds_ready, 16);
    mbar_init(acc_done, 1);
    mbar_init(do_full, 1);
    mbar_init(dp_read, 16);
    mbar_init(dq_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(do_full, TILE_BYTES);
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c)
        tma_load_3d(sDO + c * CHUNK_BYTES, &tmDO, do_full, h * DH + c * 64, q0, b);
      for (int j = 0; j < nkv; ++j) {
        const int s = j % NST;
        if (!mbar_wait(&kv_empty[s], (uint32_t)(((j / NST) & 1) ^ 1))) { atomicExch(p.err, 31); break; }
        mbar_expect_tx(&kv_full[s], 2 * TILE_BYTES);
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          tma_load_3d(sK + s * TILE_BYTES + c * CHUNK_BYTES, &tmK, &kv_full[s], h * DH + c * 64,
                      j * T, b);
          tma_load_3d(sV + s * TILE_BYTES + c * CHUNK_BYTES, &tmV, &kv_full[s], h * DH + c * 64,
                      j * T, b);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      // Phase pipeline, every MMA 128 x 128 x 16:
      //   S_0 | dP_0 | S_1 | dP_1 | dQ_0 | S_2 | dP_2 | dQ_1 | ...
      // S_{j+1} is issued once the softmax warps hold S_j in registers, dP_{j+1} once they hold
      // dP_j, dQ_j once dS_j is written; nothing the tensor pipe runs next depends on the softmax
      // work of the tile before it, so that work hides under a full tile of MMAs.
      const uint32_t idesc_s = umma_idesc_bf16(T, T, 0, 0);
      const uint32_t idesc_g = umma_idesc_bf16(T, DH, 0, 1);
      const uint32_t aK0 = smem_u32(sK), aV0 = smem_u32(sV);
      auto issue_s = [&](int st) {
        const uint32_t aK = aK0 + st * TILE_BYTES;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          const uint64_t db = umma_desc_kmajor(aK + c * CHUNK_BYTES, 128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16_ts(tmem_base + S_COL, tmem_base + QA_COL + (c * 4 + kk) * 8, db + kk * 2,
                         idesc_s, (c | kk) != 0);
        }
        umma_commit(s_full);
      };
      const uint32_t aDO = smem_u32(sDO);
      auto issue_dp = [&](int st) {
        const uint32_t aV = aV0 + st * TILE_BYTES;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          const uint64_t da = umma_desc_kmajor(aDO + c * CHUNK_BYTES, 128);
          const uint64_t db = umma_desc_kmajor(aV + c * CHUNK_BYTES, 128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(tmem_base + DP_COL, da + kk * 2, db + kk * 2, idesc_s, (c | kk) != 0);
        }
        umma_commit(dp_full);
      };
      auto issue_dq = [&](int st, bool first) {
        const uint32_t aK = aK0 + st * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < T / 16; ++kk) {
          const uint64_t dbk = umma_desc_mn128(aK + kk * 2048, CHUNK_BYTES);
          umma_bf16_ts(tmem_base + DQ_COL, tmem_base + DS_COL + kk * 8, dbk, idesc_g,
                       !first || kk != 0);
        }
        umma_commit(dq_done);
      };
      int tn = 0;
      trace_ev(p, 0, tn, 0);
      bool ok = mbar_wait(qa_ready, 0);
      if (!ok) atomicExch(p.err, 32);
      trace_ev(p, 0, tn, 1);
      if (ok && !mbar_wait(do_full, 0)) { atomicExch(p.err, 32); ok = false; }
      if (ok && !mbar_wait(&kv_full[0], 0)) { atomicExch(p.err, 33); ok = false; }
      if (ok) {
        tc_fence_after();
        issue_s(0);
        issue_dp(0);
      }
      for (int j = 0; j < nkv && ok; ++j) {
        const int s = j % NST, sn = (j + 1) % NST;
        const uint32_t par = (uint32_t)(j & 1);
        const bool more = j + 1 < nkv;
        if (more) {
          if (!mbar_wait(&kv_full[sn], (uint32_t)(((j + 1) / NST) & 1))) {
            atomicExch(p.err, 33);
            ok = false;
            break;
          }
          trace_ev(p, 0, tn, 2);
          if (!mbar_wait(s_read, par)) { atomicExch(p.err, 38); ok = false; break; }
          trace_ev(p, 0, tn, 3);
          tc_fence_after();
          issue_s(sn);
          trace_ev(p, 0, tn, 4);
          if (!mbar_wait(dp_read, par)) { atomicExch(p.err, 40); ok = false; break; }
          tc_fence_after();
          issue_dp(sn);
          trace_ev(p, 0, tn, 7);
        }
        if (!mbar_wait(ds_ready, par)) { atomicExch(p.err, 34); ok = false; break; }
        trace_ev(p, 0, tn, 5);
        tc_fence_after();
        issue_dq(s, j == 0);
        umma_commit(&kv_empty[s]);
        trace_ev(p, 0, tn, 6);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    // Sixteen softmax warps: warp (qd, c) owns TMEM lanes [32 qd, 32 qd + 32) (queries) and the
    // 32-key chunk c of every tile. Phase 1 (after S): P = exp2(S c - lse2) into registers.
    // Phase 2 (after dP): dS = P * (dP - delta), written over the chunk's first 16 dP columns as
    // packed bf16 (the A operand of dQ += dS K).
    const int qd = warp & 3;
    const int ew = warp - 2;
    const int c = ew >> 2;
    const int sub = c;
    const int row = q0 + qd * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    const size_t stat = ((size_t)b * p.H + h) * p.Lp + row;  // row < Lp always
    const float lse2 = p.lse2[stat], delta = p.delta[stat];
    bool ok = true;
    const f32x2 sc2 = f2_pack(p.scale_log2, p.scale_log2);
    const f32x2 nl2 = f2_pack(-lse2, -lse2);
    const f32x2 dl2 = f2_pack(delta, delta);
    {
      // Stage Q as a constant A operand: warp groups 0 and 1 copy one half of the row block
      // each, every thread its own query row (= TMEM lane), straight from global memory.
      const bf16* src = p.q + (((size_t)b * p.Lq + row) * p.H + h) * DH + (sub & 1) * (DH / 2);
      const uint32_t dst = lane_addr + QA_COL + (sub & 1) * (DH / 4);
#pragma unroll
      for (int w = 0; w < (sub < 2 ? DH / 64 : 0); ++w) {
        uint32_t v[16];
        if (row < p.Lq) {
          const uint4* s4 = reinterpret_cast<const uint4*>(src + w * 32);
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const uint4 u = s4[t];
            v[4 * t] = u.x; v[4 * t + 1] = u.y; v[4 * t + 2] = u.z; v[4 * t + 3] = u.w;
          }
        } else {
#pragma unroll
          for (int t = 0; t < 16; ++t) v[t] = 0u;
        }
        tmem_st16(dst + w * 16, v);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(qa_ready);
    }
    int tn = 0;
    const int rec = (ew == 0 && lane == 0) ? 1 : -1;
    for (int j = 0; j < nkv; ++j) {
      const int kv_left = p.Lk - j * T - c * 32;  // valid keys in this warp's chunk
      if (rec > 0) trace_ev(p, rec, tn, 10);
      if (!mbar_wait(s_full, (uint32_t)(j & 1))) {
        if (lane == 0) atomicExch(p.err, 35);
        ok = false;
        break;
      }
      if (rec > 0) trace_ev(p, rec, tn, 11);
      tc_fence_after();
      f32x2 pr[16];
      {
        uint32_t r[32];
        tmem_ld32(lane_addr + S_COL + c * 32, r);
        tmem_ld_wait();
        if (rec > 0) trace_ev(p, rec, tn, 12);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_read);  // S is in registers: the next S may overwrite it
        const bool use_bias =
            MASK && reinterpret_cast<const int*>(p.kbias + (size_t)p.B * p.Lkb)[b * (p.Lkb / T) + j] != 0;
        if (use_bias) {
          // the 32 keys of this warp's chunk: every lane reads the same bias values
          const float4* kb4 = reinterpret_cast<const float4*>(p.kbias + (size_t)b * p.Lkb + j * T + c * 32);
#pragma unroll
          for (int x4 = 0; x4 < 8; ++x4) {
            const float4 kb = __ldg(kb4 + x4);
            const float p0 = ex2_mufu(fmaf(__uint_as_float(r[4 * x4]), p.scale_log2, kb.x) - lse2);
            const float p1 = ex2_mufu(fmaf(__uint_as_float(r[4 * x4 + 1]), p.scale_log2, kb.y) - lse2);
            const float p2 = ex2_mufu(fmaf(__uint_as_float(r[4 * x4 + 2]), p.scale_log2, kb.z) - lse2);
            const float p3 = ex2_mufu(fmaf(__uint_as_float(r[4 * x4 + 3]), p.scale_log2, kb.w) - lse2);
            pr[2 * x4] = f2_pack(p0, p1);
            pr[2 * x4 + 1] = f2_pack(p2, p3);
          }
        } else if (kv_left >= 32) {
#pragma unroll
          for (int x = 0; x < 16; ++x) {
            f32x2 v = f2_fma(f2_pack_bits(r[2 * x], r[2 * x + 1]), sc2, nl2);
            if (x < 16 - POLY) {
              float lo, hi;
              f2_unpack(v, lo, hi);
              v = f2_pack(ex2_mufu(lo), ex2_mufu(hi));
            } else {
              v = MASK ? ex2_poly2_z(v) : ex2_poly2(v);
            }
            pr[x] = v;
          }
        } else {
#pragma unroll
          for (int x = 0; x < 16; ++x) {
            float p0 = exp2f(fmaf(__uint_as_float(r[2 * x]), p.scale_log2, -lse2));
            float p1 = exp2f(fmaf(__uint_as_float(r[2 * x + 1]), p.scale_log2, -lse2));
            if (2 * x >= kv_left) p0 = 0.f;
            if (2 * x + 1 >= kv_left) p1 = 0.f;
            pr[x] = f2_pack(p0, p1);
          }
        }
      }
      if (rec > 0) trace_ev(p, rec, tn, 13);
      if (!mbar_wait(dp_full, (uint32_t)(j & 1))) {
        if (lane == 0) atomicExch(p.err, 39);
        ok = false;
        break;
      }
      if (rec > 0) trace_ev(p, rec, tn, 14);
      tc_fence_after();
      {
        uint32_t g[32];
        tmem_ld32(lane_addr + DP_COL + c * 32, g);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dp_read);  // dP is in registers: the next dP may overwrite it
        if (rec > 0) trace_ev(p, rec, tn, 15);
        uint32_t dk_[16];
#pragma unroll
        for (int x = 0; x < 16; ++x)
          dk_[x] = f2_to_bf162(f2_mul(pr[x], f2_sub(f2_pack_bits(g[2 * x], g[2 * x + 1]), dl2)));
        // dS_{j-1} must have been consumed by dQ_{j-1} before its columns are overwritten
        if (j > 0 && !mbar_wait(dq_done, (uint32_t)((j - 1) & 1))) {
          if (lane == 0) atomicExch(p.err, 41);
          ok = false;
          break;
        }
        tc_fence_after();
        tmem_st16(lane_addr + DS_COL + c * 16, dk_);
        if (rec > 0) trace_ev(p, rec, tn, 16);
        tmem_st_wait();
        if (rec > 0) trace_ev(p, rec, tn, 17);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_ready);
      }
    }
    if (ok && !mbar_wait(acc_done, 0)) {
      if (lane == 0) atomicExch(p.err, 36);
      ok = false;
    }
    if (ok) {
      tc_fence_after();
      const size_t obase = (((size_t)b * p.Lq + row) * p.H + h) * DH;
#pragma unroll 1
      for (int c = sub; c < DH / 32; c += 4) {
        uint32_t r[32];
        tmem_ld32(lane_addr + DQ_COL + c * 32, r);
        tmem_ld_wait();
        if (row < p.Lq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float a[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) a[x] = __uint_as_float(r[g * 8 + x]) * p.scale;
            *reinterpret_cast<bf16x8*>(p.dq + obase + c * 32 + g * 8) = pack8(a);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

int* g_fab_err[64] = {nullptr};   // one error word per device
long long* g_fab_trace = nullptr;
int g_fab_trace_cap = 0;
int g_fab_trace_kernel = 0;  // 0: dQ kernel, 1: dK/dV kernel

int make_map(CUtensorMap* m, const void* ptr, int B, int L, int H, int DH) {
  uint64_t dims[3] = {(uint64_t)H * DH, (uint64_t)L, (uint64_t)B};
  uint64_t strides[2] = {(uint64_t)H * DH * 2, (uint64_t)L * H * DH * 2};
  uint32_t box[3] = {64, 128, 1};
  return make_tensor_map(m, ptr, 3, dims, strides, box, 128);
}

template <int DH, int POLY, bool MASK>
int launch_bwd_v(const CUtensorMap& q, const CUtensorMap& k, const CUtensorMap& v,
                 const CUtensorMap& d, const FaBwdParams& p, cudaStream_t st) {
  constexpr int SMEM = 6 * 128 * 128 * (DH / 64) + 2048 + 1024 + 128;
  constexpr int SMEM_DQ = 7 * 128 * 128 * (DH / 64) + 1024 + 256;  // 3 K/V stages + dO + barriers
  // The shared-memory limit is an attribute of the (kernel, device) pair: one flag per device, so
  // that a process driving several GPUs raises it on each of them.
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -5;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(fa_bwd_dkdv_kernel<DH, POLY, MASK>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return -5;
    if (cudaFuncSetAttribute(fa_bwd_dq_kernel<DH, POLY, MASK>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DQ) != cudaSuccess)
      return -5;
    configured[dev] = true;
  }
  dim3 g1((p.Lk + T - 1) / T, p.H, p.B), g2((p.Lq + T - 1) / T, p.H, p.B);
  FaBwdParams p1 = p, p2 = p;
  if (g_fab_trace_kernel == 0) p1.trace = nullptr; else p2.trace = nullptr;
  fa_bwd_dkdv_kernel<DH, POLY, MASK><<<g1, 576, SMEM, st>>>(q, k, v, d, p1);
  fa_bwd_dq_kernel<DH, POLY, MASK><<<g2, 576, SMEM_DQ, st>>>(q, k, v, d, p2);
  return (int)cudaGetLastError();
}

// Pairs (of every 16) whose 2^x runs on the FMA pipe instead of the special-function unit;
// ERI_B200_FA_BWD_POLY = 0, 4 or 8 (read once, no allocation).
int bwd_poly_pairs() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("ERI_B200_FA_BWD_POLY");
    v = e ? atoi(e) : 4;
    if (v != 0 && v != 4 && v != 8) v = 4;
  }
  return v;
}

template <int DH>
int launch_bwd(const CUtensorMap& q, const CUtensorMap& k, const CUtensorMap& v,
               const CUtensorMap& d, const FaBwdParams& p, cudaStream_t st) {
  if (p.kbias) return launch_bwd_v<DH, 4, true>(q, k, v, d, p, st);
  const int poly = bwd_poly_pairs();
  if (poly == 0) return launch_bwd_v<DH, 0, false>(q, k, v, d, p, st);
  if (poly == 8) return launch_bwd_v<DH, 8, false>(q, k, v, d, p, st);
  return launch_bwd_v<DH, 4, false>(q, k, v, d, p, st);
}

void launch_prep(const void* out, const void* dout, const float* lse, float* lse2, float* delta, int B,
                 int H, int Lq, int Lp, int DH, cudaStream_t st, long long out_ld = 0) {
  if (out_ld == 0) out_ld = (long long)H * DH;
  const long long rows = (long long)B * H * Lp;
  const int block = 256;
  const long long grid = (rows * 16 + block - 1) / block;
  fa_bwd_prep_kernel<<<(unsigned)grid, block, 0, st>>>((const bf16*)out, (const bf16*)dout, lse, lse2,
                                                       delta, B, H, Lq, Lp, DH, out_ld);
}

int bwd_entry(const void* dout, const void* q, const void* k, const void* v, const void* out,
              const float* lse, float* lse2, float* delta, void* dq, void* dk, void* dv,
              const float* kbias, int B, int H, int Lq, int Lk, int DH, float scale, void* stream,
              long long out_ld = 0) {
  if (DH != 64 && DH != 128) return -1;
  if (Lq < 1 || Lk < 1 || (Lk < 128 && !kbias)) return -2;
  if (kbias && (((uintptr_t)kbias) & 15)) return -6;
  if (out_ld && (out_ld < (long long)H * DH || out_ld % 8 || (((uintptr_t)out) & 15))) return -7;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -3;
  if (!g_fab_err[dev]) {
    if (cudaMalloc(&g_fab_err[dev], sizeof(int)) != cudaSuccess) return -3;
    cudaMemset(g_fab_err[dev], 0, sizeof(int));
  }
  cudaStream_t st = (cudaStream_t)stream;
  const int Lp = (Lq + T - 1) / T * T;
  CUtensorMap tq, tk, tv, td;
  if (make_map(&tq, q, B, Lq, H, DH) || make_map(&tk, k, B, Lk, H, DH) ||
      make_map(&tv, v, B, Lk, H, DH) || make_map(&td, dout, B, Lq, H, DH))
    return -4;
  launch_prep(out, dout, lse, lse2, delta, B, H, Lq, Lp, DH, st, out_ld);
  FaBwdParams p;
  p.B = B; p.H = H; p.Lq = Lq; p.Lk = Lk; p.Lp = Lp;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse2 = lse2; p.delta = delta; p.q = (const bf16*)q; p.dout = (const bf16*)dout;
  p.trace = g_fab_trace; p.trace_cap = g_fab_trace_cap;
  p.dq = (bf16*)dq; p.dk = (bf16*)dk; p.dv = (bf16*)dv; p.err = g_fab_err[dev];
  p.kbias = kbias; p.Lkb = (Lk + T - 1) / T * T;
  return DH == 128 ? launch_bwd<128>(tq, tk, tv, td, p, st) : launch_bwd<64>(tq, tk, tv, td, p, st);
}

}  // namespace

extern "C" {

int eri_fa_bwd_check_error() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || !g_fab_err[dev]) return 0;
  int h = 0;
  cudaMemcpy(&h, g_fab_err[dev], sizeof(int), cudaMemcpyDeviceToHost);
  if (h) cudaMemset(g_fab_err[dev], 0, sizeof(int));
  return h;
}

// Timeline tracing for performance work: `buf` holds 2 * cap int64 entries (first half: the
// MMA-issuing thread, second half: lane 0 of the first softmax warp, both of CTA (0,0,0) of the
// dQ kernel (which_kernel = 0) or the dK/dV kernel (1)), each (clock64 << 8) | event code. Pass
// nullptr to switch tracing off.
int eri_fa_bwd_set_trace(long long* buf, int cap, int which_kernel) {
  g_fab_trace = buf;
  g_fab_trace_cap = buf ? cap : 0;
  g_fab_trace_kernel = which_kernel;
  return 0;
}

// All tensors contiguous bf16 [B, L, H, DH]; lse [B, H, Lq] fp32 from the forward.
// Scratch supplied by the caller: lse2 and delta, each [B, H, Lp] fp32 with Lp = ceil(Lq/128)*128.
int eri_flash_attn_bwd(const void* dout, const void* q, const void* k, const void* v,
                       const void* out, const float* lse, float* lse2, float* delta, void* dq,
                       void* dk, void* dv, int B, int H, int Lq, int Lk, int DH, float scale,
                       void* stream) {
  return bwd_entry(dout, q, k, v, out, lse, lse2, delta, dq, dk, dv, nullptr, B, H, Lq, Lk, DH, scale,
                   stream);
}

// The same with the forward output's token stride given (see eri_flash_attn_fwd_ld); only the
// row-sum preparation reads the forward output.
int eri_flash_attn_bwd_ld(const void* dout, const void* q, const void* k, const void* v,
                          const void* out, const float* lse, float* lse2, float* delta, void* dq,
                          void* dk, void* dv, int B, int H, int Lq, int Lk, int DH, float scale,
                          long long out_ld, void* stream) {
  return bwd_entry(dout, q, k, v, out, lse, lse2, delta, dq, dk, dv, nullptr, B, H, Lq, Lk, DH, scale,
                   stream, out_ld);
}

// The same with the additive key bias of eri_flash_attn_fwd_masked (the forward's lse already
// contains it). Gradients of masked keys come out as zeros.
int eri_flash_attn_bwd_masked(const void* dout, const void* q, const void* k, const void* v,
                              const void* out, const float* lse, float* lse2, float* delta, void* dq,
                              void* dk, void* dv, const float* kbias, int B, int H, int Lq, int Lk,
                              int DH, float scale, void* stream) {
  if (!kbias) return -6;
  return bwd_entry(dout, q, k, v, out, lse, lse2, delta, dq, dk, dv, kbias, B, H, Lq, Lk, DH, scale,
                   stream);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Allocation-free attention backward (declared in flash_attn_noalloc.h).
//
// Who needs this: code that drives the library from a place where asking CUDA for memory is not
// possible or not allowed — a host application that hands this library a fixed memory budget and
// forbids any further cudaMalloc, a plug-in running inside another framework's allocator that
// must not allocate behind its back, or a real-time loop where an allocation (which may
// synchronise the device or fail under fragmentation) is unacceptable. Such callers can provide
// the inputs and outputs they own, but have nowhere to get the kernel's two scratch vectors
// (the log-sum-exp in log2 units and the row sums of O*dO). Here the scratch lives in a
// fixed-size array that is part of the loaded library image on every GPU.
//
// Limits and rules:
//  * B * H * ceil(Lq/128)*128 must not exceed ERI_FA_NOALLOC_MAX_ROWS (262144 rows; the array
//    holds two fp32 vectors of that length, 2 MiB per GPU that loads the library, kept until the
//    process exits). Larger problems are rejected with ERI_FA_NOALLOC_TOO_LARGE.
//  * The first call on each device looks up the device address of the array (and of the status
//    word) with cudaGetSymbolAddress while that device is current. Make that first call outside
//    of any stream capture.
//  * Every call on a device uses the same array. The array keeps whatever the previous call left
//    in it; this kernel overwrites every element it later reads, so nothing has to be cleared.
//    Two calls whose GPU work overlaps in time (different streams, or different host threads)
//    race on the array and corrupt each other: serialise them.
//  * No cudaMalloc / cudaFree / cudaMallocAsync and no allocating library routine is called.
// ---------------------------------------------------------------------------------------------
#define ERI_FA_NOALLOC_MAX_ROWS 262144
#define ERI_FA_NOALLOC_MAX_DEVICES 64

static __device__ __align__(256) float g_fa_noalloc_scratch[2 * ERI_FA_NOALLOC_MAX_ROWS];
static __device__ __align__(256) int g_fa_noalloc_status[64];

static float* g_fa_noalloc_scratch_addr[ERI_FA_NOALLOC_MAX_DEVICES] = {nullptr};
static int* g_fa_noalloc_status_addr[ERI_FA_NOALLOC_MAX_DEVICES] = {nullptr};

namespace {

// Tensor-map encode without the host-side cache (the cache grows a std::unordered_map).
int encode_map_uncached(CUtensorMap* m, const void* ptr, int B, int L, int H, int DH) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)H * DH, (cuuint64_t)L, (cuuint64_t)B};
  cuuint64_t strides[2] = {(cuuint64_t)H * DH * 2, (cuuint64_t)L * H * DH * 2};
  cuuint32_t box[3] = {64, 128, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides,
                  box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -1;
}

}  // namespace

extern "C" {

const char* eri_flash_attn_bwd_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -1: return "head_dim must be 64 or 128";
    case -2: return "sequence lengths must be at least 128";
    case -4: return "could not encode a TMA tensor map for one of the tensors";
    case -5: return "could not raise the kernel's shared-memory limit";
    case -6: return "ERI_FA_NOALLOC_TOO_LARGE: B*H*ceil(Lq/128)*128 exceeds the 262144-row static scratch";
    case -7: return "cudaGetSymbolAddress failed for the static scratch array";
    case -8: return "device ordinal above the supported table size";
    default: return "CUDA launch error (value is a cudaError_t)";
  }
}

int eri_flash_attn_bwd_noalloc_max_rows() { return ERI_FA_NOALLOC_MAX_ROWS; }

// Reads (and clears) the status word the kernels set when one of their bounded waits ran out.
// Synchronous device-to-host copy of 4 bytes; allocates nothing. 0 = clean.
int eri_flash_attn_bwd_noalloc_status() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= ERI_FA_NOALLOC_MAX_DEVICES) return -8;
  if (!g_fa_noalloc_status_addr[dev]) return 0;
  int h = 0;
  cudaMemcpy(&h, g_fa_noalloc_status_addr[dev], sizeof(int), cudaMemcpyDeviceToHost);
  if (h) cudaMemset(g_fa_noalloc_status_addr[dev], 0, sizeof(int));
  return h;
}

// dout, q, out, dq: [B, Lq, H, DH]; k, v, dk, dv: [B, Lk, H, DH]; all contiguous bf16 on the
// current device. lse: [B, H, Lq] fp32 as written by eri_flash_attn_fwd. Work is enqueued on
// `stream`; returns 0 or a negative code (see eri_flash_attn_bwd_noalloc_strerror).
int eri_flash_attn_bwd_noalloc(const void* dout, const void* q, const void* k, const void* v,
                               const void* out, const float* lse, void* dq, void* dk, void* dv,
                               int B, int H, int Lq, int Lk, int DH, float scale, void* stream) {
  if (DH != 64 && DH != 128) return -1;
  if (Lq < 128 || Lk < 128) return -2;
  const int Lp = (Lq + T - 1) / T * T;
  const long long rows = (long long)B * H * Lp;
  if (rows > ERI_FA_NOALLOC_MAX_ROWS) return -6;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= ERI_FA_NOALLOC_MAX_DEVICES) return -8;
  if (!g_fa_noalloc_scratch_addr[dev]) {
    // One-time set-up for this device: the array's name is only a host-side handle, the kernels
    // need its device address.
    float* sp = nullptr;
    int* ep = nullptr;
    if (cudaGetSymbolAddress((void**)&sp, g_fa_noalloc_scratch) != cudaSuccess || !sp) return -7;
    if (cudaGetSymbolAddress((void**)&ep, g_fa_noalloc_status) != cudaSuccess || !ep) return -7;
    g_fa_noalloc_status_addr[dev] = ep;
    g_fa_noalloc_scratch_addr[dev] = sp;
  }
  float* lse2 = g_fa_noalloc_scratch_addr[dev];
  float* delta = lse2 + ERI_FA_NOALLOC_MAX_ROWS;
  cudaStream_t st = (cudaStream_t)stream;
  // every check that can fail comes before the first launch, so that a rejected call leaves the
  // shared scratch untouched
  CUtensorMap tq, tk, tv, td;
  if (encode_map_uncached(&tq, q, B, Lq, H, DH) || encode_map_uncached(&tk, k, B, Lk, H, DH) ||
      encode_map_uncached(&tv, v, B, Lk, H, DH) || encode_map_uncached(&td, dout, B, Lq, H, DH))
    return -4;
  launch_prep(out, dout, lse, lse2, delta, B, H, Lq, Lp, DH, st);
  FaBwdParams p;
  p.B = B; p.H = H; p.Lq = Lq; p.Lk = Lk; p.Lp = Lp;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse2 = lse2; p.delta = delta; p.q = (const bf16*)q; p.dout = (const bf16*)dout;
  p.trace = g_fab_trace; p.trace_cap = g_fab_trace_cap;
  p.dq = (bf16*)dq; p.dk = (bf16*)dk; p.dv = (bf16*)dv; p.err = g_fa_noalloc_status_addr[dev];
  p.kbias = nullptr; p.Lkb = 0;
  return DH == 128 ? launch_bwd<128>(tq, tk, tv, td, p, st) : launch_bwd<64>(tq, tk, tv, td, p, st);
}

}  // extern "C"
