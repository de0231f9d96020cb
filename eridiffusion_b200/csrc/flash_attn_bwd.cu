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
  bf16* dq;              // [B, Lq, H, DH]
  bf16* dk;              // [B, Lk, H, DH]
  bf16* dv;
  int* err;
};

constexpr int T = 128;  // tile edge (queries and keys)

__global__ void fa_bwd_prep_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dout,
                                   const float* __restrict__ lse, float* __restrict__ lse2,
                                   float* __restrict__ delta, int B, int H, int Lq, int Lp, int DH) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int total = B * H * Lp;
  if (warp >= total) return;
  const int l = warp % Lp, h = (warp / Lp) % H, b = warp / (Lp * H);
  if (l >= Lq) {
    if (lane == 0) {
      lse2[warp] = INFINITY;
      delta[warp] = 0.f;
    }
    return;
  }
  const size_t base = (((size_t)b * Lq + l) * H + h) * DH;
  float acc = 0.f;
  for (int d = lane * 2; d < DH; d += 64) {
    float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + base + d));
    float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dout + base + d));
    acc += a.x * g.x + a.y * g.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    delta[warp] = acc;
    lse2[warp] = lse[((size_t)b * H + h) * Lq + l] * 1.4426950408889634f;
  }
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ------------------------------------------------------------------------------------- dK, dV
template <int DH, int POLY>
__global__ void __launch_bounds__(192, 1)
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
  uint64_t* sp_full = bars + 5;    // [2] one per 64-query half
  uint64_t* pds_ready = bars + 7;  // [2]
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
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sp_full[s], 1);
      mbar_init(&pds_ready[s], 4);
    }
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
      // Software pipeline over 64-query halves: while the softmax warps turn one half of
      // S^T / dP^T into P^T / dS^T, the tensor pipe runs the other half's products, and the
      // next tile's first half is issued before this tile's second half is consumed.
      const uint32_t idesc_s = umma_idesc_bf16(T, 64, 0, 0);
      const uint32_t idesc_g = umma_idesc_bf16(T, DH, 0, 1);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV);
      const uint32_t aQ0 = smem_u32(sQ), aDO0 = smem_u32(sDO);
      auto issue_sdp = [&](int st, int hf) {  // S^T and dP^T for queries [64 hf, 64 hf + 64)
        const uint32_t aQ = aQ0 + st * TILE_BYTES + hf * 8192, aDO = aDO0 + st * TILE_BYTES + hf * 8192;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          const uint64_t da = umma_desc_kmajor(aK + c * CHUNK_BYTES, 128);
          const uint64_t db = umma_desc_kmajor(aQ + c * CHUNK_BYTES, 128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(tmem_base + S_COL + hf * 64, da + kk * 2, db + kk * 2, idesc_s, (c | kk) != 0);
        }
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          const uint64_t da = umma_desc_kmajor(aV + c * CHUNK_BYTES, 128);
          const uint64_t db = umma_desc_kmajor(aDO + c * CHUNK_BYTES, 128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(tmem_base + DP_COL + hf * 64, da + kk * 2, db + kk * 2, idesc_s, (c | kk) != 0);
        }
        umma_commit(&sp_full[hf]);
      };
      auto issue_dvdk = [&](int st, int hf, bool first) {
        const uint32_t aQ = aQ0 + st * TILE_BYTES, aDO = aDO0 + st * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t dbo = umma_desc_mn128(aDO + (hf * 4 + kk) * 2048, CHUNK_BYTES);
          umma_bf16_ts(tmem_base + DV_COL, tmem_base + S_COL + hf * 64 + kk * 8, dbo, idesc_g,
                       !first || kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t dbq = umma_desc_mn128(aQ + (hf * 4 + kk) * 2048, CHUNK_BYTES);
          umma_bf16_ts(tmem_base + DK_COL, tmem_base + DP_COL + hf * 64 + kk * 8, dbq, idesc_g,
                       !first || kk != 0);
        }
      };
      bool ok = mbar_wait(kv_full, 0);
      if (!ok) atomicExch(p.err, 22);
      if (ok && !mbar_wait(&qdo_full[0], 0)) { atomicExch(p.err, 23); ok = false; }
      if (ok) {
        tc_fence_after();
        issue_sdp(0, 0);
        issue_sdp(0, 1);
      }
      for (int i = 0; i < nq && ok; ++i) {
        const int s = i & 1;
        const uint32_t par = (uint32_t)(i & 1);
        const bool more = i + 1 < nq;
        if (!mbar_wait(&pds_ready[0], par)) { atomicExch(p.err, 24); ok = false; break; }
        tc_fence_after();
        issue_dvdk(s, 0, i == 0);
        if (more) {
          if (!mbar_wait(&qdo_full[s ^ 1], (uint32_t)(((i + 1) >> 1) & 1))) {
            atomicExch(p.err, 23);
            ok = false;
            break;
          }
          tc_fence_after();
          issue_sdp(s ^ 1, 0);
        }
        if (!mbar_wait(&pds_ready[1], par)) { atomicExch(p.err, 27); ok = false; break; }
        tc_fence_after();
        issue_dvdk(s, 1, false);
        umma_commit(&qdo_empty[s]);
        if (more) issue_sdp(s ^ 1, 1);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int qd = warp & 3;
    const int tid = threadIdx.x - 64;  // 0..127
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    const size_t stat_base = ((size_t)b * p.H + h) * p.Lp;
    bool ok = true;
    for (int i = 0; i < nq; ++i) {
      const int s = i & 1;
      s_lse[s * T + tid] = -p.lse2[stat_base + i * T + tid];
      s_delta[s * T + tid] = p.delta[stat_base + i * T + tid];
      named_bar_sync(1, 128);
      // s_lse holds -lse2 so that one packed fma gives s * c - lse2 for two queries
      const float4* ls4 = reinterpret_cast<const float4*>(s_lse + s * T);
      const float4* dl4 = reinterpret_cast<const float4*>(s_delta + s * T);
      const f32x2 sc2 = f2_pack(p.scale_log2, p.scale_log2);
#pragma unroll 1
      for (int hf = 0; hf < 2 && ok; ++hf) {
        if (!mbar_wait(&sp_full[hf], (uint32_t)(i & 1))) {
          if (lane == 0) atomicExch(p.err, 25);
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
          const int c = hf * 2 + cc;  // 32-query chunk
          uint32_t r[32], g[32];
          tmem_ld32(lane_addr + S_COL + c * 32, r);
          tmem_ld32(lane_addr + DP_COL + c * 32, g);
          tmem_ld_wait();
          uint32_t pk[16], dk_[16];
#pragma unroll
          for (int x4 = 0; x4 < 8; ++x4) {
            const float4 nl = ls4[c * 8 + x4];
            const float4 dl = dl4[c * 8 + x4];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const int x = 2 * x4 + hh;
              const f32x2 nl2 = hh ? f2_pack(nl.z, nl.w) : f2_pack(nl.x, nl.y);
              const f32x2 dl2 = hh ? f2_pack(dl.z, dl.w) : f2_pack(dl.x, dl.y);
              f32x2 v = f2_fma(f2_pack_bits(r[2 * x], r[2 * x + 1]), sc2, nl2);
              if (x < 16 - POLY) {
                float lo, hi;
                f2_unpack(v, lo, hi);
                v = f2_pack(ex2_mufu(lo), ex2_mufu(hi));
              } else {
                v = ex2_poly2(v);
              }
              const f32x2 d = f2_mul(v, f2_sub(f2_pack_bits(g[2 * x], g[2 * x + 1]), dl2));
              pk[x] = f2_to_bf162(v);
              dk_[x] = f2_to_bf162(d);
            }
          }
          // packed bf16 P^T / dS^T of this half start at the half's own first column
          tmem_st16(lane_addr + S_COL + hf * 64 + cc * 16, pk);
          tmem_st16(lane_addr + DP_COL + hf * 64 + cc * 16, dk_);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pds_ready[hf]);
      }
      if (!ok) break;
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
      for (int c = 0; c < DH / 32; ++c) {
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
template <int DH, int POLY>
__global__ void __launch_bounds__(192, 1)
fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const FaBwdParams p) {
  constexpr int CHUNKS = DH / 64;
  constexpr int CHUNK_BYTES = T * 128;
  constexpr int TILE_BYTES = CHUNK_BYTES * CHUNKS;
  constexpr uint32_t S_COL = 0, DP_COL = 128, DQ_COL = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + TILE_BYTES;
  uint8_t* sK = sDO + TILE_BYTES;      // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;   // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * TILE_BYTES);
  uint64_t* qdo_full = bars + 0;
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* sp_full = bars + 5;   // [2] one per 64-key half
  uint64_t* ds_ready = bars + 7;  // [2]
  uint64_t* acc_done = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * T, h = blockIdx.y, b = blockIdx.z;
  const int nkv = (p.Lk + T - 1) / T;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sp_full[s], 1);
      mbar_init(&ds_ready[s], 4);
    }
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
      mbar_expect_tx(qdo_full, 2 * TILE_BYTES);
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        tma_load_3d(sQ + c * CHUNK_BYTES, &tmQ, qdo_full, h * DH + c * 64, q0, b);
        tma_load_3d(sDO + c * CHUNK_BYTES, &tmDO, qdo_full, h * DH + c * 64, q0, b);
      }
      for (int j = 0; j < nkv; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], (uint32_t)(((j >> 1) & 1) ^ 1))) { atomicExch(p.err, 31); break; }
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
      // Same half-tile software pipeline as the dK/dV kernel, split over 64-key halves.
      const uint32_t idesc_s = umma_idesc_bf16(T, 64, 0, 0);
      const uint32_t idesc_g = umma_idesc_bf16(T, DH, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aDO = smem_u32(sDO);
      const uint32_t aK0 = smem_u32(sK), aV0 = smem_u32(sV);
      auto issue_sdp = [&](int st, int hf) {  // S and dP for keys [64 hf, 64 hf + 64)
        const uint32_t aK = aK0 + st * TILE_BYTES + hf * 8192, aV = aV0 + st * TILE_BYTES + hf * 8192;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          const uint64_t da = umma_desc_kmajor(aQ + c * CHUNK_BYTES, 128);
          const uint64_t db = umma_desc_kmajor(aK + c * CHUNK_BYTES, 128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(tmem_base + S_COL + hf * 64, da + kk * 2, db + kk * 2, idesc_s, (c | kk) != 0);
        }
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          const uint64_t da = umma_desc_kmajor(aDO + c * CHUNK_BYTES, 128);
          const uint64_t db = umma_desc_kmajor(aV + c * CHUNK_BYTES, 128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(tmem_base + DP_COL + hf * 64, da + kk * 2, db + kk * 2, idesc_s, (c | kk) != 0);
        }
        umma_commit(&sp_full[hf]);
      };
      auto issue_dq = [&](int st, int hf, bool first) {
        const uint32_t aK = aK0 + st * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t dbk = umma_desc_mn128(aK + (hf * 4 + kk) * 2048, CHUNK_BYTES);
          umma_bf16_ts(tmem_base + DQ_COL, tmem_base + DP_COL + hf * 64 + kk * 8, dbk, idesc_g,
                       !first || kk != 0);
        }
      };
      bool ok = mbar_wait(qdo_full, 0);
      if (!ok) atomicExch(p.err, 32);
      if (ok && !mbar_wait(&kv_full[0], 0)) { atomicExch(p.err, 33); ok = false; }
      if (ok) {
        tc_fence_after();
        issue_sdp(0, 0);
        issue_sdp(0, 1);
      }
      for (int j = 0; j < nkv && ok; ++j) {
        const int s = j & 1;
        const uint32_t par = (uint32_t)(j & 1);
        const bool more = j + 1 < nkv;
        if (!mbar_wait(&ds_ready[0], par)) { atomicExch(p.err, 34); ok = false; break; }
        tc_fence_after();
        issue_dq(s, 0, j == 0);
        if (more) {
          if (!mbar_wait(&kv_full[s ^ 1], (uint32_t)(((j + 1) >> 1) & 1))) {
            atomicExch(p.err, 33);
            ok = false;
            break;
          }
          tc_fence_after();
          issue_sdp(s ^ 1, 0);
        }
        if (!mbar_wait(&ds_ready[1], par)) { atomicExch(p.err, 37); ok = false; break; }
        tc_fence_after();
        issue_dq(s, 1, false);
        umma_commit(&kv_empty[s]);
        if (more) issue_sdp(s ^ 1, 1);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int qd = warp & 3;
    const int row = q0 + qd * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    const size_t stat = ((size_t)b * p.H + h) * p.Lp + row;  // row < Lp always
    const float lse2 = p.lse2[stat], delta = p.delta[stat];
    bool ok = true;
    const f32x2 sc2 = f2_pack(p.scale_log2, p.scale_log2);
    const f32x2 nl2 = f2_pack(-lse2, -lse2);
    const f32x2 dl2 = f2_pack(delta, delta);
    for (int j = 0; j < nkv && ok; ++j) {
      const int kv_left = p.Lk - j * T;
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {
        if (!mbar_wait(&sp_full[hf], (uint32_t)(j & 1))) {
          if (lane == 0) atomicExch(p.err, 35);
          ok = false;
          break;
        }
        tc_fence_after();
        if (kv_left >= T) {
#pragma unroll 1
          for (int cc = 0; cc < 2; ++cc) {
            const int c = hf * 2 + cc;
            uint32_t r[32], g[32];
            tmem_ld32(lane_addr + S_COL + c * 32, r);
            tmem_ld32(lane_addr + DP_COL + c * 32, g);
            tmem_ld_wait();
            uint32_t dk_[16];
#pragma unroll
            for (int x = 0; x < 16; ++x) {
              f32x2 v = f2_fma(f2_pack_bits(r[2 * x], r[2 * x + 1]), sc2, nl2);
              if (x < 16 - POLY) {
                float lo, hi;
                f2_unpack(v, lo, hi);
                v = f2_pack(ex2_mufu(lo), ex2_mufu(hi));
              } else {
                v = ex2_poly2(v);
              }
              dk_[x] = f2_to_bf162(f2_mul(v, f2_sub(f2_pack_bits(g[2 * x], g[2 * x + 1]), dl2)));
            }
            tmem_st16(lane_addr + DP_COL + hf * 64 + cc * 16, dk_);
          }
        } else {
#pragma unroll 1
          for (int cc = 0; cc < 2; ++cc) {
            const int c = hf * 2 + cc;
            uint32_t r[32], g[32];
            tmem_ld32(lane_addr + S_COL + c * 32, r);
            tmem_ld32(lane_addr + DP_COL + c * 32, g);
            tmem_ld_wait();
            uint32_t dk_[16];
#pragma unroll
            for (int x = 0; x < 16; ++x) {
              float p0 = exp2f(fmaf(__uint_as_float(r[2 * x]), p.scale_log2, -lse2));
              float p1 = exp2f(fmaf(__uint_as_float(r[2 * x + 1]), p.scale_log2, -lse2));
              if (c * 32 + 2 * x >= kv_left) p0 = 0.f;
              if (c * 32 + 2 * x + 1 >= kv_left) p1 = 0.f;
              float d0 = p0 * (__uint_as_float(g[2 * x]) - delta);
              float d1 = p1 * (__uint_as_float(g[2 * x + 1]) - delta);
              dk_[x] = pack_bf162(d0, d1);
            }
            tmem_st16(lane_addr + DP_COL + hf * 64 + cc * 16, dk_);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ds_ready[hf]);
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
      for (int c = 0; c < DH / 32; ++c) {
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

int* g_fab_err = nullptr;

int make_map(CUtensorMap* m, const void* ptr, int B, int L, int H, int DH) {
  uint64_t dims[3] = {(uint64_t)H * DH, (uint64_t)L, (uint64_t)B};
  uint64_t strides[2] = {(uint64_t)H * DH * 2, (uint64_t)L * H * DH * 2};
  uint32_t box[3] = {64, 128, 1};
  return make_tensor_map(m, ptr, 3, dims, strides, box, 128);
}

template <int DH, int POLY>
int launch_bwd_v(const CUtensorMap& q, const CUtensorMap& k, const CUtensorMap& v,
                 const CUtensorMap& d, const FaBwdParams& p, cudaStream_t st) {
  constexpr int SMEM = 6 * 128 * 128 * (DH / 64) + 2048 + 1024 + 128;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(fa_bwd_dkdv_kernel<DH, POLY>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return -5;
    if (cudaFuncSetAttribute(fa_bwd_dq_kernel<DH, POLY>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return -5;
    configured = true;
  }
  dim3 g1((p.Lk + T - 1) / T, p.H, p.B), g2((p.Lq + T - 1) / T, p.H, p.B);
  fa_bwd_dkdv_kernel<DH, POLY><<<g1, 192, SMEM, st>>>(q, k, v, d, p);
  fa_bwd_dq_kernel<DH, POLY><<<g2, 192, SMEM, st>>>(q, k, v, d, p);
  return (int)cudaGetLastError();
}

// Pairs (of every 16) whose 2^x runs on the FMA pipe instead of the special-function unit;
// ERI_B200_FA_BWD_POLY = 0, 4 or 8 (read once, no allocation).
int bwd_poly_pairs() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("ERI_B200_FA_BWD_POLY");
    v = e ? atoi(e) : 8;
    if (v != 0 && v != 4 && v != 8) v = 8;
  }
  return v;
}

template <int DH>
int launch_bwd(const CUtensorMap& q, const CUtensorMap& k, const CUtensorMap& v,
               const CUtensorMap& d, const FaBwdParams& p, cudaStream_t st) {
  const int poly = bwd_poly_pairs();
  if (poly == 0) return launch_bwd_v<DH, 0>(q, k, v, d, p, st);
  if (poly == 8) return launch_bwd_v<DH, 8>(q, k, v, d, p, st);
  return launch_bwd_v<DH, 4>(q, k, v, d, p, st);
}

}  // namespace

extern "C" {

int eri_fa_bwd_check_error() {
  if (!g_fab_err) return 0;
  int h = 0;
  cudaMemcpy(&h, g_fab_err, sizeof(int), cudaMemcpyDeviceToHost);
  if (h) cudaMemset(g_fab_err, 0, sizeof(int));
  return h;
}

// All tensors contiguous bf16 [B, L, H, DH]; lse [B, H, Lq] fp32 from the forward.
// Scratch supplied by the caller: lse2 and delta, each [B, H, Lp] fp32 with Lp = ceil(Lq/128)*128.
int eri_flash_attn_bwd(const void* dout, const void* q, const void* k, const void* v,
                       const void* out, const float* lse, float* lse2, float* delta, void* dq,
                       void* dk, void* dv, int B, int H, int Lq, int Lk, int DH, float scale,
                       void* stream) {
  if (DH != 64 && DH != 128) return -1;
  if (Lq < 128 || Lk < 128) return -2;
  if (!g_fab_err) {
    if (cudaMalloc(&g_fab_err, sizeof(int)) != cudaSuccess) return -3;
    cudaMemset(g_fab_err, 0, sizeof(int));
  }
  cudaStream_t st = (cudaStream_t)stream;
  const int Lp = (Lq + T - 1) / T * T;
  {
    const long long warps = (long long)B * H * Lp;
    const int block = 256;
    const long long grid = (warps * 32 + block - 1) / block;
    fa_bwd_prep_kernel<<<(unsigned)grid, block, 0, st>>>((const bf16*)out, (const bf16*)dout, lse,
                                                         lse2, delta, B, H, Lq, Lp, DH);
  }
  CUtensorMap tq, tk, tv, td;
  if (make_map(&tq, q, B, Lq, H, DH) || make_map(&tk, k, B, Lk, H, DH) ||
      make_map(&tv, v, B, Lk, H, DH) || make_map(&td, dout, B, Lq, H, DH))
    return -4;
  FaBwdParams p;
  p.B = B; p.H = H; p.Lq = Lq; p.Lk = Lk; p.Lp = Lp;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse2 = lse2; p.delta = delta;
  p.dq = (bf16*)dq; p.dk = (bf16*)dk; p.dv = (bf16*)dv; p.err = g_fab_err;
  return DH == 128 ? launch_bwd<128>(tq, tk, tv, td, p, st) : launch_bwd<64>(tq, tk, tv, td, p, st);
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
  {
    const int block = 256;
    const long long grid = (rows * 32 + block - 1) / block;
    fa_bwd_prep_kernel<<<(unsigned)grid, block, 0, st>>>((const bf16*)out, (const bf16*)dout, lse,
                                                         lse2, delta, B, H, Lq, Lp, DH);
  }
  CUtensorMap tq, tk, tv, td;
  if (encode_map_uncached(&tq, q, B, Lq, H, DH) || encode_map_uncached(&tk, k, B, Lk, H, DH) ||
      encode_map_uncached(&tv, v, B, Lk, H, DH) || encode_map_uncached(&td, dout, B, Lq, H, DH))
    return -4;
  FaBwdParams p;
  p.B = B; p.H = H; p.Lq = Lq; p.Lk = Lk; p.Lp = Lp;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse2 = lse2; p.delta = delta;
  p.dq = (bf16*)dq; p.dk = (bf16*)dk; p.dv = (bf16*)dv; p.err = g_fa_noalloc_status_addr[dev];
  return DH == 128 ? launch_bwd<128>(tq, tk, tv, td, p, st) : launch_bwd<64>(tq, tk, tv, td, p, st);
}

}  // extern "C"
