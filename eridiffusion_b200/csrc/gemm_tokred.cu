// Token-reduction GEMM for the LoRA weight gradients:
//
//     C[Mg, r] (+)= alpha * A[T, Mg]^T B[T, r]          r = 16, 32 or 64 (the adapter rank)
//
// with both operands token-major as the training step leaves them:
//     dB[N_out, r] += dY[T, N_out]^T H[T, r]                         (C written as is)
//     dA[r, K_in]  += Ts[T, r]^T X[T, K_in] = (X^T Ts)^T             (C written transposed)
// (reference math: FluxLoraLinear backward, crates/training/src/flux/lora.rs:47-63; the reference
// issues two library GEMMs on transposed copies per adapter site).
//
// The product reads a whole activation to produce a few columns, so it is bandwidth-bound. Both
// operands are fed to tcgen05.mma as MN-major tiles straight from their row-major [T, *] layout
// (no transposed copy exists anywhere): the A tile is two 64-column slabs of 64 token rows, the B
// tile one slab whose columns beyond r are zero-filled by the TMA unit (box wider than the tensor),
// so the instruction always runs with N = 64. The token dimension is split across the CTAs of one
// thread-block cluster (grid = Mg / 128 tiles x splits, cluster = 1 x splits, splits in {1, 2, 4, 8}):
// every CTA leaves its fp32 partial tile in its own shared memory, and after one cluster barrier
// each CTA adds a 128 / splits row band of all the partials, read over distributed shared memory in
// split order, optionally adds the existing gradient (beta = 1) and writes bf16. No workspace in
// global memory, no atomics, and a fixed summation order: the result is bit-reproducible run to
// run. One launch per gradient; with programmatic dependent launch its prologue (barriers, TMEM
// allocation, descriptor prefetch) overlaps the tail of the kernel before it.
#include <cstdlib>

#include "ptx.cuh"
#include "tma_host.h"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int BM = 128, BK = 64, BN = 64, STAGES = 4;   // 96 KB of stages: two CTAs per SM
constexpr int A_BYTES = BK * BM * 2;   // two [64 tokens x 64 columns] slabs
constexpr int B_BYTES = BK * BN * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;

struct TokredParams {
  int Mg, r, T, ldc;
  int ksteps_total, splits;
  int transpose_out;   // 1: out is [r, Mg] (row stride ldc), 0: out is [Mg, r]
  int accumulate;      // 1: out += result
  float alpha;
  bf16* out;
  long long dbg_out_bytes;   // extent of `out` in bytes (debug build only; 0: unknown)
  int* err;
};

ERI_DEBUG_BOUNDS_DEFINE(tokred)

__global__ void __launch_bounds__(192, 2)
gemm_tokred_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const TokredParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tile = blockIdx.x, split = (int)cluster_ctarank();   // cluster = (1, splits, 1): rank == blockIdx.y
  const int ks0 = (int)((long long)p.ksteps_total * split / p.splits);
  const int ks1 = (int)((long long)p.ksteps_total * (split + 1) / p.splits);
  const int nks = ks1 - ks0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      griddep_wait();                    // the operands are written by the kernels before this one
      for (int i = 0; i < nks; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(&empty[s], (uint32_t)(((i / STAGES) & 1) ^ 1))) { atomicExch(p.err, 71); break; }
        uint8_t* st = smem + s * STAGE_BYTES;
        const int t0 = (ks0 + i) * BK;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        tma_load_2d(st, &tmA, &full[s], m_tile * BM, t0);
        tma_load_2d(st + BK * 128, &tmA, &full[s], m_tile * BM + 64, t0);
        tma_load_2d(st + A_BYTES, &tmB, &full[s], 0, t0);   // columns >= r arrive as zeros
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_bf16(BM, BN, 1, 1);
      bool ok = true;
      for (int i = 0; i < nks && ok; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(&full[s], (uint32_t)((i / STAGES) & 1))) { atomicExch(p.err, 72); ok = false; break; }
        tc_fence_after();
        const uint32_t a0 = smem_u32(smem + s * STAGE_BYTES), b0 = a0 + A_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk)
          umma_bf16(tmem_base, umma_desc_mn128(a0 + kk * 2048, BK * 128),
                    umma_desc_mn128(b0 + kk * 2048, BK * 128), idesc, (i | kk) != 0);
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    // this CTA's partial tile -> shared memory as [r][128] floats (the stages are free: the commit
    // that armed acc_full covers every MMA that read them)
    const int qd = warp & 3;
    const int r_in = qd * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    const bool ok = nks > 0 ? mbar_wait(acc_full, 0) : true;
    if (!ok && lane == 0) atomicExch(p.err, 73);
    tc_fence_after();
    float* part = reinterpret_cast<float*>(smem);
#pragma unroll
    for (int c = 0; c < BN / 16; ++c) {
      if (c * 16 < p.r) {
        uint32_t rr[16];
        if (ok && nks > 0) {
          tmem_ld16(lane_addr + c * 16, rr);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) rr[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) part[(c * 16 + j) * BM + r_in] = __uint_as_float(rr[j]);
      }
    }
  }
  // every CTA of the cluster has its partial in place (all threads of all CTAs arrive: the roles
  // above always fall through to here, also after a wait that ran out)
  __syncwarp();
  cluster_sync_all();
  if (warp >= 2) {
    griddep_wait();                      // `out` may be read or written only after the kernel before
    const int t = (int)threadIdx.x - 64;
    const int band = BM / p.splits;      // rows of the tile this CTA reduces: 128, 64, 32 or 16
    const uint32_t part_u32 = smem_u32(smem);
    if (p.transpose_out) {
      // item = (column j, 8 consecutive rows): out[j][row .. row + 7] is a contiguous run
      const int items = p.r * (band / 8);
      for (int it = t; it < items; it += 128) {
        const int j = it / (band / 8), g = it % (band / 8);
        const int rl = split * band + g * 8, row = m_tile * BM + rl;
        if (row >= p.Mg) continue;       // Mg is a multiple of 8: a group is inside or outside
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
#pragma unroll 8
        for (int sp = 0; sp < p.splits; ++sp) {
          const uint32_t src = map_to_cta(part_u32 + (uint32_t)(j * BM + rl) * 4u, (uint32_t)sp);
          const float4 lo = ld_shared_cluster_v4(src), hi = ld_shared_cluster_v4(src + 16);
          v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w;
          v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
        }
        bf16* o = p.out + (size_t)j * p.ldc + row;
        if (!ERI_DBG_RANGE(p.out, p.dbg_out_bytes, o, 16, 71)) continue;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= p.alpha;
        if ((reinterpret_cast<uintptr_t>(o) & 15) == 0) {
          if (p.accumulate) {
            float old[8];
            unpack8(*reinterpret_cast<const bf16x8*>(o), old);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] += old[i];
          }
          *reinterpret_cast<bf16x8*>(o) = pack8(v);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float w = v[i];
            if (p.accumulate) w += __bfloat162float(o[i]);
            o[i] = __float2bfloat16(w);
          }
        }
      }
    } else {
      // item = (row, 8 consecutive columns): out[row][j0 .. j0 + 7]
      const int items = band * (p.r / 8);
      for (int it = t; it < items; it += 128) {
        const int rl = split * band + it % band, j0 = (it / band) * 8;
        const int row = m_tile * BM + rl;
        if (row >= p.Mg) continue;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
#pragma unroll 8
        for (int sp = 0; sp < p.splits; ++sp) {
          const uint32_t src = map_to_cta(part_u32 + (uint32_t)(j0 * BM + rl) * 4u, (uint32_t)sp);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] += ld_shared_cluster_f32(src + (uint32_t)(i * BM) * 4u);
        }
        bf16* o = p.out + (size_t)row * p.ldc + j0;
        if (!ERI_DBG_RANGE(p.out, p.dbg_out_bytes, o, 16, 72)) continue;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= p.alpha;
        if (p.accumulate) {
          float old[8];
          unpack8(*reinterpret_cast<const bf16x8*>(o), old);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] += old[i];
        }
        *reinterpret_cast<bf16x8*>(o) = pack8(v);
      }
    }
  }
  // no CTA leaves (and frees its shared memory) while a peer may still read its partial
  __syncwarp();
  cluster_sync_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, BN);
  }
}

struct TokredState {
  int* err = nullptr;
  bool configured = false;
  int sms = 0;
};
TokredState g_tr[64];
int g_tokred_target = 0;   // CTAs per launch to aim for (0: one per SM)

}  // namespace

extern "C" {

int eri_gemm_tokred_check_error() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !g_tr[dev].err) return 0;
  int h = 0;
  cudaMemcpy(&h, g_tr[dev].err, sizeof(int), cudaMemcpyDeviceToHost);
  if (h) cudaMemset(g_tr[dev].err, 0, sizeof(int));
  return h;
}

// Tuning hook: the number of CTAs a launch aims for (0 restores the default).
int eri_gemm_tokred_set_target(int ctas) {
  g_tokred_target = ctas;
  return 0;
}

// a [T, Mg] (row stride lda elements), b [T, r] (row stride ldb), bf16. out: [Mg, r] or, with
// transpose_out, [r, Mg]; row stride ldc. accumulate: out += alpha * a^T b. out_bytes: extent of
// `out` from its pointer (0: unknown), checked by the bounds-checked debug build only.
// Returns -100 when the shape is outside this kernel's range (the caller uses another path).
int eri_gemm_tokred(const void* a, long long lda, const void* b, long long ldb, void* out, int ldc,
                    int T, int Mg, int r, float alpha, int transpose_out, int accumulate,
                    long long out_bytes, void* stream) {
  if (!(r == 16 || r == 32 || r == 64) || T < 64 || Mg < 128 || Mg % 8 || lda % 8 || ldb % 8) return -100;
  if (!transpose_out && ldc % 8) return -100;
  if (((uintptr_t)a | (uintptr_t)b) & 15) return -100;
  if (!transpose_out && ((uintptr_t)out & 15)) return -100;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -100;
  TokredState& s = g_tr[dev];
  cudaStream_t st = (cudaStream_t)stream;
  constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
  if (!s.configured) {
    if (cudaFuncSetAttribute(gemm_tokred_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) !=
        cudaSuccess)
      return -5;
    cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, dev);
    s.configured = true;
  }
  if (!s.err) {
    if (cudaMalloc(&s.err, sizeof(int)) != cudaSuccess) return -3;
    cudaMemsetAsync(s.err, 0, sizeof(int), st);
  }
  const int m_tiles = (Mg + BM - 1) / BM;
  const int ksteps = (T + BK - 1) / BK;
  // The token splits of one tile form a cluster (1, 2, 4 or 8 CTAs). Enough CTAs to cover the SMs,
  // but at least four K steps each so that a CTA's prologue is paid for.
  const int target = g_tokred_target > 0 ? g_tokred_target : s.sms;
  int splits = 1;
  while (splits < 8 && m_tiles * splits < target && ksteps / (splits * 2) >= 4) splits *= 2;
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {(uint64_t)Mg, (uint64_t)T};
    uint64_t strides[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {64, BK};
    if (make_tensor_map(&ta, a, 2, dims, strides, box, 128)) return -4;
  }
  {
    // the box is 64 columns wide whatever r is: columns beyond the tensor are zero-filled
    uint64_t dims[2] = {(uint64_t)r, (uint64_t)T};
    uint64_t strides[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {BN, BK};
    if (make_tensor_map(&tb, b, 2, dims, strides, box, 128)) return -6;
  }
  TokredParams p;
  p.Mg = Mg; p.r = r; p.T = T; p.ldc = ldc; p.ksteps_total = ksteps; p.splits = splits;
  p.transpose_out = transpose_out; p.accumulate = accumulate; p.alpha = alpha;
  p.dbg_out_bytes = out_bytes;
  p.out = (bf16*)out; p.err = s.err;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(m_tiles, splits);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = st;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = splits; at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 2;
  return (int)cudaLaunchKernelEx(&cfg, gemm_tokred_kernel, ta, tb, p);
}

}  // extern "C"

ERI_DEBUG_BOUNDS_EXPORT(tokred)
