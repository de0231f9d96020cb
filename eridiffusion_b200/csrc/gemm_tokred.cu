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
// so the instruction always runs with N = 64. The token dimension is split across CTAs
// (grid = Mg / 128 tiles x splits); every CTA stores its partial tile into its own slot of an fp32
// workspace (plain coalesced stores, no atomics) and the last CTA of a tile (an arrival counter)
// adds the slots in split order, optionally adds the existing gradient (beta = 1) and writes bf16.
// The summation order is fixed, so the result is bit-reproducible run to run. One launch per
// gradient.
//
// The workspace is one buffer per device shared by all calls: calls whose GPU work may overlap
// (different streams) must not use this entry point concurrently.
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
  float* ws;           // [m_tiles][splits][r][128] fp32 partial tiles (every slot is rewritten per call)
  int* counters;       // [m_tiles] arrivals (zero between calls)
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
  int* s_last = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tile = blockIdx.x, split = blockIdx.y;
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
    const int qd = warp & 3;
    const int r_in = qd * 32 + lane;
    const int row = m_tile * BM + r_in;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    float acc[BN];
    bool ok = nks > 0 ? mbar_wait(acc_full, 0) : true;
    if (!ok && lane == 0) atomicExch(p.err, 73);
    tc_fence_after();
    if (ok && nks > 0) {
#pragma unroll
      for (int c = 0; c < BN / 16; ++c) {
        uint32_t rr[16];
        tmem_ld16(lane_addr + c * 16, rr);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[c * 16 + j] = __uint_as_float(rr[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < BN; ++j) acc[j] = 0.f;
    }
    // slot of (tile, split): [r][128] floats, lanes along the row index -> coalesced
    const size_t slot_elems = (size_t)p.r * BM;
    float* tile_ws = p.ws + (size_t)m_tile * p.splits * slot_elems;
    if (p.splits > 1) {
      float* mine = tile_ws + (size_t)split * slot_elems + r_in;
#pragma unroll
      for (int j = 0; j < BN; ++j)
        if (j < p.r) __stcg(mine + (size_t)j * BM, acc[j]);
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) *s_last = (atomicAdd(p.counters + m_tile, 1) == p.splits - 1) ? 1 : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    if (p.splits == 1 || *s_last) {
      if (p.splits > 1) {
        __threadfence();
#pragma unroll
        for (int j = 0; j < BN; ++j) acc[j] = 0.f;
        for (int sp = 0; sp < p.splits; ++sp) {
          const float* src = tile_ws + (size_t)sp * slot_elems + r_in;
#pragma unroll
          for (int j = 0; j < BN; ++j)
            if (j < p.r) acc[j] += __ldcg(src + (size_t)j * BM);
        }
        if (threadIdx.x == 64) p.counters[m_tile] = 0;
      }
      if (row < p.Mg) {
        if (p.transpose_out) {
          // consecutive threads hold consecutive rows: column j of the tile is a contiguous run
#pragma unroll
          for (int j = 0; j < BN; ++j)
            if (j < p.r) {
              bf16* o = p.out + (size_t)j * p.ldc + row;
              if (!ERI_DBG_RANGE(p.out, p.dbg_out_bytes, o, 2, 71)) continue;
              float v = acc[j] * p.alpha;
              if (p.accumulate) v += __bfloat162float(*o);
              *o = __float2bfloat16(v);
            }
        } else {
          bf16* o = p.out + (size_t)row * p.ldc;
#pragma unroll
          for (int g = 0; g < BN / 8; ++g)
            if (g * 8 < p.r && ERI_DBG_RANGE(p.out, p.dbg_out_bytes, o + g * 8, 16, 72)) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = acc[g * 8 + j] * p.alpha;
              if (p.accumulate) {
                float old[8];
                unpack8(*reinterpret_cast<const bf16x8*>(o + g * 8), old);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += old[j];
              }
              *reinterpret_cast<bf16x8*>(o + g * 8) = pack8(v);
            }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, BN);
  }
}

struct TokredState {
  float* ws = nullptr;
  int* counters = nullptr;
  int* err = nullptr;
  long long ws_elems = 0;
  int n_counters = 0;
  bool configured = false;
  int sms = 0;
};
TokredState g_tr[64];
int g_tokred_target = 0;   // CTAs per launch to aim for (0: four per SM)

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
  const int m_tiles = (Mg + BM - 1) / BM;
  const int ksteps = (T + BK - 1) / BK;
  // About one CTA per SM measured best (every extra split adds a partial tile to store and re-read);
  // at least four K steps per CTA pay for its prologue.
  const int target = g_tokred_target > 0 ? g_tokred_target : s.sms;
  int splits = (target + m_tiles / 2) / m_tiles;
  if (splits > ksteps / 4) splits = ksteps / 4;
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  if (!s.err) {
    if (cudaMalloc(&s.err, sizeof(int)) != cudaSuccess) return -3;
    cudaMemsetAsync(s.err, 0, sizeof(int), st);
  }
  const long long need = splits > 1 ? (long long)m_tiles * splits * r * BM : 0;
  if (need > s.ws_elems || m_tiles > s.n_counters) {
    // grow the workspace (rare: first call and larger problems); the old buffers are released only
    // after the stream has drained, since earlier launches may still use them
    cudaStreamSynchronize(st);
    if (s.ws) cudaFree(s.ws);
    if (s.counters) cudaFree(s.counters);
    s.ws_elems = need > (8ll << 20) ? need : (8ll << 20);
    s.n_counters = m_tiles > 4096 ? m_tiles : 4096;
    if (cudaMalloc(&s.ws, (size_t)s.ws_elems * sizeof(float)) != cudaSuccess) return -3;
    if (cudaMalloc(&s.counters, (size_t)s.n_counters * sizeof(int)) != cudaSuccess) return -3;
    cudaMemsetAsync(s.counters, 0, (size_t)s.n_counters * sizeof(int), st);
  }
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
  p.out = (bf16*)out; p.ws = s.ws; p.counters = s.counters; p.err = s.err;
  dim3 grid(m_tiles, splits);
  gemm_tokred_kernel<<<grid, 192, SMEM, st>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

}  // extern "C"

ERI_DEBUG_BOUNDS_EXPORT(tokred)
