// Skinny GEMM for LoRA down-projections: out[M, N] = alpha * A[M, K] B[N, K]^T with N = 16, 32 or 64
// (the adapter rank) and K in the thousands. The problem reads a whole activation to produce a few
// columns, so it is bandwidth-bound and a 128-row tiling alone leaves most SMs idle (M / 128 CTAs).
// Here the K dimension is split across CTAs as well: grid = (M tiles, splits), each CTA runs a
// TMA -> tcgen05.mma pipeline over its K range into a 32/64-column TMEM accumulator, adds its
// partial into an fp32 workspace with global reductions, and the last CTA of each M tile (an
// arrival counter) converts the finished rows to bf16 and clears the workspace for the next call.
// One launch, no separate zero-fill or conversion kernels.
//
// The reference computes the same product as a separate library GEMM per adapter site
// (FluxLoraLinear::forward_delta, crates/training/src/flux/lora.rs:47-63).
//
// The workspace is one buffer per device shared by all calls: calls whose GPU work may overlap
// (different streams) must not use this entry point concurrently.
#include <cstdlib>

#include "ptx.cuh"
#include "tma_host.h"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int BM = 128, BK = 64, STAGES = 8;

struct SkinnyParams {
  int M, N, K, ldc;
  int ksteps_total, splits;
  float alpha;
  bf16* out;
  float* ws;          // [m_tiles * 128, BN] fp32 partial sums (zero between calls)
  int* counters;      // [m_tiles] arrivals (zero between calls)
  int* err;
};

template <int BN>
__global__ void __launch_bounds__(192, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const SkinnyParams p) {
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + (B_BYTES < 1024 ? 1024 : B_BYTES);
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
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
    tmem_alloc(tmem_slot, TMEM_COLS);
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
        if (!mbar_wait(&empty[s], (uint32_t)(((i / STAGES) & 1) ^ 1))) { atomicExch(p.err, 51); break; }
        uint8_t* st = smem + s * STAGE_BYTES;
        mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
        tma_load_2d(st, &tmA, &full[s], (ks0 + i) * BK, m_tile * BM);
        tma_load_2d(st + A_BYTES, &tmB, &full[s], (ks0 + i) * BK, 0);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_bf16(BM, BN, 0, 0);
      bool ok = true;
      for (int i = 0; i < nks && ok; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(&full[s], (uint32_t)((i / STAGES) & 1))) { atomicExch(p.err, 52); ok = false; break; }
        tc_fence_after();
        const uint32_t a0 = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t da = umma_desc_kmajor(a0, 128), db = umma_desc_kmajor(a0 + A_BYTES, 128);
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk)
          umma_bf16(tmem_base, da + kk * 2, db + kk * 2, idesc, (i | kk) != 0);
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
    if (!ok && lane == 0) atomicExch(p.err, 53);
    tc_fence_after();
    if (ok && nks > 0) {
#pragma unroll
      for (int c = 0; c < BN / 16; ++c) {
        uint32_t r[16];
        tmem_ld16(lane_addr + c * 16, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[c * 16 + j] = __uint_as_float(r[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < BN; ++j) acc[j] = 0.f;
    }
    float* wrow = p.ws + ((size_t)m_tile * BM + r_in) * BN;
    if (p.splits == 1) {
      if (row < p.M) {
        bf16* o = p.out + (size_t)row * p.ldc;
#pragma unroll
        for (int g = 0; g < BN / 8; ++g) {
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = acc[g * 8 + j] * p.alpha;
          *reinterpret_cast<bf16x8*>(o + g * 8) = pack8(v);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < BN; ++j) atomicAdd(wrow + j, acc[j]);
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) *s_last = (atomicAdd(p.counters + m_tile, 1) == p.splits - 1) ? 1 : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*s_last) {
        __threadfence();
        float4* w4 = reinterpret_cast<float4*>(wrow);
#pragma unroll
        for (int g = 0; g < BN / 8; ++g) {
          const float4 x0 = __ldcg(w4 + 2 * g), x1 = __ldcg(w4 + 2 * g + 1);
          const float v[8] = {x0.x * p.alpha, x0.y * p.alpha, x0.z * p.alpha, x0.w * p.alpha,
                              x1.x * p.alpha, x1.y * p.alpha, x1.z * p.alpha, x1.w * p.alpha};
          if (row < p.M) *reinterpret_cast<bf16x8*>(p.out + (size_t)row * p.ldc + g * 8) = pack8(v);
          w4[2 * g] = make_float4(0.f, 0.f, 0.f, 0.f);
          w4[2 * g + 1] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (threadIdx.x == 64) p.counters[m_tile] = 0;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

struct SkinnyState {
  float* ws = nullptr;
  int* counters = nullptr;
  int* err = nullptr;
  long long ws_rows = 0;
  int n_counters = 0;
};
SkinnyState g_sk[64];

template <int BN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const SkinnyParams& p, int m_tiles,
           cudaStream_t st) {
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + (B_BYTES < 1024 ? 1024 : B_BYTES);
  constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_skinny_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM) != cudaSuccess)
      return -5;
    configured = true;
  }
  dim3 grid(m_tiles, p.splits);
  gemm_skinny_kernel<BN><<<grid, 192, SMEM, st>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

int eri_gemm_skinny_check_error() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !g_sk[dev].err) return 0;
  int h = 0;
  cudaMemcpy(&h, g_sk[dev].err, sizeof(int), cudaMemcpyDeviceToHost);
  if (h) cudaMemset(g_sk[dev].err, 0, sizeof(int));
  return h;
}

// a [M, K] (row stride lda elements), b [N, K] (row stride ldb), out [M, N] (row stride ldc), bf16.
// Returns -100 when the shape is outside this kernel's range (caller uses the general GEMM).
int eri_gemm_skinny(const void* a, long long lda, const void* b, long long ldb, void* out, int ldc,
                    int M, int N, int K, float alpha, void* stream) {
  if (!(N == 16 || N == 32 || N == 64) || K < 512 || K % 8 || lda % 8 || ldb % 8 || ldc % 8 || M < 1)
    return -100;
  // Measured on B200 (M = 4608, N = 16): K = 3072 runs 22 us here against 19 us on 128-row tiles
  // alone (the reductions and the arrival counter cost more than the extra CTAs save), K = 15360
  // 45 us against 62 us, K = 21504 55 us against 84 us. Short K therefore stays on the general
  // kernel unless ERI_B200_SKINNY_MIN_K lowers the threshold (tests do).
  static int min_k = -1;
  if (min_k < 0) {
    const char* e = getenv("ERI_B200_SKINNY_MIN_K");
    min_k = e ? atoi(e) : 6144;
  }
  if (K < min_k) return -100;
  if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) return -100;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -100;
  SkinnyState& s = g_sk[dev];
  cudaStream_t st = (cudaStream_t)stream;
  const int m_tiles = (M + BM - 1) / BM;
  const int ksteps = (K + BK - 1) / BK;
  int splits = 296 / m_tiles;
  if (splits > ksteps / 8) splits = ksteps / 8;
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  if (!s.err) {
    if (cudaMalloc(&s.err, sizeof(int)) != cudaSuccess) return -3;
    cudaMemsetAsync(s.err, 0, sizeof(int), st);
  }
  const long long rows = (long long)m_tiles * BM;
  if (splits > 1 && (rows > s.ws_rows || m_tiles > s.n_counters)) {
    // grow the workspace (rare: first call and larger M); the old buffers are released only
    // after the stream has drained, since earlier launches may still use them
    cudaStreamSynchronize(st);
    if (s.ws) cudaFree(s.ws);
    if (s.counters) cudaFree(s.counters);
    s.ws_rows = rows > 8192 ? rows : 8192;
    s.n_counters = (int)(s.ws_rows / BM);
    if (cudaMalloc(&s.ws, (size_t)s.ws_rows * 64 * sizeof(float)) != cudaSuccess) return -3;
    if (cudaMalloc(&s.counters, (size_t)s.n_counters * sizeof(int)) != cudaSuccess) return -3;
    cudaMemsetAsync(s.ws, 0, (size_t)s.ws_rows * 64 * sizeof(float), st);
    cudaMemsetAsync(s.counters, 0, (size_t)s.n_counters * sizeof(int), st);
  }
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t strides[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {BK, BM};
    if (make_tensor_map(&ta, a, 2, dims, strides, box, 128)) return -4;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t strides[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {BK, (uint32_t)N};
    if (make_tensor_map(&tb, b, 2, dims, strides, box, 128)) return -4;
  }
  SkinnyParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ksteps_total = ksteps; p.splits = splits; p.alpha = alpha;
  p.out = (bf16*)out; p.ws = s.ws; p.counters = s.counters; p.err = s.err;
  if (N == 16) return launch<16>(ta, tb, p, m_tiles, st);
  if (N == 32) return launch<32>(ta, tb, p, m_tiles, st);
  return launch<64>(ta, tb, p, m_tiles, st);
}

}  // extern "C"
