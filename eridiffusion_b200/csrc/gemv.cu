// Small-M linear: y[m, n] = f(x[m, :]) . W[n, :] + b[n] for M <= 8 rows (conditioning vectors).
// Used for adaLN modulation (f = SiLU), the time / guidance / pooled-text embedders and their
// backward (d_x = d_y W, via the transposed launch below). The op is bound by one pass over W,
// so each warp streams one weight row with 16-byte loads and keeps M accumulators in registers.
// Reference call site: `modulation` = SiLU + GEMM + bias + six narrows
// (crates/training/src/flux/runtime.rs:401-463).
#include "ptx.cuh"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kMaxM = 8;

template <int M>
__global__ void gemv_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                            const bf16* __restrict__ bias, bf16* __restrict__ y, int N, int K,
                            int ldx, int ldw, int ldy, int silu_in, int act_out) {
  extern __shared__ float xs[];  // [M, K] fp32, input activation applied
  for (int i = threadIdx.x; i < M * K; i += blockDim.x) {
    int m = i / K, k = i - m * K;
    float v = __bfloat162float(x[(size_t)m * ldx + k]);
    xs[i] = silu_in ? silu_f(v) : v;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int kv = K >> 3;
  for (int n = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); n < N;
       n += gridDim.x * warps_per_cta) {
    const bf16x8* wr = reinterpret_cast<const bf16x8*>(w + (size_t)n * ldw);
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    for (int v = lane; v < kv; v += 32) {
      float wf[8];
      unpack8(wr[v], wf);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float4* xp = reinterpret_cast<const float4*>(xs + (size_t)m * K + v * 8);
        float4 a = xp[0], b = xp[1];
        acc[m] += wf[0] * a.x + wf[1] * a.y + wf[2] * a.z + wf[3] * a.w + wf[4] * b.x +
                  wf[5] * b.y + wf[6] * b.z + wf[7] * b.w;
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = warp_sum(acc[m]);
    if (lane == 0) {
      float bb = bias ? __bfloat162float(bias[n]) : 0.f;
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float v = acc[m] + bb;
        if (act_out == 1) v = silu_f(v);
        y[(size_t)m * ldy + n] = __float2bfloat16(v);
      }
    }
  }
}

}  // namespace

extern "C" int eri_gemv_bf16(const void* x, const void* w, const void* bias, void* y, int M, int N,
                             int K, int ldx, int ldw, int ldy, int silu_in, int act_out,
                             void* stream) {
  if (M < 1 || M > kMaxM || K % 8 || ldw % 8) return -1;
  const size_t smem = (size_t)M * K * sizeof(float);
  if (smem > 200 * 1024) return -2;
  const int block = 256;
  int grid = (N + 7) / 8;
  if (grid > 148 * 4) grid = 148 * 4;
  cudaStream_t st = (cudaStream_t)stream;
#define ERI_GEMV_CASE(MM)                                                                      \
  case MM: {                                                                                   \
    static bool cfg = false;                                                                   \
    if (!cfg) {                                                                                \
      cudaFuncSetAttribute(gemv_kernel<MM>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                           200 * 1024);                                                        \
      cfg = true;                                                                              \
    }                                                                                          \
    gemv_kernel<MM><<<grid, block, smem, st>>>((const bf16*)x, (const bf16*)w,                 \
                                               (const bf16*)bias, (bf16*)y, N, K, ldx, ldw,    \
                                               ldy, silu_in, act_out);                         \
    break;                                                                                     \
  }
  switch (M) {
    ERI_GEMV_CASE(1)
    ERI_GEMV_CASE(2)
    ERI_GEMV_CASE(3)
    ERI_GEMV_CASE(4)
    ERI_GEMV_CASE(5)
    ERI_GEMV_CASE(6)
    ERI_GEMV_CASE(7)
    ERI_GEMV_CASE(8)
  }
#undef ERI_GEMV_CASE
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Backward of the small-M linear (T <= 8 rows of dy).
//
//   weight gradient  dW[n, k] (+)= sum_t dy[t, n] * x[t, k]        bound by writing dW once
//   input gradient   part[s, t, k] = sum_{n in split s} dy[t, n] * W[n, k]   bound by reading W once;
//                    the caller adds the `splits` partial planes (fixed order: deterministic)
//
// Reference: the modulation / embedder linears' backward is composed from tensor ops
// (crates/training/src/flux/runtime.rs:401-463 forward; gradients through the autograd tape).
namespace {

__global__ void __launch_bounds__(128) rows_wgrad_kernel(const bf16* __restrict__ dy, int ldy, const bf16* __restrict__ x,
                                                         int ldx, bf16* __restrict__ dw, int ldw, int T, int N, int K,
                                                         int accumulate, float scale) {
  // a CTA owns 128 x 8 columns of dW and walks its rows in chunks of kChunk: the chunk's dy values are
  // staged in shared memory first, so that the row loop has no dependent global load in it
  constexpr int kChunk = 64;
  __shared__ float sdy[kMaxM][kChunk];
  const int kv = blockIdx.x * blockDim.x + threadIdx.x;   // 8 columns per thread
  const bool live = kv * 8 < K;
  float xf[kMaxM][8];
#pragma unroll
  for (int t = 0; t < kMaxM; ++t) {
    if (t < T && live) unpack8(*reinterpret_cast<const bf16x8*>(x + (size_t)t * ldx + kv * 8), xf[t]);
  }
  for (int n0 = blockIdx.y * kChunk; n0 < N; n0 += gridDim.y * kChunk) {
    const int nc = min(kChunk, N - n0);
    __syncthreads();
    for (int i = threadIdx.x; i < T * kChunk; i += blockDim.x) {
      const int t = i / kChunk, j = i - t * kChunk;
      sdy[t][j] = j < nc ? __bfloat162float(dy[(size_t)t * ldy + n0 + j]) * scale : 0.f;
    }
    __syncthreads();
    if (!live) continue;
#pragma unroll 4
    for (int j = 0; j < nc; ++j) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int t = 0; t < kMaxM; ++t) {
        if (t < T) {
          const float d = sdy[t][j];
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] = fmaf(d, xf[t][q], acc[q]);
        }
      }
      bf16x8* o = reinterpret_cast<bf16x8*>(dw + (size_t)(n0 + j) * ldw + kv * 8);
      if (accumulate) {
        float old[8];
        unpack8(*o, old);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += old[q];
      }
      *o = pack8(acc);
    }
  }
}

template <int T>
__global__ void rows_dgrad_kernel(const bf16* __restrict__ dy, int ldy, const bf16* __restrict__ w,
                                  int ldw, float* __restrict__ part, int N, int K, int rows_per_split) {
  const int kv = blockIdx.x * blockDim.x + threadIdx.x;
  if (kv * 8 >= K) return;
  const int n0 = blockIdx.y * rows_per_split;
  const int n1 = min(N, n0 + rows_per_split);
  float acc[T][8];
#pragma unroll
  for (int t = 0; t < T; ++t)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[t][j] = 0.f;
#pragma unroll 4
  for (int n = n0; n < n1; ++n) {
    float wf[8];
    unpack8(*reinterpret_cast<const bf16x8*>(w + (size_t)n * ldw + kv * 8), wf);
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const float d = __bfloat162float(dy[(size_t)t * ldy + n]);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[t][j] = fmaf(d, wf[j], acc[t][j]);
    }
  }
#pragma unroll
  for (int t = 0; t < T; ++t) {
    float4* o = reinterpret_cast<float4*>(part + ((size_t)blockIdx.y * T + t) * K + kv * 8);
    o[0] = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
    o[1] = make_float4(acc[t][4], acc[t][5], acc[t][6], acc[t][7]);
  }
}

}  // namespace

// dw[N, K] (row stride ldw) (+)= scale * dy[T, N]^T x[T, K]; T <= 8, K, ldx and ldw multiples of 8.
extern "C" int eri_rows_wgrad(const void* dy, int ldy, const void* x, int ldx, void* dw, int ldw,
                              int T, int N, int K, int accumulate, float scale, void* stream) {
  if (T < 1 || T > kMaxM || K % 8 || ldx % 8 || ldw % 8 || N < 1) return -1;
  if (((uintptr_t)x | (uintptr_t)dw) & 15) return -1;
  const int block = 128;
  // about sixteen CTAs per SM, each looping over its rows of dW with the x rows held in registers
  const int gx = (K / 8 + block - 1) / block;
  int gy = (148 * 16 + gx - 1) / gx;
  const int chunks = (N + 63) / 64;
  if (gy > chunks) gy = chunks;
  if (gy > 65535) gy = 65535;
  dim3 grid(gx, gy);
  rows_wgrad_kernel<<<grid, block, 0, (cudaStream_t)stream>>>((const bf16*)dy, ldy, (const bf16*)x, ldx,
                                                              (bf16*)dw, ldw, T, N, K, accumulate, scale);
  return (int)cudaGetLastError();
}

// part[splits, T, K] fp32 = per-split partial sums of dy[T, N] W[N, K]; returns the number of
// splits (> 0) the caller must add, or a negative error. `max_splits`: planes available in `part`.
extern "C" int eri_rows_dgrad(const void* dy, int ldy, const void* w, int ldw, float* part, int T,
                              int N, int K, int max_splits, void* stream) {
  if (T < 1 || T > kMaxM || K % 8 || ldw % 8 || N < 1 || max_splits < 1) return -1;
  if (((uintptr_t)w | (uintptr_t)part) & 15) return -1;
  const int block = 128;
  const int gx = (K / 8 + block - 1) / block;
  int splits = (148 * 6 + gx - 1) / gx;            // about six CTAs per SM
  if (splits > max_splits) splits = max_splits;
  if (splits > N) splits = N;
  const int rows = (N + splits - 1) / splits;
  splits = (N + rows - 1) / rows;
  dim3 grid(gx, splits);
  cudaStream_t st = (cudaStream_t)stream;
#define ERI_DGRAD_CASE(TT)                                                                              \
  case TT:                                                                                              \
    rows_dgrad_kernel<TT><<<grid, block, 0, st>>>((const bf16*)dy, ldy, (const bf16*)w, ldw, part, N, K, \
                                                  rows);                                                \
    break;
  switch (T) {
    ERI_DGRAD_CASE(1) ERI_DGRAD_CASE(2) ERI_DGRAD_CASE(3) ERI_DGRAD_CASE(4)
    ERI_DGRAD_CASE(5) ERI_DGRAD_CASE(6) ERI_DGRAD_CASE(7) ERI_DGRAD_CASE(8)
  }
#undef ERI_DGRAD_CASE
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? splits : -(int)e - 1000;
}
