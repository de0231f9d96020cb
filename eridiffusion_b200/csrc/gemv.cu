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
