// GroupNorm (+ optional SiLU) for channels-last activations [N, HW, C], forward and backward.
//
// Both directions are two bandwidth-bound passes over the activation:
//   column pass   per-(n, c) sums over HW, accumulated per thread in registers for a fixed group of
//                 eight channels, combined through shared-memory atomics and one global atomic per
//                 (n, c, statistic) per CTA:   forward  (sum x, sum x^2)
//                                              backward (sum dz, sum dz * xhat),  dz = dy * act'(z)
//   apply pass    forward  y  = act(xhat * w + b)
//                 backward dx = rstd * (dz * w - s1 / m - xhat * s2 / m)
// The few-kilobyte reductions between the passes (channels -> groups, parameter gradients) are done
// by the caller on the [N, C] statistics. The reference's GroupNorm is a forward-only NCHW kernel
// with one warp-shuffle reduction per group (crates/core/src/cuda/kernels/group_norm.cu); its SDXL
// ResBlocks apply SiLU as a separate pass (crates/training/src/sdxl/runtime.rs).
#include "ptx.cuh"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

struct GnArgs {
  const bf16 *x, *dy, *w, *b;
  const float *mean, *rstd;  // [N, G]
  const float *s1, *s2;      // [N, G] backward group sums (already divided by m)
  float* stats;              // [N, C, 2]
  bf16* out;
  int HW, C, G, silu;
};

__device__ __forceinline__ float act_grad(float z, int silu) {
  if (!silu) return 1.f;
  const float s = 1.f / (1.f + __expf(-z));
  return s * (1.f + z * (1.f - s));
}

template <int MODE>
__global__ void gn_colreduce_kernel(const GnArgs a, int rows_per_cta) {
  extern __shared__ float sacc[];  // [C][2]
  const int n = blockIdx.y;
  const int nvec = a.C >> 3;
  const int R = blockDim.x / nvec;  // rows handled in parallel by the CTA
  const int v = threadIdx.x % nvec, rr = threadIdx.x / nvec;
  for (int i = threadIdx.x; i < 2 * a.C; i += blockDim.x) sacc[i] = 0.f;
  __syncthreads();
  const int r0 = blockIdx.x * rows_per_cta;
  const int r1 = min(a.HW, r0 + rows_per_cta);
  float acc0[8], acc1[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc0[j] = acc1[j] = 0.f;
  float wv[8], bv[8], mu[8], rs[8];
  if (MODE == 1) {
    const int cpg = a.C / a.G;
    float t[8];
    unpack8(reinterpret_cast<const bf16x8*>(a.w)[v], wv);
    if (a.b) unpack8(reinterpret_cast<const bf16x8*>(a.b)[v], t);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      bv[j] = a.b ? t[j] : 0.f;
      const int g = (v * 8 + j) / cpg;
      mu[j] = a.mean[n * a.G + g];
      rs[j] = a.rstd[n * a.G + g];
    }
  }
  if (rr < R) {
    for (int r = r0 + rr; r < r1; r += R) {
      const size_t off = ((size_t)n * a.HW + r) * a.C;
      float xv[8];
      unpack8(reinterpret_cast<const bf16x8*>(a.x + off)[v], xv);
      if (MODE == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc0[j] += xv[j];
          acc1[j] = fmaf(xv[j], xv[j], acc1[j]);
        }
      } else {
        float g[8];
        unpack8(reinterpret_cast<const bf16x8*>(a.dy + off)[v], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mu[j]) * rs[j];
          const float dz = g[j] * act_grad(fmaf(xh, wv[j], bv[j]), a.silu);
          acc0[j] += dz;
          acc1[j] = fmaf(dz, xh, acc1[j]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      atomicAdd(&sacc[(v * 8 + j) * 2], acc0[j]);
      atomicAdd(&sacc[(v * 8 + j) * 2 + 1], acc1[j]);
    }
  }
  __syncthreads();
  float* dst = a.stats + (size_t)n * a.C * 2;
  for (int i = threadIdx.x; i < 2 * a.C; i += blockDim.x) atomicAdd(&dst[i], sacc[i]);
}

template <int MODE>
__global__ void gn_apply_kernel(const GnArgs a, long long total_vec) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total_vec) return;
  const int nvec = a.C >> 3;
  const int v = (int)(i % nvec);
  const long long row = i / nvec;
  const int n = (int)(row / a.HW);
  const int cpg = a.C / a.G;
  float xv[8], wv[8], bv[8], o[8];
  unpack8(reinterpret_cast<const bf16x8*>(a.x)[i], xv);
  unpack8(reinterpret_cast<const bf16x8*>(a.w)[v], wv);
  if (a.b) {
    unpack8(reinterpret_cast<const bf16x8*>(a.b)[v], bv);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) bv[j] = 0.f;
  }
  if (MODE == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int g = (v * 8 + j) / cpg;
      const float xh = (xv[j] - a.mean[n * a.G + g]) * a.rstd[n * a.G + g];
      const float z = fmaf(xh, wv[j], bv[j]);
      o[j] = a.silu ? z / (1.f + __expf(-z)) : z;
    }
  } else {
    float g8[8];
    unpack8(reinterpret_cast<const bf16x8*>(a.dy)[i], g8);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int g = (v * 8 + j) / cpg;
      const float rs = a.rstd[n * a.G + g];
      const float xh = (xv[j] - a.mean[n * a.G + g]) * rs;
      const float dz = g8[j] * act_grad(fmaf(xh, wv[j], bv[j]), a.silu);
      o[j] = rs * (dz * wv[j] - a.s1[n * a.G + g] - xh * a.s2[n * a.G + g]);
    }
  }
  reinterpret_cast<bf16x8*>(a.out)[i] = pack8(o);
}

template <int MODE>
int launch_colreduce(const GnArgs& a, int N, cudaStream_t st) {
  const int nvec = a.C >> 3;
  if (nvec > 1024) return -1;
  int R = 256 / nvec;
  if (R < 1) R = 1;
  const int threads = ((R * nvec + 31) / 32) * 32;
  // enough CTAs to fill the machine a few times over, at least 32 rows each
  int rows_per_cta = (int)(((long long)a.HW * N + 148 * 8 - 1) / (148 * 8));
  if (rows_per_cta < 32) rows_per_cta = 32;
  rows_per_cta = (rows_per_cta + R - 1) / R * R;
  dim3 grid((a.HW + rows_per_cta - 1) / rows_per_cta, N);
  gn_colreduce_kernel<MODE><<<grid, threads, 2 * a.C * sizeof(float), st>>>(a, rows_per_cta);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

// stats [N, C, 2] fp32 must be zero on entry. Forward: (sum x, sum x^2) per (n, c).
int eri_gn_stats_fwd(const void* x, float* stats, int N, int HW, int C, void* stream) {
  if (C % 8) return -1;
  GnArgs a = {};
  a.x = (const bf16*)x; a.stats = stats; a.HW = HW; a.C = C; a.G = 1;
  return launch_colreduce<0>(a, N, (cudaStream_t)stream);
}

int eri_gn_apply_fwd(const void* x, const void* w, const void* b, const float* mean, const float* rstd,
                     void* y, int N, int HW, int C, int G, int silu, void* stream) {
  if (C % 8 || C % G) return -1;
  GnArgs a = {};
  a.x = (const bf16*)x; a.w = (const bf16*)w; a.b = (const bf16*)b; a.mean = mean; a.rstd = rstd;
  a.out = (bf16*)y; a.HW = HW; a.C = C; a.G = G; a.silu = silu;
  const long long total = (long long)N * HW * (C >> 3);
  gn_apply_kernel<0><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a, total);
  return (int)cudaGetLastError();
}

// Backward column sums: stats[n, c] = (sum dz, sum dz * xhat), zero on entry.
int eri_gn_stats_bwd(const void* x, const void* dy, const void* w, const void* b, const float* mean,
                     const float* rstd, float* stats, int N, int HW, int C, int G, int silu,
                     void* stream) {
  if (C % 8 || C % G) return -1;
  GnArgs a = {};
  a.x = (const bf16*)x; a.dy = (const bf16*)dy; a.w = (const bf16*)w; a.b = (const bf16*)b;
  a.mean = mean; a.rstd = rstd; a.stats = stats; a.HW = HW; a.C = C; a.G = G; a.silu = silu;
  return launch_colreduce<1>(a, N, (cudaStream_t)stream);
}

// s1, s2 [N, G]: group sums of w*sum(dz) and w*sum(dz*xhat), each divided by m = HW * C / G.
int eri_gn_apply_bwd(const void* x, const void* dy, const void* w, const void* b, const float* mean,
                     const float* rstd, const float* s1, const float* s2, void* dx, int N, int HW,
                     int C, int G, int silu, void* stream) {
  if (C % 8 || C % G) return -1;
  GnArgs a = {};
  a.x = (const bf16*)x; a.dy = (const bf16*)dy; a.w = (const bf16*)w; a.b = (const bf16*)b;
  a.mean = mean; a.rstd = rstd; a.s1 = s1; a.s2 = s2; a.out = (bf16*)dx;
  a.HW = HW; a.C = C; a.G = G; a.silu = silu;
  const long long total = (long long)N * HW * (C >> 3);
  gn_apply_kernel<1><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a, total);
  return (int)cudaGetLastError();
}

}  // extern "C"
