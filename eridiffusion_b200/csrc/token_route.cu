// Token routing on the device (TREAD-style): score tokens by the L2 norm of their hidden vector,
// pick the top k per sample, gather them into a short sequence, and later re-inject the processed
// rows into the full sequence. The reference scores and selects on the host (a device-to-host copy
// of the hidden states and a CPU sort per routed step, crates/training/src/tread.rs:140-248) and
// gathers with byte-wise narrow kernels; here the selection never leaves the GPU.
//
//   eri_row_l2norm     one warp per token row -> fp32 norm
//   eri_topk_desc      one CTA per sample: bitonic sort of (score, index) keys in shared memory,
//                      first k indices written in descending-score order (ties: lower index first)
//   eri_build_inverse  inv[b, l] = position of token l in the kept list, or -1
//   eri_gather_rows    out[b, j, :] = x[b, idx[b, j], :]
//   eri_reinject_rows  out[b, l, :] = inv[b, l] >= 0 ? routed[b, inv[b, l], :] : full[b, l, :]
//                      (full == nullptr reads zeros: the scatter used by the gather's backward)
#include "ptx.cuh"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

__global__ void row_l2norm_kernel(const bf16* __restrict__ x, float* __restrict__ out, long long rows,
                                  int D) {
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * D);
  float s = 0.f;
  for (int v = lane; v < (D >> 3); v += 32) {
    float f[8];
    unpack8(xr[v], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s = fmaf(f[j], f[j], s);
  }
  s = warp_sum(s);
  if (lane == 0) out[row] = sqrtf(s);
}

// Keys: (float bits of a non-negative score) << 32 | (0xffffffff - index); sorting the 64-bit keys
// in descending order sorts by score, ties by ascending index.
__global__ void __launch_bounds__(1024) topk_desc_kernel(const float* __restrict__ scores,
                                                         int* __restrict__ idx_out, int L, int k,
                                                         int n_pow2) {
  extern __shared__ unsigned long long keys[];
  const int b = blockIdx.x;
  const float* s = scores + (size_t)b * L;
  for (int i = threadIdx.x; i < n_pow2; i += blockDim.x) {
    unsigned long long key = 0ull;  // padding sorts last
    if (i < L) {
      float v = s[i];
      if (!(v >= 0.f)) v = 0.f;  // NaN or negative scores sort with the zeros
      key = ((unsigned long long)__float_as_uint(v) << 32) | (unsigned long long)(0xffffffffu - (unsigned)i);
    }
    keys[i] = key;
  }
  __syncthreads();
  for (int size = 2; size <= n_pow2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < (n_pow2 >> 1); t += blockDim.x) {
        const int lo = 2 * t - (t & (stride - 1));  // index with the `stride` bit clear
        const int hi = lo + stride;
        const bool desc = (lo & size) == 0;
        const unsigned long long a = keys[lo], c = keys[hi];
        if ((a < c) == desc) {
          keys[lo] = c;
          keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  for (int j = threadIdx.x; j < k; j += blockDim.x)
    idx_out[(size_t)b * k + j] = (int)(0xffffffffu - (unsigned)(keys[j] & 0xffffffffull));
}

ERI_DEBUG_BOUNDS_DEFINE(route)

__global__ void build_inverse_kernel(const int* __restrict__ idx, int* __restrict__ inv, int B, int L,
                                     int k) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * k) return;
  const int b = i / k, j = i % k;
  const int l = idx[i];
  if (!ERI_DBG_INDEX(l, L, 61)) return;       // debug build: an index outside [0, L) is recorded
  if (l >= 0 && l < L) inv[(size_t)b * L + l] = j;
}

__global__ void gather_rows_kernel(const bf16* __restrict__ x, const int* __restrict__ idx,
                                   bf16* __restrict__ out, int L, int k, int D) {
  const int j = blockIdx.x, b = blockIdx.y;
  const int l = idx[(size_t)b * k + j];
  const bf16x8* src = reinterpret_cast<const bf16x8*>(x + ((size_t)b * L + l) * D);
  bf16x8* dst = reinterpret_cast<bf16x8*>(out + ((size_t)b * k + j) * D);
  if (threadIdx.x == 0) (void)ERI_DBG_INDEX(l, L, 62);   // debug build: recorded; skipped in every build
  if (l < 0 || l >= L) return;
  for (int v = threadIdx.x; v < (D >> 3); v += blockDim.x) dst[v] = src[v];
}

__global__ void reinject_rows_kernel(const bf16* __restrict__ full, const bf16* __restrict__ routed,
                                     const int* __restrict__ inv, bf16* __restrict__ out, int L, int k,
                                     int D) {
  const int l = blockIdx.x, b = blockIdx.y;
  const int j = inv[(size_t)b * L + l];
  bf16x8* dst = reinterpret_cast<bf16x8*>(out + ((size_t)b * L + l) * D);
  if (j >= k) {                                  // never valid: skipped in every build, recorded in the debug build
    if (threadIdx.x == 0) (void)ERI_DBG_VIOLATION(63, j);
    return;
  }
  if (j >= 0) {
    const bf16x8* src = reinterpret_cast<const bf16x8*>(routed + ((size_t)b * k + j) * D);
    for (int v = threadIdx.x; v < (D >> 3); v += blockDim.x) dst[v] = src[v];
  } else if (full) {
    const bf16x8* src = reinterpret_cast<const bf16x8*>(full + ((size_t)b * L + l) * D);
    for (int v = threadIdx.x; v < (D >> 3); v += blockDim.x) dst[v] = src[v];
  } else {
    bf16x8 z;
    z.u = make_uint4(0, 0, 0, 0);
    for (int v = threadIdx.x; v < (D >> 3); v += blockDim.x) dst[v] = z;
  }
}

}  // namespace

extern "C" {

int eri_row_l2norm(const void* x, float* out, long long rows, int D, void* stream) {
  if (D % 8) return -1;
  const int block = 256;
  const long long grid = (rows * 32 + block - 1) / block;
  row_l2norm_kernel<<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>((const bf16*)x, out, rows, D);
  return (int)cudaGetLastError();
}

// scores [B, L] fp32 (non-negative), idx_out [B, k] int32. L <= 16384.
int eri_topk_desc(const float* scores, int* idx_out, int B, int L, int k, void* stream) {
  if (L < 1 || L > 16384 || k < 1 || k > L) return -1;
  int n = 1;
  while (n < L) n <<= 1;
  const int smem = n * 8;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(topk_desc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             16384 * 8) != cudaSuccess)
      return -2;
    configured = true;
  }
  const int threads = n / 2 < 1024 ? (n / 2 < 32 ? 32 : n / 2) : 1024;
  topk_desc_kernel<<<B, threads, smem, (cudaStream_t)stream>>>(scores, idx_out, L, k, n);
  return (int)cudaGetLastError();
}

// inv [B, L] int32 must be filled with -1 by the caller (one memset: 0xff bytes).
int eri_build_inverse(const int* idx, int* inv, int B, int L, int k, void* stream) {
  const int n = B * k;
  build_inverse_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(idx, inv, B, L, k);
  return (int)cudaGetLastError();
}

int eri_gather_rows(const void* x, const int* idx, void* out, int B, int L, int k, int D, void* stream) {
  if (D % 8) return -1;
  dim3 grid(k, B);
  gather_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((const bf16*)x, idx, (bf16*)out, L, k, D);
  return (int)cudaGetLastError();
}

int eri_reinject_rows(const void* full, const void* routed, const int* inv, void* out, int B, int L,
                      int k, int D, void* stream) {
  if (D % 8) return -1;
  dim3 grid(L, B);
  reinject_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((const bf16*)full, (const bf16*)routed,
                                                              inv, (bf16*)out, L, k, D);
  return (int)cudaGetLastError();
}

}  // extern "C"

ERI_DEBUG_BOUNDS_EXPORT(route)
