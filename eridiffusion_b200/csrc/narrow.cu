// Strided slice gather and its gradient (slice scatter-add).
//
// The reference ships two SIMT kernels for `narrow(dim, start, len)` on tensors of rank <= 8: a
// byte-wise gather whose shape / stride arrays are allocated and copied on every call
// (crates/core/cuda/narrow_strided.cu:18-99), and a backward that scatter-adds the slice gradient
// with dtype-tagged atomics, bf16 through a 32-bit compare-and-swap loop
// (crates/core/cuda/narrow_strided_backward.cu:22-214).
//
// Here:
//  * shapes and strides travel by value in the launch parameters (no allocation, no extra copy);
//  * a slice maps every output element to ONE input element, so the backward needs no atomics at
//    all: it is a read-modify-write of disjoint addresses;
//  * the common case -- source contiguous, viewed as [outer, dim, inner] -- moves 16-byte vectors
//    with a grid sized to the 148 SMs; the general strided case falls back to one element per
//    thread with 64-bit index arithmetic.
//
// In the framework plain slices are views; these kernels serve the cases that need a materialised
// copy (a slice handed to a kernel that wants a dense operand) and the accumulation of a slice
// gradient into a larger gradient buffer.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int kMaxRank = 8;

struct StridedView {
    int rank;
    long long shape[kMaxRank];     // shape of the SLICE (output)
    long long stride[kMaxRank];    // element strides of the source tensor
    long long offset;              // element offset of the slice's first element in the source
};

// ------------------------------------------------------------------ contiguous [outer, dim, inner]
// src: [outer, dim_len, inner] -> dst: [outer, len, inner], both in units of VEC-byte words.
template <typename V>
__global__ void narrow_rows_kernel(const V* __restrict__ src, V* __restrict__ dst, long long outer,
                                   long long dim_len, long long inner, long long start, long long len) {
    const long long total = outer * len * inner;
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const long long run = len * inner;
        const long long o = i / run, r = i - o * run;
        dst[i] = src[o * dim_len * inner + start * inner + r];
    }
}

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// grad_in[o, start + j, i] += grad_out[o, j, i]; eight 16-bit or four 32-bit values per thread.
template <typename T, int PER>
__global__ void narrow_add_rows_kernel(const T* __restrict__ gout, T* __restrict__ gin, long long outer,
                                       long long dim_len, long long inner, long long start, long long len) {
    const long long total = outer * len * inner / PER;          // inner % PER == 0 (checked on the host)
    const long long step = (long long)gridDim.x * blockDim.x;
    const long long run = len * inner / PER, in_w = inner / PER;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const long long o = i / run, r = i - o * run;
        const uint4 a = reinterpret_cast<const uint4*>(gout)[i];
        uint4* dp = reinterpret_cast<uint4*>(gin) + (o * dim_len * in_w + start * in_w + r);
        uint4 b = *dp;
        const T* av = reinterpret_cast<const T*>(&a);
        T* bv = reinterpret_cast<T*>(&b);
#pragma unroll
        for (int k = 0; k < PER; ++k) bv[k] = from_f<T>(to_f<T>(bv[k]) + to_f<T>(av[k]));
        *dp = b;
    }
}

// ------------------------------------------------------------------ general strided source
__device__ __forceinline__ long long src_index(const StridedView& v, long long i) {
    long long idx = v.offset;
#pragma unroll
    for (int d = kMaxRank - 1; d >= 0; --d) {
        if (d < v.rank) {
            const long long q = i / v.shape[d];
            idx += (i - q * v.shape[d]) * v.stride[d];
            i = q;
        }
    }
    return idx;
}

template <typename W>
__global__ void narrow_strided_kernel(const W* __restrict__ src, W* __restrict__ dst, StridedView v,
                                      long long total) {
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
        dst[i] = src[src_index(v, i)];
}

template <typename T>
__global__ void narrow_add_strided_kernel(const T* __restrict__ gout, T* __restrict__ gin, StridedView v,
                                          long long total) {
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const long long j = src_index(v, i);
        gin[j] = from_f<T>(to_f<T>(gin[j]) + to_f<T>(gout[i]));
    }
}

inline int grid_for(long long total, int threads) {
    long long b = (total + threads - 1) / threads;
    const long long cap = 148LL * 8;                      // 8 resident CTAs of 256 threads per SM
    if (b > cap) b = cap;
    return b < 1 ? 1 : (int)b;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" {

// Copy of src[:, start:start+len, :] for a contiguous source viewed as [outer, dim_len, inner]
// with `elem` bytes per element. Returns 0, or a cudaError code, or -1 for bad arguments.
int eri_narrow_copy(const void* src, void* dst, long long outer, long long dim_len, long long inner,
                    long long start, long long len, int elem, void* stream) {
    if (outer < 0 || len < 0 || start < 0 || start + len > dim_len || inner < 0 || elem <= 0) return -1;
    const long long total_bytes = outer * len * inner * elem;
    if (total_bytes == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    // A row of the source is dim_len * inner * elem bytes, of which the bytes [off_b, off_b + run_b)
    // are kept. The widest word that divides all three (and the base addresses) moves the data, so
    // a slice of the LAST dimension (inner = 1) is vectorised like any other.
    const long long row_b = dim_len * inner * elem, off_b = start * inner * elem, run_b = len * inner * elem;
    int v = 16;
    while (v > 1 && (row_b % v || off_b % v || run_b % v || (reinterpret_cast<uintptr_t>(src) % v) ||
                     (reinterpret_cast<uintptr_t>(dst) % v)))
        v >>= 1;
    const long long total = outer * (run_b / v);
    const int g = grid_for(total, 256);
    switch (v) {
        case 16: narrow_rows_kernel<uint4><<<g, 256, 0, st>>>((const uint4*)src, (uint4*)dst, outer, row_b / v, 1, off_b / v, run_b / v); break;
        case 8: narrow_rows_kernel<uint2><<<g, 256, 0, st>>>((const uint2*)src, (uint2*)dst, outer, row_b / v, 1, off_b / v, run_b / v); break;
        case 4: narrow_rows_kernel<uint32_t><<<g, 256, 0, st>>>((const uint32_t*)src, (uint32_t*)dst, outer, row_b / v, 1, off_b / v, run_b / v); break;
        case 2: narrow_rows_kernel<uint16_t><<<g, 256, 0, st>>>((const uint16_t*)src, (uint16_t*)dst, outer, row_b / v, 1, off_b / v, run_b / v); break;
        default: narrow_rows_kernel<uint8_t><<<g, 256, 0, st>>>((const uint8_t*)src, (uint8_t*)dst, outer, row_b, 1, off_b, run_b); break;
    }
    return (int)cudaGetLastError();
}

// grad_in[:, start:start+len, :] += grad_out. dtype: 0 = f32, 1 = bf16, 2 = f16.
int eri_narrow_backward_add(const void* grad_out, void* grad_in, long long outer, long long dim_len,
                            long long inner, long long start, long long len, int dtype, void* stream) {
    if (outer < 0 || len < 0 || start < 0 || start + len > dim_len || inner < 0 || dtype < 0 || dtype > 2)
        return -1;
    const long long total = outer * len * inner;
    if (total == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int per = dtype == 0 ? 4 : 8;
    // in elements: row length, offset and length of the kept run; 16-byte words when all three divide
    const long long row_e = dim_len * inner, off_e = start * inner, run_e = len * inner;
    const bool vec = row_e % per == 0 && off_e % per == 0 && run_e % per == 0 && aligned16(grad_out) && aligned16(grad_in);
    StridedView v{};
    v.rank = 3;
    v.shape[0] = outer; v.shape[1] = len; v.shape[2] = inner;
    v.stride[0] = dim_len * inner; v.stride[1] = inner; v.stride[2] = 1;
    v.offset = start * inner;
    const int g = grid_for(vec ? total / per : total, 256);
    if (dtype == 0) {
        if (vec) narrow_add_rows_kernel<float, 4><<<g, 256, 0, st>>>((const float*)grad_out, (float*)grad_in, outer, row_e / 4, 4, off_e / 4, run_e / 4);
        else narrow_add_strided_kernel<float><<<g, 256, 0, st>>>((const float*)grad_out, (float*)grad_in, v, total);
    } else if (dtype == 1) {
        if (vec) narrow_add_rows_kernel<__nv_bfloat16, 8><<<g, 256, 0, st>>>((const __nv_bfloat16*)grad_out, (__nv_bfloat16*)grad_in, outer, row_e / 8, 8, off_e / 8, run_e / 8);
        else narrow_add_strided_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)grad_out, (__nv_bfloat16*)grad_in, v, total);
    } else {
        if (vec) narrow_add_rows_kernel<__half, 8><<<g, 256, 0, st>>>((const __half*)grad_out, (__half*)grad_in, outer, row_e / 8, 8, off_e / 8, run_e / 8);
        else narrow_add_strided_kernel<__half><<<g, 256, 0, st>>>((const __half*)grad_out, (__half*)grad_in, v, total);
    }
    return (int)cudaGetLastError();
}

// General form: the slice has `rank` (<= 8) dimensions `shape`, the source has element strides
// `stride` and the slice starts `offset` elements into it. `elem` in {1, 2, 4, 8, 16} bytes.
int eri_narrow_strided(const void* src, void* dst, int rank, const long long* shape, const long long* stride,
                       long long offset, int elem, void* stream) {
    if (rank < 1 || rank > kMaxRank) return -1;
    StridedView v{};
    v.rank = rank;
    v.offset = offset;
    long long total = 1;
    for (int d = 0; d < rank; ++d) {
        if (shape[d] < 0) return -1;
        v.shape[d] = shape[d];
        v.stride[d] = stride[d];
        total *= shape[d];
    }
    if (total == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int g = grid_for(total, 256);
    switch (elem) {
        case 1: narrow_strided_kernel<uint8_t><<<g, 256, 0, st>>>((const uint8_t*)src, (uint8_t*)dst, v, total); break;
        case 2: narrow_strided_kernel<uint16_t><<<g, 256, 0, st>>>((const uint16_t*)src, (uint16_t*)dst, v, total); break;
        case 4: narrow_strided_kernel<uint32_t><<<g, 256, 0, st>>>((const uint32_t*)src, (uint32_t*)dst, v, total); break;
        case 8: narrow_strided_kernel<uint2><<<g, 256, 0, st>>>((const uint2*)src, (uint2*)dst, v, total); break;
        case 16: narrow_strided_kernel<uint4><<<g, 256, 0, st>>>((const uint4*)src, (uint4*)dst, v, total); break;
        default: return -1;
    }
    return (int)cudaGetLastError();
}

// Strided form of the backward: grad_in (strided, slice at `offset`) += grad_out (dense).
int eri_narrow_backward_add_strided(const void* grad_out, void* grad_in, int rank, const long long* shape,
                                    const long long* stride, long long offset, int dtype, void* stream) {
    if (rank < 1 || rank > kMaxRank || dtype < 0 || dtype > 2) return -1;
    StridedView v{};
    v.rank = rank;
    v.offset = offset;
    long long total = 1;
    for (int d = 0; d < rank; ++d) {
        if (shape[d] < 0) return -1;
        v.shape[d] = shape[d];
        v.stride[d] = stride[d];
        total *= shape[d];
    }
    if (total == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int g = grid_for(total, 256);
    if (dtype == 0) narrow_add_strided_kernel<float><<<g, 256, 0, st>>>((const float*)grad_out, (float*)grad_in, v, total);
    else if (dtype == 1) narrow_add_strided_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)grad_out, (__nv_bfloat16*)grad_in, v, total);
    else narrow_add_strided_kernel<__half><<<g, 256, 0, st>>>((const __half*)grad_out, (__half*)grad_in, v, total);
    return (int)cudaGetLastError();
}

}  // extern "C"
