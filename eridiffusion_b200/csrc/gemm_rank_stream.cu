// out[M, N] = alpha * a[M, K] b[N, K]^T for N = 16 / 32 / 64 (a LoRA rank) as a streaming kernel.
//
// The problem is bound by reading a once (M * K * 2 bytes; 2 * N FLOP per byte), so the kernel is
// built around loads in flight, not around the tensor cores: no shared-memory operand staging, no
// tensor-memory allocation, no barriers in the main loop. One CTA of eight warps owns 16 rows of a;
// the warps split K among themselves (contiguous ranges, so each warp walks whole DRAM pages) and
// every thread keeps several 16-byte loads of a in flight. The products run on mma.sync m16n8k16:
// the instruction sums over 16 k-slots, and which column sits in which slot is free as long as a and
// b agree, so a thread's 16-byte load (8 consecutive columns of one row) feeds two instructions
// directly from registers: slots {2t, 2t+1, 2t+8, 2t+9} take columns {8t..8t+3} for the first and
// {8t+4..8t+7} for the second. b is loaded the same way (row n = lane / 4 of each 8-row group) and
// stays in L1 / L2 (N * K * 2 bytes for the whole grid). The eight partial 16 x N tiles are summed
// through shared memory at the end.
//
// The reference computes the LoRA down-projection as a separate library GEMM per adapter site
// (crates/training/src/flux/lora.rs:47-63).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

typedef __nv_bfloat16 bf16;

namespace {

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kWarps = 8;

// NT: 8-column tiles of the output (N = 8 * NT); U: 32-column steps whose loads are issued together.
// One problem of a launch. A launch may carry two with the same K and N (the image and the text stream of a
// dual-stream block): CTAs [0, ceil(M0 / 16)) work on the first, the rest on the second.
struct RankProb {
  const bf16* a;
  long long lda;
  const bf16* b;
  long long ldb;
  bf16* out;
  int ldc, M;
  float alpha;
};

template <int NT, int U>
__global__ void __launch_bounds__(kWarps * 32)
rank_stream_kernel(const RankProb p0, const RankProb p1, int grid0, int K) {
  constexpr int N = NT * 8;
  const bool second = (int)blockIdx.x >= grid0;
  const RankProb& pr = second ? p1 : p0;
  const bf16* __restrict__ a = pr.a;
  const bf16* __restrict__ b = pr.b;
  bf16* __restrict__ out = pr.out;
  const long long lda = pr.lda, ldb = pr.ldb;
  const int ldc = pr.ldc, M = pr.M;
  const float alpha = pr.alpha;
  __shared__ float red[kWarps][16][N + 1];
  // the GEMM that consumes this kernel's output may be scheduled now; it waits for this kernel's
  // completion only before it reads the output (programmatic dependent launch)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int m0 = ((int)blockIdx.x - (second ? grid0 : 0)) * 16;
  // rows past the end read the last row (valid memory) and are never stored
  const int r0 = min(m0 + g, M - 1), r1 = min(m0 + g + 8, M - 1);
  const int nsteps = K >> 5;
  const int s_begin = (int)((long long)warp * nsteps / kWarps);
  const int s_end = (int)((long long)(warp + 1) * nsteps / kWarps);
  const uint4* pa0 = reinterpret_cast<const uint4*>(a + (size_t)r0 * lda) + t;
  const uint4* pa1 = reinterpret_cast<const uint4*>(a + (size_t)r1 * lda) + t;
  const uint4* pb = reinterpret_cast<const uint4*>(b + (size_t)g * ldb) + t;
  const size_t b_tile = (size_t)ldb;   // uint4 units between 8-row groups of b: 8 rows * ldb * 2 B / 16 B

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

  // Software pipeline over batches of U steps: the loads of a for batch i + 1 are issued before the
  // products of batch i, so every thread keeps 2 * U * 32 bytes of a in flight across the loop; b
  // comes from L1 / L2 right before its use.
  uint4 cur0[U], cur1[U], nxt0[U], nxt1[U];
  auto load_a = [&](uint4 (&v0)[U], uint4 (&v1)[U], int s) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int ss = min(s + u, s_end - 1);       // the tail repeats a step; its product is dropped
      v0[u] = ld_stream16(pa0 + 4 * ss);
      v1[u] = ld_stream16(pa1 + 4 * ss);
    }
  };
  if (s_begin < s_end) load_a(cur0, cur1, s_begin);
  for (int s = s_begin; s < s_end; s += U) {
    if (s + U < s_end) load_a(nxt0, nxt1, s + U);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (s + u < s_end) {
        uint4 vb[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) vb[j] = ld_cached16(pb + j * b_tile + 4 * (s + u));
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          mma16816(acc[j], cur0[u].x, cur1[u].x, cur0[u].y, cur1[u].y, vb[j].x, vb[j].y);
          mma16816(acc[j], cur0[u].z, cur1[u].z, cur0[u].w, cur1[u].w, vb[j].z, vb[j].w);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      cur0[u] = nxt0[u];
      cur1[u] = nxt1[u];
    }
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    red[warp][g][j * 8 + 2 * t] = acc[j][0];
    red[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
    red[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
    red[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  // 16 x N outputs, two adjacent columns per thread
  for (int i = threadIdx.x; i < 16 * N / 2; i += kWarps * 32) {
    const int row = i / (N / 2), col = (i % (N / 2)) * 2;
    float v0 = 0.f, v1 = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      v0 += red[w][row][col];
      v1 += red[w][row][col + 1];
    }
    if (m0 + row < M)
      *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(m0 + row) * ldc + col) =
          __floats2bfloat162_rn(v0 * alpha, v1 * alpha);
  }
}

int launch_rank(const RankProb& p0, const RankProb& p1, int grid0, int grid1, int N, int K, cudaStream_t st) {
  const int grid = grid0 + grid1;
  if (N == 16)
    rank_stream_kernel<2, 4><<<grid, kWarps * 32, 0, st>>>(p0, p1, grid0, K);
  else if (N == 32)
    rank_stream_kernel<4, 4><<<grid, kWarps * 32, 0, st>>>(p0, p1, grid0, K);
  else
    rank_stream_kernel<8, 2><<<grid, kWarps * 32, 0, st>>>(p0, p1, grid0, K);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

// a [M, K] (row stride lda elements), b [N, K] (row stride ldb), out [M, N] (row stride ldc), bf16.
// Returns -100 when the shape is outside this kernel's range (the caller uses another kernel).
int eri_gemm_rank_stream(const void* a, long long lda, const void* b, long long ldb, void* out,
                         int ldc, int M, int N, int K, float alpha, void* stream) {
  if (!(N == 16 || N == 32 || N == 64) || M < 1 || K < 256 || K % 32 || lda % 8 || ldb % 8 || ldc % 2)
    return -100;
  if ((((uintptr_t)a | (uintptr_t)b) & 15) || ((uintptr_t)out & 3)) return -100;
  const RankProb p{(const bf16*)a, lda, (const bf16*)b, ldb, (bf16*)out, ldc, M, alpha};
  return launch_rank(p, p, (M + 15) / 16, 0, N, K, (cudaStream_t)stream);
}

// Two products with the same N and K in one launch (out_i = alpha_i * a_i b_i^T): the small second one (the
// 512-token text stream) costs a few more CTAs instead of a launch of its own.
int eri_gemm_rank_stream2(const void* a0, long long lda0, const void* b0, long long ldb0, void* out0, int ldc0,
                          int M0, float alpha0, const void* a1, long long lda1, const void* b1, long long ldb1,
                          void* out1, int ldc1, int M1, float alpha1, int N, int K, void* stream) {
  if (!(N == 16 || N == 32 || N == 64) || M0 < 1 || M1 < 1 || K < 256 || K % 32 || lda0 % 8 || ldb0 % 8 || ldc0 % 2 ||
      lda1 % 8 || ldb1 % 8 || ldc1 % 2)
    return -100;
  if ((((uintptr_t)a0 | (uintptr_t)b0 | (uintptr_t)a1 | (uintptr_t)b1) & 15) ||
      (((uintptr_t)out0 | (uintptr_t)out1) & 3))
    return -100;
  const RankProb p0{(const bf16*)a0, lda0, (const bf16*)b0, ldb0, (bf16*)out0, ldc0, M0, alpha0};
  const RankProb p1{(const bf16*)a1, lda1, (const bf16*)b1, ldb1, (bf16*)out1, ldc1, M1, alpha1};
  return launch_rank(p0, p1, (M0 + 15) / 16, (M1 + 15) / 16, N, K, (cudaStream_t)stream);
}

}  // extern "C"
