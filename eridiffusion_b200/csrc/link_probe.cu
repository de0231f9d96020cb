// Link probe: how fast can CTAs of one GPU move a buffer from / to a peer GPU, by mechanism.
//
//   mode 0  bulk pull : cp.async.bulk peer -> shared -> local (the copy role of the gather-fused GEMM)
//   mode 1  load pull : 16-byte peer loads, eight in flight per thread, plain local stores
//   mode 2  store push: local 16-byte loads, 16-byte stores to the peer (posted writes)
//   mode 3  bulk push : cp.async.bulk local -> shared -> peer
//
// The gather-fused GEMMs pick their transfer mechanism from these numbers (comm_bench --what link).
// No kernel here waits on another GPU: each CTA moves its own contiguous chunk and leaves.
#include "ptx.cuh"
#include "gather_copy.cuh"

using namespace eri;

namespace {

struct ProbeParams {
  int n_copy, n_jobs, all_flag;
  const GatherJob* jobs;
  unsigned int* flags;
  const unsigned int* flag_target;
  int* err;
};

__global__ void __launch_bounds__(192, 1) probe_bulk_kernel(ProbeParams p, int ring) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  copy_role(p, smem, ring, (int)blockIdx.x);
}

// mode 1 / 2: every thread moves 16-byte words, UNROLL loads in flight before the first store
template <int UNROLL>
__global__ void __launch_bounds__(1024, 1)
probe_ldst_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (UNROLL - 1) * stride < n16; i += UNROLL * stride) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) v[u] = src[i + u * stride];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) dst[i + u * stride] = v[u];
  }
  for (; i < n16; i += stride) dst[i] = src[i];
}

int* g_probe_err = nullptr;

}  // namespace

extern "C" {

// Moves `bytes` (a multiple of 16) from src to dst with `n_ctas` CTAs. For the bulk modes the caller
// passes a device array of GatherJob records (`jobs`, one contiguous slab each) and their count.
// Returns 0 or a CUDA error code.
int eri_link_probe(int mode, const void* src, void* dst, long long bytes, int n_ctas, const void* jobs,
                   int n_jobs, void* flags, const void* flag_target, int ring, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (n_ctas < 1 || bytes % 16) return -1;
  if (mode == 0 || mode == 3) {
    if (!g_probe_err) {
      if (cudaMalloc(&g_probe_err, sizeof(int)) != cudaSuccess) return -3;
      cudaMemset(g_probe_err, 0, sizeof(int));
    }
    if (ring < 1 || ring > 6) return -1;
    const int SMEM = ring * kCopyStageBytes + 1024 + 256;
    static int configured = 0;
    if (configured < SMEM) {
      if (cudaFuncSetAttribute(probe_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 6 * kCopyStageBytes + 1280) !=
          cudaSuccess)
        return -5;
      configured = 6 * kCopyStageBytes + 1280;
    }
    ProbeParams p;
    p.n_copy = n_ctas; p.n_jobs = n_jobs; p.all_flag = 0; p.jobs = (const GatherJob*)jobs;
    p.flags = (unsigned int*)flags; p.flag_target = (const unsigned int*)flag_target; p.err = g_probe_err;
    probe_bulk_kernel<<<n_ctas, 192, SMEM, st>>>(p, ring);
    return (int)cudaGetLastError();
  }
  probe_ldst_kernel<8><<<n_ctas, 1024, 0, st>>>((const uint4*)src, (uint4*)dst, bytes / 16);
  return (int)cudaGetLastError();
}

int eri_link_probe_check_error() {
  if (!g_probe_err) return 0;
  int h = 0;
  cudaMemcpy(&h, g_probe_err, sizeof(int), cudaMemcpyDeviceToHost);
  if (h) cudaMemset(g_probe_err, 0, sizeof(int));
  return h;
}

}  // extern "C"
