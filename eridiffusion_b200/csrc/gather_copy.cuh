// Copy role and landing-counter waits shared by the gather-fused GEMM kernels.
//
// A gather-fused launch reserves its first n_copy CTAs for copy jobs: each job moves a slab (rows of
// row_bytes, source possibly on a peer GPU) into a local landing buffer and bumps the slab's
// counter; the TMA producers of the compute CTAs wait (bounded) on the counters of the slabs they
// are about to load. The parameter type P provides n_copy, n_jobs, jobs, flags, flag_target, all_flag, err.
#pragma once
#include "ptx.cuh"

namespace eri {

struct GatherJob {
  const void* src;   // peer (or local) source, 16-byte aligned
  void* dst;         // local landing address
  int rows;
  int row_bytes;     // multiple of 16
  long long src_stride, dst_stride;  // bytes
  int flag;          // counter bumped when the job is done
  int pad;
};


__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// Bounded wait for a landing-slab counter. Returns false when the wait ran out.
template <class P>
__device__ __forceinline__ bool wait_slab(const P& p, int f) {
  const unsigned int want = p.flag_target[f];
  if (ld_acquire_gpu(p.flags + f) >= want) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 0; i < (1u << 28); ++i) {
    if (ld_acquire_gpu(p.flags + f) >= want) return true;
    if ((i & 63u) == 63u) {
      if (globaltimer_ns() - t0 > ERI_WAIT_LIMIT_NS) return false;
      // another role or CTA of this launch already gave up: do not stack a second full wait on it
      if (*reinterpret_cast<volatile int*>(p.err) != 0) return false;
    }
  }
  return false;
}

// Copy CTA: moves its jobs through a ring of shared-memory stages with bulk asynchronous copies
// (peer or local global memory -> shared -> local landing buffer). Warp 0 issues the loads, one
// row segment per lane, each stage completing on its own mbarrier; warp 1 issues the stores and
// hands the stage back once the store has read it. With 32 KB stages the ring keeps up to
// ring_stages * 32 KB of NVLink reads in flight per CTA (a 16-byte load per thread kept 3 KB in
// flight and ran at ~1 GB/s per CTA). No multicast: every copy is a plain cp.async.bulk.
constexpr int kCopyStageBytes = 32 * 1024;

__device__ __forceinline__ void bulk_g2s_plain(uint32_t dst_smem, const void* src, uint32_t bytes,
                                               uint32_t bar_smem) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst_smem), "l"(src), "r"(bytes), "r"(bar_smem)
      : "memory");
}
__device__ __forceinline__ void bulk_s2g_plain(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(src_smem), "r"(bytes)
               : "memory");
}

// A job is cut into chunks of whole rows (or, for a contiguous slab, of 32 KB pieces of one long
// row); chunk c of a job covers rows [c * rpc, ...) or bytes [c * 32 KB, ...).
struct CopyChunking {
  bool flat;        // rows are back to back in both source and destination
  long long total;  // flat: bytes of the job
  int rpc;          // strided: rows per chunk
  int nchunks;
};
__device__ __forceinline__ CopyChunking chunking(const GatherJob& job) {
  CopyChunking k;
  k.flat = job.src_stride == job.row_bytes && job.dst_stride == job.row_bytes;
  k.total = (long long)job.rows * job.row_bytes;
  if (k.flat) {
    k.rpc = 0;
    k.nchunks = (int)((k.total + kCopyStageBytes - 1) / kCopyStageBytes);
  } else {
    k.rpc = kCopyStageBytes / job.row_bytes;   // row_bytes <= 32 KB is checked on the host
    k.nchunks = (job.rows + k.rpc - 1) / k.rpc;
  }
  return k;
}

template <class P>
__device__ void copy_role(const P& p, uint8_t* smem, int ring_stages, int cta) {
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)ring_stages * kCopyStageBytes);
  uint64_t* empty = full + ring_stages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < ring_stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == 0) {
    int it = 0;
    bool ok = true;
    for (int j = cta; j < p.n_jobs && ok; j += p.n_copy) {
      const GatherJob job = p.jobs[j];
      if (job.src_stride != job.row_bytes && job.row_bytes > kCopyStageBytes) {
        if (lane == 0) atomicExch(p.err, 63);   // a strided row must fit one ring stage
        break;
      }
      const CopyChunking k = chunking(job);
      for (int c = 0; c < k.nchunks && ok; ++c, ++it) {
        const int s = it % ring_stages;
        if (!mbar_wait(&empty[s], (uint32_t)(((it / ring_stages) & 1) ^ 1))) {
          if (lane == 0) atomicExch(p.err, 61);
          ok = false;
          break;
        }
        const uint32_t dst = smem_u32(smem + (size_t)s * kCopyStageBytes);
        const uint32_t bar = smem_u32(&full[s]);
        if (k.flat) {
          const long long off = (long long)c * kCopyStageBytes;
          const uint32_t bytes = (uint32_t)min((long long)kCopyStageBytes, k.total - off);
          if (lane == 0) {
            mbar_expect_tx(&full[s], bytes);
            bulk_g2s_plain(dst, reinterpret_cast<const char*>(job.src) + off, bytes, bar);
          }
        } else {
          const int r0 = c * k.rpc, nr = min(k.rpc, job.rows - r0);
          if (lane == 0) mbar_expect_tx(&full[s], (uint32_t)nr * (uint32_t)job.row_bytes);
          __syncwarp();
          for (int r = lane; r < nr; r += 32)
            bulk_g2s_plain(dst + (uint32_t)r * (uint32_t)job.row_bytes,
                           reinterpret_cast<const char*>(job.src) + (long long)(r0 + r) * job.src_stride,
                           (uint32_t)job.row_bytes, bar);
        }
      }
    }
  } else if (warp == 1) {
    // Up to kStoreDepth stores stay in flight: a stage goes back to the loader once the store that
    // reads it is no longer among the kStoreDepth - 1 youngest groups (one store at a time capped a
    // CTA at one 32 KB chunk per store latency, ~20 GB/s).
    constexpr int kStoreDepth = 3;
    int it = 0, released = 0;
    bool ok = true;
    for (int j = cta; j < p.n_jobs && ok; j += p.n_copy) {
      const GatherJob job = p.jobs[j];
      if (job.src_stride != job.row_bytes && job.row_bytes > kCopyStageBytes) {
        if (lane == 0) atomicExch(p.err, 63);   // a strided row must fit one ring stage
        break;
      }
      const CopyChunking k = chunking(job);
      for (int c = 0; c < k.nchunks && ok; ++c, ++it) {
        const int s = it % ring_stages;
        if (!mbar_wait(&full[s], (uint32_t)((it / ring_stages) & 1))) {
          if (lane == 0) atomicExch(p.err, 62);
          ok = false;
          break;
        }
        const uint32_t src = smem_u32(smem + (size_t)s * kCopyStageBytes);
        if (k.flat) {
          const long long off = (long long)c * kCopyStageBytes;
          const uint32_t bytes = (uint32_t)min((long long)kCopyStageBytes, k.total - off);
          if (lane == 0) bulk_s2g_plain(reinterpret_cast<char*>(job.dst) + off, src, bytes);
        } else {
          const int r0 = c * k.rpc, nr = min(k.rpc, job.rows - r0);
          for (int r = lane; r < nr; r += 32)
            bulk_s2g_plain(reinterpret_cast<char*>(job.dst) + (long long)(r0 + r) * job.dst_stride,
                           src + (uint32_t)r * (uint32_t)job.row_bytes, (uint32_t)job.row_bytes);
        }
        tma_store_commit();
        tma_store_wait_read<kStoreDepth - 1>();   // all but the youngest groups have read their stage
        __syncwarp();
        for (; released <= it - (kStoreDepth - 1); ++released)
          if (lane == 0) mbar_arrive(&empty[released % ring_stages]);
      }
      // the whole job has landed in local memory before its counter moves
      tma_store_wait<0>();
      __syncwarp();
      for (; released < it; ++released)
        if (lane == 0) mbar_arrive(&empty[released % ring_stages]);
      if (lane == 0 && ok) {
        __threadfence();
        fence_proxy_async_all();
        atomicAdd(p.flags + job.flag, 1u);
        if (p.all_flag) atomicAdd(p.flags + (p.all_flag - 1), 1u);
      }
    }
  }
}

}  // namespace eri
