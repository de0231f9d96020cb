// Thin inline-PTX wrappers for the sm_100a features the kernels use:
// mbarrier, TMA (cp.async.bulk.tensor, never with cluster multicast), tcgen05
// (TMEM alloc, UMMA issue/commit, TMEM loads) and acquire/release system-scope
// accesses for flags that another GPU writes.
//
// Every wait in this file is bounded: a spin that runs out returns false and the
// caller records an error word and leaves the kernel through its normal exit.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace eri {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Programmatic dependent launch: a kernel launched with the programmatic-stream-serialization
// attribute may start while the previous kernel on the stream still runs; griddep_wait() blocks
// until that kernel has completed and its writes are visible (a no-op without the attribute).
// griddep_launch_dependents() in the earlier kernel lets the next one be scheduled right away.
__device__ __forceinline__ void griddep_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up after ERI_WAIT_LIMIT_NS of wall time (and after a hard cap on the
// number of polls, in case the timer does not advance). A legitimate wait in these kernels is
// microseconds long.
#ifndef ERI_WAIT_LIMIT_NS
#define ERI_WAIT_LIMIT_NS 2000000000ull
#endif
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 0; i < (1u << 26); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && globaltimer_ns() - t0 > ERI_WAIT_LIMIT_NS) return false;
  }
  return false;
}

// ----------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const void* desc) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(desc)) : "memory");
}
// 2-D tiled load global -> shared, completion on an mbarrier of this CTA.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* desc, uint64_t* bar,
                                            int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(bar)),
      "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* desc, uint64_t* bar,
                                            int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(bar)),
      "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const void* desc, uint64_t* bar,
                                            int32_t x, int32_t y, int32_t z, int32_t w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(bar)),
      "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// 2-D tiled store shared -> global (bulk async group).
__device__ __forceinline__ void tma_store_2d(const void* desc, const void* smem_src, int32_t x,
                                             int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, fp32 accumulate; one thread issues.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A operand from TMEM (bf16 packed), B from shared memory.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Make an mbarrier of this CTA track completion of all prior UMMAs of this thread.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets row (lane base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
      "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
      "r"(r[14]), "r"(r[15])
      : "memory");
}

// ----------------------------------------------------------------- CTA pairs (cta_group::2)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
// Loads from a shared::cluster address (this or another CTA's shared memory, see map_to_cta).
__device__ __forceinline__ float ld_shared_cluster_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_shared_cluster_v4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// TMA load whose completion bytes are credited to the barrier at `bar_cluster_addr`
// (a shared::cluster address, here always the leader CTA's barrier).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* desc,
                                                 uint32_t bar_cluster_addr, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar_cluster_addr),
      "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (once all prior UMMAs of this thread are done) on a barrier given by its shared::cluster
// address: used for the local CTA's barrier and, with the mapped address, for the peer's.
__device__ __forceinline__ void umma2_commit_addr(uint32_t bar_cluster_addr) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          bar_cluster_addr)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const void* desc,
                                                 uint32_t bar_cluster_addr, int32_t x, int32_t y,
                                                 int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar_cluster_addr),
      "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Pair MMA with the A operand read from tensor memory (each CTA's own lanes), B from the two CTAs'
// shared memory.
__device__ __forceinline__ void umma2_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major bf16 operand stored as rows of 128 bytes
// (64 bf16) with the 128-byte swizzle that TMA's SWIZZLE_128B mode writes. Groups of 8 rows
// are 1024 bytes apart (stride byte offset); the leading byte offset is unused for this mode.
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                 // leading byte offset (ignored)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;         // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                 // descriptor version for sm_100
  d |= static_cast<uint64_t>(2) << 61;                 // SWIZZLE_128B
  return d;
}
// K-major operand whose rows are `sw` bytes long (32, 64 or 128) and swizzled with the matching
// TMA swizzle mode; groups of 8 rows are 8*sw bytes apart.
__device__ __forceinline__ uint64_t umma_desc_kmajor(uint32_t saddr, uint32_t sw) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>((8 * sw) >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(sw == 128 ? 2 : (sw == 64 ? 4 : 6)) << 61;
  return d;
}
// Shared-memory matrix descriptor for an MN-major bf16 operand: the tile is stored as
// (K rows) x (64 MN elements = 128 bytes) slabs with the 128-byte swizzle; slabs that cover the
// next 64 MN elements are `mn_slab_bytes` apart, groups of 8 K-rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_mn128(uint32_t saddr, uint32_t mn_slab_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((mn_slab_bytes >> 4) & 0x3FFF) << 16;  // leading: next 64 MN
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                      // stride: next 8 K rows
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, dense, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N, int a_mn_major = 0,
                                                       int b_mn_major = 0) {
  return (1u << 4)                      // accumulator fp32
         | (1u << 7)                    // A bf16
         | (1u << 10)                   // B bf16
         | (uint32_t(a_mn_major) << 15) // A major
         | (uint32_t(b_mn_major) << 16) // B major
         | (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

// ----------------------------------------------------------------- system-scope flags
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ----------------------------------------------------------------- bounds-checked debug build
// Built with -DERI_DEBUG_BOUNDS (csrc/build.py, ERI_B200_DEBUG_BOUNDS=1) every guarded global or
// peer access first checks its byte range against the extent the host passed for that buffer; a
// violation is RECORDED (first code / count / source line / offending value, read through
// eri_<file>_debug_bounds) and the access is SKIPPED, so an indexing bug shows up as a report
// instead of a fault. In the normal build the macros expand to nothing / `true`. This is the
// stand-in for a memory checker on machines where none can be run.
#ifdef ERI_DEBUG_BOUNDS
#define ERI_DEBUG_BOUNDS_DEFINE(tag)                                                              \
  static __device__ int g_dbg_bounds[4];                                                          \
  static __device__ __forceinline__ bool eri_dbg_violation(int code, long long value, int line) { \
    if (atomicAdd(&g_dbg_bounds[1], 1) == 0) {                                                    \
      g_dbg_bounds[0] = code;                                                                     \
      g_dbg_bounds[2] = line;                                                                     \
      g_dbg_bounds[3] = (int)value;                                                               \
    }                                                                                             \
    return false;                                                                                 \
  }
// the exported reader: placed at file scope (outside any unnamed namespace) so that it is visible
#define ERI_DEBUG_BOUNDS_EXPORT(tag)                                                              \
  extern "C" int eri_##tag##_debug_bounds(int* out4) {                                            \
    int z[4] = {0, 0, 0, 0};                                                                      \
    if (cudaMemcpyFromSymbol(out4, g_dbg_bounds, sizeof(z)) != cudaSuccess) return -1;            \
    cudaMemcpyToSymbol(g_dbg_bounds, z, sizeof(z));                                               \
    return out4[1];                                                                               \
  }
#define ERI_DBG_VIOLATION(code, value) eri_dbg_violation(code, (long long)(value), __LINE__)
// true when [ptr, ptr + n) lies inside [base, base + extent) (extent 0: unknown, not checked)
#define ERI_DBG_RANGE(base, extent, ptr, n, code)                                                 \
  ((extent) == 0 ||                                                                               \
   ((const char*)(ptr) >= (const char*)(base) &&                                                  \
    (const char*)(ptr) + (n) <= (const char*)(base) + (extent)) ||                                \
   ERI_DBG_VIOLATION(code, (const char*)(ptr) - (const char*)(base)))
#define ERI_DBG_INDEX(i, n, code) (((i) >= 0 && (i) < (n)) || ERI_DBG_VIOLATION(code, i))
#else
#define ERI_DEBUG_BOUNDS_DEFINE(tag)
#define ERI_DEBUG_BOUNDS_EXPORT(tag)
#define ERI_DBG_VIOLATION(code, value) false
#define ERI_DBG_RANGE(base, extent, ptr, n, code) true
#define ERI_DBG_INDEX(i, n, code) true
#endif

// ----------------------------------------------------------------- small math helpers
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}
__device__ __forceinline__ float gelu_tanh_grad_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float x2 = x * x;
  float u = k0 * (x + k1 * x * x2);
  float t = tanhf(u);
  float du = k0 * (1.f + 3.f * k1 * x2);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float silu_grad_f(float x) {
  float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

// Eight bf16 values moved as ONE 128-bit access. The payload is a uint4 so that copying the
// struct through a pointer compiles to a single LDG.128 / STG.128; with four __nv_bfloat162
// members the compiler emitted four 32-bit accesses (4 useful bytes per 32-byte sector in the
// row-per-thread GEMM epilogue).
struct alignas(16) bf16x8 {
  uint4 u;
};
__device__ __forceinline__ float2 bf162_bits_to_float2(uint32_t w) {
  // bf16 -> fp32 is a 16-bit shift
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ void unpack8(const bf16x8& p, float (&f)[8]) {
  const uint4 u = p.u;
  float2 t;
  t = bf162_bits_to_float2(u.x); f[0] = t.x; f[1] = t.y;
  t = bf162_bits_to_float2(u.y); f[2] = t.x; f[3] = t.y;
  t = bf162_bits_to_float2(u.z); f[4] = t.x; f[5] = t.y;
  t = bf162_bits_to_float2(u.w); f[6] = t.x; f[7] = t.y;
}
__device__ __forceinline__ uint32_t pack_bf162(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 p;
  p.u = make_uint4(pack_bf162(f[0], f[1]), pack_bf162(f[2], f[3]), pack_bf162(f[4], f[5]),
                   pack_bf162(f[6], f[7]));
  return p;
}

// ---- packed fp32 pairs (two fp32 lanes per 64-bit register; sm_100 executes add / mul / fma on
// both lanes in one instruction, which halves the issue slots of softmax-style loops)
typedef uint64_t f32x2;
__device__ __forceinline__ f32x2 f2_pack(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ f32x2 f2_pack_bits(uint32_t lo, uint32_t hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 f2_sub(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^x on the special-function unit: one instruction, flushes denormal results to zero.
__device__ __forceinline__ float ex2_mufu(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for a pair on the FMA pipe (no special-function unit): round-to-nearest split x = n + f with
// f in [-0.5, 0.5] by the 1.5*2^23 trick, cubic minimax polynomial for 2^f (max relative error
// 7.5e-5, well under bf16 rounding), exponent added by an integer multiply-add. x is clamped at
// -126 so the result stays normal; the caller guarantees x <= 127.
__device__ __forceinline__ f32x2 ex2_poly2(f32x2 x) {
  float x0, x1;
  f2_unpack(x, x0, x1);
  x0 = fmaxf(x0, -126.f);
  x1 = fmaxf(x1, -126.f);
  x = f2_pack(x0, x1);
  const f32x2 magic = f2_pack(12582912.f, 12582912.f);
  const f32x2 t = f2_add(x, magic);
  const f32x2 f = f2_sub(x, f2_sub(t, magic));
  f32x2 p = f2_pack(0.0551716685f, 0.0551716685f);
  p = f2_fma(p, f, f2_pack(0.2426111251f, 0.2426111251f));
  p = f2_fma(p, f, f2_pack(0.6932609677f, 0.6932609677f));
  p = f2_fma(p, f, f2_pack(0.9999280572f, 0.9999280572f));
  uint32_t t0, t1, p0, p1;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(t0), "=r"(t1) : "l"(t));
  asm("mov.b64 {%0, %1}, %2;" : "=r"(p0), "=r"(p1) : "l"(p));
  // the low mantissa bits of t hold n (two's complement in the 23-bit field); n << 23 added to
  // the bits of p scales it by 2^n
  p0 += t0 << 23;
  p1 += t1 << 23;
  return f2_pack_bits(p0, p1);
}
// Same, with an exact zero where x < -125 (a masked key carries a bias of -1e30: its probability and
// therefore its gradients must be exactly zero, as the special-function unit gives them).
__device__ __forceinline__ f32x2 ex2_poly2_z(f32x2 x) {
  float x0, x1;
  f2_unpack(x, x0, x1);
  float r0, r1;
  f2_unpack(ex2_poly2(x), r0, r1);
  return f2_pack(x0 < -125.f ? 0.f : r0, x1 < -125.f ? 0.f : r1);
}
// round a pair to packed bf16 (low half = lo)
__device__ __forceinline__ uint32_t f2_to_bf162(f32x2 v) {
  float lo, hi;
  f2_unpack(v, lo, hi);
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

}  // namespace eri
