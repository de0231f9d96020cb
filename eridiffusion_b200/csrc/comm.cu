// Communication kernels over NVLink peer memory (one process per GPU; buffers are cudaMalloc'ed
// and exported with CUDA IPC, so every rank holds a device pointer to every peer's buffer).
//
//   fused_dp_step   data-parallel gradient reduce-scatter + global-norm clip + block-wise 8-bit
//                   AdamW on this rank's shard + all-gather of the updated parameters, ONE
//                   cooperative kernel: peers' gradient shards are pulled with 16-byte loads,
//                   reduced in fp32 registers, the squared norm is exchanged through peer slots,
//                   the update runs on the shard, and the new bf16 parameters are pushed to every
//                   peer's arena with 16-byte stores.
//   collectives     barrier, all-gather, reduce-scatter, all-reduce (two-shot), all-to-all,
//                   broadcast as pull-based peer-memory kernels.
//
// Cross-GPU synchronisation is a monotonically increasing epoch written into per-peer flag words
// (st.release.sys / ld.acquire.sys). Every wait has a wall-clock bound; when it runs out the kernel
// records (phase, peer) in a status word and continues to its normal exit, so a missing peer can
// never hang the GPU. No multimem / multicast object is bound here: plain peer loads and stores.
//
// The reference's collectives are stubs (crates/training/src/distributed.rs:155-183) and its DDP
// wrapper flattens a bucket and "all-reduces" it by dividing by the world size (:284-319).
#include <cooperative_groups.h>

#include "ptx.cuh"
#include "optim_codec.cuh"

namespace cg = cooperative_groups;
using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kMaxWorld = 16;
constexpr int kBlock = 256;  // optimizer quantisation block

struct Peers {
  void* ptr[kMaxWorld];
};

struct CommCtx {
  uint32_t* flags_local;           // [channels][world]
  uint32_t* flags_peer[kMaxWorld]; // each peer's flags_local
  int rank, world;
  uint32_t epoch;
  unsigned long long wait_ns;
  int* err;                        // status word: 0 ok, else (phase << 8) | peer
};

// Block 0 signals every peer and waits for every peer; the caller follows with grid.sync().
__device__ void cross_barrier(const CommCtx& c, int channel, cg::grid_group& grid) {
  grid.sync();  // all of this GPU's prior writes are done
  if (blockIdx.x == 0 && threadIdx.x < c.world) {
    const int p = threadIdx.x;
    __threadfence_system();
    st_release_sys(c.flags_peer[p] + channel * c.world + c.rank, c.epoch);
    const uint32_t* mine = c.flags_local + channel * c.world + p;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - c.epoch) < 0) {
      if ((++spins & 255u) == 0u && globaltimer_ns() - t0 > c.wait_ns) {
        atomicCAS(c.err, 0, ((channel + 1) << 8) | p);
        break;
      }
    }
  }
  grid.sync();
}

__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ bf16 round_bf16(float v, bool stochastic, uint32_t rnd) {
  if (!stochastic) return __float2bfloat16(v);
  uint32_t bits = __float_as_uint(v);
  if ((bits & 0x7f800000u) == 0x7f800000u) return __float2bfloat16(v);
  bits += rnd & 0xffffu;
  return __ushort_as_bfloat16((unsigned short)(bits >> 16));
}

struct FusedDpArgs {
  Peers grads;        // every rank's gradient arena (bf16)
  Peers params;       // every rank's parameter arena (bf16)
  Peers sumsq_slots;  // every rank's float[world] slot array
  float* reduced;     // local scratch: fp32 reduced gradient shard [shard_elems]
  float* sumsq_local; // local fp32 accumulator (zeroed by the kernel at exit for the next call)
  int8_t* mq;         // optimizer state of this rank's shard
  uint8_t* vq;
  float* m_absmax;
  float* v_absmax;
  long long shard_elems;  // multiple of 256
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, max_grad_norm;
  uint32_t seed;
  int stochastic;
  float* grad_norm_out;   // optional: global gradient norm of this step
  unsigned long long* stamps;  // optional: %globaltimer at the six phase boundaries (thread 0)
};

__device__ __forceinline__ void stamp(const FusedDpArgs& a, int i) {
  if (a.stamps && blockIdx.x == 0 && threadIdx.x == 0) a.stamps[i] = globaltimer_ns();
}

__global__ void __launch_bounds__(256, 4)
fused_dp_step_kernel(CommCtx c, FusedDpArgs a) {
  cg::grid_group grid = cg::this_grid();
  __shared__ float red[32];
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long gwarp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nblocks = a.shard_elems / kBlock;
  const long long shard_off = (long long)c.rank * a.shard_elems;
  const float inv_world = 1.f / (float)c.world;

  // phase 0: every rank's backward has finished writing its gradient arena
  stamp(a, 0);
  cross_barrier(c, 0, grid);
  stamp(a, 1);

  // phase 1: reduce-scatter (pull) into fp32 scratch + local sum of squares
  float ss = 0.f;
  for (long long blk = gwarp; blk < nblocks; blk += warps) {
    const long long e = blk * kBlock + lane * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // issue every peer's 16-byte load before the first add, so that one NVLink round trip is
    // paid per block instead of one per peer
    for (int i0 = 0; i0 < c.world; i0 += 8) {
      bf16x8 raw[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (i0 + i < c.world) {
          int p = c.rank + i0 + i;           // start at self, stagger peers
          if (p >= c.world) p -= c.world;
          raw[i] = *reinterpret_cast<const bf16x8*>(reinterpret_cast<const bf16*>(a.grads.ptr[p]) +
                                                   shard_off + e);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (i0 + i < c.world) {
          float f[8];
          unpack8(raw[i], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += f[j];
        }
      }
    }
    float4 o0, o1;
    o0.x = acc[0] * inv_world; o0.y = acc[1] * inv_world; o0.z = acc[2] * inv_world; o0.w = acc[3] * inv_world;
    o1.x = acc[4] * inv_world; o1.y = acc[5] * inv_world; o1.z = acc[6] * inv_world; o1.w = acc[7] * inv_world;
    ss += o0.x * o0.x + o0.y * o0.y + o0.z * o0.z + o0.w * o0.w + o1.x * o1.x + o1.y * o1.y +
          o1.z * o1.z + o1.w * o1.w;
    float4* dst = reinterpret_cast<float4*>(a.reduced + e);
    dst[0] = o0;
    dst[1] = o1;
  }
  ss = warp_sum(ss);
  if (lane == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) atomicAdd(a.sumsq_local, t);
  }
  grid.sync();
  stamp(a, 2);

  // phase 2: publish this shard's squared norm to every peer, then wait for all of them
  if (blockIdx.x == 0 && threadIdx.x < c.world) {
    const float mine = *reinterpret_cast<volatile float*>(a.sumsq_local);
    float* slot = reinterpret_cast<float*>(a.sumsq_slots.ptr[threadIdx.x]) + c.rank;
    asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(slot), "f"(mine) : "memory");
  }
  cross_barrier(c, 1, grid);
  stamp(a, 3);
  float total = 0.f;
  {
    const float* slots = reinterpret_cast<const float*>(a.sumsq_slots.ptr[c.rank]);
    for (int p = 0; p < c.world; ++p) {
      float v;
      asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(slots + p) : "memory");
      total += v;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0 && a.grad_norm_out) *a.grad_norm_out = sqrtf(total);
  const bool finite = isfinite(total);
  // A bounded wait of this launch (or of an earlier one that the host has not read yet) ran out:
  // the reduced gradient may be partial. The word was written before the grid-wide sync that ends
  // cross_barrier, so every thread of the grid reads the same value and the whole grid skips the
  // update: parameters and optimizer state stay as they were and nothing is pushed to the peers.
  const bool comm_ok = *reinterpret_cast<volatile int*>(c.err) == 0;
  float gs = 1.f;
  if (a.max_grad_norm > 0.f) gs = fminf(1.f, a.max_grad_norm / (sqrtf(total) + 1e-6f));

  // phase 3: 8-bit AdamW on the shard, push new parameters to every rank
  if (finite && comm_ok) {
    Adam8Consts k;
    adam8_consts(k, a.beta1, a.beta2, a.eps, a.bc1, a.bc2, gs);
    for (long long blk = gwarp; blk < nblocks; blk += warps) {
      const long long e = blk * kBlock + lane * 8;
      bf16* own = reinterpret_cast<bf16*>(a.params.ptr[c.rank]) + shard_off + e;
      const uint4 pw = *reinterpret_cast<const uint4*>(own);
      const float4* gp = reinterpret_cast<const float4*>(a.reduced + e);
      const float4 g0 = gp[0], g1 = gp[1];
      const f32x2 g2[4] = {f2_pack(g0.x, g0.y), f2_pack(g0.z, g0.w), f2_pack(g1.x, g1.y), f2_pack(g1.z, g1.w)};
      const uint2 mraw = *reinterpret_cast<const uint2*>(a.mq + e);
      const uint2 vraw = *reinterpret_cast<const uint2*>(a.vq + e);
      f32x2 m2[4], sv2[4], p2[4];
      float mmax, vmax;
      adam8_update8(k, g2, pw, mraw, vraw, a.m_absmax[blk], a.v_absmax[blk], a.lr, a.weight_decay, m2, sv2,
                    p2, mmax, vmax);
      mmax = warp_max(mmax);
      vmax = warp_max(vmax);
      uint2 mo, vo;
      uint4 pq;
      adam8_encode8(m2, sv2, p2, mmax, vmax, a.stochastic != 0, a.seed, (uint32_t)(shard_off + e), mo, vo, pq);
      bf16x8 po;
      po.u = pq;
      *reinterpret_cast<uint2*>(a.mq + e) = mo;
      *reinterpret_cast<uint2*>(a.vq + e) = vo;
      if (lane == 0) {
        a.m_absmax[blk] = mmax;
        a.v_absmax[blk] = vmax;
      }
      for (int i = 0; i < c.world; ++i) {
        const int q = (c.rank + i) % c.world;
        bf16* dst = reinterpret_cast<bf16*>(a.params.ptr[q]) + shard_off + e;
        *reinterpret_cast<bf16x8*>(dst) = po;
      }
    }
  }
  // phase 4: all ranks have pushed their shards (and finished reading every gradient arena)
  stamp(a, 4);
  cross_barrier(c, 2, grid);
  stamp(a, 5);
  if (blockIdx.x == 0 && threadIdx.x == 0) *a.sumsq_local = 0.f;
}

// ---------------------------------------------------------------------------- generic collectives
enum { OP_ALLGATHER = 0, OP_REDUCE_SCATTER = 1, OP_ALLREDUCE = 2, OP_ALLTOALL = 3, OP_BROADCAST = 4,
       OP_BARRIER = 5 };

struct CollArgs {
  Peers src;          // every rank's source buffer
  void* dst;          // local destination
  Peers dst_peers;    // every rank's destination (all-reduce second shot)
  long long count;    // elements per rank chunk (16-byte multiple in bytes)
  int op, dtype;      // dtype: 0 bf16, 1 fp32
  int root, avg;
};

template <typename TT>
__device__ __forceinline__ void load16(const void* p, float (&f)[8], int& n);
template <>
__device__ __forceinline__ void load16<bf16>(const void* p, float (&f)[8], int& n) {
  unpack8(*reinterpret_cast<const bf16x8*>(p), f);
  n = 8;
}
template <>
__device__ __forceinline__ void load16<float>(const void* p, float (&f)[8], int& n) {
  float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  n = 4;
}
template <typename TT>
__device__ __forceinline__ void store16(void* p, const float (&f)[8]);
template <>
__device__ __forceinline__ void store16<bf16>(void* p, const float (&f)[8]) {
  *reinterpret_cast<bf16x8*>(p) = pack8(f);
}
template <>
__device__ __forceinline__ void store16<float>(void* p, const float (&f)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}

template <typename TT>
__global__ void __launch_bounds__(256) collective_kernel(CommCtx c, CollArgs a) {
  cg::grid_group grid = cg::this_grid();
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  constexpr int EPV = 16 / sizeof(TT);  // elements per 16-byte vector
  const long long nvec = a.count / EPV;
  cross_barrier(c, 3, grid);  // sources are ready everywhere
  if (a.op == OP_ALLGATHER || a.op == OP_ALLTOALL || a.op == OP_BROADCAST) {
    const int first = a.op == OP_BROADCAST ? a.root : 0;
    const int last = a.op == OP_BROADCAST ? a.root + 1 : c.world;
    for (int i = first; i < last; ++i) {
      const int p = a.op == OP_BROADCAST ? i : (c.rank + i) % c.world;
      // all-gather: peer p's whole chunk -> dst chunk p; all-to-all: peer p's chunk `rank` -> dst chunk p
      const long long soff = a.op == OP_ALLTOALL ? (long long)c.rank * a.count : 0;
      const long long doff = a.op == OP_BROADCAST ? 0 : (long long)p * a.count;
      const uint4* s = reinterpret_cast<const uint4*>(reinterpret_cast<const TT*>(a.src.ptr[p]) + soff);
      uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<TT*>(a.dst) + doff);
      for (long long v = tid; v < nvec; v += nth) d[v] = s[v];
    }
  } else if (a.op == OP_REDUCE_SCATTER || a.op == OP_ALLREDUCE) {
    const float sc = a.avg ? 1.f / (float)c.world : 1.f;
    for (long long v = tid; v < nvec; v += nth) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      int n = 0;
      for (int i = 0; i < c.world; ++i) {
        const int p = (c.rank + i) % c.world;
        float f[8];
        load16<TT>(reinterpret_cast<const TT*>(a.src.ptr[p]) + (long long)c.rank * a.count + v * EPV, f, n);
        for (int j = 0; j < n; ++j) acc[j] += f[j];
      }
      for (int j = 0; j < n; ++j) acc[j] *= sc;
      if (a.op == OP_REDUCE_SCATTER) {
        store16<TT>(reinterpret_cast<TT*>(a.dst) + v * EPV, acc);
      } else {  // second shot: push the reduced chunk into every rank's destination
        for (int i = 0; i < c.world; ++i) {
          const int q = (c.rank + i) % c.world;
          store16<TT>(reinterpret_cast<TT*>(a.dst_peers.ptr[q]) + (long long)c.rank * a.count + v * EPV, acc);
        }
      }
    }
  }
  cross_barrier(c, 4, grid);  // everyone finished reading sources / writing destinations
}

int g_coop_blocks_fused = 0, g_coop_blocks_coll = 0;

int coop_grid(const void* fn, int& cache) {
  if (cache) return cache;
  int dev = 0, sms = 0, per = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, fn, 256, 0);
  if (per < 1) per = 1;
  if (per > 4) per = 4;
  cache = sms * per;
  return cache;
}

}  // namespace

extern "C" {

int eri_symm_malloc(long long bytes, void** out) { return (int)cudaMalloc(out, (size_t)bytes); }

// Copy-engine leg of a gather: one asynchronous device-to-device copy from a peer's (IPC-mapped)
// buffer into local memory, then ``n_flags`` 32-bit stream memory writes of ``value`` starting at
// ``flags`` (one per landing counter the copied slab covers). Both are stream operations executed by
// the copy engine / front end, not kernels, so a GEMM that is already running and waits (bounded)
// on those counters cannot starve them of SMs. Returns 0 on success.
int eri_peer_copy_flags(void* dst, const void* src, long long bytes, void* flags, int n_flags,
                        unsigned int value, void* stream) {
  typedef int (*WriteValue32Fn)(void* /*CUstream*/, unsigned long long /*CUdeviceptr*/, unsigned int,
                                unsigned int);
  static WriteValue32Fn write32 = nullptr;
  static bool looked = false;
  if (!looked) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      write32 = reinterpret_cast<WriteValue32Fn>(p);
    looked = true;
  }
  if (!write32) return -1;
  cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  for (int i = 0; i < n_flags; ++i) {
    const int r = write32(stream, (unsigned long long)(uintptr_t)flags + 4ull * i, value, 0u);
    if (r != 0) return 1000 + r;
  }
  return 0;
}
int eri_symm_free(void* p) { return (int)cudaFree(p); }
int eri_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
int eri_ipc_open_handle(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
int eri_ipc_close_handle(void* p) { return (int)cudaIpcCloseMemHandle(p); }
int eri_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }

struct EriCommCtx {
  void* flags_local;
  void* flags_peer[kMaxWorld];
  int rank, world;
  unsigned int epoch;
  unsigned long long wait_ns;
  void* err;
};

static CommCtx to_ctx(const EriCommCtx* h) {
  CommCtx c;
  c.flags_local = (uint32_t*)h->flags_local;
  for (int i = 0; i < kMaxWorld; ++i) c.flags_peer[i] = (uint32_t*)h->flags_peer[i];
  c.rank = h->rank; c.world = h->world; c.epoch = h->epoch;
  c.wait_ns = h->wait_ns ? h->wait_ns : 2000000000ull;
  c.err = (int*)h->err;
  return c;
}

struct EriFusedDpArgs {
  void* grads[kMaxWorld];
  void* params[kMaxWorld];
  void* sumsq_slots[kMaxWorld];
  void* reduced;
  void* sumsq_local;
  void* mq;
  void* vq;
  void* m_absmax;
  void* v_absmax;
  void* grad_norm_out;
  long long shard_elems;
  float lr, beta1, beta2, eps, weight_decay, max_grad_norm;
  int step;
  unsigned int seed;
  int stochastic;
  void* stamps;  // optional uint64[6]: device timer at the phase boundaries
};

int eri_fused_dp_step(const EriCommCtx* h, const EriFusedDpArgs* g, void* stream) {
  if (h->world < 1 || h->world > kMaxWorld || g->shard_elems % kBlock || g->step < 1) return -1;
  CommCtx c = to_ctx(h);
  FusedDpArgs a;
  for (int i = 0; i < kMaxWorld; ++i) {
    a.grads.ptr[i] = g->grads[i];
    a.params.ptr[i] = g->params[i];
    a.sumsq_slots.ptr[i] = g->sumsq_slots[i];
  }
  a.reduced = (float*)g->reduced; a.sumsq_local = (float*)g->sumsq_local;
  a.mq = (int8_t*)g->mq; a.vq = (uint8_t*)g->vq;
  a.m_absmax = (float*)g->m_absmax; a.v_absmax = (float*)g->v_absmax;
  a.shard_elems = g->shard_elems;
  a.lr = g->lr; a.beta1 = g->beta1; a.beta2 = g->beta2; a.eps = g->eps;
  a.weight_decay = g->weight_decay; a.max_grad_norm = g->max_grad_norm;
  a.bc1 = 1.f - powf(g->beta1, (float)g->step);
  a.bc2 = 1.f - powf(g->beta2, (float)g->step);
  a.seed = g->seed * 2654435761u + g->step; a.stochastic = g->stochastic;
  a.grad_norm_out = (float*)g->grad_norm_out;
  a.stamps = (unsigned long long*)g->stamps;
  const int grid = coop_grid((const void*)fused_dp_step_kernel, g_coop_blocks_fused);
  void* args[] = {&c, &a};
  return (int)cudaLaunchCooperativeKernel((const void*)fused_dp_step_kernel, dim3(grid), dim3(256),
                                          args, 0, (cudaStream_t)stream);
}

struct EriCollArgs {
  void* src[kMaxWorld];
  void* dst_peers[kMaxWorld];
  void* dst;
  long long count;
  int op, dtype, root, avg;
};

int eri_collective(const EriCommCtx* h, const EriCollArgs* g, void* stream) {
  if (h->world < 1 || h->world > kMaxWorld) return -1;
  const int esz = g->dtype == 0 ? 2 : 4;
  if ((g->count * esz) % 16) return -2;
  CommCtx c = to_ctx(h);
  CollArgs a;
  for (int i = 0; i < kMaxWorld; ++i) {
    a.src.ptr[i] = g->src[i];
    a.dst_peers.ptr[i] = g->dst_peers[i];
  }
  a.dst = g->dst; a.count = g->count; a.op = g->op; a.dtype = g->dtype; a.root = g->root; a.avg = g->avg;
  void* args[] = {&c, &a};
  if (g->dtype == 0) {
    const int grid = coop_grid((const void*)collective_kernel<bf16>, g_coop_blocks_coll);
    return (int)cudaLaunchCooperativeKernel((const void*)collective_kernel<bf16>, dim3(grid),
                                            dim3(256), args, 0, (cudaStream_t)stream);
  }
  static int cache_f32 = 0;
  const int grid = coop_grid((const void*)collective_kernel<float>, cache_f32);
  return (int)cudaLaunchCooperativeKernel((const void*)collective_kernel<float>, dim3(grid), dim3(256),
                                          args, 0, (cudaStream_t)stream);
}

}  // extern "C"
