// Two-CTA (cta_group::2) variant of the bf16 GEMM: a pair of CTAs on one TPC computes a 256x256
// output tile with tcgen05.mma M=256. Each CTA stages its own 128 rows of A and ONE HALF of the B
// tile (128 of the 256 columns), so a K step costs 32 KB of shared-memory fill per SM instead of
// 48 KB for the single-CTA 128x256 tile — the single-CTA kernel is bound by the latency x
// bandwidth product of its operand ring (tensor pipe ~52 % active in its profile), and the pair
// tile cuts the bytes per flop by a third and deepens the ring to six stages.
//
// Roles per CTA: warp 0 TMA producer (both CTAs; completion bytes of both land on the leader's
// `full` barrier), warp 1 UMMA issuer (leader CTA only; tcgen05.commit arrives on the `empty` /
// `acc_full` barriers of BOTH CTAs with two plain commits), warps 2-5 epilogue for the CTA's own
// 128 accumulator rows (peer epilogue warps arrive remotely on the leader's `acc_empty`).
// No multicast of any kind is used: every CTA issues its own loads.
//
// Same fused epilogue family and LoRA K step as gemm.cu (bias, GELU/SiLU + saved pre-activation,
// activation backward, gate + residual, column split, MN-major B, operand gathers, peer scatter
// through staged rows), plus:
//   * MN-major A ([K, M] row-major): with an MN-major B this is the weight-gradient product
//     dW[N_out, K_in] = dY[T, N_out]^T X[T, K_in] read straight from the token-major activations;
//     the `residual` epilogue input (same buffer as `out`) gives the beta = 1 accumulation into an
//     existing gradient.
//   * gated-linear-unit epilogue (GEGLU / SwiGLU, the reference's fused feed-forward kernel,
//     crates/training/src/sdxl/runtime.rs:249-321): the pair's two CTAs stage the B rows of the
//     FIRST and of the SECOND half of an up-projection [2*hidden, K], so one 256-column accumulator
//     holds 128 value columns next to their 128 gate columns and the epilogue writes
//     out[M, hidden] = a * act(b) (or act(a) * b) and, for backward, the raw halves.
#include "ptx.cuh"
#include "tma_host.h"
#include "gather_copy.cuh"
#include "gemm_args.h"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

struct Gemm2Params {
  int M, N, K, num_k;
  int lora_r, act, n_split;
  int ldc, ldc2, ld_pre, ldr;
  int rows_per_batch, gate_stride;
  int b_mn, a_mn;
  int glu, glu_hidden;        // glu: 0 off, 1 a*gelu(b), 2 a*silu(b), 3 gelu(a)*b, 4 silu(a)*b
  float alpha;
  const bf16* bias;
  const bf16* residual;
  const bf16* gate;
  const bf16* pre_in;
  bf16* out;
  bf16* out2;
  bf16* pre_out;
  int* err;
  unsigned long long* stamps;   // optional %globaltimer phase record of a gather launch (gemm_args.h)
  int join_round;               // gather mode: > 0 = copy clusters compute tiles from this round on
  int all_flag;                 // gather mode: 1 + index of the counter every copy job bumps (0: none)
  // gather mode (see gather_copy.cuh): the first n_copy CTAs (whole clusters) run copy jobs
  int n_copy, n_jobs;
  const GatherJob* jobs;
  unsigned int* flags;
  const unsigned int* flag_target;
  int b_flag_rows;            // rows of B per landing counter (0: B is not gathered)
  int a_flag_cols;            // K columns per counter of a K-gathered A operand (0: none)
  int a_flag_rows, a_row_groups;
  int rot_n, rot_k;           // rotation of the tile order / K order towards the local slab
  // 1: B rows [loc_lo, loc_hi) are read from this rank's own shard (tensor map tmBL, row - loc_lo);
  // 2: K range [loc_lo, loc_hi) of an MN-major B likewise; 3: K range [loc_lo, loc_hi) of the A
  // operand (tmBL then maps A[:, loc_lo:loc_hi] in its home buffer). Those slabs have no copy jobs.
  int loc_mode, loc_lo, loc_hi;
  // peer scatter epilogue (as in gemm.cu): all columns of a pair tile belong to one (part, rank) group
  int scatter_world, scatter_rank, scatter_part_cols, scatter_group_cols, scatter_local_rows;
  int scatter_mode;           // 0 column groups, 1 row slabs (see gemm_args.h)
  bf16* scatter_out[kMaxPeers];
  float* rowsq;
  int rowsq_parts;
  long long dbg_out_bytes, dbg_out2_bytes, dbg_pre_bytes, dbg_res_bytes;   // debug build only
  // Grouped launch (two plain products with the same N, K, operand majors, LoRA rank and epilogue
  // kind, e.g. the image and the text stream of a dual-stream block): tiles [0, group_tiles0) belong
  // to this problem, the rest to the second parameter block. 0: a single problem. total_tiles: all.
  int group_tiles0, total_tiles;
};

ERI_DEBUG_BOUNDS_DEFINE(gemm2)

constexpr int BM = 128;       // rows per CTA (256 per pair)
constexpr int BN = 256;       // columns per pair tile
constexpr int BNH = 128;      // B rows staged per CTA
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STG_PITCH = BN * 2 + 16;   // staged epilogue: one padded accumulator row per thread
constexpr int kGroupN = 8;

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int rot_n, int& m_blk,
                                            int& n_blk) {
  const int group_sz = kGroupN * num_m;
  const int g = t / group_sz;
  const int first_n = g * kGroupN;
  const int gw = min(num_n - first_n, kGroupN);
  const int r = t - g * group_sz;
  n_blk = first_n + r % gw;
  m_blk = r / gw;
  if (rot_n) {
    n_blk += rot_n;
    if (n_blk >= num_n) n_blk -= num_n;
  }
}
// Tile schedule of a persistent launch. Round r hands one tile to every participating cluster. In
// gather mode the copy clusters take part from round `join` on (they move slabs first), so rounds
// below `join` are `cc` tiles wide and later rounds `cc + cx`:
//   compute cluster i: tile(r) = r * cc + i                               (r <  join)
//                      tile(r) = join * cc + (r - join) * (cc + cx) + i   (r >= join)
//   copy cluster j   : starts at r = join with slot cc + j.
// Without copy clusters (cx = 0) this is the plain stride-cc walk.
struct TileSched {
  int cc, cx, join, slot, first_round;
  __device__ __forceinline__ int tile(int r) const {
    return r < join ? r * cc + slot : join * cc + (r - join) * (cc + cx) + slot;
  }
};
__device__ __forceinline__ float apply_act(float v, int act) {
  return act == 1 ? gelu_tanh_f(v) : act == 2 ? silu_f(v) : v;
}
__device__ __forceinline__ float apply_act_grad(float pre, int act) {
  return act == 3 ? gelu_tanh_grad_f(pre) : silu_grad_f(pre);
}

// STAGED: the epilogue writes each accumulator row to shared memory and sends it with one bulk
// asynchronous copy (the peer scatter, whose destination rows live on other GPUs).
template <int STAGES, bool STAGED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(320, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA_0, const __grid_constant__ CUtensorMap tmB_0,
                  const __grid_constant__ CUtensorMap tmA2_0, const __grid_constant__ CUtensorMap tmB2_0,
                  const __grid_constant__ CUtensorMap tmBL, const __grid_constant__ Gemm2Params p0,
                  const __grid_constant__ CUtensorMap tmA_1, const __grid_constant__ CUtensorMap tmB_1,
                  const __grid_constant__ CUtensorMap tmA2_1, const __grid_constant__ CUtensorMap tmB2_1,
                  const __grid_constant__ Gemm2Params p1) {
  // Launch-wide state comes from the first parameter block; inside the tile loops `p` and the
  // operand maps are re-bound per tile to the problem the tile belongs to (grouped launch).
  const Gemm2Params& p = p0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  if (p.stamps && threadIdx.x == 0) atomicMin(p.stamps + 0, (unsigned long long)globaltimer_ns());
  if ((int)blockIdx.x < p.n_copy) {
    // copy clusters (n_copy is even): both CTAs move slabs and leave; they take no part in the
    // cluster barriers or the tensor-memory allocation of the compute clusters. The copy ring reuses
    // the operand stages' shared memory; its barriers sit where the GEMM's do.
    constexpr int RING = (STAGES * STAGE_BYTES) / kCopyStageBytes;
    copy_role(p, smem, RING < 6 ? RING : 6, (int)blockIdx.x);
    if (p.stamps) {
      __syncthreads();
      if (threadIdx.x == 0) atomicMax(p.stamps + 1, (unsigned long long)globaltimer_ns());
    }
    if (p.join_round <= 0) return;
    // This cluster now joins the tile loop. The copy ring's barriers sit where the GEMM's are set up
    // below: every copy of the ring has completed (each job ends with a full store drain), so they
    // are invalidated before the memory becomes the GEMM's barriers.
    __syncthreads();
    if (threadIdx.x == 0) {
      uint64_t* rb = reinterpret_cast<uint64_t*>(smem + (size_t)(RING < 6 ? RING : 6) * kCopyStageBytes);
      for (int i = 0; i < 2 * (RING < 6 ? RING : 6); ++i) mbar_inval(&rb[i]);
    }
    __syncthreads();
  }
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  uint8_t* stg = smem + STAGES * STAGE_BYTES + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);    // leader: one arrive.expect_tx per phase (+ bytes of both CTAs)
      mbar_init(&empty[s], 1);   // one commit arrival per phase
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 2 * ((blockDim.x >> 5) - 2));  // epilogue warps x 2 CTAs (used on the leader only)
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // both CTAs' barriers are initialised before any remote use
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // GLU: a tile is 128 output columns (value rows from the first half of B, gate rows from the second)
  const int num_n = p.glu ? (p.glu_hidden + BNH - 1) / BNH : (p.N + BN - 1) / BN;
  const int tiles = p.total_tiles;     // both problems of a grouped launch
  const int k_iters = p.num_k + (p.lora_r > 0 ? 1 : 0);
  const bool was_copy = (int)blockIdx.x < p.n_copy;
  TileSched sched;
  sched.cc = ((int)gridDim.x - p.n_copy) >> 1;
  sched.cx = p.join_round > 0 ? p.n_copy >> 1 : 0;
  sched.join = p.join_round > 0 ? p.join_round : 0x3fffffff;
  sched.slot = was_copy ? sched.cc + ((int)blockIdx.x >> 1) : ((int)blockIdx.x - p.n_copy) >> 1;
  sched.first_round = was_copy ? sched.join : 0;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      bool dep_done = false;
      unsigned long long waited = 0;   // ns spent on slab counters (recorded only with p.stamps)
      bool all_landed = false;         // sticky: the gather has finished, no slab counter needs a look
      for (int r = sched.first_round; ok; ++r) {
        const int t = sched.tile(r);
        if (t >= tiles) break;
        // grouped launch: this tile's problem, its operand maps and its tile index within the problem
        const bool g1 = p0.group_tiles0 > 0 && t >= p0.group_tiles0;
        const Gemm2Params& p = g1 ? p1 : p0;
        const CUtensorMap& tmA = g1 ? tmA_1 : tmA_0;
        const CUtensorMap& tmB = g1 ? tmB_1 : tmB_0;
        const CUtensorMap& tmA2 = g1 ? tmA2_1 : tmA2_0;
        const CUtensorMap& tmB2 = g1 ? tmB2_1 : tmB2_0;
        const int num_m = (p.M + 2 * BM - 1) / (2 * BM);
        int m_blk, n_blk;
        tile_coords(g1 ? t - p0.group_tiles0 : t, num_m, num_n, p.rot_n, m_blk, n_blk);
        const int m0 = m_blk * 2 * BM + (int)rank * BM;
        const int n0 = p.glu ? n_blk * BNH + (int)rank * p.glu_hidden : n_blk * BN + (int)rank * BNH;
        const bool b_rows_local = p.loc_mode == 1 && n0 >= p.loc_lo && n0 + BNH <= p.loc_hi;
        if (p.all_flag && !all_landed) {
          all_landed = ld_acquire_gpu(p.flags + (p.all_flag - 1)) >= p.flag_target[p.all_flag - 1];
          if (all_landed) fence_proxy_async_all();
        }
        if (p.b_flag_rows && !b_rows_local && !all_landed) {
          // every slab that the B rows staged by THIS CTA touch must have landed
          const int f0 = n0 / p.b_flag_rows, f1 = (min(n0 + BNH, p.N) - 1) / p.b_flag_rows;
          const unsigned long long tw = p.stamps ? globaltimer_ns() : 0ull;
          for (int f = f0; f <= f1 && ok; ++f)
            if (!wait_slab(p, f)) {
              atomicExch(p.err, 45);
              ok = false;
            }
          if (p.stamps) waited += globaltimer_ns() - tw;
          if (!ok) break;
          fence_proxy_async_all();
        }
        int a_ready = -1;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            atomicExch(p.err, 41);
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          if (k < p.num_k) {
            int kk = k + p.rot_k;
            if (kk >= p.num_k) kk -= p.num_k;
            const bool k_local = p.loc_mode >= 2 && kk * BK >= p.loc_lo && kk * BK + BK <= p.loc_hi;
            if (p.a_flag_cols && !k_local && !all_landed) {
              int f = (kk * BK) / p.a_flag_cols;
              if (p.a_flag_rows) f = f * p.a_row_groups + min(m0, p.M - 1) / p.a_flag_rows;
              if (f != a_ready) {
                const unsigned long long tw = p.stamps ? globaltimer_ns() : 0ull;
                if (!wait_slab(p, f)) {
                  atomicExch(p.err, 46);
                  ok = false;
                  break;
                }
                if (p.stamps) waited += globaltimer_ns() - tw;
                fence_proxy_async_all();
                a_ready = f;
              }
            }
            if (leader) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);
            if (p.a_mn) {
              tma_load_2d_pair(sA, &tmA, bar, m0, kk * BK);
              tma_load_2d_pair(sA + BK * 128, &tmA, bar, m0 + 64, kk * BK);
            } else if (p.loc_mode == 3 && k_local) {
              tma_load_2d_pair(sA, &tmBL, bar, kk * BK - p.loc_lo, m0);
            } else {
              tma_load_2d_pair(sA, &tmA, bar, kk * BK, m0);
            }
            if (!p.b_mn) {
              if (b_rows_local) tma_load_2d_pair(sB, &tmBL, bar, kk * BK, n0 - p.loc_lo);
              else tma_load_2d_pair(sB, &tmB, bar, kk * BK, n0);
            } else {
              const bool bl = k_local && p.loc_mode == 2;
              const CUtensorMap* tb = bl ? &tmBL : &tmB;
              const int ky = bl ? kk * BK - p.loc_lo : kk * BK;
              tma_load_2d_pair(sB, tb, bar, n0, ky);
              tma_load_2d_pair(sB + BK * 128, tb, bar, n0 + 64, ky);
            }
          } else {
            // lora_h may still be in production by the previous kernel (dependent launch)
            if (!dep_done) {
              griddep_wait();
              dep_done = true;
            }
            if (leader) mbar_expect_tx(&full[stage], 2 * (BM + BNH) * p.lora_r * 2);
            tma_load_2d_pair(sA, &tmA2, bar, 0, m0);
            tma_load_2d_pair(sB, &tmB2, bar, 0, n0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (p.stamps && waited) {
        atomicAdd(p.stamps + 3, waited);
        atomicMax(p.stamps + 4, waited);
        atomicAdd(p.stamps + 5, 1ull);
      }
    }
  } else if (warp == 1) {
    if (leader && elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      const uint32_t idesc = umma_idesc_bf16(256, BN, p.a_mn, p.b_mn);
      const uint32_t idesc_lora = umma_idesc_bf16(256, BN, 0, 0);
      for (int r = sched.first_round; ok && sched.tile(r) < tiles; ++r, ++it) {
        const int buf = it & 1;
        const uint32_t use = (uint32_t)(it >> 1);
        if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1)) {
          atomicExch(p.err, 42);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&full[stage], phase)) {
            atomicExch(p.err, 43);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sB = sA + A_BYTES;
          if (k < p.num_k) {
            const uint64_t da = umma_desc_kmajor(sA, 128);
            if (p.a_mn) {
              // both operands token-major (weight gradient): 16 K rows are 2048 bytes apart
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk)
                umma2_bf16(d_tmem, umma_desc_mn128(sA + kk * 2048, BK * 128),
                           p.b_mn ? umma_desc_mn128(sB + kk * 2048, BK * 128)
                                  : umma_desc_kmajor(sB, 128) + kk * 2,
                           idesc, (k | kk) != 0);
            } else if (!p.b_mn) {
              const uint64_t db = umma_desc_kmajor(sB, 128);
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk)
                umma2_bf16(d_tmem, da + kk * 2, db + kk * 2, idesc, (k | kk) != 0);
            } else {
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk)
                umma2_bf16(d_tmem, da + kk * 2, umma_desc_mn128(sB + kk * 2048, BK * 128), idesc,
                           (k | kk) != 0);
            }
          } else {
            const uint32_t sw = p.lora_r * 2;
            const uint64_t da = umma_desc_kmajor(sA, sw), db = umma_desc_kmajor(sB, sw);
            for (int kk = 0; kk < p.lora_r / 16; ++kk)
              umma2_bf16(d_tmem, da + kk * 2, db + kk * 2, idesc_lora, (k | kk) != 0);
          }
          const uint32_t e = smem_u32(&empty[stage]);
          umma2_commit_addr(e);
          umma2_commit_addr(map_to_cta(e, 1));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          const uint32_t a = smem_u32(&acc_full[buf]);
          umma2_commit_addr(a);
          umma2_commit_addr(map_to_cta(a, 1));
        }
      }
    }
  } else {
    // Four epilogue warps (one per 32-row TMEM quadrant) or eight: with eight, warps w and w + 4 share a
    // quadrant and split the tile's columns in halves, which halves the time a tile spends in the epilogue
    // (~10 us with four warps: with K = 3072 that is close to the main loop's ~19 us as soon as the epilogue
    // reads or writes a second tensor). Plain launches run with eight, gather / scatter launches with four.
    const int q = warp & 3;
    const int n_half = ((int)(blockDim.x >> 5) - 2) >> 2;        // 1 or 2
    const int half = (warp - 2) >> 2;                            // 0, or 1 for the second set of four warps
    const int c_lo = n_half == 2 ? half * (BN / 64) : 0, c_hi = n_half == 2 ? c_lo + BN / 64 : BN / 32;
    int it = 0;
    for (int r = sched.first_round; sched.tile(r) < tiles; ++r, ++it) {
      const int t = sched.tile(r);
      const bool g1 = p0.group_tiles0 > 0 && t >= p0.group_tiles0;
      const Gemm2Params& p = g1 ? p1 : p0;     // this tile's problem (grouped launch)
      const int num_m = (p.M + 2 * BM - 1) / (2 * BM);
      int m_blk, n_blk;
      tile_coords(g1 ? t - p0.group_tiles0 : t, num_m, num_n, p.rot_n, m_blk, n_blk);
      const int m0 = m_blk * 2 * BM + (int)rank * BM, n0 = p.glu ? n_blk * BNH : n_blk * BN;
      const int buf = it & 1;
      const uint32_t use = (uint32_t)(it >> 1);
      if (!mbar_wait(&acc_full[buf], use & 1)) {
        if (lane == 0) atomicExch(p.err, 44);
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t acc_addr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
      if (p.glu) {
        // columns [0,128) of the accumulator: first half of the up-projection, [128,256): second half
        bf16* dst = p.out + (size_t)row * p.ldc;
        const bool act_first = p.glu >= 3;
        const int amode = (p.glu == 1 || p.glu == 3) ? 1 : 2;
#pragma unroll 1
        for (int c = (n_half == 2 ? half * (BNH / 64) : 0); c < (n_half == 2 ? (half + 1) * (BNH / 64) : BNH / 32); ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.glu_hidden) break;
          uint32_t ra[32], rb[32];
          tmem_ld32(acc_addr + c * 32, ra);
          tmem_ld32(acc_addr + BNH + c * 32, rb);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = col0 + g * 8;
              if (col < p.glu_hidden) {
                float va[8], vb[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  va[j] = __uint_as_float(ra[g * 8 + j]) * p.alpha;
                  vb[j] = __uint_as_float(rb[g * 8 + j]) * p.alpha;
                }
                if (p.bias) {
                  float b0[8], b1[8];
                  unpack8(*reinterpret_cast<const bf16x8*>(p.bias + col), b0);
                  unpack8(*reinterpret_cast<const bf16x8*>(p.bias + p.glu_hidden + col), b1);
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    va[j] += b0[j];
                    vb[j] += b1[j];
                  }
                }
                if (p.pre_out) {
                  // the halves are kept as bf16 (what the unfused path would have stored); the
                  // product below uses the same rounded values so that backward sees its inputs
                  bf16* pr = p.pre_out + (size_t)row * p.ld_pre;
                  const bf16x8 pa = pack8(va), pb = pack8(vb);
                  *reinterpret_cast<bf16x8*>(pr + col) = pa;
                  *reinterpret_cast<bf16x8*>(pr + p.glu_hidden + col) = pb;
                  unpack8(pa, va);
                  unpack8(pb, vb);
                }
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  v[j] = act_first ? apply_act(va[j], amode) * vb[j] : va[j] * apply_act(vb[j], amode);
                if (ERI_DBG_RANGE(p.out, p.dbg_out_bytes, dst + col, 16, 94))
                  *reinterpret_cast<bf16x8*>(dst + col) = pack8(v);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
        continue;
      }
      const bool second = p.n_split >= 0 && n0 >= p.n_split;
      const int act = second || p.n_split < 0 ? p.act : 0;
      const int coff = second ? p.n_split : 0;
      bf16* dst = second && p.out2 ? p.out2 + (size_t)row * p.ldc2 : p.out + (size_t)row * p.ldc;
      int dcol_off = second && p.out2 ? coff : 0;
      if (p.scatter_world && p.scatter_mode == 1) {
        // row slabs: this thread's output row belongs to rank row / slab; it lands in this rank's
        // slot of the owner's receive buffer, same columns
        const int dest = row_ok ? row / p.scatter_local_rows : 0;
        const size_t drow = (size_t)p.scatter_rank * p.scatter_local_rows + (row - dest * p.scatter_local_rows);
        dst = p.scatter_out[dest] + drow * p.ldc;
        dcol_off = 0;
      } else if (p.scatter_world) {
        // all columns of a tile belong to one (part, rank) group
        const int part = n0 / p.scatter_part_cols;
        const int within = n0 - part * p.scatter_part_cols;
        const int dest = within / p.scatter_group_cols;
        const int bidx = row_ok ? row / p.scatter_local_rows : 0;
        const int lrow = row - bidx * p.scatter_local_rows;
        const size_t drow = (size_t)bidx * p.scatter_world * p.scatter_local_rows +
                            (size_t)p.scatter_rank * p.scatter_local_rows + lrow;
        dst = p.scatter_out[dest] + drow * p.ldc;
        // destination column = part * group_cols + (col % group_cols)
        dcol_off = n0 - (part * p.scatter_group_cols + (within - dest * p.scatter_group_cols));
      }
      const bf16* gate = p.gate ? p.gate + (size_t)(row_ok ? row / p.rows_per_batch : 0) * p.gate_stride
                                : nullptr;
      uint8_t* stg_row = stg + (size_t)(q * 32 + lane) * STG_PITCH;
      if constexpr (STAGED) {
        // this thread's previous row copy must have read its staging row before it is rewritten
        if (it > 0) tma_store_wait_read<0>();
      }
      float sq = 0.f;
      // The residual / stored pre-activation of a row chunk is fetched one chunk ahead: a 16-byte load per
      // thread from its own row has nothing to overlap with when it is issued in the middle of the
      // chunk's arithmetic, and with a short K loop (K = 3072) the epilogue is on the critical path.
      const bf16* ex_res = (p.residual && row_ok) ? p.residual + (size_t)row * p.ldr : nullptr;
      const bf16* ex_pre = ((act == 3 || act == 4) && row_ok) ? p.pre_in + (size_t)row * p.ld_pre - coff : nullptr;
      uint4 nx_res[4], nx_pre[4];
      auto fetch = [&](int c) {
        const int col0 = n0 + c * 32;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int col = col0 + g * 8;
          if (col < p.N) {
            if (ex_res && ERI_DBG_RANGE(p.residual, p.dbg_res_bytes, ex_res + col, 16, 93))
              nx_res[g] = *reinterpret_cast<const uint4*>(ex_res + col);
            if (ex_pre) nx_pre[g] = *reinterpret_cast<const uint4*>(ex_pre + col);
          }
        }
      };
      if ((ex_res || ex_pre) && n0 + c_lo * 32 < p.N) fetch(c_lo);
#pragma unroll 1
      for (int c = c_lo; c < c_hi; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;
        uint4 cur_res[4], cur_pre[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          cur_res[g] = nx_res[g];
          cur_pre[g] = nx_pre[g];
        }
        if ((ex_res || ex_pre) && c + 1 < c_hi && col0 + 32 < p.N) fetch(c + 1);
        uint32_t r[32];
        tmem_ld32(acc_addr + c * 32, r);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = col0 + g * 8;
            if (col < p.N) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]) * p.alpha;
              if (p.bias) {
                float b[8];
                unpack8(*reinterpret_cast<const bf16x8*>(p.bias + col), b);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += b[j];
              }
              if (act == 1 || act == 2) {
                if (p.pre_out && ERI_DBG_RANGE(p.pre_out, p.dbg_pre_bytes,
                                               p.pre_out + (size_t)row * p.ld_pre + (col - coff), 16, 92))
                  *reinterpret_cast<bf16x8*>(p.pre_out + (size_t)row * p.ld_pre + (col - coff)) =
                      pack8(v);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = apply_act(v[j], act);
              } else if (act == 3 || act == 4) {
                float pr[8];
                bf16x8 pv;
                pv.u = cur_pre[g];
                unpack8(pv, pr);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= apply_act_grad(pr[j], act);
              }
              if (gate) {
                float gt[8];
                unpack8(*reinterpret_cast<const bf16x8*>(gate + col), gt);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= gt[j];
              }
              if (p.residual && ERI_DBG_RANGE(p.residual, p.dbg_res_bytes,
                                              p.residual + (size_t)row * p.ldr + col, 16, 93)) {
                float rs[8];
                bf16x8 rv;
                rv.u = cur_res[g];
                unpack8(rv, rs);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += rs[j];
              }
              if (p.rowsq) {
#pragma unroll
                for (int j = 0; j < 8; ++j) sq += v[j] * v[j];
              }
              if constexpr (STAGED) {
                *reinterpret_cast<bf16x8*>(stg_row + (size_t)(col - n0) * 2) = pack8(v);
              } else {
                const bool to2 = second && p.out2;
                if (ERI_DBG_RANGE(to2 ? p.out2 : p.out, to2 ? p.dbg_out2_bytes : p.dbg_out_bytes,
                                  dst + (col - dcol_off), 16, 91))
                  *reinterpret_cast<bf16x8*>(dst + (col - dcol_off)) = pack8(v);
              }
            }
          }
        }
      }
      if constexpr (STAGED) {
        // the row was written by this thread alone: order it before the async proxy reads it, then
        // one bulk copy carries the whole row to its (possibly remote) destination
        fence_proxy_async_all();
        if (row_ok) {
          const int ncols = min(BN, p.N - n0);
          bulk_s2g_plain(dst + (n0 - dcol_off), smem_u32(stg_row), (uint32_t)ncols * 2u);
        }
        tma_store_commit();
      }
      if (p.rowsq && row_ok && p.scatter_mode == 0) {
        const int part = n0 / p.scatter_part_cols;
        if (part < p.rowsq_parts) atomicAdd(p.rowsq + (size_t)part * p.M + row, sq);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
    }
    if constexpr (STAGED) tma_store_wait<0>();   // every row copy of this thread has completed
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer may still read this CTA's shared memory / signal its barriers
  if (p.stamps && threadIdx.x == 0) atomicMax(p.stamps + 2, (unsigned long long)globaltimer_ns());
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc2(tmem_base, 512);
  }
}

int g2_num_sms = 0;
int* g2_err = nullptr;
long long g2_gather_launches = 0;   // gather-mode launches that ran on this kernel (host counter)

// Operand maps of one problem: A, B, LoRA rank-r operands (H, up-matrix) and the in-place local slab.
struct Gemm2Maps {
  CUtensorMap ta, tb, ta2, tb2, tbl;
};

// p / m: the (first) problem; pg / mg: the second problem of a grouped launch (the same objects as
// p / m for a single problem: the kernel never looks at them then).
template <int STAGES, bool STAGED>
int launch2(const Gemm2Maps& m, Gemm2Params& p, const Gemm2Maps& mg, const Gemm2Params& pg, int tiles, int pdl,
            cudaStream_t st) {
  const CUtensorMap &ta = m.ta, &tb = m.tb, &ta2 = m.ta2, &tb2 = m.tb2, &tbl = m.tbl;
  p.total_tiles = tiles;
  constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256 + (STAGED ? BM * STG_PITCH : 0);
  auto kern = gemm2_bf16_kernel<STAGES, STAGED>;
  int dev = 0;
  cudaGetDevice(&dev);
  static bool configured[64] = {};
  if (dev < 0 || dev >= 64) return -36;
  if (!configured[dev]) {
    // the attribute belongs to the (function, device) pair
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return -36;
    configured[dev] = true;
  }
  if (p.n_copy > 0) {
    // The compute clusters spin on counters that the copy clusters bump, so every CTA of the grid
    // must be resident: the grid is sized by the cluster occupancy query and launched cooperatively.
    static int coop_clusters = -1;
    if (coop_clusters < 0) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(g2_num_sms / 2 * 2);
      cfg.blockDim = dim3(192);
      cfg.dynamicSmemBytes = SMEM;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      cfg.attrs = at;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
      }
      coop_clusters = n;
    }
    const int room = coop_clusters - p.n_copy / 2;
    if (room < 8) return -30;
    const int clusters = tiles < room ? tiles : room;
    void* args[] = {(void*)&ta, (void*)&tb, (void*)&ta2, (void*)&tb2, (void*)&tbl, (void*)&p,
                    (void*)&mg.ta, (void*)&mg.tb, (void*)&mg.ta2, (void*)&mg.tb2, (void*)&pg};
    cudaError_t e = cudaLaunchCooperativeKernel((const void*)kern, dim3(p.n_copy + clusters * 2),
                                                dim3(192), args, SMEM, st);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return -30;   // the caller falls back to the one-CTA kernel
    }
    ++g2_gather_launches;
    return 0;
  }
  const int max_clusters = g2_num_sms / 2;
  const int clusters = tiles < max_clusters ? tiles : max_clusters;
  // plain launches: eight epilogue warps (ERI_B200_GEMM_EPI_WARPS=4 keeps four); the staged epilogue of the
  // peer scatter keeps one thread per accumulator row
  static int epi_warps = 0;
  if (!epi_warps) {
    const char* e = getenv("ERI_B200_GEMM_EPI_WARPS");
    epi_warps = (e && e[0] == '4') ? 4 : 8;
  }
  const int threads = (STAGED || p.scatter_world) ? 192 : 64 + 32 * epi_warps;
  if (pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(clusters * 2);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, ta, tb, ta2, tb2, tbl, p, mg.ta, mg.tb, mg.ta2, mg.tb2, pg);
  }
  kern<<<clusters * 2, threads, SMEM, st>>>(ta, tb, ta2, tb2, tbl, p, mg.ta, mg.tb, mg.ta2, mg.tb2, pg);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

typedef EriGemmArgs EriGemmArgs2;

int eri_gemm2_gather_count() { return (int)g2_gather_launches; }

int eri_gemm2_check_error() {
  if (!g2_err) return 0;
  int h = 0;
  cudaMemcpy(&h, g2_err, sizeof(int), cudaMemcpyDeviceToHost);
  if (h) cudaMemset(g2_err, 0, sizeof(int));
  return h;
}

}  // extern "C"

namespace {

// Validates one problem and fills its parameter block and operand maps. Returns 0, or the negative
// code the entry points hand back (-30: the problem does not fit this kernel). `tiles_out`: its tiles.
int build_problem(const EriGemmArgs* g, Gemm2Params& p, Gemm2Maps& m, int& tiles_out) {
  const bool scatter = g->scatter_world != 0;
  if (g->rowsq && !scatter) return -30;
  if (scatter && g->scatter_mode == 1) {
    // row slabs (weight-gradient reduce-scatter): any operand majors, plain epilogue only
    if ((g->ldc * 2) % 16 || g->n_copy || g->glu || g->rowsq || g->scatter_local_rows <= 0 || g->N % 8 ||
        g->M != g->scatter_world * g->scatter_local_rows)
      return -30;
  } else if (scatter) {
    // a pair tile must sit inside one (part, rank) column group; rows leave through 16-byte aligned
    // bulk copies
    if (g->scatter_group_cols % BN || g->scatter_part_cols % BN || (g->ldc * 2) % 16 || g->n_copy ||
        g->glu || g->a_mn)
      return -30;
  }
  if (g->n_copy) {
    // gather mode: whole copy clusters, rotations in whole pair tiles / K blocks
    if (g->n_copy % 2 || g->n_copy < 0 || g->n_copy > 64) return -30;
    if (g->rot_n_rows % BN || g->rot_k_cols % BK || g->a_flag_cols % BK || g->a_flag_rows % BM) return -30;
    if (g->a_mn || g->glu) return -30;
  }
  if (g->glu) {
    // N counts the rows of the up-projection weight (both halves); the output has N / 2 columns
    if (g->glu < 1 || g->glu > 4 || g->N % 2 || (g->N / 2) % 8 || g->N / 2 < BNH || g->b_mn || g->a_mn ||
        g->n_split > 0 || g->act || g->residual || g->gate || g->out2)
      return -30;
  }
  if (g->a_mn && (g->lora_r || g->M % 8)) return -30;
  if (g->M < 256 || g->N < 256 || g->K < 64) return -30;
  // a dimension that is contiguous in memory must keep rows 16-byte aligned
  if ((!(g->a_mn && g->b_mn) && g->K % 8) || g->N % 8 || g->lda % 8 || g->ldb % 8 || g->ldc % 8) return -30;
  if (g->lora_r && g->lora_r != 16 && g->lora_r != 32 && g->lora_r != 64) return -30;
  if (g->n_split > 0 && g->n_split % BN) return -30;
  if (!g2_err) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g2_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaMalloc(&g2_err, sizeof(int)) != cudaSuccess) return -31;
    cudaMemset(g2_err, 0, sizeof(int));
  }
  memset(&p, 0, sizeof(p));
  p.M = g->M; p.N = g->N; p.K = g->K; p.num_k = (g->K + BK - 1) / BK;
  p.lora_r = g->lora_r; p.act = g->act; p.n_split = g->n_split > 0 ? g->n_split : -1;
  p.ldc = g->ldc; p.ldc2 = g->ldc2; p.ld_pre = g->ld_pre; p.ldr = g->ldr;
  p.rows_per_batch = g->rows_per_batch > 0 ? g->rows_per_batch : g->M;
  p.gate_stride = g->gate_stride; p.alpha = g->alpha; p.b_mn = g->b_mn; p.a_mn = g->a_mn ? 1 : 0;
  p.glu = g->glu; p.glu_hidden = g->glu ? g->N / 2 : 0;
  p.bias = (const bf16*)g->bias; p.residual = (const bf16*)g->residual;
  p.gate = (const bf16*)g->gate; p.pre_in = (const bf16*)g->pre_in;
  p.out = (bf16*)g->out; p.out2 = (bf16*)g->out2; p.pre_out = (bf16*)g->pre_out;
  p.err = g2_err;
  p.dbg_out_bytes = g->dbg_out_bytes; p.dbg_out2_bytes = g->dbg_out2_bytes;
  p.dbg_pre_bytes = g->dbg_pre_bytes; p.dbg_res_bytes = g->dbg_res_bytes;
  p.stamps = g->n_copy ? g->stamps : nullptr;
  p.join_round = g->n_copy ? g->join_round : 0;
  p.all_flag = g->n_copy ? g->all_flag : 0;
  p.n_copy = g->n_copy; p.n_jobs = g->n_jobs; p.jobs = (const GatherJob*)g->jobs;
  p.flags = (unsigned int*)g->flags; p.flag_target = (const unsigned int*)g->flag_target;
  p.b_flag_rows = g->b_flag_rows; p.a_flag_cols = g->a_flag_cols; p.a_flag_rows = g->a_flag_rows;
  p.a_row_groups = g->a_flag_rows > 0 ? (g->M + g->a_flag_rows - 1) / g->a_flag_rows : 0;
  p.rot_n = g->rot_n_rows / BN; p.rot_k = g->rot_k_cols / BK;
  if (scatter) {
    p.scatter_world = g->scatter_world; p.scatter_rank = g->scatter_rank;
    p.scatter_part_cols = g->scatter_part_cols; p.scatter_group_cols = g->scatter_group_cols;
    p.scatter_local_rows = g->scatter_local_rows > 0 ? g->scatter_local_rows : g->M;
    p.scatter_mode = g->scatter_mode;
    for (int i = 0; i < kMaxPeers; ++i) p.scatter_out[i] = (bf16*)g->scatter_out[i];
    p.rowsq = (float*)g->rowsq; p.rowsq_parts = g->rowsq_parts;
  }
  const bool use_local = g->n_copy && g->b_local && g->jobs_nl && g->flag_target_nl &&
                         !(((uintptr_t)g->b_local) & 15) && g->ldb_local % 8 == 0 &&
                         ((g->loc_mode == 1 && !g->b_mn && g->loc_lo % BNH == 0 && g->loc_hi % BNH == 0) ||
                          (g->loc_mode == 2 && g->b_mn && g->loc_lo % BK == 0 && g->loc_hi % BK == 0) ||
                          (g->loc_mode == 3 && g->loc_lo % BK == 0 && g->loc_hi % BK == 0));
  if (use_local) {
    p.loc_mode = g->loc_mode; p.loc_lo = g->loc_lo; p.loc_hi = g->loc_hi;
    p.n_jobs = g->n_jobs_nl; p.jobs = (const GatherJob*)g->jobs_nl;
    p.flag_target = (const unsigned int*)g->flag_target_nl;
  }

  CUtensorMap &ta = m.ta, &tb = m.tb, &ta2 = m.ta2, &tb2 = m.tb2, &tbl = m.tbl;
  if (!g->a_mn) {
    uint64_t d[2] = {(uint64_t)g->K, (uint64_t)g->M};
    uint64_t s[1] = {(uint64_t)g->lda * 2};
    uint32_t bx[2] = {BK, BM};
    if (make_tensor_map(&ta, g->a, 2, d, s, bx, 128)) return -32;
  } else {
    uint64_t d[2] = {(uint64_t)g->M, (uint64_t)g->K};     // A given as [K, M]
    uint64_t s[1] = {(uint64_t)g->lda * 2};
    uint32_t bx[2] = {64, BK};
    if (make_tensor_map(&ta, g->a, 2, d, s, bx, 128)) return -32;
  }
  if (!g->b_mn) {
    uint64_t d[2] = {(uint64_t)g->K, (uint64_t)g->N};
    uint64_t s[1] = {(uint64_t)g->ldb * 2};
    uint32_t bx[2] = {BK, BNH};
    if (make_tensor_map(&tb, g->b, 2, d, s, bx, 128)) return -33;
  } else {
    uint64_t d[2] = {(uint64_t)g->N, (uint64_t)g->K};
    uint64_t s[1] = {(uint64_t)g->ldb * 2};
    uint32_t bx[2] = {64, BK};
    if (make_tensor_map(&tb, g->b, 2, d, s, bx, 128)) return -33;
  }
  if (g->lora_r) {
    uint64_t d[2] = {(uint64_t)g->lora_r, (uint64_t)g->M};
    uint64_t s[1] = {(uint64_t)g->ld_h * 2};
    uint32_t bx[2] = {(uint32_t)g->lora_r, BM};
    if (make_tensor_map(&ta2, g->lora_h, 2, d, s, bx, g->lora_r * 2)) return -34;
    uint64_t d2[2] = {(uint64_t)g->lora_r, (uint64_t)g->N};
    uint64_t s2[1] = {(uint64_t)g->ld_lb * 2};
    uint32_t bx2[2] = {(uint32_t)g->lora_r, BNH};
    if (make_tensor_map(&tb2, g->lora_b, 2, d2, s2, bx2, g->lora_r * 2)) return -35;
  } else {
    ta2 = ta;
    tb2 = tb;
  }
  tbl = tb;
  if (use_local) {
    const uint64_t rows = (uint64_t)(g->loc_hi - g->loc_lo);
    uint64_t s[1] = {(uint64_t)g->ldb_local * 2};
    if (g->loc_mode == 1) {
      uint64_t d[2] = {(uint64_t)g->K, rows};
      uint32_t bx[2] = {BK, BNH};
      if (make_tensor_map(&tbl, g->b_local, 2, d, s, bx, 128)) return -33;
    } else if (g->loc_mode == 2) {
      uint64_t d[2] = {(uint64_t)g->N, rows};
      uint32_t bx[2] = {64, BK};
      if (make_tensor_map(&tbl, g->b_local, 2, d, s, bx, 128)) return -33;
    } else {
      uint64_t d[2] = {rows, (uint64_t)g->M};      // A[:, loc_lo:loc_hi] in its home buffer
      uint32_t bx[2] = {BK, BM};
      if (make_tensor_map(&tbl, g->b_local, 2, d, s, bx, 128)) return -33;
    }
  }
  const int n_tiles = g->glu ? (g->N / 2 + BNH - 1) / BNH : (g->N + BN - 1) / BN;
  tiles_out = ((g->M + 2 * BM - 1) / (2 * BM)) * n_tiles;
  return 0;
}

}  // namespace

extern "C" {

// Returns -30 when the problem does not fit this kernel (caller falls back to eri_gemm_bf16).
int eri_gemm2_bf16(const EriGemmArgs2* g, void* stream) {
  Gemm2Params p;
  Gemm2Maps m;
  int tiles = 0;
  const int code = build_problem(g, p, m, tiles);
  if (code) return code;
  cudaStream_t st = (cudaStream_t)stream;
  // four operand stages leave room for the 128 staged accumulator rows of the peer scatter
  if (g->scatter_world) return launch2<4, true>(m, p, m, p, tiles, 0, st);
  return launch2<6, false>(m, p, m, p, tiles, g->pdl && g->lora_r, st);
}

// Two plain products in ONE launch: the tiles of the second follow the tiles of the first in the
// persistent schedule, so a small second problem (the 512-token text stream of a dual-stream block:
// 24-96 tiles) runs in the last, partly empty round of the first instead of as a launch of its own
// that leaves most SMs idle. Both must have the same N, K, operand majors, LoRA rank, activation and
// column split, and neither may use gather, scatter, GLU or token-major A. Returns -30 when the pair
// does not qualify (the caller then launches them one by one).
int eri_gemm2_bf16_group2(const EriGemmArgs2* g0, const EriGemmArgs2* g1, void* stream) {
  const EriGemmArgs2* gs[2] = {g0, g1};
  for (const EriGemmArgs2* g : gs)
    if (g->scatter_world || g->n_copy || g->glu || g->a_mn || g->rowsq) return -30;
  if (g0->N != g1->N || g0->K != g1->K || g0->b_mn != g1->b_mn || g0->lora_r != g1->lora_r || g0->act != g1->act ||
      g0->n_split != g1->n_split || g0->alpha != g1->alpha || (g0->out2 != nullptr) != (g1->out2 != nullptr))
    return -30;
  Gemm2Params p0, p1;
  Gemm2Maps m0, m1;
  int t0 = 0, t1 = 0;
  int code = build_problem(g0, p0, m0, t0);
  if (code) return code;
  code = build_problem(g1, p1, m1, t1);
  if (code) return code;
  p0.group_tiles0 = t0;
  return launch2<6, false>(m0, p0, m1, p1, t0 + t1, g0->pdl && g1->pdl && g0->lora_r, (cudaStream_t)stream);
}

}  // extern "C"

ERI_DEBUG_BOUNDS_EXPORT(gemm2)
