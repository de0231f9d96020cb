// Persistent warp-specialised bf16 GEMM for sm_100a:  C[M,N] = epilogue(A[M,K] * op(B))
//
//   warp 0      TMA producer: cp.async.bulk.tensor tiles (128-byte swizzle) into a STAGES-deep ring
//   warp 1      UMMA issuer: tcgen05.mma (M=128, N=BN, K=16) from shared memory into TMEM;
//               tcgen05.commit releases ring slots and publishes finished accumulators
//   warps 2-5   epilogue: tcgen05.ld the fp32 accumulator (two TMEM buffers, so tile i drains
//               while tile i+1 accumulates), apply the fused epilogue, store bf16
//
// B is either [N, K] row-major (K-major operand, a weight used as y = x W^T) or [K, N] row-major
// (MN-major operand: the same weight tensor W[N_out, K_in] read as dX = dY W without a transposed
// copy).
//
// Fused epilogue (all optional): alpha, bias[N], GELU(tanh)/SiLU with the pre-activation kept
// for backward, activation backward (multiply by f'(pre)), adaLN gate + residual
// (out = R + gate[batch] * y), a column split that routes columns >= n_split (with the
// activation) to a second destination, and a peer scatter that stores each head group's columns
// straight into the owning rank's buffer over NVLink (Ulysses all-to-all folded into the QKV
// projection).
//
// LoRA: Y = X W^T + (s X A^T) B^T is one launch for the rank-r product H = s X A^T (the streaming
// kernel of gemm_rank_stream.cu) followed by the main launch, which appends one extra K step whose operands are
// H[M,r] and B[N,r]; the low-rank update lands in the same TMEM accumulator before the epilogue,
// so no [M,N] delta tensor is ever written. (Reference: two library GEMMs, a scale and an add per
// site, crates/training/src/flux/lora.rs:47-63, crates/training/src/flux/runtime.rs:555-600.)
//
// Gather mode (ZeRO-3 parameter all-gather / Ulysses reverse all-to-all fused with the GEMM):
// the first `n_copy` CTAs of the same launch do not compute; they pull slabs of an operand from
// peer GPUs (bulk asynchronous copies through a shared-memory ring, gather_copy.cuh) into a local
// landing buffer and bump a per-slab counter.
// The TMA producer of every compute CTA waits (bounded) on the counter of the slab it is about to
// load, and tile / K order start at this rank's own slab, so the math on slabs that have landed
// overlaps the transfer of the rest. The launch is cooperative, which guarantees the copy CTAs are
// resident. Remote data is always read from local memory by TMA, never with a multicast load.
#include "ptx.cuh"
#include "tma_host.h"
#include "gather_copy.cuh"
#include "gemm_args.h"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

struct GemmParams {
  int M, N, K, num_k;
  int lora_r;          // 0, 16, 32 or 64
  int act;             // 0 none, 1 GELU(tanh) fwd, 2 SiLU fwd, 3 GELU bwd, 4 SiLU bwd
  int n_split;         // columns >= n_split take the activation and go to out2 (tile aligned)
  int ldc, ldc2, ld_pre, ldr;
  int rows_per_batch, gate_stride;
  int b_mn;            // B given as [K, N] (MN-major operand)
  float alpha;
  const bf16* bias;
  const bf16* residual;
  const bf16* gate;
  const bf16* pre_in;   // indexed with (col - n_split)
  bf16* out;
  bf16* out2;           // indexed with (col - n_split)
  bf16* pre_out;        // indexed with (col - n_split)
  int* err;
  // gather mode
  int all_flag;               // 1 + index of the counter every copy job bumps (0: none)
  int n_copy;                 // leading CTAs that run copy jobs
  int n_jobs;
  const GatherJob* jobs;
  unsigned int* flags;        // per-slab counters (zeroed before the launch)
  const unsigned int* flag_target;
  int b_flag_rows;            // rows of B per slab (0: B is not gathered)
  int a_flag_cols;            // K columns per counter of a K-gathered operand (0: none)
  int a_flag_rows;            // >0: counters also split by row group of the A operand:
  int a_row_groups;           //     index = (k / a_flag_cols) * a_row_groups + m0 / a_flag_rows
  int rot_n, rot_k;           // rotation of tile order / K order towards the local slab
  int pdl;                    // launched as a programmatic dependent of the kernel that writes lora_h
  // peer scatter epilogue
  int scatter_world;          // 0: off
  int scatter_rank;
  int scatter_part_cols;      // columns of one part (q, k or v) = H * Dh
  int scatter_group_cols;     // columns of one rank's head group = (H / world) * Dh
  int scatter_local_rows;     // tokens per batch element on this rank
  bf16* scatter_out[kMaxPeers];
  float* rowsq;               // optional [rowsq_parts][M]: sum of squares of each output row over
  int rowsq_parts;            // the columns of part 0..rowsq_parts-1 (QK-norm across heads)
  long long dbg_out_bytes, dbg_out2_bytes, dbg_pre_bytes, dbg_res_bytes;   // debug build only
};

ERI_DEBUG_BOUNDS_DEFINE(gemm)

constexpr int BM = 128, BK = 64;
constexpr int kGroupN = 8;

__host__ __device__ constexpr int tmem_cols_for(int bn) {
  return 2 * bn <= 32 ? 32 : 2 * bn <= 64 ? 64 : 2 * bn <= 128 ? 128 : 2 * bn <= 256 ? 256 : 512;
}

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

__device__ __forceinline__ float apply_act(float v, int act) {
  return act == 1 ? gelu_tanh_f(v) : act == 2 ? silu_f(v) : v;
}
__device__ __forceinline__ float apply_act_grad(float pre, int act) {
  return act == 3 ? gelu_tanh_grad_f(pre) : silu_grad_f(pre);
}

// STAGED: the epilogue writes each accumulator row to shared memory first and sends it with ONE
// bulk asynchronous copy per row (BN * 2 bytes) instead of one 16-byte store per 8 columns. Used by
// the peer scatter, where a row's destination is another GPU: NVLink then carries 512-byte writes
// and the epilogue warps do not wait for remote stores before they release the accumulator.
template <int BN, int STAGES, bool STAGED>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                 const __grid_constant__ GemmParams p) {
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = tmem_cols_for(BN);
  constexpr int CH = BN >= 32 ? 32 : 16;  // accumulator columns per TMEM load

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  if ((int)blockIdx.x < p.n_copy) {
    // the copy ring reuses the operand stages' shared memory; its barriers sit where the GEMM's do
    constexpr int RING = (STAGES * STAGE_BYTES) / kCopyStageBytes;
    copy_role(p, smem, RING < 6 ? RING : 6, (int)blockIdx.x);
    return;
  }
  const int worker = blockIdx.x - p.n_copy;
  const int nworkers = gridDim.x - p.n_copy;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  // staged epilogue: one padded row per epilogue thread (the 16-byte pad spreads the rows over banks)
  constexpr int STG_PITCH = BN * 2 + 16;
  uint8_t* stg = smem + STAGES * STAGE_BYTES + 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int tiles = num_m * num_n;
  const int k_iters = p.num_k + (p.lora_r > 0 ? 1 : 0);
  const uint32_t idesc = umma_idesc_bf16(BM, BN, 0, p.b_mn);

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      bool dep_done = false;
      for (int t = worker; t < tiles && ok; t += nworkers) {
        int m_blk, n_blk;
        tile_coords(t, num_m, num_n, p.rot_n, m_blk, n_blk);
        const int m0 = m_blk * BM, n0 = n_blk * BN;
        if (p.b_flag_rows) {
          // every slab this tile's B rows touch must have landed
          const int f0 = n0 / p.b_flag_rows, f1 = (min(n0 + BN, p.N) - 1) / p.b_flag_rows;
          for (int f = f0; f <= f1 && ok; ++f)
            if (!wait_slab(p, f)) {
              atomicExch(p.err, 5);
              ok = false;
            }
          if (!ok) break;
          fence_proxy_async_all();
        }
        int a_ready = -1;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            atomicExch(p.err, 1);
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          if (k < p.num_k) {
            int kk = k + p.rot_k;
            if (kk >= p.num_k) kk -= p.num_k;
            if (p.a_flag_cols) {
              int f = (kk * BK) / p.a_flag_cols;
              if (p.a_flag_rows) f = f * p.a_row_groups + m0 / p.a_flag_rows;
              if (f != a_ready) {
                if (!wait_slab(p, f)) {
                  atomicExch(p.err, 6);
                  ok = false;
                  break;
                }
                fence_proxy_async_all();
                a_ready = f;
              }
            }
            mbar_expect_tx(&full[stage], STAGE_BYTES);
            tma_load_2d(sA, &tmA, &full[stage], kk * BK, m0);
            if (!p.b_mn) {
              tma_load_2d(sB, &tmB, &full[stage], kk * BK, n0);
            } else {
#pragma unroll
              for (int c = 0; c < (BN >= 64 ? BN / 64 : 1); ++c)
                tma_load_2d(sB + c * (BK * 128), &tmB, &full[stage], n0 + c * 64, kk * BK);
            }
          } else {
            // lora_h may still be in production by the previous kernel (dependent launch)
            if (!dep_done) {
              griddep_wait();
              dep_done = true;
            }
            mbar_expect_tx(&full[stage], (BM + BN) * p.lora_r * 2);
            tma_load_2d(sA, &tmA2, &full[stage], 0, m0);
            tma_load_2d(sB, &tmB2, &full[stage], 0, n0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      const uint32_t idesc_lora = umma_idesc_bf16(BM, BN, 0, 0);
      for (int t = worker; t < tiles && ok; t += nworkers, ++it) {
        const int buf = it & 1;
        const uint32_t use = (uint32_t)(it >> 1);
        if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1)) {
          atomicExch(p.err, 2);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&full[stage], phase)) {
            atomicExch(p.err, 3);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sB = sA + A_BYTES;
          if (k < p.num_k) {
            const uint64_t da = umma_desc_kmajor(sA, 128);
            if (!p.b_mn) {
              const uint64_t db = umma_desc_kmajor(sB, 128);
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk)
                umma_bf16(d_tmem, da + kk * 2, db + kk * 2, idesc, (k | kk) != 0);
            } else {
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk)
                umma_bf16(d_tmem, da + kk * 2, umma_desc_mn128(sB + kk * 2048, BK * 128), idesc,
                          (k | kk) != 0);
            }
          } else {
            const uint32_t sw = p.lora_r * 2;
            const uint64_t da = umma_desc_kmajor(sA, sw), db = umma_desc_kmajor(sB, sw);
            for (int kk = 0; kk < p.lora_r / 16; ++kk)
              umma_bf16(d_tmem, da + kk * 2, db + kk * 2, idesc_lora, (k | kk) != 0);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int it = 0;
    for (int t = worker; t < tiles; t += nworkers, ++it) {
      int m_blk, n_blk;
      tile_coords(t, num_m, num_n, p.rot_n, m_blk, n_blk);
      const int m0 = m_blk * BM, n0 = n_blk * BN;
      const int buf = it & 1;
      const uint32_t use = (uint32_t)(it >> 1);
      if (!mbar_wait(&acc_full[buf], use & 1)) {
        if (lane == 0) atomicExch(p.err, 4);
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const bool second = p.n_split >= 0 && n0 >= p.n_split;
      const int act = second || p.n_split < 0 ? p.act : 0;
      const int coff = second ? p.n_split : 0;
      bf16* dst = second && p.out2 ? p.out2 + (size_t)row * p.ldc2 : p.out + (size_t)row * p.ldc;
      int dcol_off = second && p.out2 ? coff : 0;
      if (p.scatter_world) {
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
#pragma unroll 1
      for (int c = 0; c < BN / CH; ++c) {
        const int col0 = n0 + c * CH;
        if (col0 >= p.N) break;
        uint32_t r[CH];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + c * CH;
        if constexpr (CH == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < CH / 8; ++g) {
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
                if (p.pre_out)
                  *reinterpret_cast<bf16x8*>(p.pre_out + (size_t)row * p.ld_pre + (col - coff)) =
                      pack8(v);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = apply_act(v[j], act);
              } else if (act == 3 || act == 4) {
                float pr[8];
                unpack8(*reinterpret_cast<const bf16x8*>(p.pre_in + (size_t)row * p.ld_pre +
                                                         (col - coff)),
                        pr);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= apply_act_grad(pr[j], act);
              }
              if (gate) {
                float gt[8];
                unpack8(*reinterpret_cast<const bf16x8*>(gate + col), gt);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= gt[j];
              }
              if (p.residual) {
                float rs[8];
                unpack8(*reinterpret_cast<const bf16x8*>(p.residual + (size_t)row * p.ldr + col),
                        rs);
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
                if (p.scatter_world ||
                    ERI_DBG_RANGE(to2 ? p.out2 : p.out, to2 ? p.dbg_out2_bytes : p.dbg_out_bytes,
                                  dst + (col - dcol_off), 16, 81))
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
      if (p.rowsq && row_ok) {
        const int part = n0 / p.scatter_part_cols;
        if (part < p.rowsq_parts) atomicAdd(p.rowsq + (size_t)part * p.M + row, sq);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if constexpr (STAGED) tma_store_wait<0>();   // every row copy of this thread has completed
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, int STAGES, bool STAGED = false>
int launch(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& a2, const CUtensorMap& b2,
           const GemmParams& p, int max_ctas, cudaStream_t stream) {
  constexpr int SMEM = STAGES * (BM * BK * 2 + BN * BK * 2) + 1024 + 256 + (STAGED ? BM * (BN * 2 + 16) : 0);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES, STAGED>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int room = max_ctas - p.n_copy;
  const int grid = p.n_copy + (tiles < room ? tiles : room);
  if (p.n_copy > 0) {
    // the compute CTAs spin on counters that the copy CTAs bump: all must be resident
    void* args[] = {(void*)&a, (void*)&b, (void*)&a2, (void*)&b2, (void*)&p};
    return (int)cudaLaunchCooperativeKernel((const void*)gemm_bf16_kernel<BN, STAGES, STAGED>, dim3(grid),
                                            dim3(192), args, SMEM, stream);
  }
  if (p.pdl && p.lora_r) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<BN, STAGES, STAGED>, a, b, a2, b2, p);
  }
  gemm_bf16_kernel<BN, STAGES, STAGED><<<grid, 192, SMEM, stream>>>(a, b, a2, b2, p);
  return (int)cudaGetLastError();
}

int g_num_sms = 0;
int* g_err_flag = nullptr;  // device word; non-zero after a wait inside a kernel ran out

}  // namespace

extern "C" {

// One-time set-up of the device error word (allocates 4 bytes). Returns 0 on success.
int eri_gemm_init() {
  if (g_err_flag) return 0;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  cudaError_t e = cudaMalloc(&g_err_flag, sizeof(int));
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(g_err_flag, 0, sizeof(int));
}

// Reads (and clears) the error word. Synchronises the device: meant for tests and for the
// trainer's per-step health check, not for the hot path.
int eri_gemm_check_error() {
  if (!g_err_flag) return 0;
  int h = 0;
  cudaMemcpy(&h, g_err_flag, sizeof(int), cudaMemcpyDeviceToHost);
  if (h) cudaMemset(g_err_flag, 0, sizeof(int));
  return h;
}

int eri_gemm_job_size() { return (int)sizeof(GatherJob); }

int eri_gemm_bf16(const EriGemmArgs* g, void* stream) {
  if (!g_err_flag) {
    int e = eri_gemm_init();
    if (e) return e;
  }
  if (g->M < 1 || g->N < 16 || g->K < 8) return -10;
  if (g->K % 8 || g->N % 8 || g->lda % 8 || g->ldb % 8 || g->ldc % 8) return -11;
  if (g->lora_r && g->lora_r != 16 && g->lora_r != 32 && g->lora_r != 64) return -12;
  int bn = g->force_bn;
  if (!bn) {
    if (g->N <= 16) bn = 16;
    else if (g->N <= 32) bn = 32;
    else if (g->N <= 64) bn = 64;
    else {
      const long long t256 = (long long)((g->M + BM - 1) / BM) * ((g->N + 255) / 256);
      bn = (g->N >= 256 && t256 >= g_num_sms) ? 256 : 128;
      if (g->N < 128) bn = 64;
    }
  }
  if (bn > g->N) return -13;
  if (g->n_split > 0 && g->n_split % bn) {
    if (g->n_split % 128 == 0) bn = 128; else if (g->n_split % 64 == 0) bn = 64; else return -14;
  }
  if (g->scatter_world) {
    while (bn > 16 && (g->scatter_group_cols % bn)) bn >>= 1;
    if (g->scatter_group_cols % bn) return -17;
  }
  if (g->b_mn && bn < 64) return -18;
  if (g->scatter_mode || g->a_mn || g->glu) return -24;   // two-CTA kernel only
  if (g->M < BM) return -15;  // box taller than the tensor: use the small-M path instead

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = g->M; p.N = g->N; p.K = g->K; p.num_k = (g->K + BK - 1) / BK;
  p.lora_r = g->lora_r; p.act = g->act; p.n_split = g->n_split > 0 ? g->n_split : -1;
  if (g->n_split == 0 && g->out2) p.n_split = 0;
  p.ldc = g->ldc; p.ldc2 = g->ldc2; p.ld_pre = g->ld_pre; p.ldr = g->ldr;
  p.rows_per_batch = g->rows_per_batch > 0 ? g->rows_per_batch : g->M;
  p.gate_stride = g->gate_stride; p.alpha = g->alpha; p.b_mn = g->b_mn;
  p.bias = (const bf16*)g->bias; p.residual = (const bf16*)g->residual;
  p.gate = (const bf16*)g->gate; p.pre_in = (const bf16*)g->pre_in;
  p.out = (bf16*)g->out; p.out2 = (bf16*)g->out2; p.pre_out = (bf16*)g->pre_out;
  p.err = g_err_flag;
  p.dbg_out_bytes = g->dbg_out_bytes; p.dbg_out2_bytes = g->dbg_out2_bytes;
  p.dbg_pre_bytes = g->dbg_pre_bytes; p.dbg_res_bytes = g->dbg_res_bytes;
  p.all_flag = g->n_copy ? g->all_flag : 0;
  p.n_copy = g->n_copy; p.n_jobs = g->n_jobs; p.jobs = (const GatherJob*)g->jobs;
  p.flags = (unsigned int*)g->flags; p.flag_target = (const unsigned int*)g->flag_target;
  p.b_flag_rows = g->b_flag_rows; p.a_flag_cols = g->a_flag_cols;
  p.a_flag_rows = g->a_flag_rows;
  p.a_row_groups = g->a_flag_rows > 0 ? (g->M + g->a_flag_rows - 1) / g->a_flag_rows : 0;
  if (p.a_flag_rows % BM) return -19;
  p.rot_n = g->rot_n_rows / bn;
  p.rot_k = g->rot_k_cols / BK;
  if (p.n_copy < 0 || p.n_copy > g_num_sms / 2) return -19;
  if (p.a_flag_cols % BK) return -19;
  p.scatter_world = g->scatter_world; p.scatter_rank = g->scatter_rank;
  p.scatter_part_cols = g->scatter_part_cols; p.scatter_group_cols = g->scatter_group_cols;
  p.scatter_local_rows = g->scatter_local_rows > 0 ? g->scatter_local_rows : g->M;
  for (int i = 0; i < kMaxPeers; ++i) p.scatter_out[i] = (bf16*)g->scatter_out[i];
  p.rowsq = (float*)g->rowsq; p.rowsq_parts = g->rowsq_parts;
  p.pdl = g->pdl;
  if (p.rowsq && p.scatter_part_cols <= 0) return -17;

  CUtensorMap ta, tb, ta2, tb2;
  {
    uint64_t d[2] = {(uint64_t)g->K, (uint64_t)g->M};
    uint64_t s[1] = {(uint64_t)g->lda * 2};
    uint32_t bx[2] = {BK, BM};
    if (make_tensor_map(&ta, g->a, 2, d, s, bx, 128)) return -20;
  }
  if (!g->b_mn) {
    uint64_t d[2] = {(uint64_t)g->K, (uint64_t)g->N};
    uint64_t s[1] = {(uint64_t)g->ldb * 2};
    uint32_t bx[2] = {BK, (uint32_t)bn};
    if (make_tensor_map(&tb, g->b, 2, d, s, bx, 128)) return -21;
  } else {
    uint64_t d[2] = {(uint64_t)g->N, (uint64_t)g->K};
    uint64_t s[1] = {(uint64_t)g->ldb * 2};
    uint32_t bx[2] = {64, BK};
    if (make_tensor_map(&tb, g->b, 2, d, s, bx, 128)) return -21;
  }
  if (g->lora_r) {
    uint64_t d[2] = {(uint64_t)g->lora_r, (uint64_t)g->M};
    uint64_t s[1] = {(uint64_t)g->ld_h * 2};
    uint32_t bx[2] = {(uint32_t)g->lora_r, BM};
    if (make_tensor_map(&ta2, g->lora_h, 2, d, s, bx, g->lora_r * 2)) return -22;
    uint64_t d2[2] = {(uint64_t)g->lora_r, (uint64_t)g->N};
    uint64_t s2[1] = {(uint64_t)g->ld_lb * 2};
    uint32_t bx2[2] = {(uint32_t)g->lora_r, (uint32_t)bn};
    if (make_tensor_map(&tb2, g->lora_b, 2, d2, s2, bx2, g->lora_r * 2)) return -23;
  } else {
    ta2 = ta;
    tb2 = tb;
  }
  cudaStream_t st = (cudaStream_t)stream;
  if (p.scatter_world && (g->ldc * 2) % 16 == 0) {
    // rows leave through bulk copies (16-byte aligned destinations: ldc and every column offset
    // are multiples of 8 elements); one operand stage less pays for the staging rows
    if (bn == 256) return launch<256, 3, true>(ta, tb, ta2, tb2, p, g_num_sms, st);
    if (bn == 128) return launch<128, 5, true>(ta, tb, ta2, tb2, p, g_num_sms, st);
  }
  switch (bn) {
    case 256: return launch<256, 4>(ta, tb, ta2, tb2, p, g_num_sms, st);
    case 128: return launch<128, 6>(ta, tb, ta2, tb2, p, g_num_sms, st);
    case 64: return launch<64, 8>(ta, tb, ta2, tb2, p, g_num_sms, st);
    case 32: return launch<32, 8>(ta, tb, ta2, tb2, p, g_num_sms, st);
    case 16: return launch<16, 8>(ta, tb, ta2, tb2, p, g_num_sms, st);
  }
  return -16;
}

}  // extern "C"

ERI_DEBUG_BOUNDS_EXPORT(gemm)
