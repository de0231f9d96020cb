// Argument block of the GEMM entry points (eri_gemm_bf16, eri_gemm2_bf16); mirrored field by field
// by ``GemmArgs`` in ops/_native.py.
#pragma once

constexpr int kMaxPeers = 16;

extern "C" {

struct EriGemmArgs {
  const void* a;        // [M, K] bf16, row stride lda
  const void* b;        // [N, K] bf16 (or [K, N] when b_mn), row stride ldb
  const void* lora_h;   // [M, r] bf16 (row stride ld_h) or null
  const void* lora_b;   // [N, r] bf16 (row stride ld_lb) or null
  const void* bias;
  const void* residual;
  const void* gate;
  const void* pre_in;
  void* out;
  void* out2;
  void* pre_out;
  long long lda, ldb, ld_h, ld_lb;
  int M, N, K, lora_r;
  int act, n_split;
  int ldc, ldc2, ld_pre, ldr;
  int rows_per_batch, gate_stride;
  int force_bn;
  float alpha;
  int b_mn;
  // gather mode (all zero / null when unused)
  int n_copy, n_jobs;
  const void* jobs;
  void* flags;
  const void* flag_target;
  int b_flag_rows, a_flag_cols, rot_n_rows, rot_k_cols;
  int a_flag_rows;   // 0, or a multiple of 128: row-group split of the K-range counters
  // peer scatter
  int scatter_world, scatter_rank, scatter_part_cols, scatter_group_cols, scatter_local_rows;
  void* scatter_out[kMaxPeers];
  void* rowsq;
  int rowsq_parts;
  // 1: launch as a programmatic dependent of the previous kernel on the stream. The caller promises
  // that this previous kernel is the one that writes lora_h and nothing else this GEMM reads; the
  // GEMM then starts its main K loop while that kernel still runs and waits for it
  // (griddepcontrol.wait) only before it loads lora_h for the rank-r step.
  int pdl;
  // Gather mode, optional: this rank's own slab of the gathered B operand is read in place through
  // a second tensor map instead of being copied into the landing buffer (two-CTA kernel only; the
  // *_nl job list and targets leave the local slab's jobs out).
  const void* b_local;        // this rank's shard: rows [loc_lo, loc_hi) of B (loc_mode 1), or of the
  long long ldb_local;        // K dimension of an MN-major B (loc_mode 2); row stride in elements
  int loc_mode, loc_lo, loc_hi;
  int n_jobs_nl;
  const void* jobs_nl;
  const void* flag_target_nl;
  // 1: A is given as [K, M] row-major (MN-major operand; row stride lda). Together with b_mn this is
  // the weight-gradient product dW = dY^T X over token-major activations (two-CTA kernel only).
  int a_mn;
  // Gated linear unit on an up-projection b = [2 * hidden, K]: out[M, hidden] = a * act(g) with a, g
  // the two halves of the projection; pre_out (optional, [M, 2 * hidden]) keeps the halves.
  // 1: a * gelu(g), 2: a * silu(g), 3: gelu(a) * g, 4: silu(a) * g (two-CTA kernel only).
  int glu;
  // Byte extents of the destination / auxiliary buffers counted from their pointers (0: unknown).
  // Only the bounds-checked debug build reads them.
  long long dbg_out_bytes, dbg_out2_bytes, dbg_pre_bytes, dbg_res_bytes;
  // Peer scatter by ROW slabs (two-CTA kernel): 0 = column groups (Ulysses head scatter, above);
  // 1 = output row r goes to rank r / scatter_local_rows, into slot scatter_rank of that rank's
  // receive buffer [world][scatter_local_rows, N] (the weight-gradient reduce-scatter of ZeRO-3
  // folded into the dW GEMM: every rank's partial slab lands at its owner as the tiles finish).
  int scatter_mode;
  // Gather mode, optional: device array of 8 unsigned 64-bit words that the launch fills with
  // %globaltimer readings (ns): [0] earliest CTA start (caller presets it to all ones), [1] latest
  // end of a copy CTA (every slab has landed), [2] latest end of a compute CTA, [3] sum and [4]
  // maximum over the compute CTAs' TMA producers of the time spent waiting for slab counters,
  // [5] number of producers that waited at all. Null: nothing is recorded.
  unsigned long long* stamps;
  // Gather mode on the two-CTA kernel: > 0 = the copy clusters join the tile loop once their slabs
  // have landed, taking tiles from this round of the persistent schedule on (the caller estimates how
  // many rounds the compute clusters finish while the copies run); 0 = they leave after copying.
  int join_round;
  // Gather mode: 1 + index of a counter in `flags` that every finished copy job bumps (its target in
  // `flag_target` is the number of jobs); 0 = none. A producer that finds it at its target stops
  // checking slab counters: after the gather has finished, a tile costs one counter load.
  int all_flag;
};

}  // extern "C"
