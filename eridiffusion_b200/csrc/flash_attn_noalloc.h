/* Allocation-free flash-attention backward.
 *
 * This entry point has no counterpart in the reference project: it exists for callers of this
 * library that cannot obtain device memory at call time. Examples: an embedding application that
 * gave the library a fixed memory budget up front and forbids later cudaMalloc calls; a plug-in
 * hosted inside another framework whose caching allocator owns all device memory, so a private
 * allocation could push the host framework into an out-of-memory failure; a latency-critical
 * loop that cannot tolerate the device synchronisation or the failure modes of an allocation.
 *
 * The regular entry point (eri_flash_attn_bwd) asks the caller for two scratch vectors. This
 * variant keeps them in a fixed array inside the library image instead, so the caller passes
 * only inputs and outputs.
 *
 * Limits:
 *   - B * H * (Lq rounded up to a multiple of 128) <= 262144 rows
 *     (eri_flash_attn_bwd_noalloc_max_rows()); bigger problems return -6.
 *   - The scratch array (2 MiB) is resident on every GPU that loads the library until exit.
 *   - The first call on each device resolves the array's device address
 *     (cudaGetSymbolAddress, with that device current): issue it before any stream capture.
 *   - All calls on a device share the array: calls whose GPU work overlaps race with each
 *     other; run them one after another. Nothing needs clearing between calls.
 *   - Neither cudaMalloc nor cudaFree nor any allocating library routine is called.
 *
 * Tensors: contiguous bf16 on the current device, dout/q/out/dq [B, Lq, H, DH],
 * k/v/dk/dv [B, Lk, H, DH], DH in {64, 128}, Lq, Lk >= 128; lse [B, H, Lq] fp32 from
 * eri_flash_attn_fwd. Returns 0 on success, a negative code otherwise.
 */
#ifndef ERI_FLASH_ATTN_NOALLOC_H
#define ERI_FLASH_ATTN_NOALLOC_H

#ifdef __cplusplus
extern "C" {
#endif

int eri_flash_attn_bwd_noalloc(const void* dout, const void* q, const void* k, const void* v,
                               const void* out, const float* lse, void* dq, void* dk, void* dv,
                               int B, int H, int Lq, int Lk, int DH, float scale, void* stream);

/* Human-readable text for a return code of the function above. */
const char* eri_flash_attn_bwd_noalloc_strerror(int code);

/* Largest accepted B * H * ceil(Lq/128)*128. */
int eri_flash_attn_bwd_noalloc_max_rows(void);

/* Reads and clears the kernels' status word (0 = no bounded wait ran out). Synchronous. */
int eri_flash_attn_bwd_noalloc_status(void);

#ifdef __cplusplus
}
#endif
#endif
