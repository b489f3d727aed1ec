/* Split-context decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference project: it is an addition of this
 * library.
 *
 * Who it is for.  The ordinary launcher, ng_attn_decode_bf16, asks its caller for a scratch
 * buffer in which the splits of a context leave their partial results before they are merged.
 * Some callers have no way of providing one: a host program that links this library through
 * its C ABI and has no device allocator of its own; a server that handed all device memory to
 * its weight and cache pools when it started and keeps nothing back; a latency-critical loop in
 * which cudaMalloc, which may synchronise the whole device, must never run.  For them the
 * variant below keeps the scratch inside the library, in a file-scope
 * `static __device__ __align__(256)` array.
 *
 * What that costs.  The array holds NG_NOALLOC_SCRATCH_FLOATS floats (4 MiB).  Every GPU on
 * which this library is loaded holds that much from load until the process exits, whether or
 * not the entry point is ever called; and the library is built once per head size, so a
 * process that uses two head sizes holds it twice.
 *
 * Limits.  A call needs n_rows * n_heads * n_splits * (head_dim + 2) floats when n_splits > 1.
 * n_rows is the number of rows of q and out, NOT the number of entries: a step that holds a
 * prompt portion beside decode tokens has more rows than entries, and the rows of the entries
 * this kernel skips count too.  The kernels find an entry's row in cu_q on the device; an
 * entry whose row is n_rows or more is skipped (its row of out is not written), so a caller
 * who passes too small an n_rows gets missing rows, never a write outside the array.  A call
 * that needs more than the array holds is refused with NG_NOALLOC_TOO_LARGE and launches
 * nothing; use fewer splits, or the ordinary launcher with scratch of your own.
 * ng_attn_decode_noalloc_max_floats returns the capacity.
 *
 * First call.  The device address of the array is looked up with cudaGetSymbolAddress the
 * first time the entry point runs on a device (once per device, with that device current), and
 * the return code of the lookup is checked.  Make that first call during start-up, outside any
 * stream capture.
 *
 * Sharing.  Every call on a device uses the same array, and the array keeps what the last
 * call left in it.  Nothing in it has to start at zero: each call writes every record before
 * the merge reads it.  Two calls that overlap on the GPU (different streams, or different host
 * threads without ordering between their streams) race on the array and give wrong results;
 * calls on one stream are safe.
 *
 * It calls no cudaMalloc, cudaFree or any other allocating routine.  Arguments are those of
 * ng_attn_decode_bf16 without `scratch`; return codes likewise, plus the two below.
 */
#pragma once
#include <cuda_runtime.h>

#define NG_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define NG_NOALLOC_TOO_LARGE 4      /* the call needs more scratch than the library holds */
#define NG_NOALLOC_SETUP_FAILED 5   /* cudaGetDevice / cudaGetSymbolAddress failed on this device */

#ifdef __cplusplus
extern "C" {
#endif

int ng_attn_decode_bf16_noalloc(const void* q, const void* k_pages, const void* v_pages, const int* table,
                                int table_stride, const int* cu_q, const int* ctx_before, void* out,
                                int n_rows, int n_entries, int nH, int nKV, int hd, int page_size, int num_pages,
                                int window, float scale, int n_splits, int max_ctx, cudaStream_t stream);

int ng_attn_decode_noalloc_max_floats(void);

#ifdef __cplusplus
}
#endif
