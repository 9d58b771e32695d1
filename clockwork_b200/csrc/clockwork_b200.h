/* C declarations of entry points of libclockwork_b200.so that are meant to be called from outside
 * the Python package.  (The Python package declares the rest itself, in clockwork_b200/ops.) */
#ifndef CLOCKWORK_B200_H
#define CLOCKWORK_B200_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Negative return codes of the entry points; positive values are cudaError_t. */
#define CW_OK 0
#define CW_ERR_BAD_SIZE (-1)
#define CW_ERR_BAD_DTYPE (-2)
#define CW_ERR_UNSUPPORTED (-3)
#define CW_ERR_SETUP (-4)
#define CW_ERR_SCRATCH_LIMIT (-5) /* the call needs more scratch than CW_NOALLOC_SCRATCH_BYTES */

/* Text for a return code of this library (static storage). */
const char* cw_error_string(int code);

/* Bytes of device memory that every GPU which loads this library sets aside, until the process
 * exits, for cw_attention_decode_noalloc. */
#define CW_NOALLOC_SCRATCH_BYTES (8u << 20)

/* Paged decode attention for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference (jasonjesuraja06/clockwork): it exists for
 * hosts that drive the kernels directly and cannot hand over scratch buffers of their own, for
 * instance a serving loop written in C that owns a fixed device-memory budget and treats any
 * cudaMalloc after start-up as a fault, or code that runs at a point where an allocation would
 * stall the whole device (cudaMalloc and cudaFree synchronise it).  The regular entry point,
 * cw_attention_decode, splits long contexts over thread blocks and needs float32 scratch for the
 * partial results plus a few counters, which its caller allocates.  Here the same kernel runs with
 * that scratch taken from a fixed array inside the library (CW_NOALLOC_SCRATCH_BYTES per GPU), so
 * the call itself allocates nothing: no cudaMalloc, no cudaFree, no library routine that allocates.
 *
 * Arguments are those of cw_attention_decode without the scratch pointers: q [S, q_stride]
 * bfloat16 (one query token per request, the first nh*hd columns are the query heads), out
 * [S, nh*hd] bfloat16, k_cache / v_cache [num_pages, page_size, nkv, hd] bfloat16, block_tables
 * int32 [S, max_blocks], ctx_lens int32 [S] (tokens of each request in the cache, its own
 * included), max_ctx an upper bound of every ctx_lens[s], split the tokens per thread block (a
 * multiple of 64, at least 128), status 4 int32 words on the device (may be null).  Inputs and
 * outputs are still the caller's.
 *
 * Limits and rules:
 *  - The scratch is sized for the finest cut the kernel allows (128 tokens per thread block),
 *    whatever `split` is: 4 * S * nh * ceil(max_ctx / 128) * (hd + 1) bytes plus 4 bytes per
 *    (request, KV head, group of 16 query heads), each of the three parts rounded up to 256 bytes.
 *    A call that needs more than CW_NOALLOC_SCRATCH_BYTES returns CW_ERR_SCRATCH_LIMIT and
 *    launches nothing.  cw_attention_decode_noalloc_fits answers the same question without a call:
 *    for 12 query heads of 128 over 2 KV heads the 8 MiB hold, for instance, 8 requests bounded by
 *    21,632 tokens or 64 requests bounded by 2,688.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress) with
 *    that device current.  Make that first call before any stream capture begins.
 *  - All calls share the one array and it keeps what the last call left; the counters in it are
 *    cleared (on the given stream) at the start of every call.  Two calls whose kernels may overlap
 *    on the GPU (different streams, or the same call from two threads) race on it: serialise them.
 */
int cw_attention_decode_noalloc(const void* q, int q_stride, void* out, const void* k_cache, const void* v_cache,
                                const int* block_tables, const int* ctx_lens, int S, int nh, int nkv, int hd,
                                int page_size, int max_blocks, int num_pages, float scale, int window, int max_ctx,
                                int split, int* status, cudaStream_t stream);

/* 1 when a call of cw_attention_decode_noalloc with these sizes fits the built-in scratch, 0 when it
 * would return CW_ERR_SCRATCH_LIMIT; CW_ERR_BAD_SIZE for sizes the kernel refuses anyway.  Touches
 * no device. */
int cw_attention_decode_noalloc_fits(int S, int nh, int nkv, int hd, int max_ctx);

#ifdef __cplusplus
}
#endif
#endif
