/* Decode attention for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference (pmrjge/quanta has no device code of its own);
 * it exists for users of this library's C ABI.
 *
 * Who needs it.  The decode attention (qb_attn_decode) cuts the keys of long contexts over several
 * blocks, which leave partial results that a second kernel merges, so it wants scratch memory from
 * its caller (n_parts = qb_attn_decode_parts(kv heads, longest context) entries per token and head).  Some callers have none to
 * give and cannot get any: a host program that handed the whole device to a pool of its own (a
 * serving process that sized its cache to the last byte and treats any later cudaMalloc as a
 * failure); a plug-in loaded into such a process through this C ABI, with no handle on that pool; a
 * latency-bound loop in which an allocation may synchronise the device or simply fail when memory is
 * fragmented.  For them the scratch lives inside the library: a file-scope
 * `static __device__ __align__(256)` array of QB_NOALLOC_SCRATCH_FLOATS floats (8 MiB), which every
 * GPU that loads the library holds until the process exits.
 *
 * Contract.
 *  - Same inputs and outputs as qb_attn_decode, without the two scratch pointers.  The call allocates
 *    nothing and calls no allocating routine (no cudaMalloc, cudaFree, no torch).
 *  - Sizes: n_dec * nq * n_parts * (hd + 2) floats must fit in the array; a larger problem is
 *    refused with QB_NOALLOC_TOO_LARGE and nothing is launched.  qb_attn_decode_noalloc_floats()
 *    returns what a call needs; qb_attn_decode_noalloc_capacity() the size of the array.
 *  - The first call on a device looks the array's device address up (cudaGetSymbolAddress, with that
 *    device current) and remembers it per device; make that first call before any stream capture
 *    begins on the device.
 *  - All calls share the one array, and it keeps the last call's contents.  Nothing in it has to
 *    start at zero: every element the merge step reads was written by the same call.  The one
 *    exception is a call that the kernel refuses in part (a page id outside the pool, recorded in the
 *    status words): then nothing is merged at all, `out` is not valid, and the status words say so.
 *    Two calls that overlap on the GPU (different streams, or the same stream from racing host
 *    threads) race on the array; run them one after the other.
 */
#pragma once
#include <cuda_runtime.h>

#define QB_NOALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u)
#define QB_NOALLOC_TOO_LARGE (-3)

#ifdef __cplusplus
extern "C" {
#endif

long long qb_attn_decode_noalloc_floats(int n_dec, int nq, int hd, int n_parts);
long long qb_attn_decode_noalloc_capacity(void);

int qb_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out, const int* dec_tok,
                           int n_dec, const int* tok_pos, const int* tok_req, const int* block_table, int bt_stride,
                           int nq, int nkv, int hd, int page_size, int num_pages, float scale, int window,
                           int n_parts, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
