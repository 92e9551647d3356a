/* Split-KV paged decode attention that allocates nothing.
 *
 * This entry point has no counterpart in the reference (luke396/somi-inference); it exists for
 * callers of this library that cannot allocate device memory when they need attention: a
 * process that handed the whole GPU to its own memory pool at start-up, a latency-critical
 * loop in which cudaMalloc's implicit device synchronisation is not acceptable, or a caller
 * that holds raw device pointers only.  It is the same computation as
 * somi_paged_attention_decode (attention_decode.cu), with the per-chunk partial results kept in
 * a file-scope device array of the library instead of caller-provided scratch.  The caller
 * still passes every input and the output.
 *
 * Limits and rules
 *  - The array holds 2 Mi float32 (8 MiB) and is resident on every GPU that loads the library,
 *    until the process exits.  A call needs n_decode * nq * max_splits * (hd + 2) floats
 *    (max_splits = ceil(longest cached length / 128) of the batch, as for the ordinary entry
 *    point); a larger call is refused with SOMI_ERR_SCRATCH_TOO_SMALL (10002) and nothing is
 *    launched.  somi_paged_attention_decode_static_capacity() returns the capacity in floats,
 *    somi_paged_attention_decode_static_strerror(code) a sentence for a return code.
 *  - The first call on a device looks the array's device address up
 *    (cudaGetSymbolAddress, with that device current) and remembers it; later calls on that
 *    device only launch kernels.  Make that first call outside any stream capture.
 *  - The array that is used is the one of the CURRENT device: make the device that owns
 *    `stream` and the pointer arguments current before the call.
 *  - The function calls no cudaMalloc, cudaFree or other allocating routine.
 *  - All calls on a device share the one array, which keeps the previous call's contents.
 *    Nothing in it has to start at zero (every slot read is written earlier in the same call),
 *    but two calls whose kernels overlap on the GPU (different streams, or threads launching
 *    at the same time) overwrite each other's partial results: serialise them.
 *  - Geometry as for somi_paged_attention_decode: bfloat16, head_dim 32/64/128, at most 16
 *    query heads per key/value head.  Returns 0, a SOMI_ERR_* code, or a cudaError_t value.
 */
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int somi_paged_attention_decode_static(
    const void* qkv,        /* bf16 [tokens, (nq + 2 nkv) * hd]: queries of the step, row-major */
    int row_stride,         /* elements between rows of qkv */
    int row_base,           /* row of the first single-token request */
    int req_base,           /* index of that request in block_table / ctx_len */
    int n_decode,           /* number of single-token requests */
    const void* kcache,     /* bf16 [pages, nkv, page_size, hd] */
    const void* vcache,     /* bf16 [pages, nkv, page_size, hd] */
    const int* block_table, /* int32 [requests, bt_stride] page ids */
    int bt_stride,
    const int* ctx_len,     /* int32 [requests]: tokens cached before this step */
    int nq, int nkv, int hd, int page_size, float scale,
    int window,             /* 0: all keys; n: the last n positions */
    int max_splits,         /* ceil(bt_stride * page_size / 128) or any bound on the chunks */
    void* out,              /* bf16 [tokens, nq * hd] */
    cudaStream_t stream);

long long somi_paged_attention_decode_static_capacity(void);
const char* somi_paged_attention_decode_static_strerror(int code);

#ifdef __cplusplus
}
#endif
