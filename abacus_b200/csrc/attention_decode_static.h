/* Decode attention without a scratch argument: abk_attention_decode_noalloc.
 *
 * This entry point has no counterpart in mottopanikeiku/abacus (whose engine has no GPU code
 * and no allocator question at all). It exists for callers that cannot get scratch memory for
 * abk_attention_decode: a host program that handed all device memory to a pool of its own at
 * start-up and has nothing left to cudaMalloc from; a latency-critical loop that must not pay
 * cudaMalloc's device-wide synchronisation; a plugin or callback that runs inside someone
 * else's process and owns no allocator there. Such a caller still passes every input and the
 * output; only the scratch is taken care of.
 *
 * The scratch lives in one array that is part of the library's device image:
 * ABK_NOALLOC_SCRATCH_BYTES (4 MiB + 16 KiB) on every GPU that loads the library, held until
 * the process exits. The call does no cudaMalloc, no cudaFree and calls nothing that allocates.
 *
 * Limits (the call refuses anything larger, with a message from abk_last_error):
 *     n_rows * n_heads * ceil(max_positions / 128) * (head_dim + 2) <= ABK_NOALLOC_MAX_FLOATS
 *     n_rows * n_kv_heads                                           <= ABK_NOALLOC_MAX_TICKETS
 * For example 8 rows, 16 heads of 128, positions below 4096: 8 * 16 * 32 * 130 = 532,480 floats.
 *
 * First call on a device: it looks up the array's device address (cudaGetSymbolAddress, with
 * that device current) and sets the kernels' shared-memory attribute. Make this first call
 * outside any stream capture. Later calls on that device only enqueue work on `stream`.
 *
 * All calls on a device share the one array. Each call first clears the part that must start
 * at zero (the tickets), on `stream`, and does not rely on anything an earlier call left. Two
 * calls that run on the GPU at the same time (different streams, or several host threads)
 * race on the array: keep calls on one device in one stream, or order them yourself.
 *
 * Arguments and result are those of abk_attention_decode (attention_decode.cu) without
 * `scratch` and `tickets`: 0 on success, a CUDA error code (> 0), or -1 (refused).
 */
#pragma once

#define ABK_NOALLOC_MAX_FLOATS (1 << 20)
#define ABK_NOALLOC_MAX_TICKETS 4096
#define ABK_NOALLOC_SCRATCH_BYTES (4 * (ABK_NOALLOC_MAX_FLOATS + ABK_NOALLOC_MAX_TICKETS))

#ifdef __cplusplus
extern "C" {
#endif

int abk_attention_decode_noalloc(const void *q, long long q_row, void *out, int n_rows, int n_heads, int n_kv_heads,
                                 int head_dim, float scale, int window, const int *token_seq, const int *token_pos,
                                 const int *seq_slot, const void *k_pool, const void *v_pool, const int *page_table,
                                 int table_width, int ring_pages, int tokens_per_page, int max_positions, int *status,
                                 void *stream);

#ifdef __cplusplus
}
#endif
