// abk_attention_decode_noalloc: the decode attention of attention_decode.cu with its scratch in a
// fixed array of this library instead of an argument. See attention_decode_static.h for who needs
// this, the limits and the rules of use. The kernels are the ones of attention_decode.cu, compiled
// into this library too; nothing in that file changes.
#include "attention_decode.cu"
#include "attention_decode_static.h"
#include <mutex>

// Partial results first, then the tickets. In host code this name is only a handle for
// cudaGetSymbolAddress, never an address a kernel could use.
static __device__ __align__(256) float abk_noalloc_scratch[ABK_NOALLOC_MAX_FLOATS + ABK_NOALLOC_MAX_TICKETS];

#define ABK_NOALLOC_MAX_DEVICES 64

// The array's address on the current device, looked up once per device.
static int noalloc_scratch_address(float **address) {
    static float *of_device[ABK_NOALLOC_MAX_DEVICES];
    static bool known[ABK_NOALLOC_MAX_DEVICES];
    static std::mutex lock;
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= ABK_NOALLOC_MAX_DEVICES) ABK_REFUSE("attention_decode_noalloc: device %d is not in 0..%d", device, ABK_NOALLOC_MAX_DEVICES - 1);
    std::lock_guard<std::mutex> guard(lock);
    if (!known[device]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, abk_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        of_device[device] = (float *)p;
        known[device] = true;
    }
    *address = of_device[device];
    return 0;
}

extern "C" int abk_attention_decode_noalloc(const void *q, long long q_row, void *out, int n_rows, int n_heads,
                                            int n_kv_heads, int head_dim, float scale, int window, const int *token_seq,
                                            const int *token_pos, const int *seq_slot, const void *k_pool,
                                            const void *v_pool, const int *page_table, int table_width, int ring_pages,
                                            int tokens_per_page, int max_positions, int *status, void *stream) {
    if (n_rows <= 0) return 0;
    if (n_heads < 1 || n_kv_heads < 1 || head_dim < 1 || max_positions < 1)
        ABK_REFUSE("attention_decode_noalloc: sizes must be positive");
    long long chunks = ((long long)max_positions + DEC_CHUNK - 1) / DEC_CHUNK;
    long long floats = (long long)n_rows * n_heads * chunks * (head_dim + 2);
    long long tickets = (long long)n_rows * n_kv_heads;
    if (floats > ABK_NOALLOC_MAX_FLOATS)
        ABK_REFUSE("attention_decode_noalloc: %d rows x %d heads x %lld chunks x (%d + 2) = %lld floats of scratch, the "
                   "built-in array holds %d; use abk_attention_decode with scratch of your own",
                   n_rows, n_heads, chunks, head_dim, floats, ABK_NOALLOC_MAX_FLOATS);
    if (tickets > ABK_NOALLOC_MAX_TICKETS)
        ABK_REFUSE("attention_decode_noalloc: %d rows x %d kv heads = %lld tickets, the built-in array holds %d",
                   n_rows, n_kv_heads, tickets, ABK_NOALLOC_MAX_TICKETS);
    float *scratch = nullptr;
    int rc = noalloc_scratch_address(&scratch);
    if (rc) return rc;
    int *ticket_words = (int *)(scratch + ABK_NOALLOC_MAX_FLOATS);
    // whatever an earlier call left (or an interrupted one did not reset): the tickets start at zero
    cudaError_t e = cudaMemsetAsync(ticket_words, 0, (size_t)tickets * sizeof(int), (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    return abk_attention_decode(q, q_row, out, n_rows, n_heads, n_kv_heads, head_dim, scale, window, token_seq,
                                token_pos, seq_slot, k_pool, v_pool, page_table, table_width, ring_pages,
                                tokens_per_page, max_positions, scratch, ticket_words, status, stream);
}
