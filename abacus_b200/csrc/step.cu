// The step function in C: one call walks a model's schedule and launches the whole step.
//
// abacus's forward() is C (src/model.c:286-327): embedding, then for each layer add_norm, the q/k/v product,
// rotate_and_cache, attention, the output product, add_norm, gate/up, SwiGLU, down, then the last norm and the
// output matrix on the wanted rows. This is that function for a batch of sequences on the GPU: the same order, each
// line a kernel launch (rotate_and_cache is a launch of its own only where neither neighbour takes it in: the q/k/v
// product of a long prompt step does it in its epilogue, decode attention in its own kernel). The kernels live in
// libraries of their own; their launchers' addresses are handed in once
// (AbkFns), as are the model's matrices, sizes and constants (AbkModel), so that a step costs the host one call
// instead of one per kernel (a few hundred, at some ten microseconds each from Python).
//
// It serves models put together from the library's own parts in abacus's arrangement: the plain frame, pre-norm
// blocks, RMSNorm, the attention mixer, the gated feed-forward. Which kernel runs a product or an attention is
// decided here by the rules of parts/linear.py, parts/mlp.py and kernels/ops.py (attention), restated; a test holds
// both ways to the same bits. A model with a part of another kind takes the way through the parts' own forward().
//
// No device code and no CUDA call of its own: every line that touches the GPU is a launcher of another library.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

enum { ABK_F32 = 0, ABK_BF16 = 1 };

// ------------------------------------------------------------------ the launchers (see the kernels' own files)
typedef int (*EmbedFn)(const int *, const void *, int, float *, int, int, int, int *, void *);
typedef int (*AddRmsnormFn)(float *, const float *, const float *, void *, int, const int *, int, int, float, void *);
typedef int (*SwigluFn)(const void *, void *, int, int, int, int, void *);
typedef int (*QkvPrepFn)(void *, int, int, int, int, int, int, const int *, const int *, const int *, const int *,
                         const float *, const float *, float, const float *, const float *, int, int, void *, void *,
                         const int *, int, int, int, void *);
typedef int (*GemmSimtFn)(const void *, int, const void *, int, void *, int, int, int, int, long long, long long, long long,
                          void *);
typedef int (*GemmRowsFn)(const void *, const void *, void *, int, int, int, int, long long, long long, long long, void *);
typedef int (*GemmRowsSwigluFn)(const void *, const void *, void *, int, int, int, long long, long long, long long, int,
                                void *);
typedef int (*GemmTcFn)(const void *, const void *, void *, int, int, int, int, long long, long long, long long, float *,
                        int *, int *, int, int, int, int, void *);
typedef int (*GemmTcSwigluFn)(const void *, const void *, void *, int, int, int, long long, long long, long long, int *,
                              void *);
typedef int (*GemmTcQkvFn)(const void *, const void *, void *, int, int, int, int, long long, long long, long long, const int *,
                           const int *, const int *, const float *, const float *, float, const float *, const float *, void *,
                           void *, const int *, int, int, int *, void *);
typedef int (*AttnGenericFn)(const void *, long long, void *, int, int, int, int, int, float, int, const int *, const int *,
                             const int *, const int *, const int *, const void *, const void *, const int *, int, int, int,
                             const void *, const void *, long long, void *);
typedef int (*AttnPrefillFn)(const void *, long long, int, void *, int, int, int, float, const int *, int, const int *,
                             const int *, const int *, const int *, const void *, const void *, long long, const int *, int,
                             int, int *, void *);
typedef int (*AttnPrefillTcFn)(const void *, long long, int, void *, int, int, int, float, const int *, int, int, float *,
                               int *, const void *, const void *, long long, const int *, int, int, int *, void *);
typedef int (*AttnDecodeRingFn)(const void *, long long, void *, int, int, int, int, float, int, const int *, const int *,
                                const int *, const void *, const void *, long long, const int *, int, int, int, int, int *,
                                void *);
typedef int (*AttnDecodeRingPrepareFn)(const void *, long long, void *, int, int, int, int, float, int, const int *, const int *,
                                       const int *, void *, void *, long long, const int *, int, int, int, int, const float *,
                                       const float *, float, const float *, const float *, int, int *, void *);
typedef int (*AttnDecodeFn)(const void *, long long, void *, int, int, int, int, float, int, const int *, const int *,
                            const int *, const void *, const void *, const int *, int, int, int, int, float *, int *, int *,
                            void *);

struct AbkFns {
    EmbedFn embed;
    AddRmsnormFn add_rmsnorm;
    SwigluFn swiglu;
    QkvPrepFn qkv_prep;
    GemmSimtFn gemm_simt;
    GemmRowsFn gemm_rows;
    GemmRowsSwigluFn gemm_rows_swiglu;
    GemmTcFn gemm_tc;
    GemmTcSwigluFn gemm_tc_swiglu;
    AttnGenericFn attention_generic;
    AttnPrefillFn attention_prefill;
    AttnPrefillTcFn attention_prefill_tc;
    AttnDecodeRingFn attention_decode_ring;
    AttnDecodeFn attention_decode;
    AttnDecodeRingPrepareFn attention_decode_ring_prepare;
    GemmTcQkvFn gemm_tc_qkv;
};

// ------------------------------------------------------------------ the model, bound once
struct AbkLinear {
    const void *w;  // [n, k], row pitch ldw (elements)
    long long ldw;
    int n, k, dtype, pad;
};
struct AbkNorm {
    const float *w;
    float eps;
    int size;
};
struct AbkAttention {
    AbkLinear qkv, q_only, o;
    const float *q_norm, *k_norm;  // null: no per-head norm
    const float *cos, *sin;        // null: no rotation
    float eps, scale;
    int n_heads, n_kv_heads, head_dim, window;  // window 0: all keys
    int rotary_dim, interleaved, table_positions, lists;  // lists: which of the step's attention lists it walks
};
struct AbkMlp {
    AbkLinear gate_up, down;
    int inter, block;
};
struct AbkBlock {
    AbkNorm norm1, norm2;
    AbkAttention att;
    AbkMlp mlp;
};
struct AbkEntry {  // one entry of the schedule and the cache it reads
    void *k, *v;   // [pages, kv heads, tokens per page, head_dim]; null: no keys and values
    const int *table;
    long long pool_rows;
    int block, owns, table_width, ring_pages, tokens_per_page, pad;
};
struct AbkModel {
    const AbkFns *fns;
    const AbkBlock *blocks;
    const AbkEntry *entries;
    const void *embed;
    AbkNorm final_norm;
    AbkLinear head;
    int *status;          // the model's status words (a token outside the vocabulary)
    float *gemm_scratch;  // split K of the tensor-memory product
    int *gemm_tickets, *kernel_status;
    float *halves;        // partial results of halved attention tiles
    int *halves_tickets, *attention_tickets;
    int dtype, hidden, vocab, n_blocks, n_entries, halves_pairs, attention_ticket_count;
    int decode_prepares;   // decode attention prepares q, k and v itself where it can (parts/attention.py: DECODE_PREPARES)
    int product_prepares;  // a prompt's q/k/v product prepares them in its epilogue where it can (PRODUCT_PREPARES)
};

// ------------------------------------------------------------------ one step
struct AbkLists {  // the attention mixer's tiles and work list for this step (parts/attention_plan.py)
    const int *tiles64, *work;
    int n_tiles64, n_work, n_halved, pad;
};
struct AbkStep {
    const int *tokens, *token_seq, *token_pos, *seq_slot, *seq_start, *seq_pos0, *seq_len_after, *logit_rows;
    const AbkLists *lists;
    float *x, *branch, *logits, *attention_partials;  // workspace: the stream, a branch's output, logits, decode partials
    void *xn, *qkv, *att, *act, *gate_up, *xn_final;
    long long partial_floats;
    int n_rows, n_logit_rows, is_decode, any_continuation, max_len_after, position_bound, n_lists, pad;
};

enum {
    STEP_OK = 0,
    STEP_REFUSED_WINDOW = -101,   // several tokens of a windowed sequence that is not at its start
    STEP_REFUSED_HALVES = -102,   // more halved tiles than the attention kernel has scratch for
    STEP_REFUSED_TICKETS = -103,  // more (row, kv head) pairs than decode attention has tickets for
    STEP_REFUSED_PARTIALS = -104, // the workspace given for decode partials is too small
    STEP_NO_LAUNCHER = -105,      // a kernel library this model was not expected to need
};
static thread_local char step_error[256];
static thread_local int step_launches;
extern "C" const char *abk_last_error() { return step_error; }
// Kernels the last abk_step of this thread launched.
extern "C" int abk_step_launches() { return step_launches; }
// Where the last failing call was: "<launcher> in schedule entry <i>" (-1: outside the layers).
static int fail(int rc, const char *what, int entry) {
    snprintf(step_error, sizeof step_error, "%s in schedule entry %d", what, entry);
    return rc;
}
#define TRY(call, what)                              \
    do {                                             \
        int rc_ = (call);                            \
        if (rc_) return fail(rc_, what, entry);      \
    } while (0)
// A launcher's call: refused with a clear code if its library was not handed in, counted if it ran.
#define LAUNCH(fn, ...) ((fn) ? (step_launches++, (fn)(__VA_ARGS__)) : STEP_NO_LAUNCHER)

static bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

// parts/linear.py: rows_kernel_wins
static bool rows_kernel_wins(int rows, const AbkLinear &l, bool gated) {
    const long long bytes = (long long)l.n * l.k * 2;
    if (rows > 16) return false;
    return bytes <= (16ll << 20) || (rows <= 8 && bytes <= (gated ? (128ll << 20) : (32ll << 20)));
}
// kernels/ops.py: gemm_rows_takes / gemm_tc_takes (x dense with row pitch ldx)
static bool rows_takes(const void *x, long long ldx, const AbkLinear &l, int rows) {
    return rows <= 64 && l.dtype == ABK_BF16 && l.k % 32 == 0 && ldx % 8 == 0 && l.ldw % 8 == 0 && aligned16(x) && aligned16(l.w);
}
static bool tc_takes(const void *x, long long ldx, const AbkLinear &l) {
    return l.dtype == ABK_BF16 && l.k % 8 == 0 && ldx % 8 == 0 && l.ldw % 8 == 0 && aligned16(x) && aligned16(l.w);
}

// parts/linear.py: Linear.forward. out[:rows] = x[:rows] . w^T; x in the model's dtype.
static int linear(const AbkModel &m, const AbkLinear &l, const void *x, long long ldx, void *out, int out_dtype, long long ldo,
                  int rows, void *stream) {
    const AbkFns &f = *m.fns;
    if (l.dtype == ABK_BF16 && rows_kernel_wins(rows, l, false) && rows_takes(x, ldx, l, rows))
        return LAUNCH(f.gemm_rows, x, l.w, out, out_dtype, rows, l.n, l.k, ldx, l.ldw, ldo, stream);
    if (tc_takes(x, ldx, l))
        return LAUNCH(f.gemm_tc, x, l.w, out, out_dtype, rows, l.n, l.k, ldx, l.ldw, ldo, m.gemm_scratch, m.gemm_tickets,
                         m.kernel_status, 0, -1, 0, -1, stream);
    return LAUNCH(f.gemm_simt, x, m.dtype, l.w, l.dtype, out, out_dtype, rows, l.n, l.k, ldx, l.ldw, ldo, stream);
}

static size_t esize(int dtype) { return dtype == ABK_BF16 ? 2 : 4; }

// parts/attention.py: Attention.forward, with kernels/ops.py: attention
static int attention(const AbkModel &m, const AbkAttention &a, const AbkEntry &e, const AbkStep &s, int entry, void *stream) {
    const AbkFns &f = *m.fns;
    const int n = s.n_rows, q_size = a.n_heads * a.head_dim, kv_size = a.n_kv_heads * a.head_dim;
    const long long row = q_size + 2 * kv_size;
    const bool writes = e.owns != 0, has_cache = e.k != nullptr;
    const int group = a.n_heads / a.n_kv_heads, hd = a.head_dim;
    const bool bf16 = m.dtype == ABK_BF16;
    // a windowed cache keeps only the last keys; a prompt reads its keys from this step's own rows
    const bool from_step = a.window > 0 && !s.is_decode;
    // kernels/ops.py: gemm_tc_qkv_takes
    const bool prepared = m.product_prepares && writes && !s.is_decode && !from_step && bf16 && n > 256 && hd == 128 &&
                          e.ring_pages == 0 && a.qkv.n == row && (!a.cos || (a.rotary_dim == hd && !a.interleaved)) &&
                          aligned16(a.q_norm) && aligned16(a.k_norm) && aligned16(a.cos) && aligned16(a.sin) && aligned16(e.k) &&
                          aligned16(e.v) && row % 8 == 0 && aligned16(s.qkv) && tc_takes(s.xn, m.hidden, a.qkv);
    if (prepared)
        TRY(LAUNCH(f.gemm_tc_qkv, s.xn, a.qkv.w, s.qkv, n, a.n_heads, a.n_kv_heads, a.qkv.k, (long long)m.hidden, a.qkv.ldw, row,
                   s.token_seq, s.token_pos, s.seq_slot, a.q_norm, a.k_norm, a.eps, a.cos, a.sin, e.k, e.v, e.table, e.table_width,
                   e.tokens_per_page, m.kernel_status, stream),
            "the q/k/v product");
    else if (writes) TRY(linear(m, a.qkv, s.xn, m.hidden, s.qkv, m.dtype, row, n, stream), "the q/k/v product");
    else TRY(linear(m, a.q_only, s.xn, m.hidden, s.qkv, m.dtype, row, n, stream), "the q product");
    const size_t decode_smem = (size_t)4 * 64 * hd * 2 + (size_t)4 * group * (hd + 2) * 4 + 64;
    const bool decode_takes = has_cache && (hd == 64 || hd == 128 || hd == 256) && e.tokens_per_page == 64 && decode_smem <= 200 * 1024;
    // kernels/ops.py: attention_decode_prepares
    const bool prepares = m.decode_prepares && s.is_decode && bf16 && decode_takes && hd != 256 && group <= 16 &&
                          (!a.cos || (a.rotary_dim == hd && !a.interleaved)) && row % 8 == 0 && aligned16(s.qkv) &&
                          aligned16(a.q_norm) && aligned16(a.k_norm) && aligned16(a.cos) && aligned16(a.sin) && aligned16(e.k) &&
                          aligned16(e.v);
    if (!prepares && !prepared)
        TRY(LAUNCH(f.qkv_prep, s.qkv, m.dtype, n, a.n_heads, a.n_kv_heads, a.head_dim, writes ? 0 : 1, s.token_seq, s.token_pos,
                   s.seq_slot, s.seq_len_after, a.q_norm, a.k_norm, a.eps, a.cos, a.sin, a.rotary_dim, a.interleaved,
                   writes ? e.k : nullptr, writes ? e.v : nullptr, writes ? e.table : nullptr, writes ? e.table_width : 0,
                   writes ? e.ring_pages : 0, writes ? e.tokens_per_page : 1, stream),
        "q/k/v preparation");
    if (from_step && (s.any_continuation || !writes)) return fail(STEP_REFUSED_WINDOW, "windowed attention", entry);
    const bool prefill_takes = has_cache && (hd == 64 || hd == 128) && e.tokens_per_page == 64 && e.ring_pages == 0;
    const AbkLists *lists = a.lists >= 0 && a.lists < s.n_lists ? &s.lists[a.lists] : nullptr;
    if (s.is_decode && !from_step && bf16 && decode_takes) {
        const int bound = s.position_bound > 0 ? s.position_bound : s.max_len_after;
        if (prepares) {
            TRY(LAUNCH(f.attention_decode_ring_prepare, s.qkv, row, s.att, n, a.n_heads, a.n_kv_heads, hd, a.scale, a.window,
                       s.token_seq, s.token_pos, s.seq_slot, e.k, e.v, e.pool_rows, e.table, e.table_width, e.ring_pages,
                       e.tokens_per_page, bound, a.q_norm, a.k_norm, a.eps, a.cos, a.sin, writes ? 1 : 0, m.kernel_status, stream),
                "decode attention");
        } else if (hd != 256 && group <= 16) {
            TRY(LAUNCH(f.attention_decode_ring, s.qkv, row, s.att, n, a.n_heads, a.n_kv_heads, hd, a.scale, a.window, s.token_seq,
                                        s.token_pos, s.seq_slot, e.k, e.v, e.pool_rows, e.table, e.table_width, e.ring_pages,
                                        e.tokens_per_page, bound, m.kernel_status, stream),
                "decode attention");
        } else {
            const long long chunks = (bound + 127) / 128, floats = (long long)n * a.n_heads * chunks * (hd + 2);
            if (floats > s.partial_floats) return fail(STEP_REFUSED_PARTIALS, "decode attention", entry);
            if ((long long)n * a.n_kv_heads > m.attention_ticket_count) return fail(STEP_REFUSED_TICKETS, "decode attention", entry);
            TRY(LAUNCH(f.attention_decode, s.qkv, row, s.att, n, a.n_heads, a.n_kv_heads, hd, a.scale, a.window, s.token_seq, s.token_pos,
                                   s.seq_slot, e.k, e.v, e.table, e.table_width, e.ring_pages, e.tokens_per_page, bound,
                                   s.attention_partials, m.attention_tickets, m.kernel_status, stream),
                "decode attention");
        }
    } else if (!s.is_decode && !from_step && a.window == 0 && bf16 && lists && prefill_takes) {
        if (hd == 128) {
            const int room = m.halves_pairs / a.n_heads;
            if (lists->n_halved > room) return fail(STEP_REFUSED_HALVES, "prefill attention", entry);
            TRY(LAUNCH(f.attention_prefill_tc, s.qkv, row, n, s.att, a.n_heads, a.n_kv_heads, hd, a.scale, lists->work, lists->n_work, room,
                                       m.halves, m.halves_tickets, e.k, e.v, e.pool_rows, e.table, e.table_width,
                                       e.tokens_per_page, m.kernel_status, stream),
                "prefill attention");
        } else {
            TRY(LAUNCH(f.attention_prefill, s.qkv, row, n, s.att, a.n_heads, a.n_kv_heads, hd, a.scale, lists->tiles64, lists->n_tiles64,
                                    s.seq_start, s.seq_pos0, s.seq_len_after, s.seq_slot, e.k, e.v, e.pool_rows, e.table,
                                    e.table_width, e.tokens_per_page, m.kernel_status, stream),
                "prefill attention");
        }
    } else {
        const char *base = (const char *)s.qkv;
        const void *k_step = from_step ? base + (size_t)q_size * esize(m.dtype) : nullptr;
        const void *v_step = from_step ? base + (size_t)(q_size + kv_size) * esize(m.dtype) : nullptr;
        TRY(LAUNCH(f.attention_generic, s.qkv, row, s.att, m.dtype, n, a.n_heads, a.n_kv_heads, hd, a.scale, a.window, s.token_seq,
                                s.token_pos, s.seq_slot, s.seq_start, s.seq_pos0, has_cache ? e.k : nullptr,
                                has_cache ? e.v : nullptr, has_cache ? e.table : nullptr, has_cache ? e.table_width : 0,
                                has_cache ? e.ring_pages : 0, has_cache ? e.tokens_per_page : 1, k_step, v_step, row, stream),
            "attention");
    }
    TRY(linear(m, a.o, s.att, q_size, s.branch, ABK_F32, m.hidden, n, stream), "the output product");
    return STEP_OK;
}

// parts/mlp.py: GatedMLP.forward
static int gated_mlp(const AbkModel &m, const AbkMlp &p, const AbkStep &s, int entry, void *stream) {
    const AbkFns &f = *m.fns;
    const int n = s.n_rows;
    const AbkLinear &gu = p.gate_up;
    const bool bf16 = m.dtype == ABK_BF16;
    if (bf16 && rows_kernel_wins(n, gu, true) && rows_takes(s.xn, m.hidden, gu, n)) {
        TRY(LAUNCH(f.gemm_rows_swiglu, s.xn, gu.w, s.act, n, p.inter, gu.k, m.hidden, gu.ldw, p.inter, p.block, stream),
            "gate/up with SwiGLU");
    } else if (bf16 && p.block == 128 && n > 256 && gu.n % 256 == 0 && p.inter % 8 == 0 && aligned16(s.act) &&
               tc_takes(s.xn, m.hidden, gu)) {
        TRY(LAUNCH(f.gemm_tc_swiglu, s.xn, gu.w, s.act, n, p.inter, gu.k, m.hidden, gu.ldw, p.inter, m.kernel_status, stream),
            "gate/up with SwiGLU");
    } else {
        TRY(linear(m, gu, s.xn, m.hidden, s.gate_up, m.dtype, 2ll * p.inter, n, stream), "the gate/up product");
        TRY(LAUNCH(f.swiglu, s.gate_up, s.act, m.dtype, n, p.inter, p.block, stream), "SwiGLU");
    }
    TRY(linear(m, p.down, s.act, p.inter, s.branch, ABK_F32, m.hidden, n, stream), "the down product");
    return STEP_OK;
}

// models/model.py: Model.forward with parts/frame.py (plain) and parts/block.py (pre_norm). src/model.c:286-327.
extern "C" int abk_step(const AbkModel *model, const AbkStep *step, void *stream) {
    const AbkModel &m = *model;
    const AbkStep &s = *step;
    const AbkFns &f = *m.fns;
    int entry = -1;
    step_error[0] = 0, step_launches = 0;
    if (s.n_rows <= 0) return STEP_OK;
    TRY(LAUNCH(f.embed, s.tokens, m.embed, m.dtype, s.x, s.n_rows, m.hidden, m.vocab, m.status, stream), "the embedding");
    const float *pending = nullptr;  // the branch output still to be added to the stream (src/model.c:297, 305, 311)
    for (entry = 0; entry < m.n_entries; entry++) {
        const AbkEntry &e = m.entries[entry];
        const AbkBlock &b = m.blocks[e.block];
        TRY(LAUNCH(f.add_rmsnorm, s.x, pending, b.norm1.w, s.xn, m.dtype, nullptr, s.n_rows, m.hidden, b.norm1.eps, stream), "add + norm");
        if (int rc = attention(m, b.att, e, s, entry, stream)) return rc;
        TRY(LAUNCH(f.add_rmsnorm, s.x, s.branch, b.norm2.w, s.xn, m.dtype, nullptr, s.n_rows, m.hidden, b.norm2.eps, stream), "add + norm");
        if (int rc = gated_mlp(m, b.mlp, s, entry, stream)) return rc;
        pending = s.branch;
    }
    entry = -1;
    if (s.n_logit_rows > 0) {
        TRY(LAUNCH(f.add_rmsnorm, s.x, pending, m.final_norm.w, s.xn_final, m.dtype, s.logit_rows, s.n_logit_rows, m.hidden,
                          m.final_norm.eps, stream),
            "the last norm");
        TRY(linear(m, m.head, s.xn_final, m.hidden, s.logits, ABK_F32, m.vocab, s.n_logit_rows, stream), "the output matrix");
    }
    return STEP_OK;
}

// Sizes of the structures, for the caller to check its own declarations against.
extern "C" int abk_step_sizeof(int which) {
    switch (which) {
    case 0: return (int)sizeof(AbkFns);
    case 1: return (int)sizeof(AbkLinear);
    case 2: return (int)sizeof(AbkNorm);
    case 3: return (int)sizeof(AbkAttention);
    case 4: return (int)sizeof(AbkMlp);
    case 5: return (int)sizeof(AbkBlock);
    case 6: return (int)sizeof(AbkEntry);
    case 7: return (int)sizeof(AbkModel);
    case 8: return (int)sizeof(AbkLists);
    case 9: return (int)sizeof(AbkStep);
    }
    return -1;
}
