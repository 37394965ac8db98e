// Causal prefill attention on the 5th-generation tensor cores (tcgen05), head size 128, bfloat16
// paged cache, no window.
//
// A CTA takes 128 query rows of one (sequence, head) and all pages of keys the last of the rows may see,
// or, for a tile that sees many (the tiles of a prompt see from 1 to all of its pages, and a kernel lasts
// as long as its longest CTA), the earlier or the later half of them: then both CTAs leave their partial
// the CTA that is through first leaves its partial result (O, maximum, sum) in scratch memory, and the other
// one adds the two, always in the same order, and stores the rows. (Pairs as thread-block clusters, with the partial
// result handed over through distributed shared memory, were measured slower: a cluster needs a free
// place on both SMs of a pair at once, and a sixth of the places stayed empty.) The CTAs run in the order
// of the work list, longest first, all heads of an entry together. A CTA walks its pages 64 keys at a time:
//   warp 0     TMA: the query tile once ([128, 128] as two swizzled boxes), then a page of keys and
//              a page of values per step into a ring of three stages;
//   warp 1     one thread issues tcgen05.mma: S = Q K^T (128 x 64, into one of two score buffers in
//              tensor memory) and O += P V (128 x 128, P from shared memory, V as an MN-major
//              operand straight from the page), S of the next page before O of this one, so that
//              the softmax of page j+1 runs under the second product of page j;
//   warps 2-9  two threads per query row, 32 of the page's 64 keys each (a warp reaches only its own
//              quarter of the lanes of tensor memory, so warps w and w + 4 share 32 rows): each reads
//              its half row of S (tcgen05.ld), masks (only pages that cross the diagonal), and swaps
//              its maximum with its partner through shared memory; both then hold the row's maximum,
//              keep the same reference, and each writes its half of P as bfloat16 into shared memory
//              in the swizzled layout the tensor core reads, keeps its half of the row's sum, and, when
//              the maximum has outgrown the reference by 2^8, rescales its half of the row of O in
//              tensor memory (tcgen05.ld / tcgen05.st) between two second products. A step of a
//              (sequence, head) is bound by this chain, not by the tensor cores: halving the row
//              halves every dependent run of instructions in it.
// Tensor memory: 2 x 64 columns of scores + 128 columns of output = 256 of 512. Every wait on an
// mbarrier is bounded; a wait that runs out sets status word 3 and the CTA winds down.
// Formula: src/model.c:197-211; softmax in float32, probabilities rounded to bfloat16 for P V.
#define ABK_DEFINE_ERROR
#include "common.cuh"
#include "tc_common.cuh"
#include "tensor_map.cuh"

#define TQ 128        // query rows per CTA
#define TK 64         // keys per step: one page
#define HD 128
#define KV_STAGES 2   // with the query tile and one P tile: 112 KB, two CTAs to an SM
#define FA_THREADS 320
#define Q_BYTES (TQ * HD * 2)       // two boxes of [128 rows, 64 columns]
#define KV_BYTES (TK * HD * 2)      // two boxes of [64 rows, 64 columns]
#define P_BYTES (TQ * TK * 2)       // one box of [128 rows, 64 columns]
#define BOX_Q (TQ * 128)            // bytes of a query box
#define BOX_KV (TK * 128)           // bytes of a key or value box

struct AttnTc {
    __nv_bfloat16 *out;  // [tokens, n_heads * HD]
    int n_heads, n_kv_heads;
    float scale_log2;
    // [n_work][8], a CTA's work: sequence of the step (-1: none), first of its 128 rows among the sequence's new
    // tokens, part (0: all pages of keys the rows see; 1, 2: the earlier and the later half), then the sequence's
    // first row in the step, its first new position, its new tokens, its slot, and for a halved tile its number
    // among the halved tiles
    const int4 *work;
    PagedCache cache;
    float *partial_o;   // [halved tiles][heads][32 groups of 4 columns][128 rows][4]: of the half that was through first
    float *partial_ml;  // [halved tiles][heads][128 rows][2]: its reference (in units of log2) and sum
    int *tickets;       // [halved tiles][heads][2]: who is through; the partial result is there. Zero before and after
    int *status;
};

// Shared-memory descriptor of a B operand whose N dimension is contiguous (values: [key][head_dim]),
// stored as boxes of [rows = keys, 64 columns] with the 128-byte swizzle: 8 keys are 1024 bytes apart
// (stride offset), the next 64 columns are `next_box` bytes on (leading offset).
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t next_box) {
    uint64_t d = (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((next_box >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// K-major operand made of boxes of [rows, 64 columns]: one box per 64 of K; inside a box +32 bytes per 16 of K.
__device__ __forceinline__ uint64_t k_major_desc(uint32_t base, uint32_t box_bytes, int k16) {
    return tc::smem_desc_k_sw128(base + (k16 / 4) * box_bytes + (k16 % 4) * 32);
}
__host__ __device__ constexpr uint32_t idesc_b_mn(int m, int n) { return tc::idesc_bf16_f32(m, n) | (1u << 16); }

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
// 2^x by the special-function unit alone (arguments here are at most 8; -inf gives 0).
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// The two warps of a quarter (64 threads) meet; the ids are literal so that the CTA asks for five barriers, not sixteen.
__device__ __forceinline__ void pair_sync(int quarter) {
    switch (quarter) {
    case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
    case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
    case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
    default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
    }
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__global__ void __launch_bounds__(FA_THREADS, 2) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map,
                                                                     const __grid_constant__ CUtensorMap k_map,
                                                                     const __grid_constant__ CUtensorMap v_map, AttnTc p) {
    extern __shared__ __align__(1024) uint8_t smem[];  // the kernel has no static shared memory: this starts aligned
    uint8_t *q_s = smem, *k_s = q_s + Q_BYTES, *v_s = k_s + KV_STAGES * KV_BYTES, *p_s = v_s + KV_STAGES * KV_BYTES;
    uint64_t *bars = (uint64_t *)(p_s + P_BYTES);
    uint64_t *q_full = bars, *k_full = bars + 1, *k_empty = k_full + KV_STAGES, *v_full = k_empty + KV_STAGES,
             *v_empty = v_full + KV_STAGES, *s_full = v_empty + KV_STAGES, *p_full = s_full + 2,
             *o_step = p_full + 2;  // o_step: the second product of a page is done
    uint32_t *tmem_holder = (uint32_t *)(o_step + 1);
    volatile int *failed = (volatile int *)(tmem_holder + 1);
    // [2 halves][128 rows]: the halves' maxima, rounded up to bfloat16 (any common bound of the row's scores
    // serves as the reference; the few bytes more that float32 would take are the difference between one and two
    // CTAs on an SM)
    __nv_bfloat16 *swap = (__nv_bfloat16 *)(tmem_holder + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef ABK_TRACE
    const unsigned long long trace_begin = abk_trace_ns();
#endif
    // Before pdl_wait(): what kernels further back than the one just before this wrote (the step's index arrays,
    // the page table), and the CTA's own set-up. The loads that do not depend on one another go out together.
    const int h = blockIdx.x % p.n_heads, entry = blockIdx.x / p.n_heads;  // all heads of an entry, then the next entry
    const int4 w0 = p.work[2 * entry], w1 = p.work[2 * entry + 1];
    const int seq = w0.x, row0 = w0.y, part = w0.z;
    if (seq < 0) return;  // padding of the work list (a captured step has a fixed length)
    const bool split = part != 0;
    const int rank = split ? part - 1 : 0;
    const long long pair = (long long)w1.w * p.n_heads + h;  // of a halved tile: which partial results and ticket are its
    // an earlier CTA gave up on a wait: do not queue up behind it (one thread looks, so that all decide alike)
    if (threadIdx.x == 0) {
        *(volatile int *)swap = *(volatile int *)(p.status + 3);
        *failed = 0;
        tc::mbar_init(q_full, 1);
        for (int s = 0; s < KV_STAGES; s++)
            tc::mbar_init(&k_full[s], 1), tc::mbar_init(&k_empty[s], 1), tc::mbar_init(&v_full[s], 1), tc::mbar_init(&v_empty[s], 1);
        for (int b = 0; b < 2; b++) tc::mbar_init(&s_full[b], 1), tc::mbar_init(&p_full[b], 256);
        tc::mbar_init(o_step, 1);
        tc::mbar_init_fence();
        tc::tma_prefetch_map(&q_map), tc::tma_prefetch_map(&k_map), tc::tma_prefetch_map(&v_map);
    }
    const int kvh = h / (p.n_heads / p.n_kv_heads);
    const int start = w0.w, pos0 = w1.x, n_new = w1.y, slot = w1.z;
    const int last_row = min(row0 + TQ - 1, n_new - 1);
    const int all_steps = (pos0 + last_row) / TK + 1;  // pages of keys the tile's last row sees
    // this CTA's pages: of a pair that shares a tile the first takes the earlier half, the second the later one
    const int cut = split ? (all_steps + 1) / 2 : all_steps;
    const int first = rank ? cut : 0, my_steps = rank ? all_steps - cut : cut;
    // the pool rows of the first 32 of them are looked up now, under the set-up
    int y_first = 0;
    if (warp == 0 && lane < my_steps) y_first = (cache_page(p.cache, slot, (first + lane) * TK) * p.n_kv_heads + kvh) * TK;
    __syncthreads();
    // A CTA that finds the flag set does none of its steps but still takes its ticket if its tile is halved.
    // swap is first written for its own purpose after the next barrier.
    const bool quit = *(volatile int *)swap != 0;
    const int n_steps = quit ? 0 : my_steps;
    if (warp == 1) tc::tmem_alloc(tmem_holder, 256);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = *tmem_holder, tmem_o = tmem + 128;
    // what a softmax thread (warps 2-9) keeps for the end; the other warps leave these as they are
    const int quarter = warp & 3, r = quarter * 32 + lane;  // its query row within the tile
    const int half = warp >= 2 ? (warp - 2) >> 2 : 0;          // which 32 of a page's 64 keys, and which 64 columns of O
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    float m = -INFINITY, l = 0.0f;  // the reference of the row's exponentials; their sum (this thread's keys; at the end the row's)
    bool ok = true;

    if (warp == 0) {
        // Keys and values have rings of their own: a stage of keys is free once the first product of its
        // page is done, a whole step before the stage of values is, so the next keys are under way that
        // much earlier and the first product of a step does not wait for its load. Every lane looks up the
        // pool row of one of the next 32 pages, so that the table's latency is paid once for all of them.
        int k_issued = 0, v_issued = 0;
        bool go = true;
        for (int base = 0; base < n_steps && go; base += 32) {
            const int y_lane = base == 0              ? y_first
                               : base + lane < n_steps ? (cache_page(p.cache, slot, (first + base + lane) * TK) * p.n_kv_heads + kvh) * TK
                                                       : 0;
            if (base == 0) {
                pdl_wait();  // q, and the keys and values of this step's tokens, come from the kernel just before
                if (lane == 0) {
                    tc::mbar_expect_tx(q_full, Q_BYTES);
                    tc::tma_load_2d(q_s, &q_map, h * HD, start + row0, q_full);
                    tc::tma_load_2d(q_s + BOX_Q, &q_map, h * HD + 64, start + row0, q_full);
                }
            }
            const int n = min(32, n_steps - base);
            for (int i = 0; i < n && go; i++) {
                const int j = base + i, s = j % KV_STAGES;
                const uint32_t parity = ((j / KV_STAGES) & 1) ^ 1;
                const int y = __shfl_sync(0xffffffffu, y_lane, i);
                int bad = 0;
                if (lane == 0) {
                    if (!tc::mbar_wait(&k_empty[s], parity)) {
                        bad = 1;
                    } else {
                        tc::mbar_expect_tx(&k_full[s], KV_BYTES);
                        tc::tma_load_2d(k_s + s * KV_BYTES, &k_map, 0, y, &k_full[s]);
                        tc::tma_load_2d(k_s + s * KV_BYTES + BOX_KV, &k_map, 64, y, &k_full[s]);
                        k_issued++;
                        if (!tc::mbar_wait(&v_empty[s], parity)) {
                            bad = 1;
                        } else {
                            tc::mbar_expect_tx(&v_full[s], KV_BYTES);
                            tc::tma_load_2d(v_s + s * KV_BYTES, &v_map, 0, y, &v_full[s]);
                            tc::tma_load_2d(v_s + s * KV_BYTES + BOX_KV, &v_map, 64, y, &v_full[s]);
                            v_issued++;
                        }
                    }
                }
                if (__shfl_sync(0xffffffffu, bad, 0)) go = false;
            }
        }
        if (!go && lane == 0) {  // let the copies in flight land before the CTA's memory goes away
            atomicOr(p.status + 3, 2);
            *failed = 1;
            for (int i = max(0, k_issued - KV_STAGES); i < k_issued; i++) tc::mbar_wait(&k_full[i % KV_STAGES], (i / KV_STAGES) & 1);
            for (int i = max(0, v_issued - KV_STAGES); i < v_issued; i++) tc::mbar_wait(&v_full[i % KV_STAGES], (i / KV_STAGES) & 1);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = tc::idesc_bf16_f32(TQ, TK), idesc_o = idesc_b_mn(TQ, HD);
            const uint32_t qa = tc::smem_addr(q_s);
            bool ok = n_steps == 0 || tc::mbar_wait(q_full, 0);
            if (!ok) atomicOr(p.status + 3, 4);
            // step j (of this CTA's): S(j) = Q K(j)^T, then O += P(j-1) V(j-1); one more turn for the last second product
            for (int j = 0; j <= n_steps && ok && n_steps > 0; j++) {
                if (j < n_steps) {
                    const int s = j % KV_STAGES, b = j & 1;
                    ok = ok && tc::mbar_wait(&k_full[s], (j / KV_STAGES) & 1);
                    if (!ok) atomicOr(p.status + 3, 8);
                    // the score buffer is free once the softmax of step j-2 has delivered its P
                    if (ok && j >= 2) {
                        ok = tc::mbar_wait(&p_full[b], ((j - 2) >> 1) & 1);
                        if (!ok) atomicOr(p.status + 3, 16);
                    }
                    if (!ok) break;
                    tc::fence_after_sync();
                    const uint32_t kb = tc::smem_addr(k_s + s * KV_BYTES);
#pragma unroll
                    for (int k16 = 0; k16 < HD / 16; k16++)
                        tc::mma_ss(tmem + b * TK, k_major_desc(qa, BOX_Q, k16), k_major_desc(kb, BOX_KV, k16), idesc_s, k16 > 0);
                    tc::mma_commit(&s_full[b]);
                    tc::mma_commit(&k_empty[s]);  // the page's keys may be replaced
                }
                if (j >= 1) {
                    const int i = j - 1, s = i % KV_STAGES, b = i & 1;
                    ok = tc::mbar_wait(&p_full[b], (i >> 1) & 1);  // P(i) is in shared memory, O is rescaled
                    ok = ok && tc::mbar_wait(&v_full[s], (i / KV_STAGES) & 1);
                    if (!ok) {
                        atomicOr(p.status + 3, 32);
                        break;
                    }
                    tc::fence_after_sync();
                    const uint32_t pa = tc::smem_addr(p_s), vb = tc::smem_addr(v_s + s * KV_BYTES);
#pragma unroll
                    for (int k16 = 0; k16 < TK / 16; k16++)
                        tc::mma_ss(tmem_o, tc::smem_desc_k_sw128(pa + k16 * 32), smem_desc_mn_sw128(vb + k16 * 2048, BOX_KV),
                                   idesc_o, i > 0 || k16 > 0);
                    tc::mma_commit(&v_empty[s]);  // the page's values may be replaced
                    tc::mma_commit(o_step);        // and the softmax warps may touch O again
                }
            }
            if (!ok) *failed = 1;
        }
    } else {
        pdl_wait();  // before anything is written to global memory
        const int col0 = half * (TK / 2);
        const int qpos = pos0 + row0 + r;
        const float GONE = __int_as_float(0x7fc00000);  // what a warp that has given up leaves for its partner
        for (int j = 0; j < n_steps; j++) {
            const int b = j & 1;
            // The two warps of a quarter meet at a barrier in every step, so they must leave the loop in the
            // same step: a warp that ran out of time says so through the value it swaps, and both go.
            bool fine = ok && tc::mbar_wait(&s_full[b], (j >> 1) & 1);
            fine = __all_sync(0xffffffffu, fine);
            if (ok && !fine) atomicOr(p.status + 3, 64);
            float s[TK / 2];
            float mx = -INFINITY;  // of the raw scores; the scale (positive) is applied to the maximum
            if (fine) {
                tc::fence_after_sync();
#pragma unroll
                for (int c0 = 0; c0 < TK / 2; c0 += 16) tc::tmem_ld16(tmem + lane_base + b * TK + col0 + c0, (uint32_t *)(s + c0));
                tc::tmem_ld_wait();
                const int key0 = (first + j) * TK;  // the page's first key
                const bool edge = key0 + TK - 1 > pos0 + row0;  // some key of this page lies after some row of the tile
                if (edge) {
#pragma unroll
                    for (int c = 0; c < TK / 2; c++)
                        if (key0 + col0 + c > qpos) s[c] = -INFINITY;
                }
                // two runs of maxima instead of one of 32 dependent instructions
                float mx2 = -INFINITY;
#pragma unroll
                for (int c = 0; c < TK / 2; c += 2) mx = fmaxf(mx, s[c]), mx2 = fmaxf(mx2, s[c + 1]);
                mx = fmaxf(mx, mx2);
            }
            const __nv_bfloat16 mine_up = __float2bfloat16_ru(fine ? mx : GONE);
            pair_sync(quarter);  // the partner has read what the step before left here
            swap[half * TQ + r] = mine_up;
            pair_sync(quarter);
            const float theirs = __bfloat162float(swap[(half ^ 1) * TQ + r]);
            if (__any_sync(0xffffffffu, !fine || theirs != theirs)) {
                ok = false;
                break;
            }
            mx = fmaxf(__bfloat162float(mine_up), theirs);
            mx *= p.scale_log2;
            // `m` is the reference the row's exponentials, its sum and its O are scaled by. It follows the
            // true maximum only when that has outgrown it by 2^8 (the probabilities stay below 256, well
            // inside bfloat16 and float32), so that O is rescaled on a few early steps only; the final
            // O / l does not depend on the reference. Both warps of a quarter see the same maxima and
            // the same references, so they decide alike.
            // The reference is always a whole number (a power of two as a factor): a key's probability is then the
            // same bits times a power of two whatever reference its step had, and rounds to the same bfloat16.
            const float cand = fmaxf(m, ceilf(mx));
            const bool move = __any_sync(0xffffffffu, cand > m + 8.0f);  // the first step: m is -inf
            const float m_new = move ? cand : m;
            const float ref = m_new == -INFINITY ? 0.0f : m_new;
            const float corr = exp2f(m - ref);
            float sum0 = 0.0f, sum1 = 0.0f;
            uint32_t packed[TK / 4];
#pragma unroll
            for (int c = 0; c < TK / 2; c += 2) {
                float p0 = ex2(fmaf(s[c], p.scale_log2, -ref)), p1 = ex2(fmaf(s[c + 1], p.scale_log2, -ref));
                sum0 += p0, sum1 += p1;
                __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
                packed[c / 2] = *(uint32_t *)&t;
            }
            l = l * corr + (sum0 + sum1);
            // P's tile and O may be touched only between two second products: wait for the one of step j-1
            if (j >= 1 && !__all_sync(0xffffffffu, tc::mbar_wait(o_step, (j - 1) & 1))) {
                atomicOr(p.status + 3, 128);
                ok = false;  // the partner hears of it at the next step's barrier (or both are through)
                continue;
            }
            // P(j) as a K-major operand: row r, 128 bytes, eight 16-byte chunks swizzled by the row; this thread's four
            uint8_t *prow = p_s + r * 128;
#pragma unroll
            for (int ch = 0; ch < 4; ch++)
                *(uint4 *)(prow + (((4 * half + ch) ^ (r & 7)) << 4)) =
                    make_uint4(packed[4 * ch], packed[4 * ch + 1], packed[4 * ch + 2], packed[4 * ch + 3]);
            if (j >= 1 && move) {
                tc::fence_after_sync();
#pragma unroll 1
                for (int c0 = 0; c0 < HD / 2; c0 += 16) {
                    uint32_t v[16];
                    tc::tmem_ld16(tmem_o + lane_base + half * (HD / 2) + c0, v);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 16; e++) v[e] = __float_as_uint(__uint_as_float(v[e]) * corr);
                    tmem_st16(tmem_o + lane_base + half * (HD / 2) + c0, v);
                }
                tmem_st_wait();
            }
            m = m_new;
            fence_async_smem();  // P written by this thread is visible to the tensor core
            tc::fence_before_sync();
            tc::mbar_arrive(&p_full[b]);
        }
        // the last second product of this CTA's pages
        if (ok && n_steps > 0 && !tc::mbar_wait(o_step, (n_steps - 1) & 1)) {
            atomicOr(p.status + 3, 256);
            ok = false;
        }
        if (!ok) *failed = 1;
        tc::fence_after_sync();
        // the row's sum is the two halves' (their reference is the same); P's tile is free now and carries them
        float *sums = (float *)p_s;
        sums[half * TQ + r] = l;
        pair_sync(quarter);
        l += sums[(half ^ 1) * TQ + r];
    }
    // A halved tile: the CTA that is through first (it takes ticket 0) leaves O (column groups of four, so that
    // the 32 rows of a warp lie side by side), reference and sum in scratch memory and raises a flag; the other
    // one waits for the flag, adds the two, always in the same order, and stores the rows.
    float w_own = 1.0f, w_other = 0.0f, l_all = l;
    const float *other_o = nullptr;
    bool store = !split;
    if (split) {
        __syncthreads();
        if (threadIdx.x == 0) *(volatile int *)swap = atomicAdd(p.tickets + 2 * pair, 1);
        __syncthreads();
        store = *(volatile int *)swap == 1;
        if (!store) {
            if (warp >= 2) {
                tc::fence_after_sync();
                float *mine_o = p.partial_o + pair * (TQ * HD);
                if (half == 0) *(float2 *)(p.partial_ml + (pair * TQ + r) * 2) = make_float2(n_steps > 0 ? m : -INFINITY, l);
#pragma unroll
                for (int c0 = 0; c0 < HD / 2; c0 += 32) {
                    uint32_t v[32];
                    tc::tmem_ld16(tmem_o + lane_base + half * (HD / 2) + c0, v);
                    tc::tmem_ld16(tmem_o + lane_base + half * (HD / 2) + c0 + 16, v + 16);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        *(uint4 *)(mine_o + (((half * (HD / 2) + c0) / 4 + q) * TQ + r) * 4) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                }
                __threadfence();
            }
            __syncthreads();
            if (threadIdx.x == 0) atomicExch(p.tickets + 2 * pair + 1, 1);  // the partial result is there
        } else {
            // the other CTA has its ticket, so it is running: its flag comes within microseconds, or something is broken
            if (threadIdx.x == 0) {
                const uint64_t t0 = tc::global_ns();
                int seen = 0;
                while (!(seen = atomicAdd(p.tickets + 2 * pair + 1, 0)) && tc::global_ns() - t0 < tc::abk_wait_limit_ns) __nanosleep(100);
                if (!seen) atomicOr(p.status + 3, 512), *failed = 1;
                p.tickets[2 * pair] = 0, p.tickets[2 * pair + 1] = 0;  // as they were, for the next launch
                *(volatile int *)swap = seen;
            }
            __syncthreads();
            if (!*(volatile int *)swap) ok = false;
            __threadfence();
            if (warp >= 2) {
                const float2 ml = __ldcg((const float2 *)(p.partial_ml + (pair * TQ + r) * 2));
                const float own_m = n_steps > 0 ? m : -INFINITY, top = fmaxf(own_m, ml.x);  // one of the two has had pages
                w_own = own_m == -INFINITY ? 0.0f : exp2f(own_m - top), w_other = ml.x == -INFINITY ? 0.0f : exp2f(ml.x - top);
                // the earlier half's share first, whoever adds them: the sum does not depend on who came second
                l_all = rank == 0 ? fmaf(w_other, ml.y, l * w_own) : fmaf(w_own, l, ml.y * w_other);
                other_o = p.partial_o + pair * (TQ * HD);
            }
        }
    }
    if (store && warp >= 2) {
        tc::fence_after_sync();
        // tcgen05.ld is a whole-warp instruction: every lane reads its row, only rows of the sequence are stored
        if (__all_sync(0xffffffffu, ok) && (n_steps > 0 || split)) {
            const bool mine = row0 + r < n_new;
            const float inv = 1.0f / l_all;
            __nv_bfloat16 *dst = p.out + ((long long)(start + row0 + r) * p.n_heads + h) * HD + half * (HD / 2);
#pragma unroll
            for (int c0 = 0; c0 < HD / 2; c0 += 32) {
                uint32_t v[32], hpk[16];
                float o[32];
                float4 t[8];
                if (other_o) {  // (under the loads from tensor memory)
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        t[q] = w_other != 0.0f ? __ldcg((const float4 *)(other_o + (((half * (HD / 2) + c0) / 4 + q) * TQ + r) * 4))
                                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
                tc::tmem_ld16(tmem_o + lane_base + half * (HD / 2) + c0, v);
                tc::tmem_ld16(tmem_o + lane_base + half * (HD / 2) + c0 + 16, v + 16);
                tc::tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; e++) o[e] = w_own == 0.0f ? 0.0f : __uint_as_float(v[e]);  // (no pages: nothing was written there)
                if (other_o) {
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        const float th[4] = {t[q].x, t[q].y, t[q].z, t[q].w};
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            o[4 * q + e] = rank == 0 ? fmaf(w_other, th[e], o[4 * q + e] * w_own) : fmaf(w_own, o[4 * q + e], th[e] * w_other);
                    }
                }
#pragma unroll
                for (int e2 = 0; e2 < 16; e2++) {
                    __nv_bfloat162 tt = __floats2bfloat162_rn(o[2 * e2] * inv, o[2 * e2 + 1] * inv);
                    hpk[e2] = *(uint32_t *)&tt;
                }
                if (mine) {
#pragma unroll
                    for (int q = 0; q < 4; q++) *(uint4 *)(dst + c0 + 8 * q) = make_uint4(hpk[4 * q], hpk[4 * q + 1], hpk[4 * q + 2], hpk[4 * q + 3]);
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (*failed && threadIdx.x == 0) atomicOr(p.status + 3, 1);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_free(tmem, 256);
    }
#ifdef ABK_TRACE
    if (threadIdx.x == 0) {  // every CTA's life: begin, end, its tile and head, its steps and its SM + 1 (a launch's record has 0 there)
        unsigned int i = atomicAdd(&abk_trace_count, 1u), sm;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
        if (i < ABK_TRACE_MAX)
            abk_trace_records[i] = {trace_begin, abk_trace_ns(), ABK_TRACE, (int)(blockIdx.x + (blockIdx.y << 16)), n_steps, (int)sm + 1};
    }
#endif
}

// qkv: the step's rows [n_rows, row_width] (q columns first); out [n_rows, n_heads * 128].
// work: int32 [n_work, 8] on the device, 16-byte aligned: what each CTA does (see AttnTc), for all heads. A halved
// tile has two entries and a number below max_halved. No window.
// scratch: float32 [abk_attention_prefill_tc_scratch_floats(max_halved, n_heads)]; tickets: int32 [2 * max_halved *
// n_heads], zero before and after. status word 3 is set if a wait ran out.
extern "C" long long abk_attention_prefill_tc_scratch_floats(int max_halved, int n_heads) {
    return (long long)max_halved * n_heads * (TQ * HD + TQ * 2);
}
extern "C" int abk_attention_prefill_tc(const void *qkv, long long row_width, int n_rows, void *out, int n_heads,
                                        int n_kv_heads, int head_dim, float scale, const int *work, int n_work,
                                        int max_halved, float *scratch, int *tickets, const void *k_pool, const void *v_pool, long long pool_rows,
                                        const int *page_table, int table_width, int tokens_per_page, int *status,
                                        void *stream) {
    if (n_work <= 0) return 0;
    if ((uintptr_t)work % 16 || (uintptr_t)scratch % 16) ABK_REFUSE("attention_prefill_tc: the work list and the scratch memory must be 16-byte aligned");
    if ((long long)n_work * n_heads > 0x7fffffffLL) ABK_REFUSE("attention_prefill_tc: %d entries for %d heads exceed a grid", n_work, n_heads);
    if (head_dim != HD) ABK_REFUSE("attention_prefill_tc: head_dim %d is not %d", head_dim, HD);
    if (tokens_per_page != TK) ABK_REFUSE("attention_prefill_tc: pages of %d tokens, not %d", tokens_per_page, TK);
    if (n_kv_heads < 1 || n_heads % n_kv_heads || n_heads > 65535) ABK_REFUSE("attention_prefill_tc: %d heads, %d kv heads", n_heads, n_kv_heads);
    if ((uintptr_t)out % 16 || (n_heads * HD * 2) % 16) ABK_REFUSE("attention_prefill_tc: the output must be 16-byte aligned");
    CUtensorMap qm, km, vm;
    int rc = tmap::bf16_rows_of_128_bytes(qkv, n_rows, row_width, row_width, TQ, &qm);
    if (!rc) rc = tmap::bf16_rows_of_128_bytes(k_pool, pool_rows, HD, HD, TK, &km);
    if (!rc) rc = tmap::bf16_rows_of_128_bytes(v_pool, pool_rows, HD, HD, TK, &vm);
    if (rc) return rc;
    AttnTc p;
    p.out = (__nv_bfloat16 *)out, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads;
    p.scale_log2 = scale * 1.4426950408889634f, p.work = (const int4 *)work, p.status = status;
    p.partial_o = scratch, p.partial_ml = scratch + (long long)max_halved * n_heads * (TQ * HD), p.tickets = tickets;
    p.cache.page_table = page_table, p.cache.table_width = table_width, p.cache.ring_pages = 0;
    p.cache.tokens_per_page = tokens_per_page;
    const int smem = Q_BYTES + 2 * KV_STAGES * KV_BYTES + P_BYTES + 1024;  // 113 KB: two CTAs to an SM, to the byte
    if (cudaError_t e = abk_allow_shared_memory((const void *)attn_prefill_tc_kernel, smem)) return (int)e;  // once per device
    abk_launch(attn_prefill_tc_kernel, dim3((unsigned)(n_work * n_heads)), dim3(FA_THREADS), smem, (cudaStream_t)stream, qm, km,
               vm, p);
    return ABK_LAUNCH_RESULT();
}
