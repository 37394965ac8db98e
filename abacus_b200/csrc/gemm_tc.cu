// out[M, N] = x[M, K] . w[N, K]^T in bfloat16 on the 5th-generation tensor cores (tcgen05),
// float32 accumulation in tensor memory, operands brought in by TMA.
//
// One CTA computes a tile D[128, BN] = P_tile . Q_tile^T over a range of K:
//   warp 0      one thread issues TMA loads of [128 x 64] of P and [BN x 64] of Q into a ring of
//               shared-memory stages (128-byte swizzle), signalling a "full" mbarrier per stage;
//   warp 1      allocates BN tensor-memory columns; one thread issues four tcgen05.mma
//               (128 x BN x 16) per stage and commits to the stage's "empty" mbarrier, and at the
//               end to the "accumulator ready" mbarrier;
//   warps 2-5   read the accumulator with tcgen05.ld (each warp its own 32 lanes) and store it.
// P and Q are the two matrices in either order: with many rows of x (prefill) P = x, so lanes are
// tokens; with few rows (decode) P = w, so the 128 lanes are output features, the tokens are the
// BN columns (16..64) and no tensor-core work is spent on padding. The weights stream through
// once either way.
//
// Split K: grid.z CTAs share a tile, each over its own K range. Up to 8 of them (and column tiles up to
// 128) are a thread-block cluster: each leaves its float32 partial tile in its own shared memory, where
// the operands were, and after a cluster barrier adds up a share of the columns over all partial tiles,
// in split order, reading the others' through distributed shared memory. Otherwise each writes its
// partial tile to scratch memory and takes a ticket, and the last one adds the partials in split order
// (so the result does not depend on which CTA came last) and stores the tile.
//
// Many rows and many tiles (a prompt): the persistent kernel below. One CTA to an SM walks over the
// tiles; tensor memory holds two accumulators, so the four epilogue warps store tile i while the
// tensor cores are on tile i + 1, and the ring of stages never drains between tiles.
//
// K may be any multiple of 8 (a TMA row pitch must be a multiple of 16 bytes); rows beyond M or
// N and columns beyond K are zero-filled by TMA. Other shapes are refused, not approximated.
// Formula: src/model.c:299, 302, 307, 309, 324.
#define ABK_DEFINE_ERROR
#include "common.cuh"
#include "tc_common.cuh"
#include <mutex>
#include <unordered_map>

#include "qkv_prep.cuh"

#define TILE_P 128
#define TILE_K 64
#define GEMM_THREADS 192

struct GemmTc {
    void *out;
    long long stride_p, stride_q;  // out element (p, q) is out[p * stride_p + q * stride_q]
    int P, Q, K;
    int k_blocks, k_blocks_per_split, splits;
    float *partials;  // [splits, tiles, BN, 128] when splits > 1
    int *tickets;     // [tiles], zero before and after the launch
    int *status;
    int vec;  // stride_q == 1 and every 16-column run of a row starts on a 16-byte boundary
    int in_cluster;  // the splits of a tile are a thread-block cluster and add up through distributed shared memory
    int weights_are_p;  // which operand is nobody's output (the weights): its first stages are asked for before pdl_wait()
};

template <int BN, int STAGES> struct GemmSmem {
    static constexpr int A_BYTES = TILE_P * TILE_K * 2, B_BYTES = BN * TILE_K * 2;
    static constexpr int BYTES = STAGES * (A_BYTES + B_BYTES) + 1024 /* alignment */ + 256 /* barriers */;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t *)&t;
}
// 16 consecutive results of one row, stored as 16-byte vectors.
__device__ __forceinline__ void store16(float *dst, const uint32_t *v) {
#pragma unroll
    for (int j = 0; j < 16; j += 4) *(uint4 *)(dst + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
}
__device__ __forceinline__ void store16(__nv_bfloat16 *dst, const uint32_t *v) {
    uint32_t h[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
        h[j] = *(uint32_t *)&t;
    }
    *(uint4 *)dst = make_uint4(h[0], h[1], h[2], h[3]);
    *(uint4 *)(dst + 8) = make_uint4(h[4], h[5], h[6], h[7]);
}

template <int BN, int STAGES, typename TO>
__global__ void __launch_bounds__(GEMM_THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_p,
                                                               const __grid_constant__ CUtensorMap map_q, GemmTc g) {
    using S = GemmSmem<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *a_tiles = smem, *b_tiles = smem + STAGES * S::A_BYTES;
    uint64_t *full = (uint64_t *)(smem + STAGES * (S::A_BYTES + S::B_BYTES));
    uint64_t *empty = full + STAGES, *acc_ready = empty + STAGES;
    uint32_t *tmem_holder = (uint32_t *)(acc_ready + 1);
    volatile int *flags = (volatile int *)(tmem_holder + 1);  // [0]: a wait ran out; [1]: ticket

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p0 = blockIdx.x * TILE_P, q0 = blockIdx.y * BN, split = blockIdx.z;
    const int kb_begin = split * g.k_blocks_per_split;
    const int kb_end = min(g.k_blocks, kb_begin + g.k_blocks_per_split);
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) tc::mbar_init(&full[s], 1), tc::mbar_init(&empty[s], 1);
        tc::mbar_init(acc_ready, 1);
        flags[0] = 0, flags[1] = 0;
        tc::mbar_init_fence();
        tc::tma_prefetch_map(&map_p), tc::tma_prefetch_map(&map_q);
    }
    if (warp == 1) tc::tmem_alloc(tmem_holder, TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = *tmem_holder;
    // barriers, tensor memory and the tensor maps are ready. The weights' first stages are asked for at once; what
    // the kernel before this one writes (the other operand) only after pdl_wait().
    if (warp == 0) {
        if (lane == 0) {
            const int ahead = min(STAGES, kb_end - kb_begin);
            for (int i = 0; i < ahead; i++) {
                tc::mbar_expect_tx(&full[i], S::A_BYTES + S::B_BYTES);
                if (g.weights_are_p) tc::tma_load_2d(a_tiles + i * S::A_BYTES, &map_p, (kb_begin + i) * TILE_K, p0, &full[i]);
                else tc::tma_load_2d(b_tiles + i * S::B_BYTES, &map_q, (kb_begin + i) * TILE_K, q0, &full[i]);
            }
            pdl_wait();
            int issued = 0;
            for (int kb = kb_begin; kb < kb_end; kb++, issued++) {
                int s = issued % STAGES;
                if (issued >= ahead) {
                    if (!tc::mbar_wait(&empty[s], ((issued / STAGES) & 1) ^ 1)) {
                        flags[0] = 1;
                        break;
                    }
                    tc::mbar_expect_tx(&full[s], S::A_BYTES + S::B_BYTES);
                }
                if (issued >= ahead || !g.weights_are_p) tc::tma_load_2d(a_tiles + s * S::A_BYTES, &map_p, kb * TILE_K, p0, &full[s]);
                if (issued >= ahead || g.weights_are_p) tc::tma_load_2d(b_tiles + s * S::B_BYTES, &map_q, kb * TILE_K, q0, &full[s]);
            }
            if (flags[0]) {  // let the copies still in flight land before the CTA's memory goes away
                for (int i = max(0, issued - STAGES); i < issued; i++) tc::mbar_wait(&full[i % STAGES], (i / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::idesc_bf16_f32(TILE_P, BN);
            int done = 0;
            for (int kb = kb_begin; kb < kb_end; kb++, done++) {
                int s = done % STAGES;
                if (!tc::mbar_wait(&full[s], (done / STAGES) & 1)) {
                    flags[0] = 1;
                    break;
                }
                tc::fence_after_sync();
                uint32_t a = tc::smem_addr(a_tiles + s * S::A_BYTES), b = tc::smem_addr(b_tiles + s * S::B_BYTES);
#pragma unroll
                for (int k = 0; k < TILE_K / 16; k++)
                    tc::mma_ss(tmem, tc::smem_desc_k_sw128(a + k * 32), tc::smem_desc_k_sw128(b + k * 32), idesc,
                               done > 0 || k > 0);
                tc::mma_commit(&empty[s]);
            }
            tc::mma_commit(acc_ready);
        }
    } else {
        // epilogue: warp w reads lanes 32 * (w % 4) .. + 31 of the accumulator
        const int quarter = warp & 3, row = quarter * 32 + lane, p = p0 + row;
        bool ok = tc::mbar_wait(acc_ready, 0);
        if (!ok) flags[0] = 1;
        tc::fence_after_sync();
        const int tiles = gridDim.x * gridDim.y, tile = blockIdx.y * gridDim.x + blockIdx.x;
        const bool direct = g.splits == 1;
        float *mine = direct || g.in_cluster ? nullptr : g.partials + ((long long)split * tiles + tile) * (BN * TILE_P);
        TO *out = (TO *)g.out;
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t v[16];
                tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + c0, v);
                tc::tmem_ld_wait();
                if (g.in_cluster) {  // the operands' stages are free: every product has read them
                    float *at = (float *)smem + row * (BN + 4) + c0;
#pragma unroll
                    for (int j = 0; j < 16; j += 4) *(uint4 *)(at + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                } else if (direct && g.vec && p < g.P && q0 + c0 + 16 <= g.Q) {
                    store16(out + (long long)p * g.stride_p + q0 + c0, v);
                } else if (direct) {
                    if (p < g.P) {
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (q0 + c0 + j < g.Q)
                                out[(long long)p * g.stride_p + (long long)(q0 + c0 + j) * g.stride_q] =
                                    from_float<TO>(__uint_as_float(v[j]));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) mine[(c0 + j) * TILE_P + row] = __uint_as_float(v[j]);
                }
            }
        }
        if (!direct && !g.in_cluster) {
            // the last CTA of this tile to get here adds up all partials, in split order
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) flags[1] = atomicAdd(&g.tickets[tile], 1);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (flags[1] == g.splits - 1) {
                __threadfence();
                if (p < g.P) {
                    const float *part = g.partials + (long long)tile * (BN * TILE_P) + row;
                    const long long split_stride = (long long)tiles * (BN * TILE_P);
                    const int cols = min(BN, g.Q - q0);
                    for (int c0 = 0; c0 < cols; c0 += 8) {
                        // eight columns at a time: all loads of a split are in flight together, and the
                        // splits are added in order, so the sum does not depend on who came last
                        float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                        for (int s0 = 0; s0 < g.splits; s0 += 4) {
                            float v[4][8];
#pragma unroll
                            for (int i = 0; i < 4; i++)
#pragma unroll
                                for (int j = 0; j < 8; j++)
                                    v[i][j] = (s0 + i < g.splits && c0 + j < cols)
                                                  ? __ldcg(part + (s0 + i) * split_stride + (c0 + j) * TILE_P)
                                                  : 0.0f;
#pragma unroll
                            for (int i = 0; i < 4; i++)
#pragma unroll
                                for (int j = 0; j < 8; j++) sum[j] += v[i][j];
                        }
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            if (c0 + j < cols)
                                out[(long long)p * g.stride_p + (long long)(q0 + c0 + j) * g.stride_q] =
                                    from_float<TO>(sum[j]);
                    }
                }
                if (threadIdx.x == 64) g.tickets[tile] = 0;
            }
        }
    }
    if (g.in_cluster) {
        // every CTA of the tile adds up its share of the columns (groups of four) over all partial tiles, in split order
        tc::cluster_sync();
        if (warp >= 2) {
            const int quarter = warp & 3, row = quarter * 32 + lane, p = p0 + row;
            const int groups = BN / 4, per = (groups + g.splits - 1) / g.splits;
            const uint32_t base = tc::smem_addr((float *)smem + row * (BN + 4));
            TO *out = (TO *)g.out;
            for (int gi = split * per; gi < min(groups, (split + 1) * per); gi++) {
                // all splits' loads are in flight before the first sum (a warp issues in order: a sum right behind
                // its load would wait out every round trip through the cluster one after the other)
                float4 t[8];
#pragma unroll
                for (int s0 = 0; s0 < 8; s0++)
                    t[s0] = s0 < g.splits ? tc::ld_cluster_f4(tc::peer_smem(base + gi * 16, s0)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                float4 sum = t[0];
#pragma unroll
                for (int s0 = 1; s0 < 8; s0++) sum.x += t[s0].x, sum.y += t[s0].y, sum.z += t[s0].z, sum.w += t[s0].w;
                const float r4[4] = {sum.x, sum.y, sum.z, sum.w};
                if (p < g.P) {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        if (q0 + gi * 4 + j < g.Q)
                            out[(long long)p * g.stride_p + (long long)(q0 + gi * 4 + j) * g.stride_q] = from_float<TO>(r4[j]);
                }
            }
        }
        tc::cluster_sync();  // nobody leaves while its partial tile may still be read
    }
    tc::fence_before_sync();
    __syncthreads();
    if (flags[0] && threadIdx.x == 0) atomicOr(g.status + 1, 1);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_free(tmem, TMEM_COLS);
    }
}

// ------------------------------------------------------------------ what may follow a product in its kernel
#define EPI_PLAIN 0
#define EPI_GATED 1  // silu(gate) * up of a tile that holds both (see the persistent kernel)
#define EPI_QKV 2    // the q/k/v product of a prompt with the step between it and attention taken in
// EPI_QKV (column tiles of 256 = two heads of 128, bfloat16 out): the rows are tokens, the columns q heads, then k
// heads, then v heads, and a thread that stores a row holds whole heads of it. It does what the preparation kernel
// does to them (src/model.c:247-259; qkv_prep.cuh, to the same bits): q and k normed over the head and rotated, q
// stored to out, k and v of a token that belongs to a sequence to their place in the paged cache and nowhere else.
struct QkvEpilogue {
    const int *token_seq, *token_pos, *seq_slot;
    const float *q_norm, *k_norm;  // [128]; null: no norm
    const float *cos, *sin;        // [positions, 64]; null: no rotation
    float eps;
    __nv_bfloat16 *k_pool, *v_pool;
    PagedCache cache;
    int n_heads, n_kv_heads;
};
// A kernel with this epilogue has eight storing warps, two to each quarter of the tile's rows (a warp reaches only its
// quarter of the lanes of tensor memory): warp `part` of a quarter takes the pairs (i, i + 64) of a head with i in
// [32 part, 32 part + 32), that is 64 of a row's 128 values, and reads all 128 only to add up their squares. A single warp
// to a scheduler cannot hide the latency of its own instructions; two, each with half of the work, take a third of the time.
// A row's angles (64 cos, 64 sin) lie 256 bytes from the next row's. A warp asks for its 32 of each for its 32 rows as soon
// as it knows the tile, before it waits for the accumulator: asynchronous copies that cover whole lines, into its own
// QKV_ANGLE_FLOATS floats of shared memory (cos of the 32 rows, then sin), from where every thread later reads its row's.
#define QKV_THREADS 320  // one warp that loads, one that multiplies, eight that store
#define QKV_ANGLE_FLOATS (2 * 32 * 32)
// Where the four angles from `c` on (a multiple of 4 below 32) of row `row` lie among a table's 32 rows of 32: the 16-byte
// pieces of a row are exchanged by the row's last three bits, so that reads of the same piece of 8 rows fall into different banks.
__device__ __forceinline__ int qkv_angle_at(int row, int c) { return row * 32 + ((((c >> 2) ^ (row & 7)) << 2)); }
// What a thread knows of its row before the accumulator is there: the token's sequence (-1: none) and position, and where its
// keys and values go in the pools (kv head 0; -1: nowhere). Looked up, like the angles, while the tile is still being multiplied.
struct QkvRow {
    int seq, pos;
    long long kept_at;
};
__device__ __forceinline__ QkvRow fetch_qkv_angles(int p, int part, const GemmTc &g, const QkvEpilogue &e, float *angles) {
    const int lane = threadIdx.x & 31;
    QkvRow r;
    r.seq = p < g.P ? e.token_seq[p] : -1;
    r.pos = p < g.P ? e.token_pos[p] : 0;  // (asked for with the sequence, not after it)
    if (r.seq < 0) r.pos = 0;
    r.kept_at = -1;
    if (r.seq >= 0 && e.k_pool) r.kept_at = cache_offset(e.cache, cache_page(e.cache, e.seq_slot[r.seq], r.pos), 0, e.n_kv_heads, r.pos, 128);
    if (!e.cos) return r;
    const int pos = r.pos;
#pragma unroll
    for (int j = 0; j < 8; j++) {  // lane l copies the 16-byte piece l % 8 of row l / 8 + 4 j
        const int row = (lane >> 3) + 4 * j, c = 4 * (lane & 7);
        const long long at = (long long)__shfl_sync(0xffffffffu, pos, row) * 64 + 32 * part + c;
        const uint32_t to_cos = tc::smem_addr(angles + qkv_angle_at(row, c)), to_sin = tc::smem_addr(angles + 32 * 32 + qkv_angle_at(row, c));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to_cos), "l"(e.cos + at) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to_sin), "l"(e.sin + at) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    return r;
}
// One row p of a tile whose first column is q0: the accumulator's 256 columns start at tensor-memory address `acc` (this
// warp's lanes). Whole warps call it, after fetch_qkv_angles() for the same rows and part.
template <int PART>
__device__ __forceinline__ void store_qkv_row(uint32_t acc, int p, int q0, const GemmTc &g, const QkvEpilogue &e, const float *angles,
                                              const QkvRow &r) {
    const int lane = threadIdx.x & 31;
    if (e.cos) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
    }
#pragma unroll 1
    for (int h = 0; h < 2; h++) {
        const int head = q0 / 128 + h;
        if (head * 128 >= g.Q) break;
        float mine[64], part[16];  // elements 32 PART .. + 31 and 64 + 32 PART .. + 31 of the head; every eight's sum of squares
#pragma unroll
        for (int c = 0; c < 4; c++) {  // 32 columns at a time
            float t[32];
            tc::tmem_ld16(acc + h * 128 + 32 * c, (uint32_t *)t);
            tc::tmem_ld16(acc + h * 128 + 32 * c + 16, (uint32_t *)t + 16);
            tc::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) t[i] = prep_through_bf16(t[i]);
#pragma unroll
            for (int l = 0; l < 4; l++) part[4 * c + l] = prep_sumsq8(t + 8 * l);
            if (c == PART || c == 2 + PART) {
#pragma unroll
                for (int i = 0; i < 32; i++) mine[(c == PART ? 0 : 32) + i] = t[i];
            }
        }
        const bool is_q = head < e.n_heads, is_k = !is_q && head < e.n_heads + e.n_kv_heads;
        const float *w = is_q ? e.q_norm : e.k_norm;
        if ((is_q || is_k) && w) {
            const float scale = prep_scale<128>(prep_fold<128>(part), e.eps);
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const float4 lo = __ldg((const float4 *)(w + 32 * PART + i)), hi = __ldg((const float4 *)(w + 64 + 32 * PART + i));
                mine[i] = prep_normed(lo.x, mine[i], scale), mine[i + 1] = prep_normed(lo.y, mine[i + 1], scale);
                mine[i + 2] = prep_normed(lo.z, mine[i + 2], scale), mine[i + 3] = prep_normed(lo.w, mine[i + 3], scale);
                mine[32 + i] = prep_normed(hi.x, mine[32 + i], scale), mine[33 + i] = prep_normed(hi.y, mine[33 + i], scale);
                mine[34 + i] = prep_normed(hi.z, mine[34 + i], scale), mine[35 + i] = prep_normed(hi.w, mine[35 + i], scale);
            }
        }
        if ((is_q || is_k) && e.cos) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const float4 c4 = *(const float4 *)(angles + qkv_angle_at(lane, i)), s4 = *(const float4 *)(angles + 32 * 32 + qkv_angle_at(lane, i));
                const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float lo = mine[i + k], hi = mine[32 + i + k];
                    mine[i + k] = prep_rotated_lower(lo, hi, cs[k], sn[k]);
                    mine[32 + i + k] = prep_rotated_upper(hi, lo, cs[k], sn[k]);
                }
            }
        }
        __nv_bfloat16 *dst = nullptr;
        if (is_q) {
            if (p < g.P) dst = (__nv_bfloat16 *)g.out + (long long)p * g.stride_p + head * 128;
        } else if (r.kept_at >= 0) {
            const int kv_head = is_k ? head - e.n_heads : head - e.n_heads - e.n_kv_heads;
            dst = (is_k ? e.k_pool : e.v_pool) + r.kept_at + (long long)kv_head * e.cache.tokens_per_page * 128;
        }
        if (dst) {
#pragma unroll
            for (int half = 0; half < 2; half++)
#pragma unroll
                for (int i = 0; i < 32; i += 8)
                    *(uint4 *)(dst + 64 * half + 32 * PART + i) =
                        make_uint4(pack2(mine[32 * half + i], mine[32 * half + i + 1]), pack2(mine[32 * half + i + 2], mine[32 * half + i + 3]),
                                   pack2(mine[32 * half + i + 4], mine[32 * half + i + 5]), pack2(mine[32 * half + i + 6], mine[32 * half + i + 7]));
        }
    }
    __syncwarp();  // every lane has read its angles before the next tile's are asked for
}

// ------------------------------------------------------------------ persistent kernel for many tiles
// Tile t is rows (t % m_tiles) * 128 and columns (t / m_tiles) * BN; CTA c takes tiles c, c + grid, ...
// Warp 0 loads, warp 1 issues the products into accumulator (i & 1) of its i-th tile, warps 2-5 store
// the accumulator of the tile before. acc_full / acc_empty hand the two accumulators back and forth.
// GATED (BN 256, bfloat16 out): the columns of a tile are the gates of 128 features and then their ups (the
// weight's rows come in such turns of 128), and what is stored is out[p, 128 t + j] = silu(gate) * up, both
// rounded to bfloat16 first, as they are where they are stored between the product and the activation: the
// feed-forward's first product and its activation in one (src/model.c:274-282, 307-308). g.Q is then the
// number of features, half of the product's columns.
template <int BN, int STAGES, typename TO, int EPI = EPI_PLAIN>
__global__ void __launch_bounds__(EPI == EPI_QKV ? QKV_THREADS : GEMM_THREADS) gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_p,
                                                                          const __grid_constant__ CUtensorMap map_q,
                                                                          GemmTc g, int m_tiles, int tiles, QkvEpilogue qkv) {
    constexpr bool GATED = EPI == EPI_GATED;
    using S = GemmSmem<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *a_tiles = smem, *b_tiles = smem + STAGES * S::A_BYTES;
    uint64_t *full = (uint64_t *)(smem + STAGES * (S::A_BYTES + S::B_BYTES));
    uint64_t *empty = full + STAGES, *acc_full = empty + STAGES, *acc_empty = acc_full + 2;
    uint32_t *tmem_holder = (uint32_t *)(acc_empty + 2);
    volatile int *flags = (volatile int *)(tmem_holder + 1);  // [0]: a wait ran out
    float *qkv_angles = (float *)(smem + STAGES * (S::A_BYTES + S::B_BYTES) + 256);  // (EPI_QKV: see store_qkv_row)
    constexpr uint32_t TMEM_COLS = 2 * BN;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) tc::mbar_init(&full[s], 1), tc::mbar_init(&empty[s], 1);
        for (int b = 0; b < 2; b++) tc::mbar_init(&acc_full[b], 1), tc::mbar_init(&acc_empty[b], EPI == EPI_QKV ? 8 : 4)  /* every storing warp */;
        flags[0] = 0;
        tc::mbar_init_fence();
        tc::tma_prefetch_map(&map_p), tc::tma_prefetch_map(&map_q);
    }
    if (warp == 1) tc::tmem_alloc(tmem_holder, TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            // the weights (the columns' operand) of the first tile's first stages are asked for before pdl_wait():
            // nobody writes them; the rows' operand comes from the kernel before
            const int ahead = min(STAGES, g.k_blocks);
            for (int i = 0; i < ahead; i++) {
                tc::mbar_expect_tx(&full[i], S::A_BYTES + S::B_BYTES);
                tc::tma_load_2d(b_tiles + i * S::B_BYTES, &map_q, i * TILE_K, ((int)blockIdx.x / m_tiles) * BN, &full[i]);
            }
            pdl_wait();
            int issued = 0;
            for (int t = blockIdx.x; t < tiles && !flags[0]; t += gridDim.x) {
                const int p0 = (t % m_tiles) * TILE_P, q0 = (t / m_tiles) * BN;
                for (int kb = 0; kb < g.k_blocks; kb++, issued++) {
                    int s = issued % STAGES;
                    if (issued >= ahead) {
                        if (!tc::mbar_wait(&empty[s], ((issued / STAGES) & 1) ^ 1)) {
                            flags[0] = 1;
                            break;
                        }
                        tc::mbar_expect_tx(&full[s], S::A_BYTES + S::B_BYTES);
                        tc::tma_load_2d(b_tiles + s * S::B_BYTES, &map_q, kb * TILE_K, q0, &full[s]);
                    }
                    tc::tma_load_2d(a_tiles + s * S::A_BYTES, &map_p, kb * TILE_K, p0, &full[s]);
                }
            }
            if (flags[0]) {  // let the copies still in flight land before the CTA's memory goes away
                for (int i = max(0, issued - STAGES); i < issued; i++) tc::mbar_wait(&full[i % STAGES], (i / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::idesc_bf16_f32(TILE_P, BN);
            int done = 0, it = 0;
            for (int t = blockIdx.x; t < tiles && !flags[0]; t += gridDim.x, it++) {
                const int b = it & 1;
                if (!tc::mbar_wait(&acc_empty[b], ((it >> 1) & 1) ^ 1)) {  // the epilogue is done with this accumulator
                    flags[0] = 1;
                    break;
                }
                tc::fence_after_sync();
                for (int kb = 0; kb < g.k_blocks; kb++, done++) {
                    int s = done % STAGES;
                    if (!tc::mbar_wait(&full[s], (done / STAGES) & 1)) {
                        flags[0] = 1;
                        break;
                    }
                    tc::fence_after_sync();
                    uint32_t a = tc::smem_addr(a_tiles + s * S::A_BYTES), bq = tc::smem_addr(b_tiles + s * S::B_BYTES);
#pragma unroll
                    for (int k = 0; k < TILE_K / 16; k++)
                        tc::mma_ss(tmem + b * BN, tc::smem_desc_k_sw128(a + k * 32), tc::smem_desc_k_sw128(bq + k * 32), idesc,
                                   kb > 0 || k > 0);
                    tc::mma_commit(&empty[s]);
                }
                if (flags[0]) break;
                tc::mma_commit(&acc_full[b]);
            }
        }
    } else {
        const int quarter = warp & 3, row = quarter * 32 + lane;
        TO *out = (TO *)g.out;
        int it = 0;
        pdl_wait();  // (what they store comes after the loads that wait anyway; this keeps the rule simple)
        for (int t = blockIdx.x; t < tiles; t += gridDim.x, it++) {
            const int b = it & 1;
            const int p = (t % m_tiles) * TILE_P + row, q0 = (t / m_tiles) * BN;
            QkvRow qkv_row = {-1, 0, -1};
            if constexpr (EPI == EPI_QKV) qkv_row = fetch_qkv_angles(p, (warp - 2) >> 2, g, qkv, qkv_angles + (warp - 2) * QKV_ANGLE_FLOATS);
            // every lane takes the same way out: the loads from tensor memory below are for whole warps
            const bool ok = __all_sync(0xffffffffu, !flags[0] && tc::mbar_wait(&acc_full[b], (it >> 1) & 1));
            if (!ok) {
                flags[0] = 1;
                break;
            }
            tc::fence_after_sync();
            if constexpr (GATED) {
                const int f0 = (t / m_tiles) * (BN / 2);  // the tile's first feature
#pragma unroll 1
                for (int c0 = 0; c0 < BN / 2; c0 += 32) {
                    uint32_t gv[32], uv[32];
                    tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + c0, gv);
                    tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + c0 + 16, gv + 16);
                    tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + BN / 2 + c0, uv);
                    tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + BN / 2 + c0 + 16, uv + 16);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float gate = __bfloat162float(__float2bfloat16_rn(__uint_as_float(gv[j])));
                        const float up = __bfloat162float(__float2bfloat16_rn(__uint_as_float(uv[j])));
                        gv[j] = __float_as_uint(silu_mul_fast(gate, up));
                    }
                    if (p < g.P && f0 + c0 + 32 <= g.Q) {
                        store16(out + (long long)p * g.stride_p + f0 + c0, gv);
                        store16(out + (long long)p * g.stride_p + f0 + c0 + 16, gv + 16);
                    }
                }
            } else if constexpr (EPI == EPI_QKV) {
                if ((warp - 2) >> 2) store_qkv_row<1>(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN, p, q0, g, qkv, qkv_angles + (warp - 2) * QKV_ANGLE_FLOATS, qkv_row);
                else store_qkv_row<0>(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN, p, q0, g, qkv, qkv_angles + (warp - 2) * QKV_ANGLE_FLOATS, qkv_row);
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t v[32];
                    tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + c0, v);
                    tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + c0 + 16, v + 16);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int h = 0; h < 32; h += 16) {
                        if (g.vec && p < g.P && q0 + c0 + h + 16 <= g.Q) {
                            store16(out + (long long)p * g.stride_p + q0 + c0 + h, v + h);
                        } else if (p < g.P) {
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (q0 + c0 + h + j < g.Q)
                                    out[(long long)p * g.stride_p + (long long)(q0 + c0 + h + j) * g.stride_q] =
                                        from_float<TO>(__uint_as_float(v[h + j]));
                        }
                    }
                }
            }
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&acc_empty[b]);
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (flags[0] && threadIdx.x == 0) atomicOr(g.status + 1, 1);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_free(tmem, TMEM_COLS);
    }
}

// ------------------------------------------------------------------ pairs of CTAs on tiles of 256 rows
// The persistent kernel above is bound by the operands' way from the L2 into shared memory: a CTA brings 128 rows of x
// and BN rows of w for every block of K. Here two CTAs of a cluster (the two SMs of a pair) work on one tile of 256 rows:
// each brings its 128 rows of x and only half of the tile's rows of w, and one tcgen05.mma.cta_group::2 of the even CTA
// multiplies what both hold, each CTA's tensor memory getting its 128 rows of the result. Per FLOP a CTA loads
// (128 + BN / 2) / (128 + BN) of what it loaded alone: two thirds at BN = 256. Every load is the CTA's own plain TMA copy
// into its own shared memory; there is no multicast. Roles as above (warp 0 loads, warp 1 of the leader multiplies, warps
// 2-5 of both store); the leader's `full` barriers count the bytes of both CTAs, its commits reach both CTAs' `empty` and
// `acc_full` barriers, and the peer's storing warps report to the leader's `acc_empty`.
// ABACUS_GEMM_PAIRS=0 keeps every product on single CTAs (for comparison).
static bool abk_pairs_off() {
    static int off = -1;
    if (off < 0) {
        const char *e = getenv("ABACUS_GEMM_PAIRS");
        off = e && e[0] == '0';
    }
    return off != 0;
}

template <int BN, int STAGES> struct PairSmem {
    static constexpr int A_BYTES = TILE_P * TILE_K * 2, B_BYTES = (BN / 2) * TILE_K * 2;
    static constexpr int BYTES = STAGES * (A_BYTES + B_BYTES) + 1024 /* alignment */ + 256 /* barriers */;
};

template <int BN, int STAGES, typename TO, int EPI = EPI_PLAIN>
__global__ void __launch_bounds__(EPI == EPI_QKV ? QKV_THREADS : GEMM_THREADS) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_p,
                                                                    const __grid_constant__ CUtensorMap map_q, GemmTc g,
                                                                    int m_tiles, int tiles, QkvEpilogue qkv) {
    constexpr bool GATED = EPI == EPI_GATED;
    using S = PairSmem<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *a_tiles = smem, *b_tiles = smem + STAGES * S::A_BYTES;
    uint64_t *full = (uint64_t *)(smem + STAGES * (S::A_BYTES + S::B_BYTES));
    uint64_t *empty = full + STAGES, *acc_full = empty + STAGES, *acc_empty = acc_full + 2;
    uint32_t *tmem_holder = (uint32_t *)(acc_empty + 2);
    volatile int *flags = (volatile int *)(tmem_holder + 1);  // [0]: a wait ran out
    float *qkv_angles = (float *)(smem + STAGES * (S::A_BYTES + S::B_BYTES) + 256);  // (EPI_QKV: see store_qkv_row)
    constexpr uint32_t TMEM_COLS = 2 * BN;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)tc::cluster_rank();  // 0: the leader, 1: its peer
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) tc::mbar_init(&full[s], 1), tc::mbar_init(&empty[s], 1);
        for (int b = 0; b < 2; b++) tc::mbar_init(&acc_full[b], 1), tc::mbar_init(&acc_empty[b], EPI == EPI_QKV ? 16 : 8);  // every storing warp of both CTAs
        flags[0] = 0;
        tc::mbar_init_fence();
        tc::tma_prefetch_map(&map_p), tc::tma_prefetch_map(&map_q);
    }
    if (warp == 1) tc::tmem_alloc_pair(tmem_holder, TMEM_COLS);
    tc::fence_before_sync();
    tc::cluster_sync();  // both CTAs' barriers are there before either signals the other's
    tc::fence_after_sync();
    const uint32_t tmem = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            // A stage is full when both CTAs' copies have landed: all of them report to the leader's barrier.
            constexpr uint32_t STAGE_BYTES = 2 * (S::A_BYTES + S::B_BYTES);
            const int ahead = min(STAGES, g.k_blocks);
            // the weights of the first tile's first stages are asked for before pdl_wait(): nobody writes them
            for (int i = 0; i < ahead; i++) {
                if (rank == 0) tc::mbar_expect_tx(&full[i], STAGE_BYTES);
                tc::tma_load_2d_pair(b_tiles + i * S::B_BYTES, &map_q, i * TILE_K, (pair / m_tiles) * BN + rank * (BN / 2),
                                     tc::peer_smem(tc::smem_addr(&full[i]), 0));
            }
            pdl_wait();
            int issued = 0;
            for (int t = pair; t < tiles && !flags[0]; t += pairs) {
                const int p0 = (t % m_tiles) * (2 * TILE_P) + rank * TILE_P, q0 = (t / m_tiles) * BN + rank * (BN / 2);
                for (int kb = 0; kb < g.k_blocks; kb++, issued++) {
                    const int s = issued % STAGES;
                    const uint32_t bar = tc::peer_smem(tc::smem_addr(&full[s]), 0);
                    if (issued >= ahead) {
                        if (!tc::mbar_wait(&empty[s], ((issued / STAGES) & 1) ^ 1)) {  // (its own: the commit reaches both)
                            flags[0] = 1;
                            break;
                        }
                        if (rank == 0) tc::mbar_expect_tx(&full[s], STAGE_BYTES);
                        tc::tma_load_2d_pair(b_tiles + s * S::B_BYTES, &map_q, kb * TILE_K, q0, bar);
                    }
                    tc::tma_load_2d_pair(a_tiles + s * S::A_BYTES, &map_p, kb * TILE_K, p0, bar);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = tc::idesc_bf16_f32(2 * TILE_P, BN);
            int done = 0, it = 0;
            for (int t = pair; t < tiles && !flags[0]; t += pairs, it++) {
                const int b = it & 1;
                if (!tc::mbar_wait(&acc_empty[b], ((it >> 1) & 1) ^ 1)) {  // both CTAs are done with this accumulator
                    flags[0] = 1;
                    break;
                }
                tc::fence_after_sync();
                for (int kb = 0; kb < g.k_blocks; kb++, done++) {
                    const int s = done % STAGES;
                    if (!tc::mbar_wait(&full[s], (done / STAGES) & 1)) {
                        flags[0] = 1;
                        break;
                    }
                    tc::fence_after_sync();
                    const uint32_t a = tc::smem_addr(a_tiles + s * S::A_BYTES), bq = tc::smem_addr(b_tiles + s * S::B_BYTES);
#pragma unroll
                    for (int k = 0; k < TILE_K / 16; k++)
                        tc::mma_ss_pair(tmem + b * BN, tc::smem_desc_k_sw128(a + k * 32), tc::smem_desc_k_sw128(bq + k * 32),
                                        idesc, kb > 0 || k > 0);
                    tc::mma_commit_pair(&empty[s]);
                }
                if (flags[0]) break;
                tc::mma_commit_pair(&acc_full[b]);
            }
        }
    } else {
        const int quarter = warp & 3, row = quarter * 32 + lane;
        TO *out = (TO *)g.out;
        int it = 0;
        pdl_wait();
        for (int t = pair; t < tiles; t += pairs, it++) {
            const int b = it & 1;
            const int p = (t % m_tiles) * (2 * TILE_P) + rank * TILE_P + row, q0 = (t / m_tiles) * BN;
            QkvRow qkv_row = {-1, 0, -1};
            if constexpr (EPI == EPI_QKV) qkv_row = fetch_qkv_angles(p, (warp - 2) >> 2, g, qkv, qkv_angles + (warp - 2) * QKV_ANGLE_FLOATS);
            const bool ok = __all_sync(0xffffffffu, !flags[0] && tc::mbar_wait(&acc_full[b], (it >> 1) & 1));
            if (!ok) {
                flags[0] = 1;
                break;
            }
            tc::fence_after_sync();
            if constexpr (GATED) {
                const int f0 = (t / m_tiles) * (BN / 2);  // the tile's first feature
#pragma unroll 1
                for (int c0 = 0; c0 < BN / 2; c0 += 32) {
                    uint32_t gv[32], uv[32];
                    tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + c0, gv);
                    tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + c0 + 16, gv + 16);
                    tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + BN / 2 + c0, uv);
                    tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + BN / 2 + c0 + 16, uv + 16);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float gate = __bfloat162float(__float2bfloat16_rn(__uint_as_float(gv[j])));
                        const float up = __bfloat162float(__float2bfloat16_rn(__uint_as_float(uv[j])));
                        gv[j] = __float_as_uint(silu_mul_fast(gate, up));
                    }
                    if (p < g.P && f0 + c0 + 32 <= g.Q) {
                        store16(out + (long long)p * g.stride_p + f0 + c0, gv);
                        store16(out + (long long)p * g.stride_p + f0 + c0 + 16, gv + 16);
                    }
                }
            } else if constexpr (EPI == EPI_QKV) {
                if ((warp - 2) >> 2) store_qkv_row<1>(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN, p, q0, g, qkv, qkv_angles + (warp - 2) * QKV_ANGLE_FLOATS, qkv_row);
                else store_qkv_row<0>(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN, p, q0, g, qkv, qkv_angles + (warp - 2) * QKV_ANGLE_FLOATS, qkv_row);
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t v[32];
                    tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + c0, v);
                    tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + c0 + 16, v + 16);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int h = 0; h < 32; h += 16) {
                        if (g.vec && p < g.P && q0 + c0 + h + 16 <= g.Q) {
                            store16(out + (long long)p * g.stride_p + q0 + c0 + h, v + h);
                        } else if (p < g.P) {
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (q0 + c0 + h + j < g.Q)
                                    out[(long long)p * g.stride_p + (long long)(q0 + c0 + h + j) * g.stride_q] =
                                        from_float<TO>(__uint_as_float(v[h + j]));
                        }
                    }
                }
            }
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive_in_cluster(tc::peer_smem(tc::smem_addr(&acc_empty[b]), 0));
        }
    }
    // Nobody leaves while the other CTA may still signal its barriers or write its tensor memory. (After a wait that ran
    // out, copies may still be on their way into this CTA's shared memory: give them a tenth of a millisecond.)
    if (flags[0]) {
        const uint64_t t0 = tc::global_ns();
        while (tc::global_ns() - t0 < 100000) __nanosleep(1000);
    }
    tc::fence_before_sync();
    tc::cluster_sync();
    if (flags[0] && threadIdx.x == 0) atomicOr(g.status + 1, 1);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_free_pair(tmem, TMEM_COLS);
    }
}

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    });
    return fn;
}

struct MapKey {
    const void *ptr;
    long long rows, cols, ld;
    int box_rows;
    bool operator==(const MapKey &o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey &k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.rows, h = h * 1000003u ^ (size_t)k.cols;
        return h * 1000003u ^ (size_t)k.ld ^ ((size_t)k.box_rows << 48);
    }
};

// A tensor map over a row-major bfloat16 matrix [rows, cols] with row pitch ld: boxes of
// [box_rows, 64] elements, 128-byte swizzle, zeros outside. Maps are kept by address and shape.
static int tensor_map(const void *ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap *out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex lock;
    MapKey key{ptr, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> guard(lock);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return 0;
    }
    EncodeTiled enc = encode_tiled();
    if (!enc) ABK_REFUSE("gemm_tc: the driver gives no cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TILE_K, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void *)ptr, dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) ABK_REFUSE("gemm_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return 0;
}

template <int BN, int STAGES, typename TO>
static int launch(const CUtensorMap &mp, const CUtensorMap &mq, const GemmTc &g, dim3 grid, cudaStream_t s) {
    auto kernel = gemm_tc_kernel<BN, STAGES, TO>;
    constexpr int bytes = GemmSmem<BN, STAGES>::BYTES;
    if (cudaError_t e = abk_allow_shared_memory((const void *)kernel, bytes)) return (int)e;  // once per device
    abk_launch_clusters(kernel, grid, dim3(GEMM_THREADS), (size_t)bytes, s, dim3(1, 1, g.in_cluster ? g.splits : 1), mp, mq, g);
    return ABK_LAUNCH_RESULT();
}

// The kernel for pairs of CTAs: m_tiles and tiles count tiles of 256 rows; one cluster of two CTAs per pair of SMs.
template <int BN, int STAGES, typename TO, int EPI = EPI_PLAIN>
static int launch_pair(const CUtensorMap &mp, const CUtensorMap &mq, const GemmTc &g, int m_tiles, int tiles, cudaStream_t s,
                       const QkvEpilogue &qkv = QkvEpilogue()) {
    auto kernel = gemm_tc_pair_kernel<BN, STAGES, TO, EPI>;
    constexpr int bytes = PairSmem<BN, STAGES>::BYTES + (EPI == EPI_QKV ? 8 * QKV_ANGLE_FLOATS * 4 : 0);
    constexpr int threads = EPI == EPI_QKV ? QKV_THREADS : GEMM_THREADS;
    if (cudaError_t e = abk_allow_shared_memory((const void *)kernel, bytes)) return (int)e;  // once per device
    const int pairs = abk_sm_count() / 2;
    abk_launch_clusters(kernel, dim3(2 * (tiles < pairs ? tiles : pairs)), dim3(threads), (size_t)bytes, s, 2, mp, mq, g,
                        m_tiles, tiles, qkv);
    return ABK_LAUNCH_RESULT();
}
// Whether a product of many rows goes to the pairs: enough tiles of 256 x 256 to give most pairs of SMs one.
static bool pairs_win(int M, int N) {
    const long long tiles = (long long)((M + 2 * TILE_P - 1) / (2 * TILE_P)) * ((N + 255) / 256);
    return M > 256 && N >= 256 && tiles >= (abk_sm_count() / 2) * 6 / 7;
}

template <int BN, int STAGES, typename TO, int EPI = EPI_PLAIN>
static int launch_persistent(const CUtensorMap &mp, const CUtensorMap &mq, const GemmTc &g, int m_tiles, int tiles,
                             cudaStream_t s, const QkvEpilogue &qkv = QkvEpilogue()) {
    auto kernel = gemm_tc_persistent_kernel<BN, STAGES, TO, EPI>;
    constexpr int bytes = GemmSmem<BN, STAGES>::BYTES + (EPI == EPI_QKV ? 8 * QKV_ANGLE_FLOATS * 4 : 0);
    constexpr int threads = EPI == EPI_QKV ? QKV_THREADS : GEMM_THREADS;
    if (cudaError_t e = abk_allow_shared_memory((const void *)kernel, bytes)) return (int)e;  // once per device
    abk_launch(kernel, dim3(tiles < abk_sm_count() ? tiles : abk_sm_count()), dim3(threads), (size_t)bytes, s, mp, mq, g, m_tiles, tiles,
               qkv);
    return ABK_LAUNCH_RESULT();
}

// act[M, N] = silu(x . gate^T) * (x . up^T), w [2 N, K] holding gate and up rows in turns of 128: the persistent
// kernel with the activation in its epilogue. Many rows only (more than 256), N a multiple of 128, act bfloat16
// with 16-byte aligned rows; other shapes are refused (the caller multiplies and activates in two steps).
extern "C" int abk_gemm_tc_swiglu(const void *x, const void *w, void *act, int M, int N, int K, long long ldx,
                                  long long ldw, long long ldo, int *status, void *stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M <= 256 || N % 128 || K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ldo % 8 || (((uintptr_t)x | (uintptr_t)w | (uintptr_t)act) & 15))
        ABK_REFUSE("gemm_tc_swiglu: %d rows, %d features, K = %d are not what the fused kernel takes", M, N, K);
    CUtensorMap mx, mw;
    int rc = tensor_map(x, M, K, ldx, TILE_P, &mx);
    if (!rc) rc = tensor_map(w, 2LL * N, K, ldw, 256, &mw);
    if (rc) return rc;
    GemmTc g;
    g.out = act, g.P = M, g.Q = N, g.K = K, g.stride_p = ldo, g.stride_q = 1;
    g.k_blocks = (K + TILE_K - 1) / TILE_K, g.k_blocks_per_split = g.k_blocks, g.splits = 1;
    g.partials = nullptr, g.tickets = nullptr, g.status = status, g.vec = 1, g.in_cluster = 0, g.weights_are_p = 0;
    if (pairs_win(M, 2 * N) && !abk_pairs_off()) {
        CUtensorMap mw_half;
        rc = tensor_map(w, 2LL * N, K, ldw, 128, &mw_half);
        if (rc) return rc;
        const int m_tiles2 = (M + 2 * TILE_P - 1) / (2 * TILE_P);
        return launch_pair<256, 6, __nv_bfloat16, EPI_GATED>(mx, mw_half, g, m_tiles2, m_tiles2 * (N / 128), (cudaStream_t)stream);
    }
    const int m_tiles = (M + TILE_P - 1) / TILE_P, tiles = m_tiles * (N / 128);
    return launch_persistent<256, 4, __nv_bfloat16, EPI_GATED>(mx, mw, g, m_tiles, tiles, (cudaStream_t)stream);
}

// qkv[M, :n_heads * 128] = the prepared q heads of x . w^T, and the prepared k and the v heads of every token that
// belongs to a sequence into the paged cache (src/model.c:299 with 247-259): the q/k/v product of a prompt with what
// stands between it and attention in its epilogue. w [(n_heads + 2 n_kv_heads) * 128, K] holds q heads, then k heads,
// then v heads, of 128 each; the k and v columns of qkv are not written. q_norm / k_norm [128] float32 or null; cos / sin
// [positions, 64] float32 or null (the rotation over the whole head in halves); pools [pages, n_kv_heads,
// tokens_per_page, 128] bfloat16, the cache's own, all kept. Many rows only (more than 256); other shapes are refused
// (the caller multiplies and prepares in two steps).
extern "C" int abk_gemm_tc_qkv(const void *x, const void *w, void *qkv, int M, int n_heads, int n_kv_heads, int K, long long ldx,
                               long long ldw, long long ldo, const int *token_seq, const int *token_pos, const int *seq_slot,
                               const float *q_norm, const float *k_norm, float eps, const float *cos, const float *sin,
                               void *k_pool, void *v_pool, const int *page_table, int table_width, int tokens_per_page,
                               int *status, void *stream) {
    if (M <= 0) return 0;
    const int N = (n_heads + 2 * n_kv_heads) * 128;
    if (M <= 256 || n_heads < 1 || n_kv_heads < 1 || K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ldo % 8 ||
        (((uintptr_t)x | (uintptr_t)w | (uintptr_t)qkv | (uintptr_t)q_norm | (uintptr_t)k_norm | (uintptr_t)cos | (uintptr_t)sin |
          (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) || !k_pool || !v_pool || !cos != !sin || tokens_per_page < 1)
        ABK_REFUSE("gemm_tc_qkv: %d rows, %d + 2 x %d heads, K = %d are not what the fused kernel takes", M, n_heads, n_kv_heads, K);
    CUtensorMap mx, mw;
    int rc = tensor_map(x, M, K, ldx, TILE_P, &mx);
    if (rc) return rc;
    GemmTc g;
    g.out = qkv, g.P = M, g.Q = N, g.K = K, g.stride_p = ldo, g.stride_q = 1;
    g.k_blocks = (K + TILE_K - 1) / TILE_K, g.k_blocks_per_split = g.k_blocks, g.splits = 1;
    g.partials = nullptr, g.tickets = nullptr, g.status = status, g.vec = 1, g.in_cluster = 0, g.weights_are_p = 0;
    QkvEpilogue e;
    e.token_seq = token_seq, e.token_pos = token_pos, e.seq_slot = seq_slot, e.q_norm = q_norm, e.k_norm = k_norm;
    e.cos = cos, e.sin = sin, e.eps = eps, e.k_pool = (__nv_bfloat16 *)k_pool, e.v_pool = (__nv_bfloat16 *)v_pool;
    e.cache.page_table = page_table, e.cache.table_width = table_width, e.cache.ring_pages = 0;
    e.cache.tokens_per_page = tokens_per_page, e.n_heads = n_heads, e.n_kv_heads = n_kv_heads;
    if (pairs_win(M, N) && !abk_pairs_off()) {
        rc = tensor_map(w, N, K, ldw, 128, &mw);
        if (rc) return rc;
        const int m_tiles2 = (M + 2 * TILE_P - 1) / (2 * TILE_P);
        return launch_pair<256, 5, __nv_bfloat16, EPI_QKV>(mx, mw, g, m_tiles2, m_tiles2 * ((N + 255) / 256), (cudaStream_t)stream, e);
    }
    rc = tensor_map(w, N, K, ldw, 256, &mw);
    if (rc) return rc;
    const int m_tiles = (M + TILE_P - 1) / TILE_P;
    return launch_persistent<256, 3, __nv_bfloat16, EPI_QKV>(mx, mw, g, m_tiles, m_tiles * ((N + 255) / 256), (cudaStream_t)stream, e);
}

template <typename TO>
static int launch_bn(int bn, const CUtensorMap &mp, const CUtensorMap &mq, const GemmTc &g, dim3 grid, cudaStream_t s) {
    switch (bn) {
    case 16: return launch<16, 6, TO>(mp, mq, g, grid, s);  // 108 KB: two CTAs share an SM
    case 32: return launch<32, 5, TO>(mp, mq, g, grid, s);
    case 64: return launch<64, 4, TO>(mp, mq, g, grid, s);
    case 128: return launch<128, 3, TO>(mp, mq, g, grid, s);
    case 256: return launch<256, 2, TO>(mp, mq, g, grid, s);
    }
    return ABK_REFUSED;
}

// Scratch the caller must provide for split K: how many floats and tickets this product may use.
extern "C" long long abk_gemm_tc_scratch_floats() { return 8ll << 20; }
extern "C" int abk_gemm_tc_scratch_tickets() { return 1 << 16; }

// x [M, K] and w [N, K] bfloat16 with row pitches ldx, ldw (elements); out [M, N] bfloat16 or
// float32 with row pitch ldo. scratch: float32 [abk_gemm_tc_scratch_floats()]; tickets: int32
// [abk_gemm_tc_scratch_tickets()], all zero; status: int32 [>= 2], word 1 is set if a wait ran out.
// force_bn / force_swap / force_splits / force_persistent (0 / -1 / 0 / -1: choose) pin the configuration, for tests.
extern "C" int abk_gemm_tc(const void *x, const void *w, void *out, int out_dtype, int M, int N, int K, long long ldx,
                           long long ldw, long long ldo, float *scratch, int *tickets, int *status, int force_bn,
                           int force_swap, int force_splits, int force_persistent, void *stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8)
        ABK_REFUSE("gemm_tc: K = %d and the row pitches %lld, %lld must be multiples of 8", K, ldx, ldw);
    if (((uintptr_t)x | (uintptr_t)w) & 15) ABK_REFUSE("gemm_tc: operands must be 16-byte aligned");
    bool swap = force_swap >= 0 ? force_swap != 0 : M <= 64;
    int bn;
    if (swap) {  // columns are tokens
        bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    } else {  // columns are output features
        long long tiles256 = (long long)((M + TILE_P - 1) / TILE_P) * ((N + 255) / 256);
        bn = N > 128 && tiles256 >= abk_sm_count() ? 256 : N > 64 ? 128 : 64;
    }
    if (force_bn) bn = force_bn;
    // many rows: the persistent kernel, column tiles of 256 if that still gives most SMs a tile, else of 128
    // (with a very long K two CTAs of the other kernel on an SM, each other's stalls covered, were measured faster)
    bool persistent = !swap && M > 256 && N >= 128 && K <= 4096 &&
                      (long long)((M + TILE_P - 1) / TILE_P) * ((N + 127) / 128) >= 96;
    if (force_persistent >= 0) persistent = force_persistent != 0 && !swap;
    // many tiles of 256 x 256: pairs of CTAs (force_persistent 2 pins them, for tests), whatever the length of K
    const bool pair = !swap && !force_bn && (force_persistent == 2 || (force_persistent < 0 && pairs_win(M, N) && !abk_pairs_off()));
    if (pair) {
        CUtensorMap mx2, mw2;
        int rc2 = tensor_map(x, M, K, ldx, TILE_P, &mx2);
        if (!rc2) rc2 = tensor_map(w, N, K, ldw, 128, &mw2);
        if (rc2) return rc2;
        GemmTc g2;
        g2.out = out, g2.P = M, g2.Q = N, g2.K = K, g2.stride_p = ldo, g2.stride_q = 1;
        g2.k_blocks = (K + TILE_K - 1) / TILE_K, g2.k_blocks_per_split = g2.k_blocks, g2.splits = 1;
        g2.partials = nullptr, g2.tickets = nullptr, g2.status = status, g2.in_cluster = 0, g2.weights_are_p = 0;
        g2.vec = ((uintptr_t)out % 16 == 0) && (ldo * (out_dtype == ABK_BF16 ? 2 : 4)) % 16 == 0;
        const int m_tiles2 = (M + 2 * TILE_P - 1) / (2 * TILE_P), tiles2 = m_tiles2 * ((N + 255) / 256);
        return out_dtype == ABK_BF16 ? launch_pair<256, 6, __nv_bfloat16>(mx2, mw2, g2, m_tiles2, tiles2, (cudaStream_t)stream)
                                     : launch_pair<256, 6, float>(mx2, mw2, g2, m_tiles2, tiles2, (cudaStream_t)stream);
    }
    if (persistent && !force_bn) bn = (long long)((M + TILE_P - 1) / TILE_P) * ((N + 255) / 256) >= 112 ? 256 : 128;
    if (persistent && bn != 128 && bn != 256) ABK_REFUSE("gemm_tc: the persistent kernel has column tiles of 128 and 256, not %d", bn);
    int P = swap ? N : M, Q = swap ? M : N;
    if (swap && M > bn && M > 256) ABK_REFUSE("gemm_tc: %d rows do not fit the swapped layout", M);
    dim3 grid((P + TILE_P - 1) / TILE_P, (Q + bn - 1) / bn, 1);
    if (grid.y > 65535) ABK_REFUSE("gemm_tc: too many column tiles (%u)", grid.y);
    int k_blocks = (K + TILE_K - 1) / TILE_K;
    long long tiles = (long long)grid.x * grid.y;
    int splits = 1;
    if (swap) {
        // A decode step: the weights are the lanes and stream through once, so what counts is that every SM has
        // weights in flight all the time. K is shared out until some 180 CTAs work (a power of two of splits, never
        // fewer than 4 blocks of 64 columns each). Measured at 16 rows, splits 1 / 2 / 4 / 8: 6144 x 2560 (48 tiles)
        // 15.7 / 11.9 / 10.6 / 11.1 us; 2560 x 9728 (20 tiles) 49 / 28 / 17.3 / 14.7 us; 6144 x 4096 (48 tiles)
        // 23.7 / 16.4 / 14.6 / 13.9 us; 19456 x 2560 (152 tiles) 23.0 / 23.2 / 26.9 / 36.9 us. With more than 32
        // columns (tokens) a partial tile costs more to add up, and beyond four splits that outweighs the gain
        // (2560 x 4096 at 64 rows: 23.7 / 16.9 / 12.3 / 15.3 us) unless the tiles are very few.
        const int want = (int)((180 + tiles / 2) / tiles);
        const int most = bn <= 32 || tiles <= 8 ? 8 : 4;
        for (splits = 1; splits * 2 <= want && splits * 2 <= most && k_blocks / (splits * 2) >= 4;) splits *= 2;
        if (want >= 3 && splits == 2 && most >= 4 && k_blocks / 4 >= 4) splits = 4;  // (3 rounds up: 48 tiles take four)
    } else if (tiles <= 32) {
        // Few tiles: share them along K, but sparingly: every split pays for its partial tile and for adding them
        // up. Measured at 64 rows with the splits as a cluster: 8 tiles (1024 x 2048) 14.3 us unsplit, 8.5 with four;
        // 32 tiles (4096 x 1024) 9.6 us unsplit, 8.6 with four; 48 tiles (6144 x 1024) 9.9 us unsplit, 12.0 with four.
        splits = 4;
        if (splits > k_blocks / 4) splits = k_blocks / 4;
        if (bn > 128 && tiles >= 16) splits = 1;  // (partial tiles through scratch memory: 2048 x 4096 x 1024 at 200 rows doubles)
        if (splits < 1) splits = 1;
    }
    if (force_splits) splits = force_splits;
    if (persistent) splits = 1;
    if (splits > k_blocks) splits = k_blocks;
    int per = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + per - 1) / per;
    if (splits > 1) {
        if (tiles > abk_gemm_tc_scratch_tickets() ||
            (long long)splits * tiles * bn * TILE_P > abk_gemm_tc_scratch_floats())
            splits = 1, per = k_blocks;
    }
    grid.z = splits;

    CUtensorMap mx, mw;
    int rc = tensor_map(x, M, K, ldx, swap ? bn : TILE_P, &mx);
    if (rc) return rc;
    rc = tensor_map(w, N, K, ldw, swap ? TILE_P : bn, &mw);
    if (rc) return rc;
    GemmTc g;
    g.out = out, g.P = P, g.Q = Q, g.K = K;
    g.stride_p = swap ? 1 : ldo, g.stride_q = swap ? ldo : 1;
    g.k_blocks = k_blocks, g.k_blocks_per_split = per, g.splits = splits;
    g.partials = scratch, g.tickets = tickets, g.status = status;
    // (a partial tile of 128 x (bn + 4) floats fits where the operands' stages were for column tiles up to 128)
    g.in_cluster = splits > 1 && splits <= 8 && bn <= 128;
    g.weights_are_p = swap ? 1 : 0;
    int esize = out_dtype == ABK_BF16 ? 2 : 4;
    g.vec = !swap && ((uintptr_t)out % 16 == 0) && (ldo * esize) % 16 == 0;
    cudaStream_t s = (cudaStream_t)stream;
    const CUtensorMap &mp = swap ? mw : mx, &mq = swap ? mx : mw;
    if (persistent) {
        const int m_tiles = grid.x, tiles = grid.x * grid.y;
        if (bn == 256) return out_dtype == ABK_BF16 ? launch_persistent<256, 4, __nv_bfloat16>(mp, mq, g, m_tiles, tiles, s)
                                                    : launch_persistent<256, 4, float>(mp, mq, g, m_tiles, tiles, s);
        return out_dtype == ABK_BF16 ? launch_persistent<128, 6, __nv_bfloat16>(mp, mq, g, m_tiles, tiles, s)
                                     : launch_persistent<128, 6, float>(mp, mq, g, m_tiles, tiles, s);
    }
    if (out_dtype == ABK_BF16) rc = launch_bn<__nv_bfloat16>(bn, mp, mq, g, grid, s);
    else rc = launch_bn<float>(bn, mp, mq, g, grid, s);
    if (rc == ABK_REFUSED) ABK_REFUSE("gemm_tc: no kernel for a column tile of %d", bn);
    return rc;
}
