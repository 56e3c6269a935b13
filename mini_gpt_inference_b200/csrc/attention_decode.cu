// Attention of single query tokens over the paged cache, split along the keys (bfloat16 cache).
//
// A decoding step reads every key and value of every live request once: it is bound by HBM
// bandwidth, and a request alone gives too little parallelism.  So the keys of a (token, kv head)
// are cut into blocks of SPLIT positions, one CTA each; the query heads that share the kv head
// (up to 16 per CTA) are the columns of one small matrix product, so grouped heads read their keys
// once.
//
// A CTA's four warps each own a quarter of the block's keys from load to result:
//
//   load    every lane copies 16-byte pieces of its warp's key and value rows from their pages
//           into shared memory (cp.async), swizzled so that the matrix loads below meet no bank
//           conflict.  Positions, block tables and every cache row but the newest were written
//           before this step began, so all of this is asked for BEFORE the wait for the kernel in
//           front (which wrote the query and the newest row); the newest row follows after it.
//   scores  S[key, head] = K q^T on warp-level mma (m16n8k16: sixteen keys are the rows of A, read
//           with ldmatrix; up to eight heads the columns of B), scaled by scale * log2 e in 32-bit;
//   softmax maximum, base-2 exponentials and their sum over the warp's keys, per head, in 32-bit,
//           inside the accumulator registers (a head's keys live in the eight lanes with equal t);
//   values  O[dim, head] = V^T P: V through ldmatrix.trans as the A operand, P rounded to bfloat16
//           and brought from the accumulator layout to the B layout by movmatrix (an 8x8 transpose
//           inside the warp).  With keys and dims as rows no row of a product is padding, whatever
//           the number of heads.
//
// The four warps' (maximum, sum, O) are combined through shared memory into the block's partial
// result, written to scratch; the CTA that arrives last at a counter of its (token, kv head)
// merges the blocks, writes the output rows and resets the counter (so the counters stay zero
// between launches).  Block edges are absolute positions (multiples of SPLIT from the first
// visible key), so what a token computes does not depend on the batch it is in.
//
// Sizes: head_dim in {16, 32, 64, 128, 256}; any number of heads and kv heads; any page size.
// Nothing here waits on another CTA, so no wait needs a bound; `status` is unused but kept in the
// interface.
#include <math.h>

#include "common.cuh"

MG_STAMP_DECLARE(attn)
MG_GUARD_DECLARE(attention_split)
#ifdef MG_STAMPS
// (the grid is three-dimensional here: stamps go by the CTA's linear index, thread 0 of each CTA)
#define MG_STAMP_ATTN(slot)                                                                                  \
    do {                                                                                                     \
        const unsigned cta_ = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;                \
        if (threadIdx.x == 0 && cta_ < MG_STAMP_CTAS) {                                                      \
            if ((slot) == 0) {                                                                               \
                long long t_;                                                                                \
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                       \
                attn_stamp_buf[cta_ * MG_STAMP_SLOTS] = t_;                                                  \
                attn_stamp_buf[cta_ * MG_STAMP_SLOTS + 1] = clock64();                                       \
            } else {                                                                                         \
                attn_stamp_buf[cta_ * MG_STAMP_SLOTS + (slot)] = clock64();                                  \
            }                                                                                                \
        }                                                                                                    \
    } while (0)
#else
#define MG_STAMP_ATTN(slot) do {} while (0)
#endif

namespace {

constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;
constexpr int HEAD_ROWS = 16;              // query heads per CTA (rows of the A operand)

// Keys per block: 16 KB per tile (32 KB at head_dim 256), so that several CTAs share an SM and a
// whole decode batch of a few thousand blocks is in flight at once; at least 16 keys per warp.
__host__ __device__ constexpr int split_keys(int head_dim) {
    return head_dim <= 32 ? 256 : (8192 / head_dim < 64 ? 64 : 8192 / head_dim);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Transpose of an 8x8 block of 16-bit values held one row per group of four lanes.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// The four warps of a CTA merge the key blocks of one (token, head).  Up to 16 blocks: warp 0 alone,
// everything it needs asked for at once (one trip to memory).  More: every warp finds the row's
// maximum, takes a quarter of the blocks (contiguous, in order; eight blocks' values and weights in
// flight per lane), and the quarters' sums meet in `scratch` (shared memory, WARPS * (D + 1) floats)
// and are added in warp order.  How the blocks are shared depends on their number only, so a token's
// result does not depend on the batch.  Every thread of the CTA must call it (it has two barriers).
template <int D>
__device__ __forceinline__ void merge_row(const float* __restrict__ part_out, const float* __restrict__ part_ml,
                                          size_t base, int splits, float* scratch, bf16* __restrict__ out_row,
                                          int warp, int lane) {
    constexpr int DPL = (D + 31) / 32;                                  // dims per lane: lane, lane + 32, ..
    if constexpr (D >= 32 && D <= 128) {
        if (splits <= 16) {
            if (warp != 0) return;                                      // (uniform: no barrier on this path)
            // Few blocks: maxima, sums and every partial value this lane needs are asked for at
            // once (one trip to memory instead of two); lane s holds the weight of block s.
            const float2 ml = lane < splits ? __ldcg(reinterpret_cast<const float2*>(part_ml) + base + lane)
                                            : make_float2(-INFINITY, 0.f);
            float x[16][DPL];
#pragma unroll
            for (int sidx = 0; sidx < 16; ++sidx)
#pragma unroll
                for (int j = 0; j < DPL; ++j)
                    x[sidx][j] = sidx < splits ? __ldcg(&part_out[(base + sidx) * D + lane + 32 * j]) : 0.f;
            const float M = warp_max(ml.x);
            const float w = lane < splits ? exp2f(ml.x - M) : 0.f;
            const float inv = 1.0f / warp_sum(w * ml.y);
            float v[DPL];
#pragma unroll
            for (int j = 0; j < DPL; ++j) v[j] = 0.f;
#pragma unroll
            for (int sidx = 0; sidx < 16; ++sidx) {                       // blocks in order
                const float ws = __shfl_sync(0xffffffffu, w, sidx);
#pragma unroll
                for (int j = 0; j < DPL; ++j) v[j] = fmaf(ws, x[sidx][j], v[j]);
            }
#pragma unroll
            for (int j = 0; j < DPL; ++j) out_row[lane + 32 * j] = __float2bfloat16_rn(v[j] * inv);
            return;
        }
    }
    float M = -INFINITY;
    for (int sidx = lane; sidx < splits; sidx += 32) M = fmaxf(M, __ldcg(&part_ml[(base + sidx) * 2]));
    M = warp_max(M);
    const int per = (splits + WARPS - 1) / WARPS;
    const int b0 = warp * per, b1 = min(splits, b0 + per);
    float v[DPL], den = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) v[j] = 0.f;
    for (int s0 = b0; s0 < b1; s0 += 8) {
        float x[8][DPL];
        float2 ml[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const bool in = s0 + u < b1;
            ml[u] = in ? __ldcg(reinterpret_cast<const float2*>(part_ml) + base + s0 + u) : make_float2(-INFINITY, 0.f);
#pragma unroll
            for (int j = 0; j < DPL; ++j)
                x[u][j] = (in && lane + 32 * j < D) ? __ldcg(&part_out[(base + s0 + u) * D + lane + 32 * j]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {                                     // blocks in order
            const float w = s0 + u < b1 ? exp2f(ml[u].x - M) : 0.f;
            den = fmaf(w, ml[u].y, den);
#pragma unroll
            for (int j = 0; j < DPL; ++j) v[j] = fmaf(w, x[u][j], v[j]);
        }
    }
    __syncthreads();                                                    // `scratch` may still be in use (the row before)
#pragma unroll
    for (int j = 0; j < DPL; ++j)
        if (lane + 32 * j < D) scratch[warp * (D + 1) + lane + 32 * j] = v[j];
    if (lane == 0) scratch[warp * (D + 1) + D] = den;
    __syncthreads();
    if (warp == 0) {
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) total += scratch[w * (D + 1) + D];        // warps in order
        const float inv = 1.0f / total;
#pragma unroll
        for (int j = 0; j < DPL; ++j)
            if (lane + 32 * j < D) {
                float y = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) y += scratch[w * (D + 1) + lane + 32 * j];
                out_row[lane + 32 * j] = __float2bfloat16_rn(y * inv);
            }
    }
}

// The merge as a kernel of its own, for grids of many waves: the attention CTAs then leave as soon
// as their partial rows are written, instead of each waiting for the old value of a counter.
template <int D>
__global__ void __launch_bounds__(THREADS)
attention_merge_kernel(const int* __restrict__ positions, const float* __restrict__ part_out,
                       const float* __restrict__ part_ml, bf16* __restrict__ out, int n_head, int window,
                       int max_splits) {
    constexpr int SPLIT = split_keys(D);
    __shared__ float scratch[WARPS * (D + 1)];
    const int token = blockIdx.x, head = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = positions[token];
    pdl_trigger();
    pdl_wait();                                                        // the partial rows come from the kernel in front
    if (p < 0) return;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int splits = (p - lo) / SPLIT + 1;
    if (splits == 1) return;                                            // the attention kernel wrote the row itself
    if (!MG_GUARDED(attention_split, MG_GUARD_POSITION, splits - 1, max_splits)) return;   // (more blocks than the scratch holds)
    const size_t pair = (size_t)token * n_head + head;
    merge_row<D>(part_out, part_ml, pair * max_splits, splits, scratch, out + pair * D, warp, lane);
}

// partial layout: out [token][head][split][D], ml [token][head][split][2]; counters [token][kv head tile]
// VSTREAM: the values are not kept beside the keys.  Their rows are only asked into the L2 cache
// before the wait and copied into the keys' place once the scores are done, so a CTA holds half
// the shared memory and twice as many CTAs are on the GPU at once: for grids that need fewer rounds
// of CTAs that way (a round's loads start only when the round before ends), at the price of one
// trip to L2 on every CTA's way.
template <int D, int NT, bool VSTREAM>   // NT: tiles of 8 query heads per CTA (1 or 2)
__global__ void __launch_bounds__(THREADS)
attention_split_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ k_pages,
                       const bf16* __restrict__ v_pages, const int* __restrict__ block_table,
                       const int* __restrict__ token_request, const int* __restrict__ positions,
                       bf16* __restrict__ out, float* __restrict__ part_out, float* __restrict__ part_ml,
                       int* __restrict__ counters, int n_head, int n_kv_head, int page_tokens, int max_pages,
                       int window, int max_splits, float scale_log2e, int head_tiles, int merge_inside,
                       int num_pages, int n_requests) {
    constexpr int SPLIT = split_keys(D);
    constexpr int KW = SPLIT / WARPS;          // keys per warp
    constexpr int CPR = D / 8;                 // 16-byte pieces per row
    constexpr int ROWB = 2 * D;                // bytes per row
    constexpr int RPL = CPR >= 8 ? 1 : 8 / CPR;        // rows per 128 bytes of shared memory
    constexpr int SWZ = CPR >= 8 ? 8 : CPR;            // piece c of row r lies at piece c ^ ((r / RPL) % SWZ)
    constexpr int OSTRIDE = D + 2;             // floats per (warp, head) partial: O, maximum, sum
    constexpr int QSTRIDE = D + 8;             // query rows 16 bytes apart in the banks
    static_assert(KW % 16 == 0, "a warp takes whole k steps of keys");
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* k_tile = smem;                                            // [SPLIT][D] bf16, swizzled
    uint8_t* v_tile = VSTREAM ? smem : smem + SPLIT * ROWB;            // VSTREAM: the values come where the keys were
    int* grow = reinterpret_cast<int*>(v_tile + SPLIT * ROWB);         // [SPLIT] cache row of each key
    bf16* q_tiles = reinterpret_cast<bf16*>(grow + SPLIT);             // [WARPS][rows][QSTRIDE]: a copy per warp
    __shared__ int is_last;

    const int token = blockIdx.x, split = blockIdx.z;
    const int kv_head = blockIdx.y / head_tiles, ht = blockIdx.y - kv_head * head_tiles;
    const int group = n_head / n_kv_head;
    const int h0 = kv_head * group + ht * HEAD_ROWS;                   // first query head of this CTA
    const int nh = min(HEAD_ROWS, group - ht * HEAD_ROWS);
    const int nh_rows = min(HEAD_ROWS, group);                         // rows the launch reserved
    float* wpart = reinterpret_cast<float*>(q_tiles + WARPS * nh_rows * QSTRIDE);   // [WARPS][nh][OSTRIDE]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    MG_STAMP_ATTN(0);
    pdl_trigger();
    int request = token_request[token];                                // asked for together with the position:
    int p = positions[token];                                          // one trip to memory, not two
    // (guarded builds: a request beyond the block tables' rows, a position beyond their width or a page
    // beyond the pool is recorded, and request 0, position 0 or page 0 is read in its place)
    if (!MG_GUARDED(attention_split, MG_GUARD_REQUEST, request, n_requests)) request = 0;
    if (p >= 0 && !MG_GUARDED(attention_split, MG_GUARD_POSITION, p, (long long)max_pages * page_tokens)) p = 0;
    if (p < 0) {                                                        // padding row of a fixed-size batch
        pdl_wait();                                                     // `out` may still be in use before
        if (split == 0)
            for (int i = tid; i < nh * D; i += THREADS)
                out[((size_t)token * n_head + h0 + i / D) * D + i % D] = __float2bfloat16_rn(0.f);
        return;
    }
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int start = lo + split * SPLIT;
    if (start > p) return;                                              // this block holds no key of the token
    const int count = min(SPLIT, p + 1 - start);
    const int splits = (p - lo) / SPLIT + 1;
    if (!MG_GUARDED(attention_split, MG_GUARD_POSITION, splits - 1, max_splits)) return;   // (more blocks than the scratch holds)
    const int* table = block_table + (size_t)request * max_pages;
    const bool holds_newest = start + count - 1 == p;
    const int old_count = holds_newest ? count - 1 : count;            // rows [0, old_count) are old

    // ---- where each key of this warp lies in the cache (a warp needs no other warp's rows) ----
    for (int i = lane; i < KW; i += 32) {
        const int r = warp * KW + i;
        if (r < count) {
            const int pos = start + r, pi = pos / page_tokens;
            int page = table[pi];
            if (!MG_GUARDED(attention_split, MG_GUARD_PAGE, page, num_pages)) page = 0;
            grow[r] = (page * n_kv_head + kv_head) * page_tokens + (pos - pi * page_tokens);
        }
    }
    __syncwarp();
    MG_STAMP_ATTN(2);
    // ---- every warp asks for its own rows: all keys first, then all values ----
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int which = 0; which < 2; ++which) {
        const bf16* pages = which == 0 ? k_pages : v_pages;
        uint8_t* tile = which == 0 ? k_tile : v_tile;
#pragma unroll 4
        for (int i = lane; i < KW * CPR; i += 32) {
            const int r = warp * KW + i / CPR, c = i % CPR;
            if (VSTREAM && which == 1) {
                // only towards L2 for now: one request per 128-byte line of the row
                if (r < old_count && (c * 16) % 128 == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(pages + (size_t)grow[r] * D + c * 8));
                continue;
            }
            uint8_t* dst = tile + r * ROWB + ((c ^ ((r / RPL) % SWZ)) * 16);
            if (r < old_count) cp_async16(smem_u32(dst), pages + (size_t)grow[r] * D + c * 8);
            else if (r >= count) *reinterpret_cast<uint4*>(dst) = zero4;            // keeps 0 * garbage out of O
        }
        if (!(VSTREAM && which == 1)) asm volatile("cp.async.commit_group;" ::: "memory");
    }
    MG_STAMP_ATTN(3);
    pdl_wait();
    MG_STAMP_ATTN(4);
    // ---- what the kernel in front wrote: the newest row (to the warp that owns it) and the
    // queries (a copy for every warp, so that no warp waits for another before the end) ----
    if (holds_newest && warp == (count - 1) / KW) {
        for (int i = lane; i < (VSTREAM ? 1 : 2) * CPR; i += 32) {     // (streamed values are copied later, the newest with them)
            const int which = i / CPR, c = i - which * CPR, r = count - 1;
            const uint4 v = *reinterpret_cast<const uint4*>((which == 0 ? k_pages : v_pages) + (size_t)grow[r] * D + c * 8);
            *reinterpret_cast<uint4*>((which == 0 ? k_tile : v_tile) + r * ROWB + ((c ^ ((r / RPL) % SWZ)) * 16)) = v;
        }
    }
    bf16* q_tile = q_tiles + warp * (nh_rows * QSTRIDE);
    {
        const size_t qkv_width = (size_t)(n_head + 2 * n_kv_head) * D;
        for (int i = lane; i < nh * CPR; i += 32) {
            const int row = i / CPR, c = i - row * CPR;
            *reinterpret_cast<uint4*>(q_tile + row * QSTRIDE + c * 8) =
                *reinterpret_cast<const uint4*>(qkv + (size_t)token * qkv_width + (size_t)(h0 + row) * D + c * 8);
        }
    }
    if (VSTREAM) asm volatile("cp.async.wait_group 0;" ::: "memory");
    else asm volatile("cp.async.wait_group 1;" ::: "memory");          // this lane's keys have landed
    __syncwarp();                                                       // the warp's keys, its newest row, its queries
    MG_STAMP_ATTN(5);

    // ---- scores, keys as rows: S[key, head] = k . q over this warp's KW keys ----
    // B operand: the queries, head nt * 8 + g in column g (heads past the group are zero columns)
    uint32_t qb[NT][D / 16][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int h = nt * 8 + g;
            qb[nt][ks][0] = h < nh ? *reinterpret_cast<const uint32_t*>(q_tile + h * QSTRIDE + ks * 16 + 2 * t) : 0u;
            qb[nt][ks][1] = h < nh ? *reinterpret_cast<const uint32_t*>(q_tile + h * QSTRIDE + ks * 16 + 8 + 2 * t) : 0u;
        }
    float s[NT][KW / 16][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int mt = 0; mt < KW / 16; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[nt][mt][i] = 0.f;
    {
        // A operand by ldmatrix.x4: matrix j = lane / 8 holds keys (j % 2) * 8 .., piece j / 2
        const int lrow = (lane & 7) + (((lane >> 3) & 1) << 3), lpiece = lane >> 4;
#pragma unroll
        for (int mt = 0; mt < KW / 16; ++mt)
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const int r = warp * KW + mt * 16 + lrow, c = ks * 2 + lpiece;
                uint32_t a[4];
                ldmatrix_x4(a, smem_u32(k_tile + r * ROWB + ((c ^ ((r / RPL) % SWZ)) * 16)));
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_bf16(s[nt][mt], a, qb[nt][ks][0], qb[nt][ks][1]);
            }
    }
    // ---- softmax over the warp's keys, per head: a lane holds heads 2t, 2t+1 (values 0, 1 and
    // 2, 3) of keys g and g + 8 of every 16; the other keys of a head are in the lanes with the same t
    float mx[NT][2], sum[NT][2];
    uint32_t pb[NT][KW / 16][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        mx[nt][0] = mx[nt][1] = -INFINITY;
#pragma unroll
        for (int mt = 0; mt < KW / 16; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = warp * KW + mt * 16 + g + ((i >> 1) << 3);
                s[nt][mt][i] = r < count ? s[nt][mt][i] * scale_log2e : -INFINITY;
                mx[nt][i & 1] = fmaxf(mx[nt][i & 1], s[nt][mt][i]);
            }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) mx[nt][i] = fmaxf(mx[nt][i], __shfl_xor_sync(0xffffffffu, mx[nt][i], o));
        sum[nt][0] = sum[nt][1] = 0.f;
#pragma unroll
        for (int mt = 0; mt < KW / 16; ++mt) {
            float e[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float m = mx[nt][i & 1];
                e[i] = m == -INFINITY ? 0.f : exp2_approx(s[nt][mt][i] - m);  // a warp past the last key holds nothing
                sum[nt][i & 1] += e[i];
            }
            // P[key, head] as the B operand of the next product needs keys along k: the 8x8 blocks
            // (keys g, heads 2t..) are transposed inside the warp
            pb[nt][mt][0] = movmatrix_trans(pack_bf16(e[0], e[1]));
            pb[nt][mt][1] = movmatrix_trans(pack_bf16(e[2], e[3]));
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) sum[nt][i] += __shfl_xor_sync(0xffffffffu, sum[nt][i], o);
    }

    MG_STAMP_ATTN(6);
    // ---- values, dims as rows: O[dim, head] = sum over keys of v[key, dim] * p[key, head] ----
    if (VSTREAM) {
        // the warp's keys are used up: its value rows (from L2 by now, the newest included) take their place
        __syncwarp();
        for (int i = lane; i < KW * CPR; i += 32) {
            const int r = warp * KW + i / CPR, c = i % CPR;
            uint8_t* dst = v_tile + r * ROWB + ((c ^ ((r / RPL) % SWZ)) * 16);
            if (r < count) cp_async16(smem_u32(dst), v_pages + (size_t)grow[r] * D + c * 8);
            else *reinterpret_cast<uint4*>(dst) = zero4;                // keeps 0 * garbage out of O
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    float o[NT][D / 16][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int dm = 0; dm < D / 16; ++dm)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[nt][dm][i] = 0.f;
    {
        // A operand by ldmatrix.x4.trans: matrix j holds keys (j / 2) * 8 .., piece j % 2
        const int lrow = (lane & 7) + (((lane >> 4) & 1) << 3), lpiece = (lane >> 3) & 1;
#pragma unroll
        for (int kk = 0; kk < KW / 16; ++kk)
#pragma unroll
            for (int dm = 0; dm < D / 16; ++dm) {
                const int r = warp * KW + kk * 16 + lrow, c = dm * 2 + lpiece;
                uint32_t a[4];
                ldmatrix_x4_trans(a, smem_u32(v_tile + r * ROWB + ((c ^ ((r / RPL) % SWZ)) * 16)));
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_bf16(o[nt][dm], a, pb[nt][kk][0], pb[nt][kk][1]);
            }
    }
    MG_STAMP_ATTN(7);
    // ---- the four warps' results meet in shared memory ----
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = nt * 8 + 2 * t + i;
            if (row < nh) {
                float* dst = wpart + ((size_t)warp * nh + row) * OSTRIDE;
#pragma unroll
                for (int dm = 0; dm < D / 16; ++dm) {
                    dst[dm * 16 + g] = o[nt][dm][i];
                    dst[dm * 16 + g + 8] = o[nt][dm][i + 2];
                }
                if (g == 0) {
                    dst[D] = mx[nt][i];
                    dst[D + 1] = sum[nt][i];
                }
            }
        }
    __syncthreads();
    const size_t pair0 = (size_t)token * n_head + h0;
    for (int e = tid; e < nh * D; e += THREADS) {
        const int row = e / D, d = e - row * D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, wpart[((size_t)w * nh + row) * OSTRIDE + D]);
        float v = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {                               // warps in order
            const float* src = wpart + ((size_t)w * nh + row) * OSTRIDE;
            const float f = src[D] == -INFINITY ? 0.f : exp2f(src[D] - m);
            v = fmaf(f, src[d], v);
            l = fmaf(f, src[D + 1], l);
        }
        if (splits == 1) {                                              // nothing to merge
            out[(pair0 + row) * D + d] = __float2bfloat16_rn(v / l);
        } else {
            const size_t slot = (pair0 + row) * max_splits + split;
            part_out[slot * D + d] = v;
            if (d == 0) {
                part_ml[slot * 2] = m;
                part_ml[slot * 2 + 1] = l;
            }
        }
    }
    MG_STAMP_ATTN(8);
    if (splits == 1 || !merge_inside) return;
    // ---- the CTA that finishes last merges the blocks of this (token, kv head) ----
    // The barrier orders every thread's partial writes before thread 0's release on the counter;
    // the CTA that reads the final count acquires, so it sees the partial rows of all blocks.
    __syncthreads();
    int* counter = counters + (size_t)token * (n_kv_head * head_tiles) + blockIdx.y;
    if (tid == 0) {
        int done;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(done) : "l"(counter) : "memory");
        is_last = (done == splits - 1);
        if (is_last) *counter = 0;                                      // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    // The heads one after the other, all four warps on each (the key tile is free now: scratch).
    for (int row = 0; row < nh; ++row)
        merge_row<D>(part_out, part_ml, (pair0 + row) * max_splits, splits, reinterpret_cast<float*>(k_tile),
                     out + (pair0 + row) * D, warp, lane);
    MG_STAMP_ATTN(9);
}

// Whether the CTA that finishes last merges the key blocks of its row (one launch), or a second
// kernel does (two launches): a grid of more than MERGE_INSIDE_CTAS CTAs takes the second form.
constexpr long long MERGE_INSIDE_CTAS = 1536;
inline bool merges_inside(int n_tokens, int n_head, int n_kv_head, int max_splits) {
    const int group = n_head / n_kv_head;
    const long long head_tiles = (group + HEAD_ROWS - 1) / HEAD_ROWS;
    return max_splits == 1 || (long long)n_tokens * n_kv_head * head_tiles * max_splits <= MERGE_INSIDE_CTAS;
}

int device_sms() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    return sms;
}

template <int D>
int launch(const void* qkv, const void* k_pages, const void* v_pages, const int* block_table,
           const int* token_request, const int* positions, void* out, float* part_out, float* part_ml,
           int* counters, int n_tokens, int n_head, int n_kv_head, int page_tokens, int max_pages, int window,
           int max_splits, float scale, int num_pages, int n_requests, cudaStream_t s) {
    const int group = n_head / n_kv_head;
    const int head_tiles = (group + HEAD_ROWS - 1) / HEAD_ROWS;
    const int nh_max = group < HEAD_ROWS ? group : HEAD_ROWS;
    const size_t rest = (size_t)WARPS * nh_max * (D + 8) * sizeof(bf16) + (size_t)split_keys(D) * sizeof(int) +
                        (size_t)WARPS * nh_max * (D + 2) * sizeof(float);
    const size_t tile = (size_t)split_keys(D) * D * sizeof(bf16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaSuccess;
        for (auto fn : {attention_split_kernel<D, 1, false>, attention_split_kernel<D, 2, false>,
                        attention_split_kernel<D, 1, true>, attention_split_kernel<D, 2, true>})
            if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "attention (split): cannot raise shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(n_tokens, n_kv_head * head_tiles, max_splits);
    const long long ctas = (long long)n_tokens * n_kv_head * head_tiles * max_splits;
    // Keys and values side by side if the whole grid is on the GPU at once that way (or if not even
    // half the shared memory per CTA would achieve it); else the values are streamed after the keys.
    auto resident = [&](bool streamed) -> long long {
        int per_sm = 0;
        const size_t bytes = (streamed ? tile : 2 * tile) + rest;
        const cudaError_t e =
            nh_max <= 8 ? (streamed ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_split_kernel<D, 1, true>, THREADS, bytes)
                                    : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_split_kernel<D, 1, false>, THREADS, bytes))
                        : (streamed ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_split_kernel<D, 2, true>, THREADS, bytes)
                                    : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_split_kernel<D, 2, false>, THREADS, bytes));
        return e == cudaSuccess ? (long long)per_sm * device_sms() : 0;
    };
    // the values are streamed after the keys wherever that saves a round of CTAs
    const long long beside = resident(false), after = resident(true);
    const bool vstream = beside > 0 && after > 0 && (ctas + after - 1) / after < (ctas + beside - 1) / beside;
    const size_t smem = (vstream ? tile : 2 * tile) + rest;
    // A grid of several waves (six CTAs fit an SM) merges in a second kernel, so that its CTAs do
    // not hold their shared memory while a counter answers; a small grid merges inside, which
    // saves a launch.
    const int merge_inside = merges_inside(n_tokens, n_head, n_kv_head, max_splits) ? 1 : 0;
    auto kernel = nh_max <= 8 ? (vstream ? attention_split_kernel<D, 1, true> : attention_split_kernel<D, 1, false>)
                              : (vstream ? attention_split_kernel<D, 2, true> : attention_split_kernel<D, 2, false>);
    cudaError_t le = mg_launch(kernel, grid, dim3(THREADS), smem, s, true, (const bf16*)qkv, (const bf16*)k_pages,
                               (const bf16*)v_pages, block_table, token_request, positions, (bf16*)out, part_out, part_ml,
                               counters, n_head, n_kv_head, page_tokens, max_pages, window, max_splits,
                               scale * 1.4426950408889634f, head_tiles, merge_inside, num_pages, n_requests);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "attention_split: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("attention_split");
    if (!merge_inside) {
        le = mg_launch(attention_merge_kernel<D>, dim3(n_tokens, n_head), dim3(THREADS), 0, s, true,
                       positions, (const float*)part_out, (const float*)part_ml, (bf16*)out, n_head, window, max_splits);
        if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "attention_merge: %s", cudaGetErrorString(le));
        MG_CHECK_LAUNCH("attention_merge");
    }
    return MG_OK;
}

}  // namespace

// Number of key blocks a context of `max_context` positions can have (with a window, at most
// the window's length counts).
MG_API int mg_attention_split_count(int max_context, int window, int head_dim) {
    int span = (window > 0 && window < max_context) ? window : max_context;
    if (span < 1) span = 1;
    return (span - 1) / split_keys(head_dim) + 1;
}

// Key positions per block at this head size (0 if the head size is not served).
MG_API int mg_attention_split_keys(int head_dim) {
    return (head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256)
               ? split_keys(head_dim) : 0;
}

// Kernels that mg_paged_attention_split() launches for these sizes: 1, or 2 when the merge of the
// key blocks runs as a kernel of its own.
MG_API int mg_attention_split_launches(int n_tokens, int n_head, int n_kv_head, int max_splits) {
    if (n_tokens <= 0 || n_kv_head <= 0 || n_head % n_kv_head != 0) return 1;
    return merges_inside(n_tokens, n_head, n_kv_head, max_splits) ? 1 : 2;
}

// Floats of scratch the split kernel needs (partial outputs, then maxima and sums).
MG_API long long mg_attention_split_scratch_floats(int n_tokens, int n_head, int head_dim, int max_splits) {
    return (long long)n_tokens * n_head * max_splits * (head_dim + 2);
}

// One query token per row (a row with position < 0 is padding: its output is zeros).
// qkv / pages / out as mg_paged_attention_generic, bfloat16 only.  `scratch` holds
// mg_attention_split_scratch_floats() floats and need not be initialised; `counters` holds
// n_tokens * n_head ints that are ZERO before the first launch (the kernel leaves them zero);
// `max_splits` = mg_attention_split_count() of the longest context; `num_pages` and `n_requests`: pages
// of the pool and rows of the block table (what guarded builds hold the indices against); `status` is not written
// (the kernel has no bounded wait).  Launches that share scratch or counters must not overlap.
MG_API int mg_paged_attention_split(const void* qkv, const void* k_pages, const void* v_pages,
                                    const int* block_table, const int* token_request, const int* positions,
                                    void* out, float* scratch, int* counters, int n_tokens, int n_head,
                                    int n_kv_head, int head_dim, int page_tokens, int max_pages, int window,
                                    int max_splits, float scale, int num_pages, int n_requests, int* status,
                                    void* stream) {
    (void)status;
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && n_kv_head > 0 && page_tokens > 0 && max_pages > 0 && max_splits > 0,
               "attention (split): bad sizes");
    MG_REQUIRE(n_head % n_kv_head == 0, "attention: n_head %d is not a multiple of n_kv_head %d", n_head, n_kv_head);
    MG_REQUIRE(n_head <= 65535 && max_splits <= 65535, "attention (split): too many heads or key blocks");
    MG_REQUIRE(scratch != nullptr && counters != nullptr, "attention (split): missing scratch");
    cudaStream_t s = (cudaStream_t)stream;
    float* part_out = scratch;
    float* part_ml = scratch + (size_t)n_tokens * n_head * max_splits * head_dim;
#define MG_SPLIT_CASE(DIM)                                                                                        \
    case DIM:                                                                                                     \
        return launch<DIM>(qkv, k_pages, v_pages, block_table, token_request, positions, out, part_out, part_ml, \
                           counters, n_tokens, n_head, n_kv_head, page_tokens, max_pages, window, max_splits,    \
                           scale, num_pages, n_requests, s)
    switch (head_dim) {
        MG_SPLIT_CASE(16);
        MG_SPLIT_CASE(32);
        MG_SPLIT_CASE(64);
        MG_SPLIT_CASE(128);
        MG_SPLIT_CASE(256);
        default:
            return mg_set_error(MG_ERR_UNSUPPORTED, "attention (split): head_dim %d is not 16, 32, 64, 128 or 256", head_dim);
    }
#undef MG_SPLIT_CASE
}
