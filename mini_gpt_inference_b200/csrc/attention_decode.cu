// Attention of single query tokens over the paged cache, split along the keys (bfloat16 cache).
//
// A decoding step reads every key and value of every live request once: it is bound by HBM
// bandwidth, and a request alone gives too little parallelism (one head is one row of work).
// So the keys of a (token, head) are cut into blocks of SPLIT positions, one CTA each.
//
// A CTA first asks for everything it will read: one warp issues a bulk asynchronous copy
// (cp.async.bulk, global -> shared, completion counted on an mbarrier) per cache page and
// per tensor, keys on one barrier and values on another, so that tens of kilobytes are in
// flight per CTA without holding registers, and the score pass starts as soon as the keys have
// landed while the values are still arriving.  Then, from shared memory:
//
//   pass 1  scores: a key row is read by head_dim / 8 neighbouring lanes, 16 bytes each, and the
//           dot product is finished with shuffles; the query is pre-scaled by scale * log2 e;
//   pass 2  the block's maximum, the base-2 exponentials and their sum, all in 32-bit;
//   pass 3  sum of p * v over the value rows, in 32-bit.
//
// Each CTA writes its unnormalised output, maximum and sum to scratch memory and bumps a counter
// of its (token, head); the CTA that arrives last merges the blocks, writes the output row and
// resets the counter (so the counters stay zero between launches).  Block edges are absolute
// positions (multiples of SPLIT from the first visible key), so what a token computes does not
// depend on the batch it is in.
//
// Sizes: head_dim in {16, 32, 64, 128, 256} (SPLIT = 256, 256, 128, 64, 32: at most 16 KB per tile);
// any number of heads and kv heads; any page size.  The wait for the copies is bounded: if it
// runs out the kernel records a code in `status` and writes nothing.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;
constexpr uint32_t SPIN_LIMIT = 4000000u;

// Keys per block: 16 KB per tile, so that seven CTAs share an SM and a whole decode batch of a
// few thousand blocks is in flight at once.
__host__ __device__ constexpr int split_keys(int head_dim) { return head_dim <= 32 ? 256 : (8192 / head_dim); }

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// partial layout: out [token][head][split][D], ml [token][head][split][2]; counters [token][head]
template <int D>
__global__ void __launch_bounds__(THREADS)
attention_split_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ k_pages,
                       const bf16* __restrict__ v_pages, const int* __restrict__ block_table,
                       const int* __restrict__ token_request, const int* __restrict__ positions,
                       bf16* __restrict__ out, float* __restrict__ part_out, float* __restrict__ part_ml,
                       int* __restrict__ counters, int n_head, int n_kv_head, int page_tokens, int max_pages,
                       int window, int max_splits, float scale_log2e, int* __restrict__ status) {
    constexpr int SPLIT = split_keys(D);
    constexpr int LPK = D / 8;                 // lanes per key row (16 bytes each)
    constexpr int KPW = 32 / LPK;              // keys per warp per round
    extern __shared__ __align__(128) uint8_t tiles[];
    bf16* k_tile = reinterpret_cast<bf16*>(tiles);                       // [SPLIT][D]
    bf16* v_tile = k_tile + SPLIT * D;
    __shared__ float scores[SPLIT];
    __shared__ float red[WARPS];
    __shared__ float acc_smem[WARPS][D];
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ int is_last;

    const int token = blockIdx.x, head = blockIdx.y, split = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Positions, block tables and every cache row but the newest were written before this step
    // began; only the query and the newest key/value row come from the kernel in front.  So the
    // block asks for its old rows right away, while that kernel is still running, and for the
    // newest row (if it holds it) after the wait.
    pdl_trigger();
    const int p = positions[token];
    if (p < 0) {                                                        // padding row of a fixed-size batch
        pdl_wait();                                                     // `out` may still be in use before
        if (split == 0)
            for (int d = tid; d < D; d += THREADS) out[((size_t)token * n_head + head) * D + d] = __float2bfloat16_rn(0.f);
        return;
    }
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int start = lo + split * SPLIT;
    if (start > p) return;                                              // this block holds no key of the token
    const int count = min(SPLIT, p + 1 - start);
    const int splits = (p - lo) / SPLIT + 1;
    const int kv_head = head / (n_head / n_kv_head);
    const int* table = block_table + (size_t)token_request[token] * max_pages;

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bars[0])) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bars[1])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // ---- ask for the keys and values of the block: one bulk copy per page and tensor ----
    const bool holds_newest = start + count - 1 == p;
    if (warp == 0) {
        const uint32_t bytes = (uint32_t)count * D * 2;
        if (lane == 0) {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&bars[0])), "r"(bytes) : "memory");
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&bars[1])), "r"(bytes) : "memory");
        }
        __syncwarp();
        const int old_end = holds_newest ? p : start + count;           // rows [start, old_end) are old
        if (old_end > start) {
            const int first_page = start / page_tokens, last_page = (old_end - 1) / page_tokens;
            for (int which = 0; which < 2; ++which) {                   // all key copies first
                const bf16* pages = which == 0 ? k_pages : v_pages;
                bf16* tile = which == 0 ? k_tile : v_tile;
                for (int pi = first_page + lane; pi <= last_page; pi += 32) {
                    const int page = table[pi];
                    const int r0 = max(start, pi * page_tokens), r1 = min(old_end, (pi + 1) * page_tokens);
                    const size_t row = ((size_t)page * n_kv_head + kv_head) * page_tokens + (r0 - pi * page_tokens);
                    bulk_copy(smem_u32(tile + (size_t)(r0 - start) * D), pages + row * D, (uint32_t)(r1 - r0) * D * 2,
                              smem_u32(&bars[which]));
                }
            }
        }
    }
    pdl_wait();
    if (holds_newest && tid < 2) {                                      // the row the kernel in front wrote
        const int pi = p / page_tokens;
        const size_t row = ((size_t)table[pi] * n_kv_head + kv_head) * page_tokens + (p - pi * page_tokens);
        bulk_copy(smem_u32((tid == 0 ? k_tile : v_tile) + (size_t)(p - start) * D), (tid == 0 ? k_pages : v_pages) + row * D,
                  (uint32_t)D * 2, smem_u32(&bars[tid]));
    }

    const int sub = lane % LPK, grp = lane / LPK;
    // this lane's 8 dims of the query, scaled
    float q[8];
    {
        const int qkv_width = (n_head + 2 * n_kv_head) * D;
        const uint4 raw = *reinterpret_cast<const uint4*>(qkv + (size_t)token * qkv_width + (size_t)head * D + sub * 8);
        unpack8(raw, q);
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] *= scale_log2e;
    }

    // ---- pass 1: scores, once the keys have landed ----
    bool ok = mbar_wait(smem_u32(&bars[0]), 0);
    for (int base = warp * KPW; base < count; base += WARPS * KPW) {
        const int j = base + grp;
        float dot = 0.f;
        if (j < count) {
            float kf[8];
            unpack8(*reinterpret_cast<const uint4*>(k_tile + (size_t)j * D + sub * 8), kf);
#pragma unroll
            for (int i = 0; i < 8; ++i) dot = fmaf(q[i], kf[i], dot);
        }
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (sub == 0 && j < count) scores[j] = dot;
    }
    __syncthreads();

    // ---- pass 2: maximum, exponentials, sum ----
    float m = -INFINITY;
    for (int j = tid; j < count; j += THREADS) m = fmaxf(m, scores[j]);
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    float l = 0.f;
    for (int j = tid; j < count; j += THREADS) {
        const float e = exp2f(scores[j] - m);
        scores[j] = e;
        l += e;
    }
    l = warp_sum(l);
    if (lane == 0) red[warp] = l;
    __syncthreads();
    l = red[0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) l += red[w];

    // ---- pass 3: sum of p * v, once the values have landed ----
    ok = mbar_wait(smem_u32(&bars[1]), 0) && ok;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int base = warp * KPW; base < count; base += WARPS * KPW) {
        const int j = base + grp;
        if (j < count) {
            float vf[8];
            unpack8(*reinterpret_cast<const uint4*>(v_tile + (size_t)j * D + sub * 8), vf);
            const float pj = scores[j];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(pj, vf[i], acc[i]);
        }
    }
    // lanes with the same `sub` hold the same dims: add them up inside the warp, then across warps
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
    }
    if (grp == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc_smem[warp][sub * 8 + i] = acc[i];
    }
    ok = __syncthreads_and(ok);
    if (!ok) {
        // the copies never arrived: report, give them a moment, leave without writing anything
        if (tid == 0) {
            atomicExch(status, 11);
            for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
        __syncthreads();
        return;
    }
    const size_t pair = (size_t)token * n_head + head;
    const size_t slot = pair * max_splits + split;
    if (splits == 1) {                                                  // nothing to merge
        const float inv = 1.0f / l;
        for (int d = tid; d < D; d += THREADS) {
            float v = acc_smem[0][d];
#pragma unroll
            for (int w = 1; w < WARPS; ++w) v += acc_smem[w][d];
            out[pair * D + d] = __float2bfloat16_rn(v * inv);
        }
        return;
    }
    for (int d = tid; d < D; d += THREADS) {
        float v = acc_smem[0][d];
#pragma unroll
        for (int w = 1; w < WARPS; ++w) v += acc_smem[w][d];
        part_out[slot * D + d] = v;
    }
    if (tid == 0) {
        part_ml[slot * 2] = m;
        part_ml[slot * 2 + 1] = l;
    }
    // ---- the CTA that finishes last merges the blocks of this (token, head) ----
    // The barrier orders every thread's partial writes before thread 0's release on the counter;
    // the CTA that reads the final count acquires, so it sees the partial rows of all blocks.
    __syncthreads();
    if (tid == 0) {
        int done;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(done) : "l"(counters + pair) : "memory");
        is_last = (done == splits - 1);
        if (is_last) counters[pair] = 0;                                // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    // Merge with all loads in flight at once: one thread per block fetches its maximum and sum,
    // then each thread adds up its share of the partial rows, eight loads at a time.
    const size_t base = pair * max_splits;
    float* ml = scores;                                                 // reuse: [splits] weights
    float M = -INFINITY;
    for (int s0 = 0; s0 < splits; s0 += THREADS) {
        const int s = s0 + tid;
        if (s < splits) M = fmaxf(M, __ldcg(&part_ml[(base + s) * 2]));
    }
    M = warp_max(M);
    if (lane == 0) red[warp] = M;
    __syncthreads();
    M = red[0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) M = fmaxf(M, red[w]);
    __syncthreads();
    float denom = 0.f;
    for (int s0 = 0; s0 < splits; s0 += THREADS) {
        const int s = s0 + tid;
        if (s < splits) {
            const float w = exp2f(__ldcg(&part_ml[(base + s) * 2]) - M);
            if (s < SPLIT) ml[s] = w;
            denom += w * __ldcg(&part_ml[(base + s) * 2 + 1]);
        }
    }
    denom = warp_sum(denom);
    if (lane == 0) red[warp] = denom;
    __syncthreads();
    denom = red[0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) denom += red[w];
    const float inv = 1.0f / denom;
    for (int d = tid; d < D; d += THREADS) {
        float v = 0.f;
        for (int s0 = 0; s0 < splits; s0 += 8) {                        // blocks in order, 8 loads in flight
            float x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) x[u] = (s0 + u < splits) ? __ldcg(&part_out[(base + s0 + u) * D + d]) : 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (s0 + u < splits) {
                    const int s = s0 + u;
                    const float w = s < SPLIT ? ml[s] : exp2f(__ldcg(&part_ml[(base + s) * 2]) - M);
                    v = fmaf(w, x[u], v);
                }
        }
        out[pair * D + d] = __float2bfloat16_rn(v * inv);
    }
}

template <int D>
int launch(const void* qkv, const void* k_pages, const void* v_pages, const int* block_table,
           const int* token_request, const int* positions, void* out, float* part_out, float* part_ml,
           int* counters, int n_tokens, int n_head, int n_kv_head, int page_tokens, int max_pages, int window,
           int max_splits, float scale, int* status, cudaStream_t s) {
    constexpr size_t smem = (size_t)2 * split_keys(D) * D * sizeof(bf16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_split_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "attention (split): cannot raise shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(n_tokens, n_head, max_splits);
    cudaError_t le = mg_launch(attention_split_kernel<D>, grid, dim3(THREADS), smem, s, true, (const bf16*)qkv,
                               (const bf16*)k_pages, (const bf16*)v_pages, block_table, token_request, positions,
                               (bf16*)out, part_out, part_ml, counters, n_head, n_kv_head, page_tokens, max_pages,
                               window, max_splits, scale * 1.4426950408889634f, status);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "attention_split: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("attention_split");
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

// Floats of scratch the split kernel needs (partial outputs, then maxima and sums).
MG_API long long mg_attention_split_scratch_floats(int n_tokens, int n_head, int head_dim, int max_splits) {
    return (long long)n_tokens * n_head * max_splits * (head_dim + 2);
}

// One query token per row (a row with position < 0 is padding: its output is zeros).
// qkv / pages / out as mg_paged_attention_generic, bfloat16 only.  `scratch` holds
// mg_attention_split_scratch_floats() floats and need not be initialised; `counters` holds
// n_tokens * n_head ints that are ZERO before the first launch (the kernel leaves them zero);
// `max_splits` = mg_attention_split_count() of the longest context; `status` receives a
// non-zero code if a wait ran out.  Launches that share scratch or counters must not overlap.
MG_API int mg_paged_attention_split(const void* qkv, const void* k_pages, const void* v_pages,
                                    const int* block_table, const int* token_request, const int* positions,
                                    void* out, float* scratch, int* counters, int n_tokens, int n_head,
                                    int n_kv_head, int head_dim, int page_tokens, int max_pages, int window,
                                    int max_splits, float scale, int* status, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && n_kv_head > 0 && page_tokens > 0 && max_pages > 0 && max_splits > 0,
               "attention (split): bad sizes");
    MG_REQUIRE(n_head % n_kv_head == 0, "attention: n_head %d is not a multiple of n_kv_head %d", n_head, n_kv_head);
    MG_REQUIRE(n_head <= 65535 && max_splits <= 65535, "attention (split): too many heads or key blocks");
    MG_REQUIRE(scratch != nullptr && counters != nullptr && status != nullptr, "attention (split): missing scratch");
    cudaStream_t s = (cudaStream_t)stream;
    float* part_out = scratch;
    float* part_ml = scratch + (size_t)n_tokens * n_head * max_splits * head_dim;
#define MG_SPLIT_CASE(DIM)                                                                                        \
    case DIM:                                                                                                     \
        return launch<DIM>(qkv, k_pages, v_pages, block_table, token_request, positions, out, part_out, part_ml, \
                           counters, n_tokens, n_head, n_kv_head, page_tokens, max_pages, window, max_splits,    \
                           scale, status, s)
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
