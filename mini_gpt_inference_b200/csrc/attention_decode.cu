// Attention of single query tokens over the paged cache, split along the keys (bfloat16 cache).
//
// A decoding step reads every key and value of every live request once: it is bound by HBM
// bandwidth, and a request alone gives too little parallelism (one head is one row of work).
// So the keys of a (token, head) are cut into blocks of SPLIT_KEYS positions, one CTA each:
//
//   pass 1  scores of the block: a key row (head_dim bf16) is read by head_dim / 8 neighbouring
//           lanes with one 16-byte load each, so a warp reads whole 512-byte lines; the dot
//           product is finished with shuffles;
//   pass 2  the block's maximum and the exponentials (base 2; the query is pre-scaled by
//           scale * log2 e), all in 32-bit;
//   pass 3  sum of p * v with the same 16-byte pattern over the value rows.
//
// Each CTA writes its unnormalised output, its maximum and its sum to scratch memory;
// a second kernel merges the blocks of a (token, head).  Block edges are absolute positions
// (multiples of SPLIT_KEYS from the first visible key), so what a token computes does not
// depend on the batch it is in.  Scores, maxima, sums and outputs accumulate in 32-bit.
//
// Sizes: head_dim in {16, 32, 64, 128, 256}; any number of heads and kv heads; any page size.
// Other head sizes are refused here (the general kernel takes them).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int SPLIT_KEYS = 256;
constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;
constexpr int UNROLL = 4;

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}

// partial layout: out [token][head][split][D], ml [token][head][split][2]
template <int D>
__global__ void __launch_bounds__(THREADS)
attention_split_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ k_pages,
                       const bf16* __restrict__ v_pages, const int* __restrict__ block_table,
                       const int* __restrict__ token_request, const int* __restrict__ positions,
                       float* __restrict__ part_out, float* __restrict__ part_ml, int n_head, int n_kv_head,
                       int page_tokens, int max_pages, int window, int max_splits, float scale_log2e) {
    constexpr int LPK = D / 8;                 // lanes per key row (16 bytes each)
    constexpr int KPW = 32 / LPK;              // keys per warp per round
    __shared__ float scores[SPLIT_KEYS];
    __shared__ float red[WARPS];
    __shared__ float acc_smem[WARPS][D];

    const int token = blockIdx.x, head = blockIdx.y, split = blockIdx.z;
    const int p = positions[token];
    if (p < 0) return;                                                  // padding row of a fixed-size batch
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int start = lo + split * SPLIT_KEYS;
    if (start > p) return;                                              // this block holds no key of the token
    const int count = min(SPLIT_KEYS, p + 1 - start);
    const int kv_head = head / (n_head / n_kv_head);
    const int* table = block_table + (size_t)token_request[token] * max_pages;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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

    // ---- pass 1: scores ----  (UNROLL independent 16-byte loads per lane are in flight at once)
    for (int base = warp * KPW; base < count; base += WARPS * KPW * UNROLL) {
        uint4 raw[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int j = base + u * WARPS * KPW + grp;
            raw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (j < count) {
                const int pos = start + j;
                const int page = table[pos / page_tokens];
                const size_t row = ((size_t)page * n_kv_head + kv_head) * page_tokens + (pos % page_tokens);
                raw[u] = *reinterpret_cast<const uint4*>(k_pages + row * D + sub * 8);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int j = base + u * WARPS * KPW + grp;
            float kf[8];
            unpack8(raw[u], kf);
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) dot = fmaf(q[i], kf[i], dot);
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (sub == 0 && j < count) scores[j] = dot;
        }
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

    // ---- pass 3: sum of p * v ----
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int base = warp * KPW; base < count; base += WARPS * KPW * UNROLL) {
        uint4 raw[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int j = base + u * WARPS * KPW + grp;
            raw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (j < count) {
                const int pos = start + j;
                const int page = table[pos / page_tokens];
                const size_t row = ((size_t)page * n_kv_head + kv_head) * page_tokens + (pos % page_tokens);
                raw[u] = *reinterpret_cast<const uint4*>(v_pages + row * D + sub * 8);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int j = base + u * WARPS * KPW + grp;
            float vf[8];
            unpack8(raw[u], vf);
            const float pj = j < count ? scores[j] : 0.f;
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
    __syncthreads();
    const size_t slot = ((size_t)token * n_head + head) * max_splits + split;
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
}

// Merge the blocks of each (token, head): out = sum_s 2^(m_s - M) acc_s / sum_s 2^(m_s - M) l_s.
template <int D>
__global__ void attention_merge_kernel(const float* __restrict__ part_out, const float* __restrict__ part_ml,
                                       const int* __restrict__ positions, bf16* __restrict__ out, int n_head,
                                       int window, int max_splits) {
    const int token = blockIdx.x, head = blockIdx.y;
    const int p = positions[token];
    if (p < 0) {                                                        // padding row: zeros
        for (int d = threadIdx.x; d < D; d += blockDim.x)
            out[((size_t)token * n_head + head) * D + d] = __float2bfloat16_rn(0.f);
        return;
    }
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int splits = (p - lo) / SPLIT_KEYS + 1;
    const size_t base = ((size_t)token * n_head + head) * max_splits;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
    float denom = 0.f;
    for (int s = 0; s < splits; ++s) denom += exp2f(part_ml[(base + s) * 2] - M) * part_ml[(base + s) * 2 + 1];
    const float inv = 1.0f / denom;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; ++s) v += exp2f(part_ml[(base + s) * 2] - M) * part_out[(base + s) * D + d];
        out[((size_t)token * n_head + head) * D + d] = __float2bfloat16_rn(v * inv);
    }
}

template <int D>
int launch(const void* qkv, const void* k_pages, const void* v_pages, const int* block_table,
           const int* token_request, const int* positions, void* out, float* part_out, float* part_ml,
           int n_tokens, int n_head, int n_kv_head, int page_tokens, int max_pages, int window, int max_splits,
           float scale, cudaStream_t s) {
    dim3 grid(n_tokens, n_head, max_splits);
    attention_split_kernel<D><<<grid, THREADS, 0, s>>>(
        (const bf16*)qkv, (const bf16*)k_pages, (const bf16*)v_pages, block_table, token_request, positions, part_out,
        part_ml, n_head, n_kv_head, page_tokens, max_pages, window, max_splits, scale * 1.4426950408889634f);
    MG_CHECK_LAUNCH("attention_split");
    attention_merge_kernel<D><<<dim3(n_tokens, n_head), D < 64 ? 32 : 64, 0, s>>>(part_out, part_ml, positions, (bf16*)out,
                                                                         n_head, window, max_splits);
    MG_CHECK_LAUNCH("attention_merge");
    return MG_OK;
}

}  // namespace

// Number of key blocks a context of `max_context` positions can have (with a window, at most
// the window's length counts).
MG_API int mg_attention_split_count(int max_context, int window) {
    int span = (window > 0 && window < max_context) ? window : max_context;
    if (span < 1) span = 1;
    return (span - 1) / SPLIT_KEYS + 1;
}

// Floats of scratch the split kernel needs: part_out then part_ml.
MG_API long long mg_attention_split_scratch_floats(int n_tokens, int n_head, int head_dim, int max_splits) {
    return (long long)n_tokens * n_head * max_splits * (head_dim + 2);
}

// One query token per row (any row may be a padding row with position < 0, which is skipped).
// qkv / pages / out as mg_paged_attention_generic, bfloat16 only.  `scratch` holds
// mg_attention_split_scratch_floats() floats; `max_splits` covers the longest context.
MG_API int mg_paged_attention_split(const void* qkv, const void* k_pages, const void* v_pages,
                                    const int* block_table, const int* token_request, const int* positions,
                                    void* out, float* scratch, int n_tokens, int n_head, int n_kv_head,
                                    int head_dim, int page_tokens, int max_pages, int window, int max_splits,
                                    float scale, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && n_kv_head > 0 && page_tokens > 0 && max_pages > 0 && max_splits > 0,
               "attention (split): bad sizes");
    MG_REQUIRE(n_head % n_kv_head == 0, "attention: n_head %d is not a multiple of n_kv_head %d", n_head, n_kv_head);
    MG_REQUIRE(n_head <= 65535 && max_splits <= 65535, "attention (split): too many heads or key blocks");
    MG_REQUIRE(scratch != nullptr, "attention (split): missing scratch");
    cudaStream_t s = (cudaStream_t)stream;
    float* part_out = scratch;
    float* part_ml = scratch + (size_t)n_tokens * n_head * max_splits * head_dim;
#define MG_SPLIT_CASE(DIM)                                                                                          \
    case DIM:                                                                                                       \
        return launch<DIM>(qkv, k_pages, v_pages, block_table, token_request, positions, out, part_out, part_ml,   \
                           n_tokens, n_head, n_kv_head, page_tokens, max_pages, window, max_splits, scale, s)
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
