// Causal attention of a ragged batch over the paged cache; the general kernel.
//
// One warp per (token, head).  The token's query attends to the keys of its own request at
// positions lo..p, p being the token's own position and lo = max(0, p - window + 1) (0
// without a window), all read from the request's pages: the keys of this step were written
// there before the launch.  Scores, the running maximum, the running sum and the output
// accumulate in 32-bit; keys are visited in blocks of 32 starting at lo, so the result of a
// (token, head) pair is the same in whichever step and batch it is computed.
//
// Any head_dim up to 256 and any number of heads and kv heads (n_head a multiple of
// n_kv_head) are accepted.  Entries of the block table are read only for positions lo..p, so
// stale or missing pages elsewhere never matter.
#include <math.h>

#include "common.cuh"

MG_GUARD_DECLARE(attention_generic)

namespace {

constexpr int WARPS = 4;
constexpr int MAX_DPL = 8;   // head_dim <= 256: at most 8 dims per lane

template <typename T>
__global__ void __launch_bounds__(32 * WARPS)
paged_attention_generic_kernel(const T* __restrict__ qkv, const T* __restrict__ k_pages,
                               const T* __restrict__ v_pages, const int* __restrict__ block_table,
                               const int* __restrict__ token_request, const int* __restrict__ positions,
                               T* __restrict__ out, int n_tokens, int n_head, int n_kv_head, int head_dim,
                               int page_tokens, int max_pages, int window, float scale, int num_pages,
                               int n_requests) {
    extern __shared__ float q_smem[];                     // [WARPS][head_dim]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int token = blockIdx.x;
    const int head = blockIdx.y * WARPS + warp;
    if (head >= n_head) return;                            // whole warp leaves together
    const int kv_head = head / (n_head / n_kv_head);
    const int qkv_width = (n_head + 2 * n_kv_head) * head_dim;
    int p = positions[token];
    if (p < 0) {                                           // padding row of a fixed-size batch
        T* pad = out + (size_t)token * n_head * head_dim + (size_t)head * head_dim;
        for (int d = lane; d < head_dim; d += 32) pad[d] = from_float<T>(0.f);
        return;
    }
    // (guarded builds: a position beyond the block table, a request beyond its rows or a page beyond
    // the pool is recorded, and position 0, request 0 or page 0 is read in its place)
    if (!MG_GUARDED(attention_generic, MG_GUARD_POSITION, p, (long long)max_pages * page_tokens)) p = 0;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    int request = token_request[token];
    if (!MG_GUARDED(attention_generic, MG_GUARD_REQUEST, request, n_requests)) request = 0;
    const int* table = block_table + (size_t)request * max_pages;

    float* q = q_smem + warp * head_dim;
    const T* qrow = qkv + (size_t)token * qkv_width + (size_t)head * head_dim;
    for (int d = lane; d < head_dim; d += 32) q[d] = to_float(qrow[d]) * scale;
    __syncwarp();

    float acc[MAX_DPL];
#pragma unroll
    for (int i = 0; i < MAX_DPL; ++i) acc[i] = 0.f;
    float run_max = -INFINITY, run_sum = 0.f;

    for (int j0 = lo; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= p;
        int row = 0;                                       // row of key j in the page storage
        float s = -INFINITY;
        if (valid) {
            int page = table[j / page_tokens];
            if (!MG_GUARDED(attention_generic, MG_GUARD_PAGE, page, num_pages)) page = 0;
            row = (page * n_kv_head + kv_head) * page_tokens + (j % page_tokens);
            const T* kr = k_pages + (size_t)row * head_dim;
            float dot = 0.f;
            for (int d = 0; d < head_dim; ++d) dot = fmaf(q[d], to_float(kr[d]), dot);
            s = dot;
        }
        const float new_max = fmaxf(run_max, warp_max(s));
        const float prob = valid ? expf(s - new_max) : 0.f;
        const float corr = expf(run_max - new_max);       // 0 in the first block (run_max = -inf)
        run_sum = run_sum * corr + warp_sum(prob);
        run_max = new_max;
#pragma unroll
        for (int i = 0; i < MAX_DPL; ++i) acc[i] *= corr;
        const int count = min(32, p - j0 + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, prob, jj);
            const int rj = __shfl_sync(0xffffffffu, row, jj);
            const T* vr = v_pages + (size_t)rj * head_dim;
#pragma unroll
            for (int i = 0; i < MAX_DPL; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
            }
        }
    }
    const float inv = 1.0f / run_sum;
    T* orow = out + (size_t)token * n_head * head_dim + (size_t)head * head_dim;
#pragma unroll
    for (int i = 0; i < MAX_DPL; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) orow[d] = from_float<T>(acc[i] * inv);
    }
}

}  // namespace

// qkv: [n_tokens, (n_head + 2 n_kv_head) * head_dim]; pages: [page, kv head, page_tokens, head_dim];
// block_table: [n_requests, max_pages]; out: [n_tokens, n_head * head_dim].  window <= 0: none.
// num_pages: pages of the pool (with n_requests, what guarded builds hold the indices against).
MG_API int mg_paged_attention_generic(const void* qkv, const void* k_pages, const void* v_pages,
                                      const int* block_table, const int* token_request,
                                      const int* positions, void* out, int n_tokens, int n_head,
                                      int n_kv_head, int head_dim, int page_tokens, int max_pages,
                                      int window, float scale, int num_pages, int n_requests, int is_bf16,
                                      void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && n_kv_head > 0 && page_tokens > 0 && max_pages > 0,
               "attention: bad sizes");
    MG_REQUIRE(n_head % n_kv_head == 0, "attention: n_head %d is not a multiple of n_kv_head %d", n_head, n_kv_head);
    MG_REQUIRE(head_dim > 0 && head_dim <= 32 * MAX_DPL, "attention: head_dim %d is outside 1..%d", head_dim, 32 * MAX_DPL);
    MG_REQUIRE(ceil_div(n_head, WARPS) <= 65535, "attention: too many heads");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, ceil_div(n_head, WARPS)), block(32 * WARPS);
    const size_t smem = (size_t)WARPS * head_dim * sizeof(float);
    if (is_bf16)
        paged_attention_generic_kernel<bf16><<<grid, block, smem, s>>>(
            (const bf16*)qkv, (const bf16*)k_pages, (const bf16*)v_pages, block_table, token_request, positions,
            (bf16*)out, n_tokens, n_head, n_kv_head, head_dim, page_tokens, max_pages, window, scale, num_pages, n_requests);
    else
        paged_attention_generic_kernel<float><<<grid, block, smem, s>>>(
            (const float*)qkv, (const float*)k_pages, (const float*)v_pages, block_table, token_request, positions,
            (float*)out, n_tokens, n_head, n_kv_head, head_dim, page_tokens, max_pages, window, scale, num_pages, n_requests);
    MG_CHECK_LAUNCH("paged_attention_generic");
    return MG_OK;
}
