// Projection of a few dozen tokens (decoding at batch 17 to 128): out[m, n] = x[m, :] . w[n, :].
//
// At this size a projection is still a stream over the weights, but the activations are no
// longer small: 64 tokens of width 2048 are 256 KB, too much for every CTA to stage whole, and a
// 128-row tensor-core tile leaves a 512-row matrix on 4 SMs.  So K is cut across the CTAs of a
// thread-block cluster: the CTA of rank r stages only columns of its K slice (1/8 of the
// activations), its 8 warps each take another tile of 8 weight rows, and a lane asks for all
// its weights (16 bytes per row and k block) before it waits for the kernel in front.  The sums
// run on warp-level mma (m16n8k16, tokens as the 16 rows of A, weight rows as the 8 columns of
// B; see linear_skinny.cu for how one 16-byte load feeds two mma's).  The partial sums of the K
// slices meet through distributed shared memory: every warp stores its tile's partial sums into
// the shared memory of the CTA that finishes that tile; after one cluster barrier that CTA adds
// them up in rank order from its own memory and applies the epilogue.
//
// Every output element sums its K terms in a fixed order (k blocks in order inside a slice,
// slices in rank order), independent of M and of the other rows.  K must be a multiple of 8.
#include <cooperative_groups.h>

#include "linear_epilogue.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int MAX_M = 128;
constexpr int TILE_N = 8;            // weight rows per warp
constexpr int WARPS = 8;             // tiles per cluster
constexpr int THREADS = WARPS * 32;

struct ClusterArgs {
    const bf16* x;                   // [M, K]
    const bf16* w;                   // [N, K]
    LinearEpilogue ep;
    int K;
    int ranks;                       // CTAs per cluster = K slices
    int per_rank;                    // k blocks per slice
    int xstride;                     // bytes between staged activation rows
};

// MG: groups of 16 tokens held: 2, 4, 6 or 8.  NTW: tiles of 8 weight rows per warp (2 for matrices of
// so many rows that one tile per warp would need several rounds of CTAs: half the CTAs, and a
// fragment of the activations feeds two tiles).
template <int MG, int NTW>
__global__ void __launch_bounds__(THREADS, 2) linear_cluster_kernel(const ClusterArgs a) {
    constexpr int MT = MG * 16;
    constexpr int CTILES = WARPS * NTW;                                            // tiles per cluster
    // k blocks (of 32) whose weights a lane holds at once: fewer where the sums take more registers,
    // so that two CTAs still share an SM
    constexpr int PRE = (MG <= 4 ? 8 : 4) / NTW;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int ranks = a.ranks;
    const int cluster_id = blockIdx.x / ranks;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint8_t* xs = smem_raw;                                                        // [MT][xstride]
    float* part = reinterpret_cast<float*>(smem_raw + (size_t)MT * a.xstride);     // [CTILES][MT][8]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int K = a.K, N = a.ep.N, M = a.ep.M;
    const int kblocks = (K + 31) / 32;
    const int b_begin = min(kblocks, rank * a.per_rank), b_end = min(kblocks, b_begin + a.per_rank);
    const int total_tiles = (N + TILE_N - 1) / TILE_N;
    const int tile0 = cluster_id * CTILES + warp * NTW;                            // this warp's first tile
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

    // this warp's weights first: they travel while the kernel in front drains
    const bf16* wrow[NTW];
    bool live[NTW];
    uint4 first_w[NTW][PRE];
#pragma unroll
    for (int h = 0; h < NTW; ++h) {
        live[h] = tile0 + h < total_tiles;
        wrow[h] = a.w + (size_t)min((tile0 + h) * TILE_N + g, N - 1) * K;
#pragma unroll
        for (int i = 0; i < PRE; ++i) {
            const int k = (b_begin + i) * 32 + 8 * t;
            first_w[h][i] = (live[h] && b_begin + i < b_end && k < K) ? *reinterpret_cast<const uint4*>(wrow[h] + k) : zero4;
        }
    }
    // the first result this thread will finish (tile `rank` of the cluster), and its bias
    const int e_m = tid / TILE_N, e_n = (cluster_id * CTILES + rank) * TILE_N + tid % TILE_N;
    const bool e_live = rank < CTILES && e_m < M && e_n < N;
    float e_bias = (e_live && a.ep.bias) ? a.ep.bias[e_n] : 0.f;
    // for the QKV projection, the cache rows of the tokens this thread finishes (inputs of the step)
    int e_slot[MT * TILE_N / THREADS];
#pragma unroll
    for (int j = 0; j < MT * TILE_N / THREADS; ++j) {
        const int m = e_m + j * (THREADS / TILE_N);
        e_slot[j] = (a.ep.k_pages != nullptr && m < M) ? a.ep.slots[m] : -1;
    }
    pdl_trigger();
    pdl_wait();
    float e_res = 0.f;
    if (e_live && a.ep.epilogue == EPI_RESIDUAL) e_res = a.ep.residual[(size_t)e_m * N + e_n];

    // ---- stage this slice of the activations; rows at and past M stay as they are ----
    {
        const int pieces = (b_end - b_begin) * 4;                                  // 16-byte pieces per row
        const int k0 = b_begin * 32;
        // (a thread asks for four pieces before it stores the first: one trip to L2 for 4 x THREADS pieces)
        for (int i0 = tid; i0 < M * pieces; i0 += 4 * THREADS) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * THREADS;
                const int m = i / pieces, pc = i - m * pieces;
                const int k = k0 + pc * 8;
                v[u] = (i < M * pieces && k < K) ? *reinterpret_cast<const uint4*>(a.x + (size_t)m * K + k) : zero4;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * THREADS;
                if (i < M * pieces) {
                    const int m = i / pieces, pc = i - m * pieces;
                    *reinterpret_cast<uint4*>(xs + (size_t)m * a.xstride + pc * 16) = v[u];
                }
            }
        }
    }
    __syncthreads();

    float c[NTW][MG][4];
#pragma unroll
    for (int h = 0; h < NTW; ++h)
#pragma unroll
        for (int mg = 0; mg < MG; ++mg)
#pragma unroll
            for (int i = 0; i < 4; ++i) c[h][mg][i] = 0.f;
    if (live[0]) {                                                                 // (a warp's tiles are live from the first on)
        for (int b0 = b_begin; b0 < b_end; b0 += PRE) {
            uint4 wv[NTW][PRE];
#pragma unroll
            for (int h = 0; h < NTW; ++h) {
                if (b0 == b_begin) {
#pragma unroll
                    for (int i = 0; i < PRE; ++i) wv[h][i] = first_w[h][i];
                } else {
#pragma unroll
                    for (int i = 0; i < PRE; ++i) {
                        const int k = (b0 + i) * 32 + 8 * t;
                        wv[h][i] = (live[h] && b0 + i < b_end && k < K) ? *reinterpret_cast<const uint4*>(wrow[h] + k) : zero4;
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < PRE; ++i) {
                if (b0 + i < b_end) {                                              // uniform in the warp
                    const int off = ((b0 + i - b_begin) * 32 + 8 * t) * 2;
#pragma unroll
                    for (int mg = 0; mg < MG; ++mg) {
                        const uint4 x0 = *reinterpret_cast<const uint4*>(xs + (size_t)(mg * 16 + g) * a.xstride + off);
                        const uint4 x1 = *reinterpret_cast<const uint4*>(xs + (size_t)(mg * 16 + g + 8) * a.xstride + off);
#pragma unroll
                        for (int h = 0; h < NTW; ++h) {
                            mma_bf16(c[h][mg], x0.x, x1.x, x0.y, x1.y, wv[h][i].x, wv[h][i].y);
                            mma_bf16(c[h][mg], x0.z, x1.z, x0.w, x1.w, wv[h][i].z, wv[h][i].w);
                        }
                    }
                }
            }
        }
    }
    // c0, c1: token 16 mg + g, rows 2t and 2t+1 of the tile; c2, c3: token 16 mg + g + 8.
    // The partial sums of a tile go straight into the shared memory of the CTA that finishes that
    // tile (rank tile % ranks), into the row of this rank: [slot][source rank][MT][8].
#pragma unroll
    for (int h = 0; h < NTW; ++h) {
        const int tl = warp * NTW + h;                                             // the tile's number in the cluster
        float* theirs = cluster.map_shared_rank(part, tl % ranks) + ((size_t)(tl / ranks) * ranks + rank) * MT * TILE_N;
#pragma unroll
        for (int mg = 0; mg < MG; ++mg) {
            *reinterpret_cast<float2*>(theirs + (mg * 16 + g) * TILE_N + 2 * t) = make_float2(c[h][mg][0], c[h][mg][1]);
            *reinterpret_cast<float2*>(theirs + (mg * 16 + g + 8) * TILE_N + 2 * t) = make_float2(c[h][mg][2], c[h][mg][3]);
        }
    }
    cluster.sync();                                    // all partial sums have arrived; nothing remote is touched after this
    // ---- the CTA of rank r finishes tiles r, r + ranks, ...: slices added in rank order ----
    for (int slot = 0; slot * ranks + rank < CTILES; ++slot) {
        const int tl = slot * ranks + rank;
        const int out_tile = cluster_id * CTILES + tl;
        if (out_tile >= total_tiles) break;
#pragma unroll
        for (int j = 0; j < MT * TILE_N / THREADS; ++j) {
            const int e = tid + j * THREADS;
            const int m = e / TILE_N, r = e - m * TILE_N;
            const int n = out_tile * TILE_N + r;
            if (m >= M || n >= N) continue;
            float v = 0.f;
            for (int s = 0; s < ranks; ++s) v += part[((size_t)(slot * ranks + s) * MT + m) * TILE_N + r];
            const bool first = slot == 0 && j == 0;
            if (a.ep.bias) v += first ? e_bias : a.ep.bias[n];
            linear_finish(a.ep, m, n, v, first, e_res, true, e_slot[j]);
        }
    }
}

}  // namespace

// Largest M this kernel takes.
MG_API int mg_linear_cluster_max_rows() { return MAX_M; }

MG_GUARD_EXPORT(linear_cluster, linear_index_fault)

// x: [M, K] bf16; w: [N, K] bf16; epilogues and the key/value sink as mg_linear_skinny.
// Returns MG_ERR_UNSUPPORTED (nothing launched) for M > 128, K % 8 != 0, operands that are not
// 16-byte aligned or a slice of activations beyond the shared memory.
MG_API int mg_linear_cluster(const void* x, const void* w, const float* bias, void* out, float* residual, int M, int N,
                             int K, int epilogue, int out_bf16, void* k_pages, void* v_pages, const int* slots,
                             int q_width, int n_kv_head, int head_dim, int page_tokens, int num_pages, void* stream) {
    if (M == 0) return MG_OK;
    MG_REQUIRE(M > 0 && N > 0 && K > 0 && x != nullptr && w != nullptr, "linear: bad arguments M=%d N=%d K=%d", M, N, K);
    MG_REQUIRE(epilogue == EPI_RESIDUAL ? residual != nullptr : out != nullptr, "linear: missing output");
    MG_REQUIRE(k_pages == nullptr || (out_bf16 && epilogue == EPI_STORE && slots && v_pages && head_dim > 0 &&
                                      n_kv_head > 0 && page_tokens > 0 && N == q_width + 2 * n_kv_head * head_dim),
               "linear: bad key/value sink");
    const int kblocks = (K + 31) / 32;
    int ranks = 1;
    while (ranks < 8 && (kblocks + ranks * 2 - 1) / (ranks * 2) >= 2) ranks *= 2;      // at least two k blocks per slice
    const int per_rank = (kblocks + ranks - 1) / ranks;
    const int slice_bytes = per_rank * 64;
    const int xstride = slice_bytes + (slice_bytes % 128 == 0 ? 64 : 0);               // rows 64 bytes apart mod 128
    const int mg = M <= 32 ? 2 : M <= 64 ? 4 : M <= 96 ? 6 : 8;
    const int tiles = (N + TILE_N - 1) / TILE_N;
    // two tiles per warp where one would make more CTAs than two rounds of them hold (up to 64 tokens:
    // beyond, the sums of two tiles do not fit the registers beside two CTAs per SM)
    const int ntw = (mg <= 4 && (long long)((tiles + WARPS - 1) / WARPS) * ranks > 2 * 296) ? 2 : 1;
    const size_t smem = (size_t)mg * 16 * xstride + (size_t)WARPS * ntw * mg * 16 * TILE_N * sizeof(float);
    if (M > MAX_M || K % 8 != 0 || smem > 200 * 1024 || ((uintptr_t)w & 15) || ((uintptr_t)x & 15))
        return mg_set_error(MG_ERR_UNSUPPORTED, "linear (cluster): needs M <= 128, K %% 8 == 0, aligned operands");
    ClusterArgs a;
    a.x = (const bf16*)x; a.w = (const bf16*)w; a.K = K; a.ranks = ranks; a.per_rank = per_rank; a.xstride = xstride;
    a.ep.bias = bias; a.ep.out = out; a.ep.residual = residual; a.ep.M = M; a.ep.N = N;
    a.ep.epilogue = epilogue; a.ep.out_bf16 = out_bf16;
    a.ep.k_pages = (bf16*)k_pages; a.ep.v_pages = (bf16*)v_pages; a.ep.slots = slots;
    a.ep.q_width = q_width; a.ep.n_kv_head = n_kv_head; a.ep.head_dim = head_dim; a.ep.page_tokens = page_tokens; a.ep.num_pages = num_pages;
    void (*kernel)(const ClusterArgs) = nullptr;
    if (ntw == 2) kernel = mg == 2 ? linear_cluster_kernel<2, 2> : linear_cluster_kernel<4, 2>;
    else kernel = mg == 2 ? linear_cluster_kernel<2, 1> : mg == 4 ? linear_cluster_kernel<4, 1>
                  : mg == 6 ? linear_cluster_kernel<6, 1> : linear_cluster_kernel<8, 1>;
    {
        // (once per variant: the attribute is cheap to set again)
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "linear (cluster): cannot raise shared memory: %s", cudaGetErrorString(e));
    }
    const int clusters = (tiles + WARPS * ntw - 1) / (WARPS * ntw);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)clusters * ranks);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ranks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.numAttrs = 1;
    if (mg_dependent_launch_enabled()) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    cfg.attrs = attr;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, kernel, a);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "linear_cluster: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("linear_cluster");
    return MG_OK;
}
