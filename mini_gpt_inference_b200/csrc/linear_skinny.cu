// Projection of a handful of tokens (decoding at small batch): out[m, n] = x[m, :] . w[n, :].
//
// With up to 16 tokens a projection is a stream over the weights: every weight is read once,
// far below what a 128-row tensor-core tile needs, and such tiles would leave most SMs idle on a
// 512- or 1536-row matrix.  Here the work is cut finely: a warp task is 8 weight rows times one
// slice of K, a CTA of 8 warps takes a few such tasks, so that a 512 x 2048 matrix still spreads
// over 64 CTAs, and each lane asks for all its weights (16-byte loads) before it waits for the
// kernel in front of it.
//
// The sums run on the tensor cores through warp-level mma (m16n8k16, bfloat16 in, 32-bit
// accumulate): the 16 rows of the A operand are the tokens, the 8 columns of B are weight rows.
// A lane's 16-byte load of weights (8 consecutive k of one row) feeds two mma's; which of the
// sixteen k slots of an mma a value takes is free as long as A and B agree, so the activations
// are read from shared memory with the same 16-byte pattern and no shuffle is needed.  What is
// left of the old cost (unpacking, 256 multiply-adds and a 32-lane reduction per lane) is two
// instructions; the K slices of a tile are added up in order through shared memory.
//
// Fused around the product, because at this size every extra kernel costs more than its work:
//   * prologue: LayerNorm of the 32-bit residual rows (optionally gathered through an index),
//     statistics in 32-bit, result rounded to bfloat16 exactly as the stand-alone kernel does;
//   * epilogue: bias, tanh-GELU, bfloat16 or 32-bit store, or add into the 32-bit residual;
//   * epilogue of the QKV projection: key and value features also go to their cache pages.
//
// Every output element sums its K terms in a fixed order (k blocks in order inside a slice,
// slices in order), independent of M and of the other rows.  K must be a multiple of 8 and the
// activations must fit the shared memory; other sizes are refused (the tensor-core GEMM takes them).
#include "linear_epilogue.cuh"

MG_STAMP_DECLARE(skinny)

namespace {

constexpr int MAX_M = 16;
constexpr int TILE_N = 8;            // weight rows per warp task
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int PRE = 8;               // k blocks (of 32) whose weights a lane holds at once
constexpr int XPAD = 64;             // bytes between activation rows beyond K bf16 (no bank conflicts)

struct SkinnyArgs {
    const bf16* x;                   // [M, K] bfloat16 activations, or null with a LayerNorm prologue
    const float* x32;                // rows to normalise (prologue), [*, K]
    const int* row_index;            // optional gather of x32 rows
    const float* gain;
    const float* shift;              // may be null
    float eps;
    const bf16* w;                   // [N, K]
    LinearEpilogue ep;
    int M, N, K;
    int k_splits;                    // warps that share one tile of 8 rows (1, 2, 4 or 8)
    int tiles_per_cta;
    // greedy choice on the way (AMAX kernels): the largest output of each token over this CTA's
    // rows goes to amax_v / amax_i [token][CTA]; rows at and past amax_limit are never chosen
    float* amax_v;
    int* amax_i;
    int amax_limit;
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// MT: token rows of the A operand: 8 (rows 8..15 are zero) or 16; a.M <= MT.  AMAX: also leave,
// per token, the largest output of this CTA's rows and its index (the first stage of an argmax
// over the rows, for the head's logits), lowest index first among equals.
template <int MT, bool AMAX>
__global__ void __launch_bounds__(THREADS) linear_skinny_kernel(const SkinnyArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int K = a.K;
    const int xstride = K * 2 + XPAD;                                         // bytes per token row
    uint8_t* xs = smem_raw;                                                   // [MT][K] bf16, padded rows
    float* partial = reinterpret_cast<float*>(smem_raw + (size_t)MT * xstride);   // [WARPS][MT][8]
    float* gain_s = partial + WARPS * MT * TILE_N;                                // [K] and [K]: LayerNorm gain and shift
    float* shift_s = gain_s + K;
    float* cand_v = shift_s + K;                                                  // [WARPS][MT] and the same of ints (AMAX)
    int* cand_i = reinterpret_cast<int*>(cand_v + WARPS * MT);
    float best_v = -INFINITY;                                                     // thread m: token m's best so far
    int best_i = 0x7fffffff;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    MG_STAMP(skinny, 0);

    const int ks = a.k_splits;
    const int tiles_per_round = WARPS / ks;
    const int my_tile_in_round = warp / ks, my_slice = warp % ks;
    const int kblocks = (K + 31) / 32;
    const int b_begin = (int)((long long)kblocks * my_slice / ks), b_end = (int)((long long)kblocks * (my_slice + 1) / ks);
    const int first_tile = blockIdx.x * a.tiles_per_cta;
    const int total_tiles = (a.N + TILE_N - 1) / TILE_N;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

    // Ask for the weights of this warp's first task before anything else: they travel from HBM
    // while the kernel in front drains and the activations are staged (and normalised) below.
    uint4 first_w[PRE];
    {
        const int tile = first_tile + my_tile_in_round;
        const bool live = my_tile_in_round < a.tiles_per_cta && tile < total_tiles;
        const bf16* wrow = a.w + (size_t)min(tile * TILE_N + g, a.N - 1) * K;
#pragma unroll
        for (int i = 0; i < PRE; ++i) {
            const int k = (b_begin + i) * 32 + 8 * t;
            first_w[i] = (live && b_begin + i < b_end && k < K) ? *reinterpret_cast<const uint4*>(wrow + k) : zero4;
        }
    }
    // The bias of the first result of this thread as well, so that the epilogue does not wait for it;
    // and, for the QKV projection, the cache row of its token (an input of the step, not a result).
    float first_bias = 0.f;
    int first_slot = -1;
    {
        const int ti = tid / (MT * TILE_N), r = tid % TILE_N;
        const int n = (first_tile + ti) * TILE_N + r;
        if (a.ep.bias && ti < tiles_per_round && ti < a.tiles_per_cta && n < a.N) first_bias = a.ep.bias[n];
        const int m = (tid % (MT * TILE_N)) / TILE_N;
        if (a.ep.k_pages != nullptr && m < a.M) first_slot = a.ep.slots[m];
    }
    // Which rows to normalise is an input of the step as well.
    int first_row = warp;
    if (a.x32 != nullptr && a.row_index != nullptr && warp < a.M) first_row = a.row_index[warp];
    // Gain and shift of the LayerNorm prologue are weights too: they go to shared memory now, so
    // that the normalisation does not wait for them after the statistics.
    const bool ln = a.x32 != nullptr;
    const bool ln_fast = ln && K % 128 == 0 && K <= 1024;                 // the row fits a warp's registers
    if (ln) {
        stage_gain_shift(gain_s, shift_s, a.gain, a.shift, K / 4, tid, THREADS);
    }
    // Weights and bias do not depend on the kernel before this one; everything below does.
    MG_STAMP(skinny, 2);
    pdl_trigger();
    pdl_wait();
    MG_STAMP(skinny, 3);
    if (ln) __syncthreads();

    // ---- stage the activations (with the LayerNorm prologue if asked) as bfloat16 ----
    // Rows at and past M stay as they are: a token's results depend on its own row only.
    if (a.x32 != nullptr) {
        for (int m = warp; m < a.M; m += WARPS) {
            uint8_t* dst = xs + (size_t)m * xstride;
            const float* src = a.x32 + (size_t)(a.row_index ? (m == warp ? first_row : a.row_index[m]) : m) * K;
            if (ln_fast) {
                // the row lives in registers between the passes: 16-byte loads, one trip to memory
                float4 v[8];
                const int n4 = K / 128;
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (i < n4) {
                        v[i] = *reinterpret_cast<const float4*>(src + (lane + 32 * i) * 4);
                        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
                    }
                const float mean = warp_sum(sum) / (float)K;
                float sq = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (i < n4) {
                        const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
                        sq += (dx * dx + dy * dy) + (dz * dz + dw * dw);
                    }
                const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)K + a.eps);
                // gain and shift of four chunks are read before the four results are stored: a store to
                // shared memory keeps the loads from shared memory behind it in their place
#pragma unroll
                for (int i0 = 0; i0 < 8; i0 += 4) {
                    float4 gn[4], sh[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (i0 + u < n4) {
                            const int c = (lane + 32 * (i0 + u)) * 4;
                            gn[u] = *reinterpret_cast<const float4*>(gain_s + c);
                            sh[u] = *reinterpret_cast<const float4*>(shift_s + c);
                        }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (i0 + u < n4) {
                            const int i = i0 + u, c = (lane + 32 * i) * 4;
                            uint2 y;
                            y.x = pack_bf16((v[i].x - mean) * rstd * gn[u].x + sh[u].x, (v[i].y - mean) * rstd * gn[u].y + sh[u].y);
                            y.y = pack_bf16((v[i].z - mean) * rstd * gn[u].z + sh[u].z, (v[i].w - mean) * rstd * gn[u].w + sh[u].w);
                            *reinterpret_cast<uint2*>(dst + c * 2) = y;
                        }
                }
                continue;
            }
            // longer or odd rows: three passes in chunks (K is a multiple of 8 here), gain and shift from shared memory
            layernorm_row_chunked<bf16>(src, K, gain_s, a.shift ? shift_s : nullptr, a.eps, reinterpret_cast<bf16*>(dst), lane);
        }
    } else {
        // (a thread asks for four pieces before it stores the first: one trip to L2 for 4 x THREADS pieces)
        const int chunks8 = K / 8, total = a.M * chunks8;
        for (int i0 = tid; i0 < total; i0 += 4 * THREADS) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * THREADS;
                if (i < total) v[u] = *reinterpret_cast<const uint4*>(a.x + (size_t)i * 8);   // (row m, piece c) is piece m * chunks8 + c
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * THREADS;
                if (i < total) {
                    const int m = i / chunks8, c = i - m * chunks8;
                    *reinterpret_cast<uint4*>(xs + (size_t)m * xstride + c * 16) = v[u];
                }
            }
        }
    }
    __syncthreads();
    MG_STAMP(skinny, 4);

    const uint8_t* xrow0 = xs + (size_t)g * xstride;
    const uint8_t* xrow1 = xs + (size_t)(g + 8) * xstride;
    for (int t0 = 0; t0 < a.tiles_per_cta; t0 += tiles_per_round) {
        const int tile = first_tile + t0 + my_tile_in_round;
        const bool active = (t0 + my_tile_in_round) < a.tiles_per_cta && tile < total_tiles;
        // the first result this thread finishes in this round, and what it adds to
        const int e_ti = tid / (MT * TILE_N), e_rem = tid - e_ti * (MT * TILE_N);
        const int e_m = e_rem / TILE_N, e_n = (first_tile + t0 + e_ti) * TILE_N + (e_rem - e_m * TILE_N);
        float e_res = 0.f;
        if (a.ep.epilogue == EPI_RESIDUAL && e_ti < tiles_per_round && t0 + e_ti < a.tiles_per_cta && e_n < a.N && e_m < a.M)
            e_res = a.ep.residual[(size_t)e_m * a.N + e_n];
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        if (active) {
            const bf16* wrow = a.w + (size_t)min(tile * TILE_N + g, a.N - 1) * K;
            for (int b0 = b_begin; b0 < b_end; b0 += PRE) {
                uint4 wv[PRE];
                if (t0 == 0 && b0 == b_begin) {
#pragma unroll
                    for (int i = 0; i < PRE; ++i) wv[i] = first_w[i];
                } else {
#pragma unroll
                    for (int i = 0; i < PRE; ++i) {
                        const int k = (b0 + i) * 32 + 8 * t;
                        wv[i] = (b0 + i < b_end && k < K) ? *reinterpret_cast<const uint4*>(wrow + k) : zero4;
                    }
                }
#pragma unroll
                for (int i = 0; i < PRE; ++i) {
                    const int k = (b0 + i) * 32 + 8 * t;
                    if (b0 + i < b_end) {                                        // uniform in the warp
                        const bool in = k < K;
                        const uint4 x0 = in ? *reinterpret_cast<const uint4*>(xrow0 + k * 2) : zero4;
                        uint4 x1 = zero4;
                        if (MT == 16 && in) x1 = *reinterpret_cast<const uint4*>(xrow1 + k * 2);
                        mma_bf16(c, x0.x, x1.x, x0.y, x1.y, wv[i].x, wv[i].y);
                        mma_bf16(c, x0.z, x1.z, x0.w, x1.w, wv[i].z, wv[i].w);
                    }
                }
            }
        }
        // c0, c1: token g, rows 2t and 2t+1 of the tile; c2, c3: token g + 8
        {
            float* mine = partial + (size_t)warp * MT * TILE_N;
            *reinterpret_cast<float2*>(mine + g * TILE_N + 2 * t) = make_float2(c[0], c[1]);
            if (MT == 16) *reinterpret_cast<float2*>(mine + (g + 8) * TILE_N + 2 * t) = make_float2(c[2], c[3]);
        }
        __syncthreads();
        MG_STAMP(skinny, 5);
        // ---- epilogue: one thread per (tile of the round, token, row) ----
        for (int e = tid; e < tiles_per_round * MT * TILE_N; e += THREADS) {
            const int ti = e / (MT * TILE_N), rem = e - ti * (MT * TILE_N);
            const int m = rem / TILE_N, r = rem - m * TILE_N;
            const int n = (first_tile + t0 + ti) * TILE_N + r;
            const bool live = (t0 + ti) < a.tiles_per_cta && n < a.N && m < a.M;
            float v = 0.f;
            if (live) {
                for (int s = 0; s < ks; ++s) v += partial[((size_t)(ti * ks + s) * MT + m) * TILE_N + r];   // slices in order
                if (a.ep.bias) v += (e == tid && t0 == 0) ? first_bias : a.ep.bias[n];
                linear_finish(a.ep, m, n, v, e == tid, e_res, e == tid, first_slot);
            }
            if constexpr (AMAX) {
                // the eight rows of a (tile, token) sit in eight neighbouring lanes
                float cv = (live && n < a.amax_limit) ? v : -INFINITY;
                int ci = (live && n < a.amax_limit) ? n : 0x7fffffff;
#pragma unroll
                for (int o = 1; o < TILE_N; o <<= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, cv, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, ci, o);
                    if (ov > cv || (ov == cv && oi < ci)) { cv = ov; ci = oi; }
                }
                if (r == 0) {
                    cand_v[ti * MT + m] = cv;
                    cand_i[ti * MT + m] = ci;
                }
            }
        }
        __syncthreads();
        if constexpr (AMAX) {
            if (tid < MT) {
                for (int ti = 0; ti < tiles_per_round; ++ti) {                   // tiles in order
                    const float cv = cand_v[ti * MT + tid];
                    const int ci = cand_i[ti * MT + tid];
                    if (cv > best_v || (cv == best_v && ci < best_i)) { best_v = cv; best_i = ci; }
                }
            }
        }
    }
    MG_STAMP(skinny, 7);
    if constexpr (AMAX) {
        if (tid < a.M) {
            a.amax_v[(size_t)tid * gridDim.x + blockIdx.x] = best_v;
            a.amax_i[(size_t)tid * gridDim.x + blockIdx.x] = best_i;
        }
    }
}

}  // namespace

// Largest M this kernel takes.
MG_API int mg_linear_skinny_max_rows() { return MAX_M; }

// How the work of an [N, K] matrix is cut: tiles of 8 rows, each shared by `ks` warps with at least
// two k blocks (of 32) per warp, so that every SM gets some and a lane holds all its weights at
// once; `tpc` tiles per CTA.  Returns the number of CTAs.
static int skinny_split(int N, int K, int* ks_out, int* tpc_out) {
    const int tiles = (N + TILE_N - 1) / TILE_N, kblocks = (K + 31) / 32;
    int ks = 1;
    while (ks < WARPS && kblocks / (ks * 2) >= 2 && (long long)tiles * (ks * 2) / WARPS <= 200) ks *= 2;
    const int per_round = WARPS / ks;
    int tpc = per_round;                                   // one round per CTA by default
    while ((tiles + tpc - 1) / tpc > 8 * 148) tpc += per_round;
    *ks_out = ks;
    *tpc_out = tpc;
    return (tiles + tpc - 1) / tpc;
}

// CTAs mg_linear_skinny launches for an [N, K] matrix: with the greedy choice on the way, its
// scratch holds M * that many floats and as many ints.
MG_API int mg_linear_skinny_ctas(int N, int K) {
    int ks, tpc;
    return skinny_split(N, K, &ks, &tpc);
}

// Shared memory the kernel needs for M tokens of width K (the caller checks it against the limit).
static size_t skinny_smem(int mt, int K) {
    return (size_t)mt * ((size_t)K * 2 + XPAD) + (size_t)WARPS * mt * TILE_N * sizeof(float) + (size_t)2 * K * sizeof(float) +
           (size_t)2 * WARPS * mt * sizeof(float);
}

MG_GUARD_EXPORT(linear_skinny, linear_index_fault)

// x: [M, K] bf16 (or null when x32 is given: then rows row_index[m] (or m) of x32 [*, K] are
// LayerNorm-ed with gain/shift/eps first).  w: [N, K] bf16.  Epilogues as mg_linear_simt.
// With k_pages given (QKV projection, bf16 out), features >= q_width also go to the cache rows
// slots[m].  Returns MG_ERR_UNSUPPORTED for M > 16, K % 8 != 0 or activations beyond shared memory.
MG_API int mg_linear_skinny(const void* x, const float* x32, const int* row_index, const float* gain,
                            const float* shift, float eps, const void* w, const float* bias, void* out,
                            float* residual, int M, int N, int K, int epilogue, int out_bf16, void* k_pages,
                            void* v_pages, const int* slots, int q_width, int n_kv_head, int head_dim,
                            int page_tokens, int num_pages, float* amax_v, int* amax_i, int amax_limit, void* stream) {
    if (M == 0) return MG_OK;
    MG_REQUIRE(M > 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    MG_REQUIRE(x != nullptr || (x32 != nullptr && gain != nullptr), "linear: missing input");
    MG_REQUIRE(epilogue == EPI_RESIDUAL ? residual != nullptr : out != nullptr, "linear: missing output");
    const int mt = M <= 8 ? 8 : 16;
    const size_t smem = skinny_smem(mt, K);
    if (M > MAX_M || K % 8 != 0 || smem > 200 * 1024 || ((uintptr_t)w & 15) || (x && ((uintptr_t)x & 15)) ||
        (x32 && !x && ((uintptr_t)x32 & 15)) || (gain && ((uintptr_t)gain & 15)) || (shift && ((uintptr_t)shift & 15)))
        return mg_set_error(MG_ERR_UNSUPPORTED, "linear (skinny): needs M <= 16, K %% 8 == 0, aligned operands");
    MG_REQUIRE(k_pages == nullptr || (out_bf16 && epilogue == EPI_STORE && slots && v_pages && head_dim > 0 &&
                                      n_kv_head > 0 && page_tokens > 0 && N == q_width + 2 * n_kv_head * head_dim),
               "linear: bad key/value sink");
    SkinnyArgs a;
    a.x = (const bf16*)x; a.x32 = x ? nullptr : x32; a.row_index = row_index; a.gain = gain; a.shift = shift; a.eps = eps;
    a.w = (const bf16*)w; a.M = M; a.N = N; a.K = K;
    a.ep.bias = bias; a.ep.out = out; a.ep.residual = residual; a.ep.M = M; a.ep.N = N;
    a.ep.epilogue = epilogue; a.ep.out_bf16 = out_bf16;
    a.ep.k_pages = (bf16*)k_pages; a.ep.v_pages = (bf16*)v_pages; a.ep.slots = slots;
    a.ep.q_width = q_width; a.ep.n_kv_head = n_kv_head; a.ep.head_dim = head_dim; a.ep.page_tokens = page_tokens; a.ep.num_pages = num_pages;
    MG_REQUIRE(amax_v == nullptr || (amax_i != nullptr && epilogue == EPI_STORE && !out_bf16),
               "linear: the greedy choice goes with 32-bit stored outputs");
    a.amax_v = amax_v; a.amax_i = amax_i; a.amax_limit = (amax_limit <= 0 || amax_limit > N) ? N : amax_limit;
    const int grid = skinny_split(N, K, &a.k_splits, &a.tiles_per_cta);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(linear_skinny_kernel<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_skinny_kernel<16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_skinny_kernel<8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_skinny_kernel<16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "linear (skinny): cannot raise shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const bool amax = amax_v != nullptr;
    const cudaError_t le =
        mt == 8 ? (amax ? mg_launch(linear_skinny_kernel<8, true>, dim3(grid), dim3(THREADS), smem, s, true, a)
                        : mg_launch(linear_skinny_kernel<8, false>, dim3(grid), dim3(THREADS), smem, s, true, a))
                : (amax ? mg_launch(linear_skinny_kernel<16, true>, dim3(grid), dim3(THREADS), smem, s, true, a)
                        : mg_launch(linear_skinny_kernel<16, false>, dim3(grid), dim3(THREADS), smem, s, true, a));
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "linear_skinny: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("linear_skinny");
    return MG_OK;
}
