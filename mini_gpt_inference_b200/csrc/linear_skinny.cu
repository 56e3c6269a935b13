// Projection of a handful of tokens (decoding at small batch): out[m, n] = x[m, :] . w[n, :].
//
// With up to 8 tokens a projection is a stream over the weights: every weight is read once and
// used M times, far below what tensor cores need, and the tensor-core tile (128 weight rows per
// CTA) would leave most SMs idle on a 512- or 1536-row matrix.  Here the work is cut finely:
// a warp task is R = 4 weight rows times one slice of K; a CTA of 8 warps takes a few such
// tasks, so that a 512 x 2048 matrix still spreads over 128 CTAs with 16-byte loads from four
// rows in flight per lane.  The activations sit in shared memory as 32-bit copies of their
// bfloat16 values; sums are 32-bit.
//
// Fused around the product, because at this size every extra kernel costs more than its work:
//   * prologue: LayerNorm of the 32-bit residual rows (optionally gathered through an index),
//     statistics in 32-bit, result rounded to bfloat16 exactly as the stand-alone kernel does;
//   * epilogue: bias, tanh-GELU, bfloat16 or 32-bit store, or add into the 32-bit residual;
//   * epilogue of the QKV projection: key and value features also go to their cache pages.
//
// Every output element sums its K terms in a fixed order (lane-strided within a slice, lanes in
// order, slices in order), independent of M and of the other rows.  K must be a multiple of 8 and M * K
// bfloat16 must fit the shared memory; other sizes are refused (the tensor-core kernel takes
// them).
#include "common.cuh"

#define EPI_STORE 0
#define EPI_GELU 1
#define EPI_RESIDUAL 2

namespace {

constexpr int MAX_M = 8;
constexpr int R = 4;                 // weight rows per warp task
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;

struct SkinnyArgs {
    const bf16* x;                   // [M, K] bfloat16 activations, or null with a LayerNorm prologue
    const float* x32;                // rows to normalise (prologue), [*, K]
    const int* row_index;            // optional gather of x32 rows
    const float* gain;
    const float* shift;              // may be null
    float eps;
    const bf16* w;                   // [N, K]
    const float* bias;               // may be null
    void* out;                       // [M, N]
    float* residual;                 // [M, N] for EPI_RESIDUAL
    int M, N, K, epilogue, out_bf16;
    int k_splits;                    // warps that share one group of R rows (1, 2, 4 or 8)
    int groups_per_cta;              // groups of R rows per CTA
    // key/value sink of the QKV projection (k_pages null: none)
    bf16* k_pages;
    bf16* v_pages;
    const int* slots;                // [M] flat cache row of each token, < 0: skip
    int q_width, n_kv_head, head_dim, page_tokens;
};

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}

template <int MT>   // rows of activations held (1, 2, 4 or 8); a.M <= MT
__global__ void __launch_bounds__(THREADS) linear_skinny_kernel(const SkinnyArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // activations [MT][K] as 32-bit values that are exact bfloat16 numbers; rows >= M are zero
    float* xs = reinterpret_cast<float*>(smem_raw);
    float* partial = xs + (size_t)MT * a.K;                                   // [WARPS][R*MT]
    float* red = partial + WARPS * R * MT;                                    // [WARPS][R*MT][33]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = a.K;

    const int ks = a.k_splits;
    const int groups_per_round = WARPS / ks;
    const int my_group_in_round = warp / ks, my_slice = warp % ks;
    // slice edges at multiples of 8 elements
    const int chunks = K / 8;
    const int c_begin = (int)((long long)chunks * my_slice / ks), c_end = (int)((long long)chunks * (my_slice + 1) / ks);
    const int first_group = blockIdx.x * a.groups_per_cta;
    const int total_groups = (a.N + R - 1) / R;

    // Ask for the first weights of this warp's first task before anything else: they travel
    // from HBM while the activations are staged (and normalised) below.
    uint4 first_w[R];
    bool have_first = false;
    {
        const int group = first_group + my_group_in_round;
        const int c = c_begin + lane;
        if (my_group_in_round < a.groups_per_cta && group < total_groups && c < c_end) {
#pragma unroll
            for (int r = 0; r < R; ++r)
                first_w[r] = *reinterpret_cast<const uint4*>(a.w + (size_t)min(group * R + r, a.N - 1) * K + c * 8);
            have_first = true;
        }
    }

    // The bias is asked for now as well, so that the epilogue does not wait on HBM for it.
    {
        const int e = tid;
        if (e < groups_per_round * R * MT && a.bias) {
            const int gi = e / (R * MT), rm = e - gi * (R * MT);
            const int n = (first_group + gi) * R + rm / MT;
            if (gi < a.groups_per_cta && n < a.N) asm volatile("prefetch.global.L1 [%0];" ::"l"(a.bias + n));
        }
    }
    // Weights and bias do not depend on the kernel before this one; everything below does.
    pdl_trigger();
    pdl_wait();

    // ---- stage the activations (with the LayerNorm prologue if asked), rounded to bfloat16 ----
    if (a.x32 != nullptr) {
        for (int m = warp; m < MT; m += WARPS) {
            float* dst = xs + (size_t)m * K;
            if (m >= a.M) {
                for (int c = lane; c < K; c += 32) dst[c] = 0.f;
                continue;
            }
            const float* src = a.x32 + (size_t)(a.row_index ? a.row_index[m] : m) * K;
            if (K % 128 == 0 && K <= 1024) {
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
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (i < n4) {
                        const int c = (lane + 32 * i) * 4;
                        const float4 g = *reinterpret_cast<const float4*>(a.gain + c);
                        float4 sh = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (a.shift) sh = *reinterpret_cast<const float4*>(a.shift + c);
                        float4 y;
                        y.x = __bfloat162float(__float2bfloat16_rn((v[i].x - mean) * rstd * g.x + sh.x));
                        y.y = __bfloat162float(__float2bfloat16_rn((v[i].y - mean) * rstd * g.y + sh.y));
                        y.z = __bfloat162float(__float2bfloat16_rn((v[i].z - mean) * rstd * g.z + sh.z));
                        y.w = __bfloat162float(__float2bfloat16_rn((v[i].w - mean) * rstd * g.w + sh.w));
                        *reinterpret_cast<float4*>(dst + c) = y;
                    }
                continue;
            }
            float sum = 0.f;
            for (int c = lane; c < K; c += 32) sum += src[c];
            const float mean = warp_sum(sum) / (float)K;
            float sq = 0.f;
            for (int c = lane; c < K; c += 32) {
                const float d = src[c] - mean;
                sq += d * d;
            }
            const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)K + a.eps);
            for (int c = lane; c < K; c += 32) {
                float v = (src[c] - mean) * rstd * a.gain[c];
                if (a.shift) v += a.shift[c];
                dst[c] = __bfloat162float(__float2bfloat16_rn(v));
            }
        }
    } else {
        const int chunks8 = K / 8;
        for (int i = tid; i < MT * chunks8; i += THREADS) {
            const int m = i / chunks8, c = i - m * chunks8;
            float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (m < a.M) unpack8(*reinterpret_cast<const uint4*>(a.x + (size_t)m * K + c * 8), f);
            float* dst = xs + (size_t)m * K + c * 8;
            *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(f[4], f[5], f[6], f[7]);
        }
    }
    __syncthreads();

    for (int g0 = 0; g0 < a.groups_per_cta; g0 += groups_per_round) {
        const int group = first_group + g0 + my_group_in_round;
        const bool active = (g0 + my_group_in_round) < a.groups_per_cta && group < total_groups;
        float acc[R][MT];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
        if (active) {
            const int n0 = group * R;
            const bf16* wrow[R];
#pragma unroll
            for (int r = 0; r < R; ++r) wrow[r] = a.w + (size_t)min(n0 + r, a.N - 1) * K;
            for (int c = c_begin + lane; c < c_end; c += 32) {
                uint4 wraw[R];
                if (g0 == 0 && have_first && c == c_begin + lane) {
#pragma unroll
                    for (int r = 0; r < R; ++r) wraw[r] = first_w[r];
                } else {
#pragma unroll
                    for (int r = 0; r < R; ++r) wraw[r] = *reinterpret_cast<const uint4*>(wrow[r] + c * 8);
                }
                float wf[R][8];
#pragma unroll
                for (int r = 0; r < R; ++r) unpack8(wraw[r], wf[r]);
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const float4 x0 = *reinterpret_cast<const float4*>(xs + (size_t)m * K + c * 8);
                    const float4 x1 = *reinterpret_cast<const float4*>(xs + (size_t)m * K + c * 8 + 4);
                    const float xf[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[r][m] = fmaf(wf[r][i], xf[i], acc[r][m]);
                }
            }
        }
        // sum over the lanes through shared memory: lane l writes its R*MT sums as a column,
        // then lane v adds up row v (33-word rows: no bank conflicts); the order is lane 0..31
        {
            float* mine = red + (size_t)warp * (R * MT) * 33;
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) mine[(r * MT + m) * 33 + lane] = acc[r][m];
            __syncwarp();
            if (lane < R * MT) {
                float total = 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j) total += mine[lane * 33 + j];
                partial[warp * (R * MT) + lane] = total;
            }
        }
        __syncthreads();
        // ---- epilogue: one thread per (group of the round, row, token) ----
        for (int e = tid; e < groups_per_round * R * MT; e += THREADS) {
            const int gi = e / (R * MT), rm = e - gi * (R * MT);
            const int r = rm / MT, m = rm - r * MT;
            const int grp = first_group + g0 + gi;
            const int n = grp * R + r;
            if ((g0 + gi) >= a.groups_per_cta || n >= a.N || m >= a.M) continue;
            float v = 0.f;
            for (int s = 0; s < ks; ++s) v += partial[(gi * ks + s) * (R * MT) + rm];   // slices in order
            if (a.bias) v += a.bias[n];
            if (a.epilogue == EPI_GELU) v = gelu_tanh(v);
            const size_t idx = (size_t)m * a.N + n;
            if (a.epilogue == EPI_RESIDUAL) {
                a.residual[idx] += v;
            } else if (a.out_bf16) {
                const bf16 hv = __float2bfloat16_rn(v);
                reinterpret_cast<bf16*>(a.out)[idx] = hv;
                if (a.k_pages != nullptr && n >= a.q_width) {
                    const int slot = a.slots[m];
                    if (slot >= 0) {
                        const int kv_width = a.n_kv_head * a.head_dim;
                        const int f = n - a.q_width;
                        const int which = f / kv_width, fi = f - which * kv_width;
                        const int h = fi / a.head_dim, d = fi - h * a.head_dim;
                        const int page = slot / a.page_tokens, off = slot - page * a.page_tokens;
                        const size_t dst = (((size_t)page * a.n_kv_head + h) * a.page_tokens + off) * a.head_dim + d;
                        (which == 0 ? a.k_pages : a.v_pages)[dst] = hv;
                    }
                }
            } else {
                reinterpret_cast<float*>(a.out)[idx] = v;
            }
        }
        __syncthreads();
    }
}

}  // namespace

// Largest M this kernel takes.
MG_API int mg_linear_skinny_max_rows() { return MAX_M; }

// x: [M, K] bf16 (or null when x32 is given: then rows row_index[m] (or m) of x32 [*, K] are
// LayerNorm-ed with gain/shift/eps first).  w: [N, K] bf16.  Epilogues as mg_linear_simt.
// With k_pages given (QKV projection, bf16 out), features >= q_width also go to the cache rows
// slots[m].  Returns MG_ERR_UNSUPPORTED for M > 8, K % 8 != 0 or activations beyond shared memory.
MG_API int mg_linear_skinny(const void* x, const float* x32, const int* row_index, const float* gain,
                            const float* shift, float eps, const void* w, const float* bias, void* out,
                            float* residual, int M, int N, int K, int epilogue, int out_bf16, void* k_pages,
                            void* v_pages, const int* slots, int q_width, int n_kv_head, int head_dim,
                            int page_tokens, void* stream) {
    if (M == 0) return MG_OK;
    MG_REQUIRE(M > 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    MG_REQUIRE(x != nullptr || (x32 != nullptr && gain != nullptr), "linear: missing input");
    MG_REQUIRE(epilogue == EPI_RESIDUAL ? residual != nullptr : out != nullptr, "linear: missing output");
    const int mt = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
    const size_t smem = ((size_t)mt * K + (size_t)WARPS * R * mt * 34) * sizeof(float);
    if (M > MAX_M || K % 8 != 0 || smem > 200 * 1024 || ((uintptr_t)w & 15) || (x && ((uintptr_t)x & 15)))
        return mg_set_error(MG_ERR_UNSUPPORTED, "linear (skinny): needs M <= 8, K %% 8 == 0, aligned operands");
    MG_REQUIRE(k_pages == nullptr || (out_bf16 && epilogue == EPI_STORE && slots && v_pages && head_dim > 0 &&
                                      n_kv_head > 0 && page_tokens > 0 && N == q_width + 2 * n_kv_head * head_dim),
               "linear: bad key/value sink");
    SkinnyArgs a;
    a.x = (const bf16*)x; a.x32 = x ? nullptr : x32; a.row_index = row_index; a.gain = gain; a.shift = shift; a.eps = eps;
    a.w = (const bf16*)w; a.bias = bias; a.out = out; a.residual = residual;
    a.M = M; a.N = N; a.K = K; a.epilogue = epilogue; a.out_bf16 = out_bf16;
    a.k_pages = (bf16*)k_pages; a.v_pages = (bf16*)v_pages; a.slots = slots;
    a.q_width = q_width; a.n_kv_head = n_kv_head; a.head_dim = head_dim; a.page_tokens = page_tokens;
    // Cut the work so that a few hundred CTAs exist: groups of R rows, each shared by k_splits warps.
    const int groups = (N + R - 1) / R;
    int ks = 1;
    while (ks < WARPS && groups * ks < 8 * 296 && (K / 8) / (ks * 2) >= 32) ks *= 2;   // keep >= 32 chunks per slice
    a.k_splits = ks;
    const int per_round = WARPS / ks;
    int gpc = per_round;                                   // one round per CTA by default
    while ((groups + gpc - 1) / gpc > 4 * 148) gpc += per_round;
    a.groups_per_cta = gpc;
    const int grid = (groups + gpc - 1) / gpc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(linear_skinny_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_skinny_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_skinny_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_skinny_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "linear (skinny): cannot raise shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t le;
    switch (mt) {
        case 1: le = mg_launch(linear_skinny_kernel<1>, dim3(grid), dim3(THREADS), smem, s, true, a); break;
        case 2: le = mg_launch(linear_skinny_kernel<2>, dim3(grid), dim3(THREADS), smem, s, true, a); break;
        case 4: le = mg_launch(linear_skinny_kernel<4>, dim3(grid), dim3(THREADS), smem, s, true, a); break;
        default: le = mg_launch(linear_skinny_kernel<8>, dim3(grid), dim3(THREADS), smem, s, true, a); break;
    }
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "linear_skinny: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("linear_skinny");
    return MG_OK;
}
