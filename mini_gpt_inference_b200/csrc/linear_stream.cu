// Projection of up to 64 tokens onto a LARGE matrix (the head: tens of thousands of rows; or any
// matrix of many megabytes):
// out[m, n] = x[m, :] . w[n, :], the weights streamed once through shared memory.
//
// The small-batch kernel (linear_skinny.cu) holds a warp's weights in registers: right for a
// matrix of a few hundred row tiles, where one round of CTAs covers it.  The head has thousands of
// tiles: there the time goes to rounds of short-lived CTAs, each of which stages the activations
// again and waits for memory once or twice with little in flight.  Here one CTA per SM stays and
// every warp runs a pipeline of its own: a tile is 8 weight rows, contiguous in memory; lane 0
// brings each row with a bulk asynchronous copy (cp.async.bulk, counted on an mbarrier) into one of
// the warp's stages, rows 64 bytes apart in the banks; the warp multiplies from shared memory with
// warp-level mma (tokens as the 16 rows of A, the 8 weight rows as the columns of B, K in blocks
// of 32 with the 16-byte pattern of the small-batch kernel) while its other stages fill.  About
// 190 KB are in flight per SM the whole time, and the first tiles are asked for before the wait
// for the kernel in front.
//
// Rows too long for whole-row stages beside the activations (width 1600, say) are cut into K chunks:
// a stage then holds the tile's 8 rows over one chunk, chunks of a tile follow one another in the
// warp's ring, and the tile's sums stay in registers from chunk to chunk.  With chunks of a few
// hundred bytes a row the copies' own cost shows; the caller limits the number of chunks.
//
// Fused as in the small-batch kernel: LayerNorm prologue (with row gather), bias / tanh-GELU /
// residual / store epilogue, the copy of key and value features to their cache rows, and the first
// stage of the greedy argmax over the rows.  A warp owns whole rows of K, so every output sums
// its terms in k order, independent of M.
// The waits are bounded: if one runs out, the kernel records a code in `status` and stops.
#include <math.h>

#include "blackwell.cuh"
#include "linear_epilogue.cuh"

namespace {

constexpr int MAX_M = 64;
constexpr int TILE_N = 8;            // weight rows per tile
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int XPAD = 64;             // bytes between rows beyond K bf16 (no bank conflicts)

struct StreamArgs {
    const bf16* x;                   // [M, K] bfloat16 activations, or null with a LayerNorm prologue
    const float* x32;                // rows to normalise (prologue), [*, K]
    const int* row_index;            // optional gather of x32 rows
    const float* gain;
    const float* shift;              // may be null
    float eps;
    const bf16* w;                   // [N, K]
    LinearEpilogue ep;
    int M, N, K;
    int tiles_per_cta;
    int stages;                      // copies (a tile's rows over one K chunk) a warp has in flight
    int kc;                          // K chunk: columns of a tile that one stage holds (a multiple of 32, or K)
    int nchunks;                     // ceil(K / kc)
    float* amax_v;                   // [M][gridDim.x * WARPS] candidates of the greedy argmax, or null
    int* amax_i;
    int amax_limit;
    int* status;
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <int MT>   // token rows held: 8 (rows 8..15 of the A operand are zero), 16, 32 or 64
__global__ void __launch_bounds__(THREADS, 1) linear_stream_kernel(const StreamArgs a) {
    constexpr int MG = MT <= 16 ? 1 : MT / 16;                          // groups of 16 tokens (one mma each)
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int K = a.K;
    const int xstride = K * 2 + XPAD;                                   // bytes per row of activations
    const int kc = a.kc, nch = a.nchunks;
    const int wstride = kc * 2 + XPAD;                                  // bytes per weight row of a stage
    const int tile_bytes = TILE_N * wstride;
    uint8_t* xs = smem_raw;                                             // [MT][xstride]
    float* gain_s = reinterpret_cast<float*>(xs + (size_t)MT * xstride);
    float* shift_s = gain_s + K;
    uint8_t* ring = reinterpret_cast<uint8_t*>(shift_s + K);            // [WARPS][stages][tile_bytes]
    __shared__ __align__(8) uint64_t bars[WARPS][4];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int stages = a.stages;
    uint8_t* my_ring = ring + (size_t)warp * stages * tile_bytes;
    const int total_tiles = (a.N + TILE_N - 1) / TILE_N;
    const int tile_begin = blockIdx.x * a.tiles_per_cta;
    const int tile_end = min(total_tiles, tile_begin + a.tiles_per_cta);
    // this warp takes tiles tile_begin + warp, + WARPS, ...
    const int n_mine = tile_begin + warp < tile_end ? (tile_end - tile_begin - warp + WARPS - 1) / WARPS : 0;
    const int n_items = n_mine * nch;                                   // (tile, K chunk), chunks of a tile in a row

    // Ask for tile j of this warp (the whole warp calls): lane 0 announces the bytes, then lane r
    // asks for weight row r with a bulk copy of its own: one instruction for the eight copies
    // (issued one after the other by a single lane they cost the warp a microsecond a tile).
    auto issue = [&](int j) {
        const int jt = j / nch, ch = j - jt * nch;
        const int tile = tile_begin + warp + jt * WARPS, s = j % stages;
        const int rows = min(TILE_N, a.N - tile * TILE_N);
        const int k0 = ch * kc, len = min(kc, K - k0);                  // len * 2 is a multiple of 16 bytes (K % 8 == 0)
        const uint32_t bar = smem_u32(&bars[warp][s]);
        if (lane == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)rows * len * 2) : "memory");
        __syncwarp();
        if (lane < rows)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(my_ring + (size_t)s * tile_bytes + (size_t)lane * wstride)),
                           "l"(a.w + ((size_t)tile * TILE_N + lane) * K + k0), "r"((uint32_t)len * 2), "r"(bar)
                         : "memory");
    };
    if (lane == 0) {
        for (int s = 0; s < stages; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bars[warp][s])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    for (int j = 0; j < stages && j < n_items; ++j) issue(j);           // weights depend on no kernel before
    // Which rows to normalise, and gain and shift, are inputs and weights as well.
    int first_row = warp;
    if (a.x32 != nullptr && a.row_index != nullptr && warp < a.M) first_row = a.row_index[warp];
    const bool ln = a.x32 != nullptr;
    const bool ln_fast = ln && K % 128 == 0 && K <= 1024;                 // the row fits a warp's registers
    if (ln) {
        stage_gain_shift(gain_s, shift_s, a.gain, a.shift, K / 4, tid, THREADS);
    }
    pdl_trigger();
    pdl_wait();
    if (ln) __syncthreads();

    // ---- stage the activations (with the LayerNorm prologue if asked) as bfloat16, once per CTA ----
    if (a.x32 != nullptr) {
        for (int m = warp; m < a.M; m += WARPS) {
            uint8_t* dst = xs + (size_t)m * xstride;
            const float* src = a.x32 + (size_t)(a.row_index ? (m == warp ? first_row : a.row_index[m]) : m) * K;
            if (ln_fast) {
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
        const int chunks8 = K / 8;
        for (int i = tid; i < a.M * chunks8; i += THREADS) {
            const int m = i / chunks8, c = i - m * chunks8;
            *reinterpret_cast<uint4*>(xs + (size_t)m * xstride + c * 16) =
                *reinterpret_cast<const uint4*>(a.x + (size_t)m * K + c * 8);
        }
    }
    __syncthreads();

    // ---- every warp walks its tiles ----
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    float best_v[MG][2];                                                 // tokens 16 mg + g and 16 mg + g + 8
    int best_i[MG][2];
#pragma unroll
    for (int mg = 0; mg < MG; ++mg)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            best_v[mg][h] = -INFINITY;
            best_i[mg][h] = 0x7fffffff;
        }
    bool good = true;
    float c[MG][4];                                                     // a tile's sums, kept over its K chunks
    for (int j = 0; j < n_items; ++j) {
        const int jt = j / nch, ch = j - jt * nch;
        const int tile = tile_begin + warp + jt * WARPS, s = j % stages;
        if (!mbar_wait(smem_u32(&bars[warp][s]), (uint32_t)(j / stages) & 1u)) {
            good = false;
            break;                                                      // uniform in the warp
        }
        const uint8_t* wrow = my_ring + (size_t)s * tile_bytes + (size_t)g * wstride;
        const int k0 = ch * kc, len = min(kc, K - k0);
        const int kblocks = (len + 31) / 32;
        if (ch == 0) {
#pragma unroll
            for (int mg = 0; mg < MG; ++mg)
#pragma unroll
                for (int i = 0; i < 4; ++i) c[mg][i] = 0.f;
        }
#pragma unroll 2
        for (int b = 0; b < kblocks; ++b) {
            const int kl = b * 32 + 8 * t;                              // column inside the chunk
            const bool in = kl < len;
            const int k = k0 + kl;
            const uint4 wv = in ? *reinterpret_cast<const uint4*>(wrow + kl * 2) : zero4;
#pragma unroll
            for (int mg = 0; mg < MG; ++mg) {
                const uint4 x0 = in ? *reinterpret_cast<const uint4*>(xs + (size_t)(mg * 16 + g) * xstride + k * 2) : zero4;
                uint4 x1 = zero4;
                if (MT >= 16 && in) x1 = *reinterpret_cast<const uint4*>(xs + (size_t)(mg * 16 + g + 8) * xstride + k * 2);
                mma_bf16(c[mg], x0.x, x1.x, x0.y, x1.y, wv.x, wv.y);
                mma_bf16(c[mg], x0.z, x1.z, x0.w, x1.w, wv.z, wv.w);
            }
        }
        __syncwarp();                                                   // every lane has read the stage
        if (j + stages < n_items) {                                     // uniform in the warp
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(j + stages);
        }
        if (ch != nch - 1) continue;                                    // the tile's other chunks first
        // c0, c1: token 16 mg + g, rows 2t and 2t+1 of the tile; c2, c3: token 16 mg + g + 8
#pragma unroll
        for (int mg = 0; mg < MG; ++mg)
#pragma unroll
            for (int h = 0; h < (MT >= 16 ? 2 : 1); ++h) {
                const int m = mg * 16 + g + 8 * h;
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int n = tile * TILE_N + 2 * t + i;
                    const bool live = m < a.M && n < a.N;               // rows past N hold stale weights
                    float v = c[mg][2 * h + i];
                    if (live) {
                        if (a.ep.bias) v += a.ep.bias[n];
                        linear_finish(a.ep, m, n, v, false, 0.f);
                    }
                    if (a.amax_v != nullptr && live && n < a.amax_limit &&
                        (v > best_v[mg][h] || (v == best_v[mg][h] && n < best_i[mg][h]))) {
                        best_v[mg][h] = v;
                        best_i[mg][h] = n;
                    }
                }
            }
    }
    if (!good) {
        // a copy never arrived: report, give copies in flight a moment to land, write no candidates
        if (lane == 0) {
            atomicExch(a.status, 41);
            for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
        __syncwarp();
    }
    if (a.amax_v != nullptr) {
        // the four lanes of a token hold different rows: the best of them, lowest index among equals
#pragma unroll
        for (int mg = 0; mg < MG; ++mg)
#pragma unroll
            for (int h = 0; h < (MT >= 16 ? 2 : 1); ++h) {
#pragma unroll
                for (int o = 1; o < 4; o <<= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best_v[mg][h], o);
                    const int oi = __shfl_xor_sync(0xffffffffu, best_i[mg][h], o);
                    if (ov > best_v[mg][h] || (ov == best_v[mg][h] && oi < best_i[mg][h])) {
                        best_v[mg][h] = ov;
                        best_i[mg][h] = oi;
                    }
                }
                const int m = mg * 16 + g + 8 * h;
                if (t == 0 && m < a.M) {
                    const size_t idx = (size_t)m * (gridDim.x * WARPS) + blockIdx.x * WARPS + warp;
                    a.amax_v[idx] = good ? best_v[mg][h] : -INFINITY;
                    a.amax_i[idx] = good ? best_i[mg][h] : 0x7fffffff;
                }
            }
    }
}

// CTAs and tiles per CTA for an [N, K] matrix on a device of `sms` SMs.
int stream_split(int N, int sms, int* tiles_per_cta) {
    const int tiles = (N + TILE_N - 1) / TILE_N;
    // (a matrix of fewer tiles than the device has warps spreads over all SMs, with idle warps)
    int ctas = sms < tiles ? sms : tiles;
    if (ctas < 1) ctas = 1;
    const int per = (tiles + ctas - 1) / ctas;
    *tiles_per_cta = per;
    return (tiles + per - 1) / per;
}

int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 0;
    }
    return sms;
}

}  // namespace

// Candidates per row that mg_linear_stream leaves for the greedy argmax (its scratch holds M times
// as many floats and as many ints); 0 if the device cannot be queried.
MG_API int mg_linear_stream_parts(int N) {
    const int sms = sm_count();
    if (sms <= 0) return 0;
    int per;
    return stream_split(N, sms, &per) * WARPS;
}

MG_GUARD_EXPORT(linear_stream, linear_index_fault)

// As mg_linear_skinny (same operands, prologue, epilogues and greedy choice), for wide matrices.
// A stage holds a tile's rows whole where two such stages per warp fit beside the activations;
// longer rows are cut into K chunks (four stages per warp), a tile's sums staying in registers from
// chunk to chunk (at most `max_chunks` of them: every row copy then moves a few hundred bytes, and
// the copies' own cost shows).  Returns MG_ERR_UNSUPPORTED (nothing launched) for M > 64,
// K % 8 != 0, operands that are not 16-byte aligned, rows that need more chunks than allowed, or
// activations that leave no room for stages of 64 columns.
MG_API int mg_linear_stream(const void* x, const float* x32, const int* row_index, const float* gain,
                            const float* shift, float eps, const void* w, const float* bias, void* out,
                            float* residual, int M, int N, int K, int epilogue, int out_bf16, void* k_pages,
                            void* v_pages, const int* slots, int q_width, int n_kv_head, int head_dim,
                            int page_tokens, int num_pages, float* amax_v, int* amax_i, int amax_limit, int max_chunks,
                            int* status, void* stream) {
    if (M == 0) return MG_OK;
    MG_REQUIRE(M > 0 && N > 0 && K > 0 && status != nullptr, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    MG_REQUIRE(x != nullptr || (x32 != nullptr && gain != nullptr), "linear: missing input");
    MG_REQUIRE(epilogue == EPI_RESIDUAL ? residual != nullptr : out != nullptr, "linear: missing output");
    MG_REQUIRE(amax_v == nullptr || (amax_i != nullptr && epilogue == EPI_STORE && !out_bf16),
               "linear: the greedy choice goes with 32-bit stored outputs");
    const int sms = sm_count();
    const int mt = M <= 8 ? 8 : M <= 16 ? 16 : M <= 32 ? 32 : 64;
    const size_t xstride = (size_t)K * 2 + XPAD;
    const size_t fixed = (size_t)mt * xstride + (size_t)2 * K * sizeof(float);
    const size_t budget = 226 * 1024;
    int stages = fixed < budget ? (int)((budget - fixed) / ((size_t)WARPS * TILE_N * xstride)) : 0;
    if (stages > 4) stages = 4;
    int kc = K;
    if (stages < 2 && fixed < budget) {
        // four stages of K chunks: TILE_N * (2 kc + XPAD) bytes each, kc a multiple of 32
        const long long per_stage = (long long)((budget - fixed) / ((size_t)WARPS * 4 * TILE_N));
        kc = (int)((per_stage - XPAD) / 2) / 32 * 32;
        stages = kc >= 64 ? 4 : 0;
    }
    const int nchunks = kc > 0 ? (K + kc - 1) / kc : 0;
    MG_REQUIRE(k_pages == nullptr || (out_bf16 && epilogue == EPI_STORE && slots && v_pages && head_dim > 0 &&
                                      n_kv_head > 0 && page_tokens > 0 && N == q_width + 2 * n_kv_head * head_dim),
               "linear: bad key/value sink");
    if (sms <= 0 || M > MAX_M || K % 8 != 0 || stages < 2 || nchunks > max_chunks || ((uintptr_t)w & 15) || (x && ((uintptr_t)x & 15)) ||
        (x32 && !x && ((uintptr_t)x32 & 15)) || (gain && ((uintptr_t)gain & 15)) || (shift && ((uintptr_t)shift & 15)))
        return mg_set_error(MG_ERR_UNSUPPORTED, "linear (stream): needs M <= 64, K %% 8 == 0, aligned operands, rows that fit");
    StreamArgs a;
    a.x = (const bf16*)x; a.x32 = x ? nullptr : x32; a.row_index = row_index; a.gain = gain; a.shift = shift; a.eps = eps;
    a.w = (const bf16*)w; a.M = M; a.N = N; a.K = K;
    a.ep.bias = bias; a.ep.out = out; a.ep.residual = residual; a.ep.M = M; a.ep.N = N;
    a.ep.epilogue = epilogue; a.ep.out_bf16 = out_bf16;
    a.ep.k_pages = (bf16*)k_pages; a.ep.v_pages = (bf16*)v_pages; a.ep.slots = slots;
    a.ep.q_width = q_width; a.ep.n_kv_head = n_kv_head; a.ep.head_dim = head_dim; a.ep.page_tokens = page_tokens; a.ep.num_pages = num_pages;
    a.amax_v = amax_v; a.amax_i = amax_i; a.amax_limit = (amax_limit <= 0 || amax_limit > N) ? N : amax_limit;
    a.status = status;
    a.stages = stages;
    a.kc = kc;
    a.nchunks = nchunks;
    const int grid = stream_split(N, sms, &a.tiles_per_cta);
    const size_t smem = fixed + (size_t)WARPS * stages * TILE_N * ((size_t)kc * 2 + XPAD);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(linear_stream_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_stream_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_stream_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_stream_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "linear (stream): cannot raise shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const cudaError_t le = mt == 8    ? mg_launch(linear_stream_kernel<8>, dim3(grid), dim3(THREADS), smem, s, true, a)
                           : mt == 16 ? mg_launch(linear_stream_kernel<16>, dim3(grid), dim3(THREADS), smem, s, true, a)
                           : mt == 32 ? mg_launch(linear_stream_kernel<32>, dim3(grid), dim3(THREADS), smem, s, true, a)
                                      : mg_launch(linear_stream_kernel<64>, dim3(grid), dim3(THREADS), smem, s, true, a);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "linear_stream: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("linear_stream");
    return MG_OK;
}
