// The rest of a pre-norm block after attention, for a handful of tokens, as ONE cooperative kernel:
//
//   x += attn . Wo^T + bo ;   h = act(LayerNorm(x) . Wfc^T + bfc) ;   x += h . Wproj^T + bproj
//
// At up to 8 tokens each of these three projections is a few microseconds of latency, not of
// work, and as separate kernels they pay a launch, a first trip to HBM for the weights and a
// drain each.  Here one CTA per SM stays resident through all three:
//
//   * at the start every CTA asks for ITS rows of all three weight matrices with bulk
//     asynchronous copies into shared memory (a few rows each: 36 KB per CTA at the 50M sizes),
//     so the weights of the later phases travel while the earlier phases compute;
//   * a phase stages the activations (a few KB, read from L2) in shared memory, each warp sums
//     R = 4 rows over a slice of K from shared memory, and one thread per output applies the
//     epilogue (bias, residual add or tanh-GELU);
//   * between the phases the CTAs meet at a grid-wide barrier (an atomic counter in global
//     memory; the launch is cooperative, so all CTAs are resident).  The wait is bounded: if it
//     runs out, a code goes to `status` and the kernel goes on to its end.
//
// LayerNorm statistics, sums, the GELU argument and the residual stream are 32-bit; activations
// are rounded to bfloat16 where the separate kernels round them, so the fused and the separate
// path agree to rounding of the summation order.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int MAX_M = 8;
constexpr int R = 4;                  // weight rows per warp task
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr uint32_t SPIN_LIMIT = 4000000u;

struct TailArgs {
    const bf16* attn;                 // [M, K1] attention output
    float* x;                         // [M, C] residual stream, updated in place
    const bf16* w_o;                  // [C, K1]
    const float* b_o;
    const float* gain;                // LayerNorm over C
    const float* shift;               // may be null
    float eps;
    const bf16* w_fc;                 // [F, C]
    const float* b_fc;
    const bf16* w_proj;               // [C, F]
    const float* b_proj;
    bf16* h;                          // [M, F] scratch
    int M, C, K1, F;
    int rows1, rows2, rows3;          // rows of each matrix per CTA (multiples of R)
    int* sync;                        // 3 ints: barrier 1, barrier 2, exits; zero between launches
    int* status;
    long long* stamps;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
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

// All CTAs of the grid meet here.  Returns false if the others did not arrive in time.
__device__ bool grid_barrier(int* counter, int expected, int* status) {
    __shared__ int ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        int seen;
        // release our writes and count ourselves in, without waiting for the old value
        asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(counter) : "memory");
        ok = 0;
        for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            if (seen >= expected) { ok = 1; break; }
        }
        if (!ok) atomicExch(status, 31);
    }
    __syncthreads();
    return ok != 0;
}

// What a projection phase does with a finished sum.
struct Epilogue {
    int gelu;                 // 0: out32[m, n] += sum + bias[n];  1: out16[m, n] = gelu(sum + bias[n])
    const float* bias;        // may be null
    float* out32;
    bf16* out16;
    int ld, M;
};

// One projection phase: out rows [row0, row0 + rows) of a [N, K] matrix whose rows lie in shared
// memory (`w_smem`, rows * K bf16), activations in `act` ([MT][K] floats).  One function for all
// three phases (not inlined), so that the later phases find its instructions cached.
template <int MT>
__device__ __noinline__ void project(const bf16* w_smem, const float* act, float* partial, float* red, int row0,
                                     int rows, int N, int K, const Epilogue ep) {
    static_assert(WARPS * R * MT <= THREADS, "one result per thread and round");
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunks = K / 8;
    int ks = 1;                                            // warps that share a group of R rows
    while (ks < WARPS && chunks / (ks * 2) >= 32) ks *= 2;
    const int per_round = WARPS / ks;
    const int groups = rows / R;
    const int my_group = warp / ks, my_slice = warp % ks;
    const int c_begin = (int)((long long)chunks * my_slice / ks), c_end = (int)((long long)chunks * (my_slice + 1) / ks);
    // the result this thread finishes in each round
    const int e_gi = tid / (R * MT), e_rm = tid - e_gi * (R * MT);
    const int e_r = e_rm / MT, e_m = e_rm - e_r * MT;
    for (int g0 = 0; g0 < groups; g0 += per_round) {
        const int e_n = row0 + (g0 + e_gi) * R + e_r;
        const bool e_live = e_gi < per_round && g0 + e_gi < groups && e_n < N && e_m < ep.M;
        float e_add = 0.f;                                 // asked for now, needed after the sums
        if (e_live) {
            if (ep.bias) e_add = ep.bias[e_n];
            if (!ep.gelu) e_add += __ldcg(ep.out32 + (size_t)e_m * ep.ld + e_n);
        }
        const int g = g0 + my_group;
        float acc[R][MT];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
        if (g < groups) {
            const bf16* wr = w_smem + (size_t)g * R * K;
            for (int c = c_begin + lane; c < c_end; c += 32) {
                float wf[R][8];
#pragma unroll
                for (int r = 0; r < R; ++r) unpack8(*reinterpret_cast<const uint4*>(wr + (size_t)r * K + c * 8), wf[r]);
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const float4 x0 = *reinterpret_cast<const float4*>(act + (size_t)m * K + c * 8);
                    const float4 x1 = *reinterpret_cast<const float4*>(act + (size_t)m * K + c * 8 + 4);
                    const float xf[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[r][m] = fmaf(wf[r][i], xf[i], acc[r][m]);
                }
            }
        }
        // sum over the lanes through shared memory (lane l writes a column, lane v adds up row v)
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
        __syncthreads();
        if (e_live) {
            float v = e_add;
            for (int s = 0; s < ks; ++s) v += partial[(e_gi * ks + s) * (R * MT) + e_rm];     // slices in order
            if (ep.gelu) ep.out16[(size_t)e_m * ep.ld + e_n] = __float2bfloat16_rn(gelu_tanh(v));
            else ep.out32[(size_t)e_m * ep.ld + e_n] = v;
        }
        __syncthreads();
    }
}

template <int MT>
__global__ void __launch_bounds__(THREADS) block_tail_kernel(const TailArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int C = a.C, K1 = a.K1, F = a.F, M = a.M;
    const int kmax = max(max(K1, C), F);
    // shared memory: weights of the three phases, activations, reduction scratch
    bf16* w1 = reinterpret_cast<bf16*>(smem_raw);
    bf16* w2 = w1 + (size_t)a.rows1 * K1;
    bf16* w3 = w2 + (size_t)a.rows2 * C;
    float* act = reinterpret_cast<float*>(w3 + (size_t)a.rows3 * F);
    float* partial = act + (size_t)MT * kmax;
    float* red = partial + WARPS * R * MT;
    __shared__ __align__(8) uint64_t wbar[3];

    const int row1 = blockIdx.x * a.rows1, row2 = blockIdx.x * a.rows2, row3 = blockIdx.x * a.rows3;
    const int n1 = max(0, min(a.rows1, C - row1)), n2 = max(0, min(a.rows2, F - row2)), n3 = max(0, min(a.rows3, C - row3));

    if (tid == 0) {
        for (int i = 0; i < 3; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&wbar[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // ask for this CTA's rows of all three matrices now (weights depend on no earlier kernel)
        const uint32_t b1 = (uint32_t)n1 * K1 * 2, b2 = (uint32_t)n2 * C * 2, b3 = (uint32_t)n3 * F * 2;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&wbar[0])), "r"(b1) : "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&wbar[1])), "r"(b2) : "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&wbar[2])), "r"(b3) : "memory");
        if (b1) asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_u32(w1)), "l"(a.w_o + (size_t)row1 * K1), "r"(b1), "r"(smem_u32(&wbar[0])) : "memory");
        if (b2) asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_u32(w2)), "l"(a.w_fc + (size_t)row2 * C), "r"(b2), "r"(smem_u32(&wbar[1])) : "memory");
        if (b3) asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_u32(w3)), "l"(a.w_proj + (size_t)row3 * F), "r"(b3), "r"(smem_u32(&wbar[2])) : "memory");
    }
    // rows of the weight tiles that lie past the matrix stay unread: their results are dropped
    __syncthreads();
    bool good = true;
    int sidx = 0;
#define STAMP() do { if (a.stamps && blockIdx.x == 0 && tid == 0) a.stamps[sidx++] = clock64(); } while (0)
    STAMP();

    // ---- phase 1: x += attn . Wo^T + bo ----
    for (int i = tid; i < MT * (K1 / 8); i += THREADS) {
        const int m = i / (K1 / 8), c = i - m * (K1 / 8);
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (m < M) unpack8(*reinterpret_cast<const uint4*>(a.attn + (size_t)m * K1 + c * 8), f);
        float* dst = act + (size_t)m * K1 + c * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
    STAMP();
    good = mbar_wait(smem_u32(&wbar[0]), 0) && good;
    __syncthreads();
    STAMP();
    project<MT>(w1, act, partial, red, row1, a.rows1, C, K1, Epilogue{0, a.b_o, a.x, nullptr, C, M});
    STAMP();
    good = grid_barrier(a.sync + 0, gridDim.x, a.status) && good;
    STAMP();

    // ---- phase 2: h = gelu(LayerNorm(x) . Wfc^T + bfc) ----
    for (int m = warp; m < MT; m += WARPS) {
        float* dst = act + (size_t)m * C;
        if (m >= M) {
            for (int c = lane; c < C; c += 32) dst[c] = 0.f;
            continue;
        }
        // one trip to L2 (other CTAs wrote x), the statistics from shared memory
        const float4* src = reinterpret_cast<const float4*>(a.x + (size_t)m * C);
        for (int c = lane; c < C / 4; c += 32) reinterpret_cast<float4*>(dst)[c] = __ldcg(src + c);
        __syncwarp();
        float sum = 0.f;
        for (int c = lane; c < C; c += 32) sum += dst[c];
        const float mean = warp_sum(sum) / (float)C;
        float sq = 0.f;
        for (int c = lane; c < C; c += 32) {
            const float d = dst[c] - mean;
            sq += d * d;
        }
        const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)C + a.eps);
        for (int c = lane; c < C; c += 32) {
            float v = (dst[c] - mean) * rstd * a.gain[c];
            if (a.shift) v += a.shift[c];
            dst[c] = __bfloat162float(__float2bfloat16_rn(v));
        }
    }
    STAMP();
    good = mbar_wait(smem_u32(&wbar[1]), 0) && good;
    __syncthreads();
    STAMP();
    project<MT>(w2, act, partial, red, row2, a.rows2, F, C, Epilogue{1, a.b_fc, nullptr, a.h, F, M});
    STAMP();
    good = grid_barrier(a.sync + 1, gridDim.x, a.status) && good;
    STAMP();

    // ---- phase 3: x += h . Wproj^T + bproj ----
    for (int i = tid; i < MT * (F / 8); i += THREADS) {
        const int m = i / (F / 8), c = i - m * (F / 8);
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (m < M) unpack8(__ldcg(reinterpret_cast<const uint4*>(a.h + (size_t)m * F + c * 8)), f);
        float* dst = act + (size_t)m * F + c * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
    STAMP();
    good = mbar_wait(smem_u32(&wbar[2]), 0) && good;
    __syncthreads();
    STAMP();
    project<MT>(w3, act, partial, red, row3, a.rows3, C, F, Epilogue{0, a.b_proj, a.x, nullptr, C, M});
    STAMP();
    if (!good && tid == 0) atomicExch(a.status, 32);

    // the last CTA to leave puts the counters back to zero for the next launch
    __syncthreads();
    if (tid == 0) {
        int seen;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(seen) : "l"(a.sync + 2) : "memory");
        if (seen == (int)gridDim.x - 1) {
            a.sync[0] = 0;
            a.sync[1] = 0;
            a.sync[2] = 0;
        }
    }
}

int round_rows(int n, int ctas) {
    int per = (n + ctas - 1) / ctas;
    return (per + R - 1) / R * R;
}

}  // namespace

static long long* g_stamps = nullptr;
MG_API int mg_block_tail_debug(long long* p) { g_stamps = p; return 0; }

// Most tokens this kernel takes.
MG_API int mg_block_tail_max_rows() { return MAX_M; }

// The fused block tail (see the top of this file).  attn: [M, K1] bf16; x: [M, C] float32, updated
// in place; w_o: [C, K1], w_fc: [F, C], w_proj: [C, F] bf16; biases and the LayerNorm shift may be
// null; h: [M, F] bf16 scratch; sync: 3 ints that are ZERO before the first launch (the kernel
// leaves them zero); status receives a non-zero code if a wait ran out.  Returns
// MG_ERR_UNSUPPORTED (nothing launched) for M > 8, sizes that are no multiple of 8, weights that
// do not fit the shared memory, or if the GPU cannot hold the whole grid at once.
MG_API int mg_block_tail(const void* attn, float* x, const void* w_o, const float* b_o, const float* gain,
                         const float* shift, float eps, const void* w_fc, const float* b_fc, const void* w_proj,
                         const float* b_proj, void* h, int M, int C, int K1, int F, int* sync, int* status,
                         void* stream) {
    if (M == 0) return MG_OK;
    MG_REQUIRE(M > 0 && C > 0 && K1 > 0 && F > 0 && attn && x && w_o && gain && w_fc && w_proj && h && sync && status,
               "block tail: bad arguments");
    if (M > MAX_M || C % 8 || K1 % 8 || F % 8 ||
        (((uintptr_t)attn | (uintptr_t)w_o | (uintptr_t)w_fc | (uintptr_t)w_proj | (uintptr_t)h) & 15))
        return mg_set_error(MG_ERR_UNSUPPORTED, "block tail: needs M <= 8, sizes in multiples of 8, aligned operands");
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            return mg_set_error(MG_ERR_CUDA, "block tail: cannot query the device");
    }
    TailArgs a;
    a.attn = (const bf16*)attn; a.x = x; a.w_o = (const bf16*)w_o; a.b_o = b_o; a.gain = gain; a.shift = shift; a.eps = eps;
    a.w_fc = (const bf16*)w_fc; a.b_fc = b_fc; a.w_proj = (const bf16*)w_proj; a.b_proj = b_proj; a.h = (bf16*)h;
    a.M = M; a.C = C; a.K1 = K1; a.F = F; a.sync = sync; a.status = status; a.stamps = g_stamps;
    // as many CTAs as the longest matrix can keep busy with R rows each, at most one per SM
    int ctas = sms;
    const int most_groups = ((C > F ? C : F) + R - 1) / R;
    if (ctas > most_groups) ctas = most_groups;
    a.rows1 = round_rows(C, ctas); a.rows2 = round_rows(F, ctas); a.rows3 = round_rows(C, ctas);
    const int mt = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
    const int kmax = K1 > C ? (K1 > F ? K1 : F) : (C > F ? C : F);
    const size_t smem = ((size_t)a.rows1 * K1 + (size_t)a.rows2 * C + (size_t)a.rows3 * F) * sizeof(bf16) +
                        ((size_t)mt * kmax + (size_t)WARPS * R * mt * 34) * sizeof(float);
    if (smem > 200 * 1024) return mg_set_error(MG_ERR_UNSUPPORTED, "block tail: weights of a CTA do not fit the shared memory");
    void (*kernel)(const TailArgs) = mt == 1 ? block_tail_kernel<1> : mt == 2 ? block_tail_kernel<2>
                                     : mt == 4 ? block_tail_kernel<4> : block_tail_kernel<8>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "block tail: cannot raise shared memory: %s", cudaGetErrorString(e));
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, smem);
    if (e != cudaSuccess || per_sm * sms < ctas)
        return mg_set_error(MG_ERR_UNSUPPORTED, "block tail: the grid of %d CTAs cannot be resident at once", ctas);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kernel, a);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "block tail: launch failed: %s", cudaGetErrorString(e));
    return MG_OK;
}
