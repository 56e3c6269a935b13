// Sampling from 32-bit logits: greedy (argmax) here; the stochastic sampler follows below.
#include <float.h>
#include <math.h>

#include "common.cuh"

namespace {

constexpr int ARGMAX_THREADS = 256;

// Largest value of a row; among equal values the lowest index wins.  NaN never wins.
__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, int limit) {
    __shared__ float best_v[ARGMAX_THREADS / 32];
    __shared__ int best_i[ARGMAX_THREADS / 32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < limit; i += blockDim.x) {
        const float x = row[i];
        if (x > v || (x == v && i < idx)) { v = x; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { best_v[warp] = v; best_i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = lane < ARGMAX_THREADS / 32 ? best_v[lane] : -INFINITY;
        idx = lane < ARGMAX_THREADS / 32 ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
    }
}

// Stage 1 of the wide argmax: block (row, part) scans its slice of the row.
__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_part_kernel(const float* __restrict__ logits, float* __restrict__ part_v, int* __restrict__ part_i,
                   int vocab, int limit, int parts, int slice) {
    __shared__ float best_v[ARGMAX_THREADS / 32];
    __shared__ int best_i[ARGMAX_THREADS / 32];
    pdl_trigger();
    pdl_wait();                                        // the logits come from the kernel in front
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int begin = blockIdx.y * slice, end = min(limit, begin + slice);
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float x = row[i];
        if (x > v || (x == v && i < idx)) { v = x; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { best_v[warp] = v; best_i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = lane < ARGMAX_THREADS / 32 ? best_v[lane] : -INFINITY;
        idx = lane < ARGMAX_THREADS / 32 ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        if (lane == 0) {
            part_v[(size_t)blockIdx.x * parts + blockIdx.y] = v;
            part_i[(size_t)blockIdx.x * parts + blockIdx.y] = idx;
        }
    }
}

// Stage 2: one warp per row merges the parts.
__global__ void argmax_merge_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                    int* __restrict__ out, int parts) {
    float v = -INFINITY;
    int idx = 0x7fffffff;
    pdl_trigger();
    pdl_wait();
    for (int k = threadIdx.x; k < parts; k += 32) {
        const float x = part_v[(size_t)blockIdx.x * parts + k];
        const int i = part_i[(size_t)blockIdx.x * parts + k];
        if (x > v || (x == v && i < idx)) { v = x; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
}

// Stage 2 for many parts (hundreds, as the head projection leaves them): a block per row.
__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_merge_block_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int* __restrict__ out,
                          int parts) {
    __shared__ float best_v[ARGMAX_THREADS / 32];
    __shared__ int best_i[ARGMAX_THREADS / 32];
    float v = -INFINITY;
    int idx = 0x7fffffff;
    pdl_trigger();
    pdl_wait();
    for (int k = threadIdx.x; k < parts; k += ARGMAX_THREADS) {
        const float x = part_v[(size_t)blockIdx.x * parts + k];
        const int i = part_i[(size_t)blockIdx.x * parts + k];
        if (x > v || (x == v && i < idx)) { v = x; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { best_v[warp] = v; best_i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = lane < ARGMAX_THREADS / 32 ? best_v[lane] : -INFINITY;
        idx = lane < ARGMAX_THREADS / 32 ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
    }
}

constexpr int ARGMAX_SLICE = 2048;

}  // namespace

// Parts a row is cut into by mg_argmax_wide; its scratch holds rows * parts floats and as many ints.
MG_API int mg_argmax_parts(int vocab) { return (vocab + ARGMAX_SLICE - 1) / ARGMAX_SLICE; }

// logits: [rows, vocab] 32-bit; ids >= limit are never chosen (limit <= 0: the whole vocabulary).
MG_API int mg_argmax(const float* logits, int* out, int rows, int vocab, int limit, void* stream) {
    if (rows == 0) return MG_OK;
    MG_REQUIRE(rows > 0 && vocab > 0, "argmax: bad sizes");
    if (limit <= 0 || limit > vocab) limit = vocab;
    argmax_kernel<<<rows, ARGMAX_THREADS, 0, (cudaStream_t)stream>>>(logits, out, vocab, limit);
    MG_CHECK_LAUNCH("argmax");
    return MG_OK;
}

// The same result with many blocks per row, for wide vocabularies and few rows: a row is cut
// into slices of 2048 ids, each scanned by a block; a second kernel merges.  The lowest index
// among equal maxima wins, as in mg_argmax.  scratch_v / scratch_i: rows * mg_argmax_parts(vocab).
MG_API int mg_argmax_wide(const float* logits, int* out, float* scratch_v, int* scratch_i, int rows, int vocab,
                          int limit, void* stream) {
    if (rows == 0) return MG_OK;
    MG_REQUIRE(rows > 0 && vocab > 0 && scratch_v && scratch_i, "argmax: bad arguments");
    if (limit <= 0 || limit > vocab) limit = vocab;
    const int parts = mg_argmax_parts(vocab);
    MG_REQUIRE(parts <= 65535, "argmax: vocabulary too wide");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t le = mg_launch(argmax_part_kernel, dim3(rows, parts), dim3(ARGMAX_THREADS), 0, s, true, logits, scratch_v,
                               scratch_i, vocab, limit, parts, ARGMAX_SLICE);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "argmax (parts): %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("argmax (parts)");
    le = mg_launch(argmax_merge_kernel, dim3(rows), dim3(32), 0, s, true, (const float*)scratch_v, (const int*)scratch_i, out,
                   parts);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "argmax (merge): %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("argmax (merge)");
    return MG_OK;
}

// The second stage alone: part_v / part_i hold `parts` candidates per row (value and index, as
// the head projection leaves them when it takes the greedy choice on its way).
MG_API int mg_argmax_merge(const float* part_v, const int* part_i, int* out, int rows, int parts, void* stream) {
    if (rows == 0) return MG_OK;
    MG_REQUIRE(rows > 0 && parts > 0 && part_v && part_i && out, "argmax (merge): bad arguments");
    const cudaError_t le =
        parts > 64 ? mg_launch(argmax_merge_block_kernel, dim3(rows), dim3(ARGMAX_THREADS), 0, (cudaStream_t)stream, true,
                               part_v, part_i, out, parts)
                   : mg_launch(argmax_merge_kernel, dim3(rows), dim3(32), 0, (cudaStream_t)stream, true, part_v, part_i, out,
                               parts);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "argmax (merge): %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("argmax (merge)");
    return MG_OK;
}

// ---- stochastic sampling -------------------------------------------------------------------------
// One block per row.  The order is the reference's (src/minigpt_infer/sampling.py:116-137):
// logits / max(temperature, 1e-6), top-k (values below the k-th largest dropped, ties pass),
// top-p (sorted descending, a token is dropped if the probability mass strictly before it
// exceeds p; the largest always stays), softmax, one draw.  A row with temperature <= 0 is
// greedy.  Instead of sorting the row, both cut-offs are found by a radix descent over the
// order-preserving bit pattern of the scaled logits: 4 passes of 8 bits with a histogram of
// counts (top-k) or of probability mass (top-p) in shared memory.  Mass is accumulated as
// 64-bit fixed point with integer atomics, so the result does not depend on the order of the
// additions.  The draw is an inverse-CDF walk in index order with a Philox4x32-10 number keyed
// by (seed, counter): the same request at the same token draws the same number whatever else
// is in the batch (the reference shares one generator across the batch,
// src/minigpt_infer/engine/engine.py:13-17).
namespace {

constexpr int SAMPLE_THREADS = 512;
constexpr float FIXED_ONE = 1099511627776.0f;   // 2^40: e in [0, 1] -> fixed point

__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint32_t mulhi32(uint32_t a, uint32_t b) { return __umulhi(a, b); }

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"); first word.
__device__ uint32_t philox_first(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1) {
    uint32_t c[4] = {c0, c1, 0u, 0u};
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = mulhi32(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
        const uint32_t hi1 = mulhi32(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
        const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c[0];
}

__device__ float block_reduce_max(float v, float* scratch) {
    v = warp_max(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = lane < SAMPLE_THREADS / 32 ? scratch[lane] : -INFINITY;
        v = warp_max(v);
        if (lane == 0) scratch[0] = v;
    }
    __syncthreads();
    return scratch[0];
}

__device__ float block_reduce_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = lane < SAMPLE_THREADS / 32 ? scratch[lane] : 0.f;
        v = warp_sum(v);
        if (lane == 0) scratch[0] = v;
    }
    __syncthreads();
    return scratch[0];
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const uint32_t* __restrict__ seed_lo, const uint32_t* __restrict__ seed_hi,
              const uint32_t* __restrict__ counter, int* __restrict__ out, int vocab, int limit, int cached) {
    extern __shared__ float row_cache[];      // the scaled row, if the launch gave room for it
    __shared__ float scratch[SAMPLE_THREADS / 32];
    __shared__ unsigned long long hist[256];
    __shared__ uint32_t sh_prefix;
    __shared__ unsigned long long sh_acc;
    __shared__ int sh_found;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* lr = logits + (size_t)row * vocab;
    const float temp = temperature[row];

    if (temp <= 0.f) {   // greedy row: lowest index among the largest
        float v = -INFINITY;
        int idx = 0x7fffffff;
        for (int i = tid; i < limit; i += SAMPLE_THREADS) {
            const float x = lr[i];
            if (x > v || (x == v && i < idx)) { v = x; idx = i; }
        }
        const float best = block_reduce_max(v, scratch);
        if (tid == 0) sh_found = 0x7fffffff;
        __syncthreads();
        if (v == best && idx != 0x7fffffff) atomicMin(&sh_found, idx);
        __syncthreads();
        if (tid == 0) out[row] = sh_found == 0x7fffffff ? 0 : sh_found;
        return;
    }

    const float safe_t = fmaxf(temp, 1e-6f);
    // One pass over global memory: the scaled row goes to shared memory (a 50304-wide row is
    // 197 KB and fits), every later pass reads it from there.
    float mx = -INFINITY;
    for (int i = tid; i < limit; i += SAMPLE_THREADS) {
        const float x = lr[i] / safe_t;
        if (cached) row_cache[i] = x;
        mx = fmaxf(mx, x);
    }
    mx = block_reduce_max(mx, scratch);     // (its barriers also publish row_cache)
#define ROW(i) (cached ? row_cache[i] : lr[i] / safe_t)

    // top-k: key of the k-th largest scaled logit
    uint32_t thr_key = 0u;
    const int k = top_k ? top_k[row] : 0;
    if (k > 0 && k < limit) {
        uint32_t prefix = 0u, mask = 0u;
        unsigned long long remaining = (unsigned long long)k;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) hist[tid] = 0ull;
            __syncthreads();
            for (int i = tid; i < limit; i += SAMPLE_THREADS) {
                const uint32_t key = order_key(ROW(i));
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1ull);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long cum = 0ull;
                int digit = 0;
                for (int b = 255; b >= 0; --b) {
                    if (cum + hist[b] >= remaining) { digit = b; break; }
                    cum += hist[b];
                }
                sh_prefix = prefix | ((uint32_t)digit << shift);
                sh_acc = remaining - cum;
            }
            __syncthreads();
            prefix = sh_prefix;
            remaining = sh_acc;
            mask |= 255u << shift;
            __syncthreads();
        }
        thr_key = prefix;
    }

    // top-p: lowest key whose mass of strictly larger keys is <= p * (mass kept by top-k)
    const float p = top_p ? top_p[row] : 1.f;
    if (p < 1.f) {
        float part = 0.f;
        for (int i = tid; i < limit; i += SAMPLE_THREADS) {
            const float x = ROW(i);
            if (order_key(x) >= thr_key) part += expf(x - mx);
        }
        const float z_k = block_reduce_sum(part, scratch);
        const unsigned long long target = (unsigned long long)((double)p * (double)z_k * (double)FIXED_ONE);
        uint32_t prefix = 0u, mask = 0u;
        unsigned long long acc = 0ull;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) hist[tid] = 0ull;
            __syncthreads();
            for (int i = tid; i < limit; i += SAMPLE_THREADS) {
                const float x = ROW(i);
                const uint32_t key = order_key(x);
                if (key >= thr_key && (key & mask) == prefix) {
                    // + 1 so that a token whose probability underflows still marks its bin
                    const unsigned long long e = (unsigned long long)(expf(x - mx) * FIXED_ONE) + 1ull;
                    atomicAdd(&hist[(key >> shift) & 255u], e);
                }
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long run = acc, chosen_acc = acc;
                int digit = -1;
                for (int b = 255; b >= 0; --b) {
                    if (hist[b] == 0ull) continue;
                    if (run > target && digit >= 0) break;
                    if (run <= target || digit < 0) { digit = b; chosen_acc = run; }
                    run += hist[b];
                }
                sh_prefix = prefix | ((uint32_t)(digit < 0 ? 0 : digit) << shift);
                sh_acc = chosen_acc;
            }
            __syncthreads();
            prefix = sh_prefix;
            acc = sh_acc;
            mask |= 255u << shift;
            __syncthreads();
        }
        if (prefix > thr_key) thr_key = prefix;
    }

    // normaliser of what is kept, then the inverse-CDF walk in index order
    float part = 0.f;
    for (int i = tid; i < limit; i += SAMPLE_THREADS) {
        const float x = ROW(i);
        if (order_key(x) >= thr_key) part += expf(x - mx);
    }
    const float z = block_reduce_sum(part, scratch);
    const uint32_t rnd = philox_first(seed_lo[row], seed_hi[row], counter[row], 0u);
    const float u = (float)(rnd >> 8) * (1.0f / 16777216.0f);      // [0, 1)
    const float target = u * z;

    if (tid == 0) sh_found = 0x7fffffff;
    __syncthreads();
    float base = 0.f;
    int last_kept = -1;
    const int warp = tid >> 5, lane = tid & 31;
    for (int t0 = 0; t0 < limit; t0 += SAMPLE_THREADS) {
        const int i = t0 + tid;
        float e = 0.f;
        if (i < limit) {
            const float x = ROW(i);
            if (order_key(x) >= thr_key) { e = expf(x - mx); if (e > 0.f) last_kept = i; }
        }
        float incl = e;                                            // inclusive scan in the warp
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        __syncthreads();
        if (lane == 31) scratch[warp] = incl;
        __syncthreads();
        float before = 0.f, total = 0.f;
        for (int w = 0; w < SAMPLE_THREADS / 32; ++w) {
            const float s = scratch[w];
            if (w < warp) before += s;
            total += s;
        }
        const float cum = base + before + incl;
        if (e > 0.f && cum > target) atomicMin(&sh_found, i);
        __syncthreads();
        if (sh_found != 0x7fffffff) break;
        base += total;
    }
    if (sh_found == 0x7fffffff) {                                  // rounding left the target just above the sum
        __syncthreads();
        if (tid == 0) sh_found = -1;
        __syncthreads();
        if (last_kept >= 0) atomicMax(&sh_found, last_kept);
        __syncthreads();
    }
    if (tid == 0) out[row] = sh_found < 0 ? 0 : sh_found;
#undef ROW
}

}  // namespace

// temperature: [rows]; top_k: [rows] int (<= 0: off) or null; top_p: [rows] (>= 1: off) or null;
// seed_lo/seed_hi/counter: [rows] 32-bit words of each row's seed and of its draw number.
MG_API int mg_sample(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                     const uint32_t* seed_lo, const uint32_t* seed_hi, const uint32_t* counter, int* out,
                     int rows, int vocab, int limit, void* stream) {
    if (rows == 0) return MG_OK;
    MG_REQUIRE(rows > 0 && vocab > 0, "sample: bad sizes");
    MG_REQUIRE(temperature && seed_lo && seed_hi && counter, "sample: missing per-row parameters");
    if (limit <= 0 || limit > vocab) limit = vocab;
    const size_t row_bytes = (size_t)limit * sizeof(float);
    const int cached = row_bytes <= 220 * 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "sample: cannot raise shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    sample_kernel<<<rows, SAMPLE_THREADS, cached ? row_bytes : 0, (cudaStream_t)stream>>>(
        logits, temperature, top_k, top_p, seed_lo, seed_hi, counter, out, vocab, limit, cached);
    MG_CHECK_LAUNCH("sample");
    return MG_OK;
}
