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

}  // namespace

// logits: [rows, vocab] 32-bit; ids >= limit are never chosen (limit <= 0: the whole vocabulary).
MG_API int mg_argmax(const float* logits, int* out, int rows, int vocab, int limit, void* stream) {
    if (rows == 0) return MG_OK;
    MG_REQUIRE(rows > 0 && vocab > 0, "argmax: bad sizes");
    if (limit <= 0 || limit > vocab) limit = vocab;
    argmax_kernel<<<rows, ARGMAX_THREADS, 0, (cudaStream_t)stream>>>(logits, out, vocab, limit);
    MG_CHECK_LAUNCH("argmax");
    return MG_OK;
}
