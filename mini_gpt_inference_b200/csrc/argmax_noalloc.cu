// Greedy choice over wide vocabularies without any allocation (see no_alloc.h for who needs it).
//
// Same two stages as the wide argmax of sampling.cu — blocks scan slices of 2048 ids, one warp
// per row merges — with the slice results kept in a file-scope device array.  In host code the
// array's name is only a handle: its device address is fetched once per device with
// cudaGetSymbolAddress and that pointer is what the kernels receive.
#include <math.h>

#include <mutex>

#include "common.cuh"
#include "no_alloc.h"

namespace {

constexpr int THREADS = 256;
constexpr int SLICE = 2048;
constexpr int MAX_DEVICES = 64;

struct __align__(8) Part {
    float value;
    int index;
};

// The scratch: one (value, index) per (row, slice).  64 KiB per GPU, for the life of the process.
static __device__ __align__(256) Part g_parts[MG_NOALLOC_MAX_PARTS];

__device__ __forceinline__ void keep_better(float& v, int& idx, float ov, int oi) {
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
}

__global__ void __launch_bounds__(THREADS)
noalloc_part_kernel(const float* __restrict__ logits, Part* __restrict__ parts, int vocab, int limit, int n_parts) {
    __shared__ float best_v[THREADS / 32];
    __shared__ int best_i[THREADS / 32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int begin = blockIdx.y * SLICE, end = min(limit, begin + SLICE);
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) keep_better(v, idx, row[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        keep_better(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { best_v[warp] = v; best_i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = lane < THREADS / 32 ? best_v[lane] : -INFINITY;
        idx = lane < THREADS / 32 ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            keep_better(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
        // every slot that the merge reads is written here, whatever the last call left in it
        if (lane == 0) parts[(size_t)blockIdx.x * n_parts + blockIdx.y] = Part{v, idx};
    }
}

__global__ void noalloc_merge_kernel(const Part* __restrict__ parts, int* __restrict__ out, int n_parts) {
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int k = threadIdx.x; k < n_parts; k += 32) {
        const Part p = parts[(size_t)blockIdx.x * n_parts + k];
        keep_better(v, idx, p.value, p.index);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        keep_better(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if (threadIdx.x == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
}

// Device address of g_parts on the current device, looked up once per device.
int scratch_pointer(Part** out) {
    static Part* pointers[MAX_DEVICES] = {};
    static std::mutex mu;
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "argmax (no alloc): cudaGetDevice: %s", cudaGetErrorString(e));
    if (device < 0 || device >= MAX_DEVICES) return mg_set_error(MG_ERR_ARG, "argmax (no alloc): device %d out of range", device);
    std::lock_guard<std::mutex> lock(mu);
    if (pointers[device] == nullptr) {
        Part* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_parts);      // the symbol of the device that is current now
        if (e != cudaSuccess || p == nullptr)
            return mg_set_error(MG_ERR_CUDA, "argmax (no alloc): cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        pointers[device] = p;
    }
    *out = pointers[device];
    return MG_OK;
}

}  // namespace

MG_API int mg_argmax_wide_noalloc(const float* logits, int* out, int rows, int vocab, int limit, void* stream) {
    if (rows == 0) return MG_OK;
    MG_REQUIRE(logits != nullptr && out != nullptr, "argmax (no alloc): missing input or output");
    MG_REQUIRE(rows > 0 && vocab > 0, "argmax (no alloc): bad sizes rows=%d vocab=%d", rows, vocab);
    const int n_parts = (vocab + SLICE - 1) / SLICE;
    MG_REQUIRE((long long)rows * n_parts <= MG_NOALLOC_MAX_PARTS && n_parts <= 65535,
               "argmax (no alloc): rows * ceil(vocab / %d) = %lld exceeds the built-in scratch of %d entries",
               SLICE, (long long)rows * n_parts, MG_NOALLOC_MAX_PARTS);
    if (limit <= 0 || limit > vocab) limit = vocab;
    Part* parts = nullptr;
    const int rc = scratch_pointer(&parts);
    if (rc != MG_OK) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    noalloc_part_kernel<<<dim3(rows, n_parts), THREADS, 0, s>>>(logits, parts, vocab, limit, n_parts);
    MG_CHECK_LAUNCH("argmax (no alloc, parts)");
    noalloc_merge_kernel<<<rows, 32, 0, s>>>(parts, out, n_parts);
    MG_CHECK_LAUNCH("argmax (no alloc, merge)");
    return MG_OK;
}
