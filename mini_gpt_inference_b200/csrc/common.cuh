// Shared helpers of the sm_100a kernel library: error reporting, type conversion, reductions.
//
// Every exported function is plain C (`extern "C"`), takes raw device pointers and a
// stream, launches asynchronously and returns 0, or a negative code after storing a
// message that `mg_last_error()` returns.  Nothing here allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MG_OK 0
#define MG_ERR_ARG -1
#define MG_ERR_CUDA -2
#define MG_ERR_UNSUPPORTED -3

#define MG_API extern "C" __attribute__((visibility("default")))

int mg_set_error(int code, const char* fmt, ...);

#define MG_REQUIRE(cond, ...)                                   \
    do {                                                        \
        if (!(cond)) return mg_set_error(MG_ERR_ARG, __VA_ARGS__); \
    } while (0)

#define MG_CHECK_LAUNCH(name)                                                       \
    do {                                                                            \
        cudaError_t e_ = cudaGetLastError();                                        \
        if (e_ != cudaSuccess)                                                      \
            return mg_set_error(MG_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e_)); \
    } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Four consecutive outputs at once (16 bytes of 32-bit values, 8 bytes of bfloat16).
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// LayerNorm of one row by one warp, for any width that is a multiple of 4: the row is read three
// times in chunks of 1024 values with 16-byte loads (the second and third time it comes from the
// L1 cache): the mean, then the biased variance of the centred values, then the affine map.
// gain and shift (shift may be null) in global or shared memory; src, gain, shift and dst
// 16-byte aligned (dst 8 for bfloat16).  A row's result depends on nothing but the row.
template <typename TOut>
__device__ __forceinline__ void layernorm_row_chunked(const float* src, int width, const float* gain, const float* shift,
                                                      float eps, TOut* dst, int lane) {
    const float4* src4 = reinterpret_cast<const float4*>(src);
    const int n4 = width / 4;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float sum = 0.f;
    for (int i0 = 0; i0 < n4; i0 += 256) {
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = i0 + lane + 32 * i;
            v[i] = c < n4 ? src4[c] : zero;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = warp_sum(sum) / (float)width;
    float sq = 0.f;
    for (int i0 = 0; i0 < n4; i0 += 256) {
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = i0 + lane + 32 * i;
            v[i] = c < n4 ? src4[c] : make_float4(mean, mean, mean, mean);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
            sq += (dx * dx + dy * dy) + (dz * dz + dw * dw);
        }
    }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)width + eps);
    for (int i0 = 0; i0 < n4; i0 += 256) {
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = i0 + lane + 32 * i;
            v[i] = c < n4 ? src4[c] : zero;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = i0 + lane + 32 * i;
            if (c < n4) {
                const float4 gn = reinterpret_cast<const float4*>(gain)[c];
                const float4 sh = shift ? reinterpret_cast<const float4*>(shift)[c] : zero;
                store4(dst + 4 * c, (v[i].x - mean) * rstd * gn.x + sh.x, (v[i].y - mean) * rstd * gn.y + sh.y,
                       (v[i].z - mean) * rstd * gn.z + sh.z, (v[i].w - mean) * rstd * gn.w + sh.w);
            }
        }
    }
}

// LayerNorm gain and shift (shift may be null: zeros) from global to shared memory by all `threads`
// threads of a CTA: a thread asks for all its values (of up to two rounds) before it stores the
// first, so that they cost one trip to memory, not one per value.  n4: floats / 4; 16-byte aligned.
__device__ __forceinline__ void stage_gain_shift(float* gain_s, float* shift_s, const float* gain, const float* shift,
                                                 int n4, int tid, int threads) {
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i0 = tid; i0 < n4; i0 += 2 * threads) {
        const int i1 = i0 + threads;
        const float4 g0 = reinterpret_cast<const float4*>(gain)[i0];
        const float4 s0 = shift ? reinterpret_cast<const float4*>(shift)[i0] : zero;
        const float4 g1 = i1 < n4 ? reinterpret_cast<const float4*>(gain)[i1] : zero;
        const float4 s1 = (i1 < n4 && shift) ? reinterpret_cast<const float4*>(shift)[i1] : zero;
        reinterpret_cast<float4*>(gain_s)[i0] = g0;
        reinterpret_cast<float4*>(shift_s)[i0] = s0;
        if (i1 < n4) {
            reinterpret_cast<float4*>(gain_s)[i1] = g1;
            reinterpret_cast<float4*>(shift_s)[i1] = s1;
        }
    }
}

// tanh-GELU evaluated in 32-bit: 0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3))).
__device__ __forceinline__ float gelu_tanh(float u) {
    const float k = 0.7978845608028654f;  // sqrt(2/pi)
    return 0.5f * u * (1.0f + tanhf(k * (u + 0.044715f * u * u * u)));
}

// tanh-GELU with the hardware's tanh (one instruction, relative error about 2^-11): for results that
// are rounded to bfloat16 (2^-8) right away, where the exact tanhf costs twenty times the instructions.
__device__ __forceinline__ float gelu_tanh_fast(float u) {
    const float k = 0.7978845608028654f;  // sqrt(2/pi)
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(k * (u + 0.044715f * u * u * u)));
    return 0.5f * u * (1.0f + th);
}

// 2^x as one instruction of the special-function unit (two units in the last place; results
// below the smallest normal number become zero).  For softmax weights, whose argument is <= 0 and
// whose result is rounded to bfloat16 or summed in 32-bit right away.
__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- programmatic dependent launch ---------------------------------------------------------
// A kernel launched with mg_launch(..., dependent = true) may start while the kernel before it on
// the stream is still running; it must call pdl_wait() before it reads anything that kernel
// wrote and before it writes anything at all.  What it does before that (index arithmetic,
// loads of weights) overlaps the predecessor's tail.  pdl_trigger() tells the successor that it
// may start.  Both are no-ops when the launch carries no such dependency.  The host switch
// mg_set_dependent_launch() turns the launch attribute on (used while a decode step is captured
// into a CUDA graph, where every predecessor is a kernel).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

int mg_dependent_launch_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t mg_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    bool dependent, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (dependent && mg_dependent_launch_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// ---- index guards (guarded builds only) ------------------------------------------------------------
// Token ids, positions, cache rows, page numbers and request numbers reach the kernels through device
// memory; the host checks them before every launch, and ordinary builds trust it.  With -DMG_GUARDS
// the kernels check them again where they use them: MG_GUARDED(name, code, value, limit) is true if
// 0 <= value < limit; else it records the first such fault of the kernel file (code, value, limit,
// block) and is false, and the caller skips the access or takes index 0 instead, so that a guarded
// build never reads or writes outside a table.  mg_<name>_index_fault() hands the record to the host
// and clears it.  In ordinary builds the macro is the constant true, the limits are unused
// parameters, and the exported reader reports nothing.
#define MG_GUARD_TOKEN 1        // token id >= vocabulary
#define MG_GUARD_POSITION 2     // position beyond the position table or the block table
#define MG_GUARD_CACHE_ROW 3    // cache row (page * page size + offset) beyond the pool
#define MG_GUARD_PAGE 4         // page number beyond the pool
#define MG_GUARD_REQUEST 5      // request number beyond the block tables' rows
#define MG_GUARD_ROW 6          // row index beyond the tensor gathered from
#define MG_GUARD_SOURCE 7       // index into the ids of the step before
#ifdef MG_GUARDS
struct MgIndexFault {
    int code;
    int block;
    long long value;
    long long limit;
};
__device__ __forceinline__ bool mg_guarded(MgIndexFault* fault, int code, long long value, long long limit) {
    if (value >= 0 && value < limit) return true;
    if (atomicCAS(&fault->code, 0, code) == 0) {
        fault->block = (int)blockIdx.x;
        fault->value = value;
        fault->limit = limit;
    }
    return false;
}
#define MG_GUARD_RECORD(var) static __device__ MgIndexFault var;
#define MG_GUARD_EXPORT(name, var)                                                                  \
    MG_API int mg_##name##_index_fault(long long* host) {                                           \
        MgIndexFault f, none = {0, 0, 0, 0};                                                        \
        if (cudaMemcpyFromSymbol(&f, var, sizeof(f)) != cudaSuccess ||                              \
            cudaMemcpyToSymbol(var, &none, sizeof(none)) != cudaSuccess)                            \
            return mg_set_error(MG_ERR_CUDA, "cannot read the index guard of " #name);              \
        host[0] = f.code; host[1] = f.block; host[2] = f.value; host[3] = f.limit;                  \
        return MG_OK;                                                                               \
    }
#define MG_GUARDED_IN(var, code, value, limit) mg_guarded(&var, (code), (long long)(value), (long long)(limit))
#else
#define MG_GUARD_RECORD(var)
#define MG_GUARD_EXPORT(name, var)                                                                  \
    MG_API int mg_##name##_index_fault(long long* host) {                                           \
        host[0] = host[1] = host[2] = host[3] = 0;                                                  \
        return MG_OK;                                                                               \
    }
#define MG_GUARDED_IN(var, code, value, limit) (true)
#endif
// a kernel file's own record and its reader, and the check against it
#define MG_GUARD_DECLARE(name) MG_GUARD_RECORD(name##_index_fault) MG_GUARD_EXPORT(name, name##_index_fault)
#define MG_GUARDED(name, code, value, limit) MG_GUARDED_IN(name##_index_fault, code, value, limit)

// ---- phase stamps (tracing builds only) ----------------------------------------------------------
// With -DMG_STAMPS a kernel file keeps a small device array of clock readings: thread 0 of each CTA
// records, at MG_STAMP(name, 0), the global nanosecond timer (one clock for all SMs and kernels) in
// slot 0 and its SM's cycle counter in slot 1, and at every other MG_STAMP(name, slot) the cycle
// counter (cheap to read, so the stamps hardly disturb what they measure; slot 1 is reserved).  An
// exported mg_<name>_stamps() copies the array to the host: where a kernel's time goes, and how long
// the hand-over between two kernels takes.
// In ordinary builds the macros expand to nothing.
#ifdef MG_STAMPS
#define MG_STAMP_SLOTS 12
#define MG_STAMP_CTAS 1024
#define MG_STAMP_DECLARE(name)                                                                      \
    static __device__ long long name##_stamp_buf[MG_STAMP_CTAS * MG_STAMP_SLOTS];                   \
    MG_API int mg_##name##_stamps(long long* host, int ctas) {                                      \
        if (ctas > MG_STAMP_CTAS) ctas = MG_STAMP_CTAS;                                             \
        return cudaMemcpyFromSymbol(host, name##_stamp_buf, sizeof(long long) * ctas * MG_STAMP_SLOTS) == cudaSuccess \
                   ? MG_OK : MG_ERR_CUDA;                                                           \
    }
#define MG_STAMP(name, slot)                                                                        \
    do {                                                                                            \
        if (threadIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && blockIdx.x < MG_STAMP_CTAS) {  \
            long long t_;                                                                           \
            if ((slot) == 0) {                                                                      \
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                              \
                name##_stamp_buf[blockIdx.x * MG_STAMP_SLOTS] = t_;                                 \
                name##_stamp_buf[blockIdx.x * MG_STAMP_SLOTS + 1] = clock64();                      \
            } else {                                                                                \
                name##_stamp_buf[blockIdx.x * MG_STAMP_SLOTS + (slot)] = clock64();                 \
            }                                                                                       \
        }                                                                                           \
    } while (0)
// the same from whichever single thread calls it (slots other than 0 and 1)
#define MG_STAMP_HERE(name, slot)                                                                   \
    do {                                                                                            \
        if (blockIdx.y == 0 && blockIdx.z == 0 && blockIdx.x < MG_STAMP_CTAS)                       \
            name##_stamp_buf[blockIdx.x * MG_STAMP_SLOTS + (slot)] = clock64();                     \
    } while (0)
#define MG_STAMP_HERE_LANE0(name, slot)                                                             \
    do {                                                                                            \
        if ((threadIdx.x & 31) == 0) MG_STAMP_HERE(name, slot);                                     \
    } while (0)
#else
#define MG_STAMP_DECLARE(name)
#define MG_STAMP(name, slot) do {} while (0)
#define MG_STAMP_HERE(name, slot) do {} while (0)
#define MG_STAMP_HERE_LANE0(name, slot) do {} while (0)
#endif
