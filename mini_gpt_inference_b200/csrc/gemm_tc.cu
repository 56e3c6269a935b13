// bfloat16 matrix product on the 5th-generation tensor cores: TMA -> shared memory ->
// tcgen05.mma -> TMEM -> epilogue.
//
//   D[p, q] = sum_k P[p, k] * Q[q, k]        P: [rows_p, K], Q: [rows_q, K], both K-major bf16
//
// One CTA computes a 128 x BN tile of D.  Thread 0 is the producer: it arms a "full"
// mbarrier with the bytes to come and issues two TMA tile loads (128 x 64 of P, BN x 64 of
// Q, 128-byte swizzle) per k block into a ring of stages.  Thread 32 is the issuer: it waits
// for a stage, issues four tcgen05.mma (K = 16 each) whose 32-bit accumulator lives in TMEM,
// and commits them to the stage's "empty" mbarrier, which frees the stage when the tensor
// core has read it.  After the last k block a commit to a third barrier tells all four warps
// that the accumulator is complete; each warp reads its 32 TMEM lanes with tcgen05.ld and
// applies the epilogue: bias, tanh-GELU, conversion, or an add into the 32-bit residual
// stream.  Edges need no special case on the load side: TMA fills what lies outside the
// matrices with zeros (also a K that is no multiple of 64); stores are predicated.
//
// Two orientations share the kernel.  For many tokens, P is the activations and Q the weights
// (a thread ends up with one token's row of features).  For a few tokens (decoding), P is
// the weights and Q the activations: the 128 rows of the tensor-core tile are filled with
// weight rows and the batch sits on the narrow side (BN = 16, 32 or 64), so no tensor-core
// work is wasted on padding and a CTA streams 128 x K weights.
//
// Every wait on an mbarrier is bounded.  If one runs out, the kernel records a code in
// `status`, skips the rest of its work, waits a moment for copies in flight, frees its TMEM
// and returns; the host reads `status` later.  No thread-block clusters and no multicast
// are used: each CTA loads its own tiles.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "blackwell.cuh"
#include "tensor_map.cuh"

MG_STAMP_DECLARE(gemm)
MG_GUARD_DECLARE(linear_tc)

#define EPI_STORE 0
#define EPI_GELU 1
#define EPI_RESIDUAL 2

namespace {

constexpr int TILE_P = 128;         // rows of P per CTA = UMMA M
constexpr int BLOCK_K = 64;         // bf16 elements per k block = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int MAX_STAGES = 8;
constexpr int P_TILE_BYTES = TILE_P * BLOCK_K * 2;

struct __align__(8) Barriers {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t accumulator;
    uint32_t tmem_base;
    uint32_t failed;
};

// Where the QKV projection also leaves the key and value features of each token: its row of
// the paged cache.  k_pages null: no such copy.
struct KvSink {
    bf16* k_pages;
    bf16* v_pages;
    const int* slots;                // [tokens] flat cache row, < 0: skip
    int q_width, n_kv_head, head_dim, page_tokens;
    int num_pages;                   // pages of the pool (what a cache row is held against in guarded builds)
};

// First element of feature n (>= q_width) of the token in cache row `slot`; *is_value says which array.
__device__ __forceinline__ size_t kv_sink_index(const KvSink& k, int slot, int n, bool* is_value) {
    const int kv_width = k.n_kv_head * k.head_dim;
    const int f = n - k.q_width;
    const int which = f / kv_width, fi = f - which * kv_width;
    const int h = fi / k.head_dim, d = fi - h * k.head_dim;
    const int page = slot / k.page_tokens, off = slot - page * k.page_tokens;
    *is_value = which != 0;
    return (((size_t)page * k.n_kv_head + h) * k.page_tokens + off) * k.head_dim + d;
}

template <int BN, bool SWAP>
__global__ void __launch_bounds__(128)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
               const float* __restrict__ bias, void* __restrict__ out_ptr, float* __restrict__ residual,
               int rows_p, int rows_q, int K, int ld_out, int epilogue, int out_bf16, int stages,
               const KvSink sink, int* __restrict__ status) {
    constexpr int Q_TILE_BYTES = BN * BLOCK_K * 2;
    constexpr int STAGE_BYTES = P_TILE_BYTES + Q_TILE_BYTES;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzle wants tiles aligned to 1024 bytes
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Barriers* bars = (Barriers*)(smem + (size_t)stages * STAGE_BYTES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int p0 = blockIdx.x * TILE_P, q0 = blockIdx.y * BN;
    const int num_kb = (K + BLOCK_K - 1) / BLOCK_K;
    // The epilogue's operands are asked for while the main loop runs: the tile's slice of the
    // bias goes to shared memory, the thread's row of the residual stream is pulled towards L2.
    __shared__ __align__(16) float bias_tile[BN];
    int cache_row = -1;                                   // of this thread's token (not SWAP)
    if (!SWAP) {
        if (sink.k_pages != nullptr && p0 + tid < rows_p) cache_row = sink.slots[p0 + tid];
        // (guarded builds: a row beyond the pool is recorded and its keys and values are not copied)
        if (cache_row >= 0 && !MG_GUARDED(linear_tc, MG_GUARD_CACHE_ROW, cache_row, (long long)sink.num_pages * sink.page_tokens))
            cache_row = -1;
        for (int j = tid; j < BN; j += 128) bias_tile[j] = (bias && q0 + j < rows_q) ? bias[q0 + j] : 0.f;
        if (epilogue == EPI_RESIDUAL && p0 + tid < rows_p) {
            const float* rrow = residual + (size_t)(p0 + tid) * ld_out + q0;
            for (int j = 0; j < BN && q0 + j < rows_q; j += 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(rrow + j));
        }
    }

    MG_STAMP(gemm, 0);
    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        mbar_init(smem_u32(&bars->accumulator), 1);
        bars->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&bars->tmem_base), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    // Barriers, tensor memory and the bias are set up while the kernel in front drains; its
    // results (the activations, the residual stream) are touched only from here on.
    MG_STAMP(gemm, 2);
    pdl_trigger();
    // The weights do not come from the kernel in front: their tiles of the first round of stages are
    // asked for before the wait (tokens x weights: the q operand; weights x tokens: the p operand).
    const int early = num_kb < stages ? num_kb : stages;
    if (tid == 0) {
        for (int kb = 0; kb < early; ++kb) {
            const uint32_t full = smem_u32(&bars->full[kb]);
            mbar_expect_tx(full, STAGE_BYTES);
            uint8_t* stage = smem + (size_t)kb * STAGE_BYTES;
            if (SWAP) tma_load_2d(smem_u32(stage), &map_p, full, kb * BLOCK_K, p0);
            else tma_load_2d(smem_u32(stage + P_TILE_BYTES), &map_q, full, kb * BLOCK_K, q0);
        }
    }
    pdl_wait();
    MG_STAMP(gemm, 3);

    if (tid == 0) {
        // ---- producer: TMA loads into the ring of stages ----
        for (int kb = 0; kb < num_kb; ++kb) {
            const int s = kb % stages;
            const uint32_t full = smem_u32(&bars->full[s]);
            uint8_t* stage = smem + (size_t)s * STAGE_BYTES;
            if (kb < early) {                             // the weights' tile is on its way already
                if (SWAP) tma_load_2d(smem_u32(stage + P_TILE_BYTES), &map_q, full, kb * BLOCK_K, q0);
                else tma_load_2d(smem_u32(stage), &map_p, full, kb * BLOCK_K, p0);
                continue;
            }
            if (!mbar_wait(smem_u32(&bars->empty[s]), ((kb / stages) & 1) ^ 1)) {
                atomicExch(status, 1);
                bars->failed = 1;
                break;
            }
            mbar_expect_tx(full, STAGE_BYTES);
            tma_load_2d(smem_u32(stage), &map_p, full, kb * BLOCK_K, p0);
            tma_load_2d(smem_u32(stage + P_TILE_BYTES), &map_q, full, kb * BLOCK_K, q0);
        }
        MG_STAMP(gemm, 4);
    } else if (tid == 32) {
        // ---- issuer: tcgen05.mma over the stages, accumulator in TMEM ----
        constexpr uint32_t idesc = instr_desc_bf16(TILE_P, BN);
        bool ok = true;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
            const int s = kb % stages;
            if (!mbar_wait(smem_u32(&bars->full[s]), (kb / stages) & 1)) {
                atomicExch(status, 2);
                bars->failed = 1;
                ok = false;
                break;
            }
            tc_fence_after();
            uint8_t* stage = smem + (size_t)s * STAGE_BYTES;
            const uint64_t desc_p = smem_desc_sw128(smem_u32(stage));
            const uint64_t desc_q = smem_desc_sw128(smem_u32(stage + P_TILE_BYTES));
#pragma unroll
            for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                // 16 elements further along K: 32 bytes inside the swizzled row
                const uint64_t step = (uint64_t)((k * UMMA_K * 2) >> 4);
                umma_bf16(tmem_base, desc_p + step, desc_q + step, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(smem_u32(&bars->empty[s]));
        }
        umma_commit(smem_u32(&bars->accumulator));
    }
    __syncwarp();

    // ---- epilogue: all four warps, each on its own 32 lanes of TMEM ----
    bool good = mbar_wait(smem_u32(&bars->accumulator), 0);
    if (!good) atomicExch(status, 3);
    good = good && (*(volatile uint32_t*)&bars->failed == 0);
    good = __all_sync(0xffffffffu, good);               // tcgen05.ld needs the whole warp
    tc_fence_after();
    MG_STAMP(gemm, 5);
    if (good) {
        const int p = p0 + warp * 32 + lane;             // this thread's row of D
        // first element of the token's cache row for kv head 0: [page][kv head][offset in page][feature]
        long long kv_row_base = 0;
        if (cache_row >= 0) {
            const int page = cache_row / sink.page_tokens;
            kv_row_base = (long long)page * sink.n_kv_head * sink.page_tokens + (cache_row - page * sink.page_tokens);
        }
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        constexpr int CHUNK = BN < 32 ? BN : 32;
        // one chunk of the accumulator (this thread's row, CHUNK columns from c0) through the epilogue
        auto finish_chunk = [&](const uint32_t (&r)[32], const int c0) {
            if (p < rows_p) {
                if (!SWAP) {
                    // p is a token, q runs over features: contiguous in the output row
                    const size_t row = (size_t)p * ld_out;
                    const int qc = q0 + c0;
                    const bool full = (CHUNK == 32) && (qc + CHUNK <= rows_q) && (ld_out % 8 == 0);
                    if (full) {
                        // whole chunk inside the matrix and 16-byte aligned: vector loads and stores
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 b4 = *reinterpret_cast<const float4*>(bias_tile + c0 + j);
                            v[j] = __uint_as_float(r[j]) + b4.x;
                            v[j + 1] = __uint_as_float(r[j + 1]) + b4.y;
                            v[j + 2] = __uint_as_float(r[j + 2]) + b4.z;
                            v[j + 3] = __uint_as_float(r[j + 3]) + b4.w;
                        }
                        if (epilogue == EPI_GELU) {
                            // results that become bfloat16 take the hardware tanh; 32-bit results the exact one
                            if (out_bf16) {
#pragma unroll
                                for (int j = 0; j < 32; ++j) v[j] = gelu_tanh_fast(v[j]);
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
                            }
                        }
                        if (epilogue == EPI_RESIDUAL) {
                            // all loads first, then the adds and stores: a load after a store to the
                            // same array cannot be moved up by the compiler, and eight dependent
                            // round trips to memory would follow one another
                            float4* dst = reinterpret_cast<float4*>(residual + row + qc);
                            float4 old[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) old[j] = dst[j];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                float4 o = old[j];
                                o.x += v[4 * j]; o.y += v[4 * j + 1]; o.z += v[4 * j + 2]; o.w += v[4 * j + 3];
                                dst[j] = o;
                            }
                        } else if (out_bf16) {
                            uint4* dst = reinterpret_cast<uint4*>((bf16*)out_ptr + row + qc);
                            int kv_which = 0, kv_h = 0, kv_d = -1;        // -1: not worked out for this chunk yet
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]);
                                __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
                                __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
                                uint4 o;
                                o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
                                o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
                                dst[j] = o;
                                if (cache_row >= 0 && qc + 8 * j >= sink.q_width) {
                                    // eight features of one head (head sizes are multiples of 8 here); the
                                    // place of the chunk's first such group is worked out once, the groups
                                    // after it step through the head, the heads and from keys to values
                                    if (kv_d < 0) {
                                        const int f = qc + 8 * j - sink.q_width, kv_width = sink.n_kv_head * sink.head_dim;
                                        kv_which = f >= kv_width ? 1 : 0;
                                        const int fi = f - kv_which * kv_width;
                                        kv_h = fi / sink.head_dim;
                                        kv_d = fi - kv_h * sink.head_dim;
                                    } else {
                                        kv_d += 8;
                                        if (kv_d >= sink.head_dim) {
                                            kv_d = 0;
                                            if (++kv_h == sink.n_kv_head) { kv_h = 0; kv_which = 1; }
                                        }
                                    }
                                    const size_t at = ((size_t)kv_row_base + (size_t)kv_h * sink.page_tokens) * sink.head_dim + kv_d;
                                    *reinterpret_cast<uint4*>((kv_which ? sink.v_pages : sink.k_pages) + at) = o;
                                }
                            }
                        } else {
                            float4* dst = reinterpret_cast<float4*>((float*)out_ptr + row + qc);
#pragma unroll
                            for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < CHUNK; ++j) {
                            const int q = qc + j;
                            if (q < rows_q) {
                                float v = __uint_as_float(r[j]) + bias_tile[c0 + j];
                                if (epilogue == EPI_GELU) v = gelu_tanh(v);
                                if (epilogue == EPI_RESIDUAL) residual[row + q] += v;
                                else if (out_bf16) {
                                    const bf16 hv = __float2bfloat16_rn(v);
                                    ((bf16*)out_ptr)[row + q] = hv;
                                    if (cache_row >= 0 && q >= sink.q_width) {
                                        bool is_value;
                                        const size_t at = kv_sink_index(sink, cache_row, q, &is_value);
                                        (is_value ? sink.v_pages : sink.k_pages)[at] = hv;
                                    }
                                } else ((float*)out_ptr)[row + q] = v;
                            }
                        }
                    }
                } else {
                    // p is a feature, q runs over tokens: a warp writes 32 neighbouring features
                    const float b = bias ? bias[p] : 0.f;
                    float old[32];
                    if (epilogue == EPI_RESIDUAL) {
                        // the residual values of the whole chunk are fetched before any is written back
#pragma unroll
                        for (int j = 0; j < CHUNK; ++j) {
                            const int q = q0 + c0 + j;
                            old[j] = q < rows_q ? residual[(size_t)q * ld_out + p] : 0.f;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < CHUNK; ++j) {
                        const int q = q0 + c0 + j;
                        if (q < rows_q) {
                            float v = __uint_as_float(r[j]) + b;
                            if (epilogue == EPI_GELU) v = gelu_tanh(v);
                            const size_t idx = (size_t)q * ld_out + p;
                            if (epilogue == EPI_RESIDUAL) residual[idx] = old[j] + v;
                            else if (out_bf16) ((bf16*)out_ptr)[idx] = __float2bfloat16_rn(v);
                            else ((float*)out_ptr)[idx] = v;
                        }
                    }
                }
            }
        };
        // Two register buffers take turns: while one chunk goes through the epilogue the next one is
        // on its way from tensor memory.
        uint32_t ra[32], rb[32];
        auto fetch = [&](uint32_t (&r)[32], const int c0) {
            if (CHUNK == 32) tmem_load_32(lane_addr + (uint32_t)c0, r);
            else tmem_load_16(lane_addr + (uint32_t)c0, r);
        };
        fetch(ra, 0);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 2 * CHUNK) {
            if (q0 + c0 >= rows_q) break;                 // uniform over the CTA
            tmem_wait_ld();
            const bool second = c0 + CHUNK < BN && q0 + c0 + CHUNK < rows_q;
            if (second) fetch(rb, c0 + CHUNK);
            finish_chunk(ra, c0);
            if (second) {
                tmem_wait_ld();
                if (c0 + 2 * CHUNK < BN && q0 + c0 + 2 * CHUNK < rows_q) fetch(ra, c0 + 2 * CHUNK);
                finish_chunk(rb, c0 + CHUNK);
            }
        }
    } else if (tid == 0) {
        // something timed out: give copies that may still be in flight a moment to land
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    MG_STAMP(gemm, 6);
    tc_fence_before();
    __syncthreads();
    MG_STAMP(gemm, 7);
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---- host side -----------------------------------------------------------------------------------
template <int BN, bool SWAP>
int launch(const void* p, const void* q, int rows_p, int rows_q, int K, const float* bias, void* out,
           float* residual, int ld_out, int epilogue, int out_bf16, const KvSink& sink, int* status,
           cudaStream_t s) {
    CUtensorMap map_p, map_q;
    int rc = tensor_map(p, rows_p, K, TILE_P, &map_p);
    if (rc != MG_OK) return rc;
    rc = tensor_map(q, rows_q, K, BN, &map_q);
    if (rc != MG_OK) return rc;
    constexpr int stage_bytes = P_TILE_BYTES + BN * BLOCK_K * 2;
    const int num_kb = (K + BLOCK_K - 1) / BLOCK_K;
    // Many tiles: a ring short enough for two CTAs per SM, so that one CTA's epilogue overlaps
    // another's main loop.  Few tiles (decoding): one CTA per SM with everything in flight.
    const long long tiles = (long long)ceil_div(rows_p, TILE_P) * ceil_div(rows_q, BN);
    int stages = ((tiles > 148 ? 100 : 200) * 1024) / stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > num_kb) stages = num_kb;
    const size_t smem = (size_t)stages * stage_bytes + sizeof(Barriers) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, SWAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "linear: cannot raise shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(ceil_div(rows_p, TILE_P), ceil_div(rows_q, BN));
    const cudaError_t le = mg_launch(gemm_tc_kernel<BN, SWAP>, grid, dim3(128), smem, s, true, map_p, map_q, bias, out,
                                     residual, rows_p, rows_q, K, ld_out, epilogue, out_bf16, stages, sink, status);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "gemm_tc: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("gemm_tc");
    return MG_OK;
}

}  // namespace

// x: [M, K] bf16, w: [N, K] bf16 (both row-major).  Epilogues as mg_linear_simt.  `status` is a
// device int that receives a non-zero code if a wait inside the kernel ran out.
// Returns MG_ERR_UNSUPPORTED (and launches nothing) for sizes or alignments TMA cannot take:
// K not a multiple of 8, pointers not 16-byte aligned.
MG_API int mg_linear_tc(const void* x, const void* w, const float* bias, void* out, float* residual, int M,
                        int N, int K, int epilogue, int out_bf16, void* k_pages, void* v_pages, const int* slots,
                        int q_width, int n_kv_head, int head_dim, int page_tokens, int num_pages, int* status,
                        void* stream) {
    if (M == 0) return MG_OK;
    MG_REQUIRE(M > 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    MG_REQUIRE(epilogue == EPI_RESIDUAL ? residual != nullptr : out != nullptr, "linear: missing output");
    MG_REQUIRE(status != nullptr, "linear: missing status word");
    if (K % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
        return mg_set_error(MG_ERR_UNSUPPORTED, "linear: tensor-core path needs K %% 8 == 0 and 16-byte aligned operands");
    cudaStream_t s = (cudaStream_t)stream;
    KvSink sink = {};
    if (k_pages != nullptr) {
        MG_REQUIRE(v_pages && slots && out_bf16 && epilogue == EPI_STORE, "linear: the key/value copy wants a bfloat16 store");
        MG_REQUIRE(head_dim > 0 && head_dim % 8 == 0 && q_width % 8 == 0 && n_kv_head > 0 && page_tokens > 0 &&
                       q_width + 2 * n_kv_head * head_dim == N,
                   "linear: key/value copy with q_width=%d n_kv_head=%d head_dim=%d N=%d", q_width, n_kv_head, head_dim, N);
        sink = KvSink{(bf16*)k_pages, (bf16*)v_pages, slots, q_width, n_kv_head, head_dim, page_tokens, num_pages};
    }
    if (M <= 64 && k_pages == nullptr) {
        // few tokens: weight rows fill the 128-row side of the tile, the batch sits on the narrow side
        if (ceil_div(N, TILE_P) > 2147483647) return mg_set_error(MG_ERR_ARG, "linear: N too large");
        if (M <= 16) return launch<16, true>(w, x, N, M, K, bias, out, residual, N, epilogue, out_bf16, sink, status, s);
        if (M <= 32) return launch<32, true>(w, x, N, M, K, bias, out, residual, N, epilogue, out_bf16, sink, status, s);
        return launch<64, true>(w, x, N, M, K, bias, out, residual, N, epilogue, out_bf16, sink, status, s);
    }
    MG_REQUIRE(ceil_div(N, 64) <= 65535, "linear: N too large for one launch (%d)", N);
    if (N <= 64 || (long long)ceil_div(M, TILE_P) * ceil_div(N, 128) < 120)
        return launch<64, false>(x, w, M, N, K, bias, out, residual, N, epilogue, out_bf16, sink, status, s);
    // Very many tokens on a large matrix: tiles of 128 x 256 (two CTAs of two stages per SM hold all 512
    // TMEM columns) ask L2 for a quarter fewer bytes per flop, which is what bounds these products
    // (measured at 1600 x 4800 / 6400: +12 to 18 % from 4,096 tokens on; nothing below, where the tiles
    // do not fill two rounds of the 296 places).
    if ((long long)ceil_div(M, TILE_P) * ceil_div(N, 256) >= 2 * 296)
        return launch<256, false>(x, w, M, N, K, bias, out, residual, N, epilogue, out_bf16, sink, status, s);
    return launch<128, false>(x, w, M, N, K, bias, out, residual, N, epilogue, out_bf16, sink, status, s);
}
