// Projection of a handful of tokens onto a large matrix (many megabytes): out[m, n] = x[m, :] . w[n, :].
//
// A matrix of 15 or 160 MB met by 8 tokens is a stream: every weight is read once, and the questions
// are how many bytes are on their way at any moment, in what shape memory is asked for them, and what
// stands between the last byte's arrival and the kernel's end.  Measured on this part with copies
// alone (no arithmetic, 160 MB, one CTA per SM, 160 KB of ring): boxes of 64 rows x 128 bytes reach
// 3.2 TB/s, boxes of 128 such rows 4.2 TB/s, boxes that hold 8 whole rows of 3200 bytes 4.7 TB/s: a
// request should be tens of kilobytes and made of long runs.  So the weights come here as whole rows:
// the matrix is seen as [row][64-column block][64] and one TMA instruction brings 8, 16 or 32 rows
// with all their blocks (16 to 36 KB, 128-byte swizzle by line) into a ring of stages.
//
// Loads of one SM are served in the order in which they were asked for, so a word asked for behind
// 150 KB of weights arrives microseconds late.  Hence the order of a CTA's requests: LayerNorm gain
// and shift and the bias of its rows at once (all loads of a thread before its first store); a.early
// boxes (about 48 KB) BEFORE the wait for the kernel in front, so that they travel while that kernel
// drains; the activations right behind that wait; then the rest of the ring; and nothing is read back
// from memory after that: a residual epilogue adds with atomics instead of read-modify-write.  The
// ring's first filling leaves a stage per lane of the ninth warp; refills are issued by one lane, in
// order, as stages come free (lanes that wait on different stages hold one another up).
//
// The weights are the mma's A operand (m16n8k16, 32-bit accumulate: 16 weight rows x 8 tokens, no
// padding of the token side), read from the swizzled stage by ldmatrix: the number of blocks per box
// is odd, one block of zeros added where needed, so that eight rows of a block lie in eight different
// swizzle phases.  The tokens are the B operand and stay in REGISTERS for the kernel's life: the CTA
// stages its slice of the activations once as bfloat16 (with the LayerNorm prologue if asked:
// statistics in 32-bit, result rounded to bfloat16 exactly as the stand-alone kernel does), each warp
// takes its fragments from there once, and the stage's bytes are the only shared-memory traffic of
// the main loop.  Two ways to share the work (template SOLO):
//   - short rows (up to 12 blocks x token tiles): a warp holds the fragments of all blocks, a box is
//     one warp's, whole, and the warp finishes its rows from its own registers;
//   - longer rows: warp w holds blocks w, w + 8, .. and all eight warps work on every box (a box
//     is summed a few hundred nanoseconds after it arrived); their partial sums meet in shared memory
//     (two buffers), and two further warps add them in warp order and run the epilogue, so that the
//     consumers never wait for anything but weights.
//
// K is cut into slices (one CTA column per slice) only for the residual epilogue, where partial sums
// can simply be added into the 32-bit residual stream (atomic adds in L2, bias by slice 0): that
// keeps long rows inside a stage and the staged activations inside shared memory.  The order of
// those additions is not fixed (the result can differ in its last bits from run to run).  Without
// slices every output element sums its K terms in a fixed order, independent of M.
//
// Epilogues as the other small-batch kernels (linear_epilogue.cuh): bias, tanh-GELU, bfloat16 or
// 32-bit store, residual add, the QKV projection's copy of keys and values to their cache rows,
// and the first stage of a greedy argmax over the rows (for the head's logits).  Up to 16 tokens;
// K a multiple of 64; any N.  Every wait is bounded: if one runs out the kernel records a code in
// `status` (51: a stage never came free, 52: a copy or the sums' buffer never came, 53: the sums
// never came) and stops.
#include <math.h>

#include "blackwell.cuh"
#include "linear_epilogue.cuh"
#include "tensor_map.cuh"

MG_STAMP_DECLARE(wide)

namespace {

constexpr int KB = 64;                           // columns per block: one 128-byte swizzled line
constexpr int CONSUMERS = 8;
constexpr int FINISHERS = 2;                     // warps that add the partial sums of a box and write its outputs
constexpr int THREADS = (CONSUMERS + 1 + FINISHERS) * 32;   // the ninth warp issues the copies
constexpr int MAX_STAGES = 32;
constexpr int XPAD = 16;                         // bytes between activation rows beyond the slice (no bank conflicts)
constexpr int MAX_SLICE_K = 2048;                // most columns of activations a CTA stages
constexpr int MAX_STAGE_BYTES = 36 * 1024;
constexpr int BIAS_SMEM = 1024;                  // bias values a CTA keeps in shared memory (more are read from memory)
constexpr int MAXB = (MAX_SLICE_K / KB + 1 + CONSUMERS - 1) / CONSUMERS;   // blocks of a box per warp: 5
constexpr int SOLO_BLOCKS = 12;                  // blocks x token tiles whose fragments a warp can hold (96 registers)
constexpr int EARLY_BYTES = 48 * 1024;           // weights asked for before the wait for the kernel in front

struct WideArgs {
    const bf16* x;                   // [M, K] bfloat16 activations, or null with a LayerNorm prologue
    const float* x32;                // rows to normalise (prologue), [*, K]
    const int* row_index;            // optional gather of x32 rows
    const float* gain;
    const float* shift;              // may be null
    float eps;
    LinearEpilogue ep;
    int M, N, K;
    int k_slices, slice_k;           // K cut into k_slices slices of slice_k columns (a multiple of 64)
    int groups;                      // CTAs per slice: CTA c has slice c % k_slices and row boxes c / k_slices, + groups, ...
    int row_boxes;                   // boxes of 8 * NTW rows that cover N
    int box_blocks;                  // 64-column blocks per box: odd, at least those of a slice
    int stages;
    int warps;                       // SOLO: consumer warps at work (stages % warps == 0)
    int early;                       // boxes asked for before the dependency wait (at least 1, at most the ring)
    float* amax_v;                   // greedy choice on the way: [token][CTA * 2 + finisher], SOLO: [token][CTA * 8 + warp]
    int* amax_i;
    int amax_limit;
    const uint8_t* next_w;           // weights of the projection that is expected to run next (may be null) ..
    int next_lines;                  // .. and their size in 128-byte lines: asked into L2 behind this kernel's own
    int* status;
};

struct __align__(8) WideBars {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t sums_full[2];           // the eight partial sums of a box are written (by buffer)
    uint64_t sums_empty[2];          // and read
    uint32_t failed;                 // a wait ran out
    uint32_t pad;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// LayerNorm of one row of up to 32 * 4 * LN_RESIDENT columns by one warp, the row held in registers
// (one trip to memory, all loads in flight at once: ln_load), statistics as layernorm_row_chunked
// has them (ln_finish; gain and shift in shared memory).
constexpr int LN_RESIDENT = 16;
__device__ __forceinline__ void ln_load(float4 (&v)[LN_RESIDENT], const float* src, int width, int lane) {
    const int n4 = width / 4;
#pragma unroll
    for (int i = 0; i < LN_RESIDENT; ++i) {
        const int c = lane + 32 * i;
        v[i] = c < n4 ? reinterpret_cast<const float4*>(src)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}
__device__ __forceinline__ void ln_finish(const float4 (&v)[LN_RESIDENT], int width, const float* gain, const float* shift,
                                          float eps, uint8_t* dst, int lane) {
    const int n4 = width / 4;
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < LN_RESIDENT; ++i) sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    const float mean = warp_sum(sum) / (float)width;
    // (the same sums in the same order as with a branch per chunk: a chunk past the row adds +0.0)
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < LN_RESIDENT; ++i) {
        const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
        const float term = (dx * dx + dy * dy) + (dz * dz + dw * dw);
        sq += lane + 32 * i < n4 ? term : 0.f;
    }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)width + eps);
    // gain and shift of four chunks are read before the four results are stored: a store to shared
    // memory keeps the loads from shared memory behind it in their place (measured: a third faster)
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i0 = 0; i0 < LN_RESIDENT; i0 += 4) {
        float4 gn[4], sh[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = (lane + 32 * (i0 + u)) * 4;
            const bool in = lane + 32 * (i0 + u) < n4;
            gn[u] = in ? *reinterpret_cast<const float4*>(gain + c) : zero;
            sh[u] = (in && shift) ? *reinterpret_cast<const float4*>(shift + c) : zero;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u, c = (lane + 32 * i) * 4;
            if (lane + 32 * i < n4) {
                uint2 y;
                y.x = pack_bf16((v[i].x - mean) * rstd * gn[u].x + sh[u].x, (v[i].y - mean) * rstd * gn[u].y + sh[u].y);
                y.y = pack_bf16((v[i].z - mean) * rstd * gn[u].z + sh[u].z, (v[i].w - mean) * rstd * gn[u].w + sh[u].w);
                *reinterpret_cast<uint2*>(dst + c * 2) = y;
            }
        }
    }
}

// MT: token rows (the mma's B operand, in tiles of 8): 8 or 16; a.M <= MT.  NTW: rows of a box / 8 (1, 2
// or 4).  SOLO: rows short enough (up to SOLO_BLOCKS / (MT / 8) blocks) that a warp holds the tokens'
// fragments of ALL blocks in registers: then a box belongs to one warp, whole (box n to warp n %
// a.warps, a.warps a divisor of the ring's length, so that a slot of the ring is always the same
// warp's and the warp meets its phases in order), and the warp finishes the rows' outputs from its
// own registers; no word passes between warps.  Otherwise all eight warps share every box (warp w
// has blocks w, w + 8, ..) and two more warps add their partial sums.
template <int MT, int NTW, bool SOLO>
__global__ void __launch_bounds__(THREADS, 1) linear_wide_kernel(const __grid_constant__ CUtensorMap map_w, const WideArgs a) {
    constexpr int ROWS = 8 * NTW;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzle wants the stages aligned to 1024 bytes
    uint8_t* ring = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int stages = a.stages;
    const int K = a.K;
    const int kbs = a.box_blocks;
    const uint32_t stage_bytes = (uint32_t)(ROWS * kbs) * 128u;
    const int slice = blockIdx.x % a.k_slices, first_box = blockIdx.x / a.k_slices;
    const int k0 = slice * a.slice_k;
    const int k_len = min(a.slice_k, K - k0);                                    // columns of this slice
    const int nkb = k_len / KB;                                                  // blocks of this slice (K % 64 == 0)
    const int xcols = nkb * KB;
    const int xstride = xcols * 2 + XPAD;
    uint8_t* xs = ring + (size_t)stages * stage_bytes;                           // [MT][xstride]
    float* gain_s = reinterpret_cast<float*>(xs + (size_t)MT * (a.slice_k * 2 + XPAD));   // [K], [K] with the prologue
    float* shift_s = gain_s + (a.x32 ? K : 0);
    float* bias_s = shift_s + (a.x32 ? K : 0);                                   // [BIAS_SMEM]: bias of this CTA's rows, box by box
    float* partial = bias_s + BIAS_SMEM;                                         // [2][8 warps][MT][ROWS]: partial sums of a box (not SOLO)
    int* slots_s = reinterpret_cast<int*>(partial + (SOLO ? 0 : 2 * CONSUMERS * MT * ROWS));   // [16]: cache rows of the tokens
    WideBars* bars = reinterpret_cast<WideBars*>(slots_s + 16);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int my_boxes = first_box < a.row_boxes ? (a.row_boxes - first_box + a.groups - 1) / a.groups : 0;
    MG_STAMP(wide, 0);

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), SOLO ? 1 : CONSUMERS);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->sums_full[b]), CONSUMERS);
            mbar_init(smem_u32(&bars->sums_empty[b]), 1);
        }
        bars->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_trigger();

    // Loads of one SM are served in the order in which they were asked for: a word asked for behind
    // 150 KB of weights arrives behind them, microseconds later.  So everything small goes first:
    // gain, shift and bias at once; the activations right after the wait for the kernel in front; and
    // only a.early boxes are asked for before that wait, the rest once the activations' loads are out
    // (named barrier 2: the consumers arrive when theirs are, the ninth warp waits for it).
    if (warp == CONSUMERS) {
        // ---- the copies.  The ring's first filling leaves a stage per lane (one instruction for all):
        // a.early boxes before the wait for the kernel in front, the rest of the ring behind the
        // consumers' loads of the activations.  After that one lane refills the stages in order as they
        // come free (lanes that wait for different stages hold one another up). ----
        auto issue = [&](int n) {
            const int s = n % stages;
            const uint32_t full = smem_u32(&bars->full[s]);
            mbar_expect_tx(full, stage_bytes);
            tma_load_3d(smem_u32(ring + (size_t)s * stage_bytes), &map_w, full, 0, k0 / KB, (first_box + n * a.groups) * ROWS);
        };
        const int fill = my_boxes < stages ? my_boxes : stages;                  // (stages <= 32)
        if (lane < a.early && lane < fill) issue(lane);
        pdl_wait();                                    // (every thread of the kernel passes the wait)
        asm volatile("bar.sync 2, %0;" ::"n"((CONSUMERS + 1) * 32) : "memory");   // the activations are asked for
        if (lane >= a.early && lane < fill) issue(lane);
        __syncwarp();
        // ---- the weights that the next projection will want: this CTA's share of them is asked into
        // L2 now, behind its own copies (requests are served in order: they do not delay these), and
        // travels while this kernel sums, writes and hands over (nothing comes back to the SM) ----
        if (a.next_w != nullptr && lane > 0) {
            const int per_cta = (a.next_lines + gridDim.x - 1) / gridDim.x;
            const int line0 = blockIdx.x * per_cta;
            for (int l = lane - 1; l < per_cta && line0 + l < a.next_lines; l += 31)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(a.next_w + (size_t)(line0 + l) * 128));
        }
        if (lane == 0) {
            MG_STAMP_HERE(wide, 9);                                             // the ring is full
            for (int n = stages; n < my_boxes; ++n) {
                if (!mbar_poll(smem_u32(&bars->empty[n % stages]), ((n / stages) & 1) ^ 1)) {
                    atomicExch(a.status, 51);                                   // a stage never came free
                    break;                                                      // (the consumers' own waits run out then)
                }
                issue(n);
            }
        }
        if (lane == 0) MG_STAMP_HERE(wide, 10);                                  // the last copy is issued
        return;
    }

    if (warp > CONSUMERS) {
        // ---- the finishers: box n belongs to finisher n % 2 (and to that half of `partial`).  It adds
        // the eight partial sums in warp order, applies the epilogue and keeps the greedy candidates;
        // the consumers never wait for memory that they wrote. ----
        pdl_wait();
        if (SOLO) return;
        constexpr int EPF = ROWS * MT / 32;                                      // results a lane finishes per box
        const int f = warp - CONSUMERS - 1;
        const bool bias_staged = a.ep.bias != nullptr && slice == 0 && my_boxes * ROWS <= BIAS_SMEM;
        const float* part = partial + (size_t)f * CONSUMERS * MT * ROWS;
        float best_v[EPF];
        int best_i[EPF];
#pragma unroll
        for (int u = 0; u < EPF; ++u) {
            best_v[u] = -INFINITY;
            best_i[u] = 0x7fffffff;
        }
        bool good = true;
        for (int n = f; n < my_boxes; n += FINISHERS) {
            if (!mbar_poll(smem_u32(&bars->sums_full[f]), (uint32_t)(n >> 1) & 1u)) {
                good = false;                                                   // uniform in the warp
                break;
            }
            const int row0 = (first_box + n * a.groups) * ROWS;
            float v[EPF];
#pragma unroll
            for (int u = 0; u < EPF; ++u) {
                const int e = lane + 32 * u;
                v[u] = 0.f;
#pragma unroll
                for (int w = 0; w < CONSUMERS; ++w) v[u] += part[(size_t)w * MT * ROWS + e];   // warps in order
            }
            __syncwarp();                                                       // every lane has its sums
            if (lane == 0) mbar_arrive(smem_u32(&bars->sums_empty[f]));
#pragma unroll
            for (int u = 0; u < EPF; ++u) {
                const int e = lane + 32 * u;
                const int m = e / ROWS, r = e % ROWS, col = row0 + r;
                if (m < a.M && col < a.N) {                                     // rows past N were read as zeros
                    float y = v[u];
                    if (bias_staged) y += bias_s[n * ROWS + r];
                    else if (a.ep.bias && slice == 0) y += a.ep.bias[col];
                    // the residual stream takes its sum as an atomic add, sliced or not: nothing is read
                    // back behind the weights (one add per element and kernel: the result is the same)
                    if (a.ep.epilogue == EPI_RESIDUAL) atomicAdd(a.ep.residual + (size_t)m * a.N + col, y);
                    else linear_finish(a.ep, m, col, y, false, 0.f, true, a.ep.k_pages != nullptr ? slots_s[m] : -1);
                    if (a.amax_v != nullptr && col < a.amax_limit && (y > best_v[u] || (y == best_v[u] && col < best_i[u]))) {
                        best_v[u] = y;
                        best_i[u] = col;
                    }
                }
            }
        }
        if (f == 0) MG_STAMP_HERE_LANE0(wide, 6);                                // (almost) the last box is finished
        if (!good && lane == 0) atomicExch(a.status, 53);                        // the sums never came: no candidates below
        if (a.amax_v != nullptr) {
            // a token's candidates of this warp sit in ROWS neighbouring lanes (result e = lane + 32 u is
            // token e / ROWS); the best, lowest index among equals, goes to slot CTA * 2 + finisher
#pragma unroll
            for (int u = 0; u < EPF; ++u) {
#pragma unroll
                for (int o = 1; o < ROWS; o <<= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best_v[u], o);
                    const int oi = __shfl_xor_sync(0xffffffffu, best_i[u], o);
                    if (ov > best_v[u] || (ov == best_v[u] && oi < best_i[u])) {
                        best_v[u] = ov;
                        best_i[u] = oi;
                    }
                }
                const int e = lane + 32 * u;
                const int m = e / ROWS;
                if (e % ROWS == 0 && m < a.M) {
                    const size_t idx = (size_t)m * (gridDim.x * FINISHERS) + blockIdx.x * FINISHERS + f;
                    a.amax_v[idx] = good ? best_v[u] : -INFINITY;
                    a.amax_i[idx] = good ? best_i[u] : 0x7fffffff;
                }
            }
        }
        return;
    }

    // ---- consumers: LayerNorm gain and shift are weights too, and so is the bias of this CTA's rows ----
    // (all loads of a thread first, then the stores: one trip to memory, not one per value)
    const bool bias_staged = a.ep.bias != nullptr && slice == 0 && my_boxes * ROWS <= BIAS_SMEM;
    {
        constexpr int PER = MAX_SLICE_K / 4 / (CONSUMERS * 32);                  // float4 of gain per thread: 2
        constexpr int BPER = BIAS_SMEM / (CONSUMERS * 32);                       // bias values per thread: 4
        const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
        float4 gv[PER], sv[PER];
        float bv[BPER];
        if (a.x32 != nullptr) {
#pragma unroll
            for (int u = 0; u < PER; ++u) {
                const int i = tid + u * CONSUMERS * 32;
                gv[u] = i < K / 4 ? reinterpret_cast<const float4*>(a.gain)[i] : zero;
                sv[u] = (i < K / 4 && a.shift) ? reinterpret_cast<const float4*>(a.shift)[i] : zero;
            }
        }
        if (bias_staged) {
#pragma unroll
            for (int u = 0; u < BPER; ++u) {
                const int i = tid + u * CONSUMERS * 32;
                const int col = (first_box + (i / ROWS) * a.groups) * ROWS + i % ROWS;
                bv[u] = (i < my_boxes * ROWS && col < a.N) ? a.ep.bias[col] : 0.f;
            }
        }
        if (a.x32 != nullptr) {
#pragma unroll
            for (int u = 0; u < PER; ++u) {
                const int i = tid + u * CONSUMERS * 32;
                if (i < K / 4) {
                    reinterpret_cast<float4*>(gain_s)[i] = gv[u];
                    reinterpret_cast<float4*>(shift_s)[i] = sv[u];
                }
            }
        }
        if (bias_staged) {
#pragma unroll
            for (int u = 0; u < BPER; ++u) {
                const int i = tid + u * CONSUMERS * 32;
                if (i < my_boxes * ROWS) bias_s[i] = bv[u];
            }
        }
    }
    MG_STAMP(wide, 2);
    pdl_wait();
    MG_STAMP(wide, 3);

    // ---- stage this slice of the activations as bfloat16; rows at and past M are zero.  Every load
    // of a thread is in flight before the first is used. ----
    if (a.ep.k_pages != nullptr && tid < 16) slots_s[tid] = tid < a.M ? a.ep.slots[tid] : -1;   // cache rows of the tokens
    if (a.x32 != nullptr) {
        // (the prologue comes with k_slices == 1: the whole row is this CTA's)
        const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
        const bool resident = K <= 32 * 4 * LN_RESIDENT;
        float4 v[LN_RESIDENT];
        if (resident && warp < a.M) ln_load(v, a.x32 + (size_t)(a.row_index ? a.row_index[warp] : warp) * K, K, lane);
        asm volatile("bar.arrive 2, %0;" ::"n"((CONSUMERS + 1) * 32) : "memory");
        asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");        // gain and shift are in place
        MG_STAMP(wide, 7);
        for (int m = warp; m < MT; m += CONSUMERS) {
            uint8_t* dst = xs + (size_t)m * xstride;
            if (m >= a.M) {
                for (int i = lane; i < xcols / 8; i += 32) *reinterpret_cast<uint4*>(dst + i * 16) = zero4;
                continue;
            }
            const float* src = a.x32 + (size_t)(a.row_index ? a.row_index[m] : m) * K;
            if (resident) {
                if (m != warp) ln_load(v, src, K, lane);                        // (a second row of this warp)
                ln_finish(v, K, gain_s, a.shift ? shift_s : nullptr, a.eps, dst, lane);
            } else {
                layernorm_row_chunked<bf16>(src, K, gain_s, a.shift ? shift_s : nullptr, a.eps, reinterpret_cast<bf16*>(dst), lane);
            }
        }
        MG_STAMP(wide, 8);
    } else {
        const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
        for (int i = tid, first = 1; i < xcols / 8 || first; i += CONSUMERS * 32, first = 0) {
            uint4 v[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m)
                v[m] = (m < a.M && i < xcols / 8) ? *reinterpret_cast<const uint4*>(a.x + (size_t)m * K + k0 + i * 8) : zero4;
            if (first) asm volatile("bar.arrive 2, %0;" ::"n"((CONSUMERS + 1) * 32) : "memory");
            if (i < xcols / 8) {
#pragma unroll
                for (int m = 0; m < MT; ++m) *reinterpret_cast<uint4*>(xs + (size_t)m * xstride + i * 16) = v[m];
            }
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");
    MG_STAMP(wide, 4);

    // ---- this warp's share of the tokens, for good: blocks warp, warp + 8, .. of the slice, as B
    // fragments (token g of a tile, columns 2t.. of a 16-column step) in registers.  Matrix q = lane / 8
    // of an x4 load is the 16-byte piece 4h + q of a block: b0, b1 of step 2h, then of step 2h + 1. ----
    constexpr int TB = SOLO ? SOLO_BLOCKS / (MT / 8) : MAXB;                     // blocks whose fragments a warp holds
    uint32_t tf[TB][MT / 8][8];
    {
        const uint32_t xs_lane = smem_u32(xs) + (uint32_t)((lane & 7) * xstride + (lane >> 3) * 16);
#pragma unroll
        for (int i = 0; i < TB; ++i) {
            const int j = SOLO ? i : warp + CONSUMERS * i;
#pragma unroll
            for (int tt = 0; tt < MT / 8; ++tt)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t four[4] = {0u, 0u, 0u, 0u};
                    if (j < nkb) ldsm_x4(four, xs_lane + (uint32_t)(tt * 8 * xstride + j * 128 + h * 64));
#pragma unroll
                    for (int q = 0; q < 4; ++q) tf[i][tt][4 * h + q] = four[q];
                }
        }
    }

    // Weights are the A operand: the box lies in the stage as [row][block][128 bytes], line = row * kbs
    // + block, 16-byte piece p of a line at p ^ (line % 8).  Boxes of 16 or 32 rows: matrix q of an x4
    // load is rows (q % 2) * 8 .. of a 16-row tile and the piece 2 * step + q / 2: a0..a3 of one step.
    // Boxes of 8 rows: matrix q is the piece 4h + q: a0, a2 of step 2h, then of step 2h + 1 (rows 8..15
    // of the mma tile are zero).  D: c0, c1: weight row g, tokens 2t, 2t + 1; c2, c3: weight row g + 8.
    const int a_row = ROWS >= 16 ? ((lane >> 3) & 1) * 8 + (lane & 7) : (lane & 7);
    const uint32_t a_piece = ROWS >= 16 ? (uint32_t)(lane >> 4) : (uint32_t)(lane >> 3);
    constexpr int TILES = ROWS >= 16 ? ROWS / 16 : 1;

    float best_v[MT / 8][2];                                                     // SOLO: tokens 8 tt + 2t and + 1
    int best_i[MT / 8][2];
#pragma unroll
    for (int tt = 0; tt < MT / 8; ++tt) {
        best_v[tt][0] = best_v[tt][1] = -INFINITY;
        best_i[tt][0] = best_i[tt][1] = 0x7fffffff;
    }
    bool good = true;
    for (int n = SOLO ? warp : 0; n < my_boxes && (!SOLO || warp < a.warps); n += SOLO ? a.warps : 1) {
        const int s = n % stages;
        // (not SOLO: every warp takes part in every box, in order: its blocks of the box's rows)
        if (!mbar_poll(smem_u32(&bars->full[s]), (uint32_t)(n / stages) & 1u)) {
            good = false;                                                       // uniform in the warp
            break;
        }
        if (n == 0) MG_STAMP(wide, 5);                                          // the first box has arrived
        const uint32_t stage = smem_u32(ring + (size_t)s * stage_bytes);
        float acc[TILES][MT / 8][2][4];                                         // two chains (even and odd steps)
#pragma unroll
        for (int ti = 0; ti < TILES; ++ti)
#pragma unroll
            for (int tt = 0; tt < MT / 8; ++tt)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[ti][tt][0][q] = acc[ti][tt][1][q] = 0.f;
#pragma unroll
        for (int i = 0; i < TB; ++i) {
            const int j = SOLO ? i : warp + CONSUMERS * i;
            if (j < nkb) {                                                      // uniform in the warp
#pragma unroll
                for (int ti = 0; ti < TILES; ++ti) {
                    const uint32_t line = (uint32_t)((ti * 16 + a_row) * kbs + j);
                    const uint32_t at = stage + line * 128u, sw = line & 7u;
                    if (ROWS >= 16) {
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            uint32_t af[4];
                            ldsm_x4(af, at + (((uint32_t)(2 * ks) + a_piece) ^ sw) * 16u);
#pragma unroll
                            for (int tt = 0; tt < MT / 8; ++tt)
                                mma_bf16(acc[ti][tt][ks & 1], af[0], af[1], af[2], af[3], tf[i][tt][2 * ks], tf[i][tt][2 * ks + 1]);
                        }
                    } else {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            uint32_t af[4];
                            ldsm_x4(af, at + (((uint32_t)(4 * h) + a_piece) ^ sw) * 16u);
#pragma unroll
                            for (int tt = 0; tt < MT / 8; ++tt) {
                                mma_bf16(acc[ti][tt][0], af[0], 0u, af[1], 0u, tf[i][tt][4 * h], tf[i][tt][4 * h + 1]);
                                mma_bf16(acc[ti][tt][1], af[2], 0u, af[3], 0u, tf[i][tt][4 * h + 2], tf[i][tt][4 * h + 3]);
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();                                                           // every lane has read the stage
        if (lane == 0) mbar_arrive(smem_u32(&bars->empty[s]));
        if (n == 0) MG_STAMP(wide, 11);                                         // this warp's share of the first box is summed
        if constexpr (SOLO) {
            // ---- the rows of this box are finished: c0, c1: row g of a 16-row tile, tokens 2t, 2t + 1; c2, c3: row g + 8 ----
            const int row0 = (first_box + n * a.groups) * ROWS;
#pragma unroll
            for (int ti = 0; ti < TILES; ++ti)
#pragma unroll
                for (int tt = 0; tt < MT / 8; ++tt)
#pragma unroll
                    for (int q = 0; q < (ROWS >= 16 ? 4 : 2); ++q) {
                        const int m = tt * 8 + 2 * t + (q & 1), r = ti * 16 + g + (q >> 1) * 8, col = row0 + r;
                        if (m < a.M && col < a.N) {                             // rows past N were read as zeros
                            float y = acc[ti][tt][0][q] + acc[ti][tt][1][q];
                            if (bias_staged) y += bias_s[n * ROWS + r];
                            else if (a.ep.bias && slice == 0) y += a.ep.bias[col];
                            if (a.ep.epilogue == EPI_RESIDUAL) atomicAdd(a.ep.residual + (size_t)m * a.N + col, y);
                            else linear_finish(a.ep, m, col, y, false, 0.f, true, a.ep.k_pages != nullptr ? slots_s[m] : -1);
                            if (a.amax_v != nullptr && col < a.amax_limit &&
                                (y > best_v[tt][q & 1] || (y == best_v[tt][q & 1] && col < best_i[tt][q & 1]))) {
                                best_v[tt][q & 1] = y;
                                best_i[tt][q & 1] = col;
                            }
                        }
                    }
            continue;
        }
        // ---- the eight partial sums of the box meet in shared memory: [buffer n % 2][warp][token][row];
        // the buffer is free once the finisher has read the sums of box n - 2 ----
        if (n >= 2 && !mbar_poll(smem_u32(&bars->sums_empty[n & 1]), (uint32_t)((n >> 1) - 1) & 1u)) {
            good = false;
            break;
        }
        {
            float* mine = partial + ((size_t)(n & 1) * CONSUMERS + warp) * MT * ROWS;
#pragma unroll
            for (int ti = 0; ti < TILES; ++ti)
#pragma unroll
                for (int tt = 0; tt < MT / 8; ++tt) {
                    const int tok = tt * 8 + 2 * t, row = ti * 16 + g;
                    mine[tok * ROWS + row] = acc[ti][tt][0][0] + acc[ti][tt][1][0];
                    mine[(tok + 1) * ROWS + row] = acc[ti][tt][0][1] + acc[ti][tt][1][1];
                    if (ROWS >= 16) {
                        mine[tok * ROWS + row + 8] = acc[ti][tt][0][2] + acc[ti][tt][1][2];
                        mine[(tok + 1) * ROWS + row + 8] = acc[ti][tt][0][3] + acc[ti][tt][1][3];
                    }
                }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars->sums_full[n & 1]));
    }
    if (!good && lane == 0) {
        atomicExch(a.status, 52);                                                // a copy or a finisher never came
        *(volatile uint32_t*)&bars->failed = 1;
    }
    if (SOLO && a.amax_v != nullptr) {
        // a token's candidates of this warp sit in the eight lanes with the same t; the best, lowest
        // index among equals, goes to slot CTA * 8 + warp
#pragma unroll
        for (int tt = 0; tt < MT / 8; ++tt)
#pragma unroll
            for (int u = 0; u < 2; ++u) {
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best_v[tt][u], o);
                    const int oi = __shfl_xor_sync(0xffffffffu, best_i[tt][u], o);
                    if (ov > best_v[tt][u] || (ov == best_v[tt][u] && oi < best_i[tt][u])) {
                        best_v[tt][u] = ov;
                        best_i[tt][u] = oi;
                    }
                }
                const int m = tt * 8 + 2 * t + u;
                if (g == 0 && m < a.M) {
                    const size_t idx = (size_t)m * (gridDim.x * CONSUMERS) + blockIdx.x * CONSUMERS + warp;
                    a.amax_v[idx] = good ? best_v[tt][u] : -INFINITY;
                    a.amax_i[idx] = good ? best_i[tt][u] : 0x7fffffff;
                }
            }
    }
}

int wide_sms() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 0;
    }
    return sms;
}

struct WidePlan {
    int k_slices, slice_k, groups, row_boxes, box_rows, box_blocks, stages, warps;
    bool solo;
    size_t smem;
    bool ok;
};

// How an [N, K] matrix is cut for M tokens: slices of K (residual epilogue without prologue only),
// rows per box, CTAs per slice, stages of the ring.  Among the cuts it takes the one whose busiest
// CTA reads the fewest bytes (a small charge per slice for its atomic adds), of equals the one with
// the larger boxes.
WidePlan wide_plan(int M, int N, int K, bool can_slice, bool prologue) {
    WidePlan best = {};
    const int sms = wide_sms();
    if (sms <= 0 || K % KB != 0) return best;
    const int mt = M <= 8 ? 8 : 16;
    const size_t budget = 226 * 1024;
    double best_cost = 0.0;
    const int most_slices = can_slice ? (K + 255) / 256 : 1;                     // slices of at least 256 columns
    for (int slices = 1; slices <= most_slices && slices <= sms; ++slices) {
        WidePlan p = {};
        p.slice_k = ((K + slices - 1) / slices + KB - 1) / KB * KB;
        p.k_slices = (K + p.slice_k - 1) / p.slice_k;
        if (p.k_slices != slices || p.slice_k > MAX_SLICE_K) continue;
        p.box_blocks = (p.slice_k / KB) | 1;                                     // odd: see the swizzle
        const size_t fixed = (size_t)mt * ((size_t)p.slice_k * 2 + XPAD) + (prologue ? (size_t)2 * K * sizeof(float) : 0) +
                             BIAS_SMEM * sizeof(float) + 16 * sizeof(int) + sizeof(WideBars) + 1024;
        if (fixed >= budget) continue;
        for (int rows = 32; rows >= 8; rows /= 2) {
            WidePlan q = p;
            const size_t stage_bytes = (size_t)rows * q.box_blocks * 128;
            if (stage_bytes > MAX_STAGE_BYTES) continue;
            q.box_rows = rows;
            q.row_boxes = (N + rows - 1) / rows;
            q.groups = sms / q.k_slices;
            if (q.groups > q.row_boxes) q.groups = q.row_boxes;
            if (q.groups < 1) continue;
            const int rounds = (q.row_boxes + q.groups - 1) / q.groups;
            q.solo = (p.slice_k / KB) * (mt / 8) <= SOLO_BLOCKS;
            // (rows of fewer than 16 blocks whose fragments do not fit a warp are left to the other
            // kernels: shared by eight warps, a box of so few blocks costs more in hand-overs than in
            // bytes; measured at K = 512 with 16 tokens: 38 us against 20 us of the row-streaming kernel)
            if (!q.solo && p.slice_k / KB < 16) continue;
            const size_t sums = q.solo ? 0 : (size_t)2 * CONSUMERS * mt * rows * sizeof(float);
            if (fixed + sums + 2 * stage_bytes > budget) continue;
            q.stages = (int)((budget - fixed - sums) / stage_bytes);
            if (q.stages > MAX_STAGES) q.stages = MAX_STAGES;
            if (q.stages > rounds) q.stages = rounds;
            if (q.stages < 3 && q.stages < rounds) continue;
            q.warps = CONSUMERS;
            if (q.solo) {
                // the warps at work divide the ring (see the kernel): of 4 to 8 warps those that keep most stages
                if (q.stages <= CONSUMERS) {
                    q.warps = q.stages;
                } else {
                    int keep = 0;
                    for (int w = 4; w <= CONSUMERS; ++w)
                        if (q.stages / w * w >= keep) {
                            keep = q.stages / w * w;
                            q.warps = w;
                        }
                    q.stages = keep;
                }
            }
            q.smem = fixed + sums + (size_t)q.stages * stage_bytes;
            const double cost = (double)rounds * stage_bytes + 4096.0 * q.k_slices;
            if (!best.ok || cost < best_cost) {
                best = q;
                best.ok = true;
                best_cost = cost;
            }
        }
    }
    return best;
}

// Launches the kernel for boxes of 8 * NTW rows (the first launch of a shape raises its shared memory).
template <int MT, int NTW, bool SOLO>
cudaError_t launch_wide_as(int grid, size_t smem, cudaStream_t s, const CUtensorMap& map_w, const WideArgs& a) {
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(linear_wide_kernel<MT, NTW, SOLO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    return mg_launch(linear_wide_kernel<MT, NTW, SOLO>, dim3(grid), dim3(THREADS), smem, s, true, map_w, a);
}

template <int NTW>
cudaError_t launch_wide(int M, bool solo, int grid, size_t smem, cudaStream_t s, const CUtensorMap& map_w, const WideArgs& a) {
    if (M <= 8) return solo ? launch_wide_as<8, NTW, true>(grid, smem, s, map_w, a) : launch_wide_as<8, NTW, false>(grid, smem, s, map_w, a);
    return solo ? launch_wide_as<16, NTW, true>(grid, smem, s, map_w, a) : launch_wide_as<16, NTW, false>(grid, smem, s, map_w, a);
}

}  // namespace

// Candidates per row that mg_linear_wide leaves for the greedy argmax of M tokens (its scratch holds
// M times as many floats and as many ints) for an [N, K] matrix, with the LayerNorm prologue or
// without; 0 if the device cannot be queried or the kernel does not take the shape.
MG_API int mg_linear_wide_parts(int M, int N, int K, int prologue) {
    const WidePlan p = wide_plan(M, N, K, false, prologue != 0);
    return p.ok ? p.groups * p.k_slices * (p.solo ? CONSUMERS : FINISHERS) : 0;
}

MG_GUARD_EXPORT(linear_wide, linear_index_fault)

// As mg_linear_skinny (same operands, prologue, epilogues and greedy choice), for matrices of many
// megabytes and up to 16 tokens.  next_w / next_lines: optionally the start and the size (in 128-byte
// lines) of memory that the caller expects to be read next (the weights of the projection behind this
// one): the kernel asks it into the L2 cache once its own copies are out; it must be readable, nothing
// else is assumed about it.  Returns MG_ERR_UNSUPPORTED (nothing launched) for M > 16,
// K % 64 != 0, operands that are not 16-byte aligned, or rows whose activations do not fit the shared
// memory beside a ring of at least three stages (K beyond 2048 without the residual epilogue, or with
// the prologue).
MG_API int mg_linear_wide(const void* x, const float* x32, const int* row_index, const float* gain,
                          const float* shift, float eps, const void* w, const float* bias, void* out,
                          float* residual, int M, int N, int K, int epilogue, int out_bf16, void* k_pages,
                          void* v_pages, const int* slots, int q_width, int n_kv_head, int head_dim,
                          int page_tokens, int num_pages, float* amax_v, int* amax_i, int amax_limit, const void* next_w,
                          int next_lines, int* status, void* stream) {
    if (M == 0) return MG_OK;
    MG_REQUIRE(M > 0 && N > 0 && K > 0 && status != nullptr, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    MG_REQUIRE(next_lines >= 0 && (next_w != nullptr || next_lines == 0), "linear: bad hint");
    MG_REQUIRE(x != nullptr || (x32 != nullptr && gain != nullptr), "linear: missing input");
    MG_REQUIRE(epilogue == EPI_RESIDUAL ? residual != nullptr : out != nullptr, "linear: missing output");
    MG_REQUIRE(amax_v == nullptr || (amax_i != nullptr && epilogue == EPI_STORE && !out_bf16),
               "linear: the greedy choice goes with 32-bit stored outputs");
    MG_REQUIRE(k_pages == nullptr || (out_bf16 && epilogue == EPI_STORE && slots && v_pages && head_dim > 0 &&
                                      n_kv_head > 0 && page_tokens > 0 && N == q_width + 2 * n_kv_head * head_dim),
               "linear: bad key/value sink");
    const bool prologue = x == nullptr;
    const WidePlan p = wide_plan(M, N, K, epilogue == EPI_RESIDUAL && !prologue, prologue);
    if (!p.ok || M > 16 || ((uintptr_t)w & 15) || (x && ((uintptr_t)x & 15)) || (x32 && !x && ((uintptr_t)x32 & 15)) ||
        (gain && ((uintptr_t)gain & 15)) || (shift && ((uintptr_t)shift & 15)))
        return mg_set_error(MG_ERR_UNSUPPORTED, "linear (wide): needs M <= 16, K %% 64 == 0, aligned operands, activations that fit");
    CUtensorMap map_w;
    const int rc = tensor_map_rows(w, N, K, p.box_rows, p.box_blocks, &map_w);
    if (rc != MG_OK) return rc;
    WideArgs a;
    a.x = (const bf16*)x; a.x32 = prologue ? x32 : nullptr; a.row_index = row_index; a.gain = gain; a.shift = shift; a.eps = eps;
    a.M = M; a.N = N; a.K = K;
    a.ep.bias = bias; a.ep.out = out; a.ep.residual = residual; a.ep.M = M; a.ep.N = N;
    a.ep.epilogue = epilogue; a.ep.out_bf16 = out_bf16;
    a.ep.k_pages = (bf16*)k_pages; a.ep.v_pages = (bf16*)v_pages; a.ep.slots = slots;
    a.ep.q_width = q_width; a.ep.n_kv_head = n_kv_head; a.ep.head_dim = head_dim; a.ep.page_tokens = page_tokens; a.ep.num_pages = num_pages;
    a.k_slices = p.k_slices; a.slice_k = p.slice_k; a.groups = p.groups; a.row_boxes = p.row_boxes;
    a.box_blocks = p.box_blocks; a.stages = p.stages; a.warps = p.warps;
    a.early = (int)(EARLY_BYTES / ((size_t)p.box_rows * p.box_blocks * 128));
    if (a.early < 1) a.early = 1;
    if (a.early > p.stages) a.early = p.stages;
    a.amax_v = amax_v; a.amax_i = amax_i; a.amax_limit = (amax_limit <= 0 || amax_limit > N) ? N : amax_limit;
    a.next_w = next_lines > 0 ? (const uint8_t*)next_w : nullptr; a.next_lines = next_lines;
    a.status = status;
    const int grid = p.groups * p.k_slices;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t le = cudaErrorInvalidValue;
    switch (p.box_rows) {
        case 8: le = launch_wide<1>(M, p.solo, grid, p.smem, s, map_w, a); break;
        case 16: le = launch_wide<2>(M, p.solo, grid, p.smem, s, map_w, a); break;
        case 32: le = launch_wide<4>(M, p.solo, grid, p.smem, s, map_w, a); break;
        default: break;
    }
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "linear_wide: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("linear_wide");
    return MG_OK;
}
