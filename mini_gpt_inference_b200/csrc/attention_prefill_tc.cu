// Causal attention of prompt portions over the paged cache on the 5th-generation tensor cores
// (bfloat16, head_dim 64).
//
// A CTA takes up to 128 consecutive query tokens of one request and one head and walks over the
// key blocks (128 positions, anchored at absolute multiples of 128) that those queries may see.
// Keys and values come straight from the cache pages by TMA (one tile load per page and
// tensor, 128-byte swizzle; keys one block ahead, values as soon as their tile is free); the keys of this very step were
// written to the pages before the launch, so a portion of a prompt and a whole prompt read the
// same numbers.  Per key block:
//
//   S = Q K^T        tcgen05.mma, 128 x 128, accumulator in TMEM;
//   softmax          every thread owns one query row: it reads its row of S from TMEM, masks
//                    keys after its own position (and before its window), keeps the running
//                    maximum and sum in 32-bit, and writes P = 2^(s - max) as bfloat16 into a
//                    swizzled shared-memory tile;
//   O_blk = P V      tcgen05.mma, 128 x 64, V taken as it lies in the page (MN-major operand);
//   O = O * corr + O_blk in registers (32-bit), corr = 2^(old max - new max).
//
// Rows of the tile that belong to no query of this work item are computed and dropped; value
// rows past the item's last key are cleared in shared memory before they are multiplied.  Pages
// that a request does not have (table entry -1, also pages a window has given back) make the
// TMA coordinate negative, which fills zeros.  All mbarrier waits are bounded; on expiry the
// kernel records a code in `status`, writes nothing more, frees its TMEM and returns.
#include <cuda.h>
#include <math.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

constexpr int D = 64;                 // head_dim of this kernel
constexpr int BQ = 128;               // query rows per CTA = UMMA M
constexpr int BK = 128;               // keys per block
constexpr int THREADS = 128;
constexpr uint32_t SPIN_LIMIT = 2000000u;
constexpr int Q_BYTES = BQ * D * 2;           // 16 KB
constexpr int KV_BYTES = BK * D * 2;          // 16 KB per tensor and stage
constexpr int P_BYTES = BQ * BK * 2;          // 32 KB
constexpr uint32_t TMEM_COLS = 256;           // S: 128 columns, O_blk: 64 columns
constexpr uint32_t O_COL = 128;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Descriptor of a tile whose rows are 128 bytes, 128-byte swizzle, 1024 bytes between groups of 8
// rows (version 1, layout type 2).  Serves K-major operands (rows = M or N index) and MN-major
// operands 64 elements wide (rows = K index) alike.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFFu);
    d |= (uint64_t)1u << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1u << 46;
    d |= (uint64_t)2u << 61;
    return d;
}
// kind::f16, D = F32, A = B = BF16, A K-major; bit 16 set: B is MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

struct __align__(8) Sync {
    uint64_t q_full, k_full[2], v_full, s_done, pv_done;
    uint32_t tmem_base;
    uint32_t failed;
};

__global__ void __launch_bounds__(THREADS)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ work,
                            const int* __restrict__ block_table, const int* __restrict__ positions,
                            bf16* __restrict__ out, float* __restrict__ partial, int n_head, int n_kv_head,
                            int page_tokens, int box_rows, int max_pages, int window, float scale_log2e,
                            int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_tile = smem;
    uint8_t* k_tiles = q_tile + Q_BYTES;              // 2 stages
    uint8_t* v_tile = k_tiles + 2 * KV_BYTES;         // 1 stage: reloaded once the product with P is done
    uint8_t* p_tile = v_tile + KV_BYTES;
    Sync* sync = (Sync*)(p_tile + P_BYTES);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int item = blockIdx.x, head = blockIdx.y;
    const int req = work[5 * item], row0 = work[5 * item + 1], n_rows = work[5 * item + 2];
    const int chunk = work[5 * item + 3], n_chunks = work[5 * item + 4];
    const int kv_head = head / (n_head / n_kv_head);
    const int pos0 = positions[row0];
    const int my_pos = pos0 + tid;                     // query position of this thread's row
    const int last_key = pos0 + n_rows - 1;
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    // the key blocks this tile may see, and this work item's share of them
    const int tile_first = lo / BK, tile_blocks = last_key / BK - tile_first + 1;
    const int first_blk = tile_first + (int)((long long)tile_blocks * chunk / n_chunks);
    const int last_blk = tile_first + (int)((long long)tile_blocks * (chunk + 1) / n_chunks) - 1;
    const int* table = block_table + (size_t)req * max_pages;

    if (tid == 0) {
        mbar_init(smem_u32(&sync->q_full), 1);
        for (int s = 0; s < 2; ++s) mbar_init(smem_u32(&sync->k_full[s]), 1);
        mbar_init(smem_u32(&sync->v_full), 1);
        mbar_init(smem_u32(&sync->s_done), 1);
        mbar_init(smem_u32(&sync->pv_done), 1);
        sync->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sync->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sync->tmem_base;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    // The work list, positions and block tables are inputs of the step; queries, keys and values
    // come from the kernels in front, and nothing is read or written of them before this wait.
    pdl_trigger();
    pdl_wait();

    // Issue the tile loads of one key block (thread 0 only): keys into a stage of the ring,
    // values into the single value tile.
    auto load_tiles = [&](int blk, bool values, int stage) {
        const uint32_t bar = values ? smem_u32(&sync->v_full) : smem_u32(&sync->k_full[stage]);
        mbar_expect_tx(bar, KV_BYTES);
        for (int r = 0; r < BK; r += box_rows) {
            const int pos = blk * BK + r;
            const int pi = pos / page_tokens;
            const int page = pi < max_pages ? table[pi] : -1;   // -1: no such page -> zeros
            const int y = (page * n_kv_head + kv_head) * page_tokens + (pos % page_tokens);
            uint8_t* dst = (values ? v_tile : k_tiles + stage * KV_BYTES) + r * (D * 2);
            tma_load_2d(smem_u32(dst), values ? &map_v : &map_k, bar, 0, y);
        }
    };

    if (tid == 0) {
        mbar_expect_tx(smem_u32(&sync->q_full), Q_BYTES);
        tma_load_2d(smem_u32(q_tile), &map_q, smem_u32(&sync->q_full), head * D, row0);
        if (first_blk <= last_blk) {
            load_tiles(first_blk, false, 0);
            load_tiles(first_blk, true, 0);
        }
    }

    float o[D];
#pragma unroll
    for (int d = 0; d < D; ++d) o[d] = 0.f;
    float run_max = -INFINITY, run_sum = 0.f;
    bool good = true;

    // S = Q K^T of one key block (thread 0 only): waits for the block's keys, issues, commits.
    auto issue_scores = [&](int it) {
        const int stage = it & 1;
        bool ok = true;
        if (it == 0) ok = mbar_wait(smem_u32(&sync->q_full), 0);
        ok = ok && mbar_wait(smem_u32(&sync->k_full[stage]), (it >> 1) & 1);
        if (!ok) { atomicExch(status, 21); sync->failed = 1; }
        tc_fence_after();
        constexpr uint32_t idesc_s = instr_desc(BQ, BK, false);
        const uint64_t dq = smem_desc_sw128(smem_u32(q_tile));
        const uint64_t dk = smem_desc_sw128(smem_u32(k_tiles + stage * KV_BYTES));
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
            umma_bf16(tmem_base, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_s, k ? 1u : 0u);
        umma_commit(smem_u32(&sync->s_done));
    };
    if (tid == 0 && first_blk <= last_blk) {
        if (first_blk + 1 <= last_blk) load_tiles(first_blk + 1, false, 1);   // keys one block ahead
        issue_scores(0);
    }

    for (int blk = first_blk, it = 0; blk <= last_blk; ++blk, ++it) {
        const int stage = it & 1;
        // The scores of this block were asked for together with the product of the block before
        // (below), so the tensor core computes them while the threads finish that block.
        if (tid == 0 && it > 0) {
            if (blk + 1 <= last_blk) load_tiles(blk + 1, false, stage ^ 1);   // keys one block ahead
            load_tiles(blk, true, 0);                       // values: the tile is free since the last product
        }
        __syncwarp();
        if (!mbar_wait(smem_u32(&sync->s_done), it & 1)) { good = false; atomicExch(status, 22); }
        tc_fence_after();

        // ---- softmax of this thread's row over the block's 128 keys ----
        const int key0 = blk * BK;
        const int hi = my_pos - key0;                                     // columns <= hi are not in the future
        const int lo_col = (window > 0) ? (my_pos - window + 1 - key0) : -1;   // columns >= lo_col are in the window
        // Blocks that lie wholly before the first query of the tile (and inside every window)
        // need no mask: the common case takes the short path.
        const bool unmasked = (key0 + BK - 1 <= pos0) && (window <= 0 || key0 >= pos0 + BQ - window);
        // first pass over the row of S: the block's maximum (four chains, so that a maximum does
        // not wait for the one before it)
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < BK / 32; ++c) {
            uint32_t r[32];
            tmem_load_32(lane_addr + (uint32_t)(c * 32), r);
            tmem_wait_ld();
            if (unmasked) {
#pragma unroll
                for (int j = 0; j < 32; ++j) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(r[j]));
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int col = c * 32 + j;
                    const bool visible = col <= hi && col >= lo_col;
                    mx[j & 3] = fmaxf(mx[j & 3], visible ? __uint_as_float(r[j]) : -INFINITY);
                }
            }
        }
        float blk_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        blk_max *= scale_log2e;                                            // scale > 0: max commutes
        const float new_max = fmaxf(run_max, blk_max);
        const bool none = new_max == -INFINITY;                            // no visible key so far
        const float corr = none ? 1.f : exp2f(run_max - new_max);
        const float shift = none ? 0.f : new_max;
        float part_sum[4] = {0.f, 0.f, 0.f, 0.f};                          // one per 16-byte chunk of a load
        uint8_t* p_row = p_tile + (tid >> 3) * 1024 + (tid & 7) * 128;
        // second pass: P = 2^(s - max) as bfloat16 into the swizzled tile, 8 keys per 16-byte chunk
#pragma unroll
        for (int c = 0; c < BK / 32; ++c) {
            uint32_t r[32];
            tmem_load_32(lane_addr + (uint32_t)(c * 32), r);
            tmem_wait_ld();
            float pv[32];
            if (unmasked) {
#pragma unroll
                for (int j = 0; j < 32; ++j) pv[j] = exp2_approx(fmaf(__uint_as_float(r[j]), scale_log2e, -shift));
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int col = c * 32 + j;
                    const bool visible = !none && col <= hi && col >= lo_col;
                    pv[j] = visible ? exp2_approx(fmaf(__uint_as_float(r[j]), scale_log2e, -shift)) : 0.f;
                }
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float p0 = pv[g * 8 + 2 * j], p1 = pv[g * 8 + 2 * j + 1];
                    part_sum[j] += p0 + p1;                                // the sum stays in 32-bit
                    const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    packed[j] = *reinterpret_cast<const uint32_t*>(&h);
                }
                const int chunk = c * 4 + g;                               // 16-byte chunk of the 128 keys
                const int atom = chunk >> 3, cc = chunk & 7;
                *reinterpret_cast<uint4*>(p_row + atom * (BQ * 128) + ((cc ^ (tid & 7)) * 16)) =
                    make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
        }
        const float blk_sum = (part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]);
        run_sum = run_sum * corr + blk_sum;
        run_max = new_max;
        // Rows of the value tile past the last key of this work item hold whatever the page held
        // before (their P is zero, but 0 * NaN would still poison the product): clear them.
        if (blk == last_key / BK && last_key - key0 + 1 < BK) {
            if (!mbar_wait(smem_u32(&sync->v_full), it & 1)) { good = false; atomicExch(status, 25); }
            if (tid > last_key - key0) {
                uint4* vrow = reinterpret_cast<uint4*>(v_tile + tid * (D * 2));
#pragma unroll
                for (int c = 0; c < D * 2 / 16; ++c) vrow[c] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        // make P visible to the tensor core, and be sure everybody has read S
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        tc_fence_before();
        __syncthreads();

        if (tid == 0) {
            tc_fence_after();
            if (!mbar_wait(smem_u32(&sync->v_full), it & 1)) { atomicExch(status, 23); sync->failed = 1; }
            tc_fence_after();
            constexpr uint32_t idesc_pv = instr_desc(BQ, D, true);
            const uint32_t p_addr = smem_u32(p_tile), v_addr = smem_u32(v_tile);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
                const uint64_t dp = smem_desc_sw128(p_addr + (k >> 2) * (BQ * 128) + (k & 3) * 32);
                const uint64_t dv = smem_desc_sw128(v_addr + k * (16 * D * 2));
                umma_bf16(tmem_base + O_COL, dp, dv, idesc_pv, k ? 1u : 0u);
            }
            umma_commit(smem_u32(&sync->pv_done));
            // everybody has read S (the barrier above): the next block's scores may overwrite it
            if (blk + 1 <= last_blk) issue_scores(it + 1);
        }
        __syncwarp();
        if (!mbar_wait(smem_u32(&sync->pv_done), it & 1)) { good = false; atomicExch(status, 24); }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_load_32(lane_addr + O_COL + (uint32_t)(c * 32), r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[c * 32 + j] = o[c * 32 + j] * corr + __uint_as_float(r[j]);
        }
        tc_fence_before();
        good = good && (*(volatile uint32_t*)&sync->failed == 0);
        if (!__syncthreads_and(good)) { good = false; break; }
    }

    if (first_blk > last_blk && tid == 0) {
        // nothing to walk (a window cut this part away): the query tile is still on its way
        if (!mbar_wait(smem_u32(&sync->q_full), 0)) { atomicExch(status, 26); good = false; }
    }
    if (good && n_chunks == 1) {
        if (tid < n_rows) {
            const float inv = run_sum > 0.f ? 1.0f / run_sum : 0.f;
            uint4* dst = reinterpret_cast<uint4*>(out + ((size_t)(row0 + tid) * n_head + head) * D);
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(o[c * 8 + 2 * j] * inv, o[c * 8 + 2 * j + 1] * inv);
                    packed[j] = *reinterpret_cast<const uint32_t*>(&h);
                }
                dst[c] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
        }
    } else if (good) {
        // one of several work items of this tile: leave the unnormalised row, its maximum and its
        // sum for the merge kernel   [item][head][D + 2][row]: neighbouring threads, neighbouring words
        float* dst = partial + ((size_t)item * n_head + head) * (D + 2) * BQ + tid;
#pragma unroll
        for (int d = 0; d < D; ++d) dst[(size_t)d * BQ] = o[d];
        dst[(size_t)D * BQ] = run_max;
        dst[(size_t)(D + 1) * BQ] = run_sum;
    }
    if (!good && tid == 0)
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);        // let copies in flight land
    tc_fence_before();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
}

// Merge the work items of each query tile that was cut along the keys: the CTA of the tile's
// first item (chunk 0) reads the partial rows of all its items and writes the output rows.
__global__ void __launch_bounds__(THREADS)
attention_prefill_merge_kernel(const int* __restrict__ work, const float* __restrict__ partial,
                               bf16* __restrict__ out, int n_head) {
    const int item = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int row0 = work[5 * item + 1], n_rows = work[5 * item + 2];
    const int chunk = work[5 * item + 3], n_chunks = work[5 * item + 4];
    pdl_trigger();
    pdl_wait();                                                       // the partial rows come from the kernel in front
    if (chunk != 0 || n_chunks == 1 || tid >= n_rows) return;
    const size_t stride = (size_t)n_head * (D + 2) * BQ;              // between items
    const float* base = partial + ((size_t)item * n_head + head) * (D + 2) * BQ + tid;
    float M = -INFINITY;
    for (int c = 0; c < n_chunks; ++c) M = fmaxf(M, base[c * stride + (size_t)D * BQ]);
    float o[D];
#pragma unroll
    for (int d = 0; d < D; ++d) o[d] = 0.f;
    float denom = 0.f;
    for (int c = 0; c < n_chunks; ++c) {                              // chunks in order
        const float* src = base + c * stride;
        const float m = src[(size_t)D * BQ];
        const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
        denom += w * src[(size_t)(D + 1) * BQ];
#pragma unroll
        for (int d = 0; d < D; ++d) o[d] = fmaf(w, src[(size_t)d * BQ], o[d]);
    }
    const float inv = denom > 0.f ? 1.0f / denom : 0.f;
    uint4* dst = reinterpret_cast<uint4*>(out + ((size_t)(row0 + tid) * n_head + head) * D);
#pragma unroll
    for (int c = 0; c < D / 8; ++c) {
        uint32_t packed[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(o[c * 8 + 2 * j] * inv, o[c * 8 + 2 * j + 1] * inv);
            packed[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        dst[c] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// Map of a row-major bfloat16 matrix [rows, cols]; boxes of box_rows x 64, 128-byte swizzle.
int make_map(const void* ptr, long long rows, long long cols, int box_rows, CUtensorMap* out) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return mg_set_error(MG_ERR_CUDA, "attention: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return mg_set_error(MG_ERR_CUDA, "attention: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return MG_OK;
}

}  // namespace

// Floats of scratch for the partial results of n_items work items.
MG_API long long mg_attention_prefill_scratch_floats(int n_items, int n_head) {
    return (long long)n_items * n_head * BQ * (D + 2);
}

// Attention of prompt portions.  work: [n_items, 5] ints on the device = (request index, first row
// of the flat batch, rows <= 128, chunk, chunks): consecutive rows of one request with consecutive
// positions; the tile's visible key blocks are cut evenly into `chunks` parts and this item walks
// part `chunk`; the items of one tile are consecutive, chunk 0 first.  `partial` holds
// mg_attention_prefill_scratch_floats() floats (may be null if no tile is cut: merge != 0 says
// whether any is).
// qkv: [n_tokens, (n_head + 2 n_kv_head) * 64] bf16; pages: [num_pages, n_kv_head, page_tokens, 64];
// out: [n_tokens, n_head * 64].  Returns MG_ERR_UNSUPPORTED unless head_dim is 64 and page_tokens
// is 8, 16, 32, 64, 128 or a multiple of 128.
MG_API int mg_attention_prefill_tc(const void* qkv, const void* k_pages, const void* v_pages, const int* work,
                                   const int* block_table, const int* positions, void* out, float* partial,
                                   int merge, int n_items,
                                   int n_tokens, int n_head, int n_kv_head, int head_dim, int page_tokens,
                                   long long num_pages, int max_pages, int window, float scale, int* status,
                                   void* stream) {
    if (n_items == 0) return MG_OK;
    MG_REQUIRE(n_items > 0 && n_tokens > 0 && n_head > 0 && n_kv_head > 0 && page_tokens > 0 && max_pages > 0 && status,
               "attention (prefill): bad arguments");
    MG_REQUIRE(!merge || partial != nullptr, "attention (prefill): tiles are cut along the keys but no scratch was given");
    MG_REQUIRE(n_head % n_kv_head == 0, "attention: n_head %d is not a multiple of n_kv_head %d", n_head, n_kv_head);
    const bool pages_ok = (page_tokens % 8 == 0) && ((page_tokens <= 128 && 128 % page_tokens == 0) || page_tokens % 128 == 0);
    if (head_dim != D || !pages_ok || n_head > 65535 || (((uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15))
        return mg_set_error(MG_ERR_UNSUPPORTED, "attention (prefill, tensor cores): needs head_dim 64 and a page size of 8..128 dividing 128 or a multiple of 128");
    const int box_rows = page_tokens < BK ? page_tokens : BK;
    const int qkv_width = (n_head + 2 * n_kv_head) * D;
    CUtensorMap map_q, map_k, map_v;
    int rc = make_map(qkv, n_tokens, qkv_width, BQ, &map_q);
    if (rc != MG_OK) return rc;
    const long long kv_rows = num_pages * n_kv_head * page_tokens;
    rc = make_map(k_pages, kv_rows, D, box_rows, &map_k);
    if (rc != MG_OK) return rc;
    rc = make_map(v_pages, kv_rows, D, box_rows, &map_v);
    if (rc != MG_OK) return rc;
    const size_t smem = Q_BYTES + 3 * KV_BYTES + P_BYTES + sizeof(Sync) + 1024;   // 97 KB: two CTAs per SM
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "attention (prefill): cannot raise shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(n_items, n_head);
    cudaError_t le = mg_launch(attention_prefill_tc_kernel, grid, dim3(THREADS), smem, (cudaStream_t)stream, true, map_q,
                               map_k, map_v, work, block_table, positions, (bf16*)out, partial, n_head, n_kv_head,
                               page_tokens, box_rows, max_pages, window, scale * 1.4426950408889634f, status);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "attention_prefill_tc: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("attention_prefill_tc");
    if (merge) {
        le = mg_launch(attention_prefill_merge_kernel, grid, dim3(THREADS), 0, (cudaStream_t)stream, true, work,
                       (const float*)partial, (bf16*)out, n_head);
        if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "attention_prefill_merge: %s", cudaGetErrorString(le));
        MG_CHECK_LAUNCH("attention_prefill_merge");
    }
    return MG_OK;
}
