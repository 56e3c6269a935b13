// Causal attention of prompt portions over the paged cache on the 5th-generation tensor cores
// (bfloat16, head_dim 64).
//
// A work item is up to 128 consecutive query tokens of one request, one head, and one chunk of
// the key positions those queries may see (the host cuts long contexts into chunks, see
// kernels/attention_plan.py); a CTA walks over its chunk in key blocks of 64 positions anchored
// at absolute multiples of 64.  The CTA's six warps have three jobs and hand over through
// mbarriers only (no __syncthreads in the loop, every wait bounded):
//
//   load warp        TMA tile loads of keys and values straight from the cache pages (one load
//                    per page and tensor, 128-byte swizzle) into a ring of four stages; the keys of
//                    this very step were written to the pages before the launch, so a portion of
//                    a prompt and a whole prompt read the same numbers;
//   issue warp       S = Q K^T by tcgen05.mma (128 x 64, accumulator in one of two TMEM buffers,
//                    issued one block ahead of the softmax), then O += P V (128 x 64, V taken as
//                    it lies in the page as an MN-major operand, accumulated in TMEM over all
//                    blocks of the chunk);
//   softmax warps    four warps, a thread per query row: the row of S comes from TMEM into
//                    registers in one trip, keys after the row's own position (and before its
//                    window) are masked, P = 2^(s - ref) goes as bfloat16 into one of two swizzled
//                    shared-memory tiles; the sum of P stays in 32-bit.
//
// `ref`, the exponent P is taken relative to, is the maximum of the row's first block.  It moves
// only if a later block's weights would leave the range 2^60 relative to it (REF_LIMIT); then the
// row's accumulator is rescaled in TMEM (tcgen05.ld, multiply, tcgen05.st) and its sum with it.
// That almost never happens, so a block costs one pass over S and none over O.  The result,
// O / sum, does not depend on ref beyond rounding.  A tile whose keys were cut into chunks leaves
// (O, ref, sum) per chunk in scratch; the chunk that finishes last (a counter per tile and head
// that resets itself) merges them.  Two CTAs share an SM.
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

#include "blackwell.cuh"

MG_GUARD_DECLARE(attention_prefill)

namespace {

constexpr int D = 64;                 // head_dim of this kernel
constexpr int BQ = 128;               // query rows per CTA = UMMA M
constexpr int BK = 64;                // keys per block
constexpr int KV_STAGES = 4;          // blocks of keys and values in flight
constexpr int SOFTMAX_THREADS = 128;   // one per query row: warps 0..3, each on its 32 lanes of TMEM
constexpr int ISSUE_WARP = 4;          // issues the tensor-core instructions
constexpr int LOAD_WARP = 5;           // issues the TMA loads
constexpr int THREADS = SOFTMAX_THREADS + 64;
constexpr int Q_BYTES = BQ * D * 2;           // 16 KB
constexpr int KV_BYTES = BK * D * 2;          // 8 KB per tensor and stage
constexpr int P_BYTES = BQ * BK * 2;          // 16 KB, two of them
constexpr uint32_t TMEM_COLS = 256;           // S: two buffers of 64 columns, O: 64 columns
constexpr uint32_t O_COL = 128;
constexpr float REF_LIMIT = 1.152921504606846976e18f;   // 2^60: a block's sum of P above it moves the row's reference
constexpr uint32_t ALIGN_SLACK = 768;         // bytes the tiles may have to move up to reach a 1024-byte boundary

struct __align__(8) Sync {
    uint64_t q_full, kv_full[KV_STAGES], kv_free[KV_STAGES], s_done[2], pv_done[2], block_done[2];
    uint32_t tmem_base;
    uint32_t failed;
    uint32_t last;            // this work item is the last of its tile to finish
};

__global__ void __launch_bounds__(THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ work,
                            const int* __restrict__ block_table, const int* __restrict__ positions,
                            bf16* __restrict__ out, float* __restrict__ partial, int* __restrict__ counters,
                            int n_head, int n_kv_head, int page_tokens, int box_rows, int max_pages, int window,
                            float scale_log2e, int* __restrict__ status, int n_tokens, int num_pages, int n_requests) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
    if (pad > ALIGN_SLACK) {                           // uniform over the CTA; nothing is held yet
        if (threadIdx.x == 0) atomicExch(status, 27);
        return;
    }
    uint8_t* smem = smem_raw + pad;
    uint8_t* q_tile = smem;
    uint8_t* k_tiles = q_tile + Q_BYTES;              // ring of KV_STAGES
    uint8_t* v_tiles = k_tiles + KV_STAGES * KV_BYTES;
    uint8_t* p_tiles = v_tiles + KV_STAGES * KV_BYTES;   // two
    Sync* sync = (Sync*)(p_tiles + 2 * P_BYTES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int item = blockIdx.x, head = blockIdx.y;
    int req = work[5 * item], row0 = work[5 * item + 1], n_rows = work[5 * item + 2];
    const int chunk = work[5 * item + 3], n_chunks = work[5 * item + 4];
    const int kv_head = head / (n_head / n_kv_head);
    // (guarded builds: a request beyond the block tables' rows, a first row beyond the batch or a page
    // beyond the pool is recorded; request 0 and row 0 are read in their place, and such a page counts
    // as missing: its keys are zeros)
    if (!MG_GUARDED(attention_prefill, MG_GUARD_REQUEST, req, n_requests)) req = 0;
    if (!MG_GUARDED(attention_prefill, MG_GUARD_ROW, n_rows - 1, BQ) || !MG_GUARDED(attention_prefill, MG_GUARD_ROW, row0, n_tokens) ||
        !MG_GUARDED(attention_prefill, MG_GUARD_ROW, row0 + n_rows - 1, n_tokens)) {
        row0 = 0;
        n_rows = 1;
    }
    const int pos0 = positions[row0];
    const int last_key = pos0 + n_rows - 1;
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    // the key blocks this tile may see, and this work item's share of them
    const int tile_first = lo / BK, tile_blocks = last_key / BK - tile_first + 1;
    const int first_blk = tile_first + (int)((long long)tile_blocks * chunk / n_chunks);
    const int last_blk = tile_first + (int)((long long)tile_blocks * (chunk + 1) / n_chunks) - 1;
    const int n_blocks = last_blk - first_blk + 1;     // may be <= 0 (a window cut this part away)
    const int* table = block_table + (size_t)req * max_pages;

    if (tid == 0) {
        mbar_init(smem_u32(&sync->q_full), 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(smem_u32(&sync->kv_full[s]), 1);
            mbar_init(smem_u32(&sync->kv_free[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&sync->s_done[s]), 1);
            mbar_init(smem_u32(&sync->pv_done[s]), 1);
            mbar_init(smem_u32(&sync->block_done[s]), SOFTMAX_THREADS);
        }
        sync->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sync->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Cache row (TMA y coordinate) of this lane's share of a key block: a tile of BK positions is
    // fetched as BK / box_rows boxes, one per lane of the loading warp.  -1 page: zeros.
    auto box_row = [&](int it) {
        const int pos = (first_blk + it) * BK + lane * box_rows;
        const int pi = pos / page_tokens;
        int page = (lane * box_rows < BK && pi < max_pages) ? table[pi] : -1;
        if (page >= 0 && !MG_GUARDED(attention_prefill, MG_GUARD_PAGE, page, num_pages)) page = -1;
        return (page * n_kv_head + kv_head) * page_tokens + (pos % page_tokens);
    };
    // The work list, positions and block tables are inputs of the step: the loading warp looks up
    // the pages of its first blocks while the kernel in front drains.
    int y_first[KV_STAGES];
    if (warp == LOAD_WARP) {
#pragma unroll
        for (int j = 0; j < KV_STAGES; ++j) y_first[j] = j < n_blocks ? box_row(j) : 0;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sync->tmem_base;
    // Queries, keys and values come from the kernels in front: nothing of them is read, and nothing
    // is written, before this wait.
    pdl_trigger();
    pdl_wait();

    float ref = -INFINITY, run_sum = 0.f;               // softmax threads: see below
    bool good = true;

    if (warp == LOAD_WARP) {
        // ---- loading warp: one TMA box per lane.  Keys and values of block j lie in stage
        // j % KV_STAGES of their rings and arm one barrier; a stage is free again when the product
        // P V of the block that held it is over (kv_free, armed by the issuing warp's commit).
        auto load_tiles = [&](int j, int y) {
            const int stage = j % KV_STAGES;
            const uint32_t bar = smem_u32(&sync->kv_full[stage]);
            if (lane == 0) mbar_expect_tx(bar, 2 * KV_BYTES);
            __syncwarp();
            if (lane * box_rows < BK) {
                const uint32_t off = stage * KV_BYTES + lane * box_rows * (D * 2);
                tma_load_2d(smem_u32(k_tiles + off), &map_k, bar, 0, y);
                tma_load_2d(smem_u32(v_tiles + off), &map_v, bar, 0, y);
            }
        };
        if (lane == 0) {
            mbar_expect_tx(smem_u32(&sync->q_full), Q_BYTES);
            tma_load_2d(smem_u32(q_tile), &map_q, smem_u32(&sync->q_full), head * D, row0);
        }
#pragma unroll
        for (int j = 0; j < KV_STAGES; ++j)
            if (j < n_blocks) load_tiles(j, y_first[j]);
        int code = 0;
        for (int j = KV_STAGES; j < n_blocks; ++j) {
            const int y = box_row(j);                     // looked up while the wait passes
            if (!warp_wait(smem_u32(&sync->kv_free[j % KV_STAGES]), (j / KV_STAGES - 1) & 1)) { code = 30; break; }
            load_tiles(j, y);
        }
        if (code != 0) {
            if (lane == 0) { atomicExch(status, code); *(volatile uint32_t*)&sync->failed = 1; }
            good = false;
        }
    } else if (warp == ISSUE_WARP) {
        // ---- issuing warp: lane 0 issues tcgen05.mma / commit; all lanes walk the same path, so
        // the warp stays converged.  Scores of block j go to S buffer j % 2, its P lies in P tile j % 2.
        auto issue_scores = [&](int j) {                // S(j) = Q K(j)^T
            const int stage = j % KV_STAGES;
            bool ok = true;
            if (j == 0) ok = warp_wait(smem_u32(&sync->q_full), 0);
            ok = ok && warp_wait(smem_u32(&sync->kv_full[stage]), (j / KV_STAGES) & 1);
            tc_fence_after();
            if (lane == 0) {
                constexpr uint32_t idesc_s = instr_desc_bf16(BQ, BK, false);
                const uint64_t dq = smem_desc_sw128(smem_u32(q_tile));
                const uint64_t dk = smem_desc_sw128(smem_u32(k_tiles + stage * KV_BYTES));
#pragma unroll
                for (int k = 0; k < D / 16; ++k)
                    umma_bf16(tmem_base + (uint32_t)((j & 1) * BK), dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_s, k ? 1u : 0u);
                umma_commit(smem_u32(&sync->s_done[j & 1]));
            }
            __syncwarp();
            return ok;
        };
        int code = 0;
        if (n_blocks > 0 && !issue_scores(0)) code = 21;
        for (int it = 0; it < n_blocks && code == 0; ++it) {
            // Block it - 1 is through the softmax (the round before waited for that): its S buffer is
            // free for S(it + 1), which the tensor core computes while the softmax of block `it` runs.
            if (it + 1 < n_blocks && !issue_scores(it + 1)) { code = 21; break; }
            // P(it) is written (and the accumulator rescaled where it had to be); the block's values
            // landed together with its keys, for which S(it) waited
            if (!warp_wait(smem_u32(&sync->block_done[it & 1]), (it >> 1) & 1)) { code = 29; break; }
            tc_fence_after();
            if (lane == 0) {
                constexpr uint32_t idesc_pv = instr_desc_bf16(BQ, D, true);
                const uint32_t p_addr = smem_u32(p_tiles + (it & 1) * P_BYTES);
                const uint32_t v_addr = smem_u32(v_tiles + (it % KV_STAGES) * KV_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    const uint64_t dp = smem_desc_sw128(p_addr + k * 32);
                    const uint64_t dv = smem_desc_sw128(v_addr + k * (16 * D * 2));
                    umma_bf16(tmem_base + O_COL, dp, dv, idesc_pv, (it | k) ? 1u : 0u);
                }
                umma_commit(smem_u32(&sync->pv_done[it & 1]));
                umma_commit(smem_u32(&sync->kv_free[it % KV_STAGES]));
            }
            __syncwarp();
        }
        if (n_blocks <= 0 && !warp_wait(smem_u32(&sync->q_full), 0)) code = 26;   // the query tile is still on its way
        if (code != 0) {
            if (lane == 0) { atomicExch(status, code); *(volatile uint32_t*)&sync->failed = 1; }
            good = false;
        }
    }

    uint32_t o[D];                                      // the accumulated row, 32-bit floats as they lie in TMEM
#pragma unroll
    for (int d = 0; d < D; ++d) o[d] = 0u;

    if (warp < SOFTMAX_THREADS / 32) {
        // ---- softmax warps: thread `tid` owns query row `tid` of the tile ----
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        const int my_pos = pos0 + tid;                     // query position of this thread's row
        uint8_t* const p_row0 = p_tiles + (tid >> 3) * 1024 + (tid & 7) * 128;
        for (int it = 0; it < n_blocks; ++it) {
            const int blk = first_blk + it;
            if (!warp_wait(smem_u32(&sync->s_done[it & 1]), (it >> 1) & 1)) { good = false; atomicExch(status, 22); break; }
            tc_fence_after();
            // the thread's row of S(it) into registers: two loads in flight, one wait
            uint32_t s[BK];
#pragma unroll
            for (int c = 0; c < BK / 32; ++c)
                tmem_load_32(lane_addr + (uint32_t)((it & 1) * BK + c * 32), *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
            tmem_wait_ld();

            const int key0 = blk * BK;
            // columns <= hi are not in the future (rows of the tile that are no query of this item see nothing)
            const int hi = tid < n_rows ? my_pos - key0 : -1;
            const int lo_col = (window > 0) ? (my_pos - window + 1 - key0) : -1;   // columns >= lo_col are in the window
            // Blocks that lie wholly before the first query of the tile (and inside every window)
            // need no mask: the common case takes the short path.
            const bool unmasked = (key0 + BK - 1 <= pos0) && (window <= 0 || key0 >= pos0 + BQ - window);
            if (!unmasked) {
                // keys this row may not see get the score -inf: they count for no maximum, their P is 2^-inf = 0
#pragma unroll
                for (int j = 0; j < BK; ++j)
                    if (j > hi || j < lo_col) s[j] = 0xff800000u;
            }
            // The row's maximum over the block, times the scale (> 0).
            auto block_max = [&]() {
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < BK; ++j) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(s[j]));
                return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2e;
            };
            // P = 2^(s * scale - shift) as bfloat16 into the block's swizzled tile (a row of 64 keys is
            // 128 bytes: eight 16-byte chunks); returns the row's sum of P (32-bit).
            uint8_t* const p_row = p_row0 + (it & 1) * P_BYTES;
            auto write_p = [&](float shift) {
                float part_sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int cc = 0; cc < BK / 8; ++cc) {
                    uint32_t packed[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int c0 = cc * 8 + 2 * j;
                        const float p0 = exp2_approx(fmaf(__uint_as_float(s[c0]), scale_log2e, -shift));
                        const float p1 = exp2_approx(fmaf(__uint_as_float(s[c0 + 1]), scale_log2e, -shift));
                        part_sum[j] += p0 + p1;
                        const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                        packed[j] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                    *reinterpret_cast<uint4*>(p_row + ((cc ^ (tid & 7)) * 16)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                }
                return (part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]);
            };

            // The output row accumulates in TMEM over the blocks, relative to a reference exponent
            // `ref`.  A row takes it from the first block in which it sees a key; nothing was summed
            // for it before, so nothing needs rescaling.
            if (ref == -INFINITY) ref = block_max();
            // The product of the block before last is over: it read the P tile that is written now.
            if (it >= 2) {
                if (!warp_wait(smem_u32(&sync->pv_done[it & 1]), ((it - 2) >> 1) & 1)) { good = false; atomicExch(status, 24); break; }
            }
            float blk_sum = write_p(ref == -INFINITY ? 0.f : ref);
            // Keys far above the reference make P large; that is harmless (O / sum does not depend on
            // the reference) until the numbers leave the range of the formats.  Long before that, the
            // reference moves up to the block's maximum: the accumulator and the sum are rescaled and
            // the block's P is computed again.  !(x <= limit) also catches a sum that is no number.
            const bool high = !(blk_sum <= REF_LIMIT);
            if (__any_sync(0xffffffffu, high)) {
                float corr = 1.f;
                if (high) {
                    const float new_ref = block_max();
                    corr = exp2f(ref - new_ref);
                    ref = new_ref;
                }
                if (it > 0) {
                    // the accumulator is complete up to the block before
                    const bool done = warp_wait(smem_u32(&sync->pv_done[(it - 1) & 1]), ((it - 1) >> 1) & 1);
                    if (!done) { good = false; atomicExch(status, 24); break; }
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t r[32];
                        tmem_load_32(lane_addr + O_COL + (uint32_t)(c * 32), r);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * corr);
                        tmem_store_32(lane_addr + O_COL + (uint32_t)(c * 32), r);
                    }
                    tmem_wait_st();
                }
                run_sum *= corr;
                blk_sum = write_p(ref);
            }
            run_sum += blk_sum;
            // Rows of the value tile past the last key of this work item hold whatever the page held
            // before (their P is zero, but 0 * NaN would still poison the product): clear them.
            if (blk == last_key / BK && last_key - key0 + 1 < BK) {
                if (!warp_wait(smem_u32(&sync->kv_full[it % KV_STAGES]), (it / KV_STAGES) & 1)) { good = false; atomicExch(status, 25); break; }
                if (tid < BK && tid > last_key - key0) {
                    uint4* vrow = reinterpret_cast<uint4*>(v_tiles + (it % KV_STAGES) * KV_BYTES + tid * (D * 2));
#pragma unroll
                    for (int c = 0; c < D * 2 / 16; ++c) vrow[c] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            // S(it) is in registers no more, P(it) is written (and the accumulator rescaled where it had
            // to be): visible to the tensor core, which may go on
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            mbar_arrive(smem_u32(&sync->block_done[it & 1]));
        }
        if (good && n_blocks > 0) {
            if (!warp_wait(smem_u32(&sync->pv_done[(n_blocks - 1) & 1]), ((n_blocks - 1) >> 1) & 1)) { good = false; atomicExch(status, 24); }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < D / 32; ++c) tmem_load_32(lane_addr + O_COL + (uint32_t)(c * 32), *reinterpret_cast<uint32_t(*)[32]>(&o[c * 32]));
            tmem_wait_ld();
        }
    }
    good = __syncthreads_and(good) && (*(volatile uint32_t*)&sync->failed == 0);
    if (good && n_chunks == 1) {
        if (tid < n_rows) {
            const float inv = run_sum > 0.f ? 1.0f / run_sum : 0.f;
            uint4* dst = reinterpret_cast<uint4*>(out + ((size_t)(row0 + tid) * n_head + head) * D);
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[c * 8 + 2 * j]) * inv,
                                                                   __uint_as_float(o[c * 8 + 2 * j + 1]) * inv);
                    packed[j] = *reinterpret_cast<const uint32_t*>(&h);
                }
                dst[c] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
        }
    } else if (n_chunks > 1 && (partial == nullptr || counters == nullptr)) {
        if (tid == 0) atomicExch(status, 31);              // a tile cut along the keys, but nowhere to leave its parts
    } else if (n_chunks > 1) {
        // One of several work items of this tile: it leaves the unnormalised row, its reference and
        // its sum   [item][head][D + 2][row]: neighbouring threads, neighbouring words.  The item that
        // finishes last (a counter per tile and head, left at zero again) merges them all.  An item
        // that failed counts too, so that the counter stays right; `status` tells the host.
        if (good && tid < BQ) {
            float* dst = partial + ((size_t)item * n_head + head) * (D + 2) * BQ + tid;
#pragma unroll
            for (int d = 0; d < D; ++d) dst[(size_t)d * BQ] = __uint_as_float(o[d]);
            dst[(size_t)D * BQ] = ref;
            dst[(size_t)(D + 1) * BQ] = run_sum;
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            int* counter = counters + (size_t)(item - chunk) * n_head + head;
            const int before = atomicAdd(counter, 1);
            sync->last = (before == n_chunks - 1) ? 1u : 0u;
            if (before == n_chunks - 1) *counter = 0;
        }
        __syncthreads();
        if (good && sync->last != 0 && tid < n_rows) {
            __threadfence();
            const size_t stride = (size_t)n_head * (D + 2) * BQ;          // between items
            const float* base = partial + ((size_t)(item - chunk) * n_head + head) * (D + 2) * BQ + tid;
            float M = -INFINITY;
            for (int c = 0; c < n_chunks; ++c) M = fmaxf(M, __ldcg(base + c * stride + (size_t)D * BQ));
            float acc[D];
#pragma unroll
            for (int d = 0; d < D; ++d) acc[d] = 0.f;
            float denom = 0.f;
            for (int c = 0; c < n_chunks; ++c) {                          // items in order
                const float* src = base + c * stride;
                const float m = __ldcg(src + (size_t)D * BQ);
                const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
                denom = fmaf(w, __ldcg(src + (size_t)(D + 1) * BQ), denom);
#pragma unroll
                for (int d = 0; d < D; ++d) acc[d] = fmaf(w, __ldcg(src + (size_t)d * BQ), acc[d]);
            }
            const float inv = denom > 0.f ? 1.0f / denom : 0.f;
            uint4* dst = reinterpret_cast<uint4*>(out + ((size_t)(row0 + tid) * n_head + head) * D);
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(acc[c * 8 + 2 * j] * inv, acc[c * 8 + 2 * j + 1] * inv);
                    packed[j] = *reinterpret_cast<const uint32_t*>(&h);
                }
                dst[c] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
        }
    }
    if (!good && tid == 0)
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);        // let copies in flight land
    tc_fence_before();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
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
// part `chunk`; the items of one tile are consecutive, chunk 0 first.  If any tile is cut
// (merge != 0), `partial` holds mg_attention_prefill_scratch_floats() floats and `counters`
// n_items * n_head ints that are zero before the call and zero again after it.
// qkv: [n_tokens, (n_head + 2 n_kv_head) * 64] bf16; pages: [num_pages, n_kv_head, page_tokens, 64];
// out: [n_tokens, n_head * 64]; n_requests: rows of the block table (guarded builds hold the work
// items' request numbers against it).  Returns MG_ERR_UNSUPPORTED unless head_dim is 64 and page_tokens
// is 8, 16, 32, 64, 128 or a multiple of 128.
MG_API int mg_attention_prefill_tc(const void* qkv, const void* k_pages, const void* v_pages, const int* work,
                                   const int* block_table, const int* positions, void* out, float* partial,
                                   int* counters, int merge, int n_items,
                                   int n_tokens, int n_head, int n_kv_head, int head_dim, int page_tokens,
                                   long long num_pages, int max_pages, int window, float scale, int n_requests,
                                   int* status, void* stream) {
    if (n_items == 0) return MG_OK;
    MG_REQUIRE(n_items > 0 && n_tokens > 0 && n_head > 0 && n_kv_head > 0 && page_tokens > 0 && max_pages > 0 && status,
               "attention (prefill): bad arguments");
    MG_REQUIRE(!merge || (partial != nullptr && counters != nullptr),
               "attention (prefill): tiles are cut along the keys but no scratch or no counters were given");
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
    const size_t smem = Q_BYTES + 2 * KV_STAGES * KV_BYTES + 2 * P_BYTES + sizeof(Sync) + ALIGN_SLACK;   // 113 KB: two CTAs per SM
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "attention (prefill): cannot raise shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(n_items, n_head);
    cudaError_t le = mg_launch(attention_prefill_tc_kernel, grid, dim3(THREADS), smem, (cudaStream_t)stream, true, map_q,
                               map_k, map_v, work, block_table, positions, (bf16*)out, partial, counters, n_head, n_kv_head,
                               page_tokens, box_rows, max_pages, window, scale * 1.4426950408889634f, status, n_tokens,
                               (int)num_pages, n_requests);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "attention_prefill_tc: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("attention_prefill_tc");
    return MG_OK;
}
