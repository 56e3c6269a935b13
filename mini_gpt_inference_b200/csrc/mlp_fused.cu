// The whole feed-forward of a handful of tokens in one kernel (decoding at small batch):
//
//     out = x + proj(gelu(fc(LayerNorm(x)))) + proj_bias
//
// As two projections this is two kernels that each stream a matrix of a megabyte or two and are
// bound by the hand-over between them, not by memory.  Here a CTA owns 16 units of the inner
// dimension: the 16 rows of fc.weight that produce them and the 16 columns of proj.weight that
// consume them.  It asks for all of these weights before it waits for the kernel in front,
// normalises the tokens' rows (every CTA does, a few KB from L2), multiplies them by its rows of
// fc.weight on warp-level mma (K cut over the eight warps, summed in order through shared
// memory), applies bias and tanh-GELU in 32-bit, rounds its 16 hidden values per token to bfloat16
// (exactly what the two-kernel path stores between the projections), multiplies them by its
// columns of proj.weight and adds the partial [tokens, width] product into the output with
// 16-byte vector reductions in L2.  x and the bias are added once per tile of eight columns, by the
// CTA whose number the tile has.  A CTA's columns of proj.weight are 32 bytes out of every 4 KB
// row, which DRAM serves badly; the kernel reads them from a copy packed once in the order its
// lanes want (mg_mlp_pack_elements), a CTA's slice one contiguous block.
//
// The output cannot be x itself: other CTAs still read x for their LayerNorm while the first
// partial sums arrive.  The caller hands three buffers that take turns: `x` (read), `out` (all
// zeros on entry, the result on exit) and `spare` (anything on entry, all zeros on exit: the
// `out` of the next call).
//
// The order in which the CTAs' partial sums meet is not fixed, so the 32-bit result can differ
// in its last bits from run to run; the two-kernel path (and the true 32-bit path) stay
// reproducible.  Sizes: up to 16 tokens, width a multiple of 8 up to 512, inner width a multiple of 8.
#include "linear_epilogue.cuh"

MG_STAMP_DECLARE(mlp)

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int FS = 16;               // inner units per CTA (two mma tiles of 8)
// A lane holds KPW k blocks (of 32) of fc.weight and NTW tiles of 8 output columns of proj.weight,
// all requested before the dependency wait: widths up to 512.  Wider models are left to the two
// streaming projections (measured at widths 768 and 1600: deeper register rings or a second round
// of loads after the wait cost more than the kernel saves).
constexpr int KPW = 2;
constexpr int NTW = 8;
constexpr int MAX_WIDTH = 32 * WARPS * KPW;
constexpr int XPAD = 64;             // bytes between activation rows beyond C bf16 (no bank conflicts)
constexpr int HSTRIDE = FS + 8;      // bf16 per row of the hidden tile (rows 16 bytes apart in the banks)

struct MlpArgs {
    const float* x;                  // [M, C] residual stream before the feed-forward
    float* out;                      // [M, C] zeros on entry
    float* spare;                    // [M, C] zeroed here
    const float* gain;
    const float* shift;              // may be null
    float eps;
    const bf16* w1;                  // [F, C]
    const float* b1;                 // [F] or null
    const bf16* w2p;                 // proj.weight packed for this kernel, see mg_mlp_pack_elements()
    const float* b2;                 // [C] or null
    int M, C, F;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Four consecutive 32-bit sums added into global memory by one reduction in L2.
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// MT: token rows of the A operand: 8 (rows 8..15 are zero) or 16; a.M <= MT.
template <int MT>
__global__ void __launch_bounds__(THREADS, 1) mlp_fused_kernel(const MlpArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int C = a.C, F = a.F;
    const int xstride = C * 2 + XPAD;                                          // bytes per token row
    uint8_t* xs = smem_raw;                                                    // [MT][C] bf16, padded rows
    float* gain_s = reinterpret_cast<float*>(smem_raw + (size_t)MT * xstride);  // [C], [C]
    float* shift_s = gain_s + C;
    float* partial = shift_s + C;                                              // [WARPS][MT][FS]
    bf16* hs = reinterpret_cast<bf16*>(partial + WARPS * MT * FS);             // [MT][HSTRIDE]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int f0 = blockIdx.x * FS;
    const int kblocks = (C + 31) / 32, ntiles = (C + 7) / 8;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    const uint2 zero2 = make_uint2(0u, 0u);
    MG_STAMP(mlp, 0);

    // ---- everything that does not depend on the kernel in front: this CTA's weights ----
    // fc.weight: warp w takes k blocks w, w + 8, ...; per k block a lane holds 8 consecutive k of
    // unit f0 + g and of unit f0 + 8 + g.
    const bf16* w1row0 = a.w1 + (size_t)min(f0 + g, F - 1) * C;
    const bf16* w1row1 = a.w1 + (size_t)min(f0 + 8 + g, F - 1) * C;
    uint4 w1a[KPW], w1b[KPW];
#pragma unroll
    for (int i = 0; i < KPW; ++i) {
        const int k = (warp + i * WARPS) * 32 + 8 * t;
        const bool in = warp + i * WARPS < kblocks && k < C;
        w1a[i] = in ? *reinterpret_cast<const uint4*>(w1row0 + k) : zero4;
        w1b[i] = in ? *reinterpret_cast<const uint4*>(w1row1 + k) : zero4;
    }
    // proj.weight: warp w takes column tiles w, w + 8, ...; per tile a lane holds units
    // f0 + 4t .. 4t + 3 of output column (tile * 8 + g).  The packed copy has them in exactly
    // this order, so a warp's load is 256 consecutive bytes and a CTA's slice one block.
    const uint2* w2slice = reinterpret_cast<const uint2*>(a.w2p) + (size_t)blockIdx.x * ntiles * 32 + lane;
    uint2 w2v[NTW];
#pragma unroll
    for (int i = 0; i < NTW; ++i)
        w2v[i] = warp + i * WARPS < ntiles ? w2slice[(size_t)(warp + i * WARPS) * 32] : zero2;
    // x and the bias are added once per column tile, by the CTA whose number the tile has (mod
    // the grid); the first such tile's bias comes now, its x right after the wait
    const int own_tile = blockIdx.x < ntiles ? (int)blockIdx.x : -1;
    const bool own_lane = own_tile >= 0 && own_tile % WARPS == warp;
    const int own_m = (t & 1) ? g + 8 : g, own_col = own_tile * 8 + 4 * (t >> 1);
    float4 own_add = make_float4(0.f, 0.f, 0.f, 0.f);
    if (own_lane && a.b2 != nullptr && own_col < C) own_add = *reinterpret_cast<const float4*>(a.b2 + own_col);
    float bias1[2] = {0.f, 0.f};                                               // of the two hidden values this thread finishes
    {
        const int e = tid * 2, unit = e % FS;
        if (a.b1 != nullptr && e < MT * FS) {
            if (f0 + unit < F) bias1[0] = a.b1[f0 + unit];
            if (f0 + unit + 1 < F) bias1[1] = a.b1[f0 + unit + 1];
        }
    }
    // (one value per round: with all of a thread's loads ahead of its stores, as the other kernels stage
    // gain and shift, a step of one token was measured 7% slower, a step of eight no faster)
    for (int i = tid; i < C / 4; i += THREADS) {
        reinterpret_cast<float4*>(gain_s)[i] = reinterpret_cast<const float4*>(a.gain)[i];
        reinterpret_cast<float4*>(shift_s)[i] =
            a.shift ? reinterpret_cast<const float4*>(a.shift)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    MG_STAMP(mlp, 2);
    pdl_wait();
    MG_STAMP(mlp, 3);
    float4 own_x = make_float4(0.f, 0.f, 0.f, 0.f);                            // asked for now, used at the very end
    if (own_lane && own_m < a.M && own_col < C) own_x = *reinterpret_cast<const float4*>(a.x + (size_t)own_m * C + own_col);
    __syncthreads();                                                           // gain and shift are in place

    // ---- the buffer of the call after this one becomes zero (nobody reads or writes it now) ----
    {
        const int total4 = a.M * C / 4;
        for (int i = blockIdx.x * THREADS + tid; i < total4; i += gridDim.x * THREADS)
            reinterpret_cast<float4*>(a.spare)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

    MG_STAMP(mlp, 8);
    // ---- LayerNorm of the tokens' rows into shared memory as bfloat16 (a warp per row) ----
    const bool ln_fast = C % 128 == 0 && C <= 1024;
    if (ln_fast) {
        constexpr int RPW = MT / WARPS;                                        // rows per warp: 1 or 2
        float4 v[RPW][8];
        const int n4 = C / 128;
#pragma unroll
        for (int r = 0; r < RPW; ++r) {                                         // all loads first: one trip to memory
            const int m = warp + r * WARPS;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i < n4 && m < a.M) v[r][i] = *reinterpret_cast<const float4*>(a.x + (size_t)m * C + (lane + 32 * i) * 4);
        }
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const int m = warp + r * WARPS;
            if (m >= a.M) continue;                                            // uniform in the warp
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i < n4) sum += (v[r][i].x + v[r][i].y) + (v[r][i].z + v[r][i].w);
            const float mean = warp_sum(sum) / (float)C;
            MG_STAMP(mlp, 9);
            float sq = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i < n4) {
                    const float dx = v[r][i].x - mean, dy = v[r][i].y - mean, dz = v[r][i].z - mean, dw = v[r][i].w - mean;
                    sq += (dx * dx + dy * dy) + (dz * dz + dw * dw);
                }
            const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)C + a.eps);
            uint8_t* dst = xs + (size_t)m * xstride;
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
                        y.x = pack2((v[r][i].x - mean) * rstd * gn[u].x + sh[u].x, (v[r][i].y - mean) * rstd * gn[u].y + sh[u].y);
                        y.y = pack2((v[r][i].z - mean) * rstd * gn[u].z + sh[u].z, (v[r][i].w - mean) * rstd * gn[u].w + sh[u].w);
                        *reinterpret_cast<uint2*>(dst + c * 2) = y;
                    }
            }
        }
    } else {
        for (int m = warp; m < a.M; m += WARPS)
            layernorm_row_chunked<bf16>(a.x + (size_t)m * C, C, gain_s, a.shift ? shift_s : nullptr, a.eps,
                                        reinterpret_cast<bf16*>(xs + (size_t)m * xstride), lane);
    }
    __syncthreads();
    MG_STAMP(mlp, 4);
    // Only now may the kernel behind this one start: its CTAs ask for their weights at once, and a
    // load of this kernel that is asked for behind those (the rows above) would also arrive behind them.
    pdl_trigger();

    // ---- hidden[token, unit] = LN(x) . fc.weight[unit]: this warp's k blocks ----
    float hc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
        const uint8_t* xrow0 = xs + (size_t)g * xstride;
        const uint8_t* xrow1 = xs + (size_t)(g + 8) * xstride;
        for (int b0 = warp; b0 < kblocks; b0 += WARPS * KPW) {
            uint4 wa[KPW], wb[KPW];
            if (b0 == warp) {
#pragma unroll
                for (int i = 0; i < KPW; ++i) { wa[i] = w1a[i]; wb[i] = w1b[i]; }
            } else {
#pragma unroll
                for (int i = 0; i < KPW; ++i) {
                    const int k = (b0 + i * WARPS) * 32 + 8 * t;
                    const bool in = b0 + i * WARPS < kblocks && k < C;
                    wa[i] = in ? *reinterpret_cast<const uint4*>(w1row0 + k) : zero4;
                    wb[i] = in ? *reinterpret_cast<const uint4*>(w1row1 + k) : zero4;
                }
            }
#pragma unroll
            for (int i = 0; i < KPW; ++i) {
                const int k = (b0 + i * WARPS) * 32 + 8 * t;
                if (b0 + i * WARPS < kblocks) {                                 // uniform in the warp
                    const bool in = k < C;
                    const uint4 x0 = (in && g < a.M) ? *reinterpret_cast<const uint4*>(xrow0 + k * 2) : zero4;
                    uint4 x1 = zero4;
                    if (MT == 16 && in && g + 8 < a.M) x1 = *reinterpret_cast<const uint4*>(xrow1 + k * 2);
                    mma_bf16(hc[0], x0.x, x1.x, x0.y, x1.y, wa[i].x, wa[i].y);
                    mma_bf16(hc[0], x0.z, x1.z, x0.w, x1.w, wa[i].z, wa[i].w);
                    mma_bf16(hc[1], x0.x, x1.x, x0.y, x1.y, wb[i].x, wb[i].y);
                    mma_bf16(hc[1], x0.z, x1.z, x0.w, x1.w, wb[i].z, wb[i].w);
                }
            }
        }
        // c0, c1: token g, units 2t and 2t + 1 of the tile; c2, c3: token g + 8
        float* mine = partial + (size_t)warp * MT * FS;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            *reinterpret_cast<float2*>(mine + g * FS + nt * 8 + 2 * t) = make_float2(hc[nt][0], hc[nt][1]);
            if (MT == 16) *reinterpret_cast<float2*>(mine + (g + 8) * FS + nt * 8 + 2 * t) = make_float2(hc[nt][2], hc[nt][3]);
        }
    }
    __syncthreads();
    MG_STAMP(mlp, 5);
    // ---- the warps' slices in order, bias, GELU in 32-bit, rounded to bfloat16 ----
    {
        const int e = tid * 2;
        if (e < MT * FS) {
            const int m = e / FS, unit = e - m * FS;
            float v0 = 0.f, v1 = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float2 p = *reinterpret_cast<const float2*>(partial + ((size_t)w * MT + m) * FS + unit);
                v0 += p.x;
                v1 += p.y;
            }
            // units past the inner width (a ragged last CTA) count as zero
            v0 = (m < a.M && f0 + unit < F) ? gelu_tanh(v0 + bias1[0]) : 0.f;
            v1 = (m < a.M && f0 + unit + 1 < F) ? gelu_tanh(v1 + bias1[1]) : 0.f;
            *reinterpret_cast<uint32_t*>(hs + m * HSTRIDE + unit) = pack2(v0, v1);
        }
    }
    __syncthreads();
    MG_STAMP(mlp, 6);

    // ---- out[token, column] += hidden . proj.weight[column, units]: this warp's column tiles ----
    {
        // A operand: k slots (2t, 2t+1) hold units 4t, 4t+1 and slots (2t+8, 2t+9) units 4t+2, 4t+3,
        // as the 8-byte loads of proj.weight above have them
        const uint2 h0 = *reinterpret_cast<const uint2*>(hs + g * HSTRIDE + 4 * t);
        uint2 h1 = zero2;
        if (MT == 16) h1 = *reinterpret_cast<const uint2*>(hs + (g + 8) * HSTRIDE + 4 * t);
        // tiles blockIdx.x, + gridDim.x, ... get x and the bias from this CTA; the first of them
        // (own_tile) has them in registers already
        int next_own = own_tile >= 0 ? own_tile + (int)gridDim.x : 0x7fffffff;
        for (int n0 = warp; n0 < ntiles; n0 += WARPS * NTW) {
            uint2 wv[NTW];
            if (n0 == warp) {
#pragma unroll
                for (int i = 0; i < NTW; ++i) wv[i] = w2v[i];
            } else {
#pragma unroll
                for (int i = 0; i < NTW; ++i)
                    wv[i] = n0 + i * WARPS < ntiles ? w2slice[(size_t)(n0 + i * WARPS) * 32] : zero2;
            }
            // all products first, then all exchanges, then all additions: the three do not wait
            // for one another tile by tile
            float c[NTW][4];
#pragma unroll
            for (int i = 0; i < NTW; ++i) {
                c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
                if (n0 + i * WARPS < ntiles) mma_bf16(c[i], h0.x, h1.x, h0.y, h1.y, wv[i].x, wv[i].y);
            }
            // c0, c1: token g, columns tile * 8 + 2t, + 1; c2, c3: token g + 8.  Neighbouring lanes trade
            // halves so that each holds four consecutive columns of one token: even t keeps token g,
            // odd t token g + 8.
            const bool odd = t & 1;
            float s0[NTW], s1[NTW];
#pragma unroll
            for (int i = 0; i < NTW; ++i) {
                s0[i] = __shfl_xor_sync(0xffffffffu, odd ? c[i][0] : c[i][2], 1);
                s1[i] = __shfl_xor_sync(0xffffffffu, odd ? c[i][1] : c[i][3], 1);
            }
            const int m = odd ? g + 8 : g;
#pragma unroll
            for (int i = 0; i < NTW; ++i) {
                const int tile = n0 + i * WARPS;
                if (tile >= ntiles) break;                                      // uniform in the warp
                while (next_own < tile) next_own += (int)gridDim.x;            // (no division on this path)
                const int col = tile * 8 + 4 * (t >> 1);
                float v0 = odd ? s0[i] : c[i][0], v1 = odd ? s1[i] : c[i][1], v2 = odd ? c[i][2] : s0[i], v3 = odd ? c[i][3] : s1[i];
                if (m < a.M && col < C) {                                       // C is a multiple of 4
                    if (tile == own_tile) {
                        v0 += own_add.x + own_x.x; v1 += own_add.y + own_x.y; v2 += own_add.z + own_x.z; v3 += own_add.w + own_x.w;
                    } else if (tile == next_own) {                              // more tiles than CTAs: further ones of mine
                        const float4 xv = *reinterpret_cast<const float4*>(a.x + (size_t)m * C + col);
                        const float4 bv = a.b2 ? *reinterpret_cast<const float4*>(a.b2 + col) : make_float4(0.f, 0.f, 0.f, 0.f);
                        v0 += xv.x + bv.x; v1 += xv.y + bv.y; v2 += xv.z + bv.z; v3 += xv.w + bv.w;
                    }
                    red_add_v4(a.out + (size_t)m * C + col, v0, v1, v2, v3);
                }
                if (i == 0) MG_STAMP(mlp, 10);
            }
        }
    }
    MG_STAMP(mlp, 7);
}

size_t mlp_smem(int mt, int C) {
    return (size_t)mt * ((size_t)C * 2 + XPAD) + (size_t)2 * C * sizeof(float) + (size_t)WARPS * mt * FS * sizeof(float) +
           (size_t)mt * HSTRIDE * sizeof(bf16);
}

}  // namespace

// Most tokens and the largest width the fused feed-forward takes.
MG_API int mg_mlp_fused_max_rows() { return 16; }
MG_API int mg_mlp_fused_max_width() { return MAX_WIDTH; }

// The kernel reads proj.weight [C, F] from a copy in the order its lanes use it: with G = ceil(F / 16)
// CTAs and C / 8 column tiles, element (((cta * C/8 + tile) * 8 + g) * 4 + t) * 4 + u of the copy is
// proj.weight[tile * 8 + g][cta * 16 + 4 * t + u] (zero where the unit is past F).  The caller makes
// that copy once per matrix; this is its length in elements.
MG_API long long mg_mlp_pack_elements(int C, int F) { return (long long)((F + FS - 1) / FS) * FS * C; }

// out = x + proj(gelu_tanh(fc(LayerNorm(x)) + b1)) + b2 for M <= 16 tokens, bfloat16 weights.
// w2_packed: proj.weight in the order of mg_mlp_pack_elements().  x, out, spare: three different
// [M, C] 32-bit buffers; out must be all zeros on entry; spare is all zeros on exit.  Returns MG_ERR_UNSUPPORTED for sizes it does not take (the caller then runs
// the two projections).
MG_API int mg_mlp_fused(const float* x, float* out, float* spare, const float* gain, const float* shift, float eps,
                        const void* w1, const float* b1, const void* w2_packed, const float* b2, int M, int C, int F,
                        void* stream) {
    if (M == 0) return MG_OK;
    MG_REQUIRE(M > 0 && C > 0 && F > 0, "feed-forward: bad sizes M=%d C=%d F=%d", M, C, F);
    MG_REQUIRE(x && out && spare && gain && w1 && w2_packed, "feed-forward: missing operand");
    MG_REQUIRE(x != out && x != spare && out != spare, "feed-forward: x, out and spare must be three buffers");
    const int mt = M <= 8 ? 8 : 16;
    const size_t smem = mlp_smem(mt, C);
    if (M > 16 || C > MAX_WIDTH || C % 8 != 0 || F % 8 != 0 || smem > 200 * 1024 || ((uintptr_t)w1 & 15) || ((uintptr_t)w2_packed & 15) ||
        ((uintptr_t)x & 15) || ((uintptr_t)out & 15) || ((uintptr_t)spare & 15) || ((uintptr_t)gain & 15) ||
        (shift && ((uintptr_t)shift & 15)) || (b2 && ((uintptr_t)b2 & 15)))
        return mg_set_error(MG_ERR_UNSUPPORTED, "feed-forward (fused): needs M <= 16, width <= 512, widths that are multiples of 8, aligned operands");
    MlpArgs a;
    a.x = x; a.out = out; a.spare = spare; a.gain = gain; a.shift = shift; a.eps = eps;
    a.w1 = (const bf16*)w1; a.b1 = b1; a.w2p = (const bf16*)w2_packed; a.b2 = b2; a.M = M; a.C = C; a.F = F;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaSuccess;
        for (auto fn : {mlp_fused_kernel<8>, mlp_fused_kernel<16>})
            if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "feed-forward (fused): cannot raise shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    const int grid = (F + FS - 1) / FS;
    cudaStream_t s = (cudaStream_t)stream;
    const cudaError_t le = mg_launch(mt == 8 ? mlp_fused_kernel<8> : mlp_fused_kernel<16>, dim3(grid), dim3(THREADS), smem, s, true, a);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "mlp_fused: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("mlp_fused");
    return MG_OK;
}
