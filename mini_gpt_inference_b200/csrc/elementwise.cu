// Row-wise kernels: embedding with position add, LayerNorm, row gather, KV page write.
#include "common.cuh"

MG_GUARD_DECLARE(elementwise)

// ---- embedding + learned position add ---------------------------------------------------
// x[n, :] = tok_emb[id[n], :] + pos_emb[pos[n], :]   (32-bit out; pos_emb may be null)
// A row with a negative position is padding of a fixed-size batch: it becomes zeros.
// With `source` given, a row whose source[n] >= 0 takes its id from previous[source[n]] (the token
// the step before sampled, still on the device) instead of ids[n].
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ pos,
                             const TW* __restrict__ tok, const TW* __restrict__ ptab,
                             float* __restrict__ out, int width, const int* __restrict__ source,
                             const int* __restrict__ previous, int vocab, int n_positions, int n_previous) {
    const int n = blockIdx.x;
    float* orow = out + (size_t)n * width;
    int p = pos[n];
    if (p < 0) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) orow[c] = 0.f;
        return;
    }
    int id = ids[n];
    if (source != nullptr) {
        const int src = source[n];
        if (src >= 0 && MG_GUARDED(elementwise, MG_GUARD_SOURCE, src, n_previous)) id = previous[src];
    }
    // (guarded builds: an index out of range is recorded and row 0 is read in its place)
    if (!MG_GUARDED(elementwise, MG_GUARD_TOKEN, id, vocab)) id = 0;
    if (ptab != nullptr && !MG_GUARDED(elementwise, MG_GUARD_POSITION, p, n_positions)) p = 0;
    const TW* trow = tok + (size_t)id * width;
    const TW* prow = ptab ? ptab + (size_t)p * width : nullptr;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = to_float(trow[c]);
        if (prow) v += to_float(prow[c]);
        orow[c] = v;
    }
}

// vocab, n_positions: rows of tok and ptab; n_previous: ids that `previous` holds (what the indices
// are held against in guarded builds).
MG_API int mg_embed(const int* ids, const int* pos, const void* tok, const void* ptab, float* out,
                    int n_tokens, int width, int weights_bf16, const int* source, const int* previous,
                    int vocab, int n_positions, int n_previous, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && width > 0 && vocab > 0, "embed: bad sizes");
    MG_REQUIRE(source == nullptr || previous != nullptr, "embed: token sources without the ids they point to");
    cudaStream_t s = (cudaStream_t)stream;
    int threads = width >= 256 ? 256 : 128;
    if (weights_bf16)
        embed_kernel<bf16><<<n_tokens, threads, 0, s>>>(ids, pos, (const bf16*)tok, (const bf16*)ptab, out, width, source,
                                                       previous, vocab, n_positions, n_previous);
    else
        embed_kernel<float><<<n_tokens, threads, 0, s>>>(ids, pos, (const float*)tok, (const float*)ptab, out, width,
                                                        source, previous, vocab, n_positions, n_previous);
    MG_CHECK_LAUNCH("embed");
    return MG_OK;
}

// ---- LayerNorm -----------------------------------------------------------------------------
// One warp per row.  Mean, then the biased variance of the centred values, then the affine
// map; all in 32-bit.  y = (x - mean) * rsqrt(var + eps) * gain (+ shift).
template <typename TOut>
__global__ void layernorm_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                 const float* __restrict__ shift, TOut* __restrict__ y,
                                 int rows, int width, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + warp;
    // widths of up to 1024 in steps of 128: the row lives in registers, one trip to memory
    const bool fast = width % 128 == 0 && width <= 1024 &&
                      (((uintptr_t)x | (uintptr_t)gain | (uintptr_t)shift | (uintptr_t)y) & 15) == 0;
    float4 gn[8], sh[8];
    if (fast) {                                        // gain and shift are weights: fetched before the wait
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < width / 128) {
                gn[i] = *reinterpret_cast<const float4*>(gain + (lane + 32 * i) * 4);
                sh[i] = shift ? *reinterpret_cast<const float4*>(shift + (lane + 32 * i) * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
    }
    pdl_trigger();
    pdl_wait();                                        // x comes from the kernel in front
    if (row >= rows) return;
    const float* xr = x + (size_t)row * width;
    TOut* yr = y + (size_t)row * width;
    if (fast) {
        float4 v[8];
        const int n4 = width / 128;
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < n4) {
                v[i] = *reinterpret_cast<const float4*>(xr + (lane + 32 * i) * 4);
                sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            }
        const float mean = warp_sum(sum) / (float)width;
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < n4) {
                const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
                sq += (dx * dx + dy * dy) + (dz * dz + dw * dw);
            }
        const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)width + eps);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < n4) {
                const int c = (lane + 32 * i) * 4;
                store4(yr + c, (v[i].x - mean) * rstd * gn[i].x + sh[i].x, (v[i].y - mean) * rstd * gn[i].y + sh[i].y,
                       (v[i].z - mean) * rstd * gn[i].z + sh[i].z, (v[i].w - mean) * rstd * gn[i].w + sh[i].w);
            }
        return;
    }
    if (width % 4 == 0 && (((uintptr_t)x | (uintptr_t)gain | (uintptr_t)shift | (uintptr_t)y) & 15) == 0) {
        layernorm_row_chunked<TOut>(xr, width, gain, shift, eps, yr, lane);     // wide rows, 16-byte loads
        return;
    }
    float sum = 0.f;
    for (int c = lane; c < width; c += 32) sum += xr[c];
    const float mean = warp_sum(sum) / (float)width;
    float sq = 0.f;
    for (int c = lane; c < width; c += 32) {
        float d = xr[c] - mean;
        sq += d * d;
    }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)width + eps);
    for (int c = lane; c < width; c += 32) {
        float v = (xr[c] - mean) * rstd * gain[c];
        if (shift) v += shift[c];
        yr[c] = from_float<TOut>(v);
    }
}

MG_API int mg_layernorm(const float* x, const float* gain, const float* shift, void* y, int rows,
                        int width, float eps, int out_bf16, void* stream) {
    if (rows == 0) return MG_OK;
    MG_REQUIRE(rows > 0 && width > 0, "layernorm: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = 4;
    dim3 grid(ceil_div(rows, warps)), block(32 * warps);
    const cudaError_t le = out_bf16 ? mg_launch(layernorm_kernel<bf16>, grid, block, 0, s, true, x, gain, shift, (bf16*)y, rows, width, eps)
                                    : mg_launch(layernorm_kernel<float>, grid, block, 0, s, true, x, gain, shift, (float*)y, rows, width, eps);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "layernorm: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("layernorm");
    return MG_OK;
}

// ---- row gather (32-bit) ----------------------------------------------------------------------
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                   float* __restrict__ out, int width, int x_rows) {
    int row = rows[blockIdx.x];
    if (!MG_GUARDED(elementwise, MG_GUARD_ROW, row, x_rows)) row = 0;
    const float* src = x + (size_t)row * width;
    float* dst = out + (size_t)blockIdx.x * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
}

MG_API int mg_gather_rows(const float* x, const int* rows, float* out, int n_rows, int width, int x_rows,
                          void* stream) {
    if (n_rows == 0) return MG_OK;
    MG_REQUIRE(n_rows > 0 && width > 0 && x_rows > 0, "gather_rows: bad sizes");
    gather_rows_kernel<<<n_rows, 128, 0, (cudaStream_t)stream>>>(x, rows, out, width, x_rows);
    MG_CHECK_LAUNCH("gather_rows");
    return MG_OK;
}

// ---- write new keys and values into their pages --------------------------------------------------
// qkv row layout: [q: H*D | k: Hkv*D | v: Hkv*D].  Pages: [page, kv head, token in page, D].
// slot = page * page_tokens + token in page; a negative slot is skipped (padding rows).
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ qkv, const int* __restrict__ slots,
                                T* __restrict__ k_pages, T* __restrict__ v_pages, int qkv_width,
                                int q_width, int n_kv_head, int head_dim, int page_tokens, int num_pages) {
    const int n = blockIdx.x;
    const int slot = slots[n];
    pdl_trigger();
    pdl_wait();                                        // qkv comes from the kernel in front
    if (slot < 0) return;
    if (!MG_GUARDED(elementwise, MG_GUARD_CACHE_ROW, slot, (long long)num_pages * page_tokens)) return;
    const int page = slot / page_tokens, off = slot - page * page_tokens;
    const int kv_width = n_kv_head * head_dim;
    const T* krow = qkv + (size_t)n * qkv_width + q_width;
    const T* vrow = krow + kv_width;
    for (int i = threadIdx.x; i < kv_width; i += blockDim.x) {
        const int h = i / head_dim, d = i - h * head_dim;
        const size_t dst = (((size_t)page * n_kv_head + h) * page_tokens + off) * head_dim + d;
        k_pages[dst] = krow[i];
        v_pages[dst] = vrow[i];
    }
}

MG_API int mg_kv_store(const void* qkv, const int* slots, void* k_pages, void* v_pages, int n_tokens,
                       int n_head, int n_kv_head, int head_dim, int page_tokens, int num_pages, int is_bf16,
                       void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && n_kv_head > 0 && head_dim > 0 && page_tokens > 0,
               "kv_store: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    const int q_width = n_head * head_dim, qkv_width = (n_head + 2 * n_kv_head) * head_dim;
    const cudaError_t le =
        is_bf16 ? mg_launch(kv_store_kernel<bf16>, dim3(n_tokens), dim3(128), 0, s, true, (const bf16*)qkv, slots, (bf16*)k_pages,
                            (bf16*)v_pages, qkv_width, q_width, n_kv_head, head_dim, page_tokens, num_pages)
                : mg_launch(kv_store_kernel<float>, dim3(n_tokens), dim3(128), 0, s, true, (const float*)qkv, slots,
                            (float*)k_pages, (float*)v_pages, qkv_width, q_width, n_kv_head, head_dim, page_tokens, num_pages);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "kv_store: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("kv_store");
    return MG_OK;
}

// ---- feed sampled tokens back without a trip to the host -------------------------------------------
// token_ids[i] = previous[source[i]] where source[i] >= 0; other rows keep what the host wrote.
__global__ void gather_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ source,
                                     const int* __restrict__ previous, int n, int n_previous) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && source[i] >= 0 && MG_GUARDED(elementwise, MG_GUARD_SOURCE, source[i], n_previous))
        token_ids[i] = previous[source[i]];
}

MG_API int mg_gather_tokens(int* token_ids, const int* source, const int* previous, int n, int n_previous,
                            void* stream) {
    if (n == 0) return MG_OK;
    MG_REQUIRE(n > 0 && token_ids && source && previous, "gather_tokens: bad arguments");
    gather_tokens_kernel<<<ceil_div(n, 128), 128, 0, (cudaStream_t)stream>>>(token_ids, source, previous, n, n_previous);
    MG_CHECK_LAUNCH("gather_tokens");
    return MG_OK;
}

// ---- a step's integers from pinned host memory ------------------------------------------------------
// dst[i] = src[i], src being page-locked host memory that the device reads over the bus.  A few
// kilobytes travel in a couple of microseconds, and unlike a copy on the DMA engine the kernel
// puts no engine switch between itself and the kernels that follow on the stream.
__global__ void copy_ints_kernel(int* __restrict__ dst, const int* __restrict__ src, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

MG_API int mg_copy_ints(int* dst, const int* src, int n, void* stream) {
    if (n == 0) return MG_OK;
    MG_REQUIRE(n > 0 && dst && src, "copy_ints: bad arguments");
    const int blocks = ceil_div(n, 256) < 64 ? ceil_div(n, 256) : 64;
    copy_ints_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(dst, src, n);
    MG_CHECK_LAUNCH("copy_ints");
    return MG_OK;
}


namespace {
__global__ void zero_fill_kernel(uint4* __restrict__ dst, long long n16, uint8_t* __restrict__ tail, int tail_bytes) {
    pdl_trigger();
    pdl_wait();                                                  // the buffer may still be in use by the kernel in front
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) dst[i] = z;
    if (blockIdx.x == 0 && (int)threadIdx.x < tail_bytes) tail[threadIdx.x] = 0;
}
}  // namespace

// dst[0 .. bytes) = 0 (dst 16-byte aligned).
MG_API int mg_zero_fill(void* dst, long long bytes, void* stream) {
    if (bytes <= 0) return MG_OK;
    MG_REQUIRE(dst != nullptr && ((uintptr_t)dst & 15) == 0, "zero fill: the buffer must be 16-byte aligned");
    const long long n16 = bytes / 16;
    const int tail = (int)(bytes - n16 * 16);
    long long blocks = (n16 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 1184) blocks = 1184;
    const cudaError_t le = mg_launch(zero_fill_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, true,
                                     (uint4*)dst, n16, (uint8_t*)dst + n16 * 16, tail);
    if (le != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "zero_fill: %s", cudaGetErrorString(le));
    MG_CHECK_LAUNCH("zero_fill");
    return MG_OK;
}
