// What the small- and mid-batch projection kernels do with a finished sum: bias is added by the
// caller; here the activation, the store (bfloat16 or 32-bit), the add into the 32-bit residual
// stream, and for the QKV projection the copy of key and value features to their cache rows.
#pragma once

#include "common.cuh"

#define EPI_STORE 0
#define EPI_GELU 1
#define EPI_RESIDUAL 2

struct LinearEpilogue {
    const float* bias;               // may be null
    void* out;                       // [M, N]
    float* residual;                 // [M, N] for EPI_RESIDUAL
    int M, N, epilogue, out_bf16;
    // key/value sink of the QKV projection (k_pages null: none)
    bf16* k_pages;
    bf16* v_pages;
    const int* slots;                // [M] flat cache row of each token, < 0: skip
    int q_width, n_kv_head, head_dim, page_tokens;
    int num_pages;                   // pages of the pool (what a cache row is held against in guarded builds)
};

// the fault record of the file that includes this (each exports its own reader)
MG_GUARD_RECORD(linear_index_fault)

// v: the sum with its bias.  `res` is the residual value if the caller fetched it already, `slot`
// the token's cache row if it did (pass have_slot = false to have it read here).
__device__ __forceinline__ void linear_finish(const LinearEpilogue& e, int m, int n, float v, bool have_res, float res,
                                              bool have_slot = false, int slot_in = -1) {
    if (e.epilogue == EPI_GELU) v = gelu_tanh(v);
    const size_t idx = (size_t)m * e.N + n;
    if (e.epilogue == EPI_RESIDUAL) {
        e.residual[idx] = (have_res ? res : e.residual[idx]) + v;
    } else if (e.out_bf16) {
        const bf16 hv = __float2bfloat16_rn(v);
        reinterpret_cast<bf16*>(e.out)[idx] = hv;
        if (e.k_pages != nullptr && n >= e.q_width) {
            const int slot = have_slot ? slot_in : e.slots[m];
            if (slot >= 0 && MG_GUARDED_IN(linear_index_fault, MG_GUARD_CACHE_ROW, slot, (long long)e.num_pages * e.page_tokens)) {
                const int kv_width = e.n_kv_head * e.head_dim;
                const int f = n - e.q_width;
                const int which = f / kv_width, fi = f - which * kv_width;
                const int h = fi / e.head_dim, d = fi - h * e.head_dim;
                const int page = slot / e.page_tokens, off = slot - page * e.page_tokens;
                const size_t dst = (((size_t)page * e.n_kv_head + h) * e.page_tokens + off) * e.head_dim + d;
                (which == 0 ? e.k_pages : e.v_pages)[dst] = hv;
            }
        }
    } else {
        reinterpret_cast<float*>(e.out)[idx] = v;
    }
}

// D[16x8] += A[16x16] . B[16x8], bfloat16 in, 32-bit accumulate (warp-level mma).
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
