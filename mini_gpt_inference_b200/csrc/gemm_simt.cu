// out[m, n] = sum_k a[m, k] * w[n, k] (+ bias[n]) with an epilogue, on the CUDA cores.
//
// This is the true 32-bit matrix product of the engine (plain FMA, no tensor-core mode of
// reduced precision) and the fallback for bfloat16 sizes the tensor-core kernels refuse.
// Every output element sums its k terms in one fixed order (k = 0, 1, 2, ...), whatever the
// number of rows or the tile it falls in, so a token's result does not depend on what else
// is in the batch.  All sizes are accepted; tiles are predicated at the edges.
#include "common.cuh"

#define EPI_STORE 0      // out = acc + bias                (TOut)
#define EPI_GELU 1       // out = gelu_tanh(acc + bias)     (TOut)
#define EPI_RESIDUAL 2   // residual += acc + bias          (32-bit, in place)

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TIn, typename TOut, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TIn* __restrict__ a, const TIn* __restrict__ w, const float* __restrict__ bias,
                 TOut* __restrict__ out, float* __restrict__ residual, int M, int N, int K) {
    __shared__ float as[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tr = tid / 16, tc = tid % 16;          // 16 x 16 threads, each 4 x 4 outputs
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // Each thread brings 4 elements of a and 4 of w per k tile: row = tid / 4, k = (tid % 4) * 4 ..
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int m = m0 + lrow, n = n0 + lrow;
            as[lk + i][lrow] = (m < M && k < K) ? to_float(a[(size_t)m * K + k]) : 0.f;
            ws[lk + i][lrow] = (n < N && k < K) ? to_float(w[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float av[TM], wv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = as[k][tr * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wv[j] = ws[k][tc * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + tr * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tc * TN + j;
            if (n >= N) continue;
            float v = acc[i][j] + (bias ? bias[n] : 0.f);
            const size_t idx = (size_t)m * N + n;
            if (EPI == EPI_GELU) v = gelu_tanh(v);
            if (EPI == EPI_RESIDUAL)
                residual[idx] += v;
            else
                out[idx] = from_float<TOut>(v);
        }
    }
}

template <typename TIn, typename TOut>
int launch(const void* a, const void* w, const float* bias, void* out, float* residual, int M, int N,
           int K, int epilogue, cudaStream_t s) {
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM)), block(256);
    const TIn* ap = (const TIn*)a;
    const TIn* wp = (const TIn*)w;
    TOut* op = (TOut*)out;
    switch (epilogue) {
        case EPI_STORE: gemm_simt_kernel<TIn, TOut, EPI_STORE><<<grid, block, 0, s>>>(ap, wp, bias, op, residual, M, N, K); break;
        case EPI_GELU: gemm_simt_kernel<TIn, TOut, EPI_GELU><<<grid, block, 0, s>>>(ap, wp, bias, op, residual, M, N, K); break;
        case EPI_RESIDUAL: gemm_simt_kernel<TIn, TOut, EPI_RESIDUAL><<<grid, block, 0, s>>>(ap, wp, bias, op, residual, M, N, K); break;
        default: return mg_set_error(MG_ERR_ARG, "linear: unknown epilogue %d", epilogue);
    }
    MG_CHECK_LAUNCH("gemm_simt");
    return MG_OK;
}

}  // namespace

// a: [M, K] and w: [N, K], both row-major and of the same type (32-bit, or bfloat16 if in_bf16).
// epilogue 0/1 write `out` [M, N] (bfloat16 if out_bf16 else 32-bit); epilogue 2 adds into the
// 32-bit `residual` [M, N].  bias may be null.
MG_API int mg_linear_simt(const void* a, const void* w, const float* bias, void* out, float* residual,
                          int M, int N, int K, int epilogue, int in_bf16, int out_bf16, void* stream) {
    if (M == 0) return MG_OK;
    MG_REQUIRE(M > 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    MG_REQUIRE(ceil_div(M, BM) <= 65535, "linear: too many rows for one launch (%d)", M);
    MG_REQUIRE(epilogue == EPI_RESIDUAL ? residual != nullptr : out != nullptr, "linear: missing output");
    cudaStream_t s = (cudaStream_t)stream;
    if (in_bf16 && out_bf16) return launch<bf16, bf16>(a, w, bias, out, residual, M, N, K, epilogue, s);
    if (in_bf16) return launch<bf16, float>(a, w, bias, out, residual, M, N, K, epilogue, s);
    MG_REQUIRE(!out_bf16, "linear: 32-bit inputs with bfloat16 output is not a path of this engine");
    return launch<float, float>(a, w, bias, out, residual, M, N, K, epilogue, s);
}
