// Matrix products on the CUDA cores: out[m,n] = sum_k A[m,k] * W[n,k].
//
// This is the product of the true 32-bit engine (float inputs, float FMA, no
// reduced-precision matrix mode) and the fallback of the bfloat16 engine for
// shapes the tensor-core kernel refuses.  Every output element is accumulated
// by one thread over k = 0..K-1 in order, so a row's result does not depend on
// how many other rows are in the call.
#include "common.cuh"

namespace mdma {

enum GemmMode : int {
    kStore = 0,        // out = acc
    kAccumulate = 1,   // out += acc        (the residual stream, float)
    kSwiGLU = 2,       // out = act(acc_gate) * acc_up, with a second weight (act: SiLU or GELU)
};

constexpr int TM = 64, TN = 64, TK = 16, PAD = 4;

template <typename TA, typename TW, typename TO, int MODE>
__global__ void __launch_bounds__(256)
gemm_nt_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, const TW* __restrict__ W2,
               TO* __restrict__ out, int ldo, int M, int N, int K, const Ending e) {
    __shared__ float As[TK][TM + PAD];
    __shared__ float Ws[TK][TN + PAD];
    __shared__ float Ws2[MODE == kSwiGLU ? TK : 1][TN + PAD];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int ty = tid / 16, tx = tid % 16;
    const int lrow = tid / 4, lk = (tid % 4) * 4;

    float acc[4][4] = {};
    float acc2[MODE == kSwiGLU ? 4 : 1][4] = {};

    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int m = m0 + lrow, n = n0 + lrow;
            As[lk + i][lrow] = (m < M && k < K) ? to_float(A[(size_t)m * lda + k]) : 0.f;
            Ws[lk + i][lrow] = (n < N && k < K) ? to_float(W[(size_t)n * K + k]) : 0.f;
            if (MODE == kSwiGLU)
                Ws2[lk + i][lrow] = (n < N && k < K) ? to_float(W2[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
            if (MODE == kSwiGLU) {
#pragma unroll
                for (int j = 0; j < 4; ++j) w[j] = Ws2[k][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc2[i][j] = fmaf(a[i], w[j], acc2[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            TO* o = out + (size_t)m * ldo + n;
            const float r = acc[i][j] + ending_bias(e.bias, e.bias_dtype, n);
            if (MODE == kStore) {
                *o = from_float<TO>(r);
            } else if (MODE == kAccumulate) {
                *o = from_float<TO>(to_float(*o) + r);
            } else {
                *o = from_float<TO>(gate_activation(r, e.act) * (acc2[i][j] + ending_bias(e.bias2, e.bias_dtype, n)));
            }
        }
    }
}

template <typename TA, typename TW, typename TO>
static int launch_gemm(int mode, const void* A, int lda, const void* W, const void* W2, void* out, int ldo,
                       int M, int N, int K, const Ending& e, cudaStream_t stream) {
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    if (mode == kStore)
        gemm_nt_kernel<TA, TW, TO, kStore><<<grid, 256, 0, stream>>>((const TA*)A, lda, (const TW*)W, nullptr, (TO*)out, ldo, M, N, K, e);
    else if (mode == kAccumulate)
        gemm_nt_kernel<TA, TW, TO, kAccumulate><<<grid, 256, 0, stream>>>((const TA*)A, lda, (const TW*)W, nullptr, (TO*)out, ldo, M, N, K, e);
    else if (mode == kSwiGLU)
        gemm_nt_kernel<TA, TW, TO, kSwiGLU><<<grid, 256, 0, stream>>>((const TA*)A, lda, (const TW*)W, (const TW*)W2, (TO*)out, ldo, M, N, K, e);
    else
        return fail("gemm_simt: unknown mode %d", mode);
    MDMA_LAUNCH_OK("gemm_simt");
    return 0;
}

}  // namespace mdma

using namespace mdma;

extern "C" int mdma_gemm_simt(int mode, const void* A, int a_dtype, int lda, const void* W, const void* W2,
                              int w_dtype, void* out, int out_dtype, int ldo, int M, int N, int K,
                              const void* bias, const void* bias2, int bias_dtype, int act, cudaStream_t stream) {
    MDMA_REQUIRE(M >= 0 && N > 0 && K > 0 && lda >= K && ldo >= N, "gemm_simt: bad sizes M=%d N=%d K=%d lda=%d ldo=%d", M, N, K, lda, ldo);
    MDMA_REQUIRE(mode != kSwiGLU || W2 != nullptr, "gemm_simt: SwiGLU needs two weights");
    MDMA_REQUIRE(mode != kAccumulate || out_dtype == kF32, "gemm_simt: the residual stream is float");
    MDMA_REQUIRE((size_t)((M + TM - 1) / TM) <= 65535, "gemm_simt: too many rows (%d)", M);
    MDMA_REQUIRE(act == kActSilu || act == kActGeluTanh, "gemm_simt: unknown activation %d", act);
    MDMA_REQUIRE(bias_dtype == kF32 || bias_dtype == kBF16, "gemm_simt: unknown bias dtype %d", bias_dtype);
    if (M == 0) return 0;
    const Ending e{bias, mode == kSwiGLU ? bias2 : nullptr, bias_dtype, act};
    if (a_dtype == kF32 && w_dtype == kF32 && out_dtype == kF32)
        return launch_gemm<float, float, float>(mode, A, lda, W, W2, out, ldo, M, N, K, e, stream);
    if (a_dtype == kBF16 && w_dtype == kBF16 && out_dtype == kBF16)
        return launch_gemm<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(mode, A, lda, W, W2, out, ldo, M, N, K, e, stream);
    if (a_dtype == kBF16 && w_dtype == kBF16 && out_dtype == kF32)
        return launch_gemm<__nv_bfloat16, __nv_bfloat16, float>(mode, A, lda, W, W2, out, ldo, M, N, K, e, stream);
    return fail("gemm_simt: unsupported dtypes a=%d w=%d out=%d", a_dtype, w_dtype, out_dtype);
}
