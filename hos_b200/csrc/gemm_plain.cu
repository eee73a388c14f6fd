// Plain matrix product on the CUDA cores: out[m, n] = sum_k A[m, k] * W[n, k], with
// 32-bit FMA accumulation whatever the storage types are.  It is the 32-bit path's
// product (no tensor-core mode of reduced precision exists in it), the reference
// that the tensor-core product is checked against, and the product for sizes the
// tensor-core kernel refuses.  Any M, N, K.
//
// Epilogues: none; soft-cap (logits); gated (W holds gate rows then up rows,
// out = act(gate) * up), so that the 2F-wide intermediate is never written.
#include "common.cuh"

namespace hos {

constexpr int BM = 64, BN = 64, BK = 16;

enum Epilogue : int { kEpiNone = 0, kEpiSoftcap = 1, kEpiGated = 2 };

template <typename TA, typename TW, typename TO, int EPI>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TO* __restrict__ out,
                  int M, int N, int K, int lda, int ldw, int ldo, float cap, int act, int gate_rows) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float Us[EPI == kEpiGated ? BK : 1][BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4] = {};
    float acc_u[EPI == kEpiGated ? 4 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k per operand: 1024 elements, 4 per thread
        for (int e = threadIdx.x; e < BM * BK; e += 256) {
            const int r = e >> 4, kk = e & 15;
            const int m = m0 + r, k = k0 + kk;
            As[kk][r] = (m < M && k < K) ? to_float(A[(size_t)m * lda + k]) : 0.f;
            const int n = n0 + r;
            Ws[kk][r] = (n < N && k < K) ? to_float(W[(size_t)n * ldw + k]) : 0.f;
            if (EPI == kEpiGated)
                Us[kk][r] = (n < N && k < K) ? to_float(W[(size_t)(gate_rows + n) * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
            if (EPI == kEpiGated) {
                float u[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) u[j] = Us[kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc_u[i][j] = fmaf(a[i], u[j], acc_u[i][j]);
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
            float v = acc[i][j];
            if (EPI == kEpiSoftcap) v = softcap_precise(v, cap);
            if (EPI == kEpiGated) {
                const float a = act == 0 ? gelu_tanh(v) : v / (1.f + expf(-v));
                v = a * acc_u[i][j];
            }
            out[(size_t)m * ldo + n] = from_float<TO>(v);
        }
    }
}

template <typename TA, typename TW, typename TO>
static int launch_plain(const void* A, const void* W, void* out, int M, int N, int K, int lda,
                        int ldw, int ldo, int epi, float cap, int act, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) HOS_REFUSE("gemm_plain: %d rows are more than one launch takes", M);
    switch (epi) {
    case kEpiNone:
        gemm_plain_kernel<TA, TW, TO, kEpiNone><<<grid, 256, 0, stream>>>(
            (const TA*)A, (const TW*)W, (TO*)out, M, N, K, lda, ldw, ldo, cap, act, 0);
        break;
    case kEpiSoftcap:
        gemm_plain_kernel<TA, TW, TO, kEpiSoftcap><<<grid, 256, 0, stream>>>(
            (const TA*)A, (const TW*)W, (TO*)out, M, N, K, lda, ldw, ldo, cap, act, 0);
        break;
    case kEpiGated:
        gemm_plain_kernel<TA, TW, TO, kEpiGated><<<grid, 256, 0, stream>>>(
            (const TA*)A, (const TW*)W, (TO*)out, M, N, K, lda, ldw, ldo, cap, act, N);
        break;
    default:
        HOS_REFUSE("gemm_plain: unknown epilogue %d", epi);
    }
    return check_launch("gemm_plain");
}

}  // namespace hos

using namespace hos;

// out[M, N] = A[M, K] . W[N, K]^T.  For the gated epilogue W has 2N rows (gate, then up).
// Leading dimensions are in elements.
extern "C" int hos_gemm_plain(const void* A, int a_dtype, const void* W, int w_dtype, void* out,
                              int out_dtype, int M, int N, int K, int lda, int ldw, int ldo,
                              int epilogue, float cap, int act, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) HOS_REFUSE("gemm_plain: K must be positive");
#define HOS_CASE(da, dw, dout, TA, TW, TO)                                         \
    if (a_dtype == da && w_dtype == dw && out_dtype == dout)                       \
        return launch_plain<TA, TW, TO>(A, W, out, M, N, K, lda, ldw, ldo, epilogue, cap, act, stream);
    HOS_CASE(kF32, kF32, kF32, float, float, float)
    HOS_CASE(kBF16, kBF16, kBF16, bf16, bf16, bf16)
    HOS_CASE(kBF16, kBF16, kF32, bf16, bf16, float)
    HOS_CASE(kBF16, kF32, kBF16, bf16, float, bf16)
    HOS_CASE(kBF16, kF32, kF32, bf16, float, float)
    HOS_CASE(kF32, kBF16, kF32, float, bf16, float)
#undef HOS_CASE
    HOS_REFUSE("gemm_plain: no kernel for dtypes A=%d W=%d out=%d", a_dtype, w_dtype, out_dtype);
}
