// CUDA-core GEMM: out = epilogue(A[M,K] * W[N,K]^T + bias).
//
// This is the matrix product of the true 32-bit path (FFMA only; no tensor-core
// mode of reduced precision) and the exact reference of the tensor-core GEMM in
// the kernel tests (bf16 inputs, float32 accumulation).  The K loop runs in one
// fixed order, so a row's result does not depend on which other rows share its
// tile or on M.
//   y = x W^T + b            (reference: nn.Linear at src/model/paged_decoder.py:49-50, 178-179, 295-299)
//   epilogues: bias, GELU(tanh|erf) (reference: src/model/paged_decoder.py:273-280),
//              residual accumulate into a float32 stream (reference: :184, :188)
#include "common.cuh"

namespace ps {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TIn* __restrict__ A, int lda, const TIn* __restrict__ W, int ldw,
                 const float* __restrict__ bias, TOut* __restrict__ out, int ldo,
                 int M, int N, int K, int act, int accumulate) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_prologue();
    A = pdl_fresh(A);
    int tid = threadIdx.x;
    int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4x4 outputs each
    int lr = tid >> 2, lk = (tid & 3) * 4;  // loader: row 0..63, k offset 0,4,8,12
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int k = k0 + lk + j;
            int m = m0 + lr, n = n0 + lr;
            As[lk + j][lr] = (m < M && k < K) ? to_float(A[(size_t)m * lda + k]) : 0.f;
            Ws[lk + j][lr] = (n < N && k < K) ? to_float(W[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            v = apply_act(v, act);
            size_t o = (size_t)m * ldo + n;
            if (accumulate) v += to_float(out[o]);
            out[o] = from_float<TOut>(v);
        }
    }
}

template <typename TIn, typename TOut>
int launch_gemm_simt(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo,
                     int M, int N, int K, int act, int accumulate, cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    return launch_pdl(gemm_simt_kernel<TIn, TOut>, grid, dim3(256), 0, s, (const TIn*)A, lda, (const TIn*)W, ldw, bias,
                      (TOut*)out, ldo, M, N, K, act, accumulate);
}

}  // namespace ps

// in_dtype: dtype of A and W. out_dtype: dtype of out. accumulate: out += result (out must be f32).
PS_EXPORT int ps_gemm_simt(const void* A, int lda, const void* W, int ldw, const float* bias, void* out,
                           int ldo, int M, int N, int K, int in_dtype, int out_dtype, int act,
                           int accumulate, void* stream) {
    if (M <= 0 || N <= 0) return PS_OK;
    if (K <= 0 || lda < K || ldw < K || ldo < N) return PS_ERR_BAD_ARGUMENT;
    if (accumulate && out_dtype != PS_F32) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    using bf = __nv_bfloat16;
    if (in_dtype == PS_F32 && out_dtype == PS_F32)
        return ps::launch_gemm_simt<float, float>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, s);
    if (in_dtype == PS_BF16 && out_dtype == PS_F32)
        return ps::launch_gemm_simt<bf, float>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, s);
    if (in_dtype == PS_BF16 && out_dtype == PS_BF16)
        return ps::launch_gemm_simt<bf, bf>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, s);
    return PS_ERR_UNSUPPORTED;
}
