// Weight-streaming GEMM for few rows (decode): out[M<=64, N] = epilogue(A[M,K] W[N,K]^T + bias), bf16.
//
// In decode every weight is read once per step and used for only M tokens: the product is bound
// by the bytes of W, not by flops. The kernel therefore maps *weight rows* to the 16-row side of
// mma.sync.m16n8k16 and tokens to the 8-column side, and streams W straight from global memory
// into registers with 16-byte loads (no shared-memory staging of W):
//   * a CTA owns 16 consecutive weight rows n0..n0+15 and all M tokens;
//   * its warps split K: warp w takes the 32-wide k steps w, w+W, ...;
//   * lane (g = lane/4, t = lane%4) loads W[n0+g][k0+8t .. +7] and W[n0+g+8][k0+8t .. +7] and, per token
//     tile, A[8*mt+g][k0+8t .. +7]: the same permutation of k on both operands, so that the 8 loaded
//     values feed two MMAs (k = 8t+0..3 -> first, 8t+4..7 -> second) without any shuffle;
//   * partial sums of the warps are added in shared memory in warp order (fixed order), then the
//     epilogue adds bias, applies GELU, and stores bf16/float32 or accumulates into a float32 stream.
// Requirements: K % 8 == 0, lda % 8 == 0, 16-byte aligned A and W. Any N; M <= 64.
#include "common.cuh"

namespace ps {

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// MT: token tiles of 8. WARPS: warps per CTA. UNROLL: k steps whose loads are issued together.
template <int MT, int WARPS, typename TOut>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W, int ldw,
                   const float* __restrict__ bias, TOut* __restrict__ out, int ldo, int M, int N, int K,
                   int act, int accumulate) {
    extern __shared__ float red[];                 // [WARPS][16][8*MT]
    constexpr int UNROLL = 4;
    pdl_prologue();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    const int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);
    const __nv_bfloat16* w0 = W + (size_t)r0 * ldw + 8 * t;
    const __nv_bfloat16* w1 = W + (size_t)r1 * ldw + 8 * t;
    const __nv_bfloat16* arow[MT];
    bool aok[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        int m = 8 * mt + g;
        aok[mt] = m < M;
        arow[mt] = A + (size_t)(aok[mt] ? m : 0) * lda + 8 * t;
    }
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;

    const int steps = (K + 31) >> 5;
    for (int s0 = warp; s0 < steps; s0 += WARPS * UNROLL) {
        uint4 wa[UNROLL], wb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            int k = (s0 + u * WARPS) << 5;
            bool ok = (s0 + u * WARPS) < steps && (k + 8 * t) < K;
            wa[u] = ok ? ldg_stream(w0 + k) : make_uint4(0, 0, 0, 0);
            wb[u] = ok ? ldg_stream(w1 + k) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            int k = (s0 + u * WARPS) << 5;
            bool ok = (s0 + u * WARPS) < steps && (k + 8 * t) < K;
            uint32_t a1[4] = {wa[u].x, wb[u].x, wa[u].y, wb[u].y};
            uint32_t a2[4] = {wa[u].z, wb[u].z, wa[u].w, wb[u].w};
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint4 x = (ok && aok[mt]) ? *reinterpret_cast<const uint4*>(arow[mt] + k) : make_uint4(0, 0, 0, 0);
                uint32_t b1[2] = {x.x, x.y};
                uint32_t b2[2] = {x.z, x.w};
                mma_bf16_16816(acc[mt], a1, b1);
                mma_bf16_16816(acc[mt], a2, b2);
            }
        }
    }
    // acc[mt][0]: (row g, token 8mt+2t), [1]: (g, +1), [2]: (g+8, 2t), [3]: (g+8, 2t+1)
    constexpr int TOK = 8 * MT;
    float* mine = red + (size_t)warp * 16 * TOK;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        int c = 8 * mt + 2 * t;
        mine[g * TOK + c] = acc[mt][0];
        mine[g * TOK + c + 1] = acc[mt][1];
        mine[(g + 8) * TOK + c] = acc[mt][2];
        mine[(g + 8) * TOK + c + 1] = acc[mt][3];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 16 * TOK; e += WARPS * 32) {
        int r = e & 15, m = e >> 4;           // weight row fastest: consecutive threads store consecutive n
        int n = n0 + r;
        if (m >= M || n >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += red[(size_t)w * 16 * TOK + r * TOK + m];
        if (bias) v += bias[n];
        v = apply_act(v, act);
        size_t o = (size_t)m * ldo + n;
        if (accumulate) v += to_float(out[o]);
        out[o] = from_float<TOut>(v);
    }
}

template <int MT, int WARPS, typename TOut>
int launch_skinny(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo,
                  int M, int N, int K, int act, int accumulate, cudaStream_t s) {
    size_t smem = (size_t)WARPS * 16 * 8 * MT * sizeof(float);
    auto kernel = gemm_skinny_kernel<MT, WARPS, TOut>;
    if (smem > 48 * 1024) {
        static bool raised = false;
        if (!raised) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
                return PS_ERR_LAUNCH;
            raised = true;
        }
    }
    return launch_pdl(kernel, dim3((N + 15) / 16), dim3(WARPS * 32), smem, s, (const __nv_bfloat16*)A, lda,
                      (const __nv_bfloat16*)W, ldw, bias, (TOut*)out, ldo, M, N, K, act, accumulate);
}

template <int MT, typename TOut>
int pick_warps(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo, int M,
               int N, int K, int act, int accumulate, cudaStream_t s) {
    int steps = (K + 31) / 32;
    if (steps <= 32)
        return launch_skinny<MT, 4, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, s);
    if (steps <= 64)
        return launch_skinny<MT, 8, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, s);
    return launch_skinny<MT, 16, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, s);
}

template <typename TOut>
int pick_tiles(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo, int M,
               int N, int K, int act, int accumulate, cudaStream_t s) {
    if (M <= 8) return pick_warps<1, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, s);
    if (M <= 16) return pick_warps<2, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, s);
    if (M <= 32) return pick_warps<4, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, s);
    return pick_warps<8, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, s);
}

}  // namespace ps

PS_EXPORT int ps_gemm_skinny(const void* A, int lda, const void* W, int ldw, const float* bias, void* out,
                             int ldo, int M, int N, int K, int out_dtype, int act, int accumulate,
                             void* stream) {
    if (M <= 0 || N <= 0) return PS_OK;
    if (M > 64) return PS_ERR_UNSUPPORTED;
    if (K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || lda < K || ldw < K || ldo < N)
        return PS_ERR_UNSUPPORTED;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return PS_ERR_UNSUPPORTED;
    if (accumulate && out_dtype != PS_F32) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == PS_F32)
        return ps::pick_tiles<float>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, s);
    if (out_dtype == PS_BF16)
        return ps::pick_tiles<__nv_bfloat16>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, s);
    return PS_ERR_UNSUPPORTED;
}
