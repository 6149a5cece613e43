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
    constexpr int UNROLL = 6;                      // K = 3072 over 16 warps is one round of loads
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


// ------------------------------------------------------------------------------------------------
// The same product with the norm of its input fused in front and the cache write fused behind:
//   A[m, :] = norm(X[rows[m] or m, :]) computed on the fly from the float32 residual stream
//             (statistics in two passes in float32, one warp per row, while the first weight
//             loads are already in flight), rounded to bfloat16 as the separate norm kernel does;
//   columns n >= q_width of the result are keys and values: they are written straight into the
//             request's page (cache layout of attention_simt.cu) instead of the output buffer.
// This removes the norm launch and the kv-append launch of a decode step.
struct KvScatter {
    __nv_bfloat16* k_pool;
    __nv_bfloat16* v_pool;
    long long page_stride;
    const int* token_item;
    const int* positions;
    const int* block_table;
    int bt_stride;
    int q_width;       // columns [0, q_width) are queries and go to `out`
    int kv_width;      // then kv_width key columns, then kv_width value columns
    int head_dim;
    int page_size;
};

struct NormInput {
    const float* x;    // float32 rows
    int ldx;
    const int* rows;   // optional gather of rows
    const float* gamma;
    const float* beta; // optional
    float eps;
    int has_mean;
};

template <int MT, int WARPS, typename TOut>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_fused_kernel(NormInput in, const __nv_bfloat16* __restrict__ W, int ldw,
                         const float* __restrict__ bias, TOut* __restrict__ out, int ldo, int M, int N, int K,
                         int act, int accumulate, KvScatter kv) {
    // shared memory: cross-warp sums [WARPS][16][8*MT] floats, then the normed rows [8*MT][K+8] bf16
    extern __shared__ __align__(16) float red[];
    constexpr int UNROLL = 6;
    constexpr int TOK = 8 * MT;
    const int lda_s = K + 8;                       // padded: 16-byte reads of 8 rows hit 8 different bank groups
    __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(red + (size_t)WARPS * 16 * TOK);
    pdl_prologue();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    const int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);
    const __nv_bfloat16* w0 = W + (size_t)r0 * ldw + 8 * t;
    const __nv_bfloat16* w1 = W + (size_t)r1 * ldw + 8 * t;
    const int steps = (K + 31) >> 5;

    // first batch of weight loads: in flight while the rows are normed
    uint4 wa[UNROLL], wb[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        int k = (warp + u * WARPS) << 5;
        bool ok = (warp + u * WARPS) < steps && (k + 8 * t) < K;
        wa[u] = ok ? ldg_stream(w0 + k) : make_uint4(0, 0, 0, 0);
        wb[u] = ok ? ldg_stream(w1 + k) : make_uint4(0, 0, 0, 0);
    }
    // norm: one warp per row; the row sits in registers (float4 pieces, all loads issued at once) when
    // K <= 1024, else it is read again from L1
    const int quads = K >> 2;
    for (int m = warp; m < M; m += WARPS) {
        const float4* xr = reinterpret_cast<const float4*>(in.x + (size_t)(in.rows ? in.rows[m] : m) * in.ldx);
        constexpr int HOLD = 8;
        float4 v[HOLD];
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < HOLD; ++i) {
            int c = lane + 32 * i;
            v[i] = c < quads ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
            sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
        for (int c = lane + 32 * HOLD; c < quads; c += 32) { float4 y = xr[c]; sum += (y.x + y.y) + (y.z + y.w); }
        const float mean = in.has_mean ? warp_sum(sum) / (float)K : 0.f;
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < HOLD; ++i) {
            if (lane + 32 * i < quads) {
                float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
                sq += (a * a + b * b) + (c * c + d * d);
            }
        }
        for (int c = lane + 32 * HOLD; c < quads; c += 32) {
            float4 y = xr[c];
            float a = y.x - mean, b = y.y - mean, cc = y.z - mean, d = y.w - mean;
            sq += (a * a + b * b) + (cc * cc + d * d);
        }
        const float rstd = rsqrtf(warp_sum(sq) / (float)K + in.eps);
        const float4* g4 = reinterpret_cast<const float4*>(in.gamma);
        const float4* b4 = reinterpret_cast<const float4*>(in.beta);
        for (int c = lane; c < quads; c += 32) {
            const int i = c >> 5;
            float4 y = (i < HOLD) ? make_float4(0.f, 0.f, 0.f, 0.f) : xr[c];
#pragma unroll
            for (int j = 0; j < HOLD; ++j) if (j == i) y = v[j];
            const float4 gm = g4[c];
            const float4 bt = in.beta ? b4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
            __nv_bfloat162 lo = __floats2bfloat162_rn((y.x - mean) * rstd * gm.x + bt.x, (y.y - mean) * rstd * gm.y + bt.y);
            __nv_bfloat162 hi = __floats2bfloat162_rn((y.z - mean) * rstd * gm.z + bt.z, (y.w - mean) * rstd * gm.w + bt.w);
            *reinterpret_cast<uint2*>(a_s + (size_t)m * lda_s + 4 * c) =
                make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
    }
    __syncthreads();

    const __nv_bfloat16* arow[MT];
    bool aok[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        int m = 8 * mt + g;
        aok[mt] = m < M;
        arow[mt] = a_s + (size_t)(aok[mt] ? m : 0) * lda_s + 8 * t;
    }
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;

    for (int s0 = warp; s0 < steps; s0 += WARPS * UNROLL) {
        if (s0 != warp) {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                int k = (s0 + u * WARPS) << 5;
                bool ok = (s0 + u * WARPS) < steps && (k + 8 * t) < K;
                wa[u] = ok ? ldg_stream(w0 + k) : make_uint4(0, 0, 0, 0);
                wb[u] = ok ? ldg_stream(w1 + k) : make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            int k = (s0 + u * WARPS) << 5;
            bool ok = (s0 + u * WARPS) < steps && (k + 8 * t) < K;
            if (!ok) continue;
            uint32_t a1[4] = {wa[u].x, wb[u].x, wa[u].y, wb[u].y};
            uint32_t a2[4] = {wa[u].z, wb[u].z, wa[u].w, wb[u].w};
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint4 x = aok[mt] ? *reinterpret_cast<const uint4*>(arow[mt] + k) : make_uint4(0, 0, 0, 0);
                uint32_t b1[2] = {x.x, x.y}, b2[2] = {x.z, x.w};
                mma_bf16_16816(acc[mt], a1, b1);
                mma_bf16_16816(acc[mt], a2, b2);
            }
        }
    }
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
        int r = e & 15, m = e >> 4;
        int n = n0 + r;
        if (m >= M || n >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += red[(size_t)w * 16 * TOK + r * TOK + m];
        if (bias) v += bias[n];
        v = apply_act(v, act);
        if (kv.k_pool && n >= kv.q_width) {
            int c = n - kv.q_width;
            __nv_bfloat16* pool = kv.k_pool;
            if (c >= kv.kv_width) { c -= kv.kv_width; pool = kv.v_pool; }
            int head = c / kv.head_dim, d = c - head * kv.head_dim;
            int p = kv.positions[m];
            int page = kv.block_table[(size_t)kv.token_item[m] * kv.bt_stride + p / kv.page_size];
            if (page >= 0)
                pool[(size_t)page * kv.page_stride + ((size_t)head * kv.page_size + (p % kv.page_size)) * kv.head_dim + d] =
                    __float2bfloat16_rn(v);
            continue;
        }
        size_t o = (size_t)m * ldo + n;
        if (accumulate) v += to_float(out[o]);
        out[o] = from_float<TOut>(v);
    }
}

template <int MT, int WARPS, typename TOut>
int launch_skinny_fused(const NormInput& in, const void* W, int ldw, const float* bias, void* out, int ldo, int M,
                        int N, int K, int act, int accumulate, const KvScatter& kv, cudaStream_t s) {
    size_t smem = (size_t)WARPS * 16 * 8 * MT * sizeof(float) + (size_t)8 * MT * (K + 8) * 2;
    auto kernel = gemm_skinny_fused_kernel<MT, WARPS, TOut>;
    if (smem > 200 * 1024) return PS_ERR_UNSUPPORTED;
    static size_t raised = 48 * 1024;
    if (smem > raised) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return PS_ERR_LAUNCH;
        raised = smem;
    }
    return launch_pdl(kernel, dim3((N + 15) / 16), dim3(WARPS * 32), smem, s, in, (const __nv_bfloat16*)W, ldw, bias,
                      (TOut*)out, ldo, M, N, K, act, accumulate, kv);
}

template <int MT, typename TOut>
int pick_warps_fused(const NormInput& in, const void* W, int ldw, const float* bias, void* out, int ldo, int M, int N,
                     int K, int act, int accumulate, const KvScatter& kv, cudaStream_t s) {
    int steps = (K + 31) / 32;
    if (steps <= 24) return launch_skinny_fused<MT, 4, TOut>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
    if (steps <= 48) return launch_skinny_fused<MT, 8, TOut>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
    return launch_skinny_fused<MT, 16, TOut>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
}

template <typename TOut>
int pick_tiles_fused(const NormInput& in, const void* W, int ldw, const float* bias, void* out, int ldo, int M, int N,
                     int K, int act, int accumulate, const KvScatter& kv, cudaStream_t s) {
    if (M <= 8) return pick_warps_fused<1, TOut>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
    if (M <= 16) return pick_warps_fused<2, TOut>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
    return pick_warps_fused<4, TOut>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
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

// out = epilogue(norm(x[rows]) W^T + bias) for at most 32 rows, with an optional cache write of the key and
// value columns (kv_* arguments; k_pool null = none). x float32 with ldx % 4 == 0, K % 8 == 0.
PS_EXPORT int ps_gemm_skinny_fused(const float* x, int ldx, const int* rows, const float* gamma, const float* beta,
                                   float eps, int has_mean, const void* W, int ldw, const float* bias, void* out,
                                   int ldo, int M, int N, int K, int out_dtype, int act, int accumulate,
                                   void* k_pool, void* v_pool, long long page_stride, const int* token_item,
                                   const int* positions, const int* block_table, int bt_stride, int q_width,
                                   int kv_width, int head_dim, int page_size, void* stream) {
    if (M <= 0 || N <= 0) return PS_OK;
    if (M > 32) return PS_ERR_UNSUPPORTED;
    if (K <= 0 || K % 8 != 0 || ldx % 4 != 0 || ldw % 8 != 0 || ldx < K || ldw < K || ldo < N) return PS_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)W & 15) || ((uintptr_t)gamma & 15) || ((uintptr_t)beta & 15))
        return PS_ERR_UNSUPPORTED;
    if (accumulate && out_dtype != PS_F32) return PS_ERR_BAD_ARGUMENT;
    if (k_pool && (q_width + 2 * kv_width != N || head_dim <= 0 || kv_width % head_dim != 0 || page_size <= 0))
        return PS_ERR_BAD_ARGUMENT;
    ps::NormInput in{x, ldx, rows, gamma, beta, eps, has_mean};
    ps::KvScatter kv{(__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, page_stride, token_item, positions, block_table,
                     bt_stride, q_width, kv_width, head_dim, page_size};
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == PS_F32)
        return ps::pick_tiles_fused<float>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
    if (out_dtype == PS_BF16)
        return ps::pick_tiles_fused<__nv_bfloat16>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
    return PS_ERR_UNSUPPORTED;
}
