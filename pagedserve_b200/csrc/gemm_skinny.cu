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

// Where output column n of a packed q|k|v product goes inside a page: the pool and the offset of (head, 0, d)
// from the row's place in the page; pool null for a query column (or no cache write at all). Integer
// divisions, done once per thread before the wait: a thread's column is the same in every epilogue round.
struct KvColumn {
    int which;      // 0: not a cache column, 1: keys, 2: values
    int offset;     // elements from the row's place in the page (a page of one layer is far below 2^31 elements)
};
__device__ __forceinline__ KvColumn kv_column(const KvScatter& kv, int n, int N) {
    KvColumn col{0, 0};
    if (kv.k_pool && n >= kv.q_width && n < N) {
        int c = n - kv.q_width;
        col.which = 1;
        if (c >= kv.kv_width) { c -= kv.kv_width; col.which = 2; }
        const int head = c / kv.head_dim, d = c - head * kv.head_dim;
        col.offset = head * kv.page_size * kv.head_dim + d;
    }
    return col;
}
// position -> (page index, place in the page); pages are almost always a power of two long
__device__ __forceinline__ void split_position(int p, int page_size, int* index, int* within) {
    if ((page_size & (page_size - 1)) == 0) {
        *index = p >> (31 - __clz(page_size));
        *within = p & (page_size - 1);
    } else {
        *index = p / page_size;
        *within = p - *index * page_size;
    }
}

// MT: token tiles of 8. WARPS: warps per CTA. UNROLL: k steps whose loads a warp issues together (a round);
// WARPS * UNROLL * 32 >= K makes it one round, so that the latency of the weights is paid once.
template <int MT, int WARPS, int UNROLL, typename TOut>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W, int ldw,
                   const float* __restrict__ bias, TOut* __restrict__ out, int ldo, int M, int N, int K,
                   int act, int accumulate, KvScatter kv) {
    // cross-warp sums [WARPS][16][8*MT] floats, then the cache address of each row [8*MT] (64-bit)
    extern __shared__ __align__(16) float red[];
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

    // what the output holds (to be added to) is fetched right after the wait, long before the epilogue needs it
    constexpr int TOK = 8 * MT;
    constexpr int EPT = (16 * TOK + WARPS * 32 - 1) / (WARPS * 32);      // epilogue elements per thread
    long long* dst_s = reinterpret_cast<long long*>(red + (size_t)WARPS * 16 * TOK);
    float prev[EPT];
    auto after_wait = [&]() {
        pdl_prologue();
        if (kv.k_pool) {
            // where a row's keys and values go: offset of (page, head 0, position in page, 0), or -1
            for (int m = threadIdx.x; m < M; m += WARPS * 32) {
                int index, within;
                split_position(kv.positions[m], kv.page_size, &index, &within);
                const int page = kv.block_table[(size_t)kv.token_row[m] * kv.bt_stride + index];
                dst_s[m] = page >= 0 ? (long long)page * kv.page_stride + (long long)within * kv.head_dim : -1;
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) arow[mt] = pdl_fresh(arow[mt]);
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const int e = threadIdx.x + j * WARPS * 32;
            const int n = n0 + (e & 15), m = e >> 4;
            prev[j] = (accumulate && e < 16 * TOK && m < M && n < N) ? to_float(out[(size_t)m * ldo + n]) : 0.f;
        }
    };
    // the bias of this thread's output column (the same in every epilogue round: the CTA's thread count is a
    // multiple of 16), fetched before the wait: its line was last touched a step ago and comes from DRAM
    const float bias_mine = bias ? bias[min(n0 + (int)(threadIdx.x & 15), N - 1)] : 0.f;
    const int steps = (K + 31) >> 5;
    bool waited = false;
    for (int s0 = warp; s0 < steps; s0 += WARPS * UNROLL) {
        uint4 wa[UNROLL], wb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            int k = (s0 + u * WARPS) << 5;
            bool ok = (s0 + u * WARPS) < steps && (k + 8 * t) < K;
            wa[u] = ok ? ldg_stream(w0 + k) : make_uint4(0, 0, 0, 0);
            wb[u] = ok ? ldg_stream(w1 + k) : make_uint4(0, 0, 0, 0);
        }
        if (!waited) {               // the first weights are on their way: now wait for the kernel that writes A
            after_wait();
            waited = true;
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
    if (!waited) after_wait();
    // acc[mt][0]: (row g, token 8mt+2t), [1]: (g, +1), [2]: (g+8, 2t), [3]: (g+8, 2t+1)
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
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int e = threadIdx.x + j * WARPS * 32;
        if (e >= 16 * TOK) break;
        int r = e & 15, m = e >> 4;           // weight row fastest: consecutive threads store consecutive n
        int n = n0 + r;
        if (m >= M || n >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += red[(size_t)w * 16 * TOK + r * TOK + m];
        v += bias_mine;
        v = apply_act(v, act);
        if (kv.k_pool && n >= kv.q_width) {        // a key or value column: into the row's page
            const KvColumn col = kv_column(kv, n, N);
            const long long base = dst_s[m];
            if (base >= 0) (col.which == 1 ? kv.k_pool : kv.v_pool)[base + col.offset] = __float2bfloat16_rn(v);
            continue;
        }
        v += prev[j];
        out[(size_t)m * ldo + n] = from_float<TOut>(v);
    }
}

template <int MT, int WARPS, int UNROLL, typename TOut>
int launch_skinny(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo,
                  int M, int N, int K, int act, int accumulate, const KvScatter& kv, cudaStream_t s) {
    size_t smem = (size_t)WARPS * 16 * 8 * MT * sizeof(float) + (size_t)8 * MT * sizeof(long long);
    auto kernel = gemm_skinny_kernel<MT, WARPS, UNROLL, TOut>;
    static size_t raised[MAX_DEVICES] = {0};
    if (!ensure_dynamic_smem((const void*)kernel, smem, raised)) return PS_ERR_LAUNCH;
    return launch_pdl(kernel, dim3((N + 15) / 16), dim3(WARPS * 32), smem, s, (const __nv_bfloat16*)A, lda,
                      (const __nv_bfloat16*)W, ldw, bias, (TOut*)out, ldo, M, N, K, act, accumulate, kv);
}

template <int MT, typename TOut>
int pick_warps(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo, int M,
               int N, int K, int act, int accumulate, const KvScatter& kv, cudaStream_t s) {
    // warps and steps per round such that the k steps of a warp are one round of loads where that is possible
    // (K up to 4,096, at most 8 rows); more token tiles keep the rounds short, their accumulators need the
    // registers
    const int steps = (K + 31) / 32;
#define PS_SKINNY(W_, U_) \
    return launch_skinny<MT, W_, U_, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s)
    if constexpr (MT >= 2) {
        if (steps <= 32) PS_SKINNY(4, 6);
        if (steps <= 64) PS_SKINNY(8, 6);
        PS_SKINNY(16, 6);
    } else {
        // One CTA per 16 output columns. The (8, 8) instance keeps 2 CTAs on an SM (128 registers), the (8, 4)
        // instance 3 (80 registers) at the price of a second round of loads: it wins wherever the grid is more
        // than the 296 CTAs of one wave of the former (8 x 4,800 x 1,600: 300 CTAs, 5.2 -> 4.2 us; 8 x 6,400 x
        // 1,600: 5.8 -> 4.7 us) and for short K (8 x 2,304 x 768: 2.02 -> 1.86 us), but not for a vocabulary's
        // thousands of CTAs at short K (15.0 vs 15.9 us).
        const int ctas = (N + 15) / 16;
        if (steps <= 24) {
            if (ctas <= 444) PS_SKINNY(8, 4);
            PS_SKINNY(4, 6);
        }
        if (steps <= 32) PS_SKINNY(8, 4);
        if (steps <= 64) {
            if (ctas > 296) PS_SKINNY(8, 4);
            PS_SKINNY(8, 8);
        }
        if (steps <= 96) PS_SKINNY(16, 6);
        PS_SKINNY(16, 8);
    }
#undef PS_SKINNY
}

template <typename TOut>
int pick_tiles(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo, int M,
               int N, int K, int act, int accumulate, const KvScatter& kv, cudaStream_t s) {
    // the MMAs of a CTA grow with the token tiles, and from 17 rows on they are what the kernel waits for:
    // every count of tiles has its own instance
#define PS_TILES(MT_) \
    return pick_warps<MT_, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s)
    switch ((M + 7) / 8) {
        case 1: PS_TILES(1);
        case 2: PS_TILES(2);
        case 3: PS_TILES(3);
        case 4: PS_TILES(4);
        case 5: PS_TILES(5);
        case 6: PS_TILES(6);
        case 7: PS_TILES(7);
        default: PS_TILES(8);
    }
#undef PS_TILES
}


// ------------------------------------------------------------------------------------------------
// The same product with the norm of its input fused in front and the cache write fused behind:
//   A[m, :] = norm(X[rows[m] or m, :]) computed on the fly from the float32 residual stream
//             (statistics in two passes in float32, one warp per row, while the first weight
//             loads are already in flight), rounded to bfloat16 as the separate norm kernel does;
//   columns n >= q_width of the result are keys and values: they are written straight into the
//             request's page (cache layout of attention_simt.cu) instead of the output buffer.
// This removes the norm launch and the kv-append launch of a decode step.

struct NormInput {
    const float* x;    // float32 rows
    int ldx;
    const int* rows;   // optional gather of rows
    const float* gamma;
    const float* beta; // optional
    float eps;
    int has_mean;
};

template <int MT, int WARPS, int UNROLL, typename TOut>
__global__ void __launch_bounds__(WARPS * 32, WARPS <= 8 ? 2 : 1)
gemm_skinny_fused_kernel(NormInput in, const __nv_bfloat16* __restrict__ W, int ldw,
                         const float* __restrict__ bias, TOut* __restrict__ out, int ldo, int M, int N, int K,
                         int act, int accumulate, KvScatter kv) {
    // shared memory: cross-warp sums [WARPS][16][8*MT] floats, the norm's scale and shift [2][K] floats,
    // the cache address of each row [8*MT] (64-bit), then the normed rows [8*MT][K+8] bf16
    extern __shared__ __align__(16) float red[];
    constexpr int TOK = 8 * MT;
    const int lda_s = K + 8;                       // padded: 16-byte reads of 8 rows hit 8 different bank groups
    float* gamma_s = red + (size_t)WARPS * 16 * TOK;
    float* beta_s = gamma_s + K;
    long long* dst_s = reinterpret_cast<long long*>(beta_s + K);
    __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(dst_s + TOK);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    const int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);
    const __nv_bfloat16* w0 = W + (size_t)r0 * ldw + 8 * t;
    const __nv_bfloat16* w1 = W + (size_t)r1 * ldw + 8 * t;
    const int steps = (K + 31) >> 5;
    const int quads = K >> 2;

    // Before the wait, what no kernel writes: the first batch of weights (to registers) and the norm's
    // scale and shift (to shared memory). They are in flight while the kernel before this one ends.
    uint4 wa[UNROLL], wb[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        int k = (warp + u * WARPS) << 5;
        bool ok = (warp + u * WARPS) < steps && (k + 8 * t) < K;
        wa[u] = ok ? ldg_stream(w0 + k) : make_uint4(0, 0, 0, 0);
        wb[u] = ok ? ldg_stream(w1 + k) : make_uint4(0, 0, 0, 0);
    }
    const float bias_mine = bias ? bias[min(n0 + (int)(threadIdx.x & 15), N - 1)] : 0.f;   // as in the kernel above
    const float inv_k = 1.0f / (float)K;       // divisions and the like happen here, off the critical path
    const KvColumn kv_col = kv_column(kv, n0 + (int)(threadIdx.x & 15), N);
    // Nothing before the wait waits for memory itself: when the kernel in front has already ended, every
    // microsecond here is on the step's critical path. Scale and shift go to shared memory by asynchronous
    // copies that are waited for where the norm needs them; a row's position and block-table row are asked for
    // here and used after the wait. (Positions and tables are written by the step's first kernel, never by the
    // kernel directly in front of this one: only that one may still be running before the wait.)
    for (int c = threadIdx.x; c < quads; c += WARPS * 32) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(gamma_s + 4 * c)),
                     "l"(in.gamma + 4 * c) : "memory");
        if (in.beta)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(beta_s + 4 * c)),
                         "l"(in.beta + 4 * c) : "memory");
        else
            reinterpret_cast<float4*>(beta_s)[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    const bool kv_row = kv.k_pool && threadIdx.x < M;
    int kv_p = 0, kv_table_row = 0;
    if (kv_row) {
        kv_p = kv.positions[threadIdx.x];
        kv_table_row = kv.token_row[threadIdx.x];
    }
    pdl_prologue();            // the rows come from the kernel before this one
    int kv_page = -1, kv_index = 0, kv_within = 0;
    if (kv_row) {
        split_position(kv_p, kv.page_size, &kv_index, &kv_within);
        kv_page = kv.block_table[(size_t)kv_table_row * kv.bt_stride + kv_index];
    }
    bool staged = false;       // scale and shift have arrived and every thread can see them
    // norm: one warp per row, two rows at a time so that their loads and reductions overlap; a row sits in
    // registers (float4 pieces, all loads issued at once) when K <= 1024, else its tail is read again from L1.
    // Statistics in two passes in float32, as the separate norm kernel does.
    // two rows per warp where a warp has more than one row; 16 warps have too few registers for that
    constexpr bool PAIR = WARPS <= 8 && TOK > WARPS;
    for (int m0 = warp; m0 < M; m0 += (PAIR ? 2 : 1) * WARPS) {
        constexpr int HOLD = 8;
        const int m1 = m0 + WARPS;
        const bool two = PAIR && m1 < M;
        const float4* xa = reinterpret_cast<const float4*>(in.x + (size_t)(in.rows ? in.rows[m0] : m0) * in.ldx);
        const float4* xb = two ? reinterpret_cast<const float4*>(in.x + (size_t)(in.rows ? in.rows[m1] : m1) * in.ldx) : xa;
        float4 va[HOLD], vb[HOLD];
#pragma unroll
        for (int i = 0; i < HOLD; ++i) {
            int c = lane + 32 * i;
            va[i] = c < quads ? xa[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < HOLD; ++i) {
            int c = lane + 32 * i;
            vb[i] = (two && c < quads) ? xb[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int i = 0; i < HOLD; ++i) {
            sum_a += (va[i].x + va[i].y) + (va[i].z + va[i].w);
            sum_b += (vb[i].x + vb[i].y) + (vb[i].z + vb[i].w);
        }
        for (int c = lane + 32 * HOLD; c < quads; c += 32) {
            float4 y = xa[c]; sum_a += (y.x + y.y) + (y.z + y.w);
            float4 z = xb[c]; sum_b += (z.x + z.y) + (z.z + z.w);
        }
        sum_a = warp_sum(sum_a);
        sum_b = warp_sum(sum_b);
        const float mean_a = in.has_mean ? sum_a * inv_k : 0.f;
        const float mean_b = in.has_mean ? sum_b * inv_k : 0.f;
        float sq_a = 0.f, sq_b = 0.f;
#pragma unroll
        for (int i = 0; i < HOLD; ++i) {
            if (lane + 32 * i < quads) {
                float a = va[i].x - mean_a, b = va[i].y - mean_a, c = va[i].z - mean_a, d = va[i].w - mean_a;
                sq_a += (a * a + b * b) + (c * c + d * d);
                a = vb[i].x - mean_b, b = vb[i].y - mean_b, c = vb[i].z - mean_b, d = vb[i].w - mean_b;
                sq_b += (a * a + b * b) + (c * c + d * d);
            }
        }
        for (int c = lane + 32 * HOLD; c < quads; c += 32) {
            float4 y = xa[c];
            float a = y.x - mean_a, b = y.y - mean_a, cc = y.z - mean_a, d = y.w - mean_a;
            sq_a += (a * a + b * b) + (cc * cc + d * d);
            y = xb[c];
            a = y.x - mean_b, b = y.y - mean_b, cc = y.z - mean_b, d = y.w - mean_b;
            sq_b += (a * a + b * b) + (cc * cc + d * d);
        }
        sq_a = warp_sum(sq_a);
        sq_b = warp_sum(sq_b);
        const float rstd_a = rsqrtf(sq_a * inv_k + in.eps);
        const float rstd_b = rsqrtf(sq_b * inv_k + in.eps);
        if (!staged) {         // every warp passes one such barrier: here, or below if it has no row
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
            staged = true;
        }
        auto put = [&](int m, int c, const float4& y, float mean, float rstd) {
            const float4 gm = reinterpret_cast<const float4*>(gamma_s)[c];
            const float4 bt = reinterpret_cast<const float4*>(beta_s)[c];
            __nv_bfloat162 lo = __floats2bfloat162_rn((y.x - mean) * rstd * gm.x + bt.x, (y.y - mean) * rstd * gm.y + bt.y);
            __nv_bfloat162 hi = __floats2bfloat162_rn((y.z - mean) * rstd * gm.z + bt.z, (y.w - mean) * rstd * gm.w + bt.w);
            *reinterpret_cast<uint2*>(a_s + (size_t)m * lda_s + 4 * c) =
                make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        };
#pragma unroll
        for (int i = 0; i < HOLD; ++i) {
            const int c = lane + 32 * i;
            if (c < quads) {
                put(m0, c, va[i], mean_a, rstd_a);
                if (two) put(m1, c, vb[i], mean_b, rstd_b);
            }
        }
        for (int c = lane + 32 * HOLD; c < quads; c += 32) {
            put(m0, c, xa[c], mean_a, rstd_a);
            if (two) put(m1, c, xb[c], mean_b, rstd_b);
        }
    }
    if (!staged) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
    }
    // where this row's keys and values go: offset of (page, head 0, position in page, 0), or -1
    if (kv_row)
        dst_s[threadIdx.x] = kv_page >= 0 ? (long long)kv_page * kv.page_stride + (long long)kv_within * kv.head_dim : -1;
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
            if ((s0 + u * WARPS) >= steps) continue;       // the same for the whole warp: the MMAs stay converged
            const bool in_k = (k + 8 * t) < K;             // a lane past the end of K feeds zeros
            uint32_t a1[4] = {wa[u].x, wb[u].x, wa[u].y, wb[u].y};
            uint32_t a2[4] = {wa[u].z, wb[u].z, wa[u].w, wb[u].w};
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint4 x = (in_k && aok[mt]) ? *reinterpret_cast<const uint4*>(arow[mt] + k) : make_uint4(0, 0, 0, 0);
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
        v += bias_mine;
        v = apply_act(v, act);
        if (kv_col.which) {
            const long long base = dst_s[m];
            if (base >= 0) (kv_col.which == 1 ? kv.k_pool : kv.v_pool)[base + kv_col.offset] = __float2bfloat16_rn(v);
            continue;
        }
        size_t o = (size_t)m * ldo + n;
        if (accumulate) v += to_float(out[o]);
        out[o] = from_float<TOut>(v);
    }
}

// Shared memory of the fused kernel for MT token tiles, WARPS warps and width K.
inline size_t skinny_fused_smem(int MT, int WARPS, int K) {
    return (size_t)WARPS * 16 * 8 * MT * sizeof(float) + (size_t)2 * K * sizeof(float) + (size_t)8 * MT * 8 +
           (size_t)8 * MT * (K + 8) * 2;
}

template <int MT, int WARPS, int UNROLL, typename TOut>
int launch_skinny_fused(const NormInput& in, const void* W, int ldw, const float* bias, void* out, int ldo, int M,
                        int N, int K, int act, int accumulate, const KvScatter& kv, cudaStream_t s) {
    size_t smem = skinny_fused_smem(MT, WARPS, K);
    auto kernel = gemm_skinny_fused_kernel<MT, WARPS, UNROLL, TOut>;
    if (smem > 200 * 1024) return PS_ERR_UNSUPPORTED;
    static size_t raised[MAX_DEVICES] = {0};
    if (!ensure_dynamic_smem((const void*)kernel, smem, raised)) return PS_ERR_LAUNCH;
    return launch_pdl(kernel, dim3((N + 15) / 16), dim3(WARPS * 32), smem, s, in, (const __nv_bfloat16*)W, ldw, bias,
                      (TOut*)out, ldo, M, N, K, act, accumulate, kv);
}

template <int MT, typename TOut>
int pick_warps_fused(const NormInput& in, const void* W, int ldw, const float* bias, void* out, int ldo, int M, int N,
                     int K, int act, int accumulate, const KvScatter& kv, cudaStream_t s) {
    // at least 8 warps: they also share the rows of the norm between them
    // UNROLL: the k steps of a warp whose weights are fetched before anything else
    int steps = (K + 31) / 32;
    if (steps <= 24) return launch_skinny_fused<MT, 8, 3, TOut>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
    if (steps <= 64) return launch_skinny_fused<MT, 8, 6, TOut>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
    return launch_skinny_fused<MT, 16, 6, TOut>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
}

template <typename TOut>
int pick_tiles_fused(const NormInput& in, const void* W, int ldw, const float* bias, void* out, int ldo, int M, int N,
                     int K, int act, int accumulate, const KvScatter& kv, cudaStream_t s) {
    if (M <= 8) return pick_warps_fused<1, TOut>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
    if (M <= 16) return pick_warps_fused<2, TOut>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
    return pick_warps_fused<4, TOut>(in, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
}


}  // namespace ps

// An optional cache write of the key and value columns rides on the epilogue (kv_* arguments as for
// ps_gemm_skinny_fused; k_pool null = none).
PS_EXPORT int ps_gemm_skinny(const void* A, int lda, const void* W, int ldw, const float* bias, void* out,
                             int ldo, int M, int N, int K, int out_dtype, int act, int accumulate,
                             void* k_pool, void* v_pool, long long page_stride, const int* token_item,
                             const int* positions, const int* block_table, int bt_stride, int q_width,
                             int kv_width, int head_dim, int page_size, void* stream) {
    if (M <= 0 || N <= 0) return PS_OK;
    if (M > 64) return PS_ERR_UNSUPPORTED;
    if (K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || lda < K || ldw < K || ldo < N)
        return PS_ERR_UNSUPPORTED;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return PS_ERR_UNSUPPORTED;
    if (accumulate && out_dtype != PS_F32) return PS_ERR_BAD_ARGUMENT;
    if (k_pool && (q_width + 2 * kv_width != N || head_dim <= 0 || kv_width % head_dim != 0 || page_size <= 0))
        return PS_ERR_BAD_ARGUMENT;
    ps::KvScatter kv{(__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, page_stride, token_item, positions, block_table,
                     bt_stride, q_width, kv_width, head_dim, page_size};
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == PS_F32)
        return ps::pick_tiles<float>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
    if (out_dtype == PS_BF16)
        return ps::pick_tiles<__nv_bfloat16>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, kv, s);
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
