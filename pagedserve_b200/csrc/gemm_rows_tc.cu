// Tensor-core GEMM for few rows (17 to 64 tokens of a decode step): out[M, N] = epilogue(A[M,K] W[N,K]^T + bias).
//
// With a few dozen rows the product is a stream of weights: every byte of W is read once and used for M
// tokens. The operands are therefore swapped: 128 consecutive WEIGHT rows are the 128-row side of
// tcgen05.mma (M = 128), the tokens are its narrow side (N = 16, 32, 48 or 64), and the accumulator in
// tensor memory is the transposed output tile, one output column per TMEM lane.
//
//   grid (column tiles of 128, 1, S); the S CTAs of a column tile are one thread-block cluster and split K:
//   CTA `rank` takes the 64-wide k-blocks [rank * kb / S, (rank + 1) * kb / S), so that a product with few
//   output columns (the 768 of a model's width) still has its weights streamed by many SMs.
//   TMA (128-byte swizzle, no multicast) brings the CTA's weight tiles, all of them in flight at once where
//   they fit (those of the first stages before the wait on the kernel before: weights are static), and the
//   token rows [NT, 64] of each k-block; one thread issues the MMAs; the 128 threads read the accumulator
//   (thread = output column) and park it in shared memory as partial[token][column].
//   After a cluster barrier, CTA `rank` finishes columns [rank * 128 / S, (rank + 1) * 128 / S) of the tile:
//   it adds the S partial sums of each element in rank order out of the CTAs' shared memory (distributed
//   shared memory: no scratch in global memory, no atomics, one fixed order), then bias, GELU, and stores
//   bfloat16 / float32, accumulates into the float32 residual stream, or sends key and value columns of a
//   packed q|k|v projection into the pages.
//
// The split depends on N and K only, never on M: a row's result does not depend on the rows beside it.
// Every mbarrier wait is bounded; a CTA that gives up still takes part in both cluster barriers (its
// partial sums are zero and *status says so), frees its tensor memory and returns.
//
// Replaces the cuBLAS nn.Linear calls of the reference in decode (src/model/paged_decoder.py:49-50, 178-179,
// 295-299) with bias (:52), GELU (:273-280) and residual add (:184, :188) in the epilogue.
#include <cuda.h>

#include "common.cuh"

namespace ps {
namespace rows {

constexpr int TILE_N = 128;            // weight rows (output columns) per CTA = the M of the MMA
constexpr int BK = 64;                 // bf16 elements per k-block = one 128-byte swizzle row
constexpr int THREADS = 128;
constexpr int MAX_STAGES = 8;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
constexpr uint64_t WAIT_LIMIT_NS = 200ull * 1000 * 1000;      // 0.2 s: far beyond any legitimate wait here
// false: the wait ran out, or another thread of this CTA gave up (abort flag set)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = global_timer_ns();
    while (true) {
#pragma unroll 1
        for (int spin = 0; spin < 64; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - start > WAIT_LIMIT_NS) { *abort_flag = 1; return false; }
    }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t desc = (uint64_t)((smem_addr >> 4) & 0x3FFF);
    desc |= (uint64_t)1 << 16;                     // leading byte offset (unused with swizzle), 16-byte units
    desc |= (uint64_t)(1024 >> 4) << 32;           // stride byte offset between 8-row groups
    desc |= (uint64_t)1 << 46;                     // descriptor version of sm_100
    desc |= (uint64_t)2 << 61;                     // SWIZZLE_128B
    return desc;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ float gelu_tanh_fast(float x) {       // tanh.approx: exact enough before a bf16 rounding
    float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x), th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(inner));
    return 0.5f * x * (1.0f + th);
}

template <int NT> struct Config {
    static constexpr int W_BYTES = TILE_N * BK * 2;                  // 16 KB
    static constexpr int A_BYTES = NT * BK * 2;
    static constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
    static constexpr int TMEM_COLS = NT <= 32 ? 32 : 64;
    static constexpr int PARTIAL_BYTES = NT * TILE_N * 4;            // partial[token][column], float32
    static size_t smem(int stages) { return (size_t)stages * STAGE_BYTES + PARTIAL_BYTES + 1024 + 256; }
};

// NT: token rows of the MMA (a multiple of 16 that covers M). splits: CTAs per cluster (1 = no cluster).
template <int NT, typename TOut>
__global__ void __launch_bounds__(THREADS)
gemm_rows_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                 const float* __restrict__ bias, TOut* __restrict__ out, int ldo, int M, int N, int K, int act,
                 int accumulate, int* __restrict__ status, KvScatter kv, int splits, int stages) {
    using Cfg = Config<NT>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* partial = reinterpret_cast<float*>(tiles + (size_t)stages * Cfg::STAGE_BYTES);     // [NT][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(partial) + Cfg::PARTIAL_BYTES);
    uint64_t* full = bars;                       // [MAX_STAGES]  TMA -> MMA
    uint64_t* empty = bars + MAX_STAGES;         // [MAX_STAGES]  MMA -> TMA
    uint64_t* acc_full = bars + 2 * MAX_STAGES;  // MMA -> everybody: the accumulator is complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = splits > 1 ? (int)cluster_rank() : 0;
    const int n0 = blockIdx.x * TILE_N;
    const int num_kb = (K + BK - 1) / BK;
    const int kb0 = (int)((long long)rank * num_kb / splits), kb1 = (int)((long long)(rank + 1) * num_kb / splits);
    const int my_kb = kb1 - kb0;

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        *abort_flag = 0;
        for (int s = 0; s < MAX_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------ TMA producer
        // weights do not depend on the kernel before this one: the first stages' tiles go out before the wait
        const int early = min(stages, my_kb);
        for (int it = 0; it < early; ++it) {
            mbar_expect_tx(&full[it], Cfg::STAGE_BYTES);
            tma_load_2d(tiles + (size_t)it * Cfg::STAGE_BYTES, &map_w, (kb0 + it) * BK, n0, &full[it]);
        }
        pdl_prologue();
        for (int it = 0; it < my_kb; ++it) {
            const int s = it % stages;
            unsigned char* stage = tiles + (size_t)s * Cfg::STAGE_BYTES;
            if (it >= early) {
                if (!mbar_wait(&empty[s], ((it / stages) & 1) ^ 1, abort_flag)) { atomicExch(status, 21); break; }
                mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
                tma_load_2d(stage, &map_w, (kb0 + it) * BK, n0, &full[s]);
            }
            tma_load_2d(stage + Cfg::W_BYTES, &map_a, (kb0 + it) * BK, 0, &full[s]);
        }
    } else {
        pdl_prologue();
    }
    if (warp == 1 && lane == 0) {
        // ------------------------------------------------ MMA issuer
        // instruction descriptor: D = f32, A = B = bf16, both K-major, N = NT tokens, M = 128 weight rows
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) |
                                   ((uint32_t)(TILE_N >> 4) << 24);
        bool ok = true;
        for (int it = 0; it < my_kb; ++it) {
            const int s = it % stages;
            if (!mbar_wait(&full[s], (it / stages) & 1, abort_flag)) { ok = false; atomicExch(status, 22); break; }
            tc_fence_after();
            const uint32_t w_addr = smem_u32(tiles + (size_t)s * Cfg::STAGE_BYTES);
            const uint64_t desc_w = umma_desc(w_addr), desc_a = umma_desc(w_addr + Cfg::W_BYTES);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)          // 16 bf16 = 32 bytes = 2 units of the address field
                umma_bf16(tmem_base, desc_w + 2 * k, desc_a + 2 * k, idesc, (it | k) ? 1u : 0u);
            umma_commit(&empty[s]);                     // stage free once these MMAs have read it
        }
        if (ok && my_kb > 0) umma_commit(acc_full);
        else mbar_arrive(acc_full);                     // nothing to wait for (no k-block here, or gave up)
    }
    // ------------------------------------------------ everybody: the epilogue's constants, fetched while the weights arrive
    // a thread finishes 4 consecutive columns of one token at a time: the S partial sums of the four come as
    // S independent 16-byte loads (all in flight together), added in rank order
    const int share = TILE_N / splits;                            // splits is 1, 2, 4 or 8: 128 .. 16 columns
    const int groups = share >> 2;                                // groups of 4 columns in the share
    const int c4 = (threadIdx.x % groups) * 4, first_token = threadIdx.x / groups, token_step = THREADS / groups;
    const int column = rank * share + c4;
    const int n = n0 + column;
    float b[4] = {0.f, 0.f, 0.f, 0.f};
    if (bias) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (n + j < N) b[j] = bias[n + j];
    }
    // where key / value columns go: which pool, head and offset inside the head (a group of 4 lies in one
    // head: head sizes and the query width are multiples of 4 here, else the scalar path below is taken)
    const bool whole = n + 3 < N;
    bool to_pages = false;
    __nv_bfloat16* pool = nullptr;
    long long head_offset = 0;
    if (kv.k_pool && n >= kv.q_width && n < N) {
        to_pages = true;
        int idx = n - kv.q_width;
        pool = kv.k_pool;
        if (idx >= kv.kv_width) { idx -= kv.kv_width; pool = kv.v_pool; }
        const int head = idx / kv.head_dim;
        head_offset = (long long)head * kv.page_size * kv.head_dim + (idx - head * kv.head_dim);
    }
    const bool kv_vector = to_pages && whole && (kv.head_dim & 3) == 0 && (kv.q_width & 3) == 0 &&
                           (kv.kv_width & 3) == 0 && (kv.page_stride & 3) == 0;
    const bool out_vector = whole && (ldo & 3) == 0 && (((uintptr_t)out) & 15) == 0;
    // ------------------------------------------------ everybody: accumulator -> partial[token][column]
    bool have = my_kb > 0;
    if (!mbar_wait(acc_full, 0, abort_flag)) {
        have = false;
        if (lane == 0) atomicExch(status, 23);
    }
    if (*abort_flag) have = false;
    have = __all_sync(0xffffffffu, have);                               // the TMEM load below is warp-wide
    tc_fence_after();
    {
        const int column = warp * 32 + lane;                          // TMEM lane = column of the tile
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll
        for (int c = 0; c < NT; c += 16) {
            uint32_t r[16];
            if (have) {                                               // uniform per CTA
                tmem_ld16(taddr + c, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) partial[(c + j) * TILE_N + column] = __uint_as_float(r[j]);
        }
    }
    tc_fence_before();
    if (splits > 1) cluster_sync_all(); else __syncthreads();
    // ------------------------------------------------ this CTA's share of the tile's columns, all tokens
    {
        for (int t = first_token; t < M; t += token_step) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            const float* mine = &partial[t * TILE_N + column];
            if (splits > 1) {
                float4 part[8];
#pragma unroll
                for (int r = 0; r < 8; ++r)
                    if (r < splits) part[r] = ld_cluster_f32x4(mine, r);
#pragma unroll
                for (int r = 0; r < 8; ++r)
                    if (r < splits) { v[0] += part[r].x; v[1] += part[r].y; v[2] += part[r].z; v[3] += part[r].w; }
            } else {
                const float4 own = *reinterpret_cast<const float4*>(mine);
                v[0] = own.x; v[1] = own.y; v[2] = own.z; v[3] = own.w;
            }
            if (n >= N) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[j] += b[j];
                if (act == PS_ACT_GELU_TANH) v[j] = sizeof(TOut) == 2 ? gelu_tanh_fast(v[j]) : gelu_tanh(v[j]);
                else if (act == PS_ACT_GELU_ERF) v[j] = gelu_erf(v[j]);
            }
            if (to_pages) {
                const int p = kv.positions[t];
                const int page = kv.block_table[(size_t)kv.token_row[t] * kv.bt_stride + p / kv.page_size];
                if (page < 0) continue;
                __nv_bfloat16* dst = pool + (long long)page * kv.page_stride +
                                     (long long)(p % kv.page_size) * kv.head_dim + head_offset;
                if (kv_vector) {
                    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
                    uint2 pack;
                    pack.x = *reinterpret_cast<uint32_t*>(&lo);
                    pack.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(dst) = pack;
                } else {
                    // columns of the group may lie in different heads or pools: one at a time
                    for (int j = 0; j < 4 && n + j < N; ++j) {
                        int idx = n + j - kv.q_width;
                        __nv_bfloat16* pl = kv.k_pool;
                        if (idx >= kv.kv_width) { idx -= kv.kv_width; pl = kv.v_pool; }
                        const int head = idx / kv.head_dim;
                        pl[(long long)page * kv.page_stride + (long long)(p % kv.page_size) * kv.head_dim +
                           (long long)head * kv.page_size * kv.head_dim + (idx - head * kv.head_dim)] =
                            __float2bfloat16_rn(v[j]);
                    }
                }
                continue;
            }
            TOut* dst = out + (size_t)t * ldo + n;
            if (out_vector) {
                if constexpr (sizeof(TOut) == 4) {
                    float4 o = make_float4(v[0], v[1], v[2], v[3]);
                    if (accumulate) {
                        const float4 old = *reinterpret_cast<const float4*>(dst);
                        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                    }
                    *reinterpret_cast<float4*>(dst) = o;
                } else {
                    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
                    uint2 pack;
                    pack.x = *reinterpret_cast<uint32_t*>(&lo);
                    pack.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(dst) = pack;
                }
            } else {
                for (int j = 0; j < 4 && n + j < N; ++j) {
                    float x = v[j];
                    if (accumulate) x += to_float(dst[j]);
                    dst[j] = from_float<TOut>(x);
                }
            }
        }
    }
    if (splits > 1) cluster_sync_all(); else __syncthreads();        // nobody leaves while its partial sums are read
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// A row-major [rows, K] bf16 matrix with leading dimension ld; boxes of box_rows x 64 elements, 128-byte
// swizzle; what lies outside the matrix reads as zero.
static bool make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// CTAs per column tile: as many as keep the grid within one wave of 148 SMs, at most 8 (a portable
// cluster) and at most one per k-block. A function of N and K alone.
static int pick_splits(int N, int K) {
    const int tiles = (N + TILE_N - 1) / TILE_N, num_kb = (K + BK - 1) / BK;
    int splits = 1;
    while (splits < 8 && tiles * splits * 2 <= 148 && splits * 2 <= num_kb) splits *= 2;
    return splits;
}

template <int NT, typename TOut>
int launch(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo, int M, int N, int K,
           int act, int accumulate, int* status, const KvScatter& kv, int splits, cudaStream_t stream) {
    CUtensorMap map_w, map_a;
    if (!make_map(&map_w, W, N, K, ldw, TILE_N) || !make_map(&map_a, A, M, K, lda, NT)) return PS_ERR_LAUNCH;
    const int num_kb = (K + BK - 1) / BK;
    const int per_cta = (num_kb + splits - 1) / splits;
    // all of a CTA's k-blocks in flight at once where they fit; two CTAs per SM when that leaves room
    int stages = per_cta < MAX_STAGES ? per_cta : MAX_STAGES;
    if (stages < 1) stages = 1;
    const size_t smem = Config<NT>::smem(stages);
    auto kernel = gemm_rows_kernel<NT, TOut>;
    static size_t raised[MAX_DEVICES] = {0};
    if (!ensure_dynamic_smem((const void*)kernel, smem, raised)) return PS_ERR_LAUNCH;
    const int tiles = (N + TILE_N - 1) / TILE_N;
    return launch_pdl_cluster(kernel, dim3(tiles, 1, splits), dim3(THREADS), smem, stream, splits, map_w, map_a, bias,
                              (TOut*)out, ldo, M, N, K, act, accumulate, status, kv, splits, stages);
}

template <typename TOut>
int pick(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo, int M, int N, int K,
         int act, int accumulate, int* status, const KvScatter& kv, int splits, cudaStream_t stream) {
    if (M <= 16) return launch<16, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, kv, splits, stream);
    if (M <= 32) return launch<32, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, kv, splits, stream);
    if (M <= 48) return launch<48, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, kv, splits, stream);
    return launch<64, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, kv, splits, stream);
}

}  // namespace rows
}  // namespace ps

// M <= 64 rows. status: device int32 that a bounded wait sets when it runs out (must not be null).
// splits: 0 = choose from N and K, else 1, 2, 4 or 8 CTAs per column tile (for measurements).
// The last eleven arguments describe the cache write of a packed q|k|v projection (k_pool null: none):
// columns [0, q_width) go to `out`, then kv_width key and kv_width value columns go into the pages.
PS_EXPORT int ps_gemm_rows_tc(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo,
                              int M, int N, int K, int out_dtype, int act, int accumulate, int* status, int splits,
                              void* k_pool, void* v_pool, long long page_stride, const int* token_row,
                              const int* positions, const int* block_table, int bt_stride, int q_width,
                              int kv_width, int head_dim, int page_size, void* stream) {
    if (M <= 0 || N <= 0) return PS_OK;
    if (!status || M > 64) return PS_ERR_BAD_ARGUMENT;
    // TMA: 16-byte aligned base, row stride a multiple of 16 bytes
    if (K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || lda < K || ldw < K || ldo < N)
        return PS_ERR_UNSUPPORTED;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return PS_ERR_UNSUPPORTED;
    if (accumulate && out_dtype != PS_F32) return PS_ERR_BAD_ARGUMENT;
    if (splits == 0) splits = ps::rows::pick_splits(N, K);
    if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return PS_ERR_BAD_ARGUMENT;
    ps::KvScatter kv = {};
    if (k_pool) {
        if (!v_pool || !token_row || !positions || !block_table) return PS_ERR_BAD_ARGUMENT;
        // (the epilogue works on groups of 4 columns; a group must not straddle queries, keys and values)
        if (q_width + 2 * kv_width != N || head_dim <= 0 || kv_width % head_dim != 0 || page_size <= 0 ||
            out_dtype != PS_BF16 || q_width % 4 != 0 || kv_width % 4 != 0)
            return PS_ERR_UNSUPPORTED;
        kv = ps::KvScatter{(__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, page_stride, token_row, positions,
                           block_table, bt_stride, q_width, kv_width, head_dim, page_size};
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == PS_F32)
        return ps::rows::pick<float>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, kv, splits, s);
    if (out_dtype == PS_BF16)
        return ps::rows::pick<__nv_bfloat16>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, kv,
                                             splits, s);
    return PS_ERR_UNSUPPORTED;
}
