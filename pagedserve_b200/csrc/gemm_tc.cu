// Tensor-core GEMM for sm_100a: out[M,N] = epilogue(A[M,K] W[N,K]^T + bias), bfloat16 in, float32 accumulate.
//
//   TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast)  ->  shared memory ring of STAGES k-blocks
//   tcgen05.mma.cta_group::1.kind::f16 (M=128, N=BN, K=16), issued by one thread, accumulating in TMEM
//   tcgen05.ld 32x32b -> registers -> bias / GELU / residual-accumulate epilogue -> global memory
//
// The kernel is persistent: one CTA per SM walks the output tiles (n fastest, so neighbouring CTAs share
// the same rows of A in L2). TMEM holds two accumulators of BN columns; while the four epilogue warps
// drain one, the MMA warp fills the other.
//   warp 0: TMA producer (one lane)          warp 1: TMEM allocation + MMA issue (one lane)
//   warps 2..9: epilogue in two teams of four; warp w owns TMEM lanes 32*(w%4) .. +31 (= rows of the tile),
//               team (w-2)/4 takes every other 128-byte column group of the accumulator
// A k-block is 64 bf16 = one 128-byte swizzle row; the K loop of an output element runs in one fixed
// order whatever M is, so a row's result does not depend on the rows beside it.
// Output: the epilogue warps stage 128 rows x 128 bytes of results in shared memory (swizzled, so that a
// warp's 16-byte writes fall on different banks) and one thread hands them to TMA: a plain tensor store for
// bfloat16 / float32 results, or a reducing store (cp.reduce.async.bulk.tensor ... .add) when the product is
// accumulated into the float32 residual stream - the add happens in L2 and the SM never reads the stream.
// Outputs whose row pitch is not a multiple of 16 bytes (a vocabulary of 50257) are stored from registers.
// Every mbarrier wait is bounded: when one runs out the CTA sets *status, stops, frees its TMEM and returns.
//
// Replaces the cuBLAS nn.Linear calls of the reference (src/model/paged_decoder.py:49-50, 178-179, 295-299)
// with their bias add, GELU (:273-280) and residual add (:184, :188) fused into the epilogue.
#include <cuda.h>

#include "common.cuh"

namespace ps {
namespace tc {

constexpr int BM = 128;
constexpr int BK = 64;                 // bf16 elements per k-block = 128 bytes
constexpr int THREADS = 320;           // TMA warp, MMA warp, two teams of four epilogue warps

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
// false: the wait ran out, or another role of this CTA gave up (abort flag set)
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
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void team_sync(int team) {             // the 128 threads of one epilogue team
    asm volatile("bar.sync %0, 128;" ::"r"(team + 1) : "memory");
}
__device__ __forceinline__ float gelu_tanh_fast(float x) {       // tanh.approx: exact enough before a bf16 rounding
    float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x), th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(inner));
    return 0.5f * x * (1.0f + th);
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

template <int BN> struct Config {
    static constexpr int STAGE_BYTES = BM * BK * 2 + BN * BK * 2;
    static constexpr int STAGES = BN > 128 ? 4 : (BN >= 96 ? 5 : 6);
    // two accumulators of BN columns; an allocation is a power of two of at least 32 columns
    static constexpr int TMEM_COLS = 2 * BN <= 32 ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));
    // Results on their way out: buffers of 128 rows x 128 bytes, STAGING_BUFS for each of the two epilogue teams,
    // so that a team fills one while TMA still reads the one before (256-wide tiles have no room for that)
    static constexpr int STAGING_BUFS = BN == 256 ? 1 : 2;
    static constexpr int STAGING_BYTES = 2 * STAGING_BUFS * BM * 128;
    // column groups (128 bytes of output per row) that one of the two epilogue teams takes, at most: 32-column
    // groups of float32 results (the narrower kind), every other one; and 32-column reads per group, at most
    static constexpr int GROUPS_PER_TEAM = (BN / 32 + 1) / 2;
    static constexpr int HALVES_MAX = 2;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + STAGING_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
};

template <int BN, typename TOut, bool TMA_OUT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_out, const float* __restrict__ bias, TOut* __restrict__ out,
               int ldo, int M, int N, int K, int act, int accumulate, int* __restrict__ status, KvScatter kv) {
    using Cfg = Config<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* staging = tiles + (size_t)STAGES * Cfg::STAGE_BYTES;              // [2][128 rows][128 bytes]
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + Cfg::STAGING_BYTES);
    uint64_t* full = bars;                     // [STAGES]  TMA -> MMA
    uint64_t* empty = bars + STAGES;           // [STAGES]  MMA -> TMA
    uint64_t* acc_full = bars + 2 * STAGES;    // [2]       MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;        // [2]       epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    // Set-up (barriers, tensor memory) and the first weight tiles do not depend on the kernel before this one:
    // they happen before the wait and overlap its end.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (N + BN - 1) / BN, tiles_m = (M + BM - 1) / BM;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 256); }
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

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            // the weight tiles of the first stages (of this CTA's first tile) go out before the wait
            const uint32_t early = ((int)blockIdx.x < num_tiles) ? (uint32_t)min(STAGES, num_kb) : 0u;
            for (uint32_t kb = 0; kb < early; ++kb) {
                const int n0 = ((int)blockIdx.x % tiles_n) * BN;
                mbar_expect_tx(&full[kb], Cfg::STAGE_BYTES);
                tma_load_2d(tiles + (size_t)kb * Cfg::STAGE_BYTES + BM * BK * 2, &map_w, (int)kb * BK, n0, &full[kb]);
            }
            pdl_prologue();
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    unsigned char* a_dst = tiles + (size_t)s * Cfg::STAGE_BYTES;
                    if (it >= early) {
                        if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { ok = false; atomicExch(status, 11); break; }
                        mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
                        tma_load_2d(a_dst + BM * BK * 2, &map_w, kb * BK, n0, &full[s]);
                    }
                    tma_load_2d(a_dst, &map_a, kb * BK, m0, &full[s]);
                }
            }
        } else {
            pdl_prologue();
        }
    } else if (warp == 1) {
        pdl_prologue();
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            // instruction descriptor: D = f32, A = B = bf16, both K-major, N = BN, M = 128
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                       ((uint32_t)(BM >> 4) << 24);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                if (!mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, abort_flag)) { ok = false; atomicExch(status, 12); break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full[s], (it / STAGES) & 1, abort_flag)) { ok = false; atomicExch(status, 13); break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + (size_t)s * Cfg::STAGE_BYTES);
                    const uint64_t desc_a = umma_desc(a_addr), desc_b = umma_desc(a_addr + BM * BK * 2);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)      // 16 bf16 = 32 bytes = 2 units of the address field
                        umma_bf16(tmem_d, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb | k) ? 1u : 0u);
                    umma_commit(&empty[s]);                 // stage free once these MMAs have read it
                }
                if (ok) umma_commit(&acc_full[buf]);        // accumulator complete
            }
        }
    } else {
        // ------------------------------------------------ epilogue: warps 2..9
        pdl_prologue();
        const int quarter = warp & 3;                       // TMEM lanes 32*quarter .. +31
        const int team = (warp - 2) >> 2;                   // which column groups this warp takes
        uint32_t local = 0;
        [[maybe_unused]] uint32_t chunk = 0;                // column groups this team has sent out so far
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            const int buf = local & 1;
            // a q|k|v product whose key and value columns go straight into the pages: where this row's go
            // (offset of page, head 0, position in page, 0), looked up while the tile is still being computed
            long long kv_base = -1;
            if constexpr (TMA_OUT && sizeof(TOut) == 2) {
                const int row = m0 + quarter * 32 + lane;
                if (kv.k_pool && row < M && n0 + BN > kv.q_width) {
                    const int p = kv.positions[row];
                    const int page = kv.block_table[(size_t)kv.token_row[row] * kv.bt_stride + p / kv.page_size];
                    if (page >= 0) kv_base = (long long)page * kv.page_stride + (long long)(p % kv.page_size) * kv.head_dim;
                }
            }
            // The bias of this team's column groups, fetched while the tile is still being computed: lane j
            // holds the values of columns j, 32 + j, ... of each group and hands them out by shuffle below (a
            // first touch of these lines after the accumulator is complete costs about a microsecond per group).
            [[maybe_unused]] float bias_lane[TMA_OUT ? Cfg::GROUPS_PER_TEAM * Cfg::HALVES_MAX : 1];
            if constexpr (TMA_OUT) {
                constexpr int COLS = 128 / (int)sizeof(TOut);
#pragma unroll
                for (int g = 0; g < Cfg::GROUPS_PER_TEAM * (COLS / 32); ++g) {
                    const int n = n0 + (team + 2 * (g / (COLS / 32))) * COLS + 32 * (g % (COLS / 32)) + lane;
                    bias_lane[g] = (bias && n < N && (team + 2 * (g / (COLS / 32))) * COLS < BN) ? bias[n] : 0.f;
                }
            }
            if (!mbar_wait(&acc_full[buf], (local >> 1) & 1, abort_flag)) { ok = false; if (lane == 0) atomicExch(status, 14); break; }
            tc_fence_after();
            const int m = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN);
            if constexpr (TMA_OUT) {
                // columns per staged buffer: 128 bytes of output per row
                constexpr int COLS = 128 / (int)sizeof(TOut);
                const int r = quarter * 32 + lane;                        // row of the tile = row of the buffer
                const bool leader = (quarter == 2 && lane == 0);          // first warp of the team (warps 2 and 6)
                bool released = false;
#pragma unroll
                for (int group = 0; group < Cfg::GROUPS_PER_TEAM; ++group) {
                    const int c = (team + 2 * group) * COLS;
                    if (c >= BN) break;
                    unsigned char* stage_buf =
                        staging + (size_t)(team * Cfg::STAGING_BUFS + chunk % Cfg::STAGING_BUFS) * (BM * 128);
                    ++chunk;
                    // the buffer is free once TMA has read the group sent from it (one group per chunk)
                    if (leader) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(Cfg::STAGING_BUFS - 1) : "memory");
                    team_sync(team);
#pragma unroll
                    for (int half = 0; half < COLS / 32; ++half) {
                        uint32_t rr[32];
                        tmem_ld32(taddr + c + 32 * half, rr);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (c + 2 * COLS >= BN && half == COLS / 32 - 1) {   // this team's last read of the accumulator
                            tc_fence_before();
                            mbar_arrive(&acc_empty[buf]);
                            released = true;
                        }
                        const int n = n0 + c + 32 * half;
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(rr[j]);
                        if (bias) {
                            const float mine = bias_lane[group * (COLS / 32) + half];
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] += __shfl_sync(0xffffffffu, mine, j);
                        }
                        if (act == PS_ACT_GELU_TANH) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = sizeof(TOut) == 2 ? gelu_tanh_fast(v[j]) : gelu_tanh(v[j]);
                        } else if (act == PS_ACT_GELU_ERF) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
                        }
                        // 16-byte pieces of the row, XOR-swizzled by the row as the tensor map expects
                        if constexpr (sizeof(TOut) == 2) {
                            const bool to_pages = kv.k_pool && n >= kv.q_width;      // key / value columns
#pragma unroll
                            for (int piece = 0; piece < 4; ++piece) {
                                uint4 pack;
                                __nv_bfloat162 p0 = __floats2bfloat162_rn(v[8 * piece], v[8 * piece + 1]);
                                __nv_bfloat162 p1 = __floats2bfloat162_rn(v[8 * piece + 2], v[8 * piece + 3]);
                                __nv_bfloat162 p2 = __floats2bfloat162_rn(v[8 * piece + 4], v[8 * piece + 5]);
                                __nv_bfloat162 p3 = __floats2bfloat162_rn(v[8 * piece + 6], v[8 * piece + 7]);
                                pack.x = *reinterpret_cast<uint32_t*>(&p0); pack.y = *reinterpret_cast<uint32_t*>(&p1);
                                pack.z = *reinterpret_cast<uint32_t*>(&p2); pack.w = *reinterpret_cast<uint32_t*>(&p3);
                                if (to_pages) {
                                    // 8 columns of one head (head sizes are multiples of 16, pieces start on multiples of 8)
                                    int idx = n + 8 * piece - kv.q_width;
                                    __nv_bfloat16* pool = kv.k_pool;
                                    if (idx >= kv.kv_width) { idx -= kv.kv_width; pool = kv.v_pool; }
                                    const int head = idx / kv.head_dim, d = idx - head * kv.head_dim;
                                    if (kv_base >= 0 && n + 8 * piece < N)
                                        *reinterpret_cast<uint4*>(pool + kv_base + (long long)head * kv.page_size * kv.head_dim + d) = pack;
                                } else {
                                    const int slot = (4 * half + piece) ^ (r & 7);
                                    *reinterpret_cast<uint4*>(stage_buf + r * 128 + slot * 16) = pack;
                                }
                            }
                        } else {
#pragma unroll
                            for (int piece = 0; piece < 8; ++piece) {
                                const int slot = piece ^ (r & 7);
                                *reinterpret_cast<float4*>(stage_buf + r * 128 + slot * 16) =
                                    make_float4(v[4 * piece], v[4 * piece + 1], v[4 * piece + 2], v[4 * piece + 3]);
                            }
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    team_sync(team);
                    if (leader) {
                        // (key and value columns of a scattering q|k|v product were written by the rows themselves;
                        // the query width is a multiple of the 64-column group, so a group is all one or the other)
                        if (n0 + c < N && !(sizeof(TOut) == 2 && kv.k_pool && n0 + c >= kv.q_width)) {
                            if (accumulate) tma_reduce_add_2d(&map_out, stage_buf, n0 + c, m0);
                            else tma_store_2d(&map_out, stage_buf, n0 + c, m0);
                        }
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
                if (!released) {                                          // a team without a column group (BN < 2 groups)
                    tc_fence_before();
                    mbar_arrive(&acc_empty[buf]);
                }
                continue;
            }
            TOut* orow = out + (size_t)m * ldo;
#pragma unroll 1
            for (int c = 32 * team; c < BN; c += 64) {      // the two teams take alternate 32-column chunks
                uint32_t r[32];
                tmem_ld32(taddr + c, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c + 64 >= BN) {                          // this team's last read: hand TMEM back
                    tc_fence_before();
                    mbar_arrive(&acc_empty[buf]);
                }
                const int n = n0 + c;
                if (m < M && n < N) {
                    const bool full_chunk = n + 32 <= N;
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (bias) {
                        if (full_chunk && ((((uintptr_t)(bias + n)) & 15) == 0)) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 b4 = *reinterpret_cast<const float4*>(bias + n + j);
                                v[j] += b4.x; v[j + 1] += b4.y; v[j + 2] += b4.z; v[j + 3] += b4.w;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (n + j < N) v[j] += bias[n + j];
                        }
                    }
                    if (act != PS_ACT_NONE) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], act);
                    }
                    if constexpr (sizeof(TOut) == 2) {
                        if (full_chunk && ((((uintptr_t)(orow + n)) & 15) == 0)) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 pack;
                                __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]);
                                __nv_bfloat162 p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                                __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
                                __nv_bfloat162 p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                                pack.x = *reinterpret_cast<uint32_t*>(&p0);
                                pack.y = *reinterpret_cast<uint32_t*>(&p1);
                                pack.z = *reinterpret_cast<uint32_t*>(&p2);
                                pack.w = *reinterpret_cast<uint32_t*>(&p3);
                                *reinterpret_cast<uint4*>(orow + n + j) = pack;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (n + j < N) orow[n + j] = from_float<TOut>(v[j]);
                        }
                    } else {
                        if (full_chunk && ((((uintptr_t)(orow + n)) & 15) == 0)) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                float4* dst = reinterpret_cast<float4*>(orow + n + j);
                                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                                if (accumulate) {
                                    float4 old = *dst;
                                    o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                                }
                                *dst = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (n + j < N) {
                                    float x = v[j];
                                    if (accumulate) x += to_float(orow[n + j]);
                                    orow[n + j] = from_float<TOut>(x);
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    // shared memory must outlive TMA's reads of it; the writes themselves are complete when the grid is
    if (TMA_OUT && (warp == 2 || warp == 6) && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    tc_fence_before();
    __syncthreads();
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

// A row-major [rows, K] bf16 matrix with leading dimension ld; boxes of box_rows x 64 elements, 128-byte swizzle.
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

// The output [M, N] (row pitch ldo elements) in boxes of 128 rows x 128 bytes, 128-byte swizzle.
static bool make_out_map(CUtensorMap* map, void* base, int M, int N, int ldo, int elem_bytes) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)ldo * elem_bytes};
    cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)BM};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims,
              strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int sm_count() {
    static int count = 0;
    if (!count) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
        if (count <= 0) count = 1;
    }
    return count;
}

template <int BN, typename TOut, bool TMA_OUT>
int launch_kernel(const CUtensorMap& map_a, const CUtensorMap& map_w, const CUtensorMap& map_out, const float* bias,
                  void* out, int ldo, int M, int N, int K, int act, int accumulate, int* status, const KvScatter& kv,
                  cudaStream_t stream) {
    auto kernel = gemm_tc_kernel<BN, TOut, TMA_OUT>;
    static size_t raised[MAX_DEVICES] = {0};
    if (!ensure_dynamic_smem((const void*)kernel, (size_t)Config<BN>::SMEM, raised)) return PS_ERR_LAUNCH;
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    return launch_pdl(kernel, dim3(grid), dim3(THREADS), Config<BN>::SMEM, stream, map_a, map_w, map_out, bias,
                      (TOut*)out, ldo, M, N, K, act, accumulate, status, kv);
}

template <int BN, typename TOut>
int launch(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo, int M, int N, int K,
           int act, int accumulate, int* status, const KvScatter& kv, cudaStream_t stream) {
    CUtensorMap map_a, map_w, map_out;
    if (!make_map(&map_a, A, M, K, lda, BM) || !make_map(&map_w, W, N, K, ldw, BN)) return PS_ERR_LAUNCH;
    // TMA can write the output when its rows start on 16-byte boundaries
    const bool tma_out = (((uintptr_t)out & 15) == 0) && (((size_t)ldo * sizeof(TOut)) % 16 == 0) &&
                         make_out_map(&map_out, out, M, N, ldo, (int)sizeof(TOut));
    if (tma_out)
        return launch_kernel<BN, TOut, true>(map_a, map_w, map_out, bias, out, ldo, M, N, K, act, accumulate, status, kv, stream);
    if (kv.k_pool) return PS_ERR_UNSUPPORTED;      // the cache write lives in the TMA-store epilogue only
    map_out = map_a;    // unused
    return launch_kernel<BN, TOut, false>(map_a, map_w, map_out, bias, out, ldo, M, N, K, act, accumulate, status, kv, stream);
}

template <typename TOut>
int pick(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo, int M, int N, int K,
         int act, int accumulate, int* status, int bn, const KvScatter& kv, cudaStream_t stream) {
    if (bn == 0) {
        const int tiles_m = (M + BM - 1) / BM;
        // widest tile that still gives the SMs enough tiles (measured on B200: 128 wide wins until the
        // grid falls below half the SMs; 256 wide needs two full waves)
        const int t128 = tiles_m * ((N + 127) / 128), t96 = tiles_m * ((N + 95) / 96);
        const int t256 = tiles_m * ((N + 255) / 256);
        if (t256 >= 2 * sm_count()) bn = 256;
        // bfloat16 output whose 256-wide tiles are one wave while 128-wide ones would be two rounds per CTA: an
        // MMA of 128 x N x 16 takes about 130 clocks whatever N is, so one wide tile costs half of two narrow
        // ones (2,048 x 2,304 x 768: 12.4 -> 9.9 us inside a prefill step)
        else if (sizeof(TOut) == 2 && t256 <= sm_count() && t128 > sm_count()) bn = 256;
        // bfloat16 output of a deep product (K of 1,024 and more, where the main loop outweighs what a CTA does
        // once): rounds of tiles per CTA times what a tile of each width costs beside one of 128 (measured alone:
        // 1,024 x 4,800 x 1,600 takes 30.1 / 26.7 / 28.4 us at 128 / 192 / 256 columns, 2,048 x 3,072 x 1,024
        // 23.0 / 21.4 / 23.0, 2,048 x 4,096 x 1,024 28.9 / 28.4 / 23.9)
        else if (sizeof(TOut) == 2 && K >= 1024 && t128 > sm_count()) {
            const int t192 = tiles_m * ((N + 191) / 192);
            auto rounds = [&](int tiles) { return (tiles + sm_count() - 1) / sm_count(); };
            const int c128 = rounds(t128) * 100, c192 = rounds(t192) * 130, c256 = rounds(t256) * 145;
            bn = (c128 <= c192 && c128 <= c256) ? 128 : (c192 <= c256 ? 192 : 256);
        }
        // float32 output (the products that add into the residual stream, N = the model width): 96 wide when
        // that fills more of one wave (2,048 x 768: 128 CTAs instead of 96)
        else if (sizeof(TOut) == 4 && t128 < sm_count() && t96 <= sm_count() && t96 > t128 && 2 * t128 >= sm_count())
            bn = 96;
        else if (2 * t128 >= sm_count()) bn = 128;
        else bn = 64;
    }
    if (bn == 256) return launch<256, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, kv, stream);
    if (bn == 192) return launch<192, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, kv, stream);
    if (bn == 128) return launch<128, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, kv, stream);
    if constexpr (sizeof(TOut) == 4) {      // 96 columns are three 32-column groups of float32; bfloat16 groups are 64 wide
        if (bn == 96) return launch<96, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, kv, stream);
    }
    if (bn == 64) return launch<64, TOut>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, kv, stream);
    return PS_ERR_BAD_ARGUMENT;
}

}  // namespace tc
}  // namespace ps

// status: device int32 that a bounded wait sets when it runs out (must not be null).
// bn: 0 = choose, else 64, 96 (float32 output only), 128, 192 or 256 (the N extent of the MMA tile).
static int gemm_tc_entry(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo, int M,
                         int N, int K, int out_dtype, int act, int accumulate, int* status, int bn,
                         const ps::KvScatter& kv, void* stream) {
    if (M <= 0 || N <= 0) return PS_OK;
    if (!status) return PS_ERR_BAD_ARGUMENT;
    // TMA: 16-byte aligned base, row stride a multiple of 16 bytes
    if (K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || lda < K || ldw < K || ldo < N)
        return PS_ERR_UNSUPPORTED;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return PS_ERR_UNSUPPORTED;
    if (accumulate && out_dtype != PS_F32) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == PS_F32) {
        if (kv.k_pool) return PS_ERR_UNSUPPORTED;
        return ps::tc::pick<float>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, bn, kv, s);
    }
    if (out_dtype == PS_BF16)
        return ps::tc::pick<__nv_bfloat16>(A, lda, W, ldw, bias, out, ldo, M, N, K, act, accumulate, status, bn, kv, s);
    return PS_ERR_UNSUPPORTED;
}

PS_EXPORT int ps_gemm_tc(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo, int M,
                         int N, int K, int out_dtype, int act, int accumulate, int* status, int bn, void* stream) {
    ps::KvScatter none = {};
    return gemm_tc_entry(A, lda, W, ldw, bias, out, ldo, M, N, K, out_dtype, act, accumulate, status, bn, none, stream);
}

// The packed q|k|v projection of a step with prompt portions: columns [0, q_width) go to `out` (bfloat16), the
// key and value columns (kv_width each) go straight into the pages of each row's request. q_width must be a
// multiple of 64 and head_dim of 8; `out` rows must start on 16-byte boundaries.
PS_EXPORT int ps_gemm_tc_qkv(const void* A, int lda, const void* W, int ldw, const float* bias, void* out, int ldo,
                             int M, int N, int K, int* status, void* k_pool, void* v_pool, long long page_stride,
                             const int* token_item, const int* positions, const int* block_table, int bt_stride,
                             int q_width, int kv_width, int head_dim, int page_size, void* stream) {
    if (!k_pool || !v_pool || !token_item || !positions || !block_table) return PS_ERR_BAD_ARGUMENT;
    if (q_width + 2 * kv_width != N || q_width % 64 != 0 || head_dim <= 0 || head_dim % 8 != 0 ||
        kv_width % head_dim != 0 || page_size <= 0)
        return PS_ERR_UNSUPPORTED;
    ps::KvScatter kv{(__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, page_stride, token_item, positions, block_table,
                     bt_stride, q_width, kv_width, head_dim, page_size};
    return gemm_tc_entry(A, lda, W, ldw, bias, out, ldo, M, N, K, PS_BF16, PS_ACT_NONE, 0, status, 0, kv, stream);
}
