// Causal attention of prompt portions over the paged cache on tcgen05 tensor cores (bfloat16, head size 64 or 128).
//
// One CTA per (block of 128 query tokens of one request, head); key tiles of 128 keys aligned to absolute
// positions, read from the request's pages through the block table, so a portion that continues a cached
// prompt needs no gather (the reference gathers past K/V and materialises the scores:
// src/model/paged_attention.py:262-295, 396-420).
//   S = Q K^T   tcgen05.mma, A = Q tile and B = K tile in shared memory (K-major, 128-byte swizzle), S in TMEM
//   softmax     256 threads, two per query row (64 keys of the tile each; the two warps of a pair share a TMEM
//               lane quarter): tcgen05.ld of its half of the S row, scale, mask, maximum (exchanged with the
//               partner through shared memory), exp2 and sum in float32, P rounded to bfloat16 and written
//               back to TMEM (tcgen05.st). One thread per row was bound by the length of that thread's chain
//               (2 x 1,024 keys: 23.5 us with one thread per row)
//   O += P V    tcgen05.mma with A = P from TMEM and B = the V tile in shared memory (MN-major descriptor:
//               V rows are keys, the head dim is contiguous), accumulating in TMEM; when a tile raises a
//               row's running maximum the row's thread first rescales its O row in TMEM (skipped by a whole
//               warp when none of its 32 rows changed, which is the common case after the first tiles)
// TMA brings the Q tile from the step's q|k|v buffer and, page by page, the K and V tiles from the pool
// (one box of page_size x 64 per page; no multicast); two K/V stages.
//   warp 0: TMA producer      warp 1: TMEM allocation + MMA issue      warps 2..9: softmax rows / output
// mma.sync on this GPU gives about 1/15 of the tcgen05 rate (measured: 112 TFLOP/s at best for the mma.sync
// kernel in csrc/attention_prefill.cu), which is why prompt attention is here. Head sizes other than 64 and
// 128, or pages below 8 tokens, stay with that kernel.
// Every mbarrier wait is bounded; a wait that runs out sets *status and the CTA frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"

namespace ps {
namespace pftc {

constexpr int BQ = 128, BKEY = 128, KV_STAGES = 2;
constexpr uint64_t WAIT_LIMIT_NS = 200ull * 1000 * 1000;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = timer_ns();
    while (true) {
#pragma unroll 1
        for (int spin = 0; spin < 64; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (timer_ns() - start > WAIT_LIMIT_NS) { *abort_flag = 1; return false; }
    }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// shared-memory operand descriptors, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
    uint64_t desc = (uint64_t)((smem_addr >> 4) & 0x3FFF);
    desc |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    desc |= (uint64_t)(1024 >> 4) << 32;
    desc |= (uint64_t)1 << 46;
    desc |= (uint64_t)2 << 61;
    return desc;
}
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(acc) : "memory");
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ float ex2(float x) {                  // 2^x, hardware approximation, flushes denormals
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// four loads of 32 columns issued back to back, one wait: their latencies overlap
__device__ __forceinline__ void tmem_ld128(uint32_t taddr, uint32_t (&r)[128]) {
    tmem_ld32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
    tmem_ld32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
    tmem_ld32(taddr + 64, *reinterpret_cast<uint32_t(*)[32]>(&r[64]));
    tmem_ld32(taddr + 96, *reinterpret_cast<uint32_t(*)[32]>(&r[96]));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// COLS columns: loads of 32 issued back to back, one wait
template <int COLS>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[COLS]) {
#pragma unroll
    for (int c = 0; c < COLS; c += 32) tmem_ld32(taddr + c, *reinterpret_cast<uint32_t(*)[32]>(&r[c]));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The two threads of a row hand each other a float through shared memory: a slot holds (tag << 32 | bits),
// written with one 64-bit store; the reader polls until the tag is the one it expects. Polling is bounded like
// every other wait of the kernel (a plain barrier between the two warps could not be left on an abort).
__device__ __forceinline__ void slot_put(unsigned long long* slot, uint32_t tag, float value) {
    *reinterpret_cast<volatile unsigned long long*>(slot) = ((unsigned long long)tag << 32) | __float_as_uint(value);
}
__device__ __forceinline__ bool slot_get(const unsigned long long* slot, uint32_t tag, float& value,
                                         volatile int* abort_flag) {
    const volatile unsigned long long* vs = reinterpret_cast<const volatile unsigned long long*>(slot);
    unsigned long long v = *vs;
    if ((uint32_t)(v >> 32) != tag) {
        const uint64_t start = timer_ns();
        while (true) {
#pragma unroll 1
            for (int spin = 0; spin < 64; ++spin) {
                v = *vs;
                if ((uint32_t)(v >> 32) == tag) break;
            }
            if ((uint32_t)(v >> 32) == tag) break;
            if (*abort_flag) return false;
            if (timer_ns() - start > WAIT_LIMIT_NS) { *abort_flag = 1; return false; }
        }
    }
    value = __uint_as_float((uint32_t)v);
    return true;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// SPLIT: threads per query row (1: two CTAs per SM at head size 64, best when there are many query blocks;
// 2: one CTA per SM, each row's chain half as long, best when few blocks decide the duration).
template <int HD, int SPLIT>
struct Layout {
    static constexpr int ROW_THREADS = 128 * SPLIT, THREADS = 64 + ROW_THREADS;
    static constexpr int COLS = BKEY / SPLIT;                         // keys of a tile per row thread
    static constexpr int KCH = HD / 64;                               // 64-wide pieces of the head dim
    static constexpr int Q_BYTES = BQ * HD * 2;                       // [KCH][128 rows][128 bytes]
    static constexpr int KV_BYTES = BKEY * HD * 2;                    // one K or V tile, same arrangement
    static constexpr int STAGE_BYTES = 2 * KV_BYTES;                  // K then V
    // after the tiles: barriers (256 bytes), then what row partners exchange: [2 tiles][SPLIT][128] slots
    static constexpr int EXCHANGE_BYTES = 2 * SPLIT * BQ * 8;
    static constexpr size_t SMEM = Q_BYTES + (size_t)KV_STAGES * STAGE_BYTES + 1024 + 256 + EXCHANGE_BYTES;
    // TMEM columns: S (128 fp32) | P (64 columns of packed bf16 pairs) | O_j (HD fp32)
    static constexpr int S_COL = 0, P_COL = 128, O_COL = 192;
    static constexpr int TMEM_COLS = HD == 64 ? 256 : 512;
};

template <int HD, int SPLIT>
__global__ void __launch_bounds__(64 + 128 * SPLIT, (HD == 64 && SPLIT == 1) ? 2 : 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            __nv_bfloat16* __restrict__ out, int out_stride, const int* __restrict__ q_start,
                            const int* __restrict__ kv_len, const int* __restrict__ block_table, int bt_stride,
                            const int* __restrict__ item_row, int first_item, int n_items, int n_heads,
                            int n_kv_heads, int page_size, int window,
                            float scale_log2, long long k_row_base, long long v_row_base, long long page_rows,
                            int* __restrict__ status) {
    using L = Layout<HD, SPLIT>;
    constexpr int ROW_THREADS = L::ROW_THREADS, THREADS = L::THREADS, COLS = L::COLS;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;
    unsigned char* kv_s = base + L::Q_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + (size_t)KV_STAGES * L::STAGE_BYTES);
    uint64_t* q_full = bars;                  // TMA -> MMA
    uint64_t* kv_full = bars + 1;             // [KV_STAGES] TMA -> MMA
    uint64_t* kv_empty = kv_full + KV_STAGES; // [KV_STAGES] MMA -> TMA
    uint64_t* s_full = kv_empty + KV_STAGES;  // MMA -> softmax: S is complete
    uint64_t* p_ready = s_full + 1;           // softmax (all row threads) -> MMA: P is in TMEM, S and O_j are consumed
    uint64_t* o_full = p_ready + 1;           // MMA -> softmax: O_j is complete
    uint64_t* s_free = o_full + 1;            // softmax (all row threads) -> MMA: S is in registers, the next S may land
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    unsigned long long* exchange = reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(bars) + 256);

    pdl_prologue();
    // which (item, query block) is this CTA? late blocks see most keys: they come first
    int block = blockIdx.y, item = -1, qb = 0;
    for (int i = first_item; i < first_item + n_items; ++i) {
        int blocks = (q_start[i + 1] - q_start[i] + BQ - 1) / BQ;
        if (block < blocks) { item = i; qb = blocks - 1 - block; break; }
        block -= blocks;
    }
    if (item < 0) return;
    const int h = blockIdx.x, g = h / (n_heads / n_kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qs = q_start[item], q_len = q_start[item + 1] - qs;
    const int pos0 = kv_len[item] - q_len + qb * BQ;              // position of the block's first query
    const int rows = min(BQ, q_len - qb * BQ);
    const int tok0 = qs + qb * BQ;
    const int hi = pos0 + rows - 1;
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int kb_first = lo / BKEY, kb_last = hi / BKEY;
    // the item's block-table row: item_row[item] where the table is kept by request slot, else the item itself
    const int* bt = block_table + (size_t)(item_row ? item_row[item] : item) * bt_stride;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
        mbar_init(s_full, 1);
        mbar_init(p_ready, ROW_THREADS);
        mbar_init(o_full, 1);
        mbar_init(s_free, ROW_THREADS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < 2 * SPLIT * BQ; i += THREADS) exchange[i] = 0ull;      // tag 0 = nothing yet
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer: lane pg fetches page pg of a tile
        if (lane == 0) {
            mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
            for (int c = 0; c < L::KCH; ++c)
                tma_load_2d(q_s + c * (BQ * 128), &map_q, h * HD + 64 * c, tok0, q_full);
        }
        const uint32_t page_bytes = (uint32_t)page_size * 128;
        uint32_t it = 0;
        for (int kb = kb_first; kb <= kb_last; ++kb, ++it) {
            const int s = it % KV_STAGES;
            const int key0 = kb * BKEY;
            // pages of the tile that hold a key of [lo, hi]; the rest of the tile keeps stale data (masked)
            const int pg_lo = max(lo, key0) / page_size - key0 / page_size;
            const int pg_hi = min(hi, key0 + BKEY - 1) / page_size - key0 / page_size;
            // the page id is read before the wait: the table lookups of all pages run in parallel and overlap it
            long long page = 0;
            if (lane >= pg_lo && lane <= pg_hi) page = bt[key0 / page_size + lane];
            if (!mbar_wait(&kv_empty[s], ((it / KV_STAGES) & 1) ^ 1, abort_flag)) { if (lane == 0) atomicExch(status, 31); break; }
            unsigned char* k_dst = kv_s + (size_t)s * L::STAGE_BYTES;
            unsigned char* v_dst = k_dst + L::KV_BYTES;
            if (lane == 0) mbar_expect_tx(&kv_full[s], 2u * L::KCH * page_bytes * (uint32_t)(pg_hi - pg_lo + 1));
            __syncwarp();
            if (lane >= pg_lo && lane <= pg_hi) {
                const long long row = page * page_rows + (long long)g * page_size;
#pragma unroll
                for (int c = 0; c < L::KCH; ++c) {
                    tma_load_2d(k_dst + c * (BKEY * 128) + lane * page_bytes, &map_kv, 64 * c, (int)(k_row_base + row), &kv_full[s]);
                    tma_load_2d(v_dst + c * (BKEY * 128) + lane * page_bytes, &map_kv, 64 * c, (int)(v_row_base + row), &kv_full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            // S = Q K^T: D f32, A/B bf16, both K-major, N = 128, M = 128
            constexpr uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BKEY >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
            // O_j = P V: A from TMEM (K-major), B = V MN-major (bit 16), N = HD
            constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            if (!ok) atomicExch(status, 32);
            // S = Q K^T of tile `t` (its K tile must have landed); completion is signalled on s_full
            auto issue_qk = [&](uint32_t t) -> bool {
                const int st = t % KV_STAGES;
                if (!mbar_wait(&kv_full[st], (t / KV_STAGES) & 1, abort_flag)) { atomicExch(status, 33); return false; }
                tc_fence_after();
                const uint32_t k_addr = smem_u32(kv_s + (size_t)st * L::STAGE_BYTES);
#pragma unroll
                for (int c = 0; c < L::KCH; ++c)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_ss(tmem_base + L::S_COL, desc_sw128(smem_u32(q_s) + c * (BQ * 128), 16) + 2 * k,
                                desc_sw128(k_addr + c * (BKEY * 128), 16) + 2 * k, idesc_qk, (c | k) ? 1u : 0u);
                umma_commit(s_full);
                return true;
            };
            const uint32_t n_tiles = (uint32_t)(kb_last - kb_first + 1);
            if (ok) ok = issue_qk(0);
            for (uint32_t it = 0; it < n_tiles && ok; ++it) {
                const int s = it % KV_STAGES;
                // the scores of the next tile are computed while the rows work on this one: S is free as
                // soon as every row has it in registers
                if (it + 1 < n_tiles) {
                    if (!mbar_wait(s_free, it & 1, abort_flag)) { atomicExch(status, 34); break; }
                    if (!issue_qk(it + 1)) break;
                }
                // P of this tile is in TMEM (and O rescaled): O += P V over the 128 keys, 16 keys = 2048 bytes of V
                if (!mbar_wait(p_ready, it & 1, abort_flag)) { atomicExch(status, 35); break; }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(kv_s + (size_t)s * L::STAGE_BYTES) + L::KV_BYTES;
#pragma unroll
                for (int k = 0; k < BKEY / 16; ++k)
                    umma_ts(tmem_base + L::O_COL, tmem_base + L::P_COL + 8 * k,
                            desc_sw128(v_addr, BKEY * 128) + (uint64_t)((2048 * k) >> 4), idesc_pv, (it | k) ? 1u : 0u);
                umma_commit(&kv_empty[s]);
                umma_commit(o_full);
            }
        }
    } else {
        // ------------------------------------------------ softmax rows: warps 2.., SPLIT threads per row
        const int quarter = warp & 3;
        const int half = SPLIT == 2 ? (warp - 2) >> 2 : 0;        // which keys of a tile / which output columns
        const int r = quarter * 32 + lane;                        // query row of the tile = TMEM lane
        const int pos = pos0 + r;
        const int col0 = half * COLS;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        constexpr int OCOLS = HD / SPLIT;                         // columns of O that this thread owns
        float m_run = -INFINITY, l_run = 0.f;                     // l_run: the sum over this thread's keys only
        bool ok = true;
        uint32_t it = 0;
        for (int kb = kb_first; kb <= kb_last && ok; ++kb, ++it) {
            const int key0 = kb * BKEY + col0;                    // first key of this thread's half
            if (!mbar_wait(s_full, it & 1, abort_flag)) { ok = false; if (lane == 0) atomicExch(status, 36); break; }
            tc_fence_after();
            // this thread's 64 raw scores in registers (one TMEM round trip)
            uint32_t sr[COLS];
            tmem_ld_cols<COLS>(lane_base + L::S_COL + col0, sr);
            tc_fence_before();
            mbar_arrive(s_free);                                  // the next tile's scores may overwrite S
            const bool need_mask = (key0 + COLS - 1 > pos0) || (window > 0 && key0 < pos0 + rows - window) || rows < BQ;
            if (need_mask) {
                // keys this row may see: [max(lo_row, lo), pos]; everything else becomes -inf
                const int first_ok = (r < rows) ? max(lo, window > 0 ? pos - window + 1 : 0) - key0 : COLS;
                const int last_ok = (r < rows) ? pos - key0 : -1;
#pragma unroll
                for (int j = 0; j < COLS; ++j)
                    if (j < first_ok || j > last_ok) sr[j] = 0xff800000u;        // -inf
            }
            // maximum (four independent chains), in raw units; the scale is positive
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int j = 0; j < COLS; j += 4) {
                mx0 = fmaxf(mx0, __uint_as_float(sr[j]));
                mx1 = fmaxf(mx1, __uint_as_float(sr[j + 1]));
                mx2 = fmaxf(mx2, __uint_as_float(sr[j + 2]));
                mx3 = fmaxf(mx3, __uint_as_float(sr[j + 3]));
            }
            float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            // the row's other thread holds the maximum of the other keys (two buffers: a thread that runs
            // ahead into the next tile writes the other one)
            if constexpr (SPLIT == 2) {
                slot_put(exchange + ((it & 1) * SPLIT + half) * BQ + r, it + 1, mx);
                float mx_other;
                if (!slot_get(exchange + ((it & 1) * SPLIT + (half ^ 1)) * BQ + r, it + 1, mx_other, abort_flag)) {
                    ok = false;
                    atomicExch(status, 38);
                    break;
                }
                mx = fmaxf(mx, mx_other);
            }
            mx *= scale_log2;
            const float m_new = fmaxf(m_run, mx);
            const float base_m = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = ex2(m_run - base_m);
            m_run = m_new;
            // probabilities p = 2^(s * scale - m): one FMA and one ex2 per score; P (bf16 pairs) into TMEM
            const float neg_m = -base_m;
            float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
            for (int c = 0; c < COLS; c += 64) {
                uint32_t pr[32];
#pragma unroll
                for (int j = 0; j < 64; j += 4) {
                    const float p0 = ex2(fmaf(__uint_as_float(sr[c + j]), scale_log2, neg_m));
                    const float p1 = ex2(fmaf(__uint_as_float(sr[c + j + 1]), scale_log2, neg_m));
                    const float p2 = ex2(fmaf(__uint_as_float(sr[c + j + 2]), scale_log2, neg_m));
                    const float p3 = ex2(fmaf(__uint_as_float(sr[c + j + 3]), scale_log2, neg_m));
                    sum0 += p0; sum1 += p1; sum2 += p2; sum3 += p3;
                    __nv_bfloat162 lo2 = __floats2bfloat162_rn(p0, p1), hi2 = __floats2bfloat162_rn(p2, p3);
                    pr[j >> 1] = *reinterpret_cast<uint32_t*>(&lo2);
                    pr[(j >> 1) + 1] = *reinterpret_cast<uint32_t*>(&hi2);
                }
                tmem_st32(lane_base + L::P_COL + ((col0 + c) >> 1), pr);
            }
            const float sum = (sum0 + sum1) + (sum2 + sum3);
            l_run = l_run * corr + sum;
            // O of the earlier tiles (complete: o_full of the last tile was waited below) follows the new maximum;
            // both threads of a row see the same corr and rescale their own columns
            if (it > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
                for (int c = 0; c < OCOLS; c += 32) {
                    uint32_t orr[32];
                    tmem_ld32(lane_base + L::O_COL + half * OCOLS + c, orr);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; ++j) orr[j] = __float_as_uint(__uint_as_float(orr[j]) * corr);
                    tmem_st32(lane_base + L::O_COL + half * OCOLS + c, orr);
                }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            // V rows of keys outside [lo, hi] hold stale shared memory or stale cache contents: 0 * garbage
            // must stay 0, so the row's threads clear them (half a row each) before the product reads the tile
            {
                const int key = kb * BKEY + r;
                if (key > hi || key < lo) {
                    unsigned char* v_tile = kv_s + (size_t)(it % KV_STAGES) * L::STAGE_BYTES + L::KV_BYTES;
#pragma unroll
                    for (int c = 0; c < L::KCH; ++c) {
                        uint4* row = reinterpret_cast<uint4*>(v_tile + c * (BKEY * 128) + r * 128);
#pragma unroll
                        for (int i = 0; i < 8 / SPLIT; ++i) row[half * (8 / SPLIT) + i] = make_uint4(0, 0, 0, 0);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            tc_fence_before();
            mbar_arrive(p_ready);
            // the product of this tile must be complete before O is touched again (or read at the end)
            if (!mbar_wait(o_full, it & 1, abort_flag)) { ok = false; if (lane == 0) atomicExch(status, 37); break; }
            tc_fence_after();
        }
        // the row's sum is the sum of its two threads' sums (same running maximum in both)
        if (ok && SPLIT == 2) {
            slot_put(exchange + ((it & 1) * SPLIT + half) * BQ + r, 0x7fffffffu, l_run);
            float l_other = 0.f;
            if (!slot_get(exchange + ((it & 1) * SPLIT + (half ^ 1)) * BQ + r, 0x7fffffffu, l_other, abort_flag)) {
                ok = false;
                atomicExch(status, 39);
            }
            l_run += l_other;
        }
        if (ok) {
            // the whole warp reads its O rows from TMEM (the load is warp-wide); rows of the portion store
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            __nv_bfloat16* orow = out + (size_t)(tok0 + r) * out_stride + h * HD + half * OCOLS;
#pragma unroll
            for (int c = 0; c < OCOLS; c += 32) {
                uint32_t orr[32];
                tmem_ld32(lane_base + L::O_COL + half * OCOLS + c, orr);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (r < rows) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint4 pack;
                        __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(orr[d]) * inv, __uint_as_float(orr[d + 1]) * inv);
                        __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(orr[d + 2]) * inv, __uint_as_float(orr[d + 3]) * inv);
                        __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(orr[d + 4]) * inv, __uint_as_float(orr[d + 5]) * inv);
                        __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(orr[d + 6]) * inv, __uint_as_float(orr[d + 7]) * inv);
                        pack.x = *reinterpret_cast<uint32_t*>(&p0); pack.y = *reinterpret_cast<uint32_t*>(&p1);
                        pack.z = *reinterpret_cast<uint32_t*>(&p2); pack.w = *reinterpret_cast<uint32_t*>(&p3);
                        *reinterpret_cast<uint4*>(orow + c + d) = pack;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)L::TMEM_COLS) : "memory");
    }
}

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
// rows x cols bf16 matrix with row pitch ld (elements); boxes of box_rows x 64 elements, 128-byte swizzle
static bool make_map(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int HD, int SPLIT>
int launch(const void* q, int q_stride, int T, void* out, int out_stride, const void* pool, long long pool_rows,
           long long k_row_base, long long v_row_base, long long page_rows, const int* q_start, const int* kv_len,
           const int* block_table, int bt_stride, const int* item_row, int first_item, int n_items, int max_blocks,
           int n_heads, int n_kv_heads, int page_size, int window, float scale, int* status, cudaStream_t stream) {
    CUtensorMap map_q, map_kv;
    if (!make_map(&map_q, q, T, n_heads * HD, q_stride, BQ)) return PS_ERR_LAUNCH;
    if (!make_map(&map_kv, pool, pool_rows, HD, HD, page_size)) return PS_ERR_LAUNCH;
    using L = Layout<HD, SPLIT>;
    auto kernel = prefill_attention_tc_kernel<HD, SPLIT>;
    static size_t raised[MAX_DEVICES] = {0};
    if (!ensure_dynamic_smem((const void*)kernel, (size_t)L::SMEM, raised)) return PS_ERR_LAUNCH;
    // heads vary fastest: the heaviest query blocks of all heads are scheduled first
    return launch_pdl(kernel, dim3(n_heads, max_blocks), dim3(L::THREADS), L::SMEM, stream, map_q, map_kv,
                      (__nv_bfloat16*)out, out_stride, q_start, kv_len, block_table, bt_stride, item_row, first_item,
                      n_items, n_heads, n_kv_heads, page_size, window, scale * 1.4426950408889634f, k_row_base,
                      v_row_base, page_rows, status);
}

}  // namespace pftc
}  // namespace ps

// q: the step's flat [T, >= n_heads*head_dim] buffer (row pitch q_stride). pool: base of the cache group's pool,
// seen as pool_rows rows of head_dim elements; a page's rows start at page * page_rows; within a page the K rows
// of this cache layer start at k_row_base and the V rows at v_row_base, kv head g at + g * page_size.
// max_blocks >= sum over the items of ceil(q_len / 128). Head sizes 64 and 128, pages of 8..64 tokens.
// row_threads: threads per query row, 1 or 2 (0: chosen here).
// item_row (may be null): the block-table row of each item, where the table is kept by request slot.
PS_EXPORT int ps_prefill_attention_tc(const void* q, int q_stride, int T, void* out, int out_stride, const void* pool,
                                      long long pool_rows, long long k_row_base, long long v_row_base,
                                      long long page_rows, const int* q_start, const int* kv_len,
                                      const int* block_table, int bt_stride, const int* item_row, int first_item,
                                      int n_items,
                                      int max_blocks, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                      int window, float scale, int row_threads, int* status, void* stream) {
    if (n_items <= 0 || max_blocks <= 0) return PS_OK;
    if (row_threads < 0 || row_threads > 2) return PS_ERR_BAD_ARGUMENT;
    if (!status) return PS_ERR_BAD_ARGUMENT;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || max_blocks > 65535) return PS_ERR_BAD_ARGUMENT;
    if (head_dim != 64 && head_dim != 128) return PS_ERR_UNSUPPORTED;
    if (page_size < 8 || page_size > 64 || (page_size & (page_size - 1))) return PS_ERR_UNSUPPORTED;
    if (q_stride % 8 != 0 || out_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)pool & 15))
        return PS_ERR_UNSUPPORTED;
    if (pool_rows >= (1ll << 31)) return PS_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    // Few query blocks: the duration is that of the block with most keys, so every row gets two threads.
    // Many blocks: throughput counts, one thread per row leaves room for two CTAs per SM (head size 64).
    // Measured, 12 heads of 64: 2 x 1,024 tokens 17.6 (two) vs 23.5 us (one); 8 x 1,024: 66.9 vs 53.7 us.
    // row_threads 0 leaves the choice to a count of the blocks.
    const bool two = row_threads ? row_threads == 2 : (long long)max_blocks * n_heads <= 148;
#define PS_PFTC_LAUNCH(HD, SPLIT)                                                                                     \
    return ps::pftc::launch<HD, SPLIT>(q, q_stride, T, out, out_stride, pool, pool_rows, k_row_base, v_row_base,     \
                                       page_rows, q_start, kv_len, block_table, bt_stride, item_row, first_item,      \
                                       n_items, max_blocks, n_heads, n_kv_heads, page_size, window, scale, status, s)
    if (head_dim == 64) {
        if (two) PS_PFTC_LAUNCH(64, 2);
        PS_PFTC_LAUNCH(64, 1);
    }
    if (two) PS_PFTC_LAUNCH(128, 2);
    PS_PFTC_LAUNCH(128, 1);
#undef PS_PFTC_LAUNCH
}
