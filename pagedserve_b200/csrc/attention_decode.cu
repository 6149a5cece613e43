// Paged attention for few query tokens (decode steps and short portions), bfloat16, split along keys.
//
// One CTA per (token, head, key split). The reference launches one program per (request, head) that
// walks the whole context (src/kernels/triton_paged_attention.py:225-320, grid at :530): at batch 1
// that is 12 programs for 148 SMs. Here the keys of a token are cut into chunks of `chunk_keys` keys
// aligned to absolute positions (128 keys at head size 64); a split is a whole number of chunks and
// is one CTA of 4 warps; the last CTA of a (token, head) to finish merges the partial
// (max, sum, acc) states in split order. With one split the output is written directly.
//
// A chunk's K and V blocks are brought into shared memory page by page with bulk asynchronous copies
// (cp.async.bulk, completion on an mbarrier): a page's keys of one head are contiguous, so a chunk is
// 2 * chunk_keys / page_size copies and all of them are in flight at once. Thread j then owns key j
// for the scores (16-byte reads of its row in an order rotated by j, which keeps the reads free of
// bank conflicts), the four warps share the keys for p.V with lanes on head dims. Softmax state and
// accumulators are float32 (reference: triton_paged_attention.py:219-223, 275-320).
//
// Every wait on the mbarrier is bounded; a wait that runs out sets *status and the CTA stops waiting.
//
// Scratch (only when splits > 1): part_acc[T][H][S][hd] f32, part_ml[T][H][S][2] f32, counters[T*H] int32
// (zero before the first use; the merging CTA sets its counter back to zero).
#include "common.cuh"

namespace ps {

constexpr int DEC_WARPS = 4;
constexpr int DEC_THREADS = DEC_WARPS * 32;

// elements between units in shared memory: the unit's bytes padded so that the stride is 16 (mod 128)
__host__ __device__ inline int attention_unit_stride(int unit, int head_dim) {
    const int bytes = unit * head_dim * 2;
    return (bytes + ((16 - bytes % 128) + 128) % 128) / 2;
}

__host__ __device__ inline int attention_chunk_keys(int head_dim, int page_size) {
    int keys = head_dim <= 64 ? 128 : (head_dim <= 128 ? 64 : 32);     // a power of two, K + V of a chunk <= 32 KB
    if (keys < page_size) keys = page_size;
    return keys;
}

__device__ __forceinline__ float ldcg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return done != 0;
}
// false if the wait ran out
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (int spin = 0; spin < (1 << 22); ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Scores and p.V on tensor cores although there is one query: keys (then head dims) sit on the 16-row
// side of mma.sync.m16n8k16 and the query (then the probabilities) is column 0 of the 8-column side.
//   S^T[key]  = sum_d K[key][d] q[d]        A = K rows from shared memory (ldmatrix),   B = q in lanes g == 0
//   O^T[d]    = sum_key V[key][d] p[key]    A = V^T (ldmatrix.trans),                   B = p in lanes g == 0
// A chunk is copied in units of U consecutive keys of one page (one bulk copy for K, one for V; U = 16 at
// head size 64). In shared memory the units lie `unit_stride` bytes apart with unit_stride = 16 (mod 128),
// and MMA row m of the chunk is key (m mod NU) * U + m / NU (NU units per chunk): the 8 rows of every
// ldmatrix then come from 8 different units and fall on 8 different bank groups, although each unit is a
// plain contiguous copy. Keys outside [lo, p] have their V rows zeroed and their scores masked.
// KS: head-dim steps of 16 the kernel is compiled for (head_dim <= 16 * KS); fewer steps, fewer registers.
// How the partial states of the splits of one (token, head) are merged:
//   n_splits == 1            nothing to merge;
//   cluster == n_splits > 1  the splits are one thread-block cluster; the first active CTA reads the others'
//                            (max, sum, acc) from their shared memory after a cluster barrier: no trip to
//                            global memory, no atomics;
//   cluster <= 1 < n_splits  through part_acc / part_ml / counters in global memory, merged by the CTA that
//                            finishes last.
// q_start / kv_len (both or neither): with them the kernel knows which keys of a request are older than
// this step (positions below kv_len - new tokens). A first chunk made of such keys only is fetched BEFORE
// the wait for the kernel that writes this step's q, k and v, so the fetch overlaps that kernel.
// GROUPS > 1: the CTA is GROUPS teams of 128 threads with chunk buffers of their own; team i takes chunks
// first + i, first + i + GROUPS, ... of the CTA's range, all teams at once, and the teams' states are merged
// through shared memory behind one barrier. With few (token, head) pairs (at most one per SM) the whole context
// of a pair is then one CTA (n_splits = 1) and nothing is handed over through global memory: publishing a
// partial state, the fence, the counter and the last CTA's reads cost about 2.5 us per layer at batch 8.
template <int KS, int GROUPS = 1>
__global__ void __launch_bounds__(DEC_THREADS * GROUPS, GROUPS > 1 ? 1 : (KS == 4 ? 6 : (KS == 8 ? 4 : 2)))
paged_attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                              __nv_bfloat16* __restrict__ out, int out_stride,
                              const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                              long long page_stride, const int* __restrict__ token_item,
                              const int* __restrict__ positions, const int* __restrict__ block_table,
                              int bt_stride, int n_heads, int n_kv_heads, int head_dim, int page_size,
                              int window, float scale_log2, int chunk_keys, int split_chunks, int n_splits,
                              float* __restrict__ part_acc, float* __restrict__ part_ml,
                              int* __restrict__ counters, int* __restrict__ status,
                              const int* __restrict__ q_start, const int* __restrict__ kv_len, int cluster,
                              const int* __restrict__ token_row) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // page_size, chunk_keys and the unit are powers of two: shifts and masks instead of divisions
    const int unit = min(page_size, chunk_keys >> 3);                                // keys per copy
    const int unit_log2 = 31 - __clz(unit), page_log2 = 31 - __clz(page_size), chunk_log2 = 31 - __clz(chunk_keys);
    const int n_units = chunk_keys >> unit_log2;                                     // a power of two >= 8
    const int units_log2 = chunk_log2 - unit_log2;
    const int unit_elems = attention_unit_stride(unit, head_dim);                    // padded unit, elements
    // One stage of chunk buffers: measured on B200, a second stage (copying the next chunk during the
    // compute of this one) halves the CTAs per SM and was slower at every batch size (batch 64: 44 vs 36 us).
    constexpr int THREADS = DEC_THREADS * GROUPS;
    const int tid_all = threadIdx.x;                                                 // thread of the CTA
    const int grp = GROUPS > 1 ? tid_all / DEC_THREADS : 0;                          // its team
    const int tid = GROUPS > 1 ? tid_all % DEC_THREADS : tid_all;                    // thread of the team
    const size_t team_elems = (size_t)2 * n_units * unit_elems + chunk_keys;         // K, V, probabilities
    __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw) + grp * team_elems;   // [n_units][unit_elems]
    __nv_bfloat16* v_s = k_s + (size_t)n_units * unit_elems;
    __nv_bfloat16* p_s = v_s + (size_t)n_units * unit_elems;                         // [chunk_keys] probabilities
    // [GROUPS][head_dim] accumulators; the first row becomes the CTA's merged output
    float* o_all = reinterpret_cast<float*>(reinterpret_cast<__nv_bfloat16*>(smem_raw) + GROUPS * team_elems);
    float* o_s = o_all;
    __shared__ float red_a_all[GROUPS][DEC_WARPS], red_b_all[GROUPS][DEC_WARPS];
    float* red_a = red_a_all[grp];
    float* red_b = red_b_all[grp];
    __shared__ float ml_team[GROUPS][2];                                             // (max, sum) of each team
    __shared__ float ml_pub[2];                                                      // (max, sum) for the cluster
    __shared__ __align__(8) uint64_t bar_all[GROUPS];
    uint64_t& bar = bar_all[grp];
    __shared__ int last_flag;
    auto team_sync = [&]() {                                                         // the 128 threads of a team
        if constexpr (GROUPS == 1) __syncthreads();
        else asm volatile("bar.sync %0, 128;" ::"r"(grp + 1) : "memory");
    };

    // ---- before the wait: only what no kernel of this step writes (positions, tables, older keys)
    const int t = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    const int lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, tq = lane & 3;
    const int p = positions[t];
    const int item = token_item[t];
    const int first_new = (q_start && kv_len) ? kv_len[item] - (q_start[item + 1] - q_start[item]) : 0;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int first_chunk = lo >> chunk_log2, last_chunk = p >> chunk_log2;
    const int first_split = first_chunk / split_chunks, last_split = last_chunk / split_chunks;
    const int n_active = last_split - first_split + 1;
    if (last_split >= n_splits) {
        // The grid is too shallow for this token's newest keys (the caller's bound on the context was too
        // low). Every CTA of the (token, head) sees the same: none computes, merges or touches a counter,
        // the output stays unwritten and the status word says why.
        if (status && tid == 0 && split == 0) atomicExch(status, 3);
        return;
    }
    const bool active = split >= first_split && split <= last_split;
    const bool by_cluster = cluster > 1 && n_active > 1;
    if (!active && !by_cluster) return;                                // no keys here and nobody waits for us
    const int chunk_lo = (active ? max(first_chunk, split * split_chunks) : 1) + grp;   // this team's first chunk
    const int chunk_hi = active ? min(last_chunk, (split + 1) * split_chunks - 1) : 0;

    const int g = h / (n_heads / n_kv_heads);
    // the token's block-table row: token_row[t] where the table is kept by request slot, else its item
    const int* bt = block_table + (size_t)(token_row ? token_row[t] : item) * bt_stride;
    const uint32_t unit_bytes = (uint32_t)unit * head_dim * 2;
    if (tid == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Copies of one chunk: thread u brings unit u (K and V) if it holds keys of [lo, p]. `part` selects the
    // units made only of keys older than this step (0: fetched before the wait), the others (1: after it),
    // or all (2). The chunk's barrier expects the bytes of all its units once.
    auto issue_chunk = [&](int chunk, int part) {
        const int key0 = chunk << chunk_log2;
        const int j_lo = max(lo, key0) - key0, j_hi = min(p, key0 + chunk_keys - 1) - key0;
        const int u_lo = j_lo >> unit_log2, u_hi = j_hi >> unit_log2;
        if (tid == 0 && part != 1) mbar_expect_tx(&bar, 2u * unit_bytes * (uint32_t)(u_hi - u_lo + 1));
        if (tid >= u_lo && tid <= u_hi) {
            const int key = key0 + (tid << unit_log2);
            const bool old = key + unit <= first_new;
            if (part == 2 || (part == 0) == old) {
                const int page = bt[key >> page_log2];
                const long long src = (long long)page * page_stride +
                                      ((long long)g * page_size + (key & (page_size - 1))) * head_dim;
                bulk_copy_g2s(k_s + (size_t)tid * unit_elems, k_pool + src, unit_bytes, &bar);
                bulk_copy_g2s(v_s + (size_t)tid * unit_elems, v_pool + src, unit_bytes, &bar);
            }
        }
    };
    // the first chunk's older units go out now, the rest of it after the wait
    const bool mine = active && chunk_lo <= chunk_hi;                 // this team has a chunk at all
    const bool early = mine && (chunk_lo << chunk_log2) < first_new;
    if (early) issue_chunk(chunk_lo, 0);

    pdl_prologue();
    q = pdl_fresh(q);
    k_pool = pdl_fresh(k_pool);
    v_pool = pdl_fresh(v_pool);
    if (mine) issue_chunk(chunk_lo, early ? 1 : 2);

    // the query as B fragments: lanes with g == 0 hold q[16 ks + 2 t .. +1] and q[16 ks + 2 t + 8 .. +9]
    const int ksteps = head_dim >> 4;                              // <= KS
    uint32_t qb[KS][2];
    {
        const __nv_bfloat16* qrow = q + (size_t)t * q_stride + h * head_dim;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qb[ks][0] = qb[ks][1] = 0u;
            if (ks < ksteps && gq == 0) {
                qb[ks][0] = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * tq);
                qb[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * tq + 8);
            }
        }
    }

    // this warp owns the output rows (head dims) of m-tiles warp, warp + 4, ...
    constexpr int OT = (KS + DEC_WARPS - 1) / DEC_WARPS;          // output tiles per warp
    float o_acc[OT][4];
#pragma unroll
    for (int i = 0; i < OT; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const int key_tiles = chunk_keys >> 4;
    const int unit_mask = n_units - 1;
    // MMA row m of a chunk is key (m % n_units) * unit + m / n_units and lies at element
    // (m % n_units) * unit_elems + (m / n_units) * head_dim of the chunk buffers
    auto row_elem = [&](int m) { return (size_t)(m & unit_mask) * unit_elems + (size_t)(m >> units_log2) * head_dim; };
    auto row_key = [&](int m) { return ((m & unit_mask) << unit_log2) + (m >> units_log2); };
    uint32_t phase = 0;
    bool ok = true;

    for (int chunk = chunk_lo; chunk <= chunk_hi; chunk += GROUPS) {
        const int key0 = chunk << chunk_log2;
        const int j_lo = max(lo, key0) - key0, j_hi = min(p, key0 + chunk_keys - 1) - key0;   // valid keys of the chunk
        if (chunk != chunk_lo) issue_chunk(chunk, 2);
        if (ok && !mbar_wait_bounded(&bar, phase)) {
            ok = false;
            if (status) atomicExch(status, 2);
        }
        phase ^= 1;
        if (tid < chunk_keys) {
            // rows of keys outside [j_lo, j_hi] hold stale or no data: 0 * garbage must stay 0
            const int key = row_key(tid);
            if (key < j_lo || key > j_hi) {
                const size_t off = row_elem(tid);
                uint4* vz = reinterpret_cast<uint4*>(v_s + off);
                uint4* kz = reinterpret_cast<uint4*>(k_s + off);
                for (int c = 0; c < (head_dim >> 3); ++c) { vz[c] = make_uint4(0, 0, 0, 0); kz[c] = make_uint4(0, 0, 0, 0); }
            }
        }
        team_sync();
        // ---- scores: key tiles warp, warp + 4, ... ; lanes with t == 0 end up with keys g and g + 8
        float sc[2][2];                                           // [tile of this warp][row g / g+8]
        float wmax = -INFINITY;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int mt = warp + DEC_WARPS * i;
            sc[i][0] = sc[i][1] = -INFINITY;
            if (mt < key_tiles) {
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                const __nv_bfloat16* arow = k_s + row_elem(16 * mt + (lane & 15)) + (lane >> 4) * 8;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    if (ks < ksteps) {
                        uint32_t a[4];
                        ldsm_x4(a, arow + 16 * ks);
                        mma_16816(c, a, qb[ks][0], qb[ks][1]);
                    }
                }
                const int ka = row_key(16 * mt + gq), kb = row_key(16 * mt + gq + 8);   // MMA rows -> keys of the chunk
                if (tq == 0 && ok) {
                    if (ka >= j_lo && ka <= j_hi) sc[i][0] = c[0] * scale_log2;
                    if (kb >= j_lo && kb <= j_hi) sc[i][1] = c[2] * scale_log2;
                }
                wmax = fmaxf(wmax, fmaxf(sc[i][0], sc[i][1]));
            }
        }
        wmax = warp_max(wmax);
        if (lane == 0) red_a[warp] = wmax;
        team_sync();
        const float cmax = fmaxf(fmaxf(red_a[0], red_a[1]), fmaxf(red_a[2], red_a[3]));
        const float m_new = fmaxf(m_run, cmax);
        float wsum = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int mt = warp + DEC_WARPS * i;
            if (mt < key_tiles && tq == 0) {
                const float pa = (sc[i][0] == -INFINITY) ? 0.f : exp2f(sc[i][0] - m_new);
                const float pb = (sc[i][1] == -INFINITY) ? 0.f : exp2f(sc[i][1] - m_new);
                p_s[16 * mt + gq] = __float2bfloat16_rn(pa);
                p_s[16 * mt + gq + 8] = __float2bfloat16_rn(pb);
                wsum += pa + pb;
            }
        }
        wsum = warp_sum(wsum);
        if (lane == 0) red_b[warp] = wsum;
        team_sync();
        const float csum = (red_b[0] + red_b[1]) + (red_b[2] + red_b[3]);
        const float corr = (m_new == -INFINITY) ? 1.f : exp2f(m_run - m_new);
        l_run = l_run * corr + csum;
        m_run = m_new;
        // ---- O^T += V^T p : this warp's head-dim tiles, all key steps of the chunk
#pragma unroll
        for (int i = 0; i < OT; ++i) {
            const int dt = warp + DEC_WARPS * i;
            if (dt < ksteps) {
                o_acc[i][0] *= corr; o_acc[i][1] *= corr; o_acc[i][2] *= corr; o_acc[i][3] *= corr;
                const int col = (2 * dt + ((lane >> 3) & 1)) * 8;
                const int r = (lane & 7) + ((lane >> 4) & 1) * 8;
                for (int kk = 0; kk < key_tiles; ++kk) {
                    uint32_t a[4];
                    ldsm_x4_trans(a, v_s + row_elem(16 * kk + r) + col);
                    uint32_t b0 = 0u, b1 = 0u;
                    if (gq == 0) {
                        b0 = *reinterpret_cast<const uint32_t*>(p_s + 16 * kk + 2 * tq);
                        b1 = *reinterpret_cast<const uint32_t*>(p_s + 16 * kk + 2 * tq + 8);
                    }
                    mma_16816(o_acc[i], a, b0, b1);
                }
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        team_sync();                                      // the buffers may be overwritten now
    }
    // column 0 of the accumulators is the output: lanes with t == 0 hold head dims 16 dt + g and + 8
#pragma unroll
    for (int i = 0; i < OT; ++i) {
        const int dt = warp + DEC_WARPS * i;
        if (dt < ksteps && tq == 0) {
            o_all[grp * head_dim + 16 * dt + gq] = o_acc[i][0];
            o_all[grp * head_dim + 16 * dt + gq + 8] = o_acc[i][2];
        }
    }
    if constexpr (GROUPS > 1) {
        // the teams' states become the CTA's: weights from the maxima, then the weighted sums (team order)
        if (tid == 0) { ml_team[grp][0] = m_run; ml_team[grp][1] = l_run; }
        __syncthreads();
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < GROUPS; ++i) M = fmaxf(M, ml_team[i][0]);
        float w[GROUPS], L = 0.f;
#pragma unroll
        for (int i = 0; i < GROUPS; ++i) {
            w[i] = (ml_team[i][0] == -INFINITY) ? 0.f : exp2f(ml_team[i][0] - M);
            L += ml_team[i][1] * w[i];
        }
        for (int d = tid_all; d < head_dim; d += THREADS) {
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < GROUPS; ++i) o += o_all[i * head_dim + d] * w[i];
            o_all[d] = o;                                  // thread d alone reads and writes column d
        }
        m_run = M;
        l_run = L;
    }
    if (tid_all == 0) { ml_pub[0] = m_run; ml_pub[1] = l_run; }
    __syncthreads();
    if (n_splits == 1 || n_active == 1) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        for (int d = tid_all; d < head_dim; d += THREADS)
            out[(size_t)t * out_stride + h * head_dim + d] = __float2bfloat16_rn(o_s[d] * inv);
        return;
    }
    if (by_cluster) {
        // every CTA of the cluster has published (max, sum, acc) in its shared memory (idle ones: -inf, 0, 0)
        cluster_sync_all();
        if (split == first_split) {
            // everything the merge needs is asked for at once (a portable cluster has at most 8 CTAs): one trip
            // through distributed shared memory instead of one per value
            constexpr int MAXC = 8;
            float mr[MAXC], lr[MAXC], ov[MAXC];
#pragma unroll
            for (int i = 0; i < MAXC; ++i) {
                const int r = first_split + i;
                const bool on = r <= last_split;
                mr[i] = on ? ld_cluster_f32(&ml_pub[0], r) : -INFINITY;
                lr[i] = on ? ld_cluster_f32(&ml_pub[1], r) : 0.f;
                ov[i] = (on && tid_all < head_dim) ? ld_cluster_f32(&o_s[tid_all], r) : 0.f;
            }
            float M = -INFINITY;
#pragma unroll
            for (int i = 0; i < MAXC; ++i) M = fmaxf(M, mr[i]);
            float L = 0.f;
#pragma unroll
            for (int i = 0; i < MAXC; ++i) {
                mr[i] = (mr[i] == -INFINITY) ? 0.f : exp2f(mr[i] - M);        // now the weight of split i
                L += lr[i] * mr[i];
            }
            const float inv = L > 0.f ? 1.f / L : 0.f;
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < MAXC; ++i) o += ov[i] * mr[i];
            float more = 0.f;                                         // head dim tid_all + 128 (head_dim <= 256)
            if (tid_all + THREADS < head_dim) {
#pragma unroll
                for (int i = 0; i < MAXC; ++i)
                    if (first_split + i <= last_split) more += ld_cluster_f32(&o_s[tid_all + THREADS], first_split + i) * mr[i];
            }
            // the others' shared memory has been read: they may leave while the result is written
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            if (tid_all < head_dim) out[(size_t)t * out_stride + h * head_dim + tid_all] = __float2bfloat16_rn(o * inv);
            if (tid_all + THREADS < head_dim)
                out[(size_t)t * out_stride + h * head_dim + tid_all + THREADS] = __float2bfloat16_rn(more * inv);
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            return;
        }
        cluster_sync_all();                                   // nobody's shared memory goes away before it was read
        return;
    }
    // several splits hold keys of this token: publish the partial state
    const size_t slot = ((size_t)t * n_heads + h) * n_splits + split;
    for (int d = tid_all; d < head_dim; d += THREADS) part_acc[slot * head_dim + d] = o_s[d];
    if (tid_all == 0) { part_ml[slot * 2] = m_run; part_ml[slot * 2 + 1] = l_run; }
    __threadfence();
    __syncthreads();
    if (tid_all == 0) {
        int prev = atomicAdd(&counters[t * n_heads + h], 1);
        last_flag = (prev == n_active - 1);
        if (last_flag) counters[t * n_heads + h] = 0;
    }
    __syncthreads();
    if (!last_flag) return;
    // (no fence on this side: the partial states below are read with ld.global.cg, from L2, where the other
    // CTAs' stores were performed before their fences let their counter increments through)
    const size_t base = ((size_t)t * n_heads + h) * n_splits + first_split;
    // the partial accumulators are asked for first (they do not depend on the maxima), then the (max, sum)
    // pairs; the weight of each split is computed once and shared
    constexpr int HOLD = 8;                                   // splits whose values a thread keeps in flight
    const int d0 = tid_all;                                       // head dims d0, d0 + 128, ... belong to this thread
    float held[HOLD];
    if (d0 < head_dim) {
#pragma unroll
        for (int i = 0; i < HOLD; ++i)
            held[i] = i < n_active ? ldcg_f32(part_acc + (base + i) * head_dim + d0) : 0.f;
    }
    if (n_active <= HOLD) {
        // few splits (the usual case): every thread takes the (max, sum) pairs too and weighs for itself:
        // one trip to L2 for everything, no shared memory, no barrier
        float mh[HOLD], lh[HOLD];
#pragma unroll
        for (int i = 0; i < HOLD; ++i) {
            mh[i] = -INFINITY;
            lh[i] = 0.f;
            if (i < n_active)
                asm volatile("ld.global.cg.v2.f32 {%0, %1}, [%2];" : "=f"(mh[i]), "=f"(lh[i]) : "l"(part_ml + (base + i) * 2));
        }
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < HOLD; ++i) M = fmaxf(M, mh[i]);
        float L = 0.f;
#pragma unroll
        for (int i = 0; i < HOLD; ++i) {
            mh[i] = (i < n_active) ? exp2f(mh[i] - M) : 0.f;           // now the weight of split i
            L += lh[i] * mh[i];
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        for (int d = d0, round = 0; d < head_dim; d += THREADS, ++round) {
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < HOLD; ++i) {
                if (i < n_active)
                    o += (round == 0 ? held[i] : ldcg_f32(part_acc + (base + i) * head_dim + d)) * mh[i];
            }
            out[(size_t)t * out_stride + h * head_dim + d] = __float2bfloat16_rn(o * inv);
        }
        return;
    }
    float* w_s = reinterpret_cast<float*>(smem_raw);          // the chunk buffers are free now: [n_active] weights
    float* ml_s = w_s + n_active;                             // then [n_active][2]
    const bool staged = 3 * n_active * 4 <= 2 * chunk_keys * head_dim;      // always, unless a huge split count
    if (staged) {
        for (int i = tid_all; i < 2 * n_active; i += THREADS) ml_s[i] = ldcg_f32(part_ml + base * 2 + i);
        __syncthreads();
        if (tid_all < 32) {
            float M = -INFINITY;
            for (int i = lane; i < n_active; i += 32) M = fmaxf(M, ml_s[2 * i]);
            M = warp_max(M);
            float L = 0.f;
            for (int i = lane; i < n_active; i += 32) {
                const float w = exp2f(ml_s[2 * i] - M);
                w_s[i] = w;
                L += ml_s[2 * i + 1] * w;
            }
            L = warp_sum(L);
            if (lane == 0) red_a[0] = L > 0.f ? 1.f / L : 0.f;
        }
        __syncthreads();
        const float inv = red_a[0];
        for (int d = d0, round = 0; d < head_dim; d += THREADS, ++round) {
            float o = 0.f;
            if (round == 0) {
#pragma unroll
                for (int i = 0; i < HOLD; ++i)
                    if (i < n_active) o += held[i] * w_s[i];
                for (int i = HOLD; i < n_active; ++i) o += ldcg_f32(part_acc + (base + i) * head_dim + d) * w_s[i];
            } else {
                for (int i = 0; i < n_active; ++i) o += ldcg_f32(part_acc + (base + i) * head_dim + d) * w_s[i];
            }
            out[(size_t)t * out_stride + h * head_dim + d] = __float2bfloat16_rn(o * inv);
        }
        return;
    }
    float M = -INFINITY;
    for (int i = 0; i < n_active; ++i) M = fmaxf(M, ldcg_f32(part_ml + (base + i) * 2));
    float L = 0.f;
    for (int i = 0; i < n_active; ++i)
        L += ldcg_f32(part_ml + (base + i) * 2 + 1) * exp2f(ldcg_f32(part_ml + (base + i) * 2) - M);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int d = tid_all; d < head_dim; d += THREADS) {
        float o = 0.f;
        for (int i = 0; i < n_active; ++i)
            o += ldcg_f32(part_acc + (base + i) * head_dim + d) * exp2f(ldcg_f32(part_ml + (base + i) * 2) - M);
        out[(size_t)t * out_stride + h * head_dim + d] = __float2bfloat16_rn(o * inv);
    }
}

}  // namespace ps

// Keys per chunk for a head size and page size: splits are whole numbers of chunks.
PS_EXPORT int ps_attention_chunk_keys(int head_dim, int page_size) {
    if (head_dim <= 0 || page_size <= 0) return 0;
    return ps::attention_chunk_keys(head_dim, page_size);
}

// split_tiles: tiles of 32 keys per split (split_tiles * 32 must be a multiple of the chunk size);
// n_splits: grid depth, at least ceil(longest context / split length).
// With n_splits == 1 the scratch pointers may be null. status (may be null) is set non-zero if a
// bounded wait ran out.
static int launch_attention_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_pool,
                                   const void* v_pool, long long page_stride, const int* token_item,
                                   const int* positions, const int* block_table, int bt_stride, int T, int n_heads,
                                   int n_kv_heads, int head_dim, int page_size, int window, float scale,
                                   int split_tiles, int n_splits, float* part_acc, float* part_ml, int* counters,
                                   int* status, void* stream, const int* q_start = nullptr,
                                   const int* kv_len = nullptr, int cluster = 1, const int* token_row = nullptr) {
    if (T <= 0) return PS_OK;
    if ((q_start == nullptr) != (kv_len == nullptr)) return PS_ERR_BAD_ARGUMENT;
    if (cluster > 1 && (cluster != n_splits || cluster > 8 || (cluster & (cluster - 1)))) return PS_ERR_BAD_ARGUMENT;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return PS_ERR_BAD_ARGUMENT;
    if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 256) return PS_ERR_UNSUPPORTED;
    if (page_size <= 0 || page_size > 64 || (page_size & (page_size - 1))) return PS_ERR_UNSUPPORTED;
    if (n_heads > 65535 || n_splits > 65535 || n_splits < 1 || split_tiles < 1) return PS_ERR_UNSUPPORTED;
    if (n_splits > 1 && cluster <= 1 && (!part_acc || !part_ml || !counters)) return PS_ERR_BAD_ARGUMENT;
    if (q_stride % 8 != 0 || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) || page_stride % 8 != 0)
        return PS_ERR_UNSUPPORTED;
    const int chunk_keys = ps::attention_chunk_keys(head_dim, page_size);
    if ((split_tiles * 32) % chunk_keys != 0) return PS_ERR_BAD_ARGUMENT;
    int split_chunks = split_tiles * 32 / chunk_keys;
    const int unit = page_size < (chunk_keys >> 3) ? page_size : (chunk_keys >> 3);
    const size_t team_bytes = (size_t)(chunk_keys / unit) * ps::attention_unit_stride(unit, head_dim) * 2 * 2 +
                              (size_t)chunk_keys * 2;
    // Few (token, head) pairs, at most one per SM: the whole context of a pair is one CTA of TEAMS teams that
    // work on TEAMS chunks at once and merge through shared memory, instead of n_splits CTAs that merge
    // through global memory. (Head sizes up to 64 only: the teams of one CTA share an SM's registers.)
    constexpr int TEAMS = 6;
    static int sm_count = 0;
    if (!sm_count) {
        int device = 0;
        cudaGetDevice(&device);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sm_count <= 0)
            sm_count = 1;
    }
    // (a pair's chunks are walked in rounds of TEAMS: beyond two rounds, i.e. contexts of more than 12 chunks, the
    // split form's parallelism over more SMs is worth its merge again)
    const bool teams = head_dim <= 64 && cluster <= 1 && n_splits > 1 && (long long)T * n_heads <= sm_count &&
                       (long long)n_splits * split_chunks <= 2 * TEAMS;
    int groups = 1;
    if (teams) {
        groups = TEAMS;
        split_chunks *= n_splits;
        n_splits = 1;
    }
    dim3 grid(T, n_heads, n_splits);
    size_t smem = (size_t)groups * (team_bytes + (size_t)head_dim * 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (teams) {
        auto kernel = ps::paged_attention_decode_kernel<4, TEAMS>;
        static size_t raised[ps::MAX_DEVICES] = {0};
        if (!ps::ensure_dynamic_smem((const void*)kernel, smem, raised)) return PS_ERR_LAUNCH;
        return ps::launch_pdl_cluster(kernel, grid, dim3(ps::DEC_THREADS * TEAMS), smem, s, 1,
                                      (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,
                                      (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, page_stride,
                                      token_item, positions, block_table, bt_stride, n_heads, n_kv_heads, head_dim,
                                      page_size, window, scale * 1.4426950408889634f, chunk_keys, split_chunks,
                                      n_splits, part_acc, part_ml, counters, status, q_start, kv_len, 1, token_row);
    }
#define PS_DECODE_LAUNCH(KS)                                                                                          \
    {                                                                                                                \
        auto kernel = ps::paged_attention_decode_kernel<KS>;                                                         \
        static size_t raised[ps::MAX_DEVICES] = {0};                                                                 \
        if (!ps::ensure_dynamic_smem((const void*)kernel, smem, raised)) return PS_ERR_LAUNCH;                       \
        return ps::launch_pdl_cluster(kernel, grid, dim3(ps::DEC_THREADS), smem, s, cluster,                         \
                                      (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,             \
                                      (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, page_stride,        \
                                      token_item, positions, block_table, bt_stride, n_heads, n_kv_heads, head_dim,   \
                                      page_size, window, scale * 1.4426950408889634f, chunk_keys, split_chunks,       \
                                      n_splits, part_acc, part_ml, counters, status, q_start, kv_len, cluster,        \
                                      token_row);                                                                     \
    }
    if (head_dim <= 64) PS_DECODE_LAUNCH(4)
    if (head_dim <= 128) PS_DECODE_LAUNCH(8)
    PS_DECODE_LAUNCH(16)
#undef PS_DECODE_LAUNCH
}

PS_EXPORT int ps_paged_attention_decode(const void* q, int q_stride, void* out, int out_stride,
                                        const void* k_pool, const void* v_pool, long long page_stride,
                                        const int* token_item, const int* positions, const int* block_table,
                                        int bt_stride, int T, int n_heads, int n_kv_heads, int head_dim,
                                        int page_size, int window, float scale, int split_tiles, int n_splits,
                                        float* part_acc, float* part_ml, int* counters, void* stream) {
    return launch_attention_decode(q, q_stride, out, out_stride, k_pool, v_pool, page_stride, token_item, positions,
                                   block_table, bt_stride, T, n_heads, n_kv_heads, head_dim, page_size, window, scale,
                                   split_tiles, n_splits, part_acc, part_ml, counters, nullptr, stream);
}

// The same with a device status word that a bounded wait sets when it runs out.
PS_EXPORT int ps_paged_attention_decode_checked(const void* q, int q_stride, void* out, int out_stride,
                                                const void* k_pool, const void* v_pool, long long page_stride,
                                                const int* token_item, const int* positions,
                                                const int* block_table, int bt_stride, int T, int n_heads,
                                                int n_kv_heads, int head_dim, int page_size, int window,
                                                float scale, int split_tiles, int n_splits, float* part_acc,
                                                float* part_ml, int* counters, int* status, void* stream) {
    return launch_attention_decode(q, q_stride, out, out_stride, k_pool, v_pool, page_stride, token_item, positions,
                                   block_table, bt_stride, T, n_heads, n_kv_heads, head_dim, page_size, window, scale,
                                   split_tiles, n_splits, part_acc, part_ml, counters, status, stream);
}

// The general entry. cluster > 1: the n_splits = cluster (2, 4 or 8) splits of a (token, head) are one
// thread-block cluster and merge through shared memory (no scratch needed); cluster <= 1: any n_splits, merged
// through the scratch arrays. q_start / kv_len (per item, may both be null) tell which keys are older than
// this step, so that a first chunk of such keys is fetched before the wait on the kernel before.
// token_row (may be null): the block-table row of each token, where the table is kept by request slot
// instead of by item.
PS_EXPORT int ps_paged_attention_decode_ex(const void* q, int q_stride, void* out, int out_stride,
                                           const void* k_pool, const void* v_pool, long long page_stride,
                                           const int* token_item, const int* token_row, const int* positions,
                                           const int* block_table, int bt_stride, const int* q_start,
                                           const int* kv_len, int T,
                                           int n_heads, int n_kv_heads, int head_dim, int page_size, int window,
                                           float scale, int split_tiles, int n_splits, int cluster,
                                           float* part_acc, float* part_ml, int* counters, int* status,
                                           void* stream) {
    return launch_attention_decode(q, q_stride, out, out_stride, k_pool, v_pool, page_stride, token_item, positions,
                                   block_table, bt_stride, T, n_heads, n_kv_heads, head_dim, page_size, window, scale,
                                   split_tiles, n_splits, part_acc, part_ml, counters, status, stream, q_start, kv_len,
                                   cluster < 1 ? 1 : cluster, token_row);
}

// ------------------------------------------------------------------------------------------------
// The variant that allocates nothing (see attention_decode_noalloc.h for who needs it and the rules).
// ------------------------------------------------------------------------------------------------
#include <stdio.h>

#include "attention_decode_noalloc.h"

// The scratch of the split kernel, inside the library image: counters | (max, sum) pairs | partial
// accumulators. In host code this name is only a stand-in for the symbol; the address a kernel can
// use comes from cudaGetSymbolAddress, looked up once per device below.
static __device__ __align__(256) unsigned char ps_noalloc_scratch[PS_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
void* g_noalloc_base[kMaxDevices] = {nullptr};

int refuse(char* message, int capacity, int code, const char* format, long long a, long long b) {
    if (message && capacity > 0) snprintf(message, (size_t)capacity, format, a, b);
    return code;
}

// Device address of the scratch array for the current device (first call on a device looks it up).
int noalloc_scratch(void** base, char* message, int capacity) {
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess || device < 0 || device >= kMaxDevices)
        return refuse(message, capacity, PS_ERR_SETUP, "cannot identify the current device (cuda error %lld, device %lld)",
                      (long long)err, (long long)device);
    if (!g_noalloc_base[device]) {
        void* ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, ps_noalloc_scratch);
        if (err != cudaSuccess || !ptr)
            return refuse(message, capacity, PS_ERR_SETUP,
                          "cudaGetSymbolAddress failed for the scratch array (cuda error %lld) on device %lld",
                          (long long)err, (long long)device);
        g_noalloc_base[device] = ptr;
    }
    *base = g_noalloc_base[device];
    return PS_OK;
}

}  // namespace

PS_EXPORT int ps_paged_attention_decode_noalloc(const void* q, int q_stride, void* out, int out_stride,
                                                const void* k_pool, const void* v_pool, long long page_stride,
                                                const int* token_item, const int* positions,
                                                const int* block_table, int bt_stride, int T, int n_heads,
                                                int n_kv_heads, int head_dim, int page_size, int window,
                                                float scale, int split_tiles, int n_splits, void* stream,
                                                char* message, int message_capacity) {
    if (message && message_capacity > 0) message[0] = 0;
    if (T <= 0) return PS_OK;
    if (n_heads <= 0 || n_splits < 1)
        return refuse(message, message_capacity, PS_ERR_BAD_ARGUMENT, "n_heads (%lld) and n_splits (%lld) must be positive",
                      n_heads, n_splits);
    const long long rows = (long long)T * n_heads;
    const long long partials = rows * n_splits;
    if (head_dim > PS_NOALLOC_MAX_HEAD_DIM)
        return refuse(message, message_capacity, PS_ERR_SCRATCH_LIMIT,
                      "head_dim %lld exceeds the fixed scratch's limit of %lld", head_dim, PS_NOALLOC_MAX_HEAD_DIM);
    if (rows > PS_NOALLOC_MAX_ROWS)
        return refuse(message, message_capacity, PS_ERR_SCRATCH_LIMIT,
                      "T * n_heads = %lld exceeds the fixed scratch's limit of %lld rows", rows, PS_NOALLOC_MAX_ROWS);
    if (partials > PS_NOALLOC_MAX_PARTIALS)
        return refuse(message, message_capacity, PS_ERR_SCRATCH_LIMIT,
                      "T * n_heads * n_splits = %lld exceeds the fixed scratch's limit of %lld partial states",
                      partials, PS_NOALLOC_MAX_PARTIALS);
    void* base = nullptr;
    int rc = noalloc_scratch(&base, message, message_capacity);
    if (rc != PS_OK) return rc;
    int* counters = reinterpret_cast<int*>(base);
    float* part_ml = reinterpret_cast<float*>(static_cast<unsigned char*>(base) + PS_NOALLOC_MAX_ROWS * 4);
    float* part_acc = part_ml + PS_NOALLOC_MAX_PARTIALS * 2;
    int* status = reinterpret_cast<int*>(static_cast<unsigned char*>(base) + PS_NOALLOC_STATUS_OFFSET);
    // the counters must start at zero whatever an earlier call left behind
    if (cudaMemsetAsync(counters, 0, (size_t)rows * sizeof(int), (cudaStream_t)stream) != cudaSuccess)
        return refuse(message, message_capacity, PS_ERR_LAUNCH, "clearing the counters failed (%lld rows, %lld)", rows, 0);
    rc = ps_paged_attention_decode_checked(q, q_stride, out, out_stride, k_pool, v_pool, page_stride, token_item,
                                           positions, block_table, bt_stride, T, n_heads, n_kv_heads, head_dim,
                                           page_size, window, scale, split_tiles, n_splits, part_acc, part_ml,
                                           counters, status, stream);
    if (rc != PS_OK)
        return refuse(message, message_capacity, rc, "the attention kernel refused its arguments (status %lld, %lld)", rc, 0);
    return PS_OK;
}

PS_EXPORT int ps_paged_attention_decode_noalloc_status(int* value, int clear, void* stream) {
    if (!value) return PS_ERR_BAD_ARGUMENT;
    void* base = nullptr;
    int rc = noalloc_scratch(&base, nullptr, 0);
    if (rc != PS_OK) return rc;
    int* status = reinterpret_cast<int*>(static_cast<unsigned char*>(base) + PS_NOALLOC_STATUS_OFFSET);
    cudaStream_t s = (cudaStream_t)stream;
    if (cudaMemcpyAsync(value, status, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess) return PS_ERR_LAUNCH;
    if (clear && cudaMemsetAsync(status, 0, sizeof(int), s) != cudaSuccess) return PS_ERR_LAUNCH;
    if (cudaStreamSynchronize(s) != cudaSuccess) return PS_ERR_LAUNCH;
    return PS_OK;
}
