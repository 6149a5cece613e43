// Causal attention of prompt portions over the paged cache on tensor cores (bfloat16).
//
// One CTA (8 warps = two groups of 4) per (block of 64 query tokens of one request, head). Both groups hold the
// same 64 queries (16 rows per warp); group 0 walks the even key tiles, group 1 the odd ones, each with its own
// double-buffered K/V tiles and its own named barrier; at the end group 0 merges the two (max, sum, O) states.
// This halves the chain of dependent MMAs of the longest CTA (the last query block of a long prompt). The step's keys and values are
// already in the pages, so the kernel reads every key, old or new, through the block table: a portion
// that continues a cached prompt needs no gather (the reference concatenates gathered past K/V and
// materialises the scores: src/model/paged_attention.py:262-295, 396-420), and fresh prompts need no
// grouping by length (:356-394).
//   S = Q K^T and O += P V with mma.sync.m16n8k16 (bf16 in, float32 accumulate); each warp owns 16 query rows;
//   key tiles of 64 keys aligned to absolute positions, double-buffered in shared memory with cp.async;
//   online softmax in float32 with exp2 (scores pre-scaled by scale * log2 e);
//   masks: key_pos > query_pos, key_pos <= query_pos - window, rows beyond the portion.
// Rows of shared memory are padded by 16 bytes, which keeps ldmatrix free of bank conflicts for every
// head size that is a multiple of 16.
#include "common.cuh"

namespace ps {
namespace pf {

constexpr int BQ = 64, BKEY = 64, GROUP = 128, THREADS = 256;   // 2 groups x 4 warps x 16 query rows

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    int bytes = valid ? 16 : 0;                       // 0: fill the 16 bytes with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void group_sync(int group) {           // barrier of one 128-thread group
    asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(GROUP) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(THREADS)
prefill_attention_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                         int out_stride, const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, long long page_stride,
                         const int* __restrict__ q_start, const int* __restrict__ kv_len,
                         const int* __restrict__ block_table, int bt_stride, const int* __restrict__ item_row,
                         int first_item, int n_items, int n_heads, int n_kv_heads, int page_size, int window,
                         float scale_log2) {
    constexpr int RS = HD + 8;                         // padded row, in elements
    constexpr int CH = HD / 8;                         // 16-byte pieces of a row
    constexpr int KS = HD / 16;                        // k steps over the head dim
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [BQ][RS]
    const int wg = threadIdx.x >> 7;                                           // warp group 0 / 1
    __nv_bfloat16* k_s = q_s + BQ * RS + wg * (4 * BKEY * RS);                 // this group's [2][BKEY][RS]
    __nv_bfloat16* v_s = k_s + 2 * BKEY * RS;                                  // this group's [2][BKEY][RS]

    pdl_prologue();
    q = pdl_fresh(q);
    k_pool = pdl_fresh(k_pool);
    v_pool = pdl_fresh(v_pool);
    // which (item, query block) is this CTA?
    int block = blockIdx.x, item = -1, qb = 0;
    for (int i = first_item; i < first_item + n_items; ++i) {
        int blocks = (q_start[i + 1] - q_start[i] + BQ - 1) / BQ;
        if (block < blocks) { item = i; qb = blocks - 1 - block; break; }   // late blocks see most keys: first
        block -= blocks;
    }
    if (item < 0) return;
    const int h = blockIdx.y, g = h / (n_heads / n_kv_heads);
    const int tid = threadIdx.x & (GROUP - 1), lane = tid & 31, warp = tid >> 5;   // within the group
    const int qs = q_start[item], q_len = q_start[item + 1] - qs;
    const int pos0 = kv_len[item] - q_len + qb * BQ;              // position of the block's first query
    const int rows = min(BQ, q_len - qb * BQ);                    // valid query rows of the block
    const int tok0 = qs + qb * BQ;
    const int hi = pos0 + rows - 1;                                // last key any row may see
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int kb_first = lo / BKEY, kb_last = hi / BKEY;
    // the item's block-table row: item_row[item] where the table is kept by request slot, else the item itself
    const int* bt = block_table + (size_t)(item_row ? item_row[item] : item) * bt_stride;

    // ---- Q tile
    for (int c = threadIdx.x; c < BQ * CH; c += THREADS) {
        int r = c / CH, piece = c % CH;
        bool ok = r < rows;
        const __nv_bfloat16* src = q + (size_t)(tok0 + (ok ? r : 0)) * q_stride + h * HD + piece * 8;
        cp_async16(q_s + r * RS + piece * 8, src, ok);
    }
    auto load_kv = [&](int kb, int buf) {
        const int key0 = kb * BKEY;
        for (int c = tid; c < BKEY * CH; c += GROUP) {
            int r = c / CH, piece = c % CH;
            int key = key0 + r;
            bool ok = key <= hi && key >= lo;
            long long off = 0;
            if (ok) {
                int page = bt[key / page_size];
                off = (long long)page * page_stride + ((long long)g * page_size + (key % page_size)) * HD + piece * 8;
            }
            cp_async16(k_s + (buf * BKEY + r) * RS + piece * 8, k_pool + off, ok);
            cp_async16(v_s + (buf * BKEY + r) * RS + piece * 8, v_pool + off, ok);
        }
    };
    if (kb_first + wg <= kb_last) load_kv(kb_first + wg, 0);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();                                   // the Q tile (loaded by all 256 threads) is in place

    uint32_t qf[KS][4];
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int gq = lane >> 2, tq = lane & 3;
    const int row0 = warp * 16 + gq, row1 = row0 + 8;            // the two query rows of this thread
    const int pos_r0 = pos0 + row0, pos_r1 = pos0 + row1;

#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
        ldmatrix_x4(qf[ks], q_s + (warp * 16 + (lane & 15)) * RS + (ks * 2 + (lane >> 4)) * 8);
    for (int kb = kb_first + wg; kb <= kb_last; kb += 2) {
        const int buf = ((kb - kb_first) >> 1) & 1;
        if (kb + 2 <= kb_last) load_kv(kb + 2, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        group_sync(wg);
        // ---- S = Q K^T for 16 rows x 64 keys
        float s[BKEY / 8][4];
#pragma unroll
        for (int nt = 0; nt < BKEY / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
        const __nv_bfloat16* kbuf = k_s + buf * BKEY * RS;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int nt = 0; nt < BKEY / 8; nt += 2) {
                uint32_t b[4];
                ldmatrix_x4(b, kbuf + (8 * (nt + (lane >> 4)) + (lane & 7)) * RS + (ks * 2 + ((lane >> 3) & 1)) * 8);
                mma16816(s[nt], qf[ks], b[0], b[1]);
                mma16816(s[nt + 1], qf[ks], b[2], b[3]);
            }
        }
        // ---- scale, mask, online softmax
        const int key0 = kb * BKEY;
        const bool need_mask = (key0 + BKEY - 1 > pos0) || (window > 0 && key0 < pos0 + rows - 1 - window + 1) ||
                               rows < BQ;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < BKEY / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[nt][e] * scale_log2;
                if (need_mask) {
                    int key = key0 + nt * 8 + tq * 2 + (e & 1);
                    int pos = (e < 2) ? pos_r0 : pos_r1;
                    int row = (e < 2) ? row0 : row1;
                    bool ok = key <= pos && row < rows && (window <= 0 || key > pos - window);
                    if (!ok) v = -INFINITY;
                }
                s[nt][e] = v;
            }
            mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        const float base0 = (mn0 == -INFINITY) ? 0.f : mn0, base1 = (mn1 == -INFINITY) ? 0.f : mn1;
        const float corr0 = exp2f(m_run[0] - base0), corr1 = exp2f(m_run[1] - base1);
        m_run[0] = mn0; m_run[1] = mn1;
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < BKEY / 8; ++nt) {
            s[nt][0] = exp2f(s[nt][0] - base0); s[nt][1] = exp2f(s[nt][1] - base0);
            s[nt][2] = exp2f(s[nt][2] - base1); s[nt][3] = exp2f(s[nt][3] - base1);
            sum0 += s[nt][0] + s[nt][1];
            sum1 += s[nt][2] + s[nt][3];
        }
        l_run[0] = l_run[0] * corr0 + sum0;
        l_run[1] = l_run[1] * corr1 + sum1;
#pragma unroll
        for (int dn = 0; dn < HD / 8; ++dn) {
            o[dn][0] *= corr0; o[dn][1] *= corr0; o[dn][2] *= corr1; o[dn][3] *= corr1;
        }
        // ---- O += P V
        const __nv_bfloat16* vbuf = v_s + buf * BKEY * RS;
#pragma unroll
        for (int kk = 0; kk < BKEY / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dn = 0; dn < HD / 8; dn += 2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vbuf + (16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8) * RS + (dn + (lane >> 4)) * 8);
                mma16816(o[dn], a, b[0], b[1]);
                mma16816(o[dn + 1], a, b[2], b[3]);
            }
        }
        group_sync(wg);                                // this buffer is refilled two iterations on
    }
    cp_async_wait<0>();
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
    // ---- merge the two groups: group 1 hands its state over through its (now free) K/V buffers
    __syncthreads();
    float* o1 = reinterpret_cast<float*>(q_s + BQ * RS + 4 * BKEY * RS);       // [BQ][HD] of group 1
    float* ml1 = o1 + BQ * HD;                                                  // [BQ][2]
    if (wg == 1) {
#pragma unroll
        for (int dn = 0; dn < HD / 8; ++dn) {
            const int d = dn * 8 + tq * 2;
            *reinterpret_cast<float2*>(o1 + row0 * HD + d) = make_float2(o[dn][0], o[dn][1]);
            *reinterpret_cast<float2*>(o1 + row1 * HD + d) = make_float2(o[dn][2], o[dn][3]);
        }
        if (tq == 0) {
            ml1[2 * row0] = m_run[0]; ml1[2 * row0 + 1] = l_run[0];
            ml1[2 * row1] = m_run[1]; ml1[2 * row1 + 1] = l_run[1];
        }
    }
    __syncthreads();
    if (wg == 1) return;
    {
        const float ma = ml1[2 * row0], la = ml1[2 * row0 + 1], mb = ml1[2 * row1], lb = ml1[2 * row1 + 1];
        const float n0 = fmaxf(m_run[0], ma), n1 = fmaxf(m_run[1], mb);
        const float b0 = (n0 == -INFINITY) ? 0.f : n0, b1 = (n1 == -INFINITY) ? 0.f : n1;
        const float s0 = exp2f(m_run[0] - b0), t0 = exp2f(ma - b0), s1 = exp2f(m_run[1] - b1), t1 = exp2f(mb - b1);
        l_run[0] = l_run[0] * s0 + la * t0;
        l_run[1] = l_run[1] * s1 + lb * t1;
#pragma unroll
        for (int dn = 0; dn < HD / 8; ++dn) {
            const int d = dn * 8 + tq * 2;
            const float2 pa = *reinterpret_cast<const float2*>(o1 + row0 * HD + d);
            const float2 pb = *reinterpret_cast<const float2*>(o1 + row1 * HD + d);
            o[dn][0] = o[dn][0] * s0 + pa.x * t0; o[dn][1] = o[dn][1] * s0 + pa.y * t0;
            o[dn][2] = o[dn][2] * s1 + pb.x * t1; o[dn][3] = o[dn][3] * s1 + pb.y * t1;
        }
    }
    // ---- normalise and store
    const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
    for (int dn = 0; dn < HD / 8; ++dn) {
        const int d = dn * 8 + tq * 2;
        if (row0 < rows)
            *reinterpret_cast<uint32_t*>(out + (size_t)(tok0 + row0) * out_stride + h * HD + d) =
                pack_bf16(o[dn][0] * inv0, o[dn][1] * inv0);
        if (row1 < rows)
            *reinterpret_cast<uint32_t*>(out + (size_t)(tok0 + row1) * out_stride + h * HD + d) =
                pack_bf16(o[dn][2] * inv1, o[dn][3] * inv1);
    }
}

template <int HD>
int launch(const void* q, int q_stride, void* out, int out_stride, const void* k_pool, const void* v_pool,
           long long page_stride, const int* q_start, const int* kv_len, const int* block_table, int bt_stride,
           const int* item_row, int first_item, int n_items, int max_blocks, int n_heads, int n_kv_heads,
           int page_size, int window, float scale, cudaStream_t stream) {
    constexpr int RS = HD + 8;
    size_t smem = (size_t)(BQ + 8 * BKEY) * RS * 2;
    auto kernel = prefill_attention_kernel<HD>;
    static size_t raised[MAX_DEVICES] = {0};
    if (!ensure_dynamic_smem((const void*)kernel, smem, raised)) return PS_ERR_LAUNCH;
    return launch_pdl(kernel, dim3(max_blocks, n_heads), dim3(THREADS), smem, stream, (const __nv_bfloat16*)q, q_stride,
                      (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
                      page_stride, q_start, kv_len, block_table, bt_stride, item_row, first_item, n_items, n_heads,
                      n_kv_heads, page_size, window, scale * 1.4426950408889634f);
}

}  // namespace pf
}  // namespace ps

// Attention for items [first_item, first_item + n_items) of the step. q_start[i] is the flat index of item
// i's first token, kv_len[i] its length after the step. max_blocks >= sum over items of ceil(q_len / 64).
// q and out point at row 0 of the step's flat token arrays. Head sizes: multiples of 16 up to 128.
// item_row (may be null): the block-table row of each item, where the table is kept by request slot.
PS_EXPORT int ps_prefill_attention(const void* q, int q_stride, void* out, int out_stride, const void* k_pool,
                                   const void* v_pool, long long page_stride, const int* q_start, const int* kv_len,
                                   const int* block_table, int bt_stride, const int* item_row, int first_item,
                                   int n_items,
                                   int max_blocks, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                   int window, float scale, void* stream) {
    if (n_items <= 0 || max_blocks <= 0) return PS_OK;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads > 65535) return PS_ERR_BAD_ARGUMENT;
    if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 128) return PS_ERR_UNSUPPORTED;
    if (page_size <= 0 || page_size > 64 || (page_size & (page_size - 1))) return PS_ERR_UNSUPPORTED;
    if (q_stride % 8 != 0 || out_stride % 2 != 0 || page_stride % 8 != 0) return PS_ERR_UNSUPPORTED;
    if (((uintptr_t)q & 15) || ((uintptr_t)out & 3) || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15))
        return PS_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
#define PS_PF_CASE(D)                                                                                              \
    case D:                                                                                                        \
        return ps::pf::launch<D>(q, q_stride, out, out_stride, k_pool, v_pool, page_stride, q_start, kv_len,       \
                                 block_table, bt_stride, item_row, first_item, n_items, max_blocks, n_heads,       \
                                 n_kv_heads, page_size, window, scale, s);
    switch (head_dim) {
        PS_PF_CASE(16) PS_PF_CASE(32) PS_PF_CASE(48) PS_PF_CASE(64)
        PS_PF_CASE(80) PS_PF_CASE(96) PS_PF_CASE(112) PS_PF_CASE(128)
    }
#undef PS_PF_CASE
    return PS_ERR_UNSUPPORTED;
}
