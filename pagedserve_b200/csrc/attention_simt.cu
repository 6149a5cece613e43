// Paged KV append and a general paged causal attention on CUDA cores.
//
// Cache layout of one cache layer: page p, kv head g, in-page offset o, dim d at
//   pool[p * page_stride + (g * page_size + o) * head_dim + d]
// (the reference keeps [layers, blocks, heads, block, head_dim] pools:
//  src/model/kv_manager.py:77-86).
//
// attention: one CTA per (token, head). A token at position p of its request attends
// keys max(0, p-window+1) .. p read from the request's pages through the block table;
// it makes no difference whether the token is a decode token or part of a prompt
// portion, so a position's result does not depend on how the prompt was cut.
// token_item[t] is the row of block_table that holds the pages of token t's request: the
// request's slot where the table is kept by slot, the token's item where it is built per step.
//   s = (q.k) * scale, softmax in float32, o = p.v
//   (reference: src/model/paged_attention.py:262-295; src/kernels/triton_paged_attention.py:219-331)
// Keys are visited in tiles of 32 aligned to absolute positions; warp w takes tiles with
// tile % 4 == w; the four partial (max, sum, acc) states are merged in warp order. The
// order of every sum therefore depends only on p.
#include "common.cuh"

namespace ps {

template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k_src, const T* __restrict__ v_src, int src_stride,
                                 const int* __restrict__ token_item, const int* __restrict__ positions,
                                 const int* __restrict__ block_table, int bt_stride,
                                 T* __restrict__ k_pool, T* __restrict__ v_pool, long long page_stride,
                                 int n_kv_heads, int head_dim, int page_size) {
    pdl_prologue();
    k_src = pdl_fresh(k_src);
    v_src = pdl_fresh(v_src);
    int t = blockIdx.x;
    int item = token_item[t];
    int p = positions[t];
    int page = block_table[(size_t)item * bt_stride + p / page_size];
    if (page < 0) return;
    int off = p % page_size;
    int width = n_kv_heads * head_dim;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        int g = c / head_dim, d = c - g * head_dim;
        size_t dst = (size_t)page * page_stride + ((size_t)g * page_size + off) * head_dim + d;
        k_pool[dst] = k_src[(size_t)t * src_stride + c];
        v_pool[dst] = v_src[(size_t)t * src_stride + c];
    }
}

// The same copy in 16-byte pieces: thread = (token, k or v, piece).
template <typename T>
__global__ void __launch_bounds__(256)
kv_append_vec_kernel(const T* __restrict__ k_src, const T* __restrict__ v_src, int src_stride,
                     const int* __restrict__ token_item, const int* __restrict__ positions,
                     const int* __restrict__ block_table, int bt_stride, T* __restrict__ k_pool,
                     T* __restrict__ v_pool, long long page_stride, int T_tokens, int n_kv_heads, int head_dim,
                     int page_size) {
    pdl_prologue();
    k_src = pdl_fresh(k_src);
    v_src = pdl_fresh(v_src);
    constexpr int PER = 16 / sizeof(T);                       // elements per piece
    const int pieces = n_kv_heads * head_dim / PER;           // per token and tensor
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)T_tokens * 2 * pieces) return;
    const int piece = (int)(idx % pieces);
    const int which = (int)((idx / pieces) & 1);
    const int t = (int)(idx / (2 * pieces));
    const int p = positions[t];
    const int page = block_table[(size_t)token_item[t] * bt_stride + p / page_size];
    if (page < 0) return;
    const int c = piece * PER, g = c / head_dim, d = c - g * head_dim;
    const size_t dst = (size_t)page * page_stride + ((size_t)g * page_size + (p % page_size)) * head_dim + d;
    const T* src = (which ? v_src : k_src) + (size_t)t * src_stride + c;
    T* pool = which ? v_pool : k_pool;
    *reinterpret_cast<uint4*>(pool + dst) = *reinterpret_cast<const uint4*>(src);
}

template <typename T>
int launch_kv_append(const void* k_src, const void* v_src, int src_stride, const int* token_item,
                     const int* positions, const int* block_table, int bt_stride, void* k_pool, void* v_pool,
                     long long page_stride, int T_tokens, int n_kv_heads, int head_dim, int page_size,
                     cudaStream_t s) {
    constexpr int PER = 16 / sizeof(T);
    const bool aligned = (((uintptr_t)k_src | (uintptr_t)v_src | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0 &&
                         src_stride % PER == 0 && page_stride % PER == 0 && head_dim % PER == 0;
    if (aligned) {
        long long total = (long long)T_tokens * 2 * (n_kv_heads * head_dim / PER);
        return launch_pdl(kv_append_vec_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s,
                          (const T*)k_src, (const T*)v_src, src_stride, token_item, positions, block_table, bt_stride,
                          (T*)k_pool, (T*)v_pool, page_stride, T_tokens, n_kv_heads, head_dim, page_size);
    }
    int nt = n_kv_heads * head_dim >= 256 ? 256 : 128;
    return launch_pdl(kv_append_kernel<T>, dim3(T_tokens), dim3(nt), 0, s, (const T*)k_src, (const T*)v_src, src_stride,
                      token_item, positions, block_table, bt_stride, (T*)k_pool, (T*)v_pool, page_stride, n_kv_heads,
                      head_dim, page_size);
}

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_HD = 256;

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_simt_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                            const T* __restrict__ k_pool, const T* __restrict__ v_pool, long long page_stride,
                            const int* __restrict__ token_item, const int* __restrict__ positions,
                            const int* __restrict__ block_table, int bt_stride,
                            int n_heads, int n_kv_heads, int head_dim, int page_size, int window, float scale) {
    extern __shared__ float smem[];
    float* q_s = smem;                                   // [head_dim]
    float* acc_s = smem + head_dim;                      // [ATT_WARPS][head_dim]
    __shared__ float m_s[ATT_WARPS], l_s[ATT_WARPS];

    pdl_prologue();
    q = pdl_fresh(q);
    k_pool = pdl_fresh(k_pool);
    v_pool = pdl_fresh(v_pool);
    int t = blockIdx.x, h = blockIdx.y;
    int g = h / (n_heads / n_kv_heads);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int item = token_item[t];
    int p = positions[t];
    const int* bt = block_table + (size_t)item * bt_stride;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x)
        q_s[d] = to_float(q[(size_t)t * q_stride + h * head_dim + d]);
    __syncthreads();

    int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    int first_tile = lo >> 5, last_tile = p >> 5;
    constexpr int NACC = ATT_MAX_HD / 32;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int tile = first_tile + ((warp - first_tile) & (ATT_WARPS - 1)); tile <= last_tile; tile += ATT_WARPS) {
        int kpos = (tile << 5) + lane;
        bool valid = kpos >= lo && kpos <= p;
        long long row = 0;
        float s = -INFINITY;
        if (valid) {
            int page = bt[kpos / page_size];
            row = (long long)page * page_stride + ((long long)g * page_size + (kpos % page_size)) * head_dim;
            const T* kr = k_pool + row;
            float dot = 0.f;
            for (int d = 0; d < head_dim; ++d) dot = fmaf(q_s[d], to_float(kr[d]), dot);
            s = dot * scale;
        }
        float m_new = fmaxf(m, warp_max(s));
        float corr = expf(m - m_new);          // m == -inf on the first tile -> 0
        float pr = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(pr);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= corr;
        m = m_new;
        unsigned mask = __ballot_sync(0xffffffffu, valid);
        for (int j = 0; j < 32; ++j) {
            if (!((mask >> j) & 1u)) continue;
            float pj = __shfl_sync(0xffffffffu, pr, j);
            long long rj = __shfl_sync(0xffffffffu, row, j);
            const T* vr = v_pool + rj;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
            }
        }
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        int d = lane + 32 * i;
        if (d < head_dim) acc_s[warp * head_dim + d] = acc[i];
    }
    __syncthreads();
    float big = m_s[0];
#pragma unroll
    for (int w = 1; w < ATT_WARPS; ++w) big = fmaxf(big, m_s[w]);
    float total = 0.f;
    float wgt[ATT_WARPS];
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
        wgt[w] = (m_s[w] == -INFINITY) ? 0.f : expf(m_s[w] - big);
        total += l_s[w] * wgt[w];
    }
    float inv = 1.f / total;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) o += acc_s[w * head_dim + d] * wgt[w];
        out[(size_t)t * out_stride + h * head_dim + d] = from_float<T>(o * inv);
    }
}

}  // namespace ps

static int check_attention_sizes(int n_heads, int n_kv_heads, int head_dim, int page_size) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return PS_ERR_BAD_ARGUMENT;
    if (head_dim <= 0 || head_dim > ps::ATT_MAX_HD) return PS_ERR_UNSUPPORTED;      // any head size up to the limit
    if (page_size <= 0 || page_size > 64 || (page_size & (page_size - 1))) return PS_ERR_UNSUPPORTED;
    return PS_OK;
}

PS_EXPORT int ps_kv_append(const void* k_src, const void* v_src, int src_stride, const int* token_item,
                           const int* positions, const int* block_table, int bt_stride, void* k_pool,
                           void* v_pool, long long page_stride, int T, int n_kv_heads, int head_dim,
                           int page_size, int dtype, void* stream) {
    if (T <= 0) return PS_OK;
    int rc = check_attention_sizes(n_kv_heads, n_kv_heads, head_dim, page_size);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PS_F32)
        return ps::launch_kv_append<float>(k_src, v_src, src_stride, token_item, positions, block_table, bt_stride,
                                           k_pool, v_pool, page_stride, T, n_kv_heads, head_dim, page_size, s);
    if (dtype == PS_BF16)
        return ps::launch_kv_append<__nv_bfloat16>(k_src, v_src, src_stride, token_item, positions, block_table,
                                                   bt_stride, k_pool, v_pool, page_stride, T, n_kv_heads, head_dim,
                                                   page_size, s);
    return PS_ERR_UNSUPPORTED;
}

PS_EXPORT int ps_paged_attention_simt(const void* q, int q_stride, void* out, int out_stride,
                                      const void* k_pool, const void* v_pool, long long page_stride,
                                      const int* token_item, const int* positions, const int* block_table,
                                      int bt_stride, int T, int n_heads, int n_kv_heads, int head_dim,
                                      int page_size, int window, float scale, int dtype, void* stream) {
    if (T <= 0) return PS_OK;
    int rc = check_attention_sizes(n_heads, n_kv_heads, head_dim, page_size);
    if (rc) return rc;
    if (n_heads > 65535) return PS_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, n_heads);
    size_t smem = (size_t)(1 + ps::ATT_WARPS) * head_dim * sizeof(float);
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::paged_attention_simt_kernel<float>, grid, dim3(ps::ATT_WARPS * 32), smem, s,
                              (const float*)q, q_stride, (float*)out, out_stride, (const float*)k_pool,
                              (const float*)v_pool, page_stride, token_item, positions, block_table, bt_stride,
                              n_heads, n_kv_heads, head_dim, page_size, window, scale);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::paged_attention_simt_kernel<__nv_bfloat16>, grid, dim3(ps::ATT_WARPS * 32), smem, s,
                              (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,
                              (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, page_stride, token_item,
                              positions, block_table, bt_stride, n_heads, n_kv_heads, head_dim, page_size, window,
                              scale);
    return PS_ERR_UNSUPPORTED;
}
