// Paged attention for few query tokens (decode steps and short portions), bfloat16, split along keys.
//
// One CTA per (token, head, key split). The reference launches one program per (request, head) that
// walks the whole context (src/kernels/triton_paged_attention.py:225-320, grid at :530): at batch 1
// that is 12 programs for 148 SMs. Here the keys of a token are cut into splits of `split_tiles`
// tiles of 32 keys, aligned to absolute positions; every split is a CTA of 4 warps, the warps take
// the split's tiles in turn, and the last CTA of a (token, head) to finish merges the partial
// (max, sum, acc) states in split order. With one split the output is written directly.
//
// Inside a tile lane j owns key j for the scores (its whole K row, 16-byte loads, no shuffles in the
// dot product), then lanes own head dims for p.V (coalesced 4-byte loads, p broadcast by shuffle).
// Softmax state and accumulators are float32 (reference: triton_paged_attention.py:219-223, 275-320).
//
// Scratch (only when splits > 1): part_acc[T][H][S][hd] f32, part_ml[T][H][S][2] f32, counters[T*H] int32
// (zero before the first use; the merging CTA sets its counter back to zero).
#include "common.cuh"

namespace ps {

constexpr int DEC_WARPS = 4;

__device__ __forceinline__ float ldcg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                              __nv_bfloat16* __restrict__ out, int out_stride,
                              const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                              long long page_stride, const int* __restrict__ token_item,
                              const int* __restrict__ positions, const int* __restrict__ block_table,
                              int bt_stride, int n_heads, int n_kv_heads, int head_dim, int page_size,
                              int window, float scale_log2, int split_tiles, int n_splits,
                              float* __restrict__ part_acc, float* __restrict__ part_ml,
                              int* __restrict__ counters) {
    extern __shared__ float smem[];
    float* q_s = smem;                       // [head_dim]
    float* acc_s = smem + head_dim;          // [DEC_WARPS][head_dim]
    __shared__ float m_s[DEC_WARPS], l_s[DEC_WARPS];
    __shared__ int last_flag;

    const int t = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p = positions[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int first_tile = lo >> 5, last_tile = p >> 5;
    const int first_split = first_tile / split_tiles, last_split = last_tile / split_tiles;
    if (split < first_split || split > last_split) return;          // no keys here
    const int n_active = last_split - first_split + 1;
    const int tile_lo = max(first_tile, split * split_tiles);
    const int tile_hi = min(last_tile, (split + 1) * split_tiles - 1);

    const int g = h / (n_heads / n_kv_heads);
    const int* bt = block_table + (size_t)token_item[t] * bt_stride;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x)
        q_s[d] = __bfloat162float(q[(size_t)t * q_stride + h * head_dim + d]) * scale_log2;
    __syncthreads();

    float acc[4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int chunks = head_dim >> 3;

    for (int tile = tile_lo + warp; tile <= tile_hi; tile += DEC_WARPS) {
        const int kpos = (tile << 5) + lane;
        const bool valid = kpos >= lo && kpos <= p;
        long long row = 0;
        float s = -INFINITY;
        if (valid) {
            int page = bt[kpos / page_size];
            row = (long long)page * page_stride + ((long long)g * page_size + (kpos % page_size)) * head_dim;
            const uint4* kr = reinterpret_cast<const uint4*>(k_pool + row);
            float dot = 0.f;
#pragma unroll 4
            for (int c = 0; c < chunks; ++c) {
                uint4 kv = kr[c];
                const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kv);
                const float4 qa = *reinterpret_cast<const float4*>(q_s + 8 * c);
                const float4 qb = *reinterpret_cast<const float4*>(q_s + 8 * c + 4);
                float2 f0 = __bfloat1622float2(k2[0]), f1 = __bfloat1622float2(k2[1]);
                float2 f2 = __bfloat1622float2(k2[2]), f3 = __bfloat1622float2(k2[3]);
                dot = fmaf(qa.x, f0.x, dot); dot = fmaf(qa.y, f0.y, dot);
                dot = fmaf(qa.z, f1.x, dot); dot = fmaf(qa.w, f1.y, dot);
                dot = fmaf(qb.x, f2.x, dot); dot = fmaf(qb.y, f2.y, dot);
                dot = fmaf(qb.z, f3.x, dot); dot = fmaf(qb.w, f3.y, dot);
            }
            s = dot;                                   // already in log2 units
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = exp2f(m - m_new);
        const float pr = valid ? exp2f(s - m_new) : 0.f;
        l = l * corr + warp_sum(pr);
#pragma unroll
        for (int i = 0; i < 4; ++i) { acc[i][0] *= corr; acc[i][1] *= corr; }
        m = m_new;
        const unsigned mask = __ballot_sync(0xffffffffu, valid);
        const int first = __ffs(mask) - 1, count = __popc(mask);      // valid keys are one contiguous run
#pragma unroll 8
        for (int j = first; j < first + count; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            const long long rj = __shfl_sync(0xffffffffu, row, j);
            const __nv_bfloat162* vr = reinterpret_cast<const __nv_bfloat162*>(v_pool + rj);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int d2 = lane + 32 * i;                // index of the bf16 pair
                if (2 * d2 < head_dim) {
                    float2 v = __bfloat1622float2(vr[d2]);
                    acc[i][0] = fmaf(pj, v.x, acc[i][0]);
                    acc[i][1] = fmaf(pj, v.y, acc[i][1]);
                }
            }
        }
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int d = 2 * (lane + 32 * i);
        if (d < head_dim) {
            acc_s[warp * head_dim + d] = acc[i][0];
            acc_s[warp * head_dim + d + 1] = acc[i][1];
        }
    }
    __syncthreads();
    float big = m_s[0];
#pragma unroll
    for (int w = 1; w < DEC_WARPS; ++w) big = fmaxf(big, m_s[w]);
    float wgt[DEC_WARPS];
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
        wgt[w] = (m_s[w] == -INFINITY) ? 0.f : exp2f(m_s[w] - big);
        total += l_s[w] * wgt[w];
    }
    if (n_splits == 1 || n_active == 1) {
        const float inv = 1.f / total;
        for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; ++w) o += acc_s[w * head_dim + d] * wgt[w];
            out[(size_t)t * out_stride + h * head_dim + d] = __float2bfloat16_rn(o * inv);
        }
        return;
    }
    // several splits hold keys of this token: publish the partial state
    const size_t slot = ((size_t)t * n_heads + h) * n_splits + split;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) o += acc_s[w * head_dim + d] * wgt[w];
        part_acc[slot * head_dim + d] = o;
    }
    if (threadIdx.x == 0) { part_ml[slot * 2] = big; part_ml[slot * 2 + 1] = total; }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int prev = atomicAdd(&counters[t * n_heads + h], 1);
        last_flag = (prev == n_active - 1);
        if (last_flag) counters[t * n_heads + h] = 0;
    }
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    const size_t base = ((size_t)t * n_heads + h) * n_splits;
    float M = -INFINITY;
    for (int sidx = first_split; sidx <= last_split; ++sidx) M = fmaxf(M, ldcg_f32(part_ml + (base + sidx) * 2));
    float L = 0.f;
    for (int sidx = first_split; sidx <= last_split; ++sidx)
        L += ldcg_f32(part_ml + (base + sidx) * 2 + 1) * exp2f(ldcg_f32(part_ml + (base + sidx) * 2) - M);
    const float inv = 1.f / L;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float o = 0.f;
        for (int sidx = first_split; sidx <= last_split; ++sidx)
            o += ldcg_f32(part_acc + (base + sidx) * head_dim + d) * exp2f(ldcg_f32(part_ml + (base + sidx) * 2) - M);
        out[(size_t)t * out_stride + h * head_dim + d] = __float2bfloat16_rn(o * inv);
    }
}

}  // namespace ps

// split_tiles: tiles of 32 keys per split; n_splits: grid depth = ceil(max tiles / split_tiles).
// With n_splits == 1 the scratch pointers may be null.
PS_EXPORT int ps_paged_attention_decode(const void* q, int q_stride, void* out, int out_stride,
                                        const void* k_pool, const void* v_pool, long long page_stride,
                                        const int* token_item, const int* positions, const int* block_table,
                                        int bt_stride, int T, int n_heads, int n_kv_heads, int head_dim,
                                        int page_size, int window, float scale, int split_tiles, int n_splits,
                                        float* part_acc, float* part_ml, int* counters, void* stream) {
    if (T <= 0) return PS_OK;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return PS_ERR_BAD_ARGUMENT;
    if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 256) return PS_ERR_UNSUPPORTED;
    if (page_size <= 0 || page_size > 64 || (page_size & (page_size - 1))) return PS_ERR_UNSUPPORTED;
    if (n_heads > 65535 || n_splits > 65535 || n_splits < 1 || split_tiles < 1) return PS_ERR_UNSUPPORTED;
    if (n_splits > 1 && (!part_acc || !part_ml || !counters)) return PS_ERR_BAD_ARGUMENT;
    if (q_stride % 8 != 0 || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) || page_stride % 8 != 0)
        return PS_ERR_UNSUPPORTED;
    dim3 grid(T, n_heads, n_splits);
    size_t smem = (size_t)(1 + ps::DEC_WARPS) * head_dim * sizeof(float);
    ps::paged_attention_decode_kernel<<<grid, ps::DEC_WARPS * 32, smem, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,
        (const __nv_bfloat16*)v_pool, page_stride, token_item, positions, block_table, bt_stride, n_heads,
        n_kv_heads, head_dim, page_size, window, scale * 1.4426950408889634f, split_tiles, n_splits, part_acc,
        part_ml, counters);
    return ps::launch_status();
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
    // the counters must start at zero whatever an earlier call left behind
    if (cudaMemsetAsync(counters, 0, (size_t)rows * sizeof(int), (cudaStream_t)stream) != cudaSuccess)
        return refuse(message, message_capacity, PS_ERR_LAUNCH, "clearing the counters failed (%lld rows, %lld)", rows, 0);
    rc = ps_paged_attention_decode(q, q_stride, out, out_stride, k_pool, v_pool, page_stride, token_item, positions,
                                   block_table, bt_stride, T, n_heads, n_kv_heads, head_dim, page_size, window,
                                   scale, split_tiles, n_splits, part_acc, part_ml, counters, stream);
    if (rc != PS_OK)
        return refuse(message, message_capacity, rc, "the attention kernel refused its arguments (status %lld, %lld)", rc, 0);
    return PS_OK;
}
