// Embedding gather (token table + optional learned position table) and LayerNorm.
//
// The residual stream is float32 in every mode: the sum of the two embeddings,
// every residual add and all norm statistics are 32-bit.
//   embedding : h[t] = wte[id_t] + wpe[pos_t]      (reference: src/model/paged_decoder.py:306-314)
//   layernorm : (x-mean)/sqrt(var+eps)*g+b, biased variance, two passes over registers
//               (reference: src/kernels/triton_residual_layernorm.py:25-40)
#include "common.cuh"

namespace ps {

template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ pos,
                             const T* __restrict__ wte, const T* __restrict__ wpe,
                             float* __restrict__ out, int H, int V, int P, int* __restrict__ status) {
    pdl_prologue();
    ids = pdl_fresh(ids);
    pos = pdl_fresh(pos);
    int t = blockIdx.x;
    int id = ids[t];
    int p = pos ? pos[t] : 0;
    bool bad = (id < 0 || id >= V) || (wpe && (p < 0 || p >= P));
    if (bad) {
        if (threadIdx.x == 0 && status) atomicExch(status, 1);
        for (int c = threadIdx.x; c < H; c += blockDim.x) out[(size_t)t * H + c] = 0.f;
        return;
    }
    const T* e = wte + (size_t)id * H;
    const T* q = wpe ? wpe + (size_t)p * H : nullptr;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = to_float(e[c]);
        if (q) v += to_float(q[c]);
        out[(size_t)t * H + c] = v;
    }
}

// One CTA per row. Row kept in registers when H <= NT*MAXV, else re-read.
template <typename TOut, int NT>
__global__ void layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 float eps, TOut* __restrict__ out, int H, int has_mean) {
    __shared__ float red[NT / 32];
    __shared__ float bcast;
    pdl_prologue();
    x = pdl_fresh(x);
    int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    const float* xr = x + (size_t)src * H;
    constexpr int MAXV = 8;
    float vals[MAXV];
    float sum = 0.f;
    bool in_regs = H <= NT * MAXV;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        int c = threadIdx.x + i * NT;
        vals[i] = (in_regs && c < H) ? xr[c] : 0.f;
        sum += vals[i];
    }
    if (!in_regs) {
        sum = 0.f;
        for (int c = threadIdx.x; c < H; c += NT) sum += xr[c];
    }
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float mean = 0.f;
    if (has_mean) {
        sum = warp_sum(sum);
        if (lane == 0) red[warp] = sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            float s = 0.f;
            for (int w = 0; w < NT / 32; ++w) s += red[w];
            bcast = s * (1.0f / (float)H);
        }
        __syncthreads();
        mean = bcast;
        __syncthreads();
    }
    float sq = 0.f;
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            int c = threadIdx.x + i * NT;
            float d = (c < H) ? vals[i] - mean : 0.f;
            sq += d * d;
        }
    } else {
        for (int c = threadIdx.x; c < H; c += NT) {
            float d = xr[c] - mean;
            sq += d * d;
        }
    }
    sq = warp_sum(sq);
    if (lane == 0) red[warp] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int w = 0; w < NT / 32; ++w) s += red[w];
        bcast = rsqrtf(s * (1.0f / (float)H) + eps);
    }
    __syncthreads();
    float rstd = bcast;
    TOut* o = out + (size_t)r * H;
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            int c = threadIdx.x + i * NT;
            if (c < H) {
                float v = (vals[i] - mean) * rstd * gamma[c];
                if (beta) v += beta[c];
                o[c] = from_float<TOut>(v);
            }
        }
    } else {
        for (int c = threadIdx.x; c < H; c += NT) {
            float v = (xr[c] - mean) * rstd * gamma[c];
            if (beta) v += beta[c];
            o[c] = from_float<TOut>(v);
        }
    }
}

// Many rows (prefill): one warp per row, the row held in registers (H <= 32 * 4 * WMAX), float4 loads,
// no shared memory and no block-wide barrier. Same two-pass statistics as above.
template <typename TOut, int WMAX>
__global__ void __launch_bounds__(256)
layernorm_warp_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ gamma,
                      const float* __restrict__ beta, float eps, TOut* __restrict__ out, int n_rows, int H,
                      int has_mean) {
    // the norm's scale and shift are weights: they are fetched before the wait on the kernel that writes x
    const int lane = threadIdx.x & 31;
    const int quads = H >> 2;
    const float inv_h = 1.0f / (float)H;          // the division, before the wait
    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    const float4* b4 = reinterpret_cast<const float4*>(beta);
    float4 g[WMAX], b[WMAX];
#pragma unroll
    for (int i = 0; i < WMAX; ++i) {
        const int c = lane + 32 * i;
        g[i] = c < quads ? g4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        b[i] = (beta && c < quads) ? b4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_prologue();
    x = pdl_fresh(x);
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * H);
    float4 v[WMAX];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < WMAX; ++i) {
        int c = lane + 32 * i;
        v[i] = c < quads ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = has_mean ? warp_sum(sum) * inv_h : 0.f;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < WMAX; ++i) {
        if (lane + 32 * i < quads) {
            float a = v[i].x - mean, b2 = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
            sq += (a * a + b2 * b2) + (c * c + d * d);
        }
    }
    const float rstd = rsqrtf(warp_sum(sq) * inv_h + eps);
    TOut* o = out + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < WMAX; ++i) {
        int c = lane + 32 * i;
        if (c < quads) {
            float y0 = (v[i].x - mean) * rstd * g[i].x + b[i].x, y1 = (v[i].y - mean) * rstd * g[i].y + b[i].y;
            float y2 = (v[i].z - mean) * rstd * g[i].z + b[i].z, y3 = (v[i].w - mean) * rstd * g[i].w + b[i].w;
            if constexpr (sizeof(TOut) == 2) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
                uint2 pack = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                *reinterpret_cast<uint2*>(o + 4 * c) = pack;
            } else {
                *reinterpret_cast<float4*>(o + 4 * c) = make_float4(y0, y1, y2, y3);
            }
        }
    }
}

template <typename TOut>
int launch_layernorm(const float* x, const int* rows, int n_rows, int H, const float* gamma, const float* beta,
                     float eps, int has_mean, TOut* out, cudaStream_t s) {
    const bool aligned = H % 4 == 0 && (((uintptr_t)x | (uintptr_t)gamma | (uintptr_t)beta | (uintptr_t)out) & 15) == 0;
    // Which kernel runs depends on the width and the alignment alone, never on the number of rows: a row's
    // result is the same bits whatever else is in the batch.
    if (aligned && H <= 32 * 4 * 16) {
        // a few dozen rows (a decode step): two rows per CTA, so that the rows spread over many SMs and each
        // warp's trips to memory are short; many rows (a prompt): eight per CTA
        const int warps = n_rows <= 256 ? 2 : 8;
        dim3 grid((n_rows + warps - 1) / warps), block(32 * warps);
        if (H <= 32 * 4 * 8)
            return launch_pdl(layernorm_warp_kernel<TOut, 8>, grid, block, 0, s, x, rows, gamma, beta, eps, out,
                              n_rows, H, has_mean);
        return launch_pdl(layernorm_warp_kernel<TOut, 16>, grid, block, 0, s, x, rows, gamma, beta, eps, out,
                          n_rows, H, has_mean);
    }
    return launch_pdl(layernorm_kernel<TOut, 256>, dim3(n_rows), dim3(256), 0, s, x, rows, gamma, beta, eps, out, H,
                      has_mean);
}

}  // namespace ps

PS_EXPORT int ps_embed(const int* ids, const int* pos, const void* wte, const void* wpe, float* out,
                       int T, int H, int V, int P, int dtype, int* status, void* stream) {
    if (T <= 0) return PS_OK;
    if (H <= 0 || V <= 0) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    int nt = H >= 256 ? 256 : 128;
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::embed_kernel<float>, dim3(T), dim3(nt), 0, s, ids, pos, (const float*)wte,
                              (const float*)wpe, out, H, V, P, status);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::embed_kernel<__nv_bfloat16>, dim3(T), dim3(nt), 0, s, ids, pos,
                              (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, out, H, V, P, status);
    return PS_ERR_UNSUPPORTED;
}

// out[r] = norm(x[rows ? rows[r] : r]); has_mean = 0 gives the RMS form; beta may be null.
PS_EXPORT int ps_layernorm(const float* x, const int* rows, int n_rows, int H, const float* gamma,
                           const float* beta, float eps, int has_mean, void* out, int out_dtype,
                           void* stream) {
    if (n_rows <= 0) return PS_OK;
    if (H <= 0) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == PS_F32)
        return ps::launch_layernorm<float>(x, rows, n_rows, H, gamma, beta, eps, has_mean, (float*)out, s);
    if (out_dtype == PS_BF16)
        return ps::launch_layernorm<__nv_bfloat16>(x, rows, n_rows, H, gamma, beta, eps, has_mean,
                                                   (__nv_bfloat16*)out, s);
    return PS_ERR_UNSUPPORTED;
}
