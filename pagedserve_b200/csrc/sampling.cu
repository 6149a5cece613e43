// Sampling over float32 logits: greedy argmax and temperature sampling by the Gumbel-max rule.
//
// The reference samples greedily only (argmax on device then a host read:
// src/scheduler/orca_scheduler.py:250). Temperature sampling here draws token
//   argmax_i ( logit_i / T + g_i ),  g_i = -log(-log(u_i)),
// with u_i from a counter-based generator keyed by (seed, position, i): the draw does not
// depend on what else is in the batch or on the order in which rows are processed.
//   key = mix(mix(seed) ^ position);  r = mix(key + i);  u = ((r >> 41) + 0.5) / 2^23
// where mix is the splitmix64 finaliser. Ties go to the lowest index.
#include "common.cuh"

namespace ps {

__host__ __device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__device__ __forceinline__ float gumbel(unsigned long long key, int i) {
    unsigned long long r = mix64(key + (unsigned long long)i);
    float u = ((float)(r >> 41) + 0.5f) * (1.0f / 8388608.0f);
    return -logf(-logf(u));
}

// One row per thread-block cluster of gridDim.z CTAs: each CTA scans its share of the vocabulary, the first
// CTA of the cluster takes the best of the shares out of the others' shared memory (no scratch, no atomics,
// the same result whatever the split). One CTA per row reads a 50,257-wide row through a single SM (11 us
// inside a decode step of batch 8); eight per row bring that to the latency of a few trips.
template <int NT>
__global__ void __launch_bounds__(NT)
sample_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
              const unsigned long long* __restrict__ seed, const int* __restrict__ position, int pos_offset,
              int* __restrict__ out) {
    __shared__ float best_v[NT / 32];
    __shared__ int best_i[NT / 32];
    __shared__ float share_v;
    __shared__ int share_i;
    pdl_prologue();
    logits = pdl_fresh(logits);
    const int r = blockIdx.x, split = blockIdx.z, splits = gridDim.z;
    const float* row = logits + (size_t)r * ld;
    float temp = temperature ? temperature[r] : 0.f;
    unsigned long long key = 0;
    float inv_t = 1.f;
    if (temp > 0.f) {
        key = mix64(mix64(seed[r]) ^ (unsigned long long)(long long)(position[r] + pos_offset));
        inv_t = 1.0f / temp;
    }
    const int share = (V + splits - 1) / splits;
    const int begin = split * share, end = min(V, begin + share);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    auto take = [&](float v, int i) {
        if (temp > 0.f) v = v * inv_t + gumbel(key, i);
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    };
    int i = begin + threadIdx.x;
    constexpr int FLIGHT = 8;                          // loads in flight: a share of a wide row in three trips
    for (; i + (FLIGHT - 1) * NT < end; i += FLIGHT * NT) {
        float v[FLIGHT];
#pragma unroll
        for (int j = 0; j < FLIGHT; ++j) v[j] = row[i + j * NT];
#pragma unroll
        for (int j = 0; j < FLIGHT; ++j) take(v[j], i + j * NT);
    }
    {
        // the rest, again all at once
        float v[FLIGHT];
#pragma unroll
        for (int j = 0; j < FLIGHT; ++j) v[j] = (i + j * NT < end) ? row[i + j * NT] : 0.f;
#pragma unroll
        for (int j = 0; j < FLIGHT; ++j)
            if (i + j * NT < end) take(v[j], i + j * NT);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < NT / 32; ++w)
            if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
        share_v = bv;
        share_i = bi;
    }
    if (splits == 1) {
        if (threadIdx.x == 0) out[r] = (bi == 0x7fffffff) ? 0 : bi;
        return;
    }
    cluster_sync_all();
    if (split == 0 && threadIdx.x == 0) {
        for (int s = 1; s < splits; ++s) {
            const float ov = ld_cluster_f32(&share_v, s);
            const int oi = (int)ld_cluster_u32(&share_i, s);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        out[r] = (bi == 0x7fffffff) ? 0 : bi;
    }
    cluster_sync_all();                                  // the shares stay until they were read
}

}  // namespace ps

// position[r] + pos_offset keys the noise of row r (the index of the token being drawn).
PS_EXPORT int ps_sample(const float* logits, int ld, int R, int V, const float* temperature,
                        const unsigned long long* seed, const int* position, int pos_offset, int* out,
                        void* stream) {
    if (R <= 0) return PS_OK;
    if (V <= 0 || ld < V) return PS_ERR_BAD_ARGUMENT;
    if (R > 65535) return PS_ERR_UNSUPPORTED;
    // a wide vocabulary is shared out over a cluster of 8 CTAs per row (fewer when there are many rows)
    const int splits = V >= 8192 ? (R <= 256 ? 8 : (R <= 1024 ? 4 : 2)) : 1;
    return ps::launch_pdl_cluster(ps::sample_kernel<256>, dim3(R, 1, splits), dim3(256), 0, (cudaStream_t)stream,
                                  splits, logits, ld, V, temperature, seed, position, pos_offset, out);
}
