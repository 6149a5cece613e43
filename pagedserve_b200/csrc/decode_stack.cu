// The whole decode step of a pre-norm attention + MLP stack as ONE persistent kernel.
//
// Why: at batch 1..64 a decode step of a 124M..1.5B model is a chain of ~5 tiny dependent kernels per
// layer. Each costs a launch gap plus several dependent trips to L2 even inside a CUDA graph; measured
// on B200 the 64-kernel step of GPT-2 124M took 440..590 us against 35..55 us of memory time. Here the
// CTAs of one cooperative launch stay resident for the whole step (and for several steps) and move
// from phase to phase through a grid barrier:
//
//   per layer  P1  norm1(h) staged to shared memory -> q|k|v projection (+bias); q to a buffer, k/v into pages
//              P2  split-key paged attention (bulk async copies of K/V chunks), last split merges
//              P3  attention output projection + bias, accumulated into the float32 stream h
//              P4  norm2(h) staged -> up projection + bias + GELU
//              P5  down projection + bias, accumulated into h
//   then       P6  final norm staged -> LM head; logits stored and/or reduced to a per-row best candidate
//              P7  sampled token written, fed back as the next input, positions advanced (device loop)
//
// Products map weight rows to the 16-row side of mma.sync.m16n8k16 and stream the weights to registers
// with 16-byte loads (as csrc/gemm_skinny.cu); a CTA owns a 16-row tile and its 4 warps split K; the
// next phase's weights are prefetched into L2 before the barrier. Every sum runs in a fixed order.
// Math follows the reference's block (src/model/paged_decoder.py:230-252): LayerNorm, packed QKV,
// softmax(q k^T * scale) v over the request's pages, projections with bias, GELU, two residual adds.
//
// The grid barrier and the mbarrier waits are bounded (0.2 s): a wait that runs out sets *status and
// every CTA leaves the kernel.
#include <cooperative_groups.h>

#include "common.cuh"

namespace ps {
namespace stack {

constexpr int THREADS = 128, WARPS = 4;
constexpr uint64_t WAIT_LIMIT_NS = 200ull * 1000 * 1000;

struct LayerWeights {
    const float* ln1_g; const float* ln1_b; const float* ln2_g; const float* ln2_b;
    const __nv_bfloat16* w_qkv; const float* b_qkv;
    const __nv_bfloat16* w_out; const float* b_out;
    const __nv_bfloat16* w_up; const float* b_up;
    const __nv_bfloat16* w_down; const float* b_down;
    __nv_bfloat16* k_pool; __nv_bfloat16* v_pool;
};

struct Params {
    int B, H, n_heads, n_kv_heads, head_dim, I, V, n_layers, page_size, window, act, n_positions;
    int ln_has_mean, stage_in_smem, n_steps, want_logits, do_sample;
    float eps, scale_log2;
    long long page_stride;
    const LayerWeights* layers;
    const __nv_bfloat16* wte; const __nv_bfloat16* wpe; const float* lnf_g; const float* lnf_b;
    const __nv_bfloat16* lm_head;
    int* token_ids; int* positions; int* kv_len; const int* block_table; int bt_stride;
    float* h; __nv_bfloat16* xn; __nv_bfloat16* q; __nv_bfloat16* attn; __nv_bfloat16* inner;
    float* part_acc; float* part_ml; int* counters; int chunk_keys, split_chunks, n_splits;
    float* logits;
    const float* temperature; const unsigned long long* seed;
    unsigned long long* best; int* sampled; int* history; int* step_counter; int max_steps;
    unsigned int* barrier; int* status;
    int skip_mask;        // timing aid: phases whose bit is set do no work (1 norm, 2 qkv, 4 attention, 8 out, 16 up, 32 down, 64 head)
    int ctas_per_sm;      // 0 = as many as fit, up to 3
};

__device__ __forceinline__ uint64_t timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
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
// order-preserving float -> uint, then the lowest index wins ties
__device__ __forceinline__ unsigned long long pack_candidate(float v, int n) {
    unsigned int u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)n);
}

// ---- grid barrier: monotone counter, zeroed by the host before the launch -----------------------
struct GridSync {
    unsigned int* counter;
    unsigned int epoch;
    unsigned int blocks;
    int* status;
    bool ok;
};
__device__ __forceinline__ void grid_barrier(GridSync& g) {
    __syncthreads();
    if (threadIdx.x == 0 && g.ok) {
        // arrivals count on counter[0]; the last arriver publishes the epoch in counter[32] (another
        // 128-byte line), which is all the waiting CTAs read: polls do not queue behind the atomics
        const unsigned int target = (g.epoch + 1) * g.blocks;
        unsigned int old;
        asm volatile("atom.add.release.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(g.counter) : "memory");
        if (old + 1 == target)
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(g.counter + 32), "r"(g.epoch + 1) : "memory");
        const uint64_t start = timer_ns();
        unsigned int seen;
        int spins = 0;
        while (true) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(g.counter + 32) : "memory");
            if (seen >= g.epoch + 1) break;
            if ((++spins & 255) == 0) {
                if (*(volatile int*)g.status != 0 || timer_ns() - start > WAIT_LIMIT_NS) {
                    atomicExch(g.status, 21);
                    g.ok = false;
                    break;
                }
            }
        }
    }
    g.epoch += 1;
    // thread 0's verdict to the whole CTA
    __shared__ int verdict;
    if (threadIdx.x == 0) verdict = g.ok ? 1 : 0;
    __syncthreads();
    g.ok = verdict != 0;
}

// ---- norm of all rows into shared memory (bf16, rows padded by 8 elements) ------------------------
// source: float32 rows of h, or (layer 0) the embedding sum wte[id] + wpe[pos], which CTA 0 also writes to h.
__device__ void stage_norm(const Params& p, const float* gamma, const float* beta, bool from_embedding,
                           __nv_bfloat16* a_s, int lda_s) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int H = p.H;
    for (int m = warp; m < p.B; m += WARPS) {
        const float* hr = p.h + (size_t)m * H;
        const __nv_bfloat16* e = nullptr;
        const __nv_bfloat16* pe = nullptr;
        if (from_embedding) {
            int id = p.token_ids[m], pos = p.positions[m];
            id = min(max(id, 0), p.V - 1);
            pos = min(max(pos, 0), p.n_positions - 1);
            e = p.wte + (size_t)id * H;
            if (p.wpe) pe = p.wpe + (size_t)pos * H;
        }
        float sum = 0.f;
        for (int k = lane; k < H; k += 32) {
            float v = from_embedding ? (__bfloat162float(e[k]) + (pe ? __bfloat162float(pe[k]) : 0.f)) : hr[k];
            sum += v;
        }
        const float mean = p.ln_has_mean ? warp_sum(sum) / (float)H : 0.f;
        float sq = 0.f;
        for (int k = lane; k < H; k += 32) {
            float v = from_embedding ? (__bfloat162float(e[k]) + (pe ? __bfloat162float(pe[k]) : 0.f)) : hr[k];
            float d = v - mean;
            sq += d * d;
        }
        const float rstd = rsqrtf(warp_sum(sq) / (float)H + p.eps);
        for (int k = lane; k < H; k += 32) {
            float v = from_embedding ? (__bfloat162float(e[k]) + (pe ? __bfloat162float(pe[k]) : 0.f)) : hr[k];
            float y = (v - mean) * rstd * gamma[k];
            if (beta) y += beta[k];
            a_s[(size_t)m * lda_s + k] = __float2bfloat16_rn(y);
            if (from_embedding && blockIdx.x == 0) p.h[(size_t)m * H + k] = v;
        }
    }
    __syncthreads();
}

// the same norm written to a global bf16 buffer, rows spread over the CTAs (used when the rows do not fit
// in shared memory); needs a grid barrier afterwards
__device__ void norm_to_global(const Params& p, const float* gamma, const float* beta, bool from_embedding) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int H = p.H;
    for (int m = blockIdx.x * WARPS + warp; m < p.B; m += gridDim.x * WARPS) {
        const float* hr = p.h + (size_t)m * H;
        const __nv_bfloat16* e = nullptr;
        const __nv_bfloat16* pe = nullptr;
        if (from_embedding) {
            int id = min(max(p.token_ids[m], 0), p.V - 1), pos = min(max(p.positions[m], 0), p.n_positions - 1);
            e = p.wte + (size_t)id * H;
            if (p.wpe) pe = p.wpe + (size_t)pos * H;
        }
        float sum = 0.f;
        for (int k = lane; k < H; k += 32)
            sum += from_embedding ? (__bfloat162float(e[k]) + (pe ? __bfloat162float(pe[k]) : 0.f)) : hr[k];
        const float mean = p.ln_has_mean ? warp_sum(sum) / (float)H : 0.f;
        float sq = 0.f;
        for (int k = lane; k < H; k += 32) {
            float v = from_embedding ? (__bfloat162float(e[k]) + (pe ? __bfloat162float(pe[k]) : 0.f)) : hr[k];
            sq += (v - mean) * (v - mean);
        }
        const float rstd = rsqrtf(warp_sum(sq) / (float)H + p.eps);
        for (int k = lane; k < H; k += 32) {
            float v = from_embedding ? (__bfloat162float(e[k]) + (pe ? __bfloat162float(pe[k]) : 0.f)) : hr[k];
            float y = (v - mean) * rstd * gamma[k];
            if (beta) y += beta[k];
            p.xn[(size_t)m * H + k] = __float2bfloat16_rn(y);
            if (from_embedding) p.h[(size_t)m * H + k] = v;
        }
    }
}

// ---- products ---------------------------------------------------------------------------------
enum Epilogue { EPI_QKV = 0, EPI_ACCUMULATE = 1, EPI_ACT = 2, EPI_LOGITS = 3 };

struct Product {
    const __nv_bfloat16* a;   // activations [B, K]: shared or global memory (generic address)
    int lda;
    const __nv_bfloat16* w;   // [N, K]
    const float* bias;
    int N, K;
    int epilogue;
    // outputs
    float* out_f32; __nv_bfloat16* out_bf16; int ldo;
    __nv_bfloat16* k_pool; __nv_bfloat16* v_pool;     // EPI_QKV
};

__device__ __forceinline__ void prefetch_tiles(const __nv_bfloat16* w, int N, int K) {
    // the 16-row tiles this CTA will own in the coming product: one prefetch per 128-byte line
    const int tiles = (N + 15) >> 4;
    const int lines_per_row = (K * 2 + 127) >> 7;
    int done = 0;
    for (int tile = blockIdx.x; tile < tiles && done < 2; tile += gridDim.x, ++done) {   // two tiles are enough
        const int rows = min(16, N - tile * 16);
        for (int i = threadIdx.x; i < rows * lines_per_row; i += THREADS) {
            int r = i / lines_per_row, l = i - r * lines_per_row;
            prefetch_l2(reinterpret_cast<const char*>(w + (size_t)(tile * 16 + r) * K) + (size_t)l * 128);
        }
    }
}

template <int MT>
__device__ void run_product(const Params& p, const Product& g, float* red, unsigned long long* cta_best) {
    constexpr int TOK = 8 * MT;
    constexpr int UNROLL = 6;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gq = lane >> 2, t = lane & 3;
    const int steps = (g.K + 31) >> 5;
    const int tiles = (g.N + 15) >> 4;
    bool aok[MT];
    const __nv_bfloat16* arow[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        int m = 8 * mt + gq;
        aok[mt] = m < p.B;
        arow[mt] = g.a + (size_t)(aok[mt] ? m : 0) * g.lda + 8 * t;
    }
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int n0 = tile * 16;
        const int r0 = min(n0 + gq, g.N - 1), r1 = min(n0 + gq + 8, g.N - 1);
        const __nv_bfloat16* w0 = g.w + (size_t)r0 * g.K + 8 * t;
        const __nv_bfloat16* w1 = g.w + (size_t)r1 * g.K + 8 * t;
        float acc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) { acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f; }
        for (int s0 = warp; s0 < steps; s0 += WARPS * UNROLL) {
            uint4 wa[UNROLL], wb[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                int k = (s0 + u * WARPS) << 5;
                bool ok = (s0 + u * WARPS) < steps && (k + 8 * t) < g.K;
                wa[u] = ok ? ldg_stream16(w0 + k) : make_uint4(0, 0, 0, 0);
                wb[u] = ok ? ldg_stream16(w1 + k) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                int k = (s0 + u * WARPS) << 5;
                bool ok = (s0 + u * WARPS) < steps && (k + 8 * t) < g.K;
                if (!ok) continue;
                uint32_t a1[4] = {wa[u].x, wb[u].x, wa[u].y, wb[u].y};
                uint32_t a2[4] = {wa[u].z, wb[u].z, wa[u].w, wb[u].w};
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    uint4 x = aok[mt] ? *reinterpret_cast<const uint4*>(arow[mt] + k) : make_uint4(0, 0, 0, 0);
                    uint32_t b1[2] = {x.x, x.y}, b2[2] = {x.z, x.w};
                    mma16816(acc[mt], a1, b1);
                    mma16816(acc[mt], a2, b2);
                }
            }
        }
        float* mine = red + (size_t)warp * 16 * TOK;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            int c = 8 * mt + 2 * t;
            mine[gq * TOK + c] = acc[mt][0];
            mine[gq * TOK + c + 1] = acc[mt][1];
            mine[(gq + 8) * TOK + c] = acc[mt][2];
            mine[(gq + 8) * TOK + c + 1] = acc[mt][3];
        }
        __syncthreads();
        for (int e = threadIdx.x; e < 16 * TOK; e += THREADS) {
            const int r = e & 15, m = e >> 4;
            const int n = n0 + r;
            const bool live = m < p.B && n < g.N;
            float v = 0.f;
            if (live) {
                v = (red[r * TOK + m] + red[16 * TOK + r * TOK + m]) +
                    (red[2 * 16 * TOK + r * TOK + m] + red[3 * 16 * TOK + r * TOK + m]);
                if (g.bias) v += g.bias[n];
            }
            if (g.epilogue == EPI_QKV) {
                if (!live) continue;
                const int q_width = p.n_heads * p.head_dim, kv_width = p.n_kv_heads * p.head_dim;
                if (n < q_width) {
                    g.out_bf16[(size_t)m * g.ldo + n] = __float2bfloat16_rn(v);
                } else {
                    int c = n - q_width;
                    __nv_bfloat16* pool = g.k_pool;
                    if (c >= kv_width) { c -= kv_width; pool = g.v_pool; }
                    const int head = c / p.head_dim, d = c - head * p.head_dim;
                    const int pos = p.positions[m];
                    const int page = p.block_table[(size_t)m * p.bt_stride + pos / p.page_size];
                    if (page >= 0)
                        pool[(size_t)page * p.page_stride +
                             ((size_t)head * p.page_size + (pos % p.page_size)) * p.head_dim + d] = __float2bfloat16_rn(v);
                }
            } else if (g.epilogue == EPI_ACCUMULATE) {
                if (live) g.out_f32[(size_t)m * g.ldo + n] += v;
            } else if (g.epilogue == EPI_ACT) {
                if (live) g.out_bf16[(size_t)m * g.ldo + n] = __float2bfloat16_rn(apply_act(v, p.act));
            } else {
                if (live && p.want_logits) g.out_f32[(size_t)m * g.ldo + n] = v;
                if (p.do_sample) {
                    // candidate of this column for row m; the 16 columns of a row sit in 16 neighbouring lanes
                    unsigned long long cand = 0;
                    if (live) {
                        float score = v;
                        const float temp = p.temperature[m];
                        if (temp > 0.f) {
                            const unsigned long long key =
                                mix64(mix64(p.seed[m]) ^ (unsigned long long)(long long)(p.positions[m] + 1));
                            score = v * (1.0f / temp) + gumbel(key, n);
                        }
                        cand = pack_candidate(score, n);
                    }
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) {
                        unsigned long long other = __shfl_xor_sync(0xffffffffu, cand, o);
                        cand = other > cand ? other : cand;
                    }
                    if (r == 0 && m < p.B && cand > cta_best[m]) cta_best[m] = cand;   // one writer per m
                }
            }
        }
        __syncthreads();
    }
}

// ---- attention over the pages: items (token, head, split) spread over the CTAs ------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = timer_ns();
    while (true) {
        for (int spin = 0; spin < 64; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (timer_ns() - start > WAIT_LIMIT_NS) return false;
    }
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ float ldcg_f32(const float* q) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(q));
    return v;
}

__device__ void run_attention(const Params& p, const LayerWeights& lw, unsigned char* smem, uint64_t* bar,
                              uint32_t& phase, bool& ok) {
    const int hd = p.head_dim, chunk_keys = p.chunk_keys;
    __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem);
    __nv_bfloat16* v_s = k_s + (size_t)chunk_keys * hd;
    float* q_s = reinterpret_cast<float*>(v_s + (size_t)chunk_keys * hd);
    float* p_s = q_s + hd;
    float* acc_s = p_s + chunk_keys;
    __shared__ float red_a[WARPS], red_b[WARPS];
    __shared__ int last_flag;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int items = p.B * p.n_heads * p.n_splits;
    const int row_chunks = hd >> 3;
    const int pages_per_chunk = chunk_keys / p.page_size;
    const uint32_t block_bytes = (uint32_t)p.page_size * hd * 2;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int split = item % p.n_splits;
        const int h = (item / p.n_splits) % p.n_heads;
        const int b = item / (p.n_splits * p.n_heads);
        const int pos = p.positions[b];
        const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
        const int first_chunk = lo / chunk_keys, last_chunk = pos / chunk_keys;
        const int first_split = first_chunk / p.split_chunks, last_split = last_chunk / p.split_chunks;
        if (split < first_split || split > last_split) continue;
        const int n_active = last_split - first_split + 1;
        const int chunk_lo = max(first_chunk, split * p.split_chunks);
        const int chunk_hi = min(last_chunk, (split + 1) * p.split_chunks - 1);
        const int g = h / (p.n_heads / p.n_kv_heads);
        const int* bt = p.block_table + (size_t)b * p.bt_stride;
        const int q_width = p.n_heads * hd;
        for (int d = tid; d < hd; d += THREADS)
            q_s[d] = __bfloat162float(p.q[(size_t)b * q_width + h * hd + d]) * p.scale_log2;
        __syncthreads();
        float acc[4][2];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;
        for (int chunk = chunk_lo; chunk <= chunk_hi; ++chunk) {
            const int key0 = chunk * chunk_keys;
            const int pg_first = max(lo, key0) / p.page_size - key0 / p.page_size;
            const int pg_last = min(pos, key0 + chunk_keys - 1) / p.page_size - key0 / p.page_size;
            if (tid == 0) mbar_expect_tx(bar, 2u * block_bytes * (uint32_t)(pg_last - pg_first + 1));
            if (tid >= pg_first && tid <= pg_last && tid < pages_per_chunk) {
                const int page = bt[key0 / p.page_size + tid];
                const long long base = (long long)page * p.page_stride + (long long)g * p.page_size * hd;
                bulk_copy_g2s(k_s + (size_t)tid * p.page_size * hd, lw.k_pool + base, block_bytes, bar);
                bulk_copy_g2s(v_s + (size_t)tid * p.page_size * hd, lw.v_pool + base, block_bytes, bar);
            }
            if (ok && !mbar_wait_bounded(bar, phase)) {
                ok = false;
                atomicExch(p.status, 22);
            }
            phase ^= 1;
            const int kpos = key0 + tid;
            const bool valid = ok && tid < chunk_keys && kpos >= lo && kpos <= pos;
            float s = -INFINITY;
            if (valid) {
                const __nv_bfloat16* kr = k_s + (size_t)tid * hd;
                float dot = 0.f;
                const int rot = tid % row_chunks;
                for (int c = 0; c < row_chunks; ++c) {
                    int cc = c + rot;
                    if (cc >= row_chunks) cc -= row_chunks;
                    const uint4 kv = *reinterpret_cast<const uint4*>(kr + 8 * cc);
                    const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kv);
                    const float4 qa = *reinterpret_cast<const float4*>(q_s + 8 * cc);
                    const float4 qb = *reinterpret_cast<const float4*>(q_s + 8 * cc + 4);
                    float2 f0 = __bfloat1622float2(k2[0]), f1 = __bfloat1622float2(k2[1]);
                    float2 f2 = __bfloat1622float2(k2[2]), f3 = __bfloat1622float2(k2[3]);
                    dot = fmaf(qa.x, f0.x, dot); dot = fmaf(qa.y, f0.y, dot);
                    dot = fmaf(qa.z, f1.x, dot); dot = fmaf(qa.w, f1.y, dot);
                    dot = fmaf(qb.x, f2.x, dot); dot = fmaf(qb.y, f2.y, dot);
                    dot = fmaf(qb.z, f3.x, dot); dot = fmaf(qb.w, f3.y, dot);
                }
                s = dot;
            }
            float wmax = warp_max(s);
            if (lane == 0) red_a[warp] = wmax;
            __syncthreads();
            const float cmax = fmaxf(fmaxf(red_a[0], red_a[1]), fmaxf(red_a[2], red_a[3]));
            const float m_new = fmaxf(m_run, cmax);
            const float pr = valid ? exp2f(s - m_new) : 0.f;
            if (tid < chunk_keys) p_s[tid] = pr;
            float wsum = warp_sum(pr);
            if (lane == 0) red_b[warp] = wsum;
            __syncthreads();
            const float csum = (red_b[0] + red_b[1]) + (red_b[2] + red_b[3]);
            const float corr = (m_new == -INFINITY) ? 1.f : exp2f(m_run - m_new);
            l_run = l_run * corr + csum;
            m_run = m_new;
#pragma unroll
            for (int i = 0; i < 4; ++i) { acc[i][0] *= corr; acc[i][1] *= corr; }
            const int j_lo = max(lo, key0) - key0, j_hi = min(pos, key0 + chunk_keys - 1) - key0;
            int j = j_lo + ((warp - j_lo) & (WARPS - 1));
            if (ok)
                for (; j <= j_hi; j += WARPS) {
                    const float pj = p_s[j];
                    const __nv_bfloat162* vr = reinterpret_cast<const __nv_bfloat162*>(v_s + (size_t)j * hd);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        int d2 = lane + 32 * i;
                        if (2 * d2 < hd) {
                            float2 v = __bfloat1622float2(vr[d2]);
                            acc[i][0] = fmaf(pj, v.x, acc[i][0]);
                            acc[i][1] = fmaf(pj, v.y, acc[i][1]);
                        }
                    }
                }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int d = 2 * (lane + 32 * i);
            if (d < hd) {
                acc_s[warp * hd + d] = acc[i][0];
                acc_s[warp * hd + d + 1] = acc[i][1];
            }
        }
        __syncthreads();
        __nv_bfloat16* orow = p.attn + (size_t)b * q_width + h * hd;
        if (p.n_splits == 1 || n_active == 1) {
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            for (int d = tid; d < hd; d += THREADS)
                orow[d] = __float2bfloat16_rn(((acc_s[d] + acc_s[hd + d]) + (acc_s[2 * hd + d] + acc_s[3 * hd + d])) * inv);
            __syncthreads();
            continue;
        }
        const size_t slot = ((size_t)b * p.n_heads + h) * p.n_splits + split;
        for (int d = tid; d < hd; d += THREADS)
            p.part_acc[slot * hd + d] = (acc_s[d] + acc_s[hd + d]) + (acc_s[2 * hd + d] + acc_s[3 * hd + d]);
        if (tid == 0) { p.part_ml[slot * 2] = m_run; p.part_ml[slot * 2 + 1] = l_run; }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            int prev = atomicAdd(&p.counters[b * p.n_heads + h], 1);
            last_flag = (prev == n_active - 1);
            if (last_flag) p.counters[b * p.n_heads + h] = 0;
        }
        __syncthreads();
        if (last_flag) {
            __threadfence();
            const size_t base = ((size_t)b * p.n_heads + h) * p.n_splits;
            float M = -INFINITY;
            for (int s2 = first_split; s2 <= last_split; ++s2) M = fmaxf(M, ldcg_f32(p.part_ml + (base + s2) * 2));
            float L = 0.f;
            for (int s2 = first_split; s2 <= last_split; ++s2)
                L += ldcg_f32(p.part_ml + (base + s2) * 2 + 1) * exp2f(ldcg_f32(p.part_ml + (base + s2) * 2) - M);
            const float inv = L > 0.f ? 1.f / L : 0.f;
            for (int d = tid; d < hd; d += THREADS) {
                float o = 0.f;
                for (int s2 = first_split; s2 <= last_split; ++s2)
                    o += ldcg_f32(p.part_acc + (base + s2) * hd + d) * exp2f(ldcg_f32(p.part_ml + (base + s2) * 2) - M);
                orow[d] = __float2bfloat16_rn(o * inv);
            }
        }
        __syncthreads();
    }
}

// ---- the kernel -------------------------------------------------------------------------------
template <int MT>
__global__ void __launch_bounds__(THREADS, 3) decode_stack_kernel(const Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    // shared memory: [ attention buffers | staged activations ] and the cross-warp reduction area after them
    __shared__ __align__(8) uint64_t bar;
    __shared__ unsigned long long cta_best[8 * MT];
    constexpr int TOK = 8 * MT;
    const int lda_s = p.H + 8;
    const size_t stage_bytes = p.stage_in_smem ? (size_t)TOK * lda_s * 2 : 0;
    const size_t attn_bytes = (size_t)p.chunk_keys * p.head_dim * 4 + (size_t)(p.head_dim + p.chunk_keys + WARPS * p.head_dim) * 4;
    const size_t area = ((stage_bytes > attn_bytes ? stage_bytes : attn_bytes) + 127) & ~(size_t)127;
    __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(smem);
    float* red = reinterpret_cast<float*>(smem + area);

    GridSync sync{p.barrier, 0u, gridDim.x, p.status, true};
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < TOK; i += THREADS) cta_best[i] = 0ull;
    if (p.stage_in_smem)   // rows beyond the batch stay zero for good
        for (int i = threadIdx.x; i < TOK * lda_s / 2; i += THREADS) reinterpret_cast<uint32_t*>(a_s)[i] = 0u;
    __syncthreads();
    uint32_t phase = 0;
    bool attn_ok = true;
    const int q_width = p.n_heads * p.head_dim, kv_width = p.n_kv_heads * p.head_dim;

    for (int step = 0; step < p.n_steps && sync.ok; ++step) {
        for (int l = 0; l < p.n_layers && sync.ok; ++l) {
            const LayerWeights& lw = p.layers[l];
            // P1: norm1 -> q|k|v
            Product g{};
            if (p.stage_in_smem) {
                if (!(p.skip_mask & 1)) stage_norm(p, lw.ln1_g, lw.ln1_b, l == 0, a_s, lda_s);
                g.a = a_s; g.lda = lda_s;
            } else {
                norm_to_global(p, lw.ln1_g, lw.ln1_b, l == 0);
                grid_barrier(sync);
                g.a = p.xn; g.lda = p.H;
            }
            g.w = lw.w_qkv; g.bias = lw.b_qkv; g.N = q_width + 2 * kv_width; g.K = p.H; g.epilogue = EPI_QKV;
            g.out_bf16 = p.q; g.ldo = q_width; g.k_pool = lw.k_pool; g.v_pool = lw.v_pool;
            if (!(p.skip_mask & 2)) run_product<MT>(p, g, red, cta_best);
            prefetch_tiles(lw.w_out, p.H, q_width);
            grid_barrier(sync);
            // P2: attention
            if (!(p.skip_mask & 4)) run_attention(p, lw, smem, &bar, phase, attn_ok);
            grid_barrier(sync);
            // P3: output projection into the stream
            g = Product{};
            g.a = p.attn; g.lda = q_width; g.w = lw.w_out; g.bias = lw.b_out; g.N = p.H; g.K = q_width;
            g.epilogue = EPI_ACCUMULATE; g.out_f32 = p.h; g.ldo = p.H;
            if (!(p.skip_mask & 8)) run_product<MT>(p, g, red, cta_best);
            prefetch_tiles(lw.w_up, p.I, p.H);
            grid_barrier(sync);
            // P4: norm2 -> up projection + GELU
            g = Product{};
            if (p.stage_in_smem) {
                if (!(p.skip_mask & 1)) stage_norm(p, lw.ln2_g, lw.ln2_b, false, a_s, lda_s);
                g.a = a_s; g.lda = lda_s;
            } else {
                norm_to_global(p, lw.ln2_g, lw.ln2_b, false);
                grid_barrier(sync);
                g.a = p.xn; g.lda = p.H;
            }
            g.w = lw.w_up; g.bias = lw.b_up; g.N = p.I; g.K = p.H; g.epilogue = EPI_ACT; g.out_bf16 = p.inner; g.ldo = p.I;
            if (!(p.skip_mask & 16)) run_product<MT>(p, g, red, cta_best);
            prefetch_tiles(lw.w_down, p.H, p.I);
            grid_barrier(sync);
            // P5: down projection into the stream
            g = Product{};
            g.a = p.inner; g.lda = p.I; g.w = lw.w_down; g.bias = lw.b_down; g.N = p.H; g.K = p.I;
            g.epilogue = EPI_ACCUMULATE; g.out_f32 = p.h; g.ldo = p.H;
            if (!(p.skip_mask & 32)) run_product<MT>(p, g, red, cta_best);
            if (l + 1 < p.n_layers) prefetch_tiles(p.layers[l + 1].w_qkv, q_width + 2 * kv_width, p.H);
            else prefetch_tiles(p.lm_head, p.V, p.H);
            grid_barrier(sync);
        }
        // P6: final norm -> LM head
        Product g{};
        if (p.stage_in_smem) {
            stage_norm(p, p.lnf_g, p.lnf_b, p.n_layers == 0, a_s, lda_s);
            g.a = a_s; g.lda = lda_s;
        } else {
            norm_to_global(p, p.lnf_g, p.lnf_b, p.n_layers == 0);
            grid_barrier(sync);
            g.a = p.xn; g.lda = p.H;
        }
        g.w = p.lm_head; g.bias = nullptr; g.N = p.V; g.K = p.H; g.epilogue = EPI_LOGITS; g.out_f32 = p.logits; g.ldo = p.V;
        if (!(p.skip_mask & 64)) run_product<MT>(p, g, red, cta_best);
        if (p.do_sample) {
            for (int m = threadIdx.x; m < p.B; m += THREADS) {
                if (cta_best[m]) atomicMax(&p.best[m], cta_best[m]);
                cta_best[m] = 0ull;
            }
        }
        if (p.n_layers > 0) prefetch_tiles(p.layers[0].w_qkv, q_width + 2 * kv_width, p.H);
        grid_barrier(sync);
        // P7: the winners become the next inputs
        if (p.do_sample) {
            if (blockIdx.x == 0) {
                const int at = *p.step_counter;
                for (int m = threadIdx.x; m < p.B; m += THREADS) {
                    const unsigned long long won = p.best[m];
                    const int token = (int)(0xFFFFFFFFu - (unsigned int)(won & 0xFFFFFFFFull));
                    p.best[m] = 0ull;
                    p.sampled[m] = token;
                    p.token_ids[m] = token;
                    p.positions[m] += 1;
                    p.kv_len[m] += 1;
                    if (at < p.max_steps) p.history[(size_t)at * p.B + m] = token;
                }
                __syncthreads();
                if (threadIdx.x == 0) *p.step_counter = at + 1;
            }
            if (step + 1 < p.n_steps) grid_barrier(sync);
        }
    }
    if (!attn_ok && threadIdx.x == 0) atomicExch(p.status, 22);
}

template <int MT>
int launch(const Params& p, int sm_limit, cudaStream_t stream) {
    auto kernel = decode_stack_kernel<MT>;
    constexpr int TOK = 8 * MT;
    const size_t stage_bytes = p.stage_in_smem ? (size_t)TOK * (p.H + 8) * 2 : 0;
    const size_t attn_bytes = (size_t)p.chunk_keys * p.head_dim * 4 + (size_t)(p.head_dim + p.chunk_keys + WARPS * p.head_dim) * 4;
    const size_t area = ((stage_bytes > attn_bytes ? stage_bytes : attn_bytes) + 127) & ~(size_t)127;
    const size_t smem = area + (size_t)WARPS * 16 * TOK * 4;
    static size_t raised = 0;
    if (smem > 48 * 1024 && smem > raised) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return PS_ERR_LAUNCH;
        raised = smem;
    }
    int device = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, smem) != cudaSuccess || per_sm < 1)
        return PS_ERR_LAUNCH;
    if (per_sm > 3) per_sm = 3;
    if (p.ctas_per_sm > 0 && p.ctas_per_sm < per_sm) per_sm = p.ctas_per_sm;
    if (sm_limit > 0 && sm_limit < sms) sms = sm_limit;
    dim3 grid(sms * per_sm);
    if (cudaMemsetAsync(p.barrier, 0, 64 * sizeof(unsigned int), stream) != cudaSuccess) return PS_ERR_LAUNCH;
    void* args[] = {const_cast<Params*>(&p)};
    cudaError_t e = cudaLaunchCooperativeKernel((void*)kernel, grid, dim3(THREADS), args, smem, stream);
    return e == cudaSuccess ? PS_OK : PS_ERR_LAUNCH;
}

}  // namespace stack
}  // namespace ps

// sizeof the two structs, so that the Python side can check its mirror of the layout
PS_EXPORT int ps_decode_stack_sizes(int* layer_bytes, int* params_bytes) {
    *layer_bytes = (int)sizeof(ps::stack::LayerWeights);
    *params_bytes = (int)sizeof(ps::stack::Params);
    return PS_OK;
}

// params: host pointer to a Params struct (device pointers inside). B <= 64.
PS_EXPORT int ps_decode_stack(const void* params, int sm_limit, void* stream) {
    const ps::stack::Params& p = *reinterpret_cast<const ps::stack::Params*>(params);
    if (p.B <= 0 || p.n_steps <= 0) return PS_OK;
    if (p.B > 64) return PS_ERR_UNSUPPORTED;
    if (p.H % 8 != 0 || p.I % 8 != 0 || p.head_dim % 16 != 0 || p.head_dim > 256) return PS_ERR_UNSUPPORTED;
    if (p.n_heads % p.n_kv_heads != 0 || p.page_size <= 0 || (p.page_size & (p.page_size - 1)) || p.page_size > 64)
        return PS_ERR_UNSUPPORTED;
    if (p.chunk_keys % p.page_size != 0 || p.chunk_keys > ps::stack::THREADS) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (p.B <= 8) return ps::stack::launch<1>(p, sm_limit, s);
    if (p.B <= 16) return ps::stack::launch<2>(p, sm_limit, s);
    if (p.B <= 32) return ps::stack::launch<4>(p, sm_limit, s);
    return ps::stack::launch<8>(p, sm_limit, s);
}
