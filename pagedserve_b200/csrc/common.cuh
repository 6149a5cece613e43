// Shared helpers for the sm_100a kernels of pagedserve_b200.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstring>
#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include <stdint.h>
#include <stdlib.h>

#define PS_OK 0
#define PS_ERR_BAD_ARGUMENT 1
#define PS_ERR_UNSUPPORTED 2
#define PS_ERR_LAUNCH 3

// dtype codes shared with the Python side
#define PS_F32 0
#define PS_BF16 1

// activation codes
#define PS_ACT_NONE 0
#define PS_ACT_GELU_TANH 1
#define PS_ACT_GELU_ERF 2

#define PS_EXPORT extern "C" __attribute__((visibility("default")))

namespace ps {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
__device__ __forceinline__ float gelu_tanh(float x) {
    const float k = 0.7978845608028654f;
    float inner = k * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(inner));
}
// 0.5 x (1 + erf(x / sqrt 2))
__device__ __forceinline__ float gelu_erf(float x) {
    return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
}
__device__ __forceinline__ float apply_act(float x, int act) {
    if (act == PS_ACT_GELU_TANH) return gelu_tanh(x);
    if (act == PS_ACT_GELU_ERF) return gelu_erf(x);
    return x;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Where the key and value columns of a packed q|k|v projection go when the product's own epilogue writes them
// into the pages (k_pool null = nowhere: everything goes to the output buffer).
struct KvScatter {
    __nv_bfloat16* k_pool;
    __nv_bfloat16* v_pool;
    long long page_stride;
    const int* token_row;     // per token: the row of block_table that holds its request's pages
    const int* positions;
    const int* block_table;
    int bt_stride;
    int q_width;       // columns [0, q_width) are queries and go to `out`
    int kv_width;      // then kv_width key columns, then kv_width value columns
    int head_dim;
    int page_size;
};

// Thread-block clusters: CTAs of a cluster read each other's shared memory after a cluster barrier.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t ld_cluster_u32(const void* local, int rank) {
    uint32_t remote, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ float ld_cluster_f32(const float* local, int rank) {
    return __uint_as_float(ld_cluster_u32(local, rank));
}
// 16 bytes at once (local must be 16-byte aligned). Not volatile: independent loads may be in flight together;
// the cluster barrier before them orders them behind the writes they read.
__device__ __forceinline__ float4 ld_cluster_f32x4(const float* local, int rank) {
    uint32_t remote;
    float4 v;
    asm("mapa.shared::cluster.u32 %0, %1, %2;"
        : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}

// Programmatic dependent launch (on unless PAGEDSERVE_B200_PDL=0). A kernel calls pdl_wait() before it
// touches memory that an earlier kernel wrote: it returns when all earlier kernels have completed and their
// writes are visible. What a kernel does before pdl_wait() (reading weights, which no kernel writes) overlaps
// the end of the kernel before it. pdl_launch() lets the next kernel in the stream begin to launch: its CTAs
// are scheduled as SM resources free up and run up to their own pdl_wait(). Because every kernel calls
// pdl_launch() after its pdl_wait(), at most two kernels are resident at a time. Without the launch
// attribute both instructions do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_prologue() {
    pdl_wait();
    pdl_launch();
}
// A pointer to data that an earlier kernel of the step wrote goes through pdl_fresh() after pdl_wait():
// loads through a `const __restrict__` pointer count as loads of memory that never changes, which the
// compiler may move above the wait; the value returned here does not exist before the wait.
template <typename T>
__device__ __forceinline__ T* pdl_fresh(T* p) {
    asm volatile("" : "+l"(p) : : "memory");
    return p;
}

// PAGEDSERVE_B200_PDL: unset or 1 = programmatic dependent launch for every kernel, 0 = for none; any other
// value is a comma-separated list of pieces of kernel names that get it (for finding out which kernel gains
// or misbehaves).
inline bool pdl_name_listed(const void* kernel, const char* env) {
    const char* name = nullptr;
    if (cudaFuncGetName(&name, kernel) != cudaSuccess || !name) return false;
    const char* piece = env;
    while (*piece) {
        const char* end = strchr(piece, ',');
        size_t n = end ? (size_t)(end - piece) : strlen(piece);
        if (n > 0 && n < 128) {
            char buffer[128];
            memcpy(buffer, piece, n);
            buffer[n] = 0;
            if (strstr(name, buffer)) return true;
        }
        if (!end) break;
        piece = end + 1;
    }
    return false;
}

// The decision is per kernel (the launcher below is one template instance for all kernels of one signature,
// so a static inside it would let the first kernel decide for the others).
inline bool pdl_enabled_for(const void* kernel) {
    static const char* const env = getenv("PAGEDSERVE_B200_PDL");
    static const int mode = (!env || !*env || !strcmp(env, "1")) ? 1 : (!strcmp(env, "0") ? 0 : 2);
    if (mode != 2) return mode == 1;
    static std::mutex lock;
    static std::unordered_map<const void*, bool> decided;
    std::lock_guard<std::mutex> guard(lock);
    auto found = decided.find(kernel);
    if (found != decided.end()) return found->second;
    const bool listed = pdl_name_listed(kernel, env);
    decided.emplace(kernel, listed);
    return listed;
}

// A kernel that needs more than 48 KB of dynamic shared memory has its limit raised once per device:
// `raised` is the call site's own static table (one per kernel instantiation) of what each device allows.
constexpr int MAX_DEVICES = 64;
inline bool ensure_dynamic_smem(const void* kernel, size_t smem, size_t (&raised)[MAX_DEVICES]) {
    if (smem <= 48 * 1024) return true;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return false;
    if (smem <= raised[device]) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return false;
    raised[device] = smem;
    return true;
}

// Launch with the programmatic-stream-serialization attribute (kept when a stream is captured into a
// CUDA graph, where it becomes a programmatic dependency edge).
template <typename... KArgs, typename... Args>
inline int launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              int cluster_z, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    // Measured on B200 with the 64-kernel decode graph of GPT-2 124M at batch 8: 362 us per step with it,
    // 414 us without. (A first form, in which every kernel let its successor launch before its own wait, so
    // that many kernels sat resident at once, was slower than no early launch at all.)
    const bool enabled = pdl_enabled_for((const void*)kernel);
    cudaLaunchAttribute attribute[2];
    int count = 0;
    if (enabled) {
        attribute[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    if (cluster_z > 1) {             // thread-block clusters of (1, 1, cluster_z) CTAs
        attribute[count].id = cudaLaunchAttributeClusterDimension;
        attribute[count].val.clusterDim.x = 1;
        attribute[count].val.clusterDim.y = 1;
        attribute[count].val.clusterDim.z = (unsigned)cluster_z;
        ++count;
    }
    config.attrs = attribute;
    config.numAttrs = count;
    cudaError_t e = cudaLaunchKernelEx(&config, kernel, KArgs(args)...);
    return e == cudaSuccess ? PS_OK : PS_ERR_LAUNCH;
}

template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                      Args... args) {
    return launch_pdl_cluster(kernel, grid, block, smem, stream, 1, args...);
}

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? PS_OK : PS_ERR_LAUNCH;
}

}  // namespace ps
