// Shared helpers of the sm_100a kernels: element types, loads that widen to float,
// warp and block reductions, and the error convention of the C entry points.
//
// Every entry point is `extern "C" int qt_*(..., void* stream)`: it checks its
// arguments, launches on `stream`, and returns 0 or a negative code whose text
// qt_last_error() (in each library) gives.  Nothing allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <utility>

#define QT_OK 0
#define QT_ERR_ARG -1
#define QT_ERR_LAUNCH -2
#define QT_ERR_UNSUPPORTED -3

// element types of activations, weights and caches
#define QT_F32 0
#define QT_BF16 1

namespace qt {

static thread_local char g_error[512] = "";

#define QT_FAIL(code, ...)                                   \
    do {                                                     \
        snprintf(qt::g_error, sizeof(qt::g_error), __VA_ARGS__); \
        return (code);                                       \
    } while (0)

#define QT_REQUIRE(cond, ...)                     \
    do {                                          \
        if (!(cond)) QT_FAIL(QT_ERR_ARG, __VA_ARGS__); \
    } while (0)

#define QT_CHECK_LAUNCH(name)                                                          \
    do {                                                                               \
        cudaError_t err__ = cudaGetLastError();                                        \
        if (err__ != cudaSuccess)                                                      \
            QT_FAIL(QT_ERR_LAUNCH, "%s: launch failed: %s", name, cudaGetErrorString(err__)); \
    } while (0)

#define QT_DEFINE_LAST_ERROR(libname)                                   \
    extern "C" const char* qt_last_error_##libname() { return qt::g_error; }

// Programmatic dependent launch.  Every kernel is launched so that it may start while the kernel before
// it in the stream is still draining; it announces its own dependents at once and, before it touches
// anything a predecessor wrote (or writes anything a predecessor may still read), waits for the
// predecessors to finish.  Work that depends on nothing earlier (set-up, weight prefetch) runs ahead of
// that wait.  QT_B200_PDL=0 in the environment turns the launch attribute off; the wait is then a no-op.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Streaming multiprocessors of the current device (asked once per device).
inline int sm_count() {
    static int counts[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 1;
    if (counts[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 1;
        counts[device] = n;
    }
    return counts[device];
}

inline bool pdl_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* env = getenv("QT_B200_PDL");
        enabled = (env && env[0] == '0') ? 0 : 1;
    }
    return enabled != 0;
}

template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);   // errors surface in QT_CHECK_LAUNCH
}

// The same with the blocks grouped into thread-block clusters of `cluster_x` along x (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
inline void launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster_x,
                                  Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = cluster_x;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);   // errors surface in QT_CHECK_LAUNCH
}

// Thread-block cluster helpers: rank and size along the cluster, the address of a shared-memory word of another
// block of the cluster, a store to it, and the cluster-wide barrier (release/acquire: stores before it are seen after it).
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_size() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_store_float(const float* local, uint32_t rank, float value) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(value) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// A block may touch another block's shared memory only once that block has started.  Every thread arrives here at
// kernel entry and waits just before its block's first remote access; by then every block of the cluster has arrived,
// so it runs.  (A second, release/acquire barrier still has to follow the remote stores before they are read.)
__device__ __forceinline__ void cluster_arrive_started() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_started() { asm volatile("barrier.cluster.wait.aligned;" ::: "memory"); }

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Gate activations of a gated feed-forward, out = act(gate) * up (a parameter of the part, a code here).
#define QT_ACT_SILU 0
#define QT_ACT_GELU_TANH 1
#define QT_ACT_GELU 2
#define QT_ACT_RELU 3
#define QT_ACT_COUNT 4

// act(g) in float.  FAST takes the hardware approximations of exp and division for SiLU (2 ulp of float, for results
// that are rounded to bfloat16 anyway); the other activations are the library's forms.
template <bool FAST>
__device__ __forceinline__ float gate_activation(float g, int act) {
    switch (act) {
        case QT_ACT_GELU_TANH: return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
        case QT_ACT_GELU: return 0.5f * g * (1.f + erff(g * 0.7071067811865476f));
        case QT_ACT_RELU: return fmaxf(g, 0.f);
        default: return FAST ? __fdividef(g, 1.f + __expf(-g)) : g / (1.f + expf(-g));
    }
}

// Sum of `n_splits` partial results stored `split_stride` elements apart (split-K GEMM output).
template <typename T>
__device__ __forceinline__ float load_sum(const T* base, size_t index, int n_splits, size_t split_stride) {
    float acc = to_float(base[index]);
    for (int s = 1; s < n_splits; ++s) acc += to_float(base[index + (size_t)s * split_stride]);
    return acc;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

// Block-wide sum for blocks of up to 1024 threads; `scratch` holds 32 floats.  All threads get the sum.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = (lane < nwarps) ? scratch[lane] : 0.f;
    total = warp_sum(total);
    return total;
}

// Where position `pos` of a sequence lives in a paged cache.
//   block_table   this sequence's row of page numbers
//   ring_tokens   0: position p is element p; else element p % ring_tokens (windowed group)
// Layout of one cache entry: [pages][kv_heads][page_tokens][head_dim].
__device__ __forceinline__ size_t cache_offset(const int* block_table, int pos, int ring_tokens, int page_tokens,
                                               int kv_heads, int kv_head, int head_dim) {
    const int slot_pos = ring_tokens > 0 ? pos % ring_tokens : pos;
    const int page = block_table[slot_pos / page_tokens];
    return (((size_t)page * kv_heads + kv_head) * page_tokens + (slot_pos % page_tokens)) * (size_t)head_dim;
}

}  // namespace qt

// Calls `body` with `T` bound to the element type named by the runtime code.
#define QT_DISPATCH_DTYPE(dtype, name, ...)                         \
    [&]() -> int {                                                  \
        if ((dtype) == QT_F32) {                                    \
            using T = float;                                        \
            __VA_ARGS__                                             \
        } else if ((dtype) == QT_BF16) {                            \
            using T = __nv_bfloat16;                                \
            __VA_ARGS__                                             \
        }                                                           \
        QT_FAIL(QT_ERR_ARG, "%s: unknown element type %d", name, (int)(dtype)); \
    }()
