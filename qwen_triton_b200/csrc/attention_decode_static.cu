// Implementation of qt_attention_decode_static: the split-KV decode attention of attention_mma.cuh
// with its scratch in a static device array, for callers that cannot allocate (see the header).
#include "attention_decode_static.h"

#include "attention_mma.cuh"

#include <mutex>

using namespace qt;
using namespace qt_mma;

// The scratch of every call: partial accumulators first, then the (max, sum) pairs.  In host code this
// name is only a handle for cudaGetSymbolAddress; the address a kernel may use is looked up per device.
static __device__ __align__(256) float g_static_scratch[QT_STATIC_SCRATCH_FLOATS];

namespace {

constexpr int MAX_DEVICES = 64;
float* g_scratch_address[MAX_DEVICES] = {};
std::mutex g_setup_lock;

// Once per device, with that device current: the device address of the scratch array, and the
// shared-memory limit of the two kernel variants.
int setup_device(int device, float** scratch) {
    std::lock_guard<std::mutex> guard(g_setup_lock);
    if (g_scratch_address[device] == nullptr) {
        float* address = nullptr;
        cudaError_t err = cudaGetSymbolAddress((void**)&address, g_static_scratch);
        if (err != cudaSuccess || address == nullptr)
            QT_FAIL(QT_ERR_LAUNCH, "attention_decode_static: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(err));
        err = cudaFuncSetAttribute(attention_decode_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
        if (err == cudaSuccess)
            err = cudaFuncSetAttribute(attention_decode_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
        if (err != cudaSuccess)
            QT_FAIL(QT_ERR_LAUNCH, "attention_decode_static: cannot raise shared memory on device %d: %s", device, cudaGetErrorString(err));
        g_scratch_address[device] = address;
    }
    *scratch = g_scratch_address[device];
    return QT_OK;
}

}  // namespace

extern "C" int qt_attention_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                          const int* block_table, int max_blocks, const int* seq_len, int n_seqs, int nq,
                                          int nkv, int d, int page_tokens, int ring_tokens, int window, float scale,
                                          int n_splits, void* stream) {
    if (n_seqs == 0) return QT_OK;
    QT_REQUIRE(n_seqs > 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention_decode_static: bad head counts nq=%d nkv=%d (B=%d)", nq, nkv, n_seqs);
    QT_REQUIRE(d >= 16 && d <= 128 && d % 16 == 0, "attention_decode_static: head_dim=%d is not a multiple of 16 up to 128", d);
    QT_REQUIRE(page_tokens == PAGE, "attention_decode_static: pages of %d tokens (this kernel walks pages of %d)", page_tokens, PAGE);
    QT_REQUIRE(ring_tokens >= 0 && ring_tokens % PAGE == 0, "attention_decode_static: the ring of %d tokens is not a whole number of pages", ring_tokens);
    QT_REQUIRE(ring_tokens == 0 || (window > 0 && ring_tokens >= window), "attention_decode_static: a ring of %d tokens cannot hold a window of %d", ring_tokens, window);
    QT_REQUIRE(n_seqs <= 65535 && n_splits >= 1 && n_splits <= 65535, "attention_decode_static: n_seqs=%d, n_splits=%d", n_seqs, n_splits);
    QT_REQUIRE((long long)nkv * ((nq / nkv + 15) / 16) <= 65535, "attention_decode_static: nkv=%d with groups of %d heads is more than one launch takes", nkv, nq / nkv);
    const long long slots = (long long)n_seqs * nq * n_splits;
    const long long needed = slots * (d + 2);
    QT_REQUIRE(needed <= (long long)QT_STATIC_SCRATCH_FLOATS,
               "attention_decode_static: this call needs %lld floats of scratch (n_seqs * nq * n_splits * (d + 2)), the built-in array holds %lld; "
               "use fewer splits or a smaller batch, or call qt_attention_decode_mma with scratch of your own",
               needed, (long long)QT_STATIC_SCRATCH_FLOATS);
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    QT_REQUIRE(err == cudaSuccess && device >= 0 && device < MAX_DEVICES, "attention_decode_static: no usable current device (%s)", cudaGetErrorString(err));
    float* scratch = nullptr;
    int rc = setup_device(device, &scratch);
    if (rc) return rc;
    float* part_acc = scratch;
    float* part_ml = scratch + slots * d;

    MmaParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out,
                block_table, max_blocks, nullptr, nullptr, seq_len, n_seqs, nq, nkv, d, ring_tokens, window, scale,
                n_splits, part_acc, part_ml, DEC_MAX_STAGES};
    const int lds = d + PAD;
    const size_t stage = 2 * (size_t)PAGE * lds * 2;
    size_t smem = 16 * lds * 2 + DEC_MAX_STAGES * stage;
    const size_t merge = 16 * lds * 2 + (size_t)4 * 16 * d * 4 + 4 * 16 * 2 * 4;
    if (merge > smem) smem = merge;
    const int group = nq / nkv;
    dim3 grid(n_splits, nkv * ((group + 15) / 16), n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    if (d <= 64) launch_kernel(attention_decode_mma_kernel<64>, grid, dim3(128), smem, s, p);
    else launch_kernel(attention_decode_mma_kernel<128>, grid, dim3(128), smem, s, p);
    QT_CHECK_LAUNCH("attention_decode_static");
    if (n_splits > 1) {
        launch_kernel(attention_combine_mma_kernel, dim3(n_seqs * nq), dim3(128), 0, s, (const float*)part_acc, (const float*)part_ml,
                      (__nv_bfloat16*)out, n_splits, d);
        QT_CHECK_LAUNCH("attention_decode_static (merge)");
    }
    return QT_OK;
}

QT_DEFINE_LAST_ERROR(attention_decode_static)
