// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16, float
// accumulation), for head sizes that are multiples of 16 up to 128 and pages of 64 tokens.
//
//  * decode: one query token per sequence.  A block takes one kv head, up to 16 of its query
//    heads (the MMA's 16 rows: the whole group shares one read of the keys and values) and a
//    range of keys.  Two kernels: in the one that serves the engine every warp walks a range of
//    its own, 32 keys at a time through its own two-stage cp.async ring, with one online softmax
//    per tile and no barrier until the warps of a block merge; in the older one the four warps
//    of a block share each page's tile, 16 keys per warp.  Partial results of the blocks of a
//    (sequence, kv head) go to float scratch and are merged by the combine kernel.
//  * prefill: packed sequences with a past.  A block takes 64 query rows of one head (16 per
//    warp) and walks the pages its rows can see, double-buffered.
//
// Key j is visible to the query at absolute position p iff j <= p and, in a windowed group,
// j > p - window.  Softmax runs in float in the base-2 domain.  Other element types, head sizes
// and page sizes take the generic kernels of attention.cu.
//
// Counterpart in luozoupi/Qwen-Triton: kernels/flash_attention.py:54-152.
#include "attention_mma.cuh"

using namespace qt;
using namespace qt_mma;

namespace {

int check(const char* name, int n_seqs, int nq, int nkv, int d, int page_tokens, int ring_tokens, int window) {
    QT_REQUIRE(n_seqs > 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "%s: bad head counts nq=%d nkv=%d (B=%d)", name, nq, nkv, n_seqs);
    QT_REQUIRE(d >= 16 && d <= 128 && d % 16 == 0, "%s: head_dim=%d is not a multiple of 16 up to 128 (use the generic kernel)", name, d);
    QT_REQUIRE(page_tokens == PAGE, "%s: pages of %d tokens (this kernel walks pages of %d)", name, page_tokens, PAGE);
    QT_REQUIRE(ring_tokens >= 0 && ring_tokens % PAGE == 0, "%s: the ring of %d tokens is not a whole number of pages", name, ring_tokens);
    QT_REQUIRE(ring_tokens == 0 || (window > 0 && ring_tokens >= window), "%s: a ring of %d tokens cannot hold a window of %d", name, ring_tokens, window);
    QT_REQUIRE(n_seqs <= 65535 && nq <= 65535, "%s: too many sequences or heads for one launch", name);
    return QT_OK;
}

// Depth of the decode kernel's tile ring.  Two stages leave room for three blocks per SM at head size 128, which
// measured faster than three stages and two blocks (the kernel is bound by latency, not by bytes in flight);
// QT_B200_DECODE_STAGES=3 selects the deeper ring.
int decode_stages() {
    static int stages = 0;
    if (stages == 0) {
        const char* env = getenv("QT_B200_DECODE_STAGES");
        stages = (env && env[0] == '3') ? 3 : 2;
    }
    return stages;
}

template <typename K>
int raise_smem(K kernel, size_t bytes, const char* name) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "%s: cannot raise shared memory to %zu: %s", name, bytes, cudaGetErrorString(err));
    return QT_OK;
}

}  // namespace

extern "C" int qt_attention_decode_mma(const void* q, const void* k_cache, const void* v_cache, void* out,
                                       const int* block_table, int max_blocks, const int* seq_len, int n_seqs, int nq,
                                       int nkv, int d, int page_tokens, int ring_tokens, int window, float scale,
                                       int n_splits, float* part_acc, float* part_ml, void* stream) {
    if (n_seqs == 0) return QT_OK;
    int rc = check("attention_decode_mma", n_seqs, nq, nkv, d, page_tokens, ring_tokens, window);
    if (rc) return rc;
    QT_REQUIRE(n_splits >= 1 && n_splits <= 65535, "attention_decode_mma: n_splits=%d", n_splits);
    QT_REQUIRE(n_splits == 1 || (part_acc && part_ml), "attention_decode_mma: split results need scratch memory");
    MmaParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out,
                block_table, max_blocks, nullptr, nullptr, seq_len, n_seqs, nq, nkv, d, ring_tokens, window, scale,
                n_splits, part_acc, part_ml, decode_stages()};
    const int lds = d + PAD;
    const size_t stage = 2 * (size_t)PAGE * lds * 2;
    size_t smem = 16 * lds * 2 + p.stages * stage;
    const size_t merge = 16 * lds * 2 + (size_t)4 * 16 * d * 4 + 4 * 16 * 2 * 4;
    if (merge > smem) smem = merge;
    const int group = nq / nkv;
    dim3 grid(n_splits, nkv * ((group + 15) / 16), n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    if (d <= 64) {
        static bool ok = false;
        if (!ok) { rc = raise_smem(attention_decode_mma_kernel<64>, 100 * 1024, "attention_decode_mma"); if (rc) return rc; ok = true; }
        launch_kernel(attention_decode_mma_kernel<64>, dim3(grid), dim3(128), smem, s, p);
    } else {
        static bool ok = false;
        if (!ok) { rc = raise_smem(attention_decode_mma_kernel<128>, 128 * 1024, "attention_decode_mma"); if (rc) return rc; ok = true; }
        launch_kernel(attention_decode_mma_kernel<128>, dim3(grid), dim3(128), smem, s, p);
    }
    QT_CHECK_LAUNCH("attention_decode_mma");
    if (n_splits > 1) {
        launch_kernel(attention_combine_mma_kernel, dim3(n_seqs * nq), dim3(128), 0, s, part_acc, part_ml, (__nv_bfloat16*)out, n_splits, d);
        QT_CHECK_LAUNCH("attention_combine_mma");
    }
    return QT_OK;
}

// The decode kernel that gives every warp a key range of its own: `n_splits` blocks of `warps` warps per
// (sequence, kv head).  Two to eight blocks form a cluster and merge in the first block's shared memory (one
// launch, no scratch); more go through scratch and the combine kernel.
extern "C" int qt_attention_decode_ws(const void* q, const void* k_cache, const void* v_cache, void* out,
                                      const int* block_table, int max_blocks, const int* seq_len, int n_seqs, int nq,
                                      int nkv, int d, int page_tokens, int ring_tokens, int window, float scale,
                                      int n_splits, int warps, float* part_acc, float* part_ml, void* stream) {
    if (n_seqs == 0) return QT_OK;
    int rc = check("attention_decode_ws", n_seqs, nq, nkv, d, page_tokens, ring_tokens, window);
    if (rc) return rc;
    QT_REQUIRE(n_splits >= 1 && n_splits <= 65535, "attention_decode_ws: n_splits=%d", n_splits);
    QT_REQUIRE(warps >= 1 && warps <= WS_MAX_WARPS, "attention_decode_ws: %d warps per block (1 to %d)", warps, WS_MAX_WARPS);
    QT_REQUIRE(scale > 0.f, "attention_decode_ws: the score scale must be positive (the row maximum is taken before scaling)");
    // Up to eight blocks per (sequence, kv head) run as one cluster and merge through the first block's shared memory;
    // more than that (or QT_B200_DECODE_CLUSTER=0) go through scratch and the combine kernel.
    static const bool cluster_allowed = [] { const char* env = getenv("QT_B200_DECODE_CLUSTER"); return !(env && env[0] == '0'); }();
    const int lds = d + PAD;
    const int group = nq / nkv;
    const int rows_most = group < 16 ? group : 16;
    const size_t rings = 16 * (size_t)lds * 2 + (size_t)warps * 4 * WS_TILE * lds * 2;
    const size_t inboxes = (size_t)n_splits * (rows_most * d + 2 * rows_most) * sizeof(float);
    const bool cluster = cluster_allowed && n_splits >= 2 && n_splits <= 8 && rings + inboxes <= 227 * 1024;
    QT_REQUIRE(n_splits == 1 || cluster || (part_acc && part_ml), "attention_decode_ws: split results need scratch memory");
    MmaParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out,
                block_table, max_blocks, nullptr, nullptr, seq_len, n_seqs, nq, nkv, d, ring_tokens, window, scale,
                n_splits, part_acc, part_ml, 2, cluster ? 1 : 0};
    const size_t smem = rings + (cluster ? inboxes : 0);
    dim3 grid(n_splits, nkv * ((group + 15) / 16), n_seqs), block(32 * warps);
    cudaStream_t s = (cudaStream_t)stream;
#define QT_LAUNCH_WS(DMAX, EXACT)                                                                                        \
    do {                                                                                                                 \
        static bool ok = false;                                                                                          \
        if (!ok) { rc = raise_smem(attention_decode_ws_kernel<DMAX, EXACT>, 227 * 1024, "attention_decode_ws"); if (rc) return rc; ok = true; } \
        if (cluster) launch_kernel_cluster(attention_decode_ws_kernel<DMAX, EXACT>, grid, block, smem, s, (unsigned)n_splits, p); \
        else launch_kernel(attention_decode_ws_kernel<DMAX, EXACT>, grid, block, smem, s, p);                             \
    } while (0)
    if (d == 128) QT_LAUNCH_WS(128, true);
    else if (d == 64) QT_LAUNCH_WS(64, true);
    else if (d < 64) QT_LAUNCH_WS(64, false);
    else QT_LAUNCH_WS(128, false);
#undef QT_LAUNCH_WS
    QT_CHECK_LAUNCH("attention_decode_ws");
    if (n_splits > 1 && !cluster) {
        launch_kernel(attention_combine_mma_kernel, dim3(n_seqs * nq), dim3(128), 0, s, part_acc, part_ml, (__nv_bfloat16*)out, n_splits, d);
        QT_CHECK_LAUNCH("attention_combine_mma");
    }
    return QT_OK;
}

extern "C" int qt_attention_prefill_mma(const void* q, const void* k_cache, const void* v_cache, void* out,
                                        const int* block_table, int max_blocks, const int* seq_start, const int* seq_past,
                                        int n_seqs, int max_q_len, int nq, int nkv, int d, int page_tokens, int ring_tokens,
                                        int window, float scale, void* stream) {
    if (n_seqs == 0 || max_q_len == 0) return QT_OK;
    int rc = check("attention_prefill_mma", n_seqs, nq, nkv, d, page_tokens, ring_tokens, window);
    if (rc) return rc;
    MmaParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out,
                block_table, max_blocks, seq_start, seq_past, nullptr, n_seqs, nq, nkv, d, ring_tokens, window, scale,
                1, nullptr, nullptr, 2};
    const int lds = d + PAD;
    const size_t smem = (size_t)4 * PAGE * lds * 2;
    dim3 grid((max_q_len + PF_BQ - 1) / PF_BQ, nq, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    if (d <= 64) {
        static bool ok = false;
        if (!ok) { rc = raise_smem(attention_prefill_mma_kernel<64>, 100 * 1024, "attention_prefill_mma"); if (rc) return rc; ok = true; }
        launch_kernel(attention_prefill_mma_kernel<64>, dim3(grid), dim3(128), smem, s, p);
    } else {
        static bool ok = false;
        if (!ok) { rc = raise_smem(attention_prefill_mma_kernel<128>, 100 * 1024, "attention_prefill_mma"); if (rc) return rc; ok = true; }
        launch_kernel(attention_prefill_mma_kernel<128>, dim3(grid), dim3(128), smem, s, p);
    }
    QT_CHECK_LAUNCH("attention_prefill_mma");
    return QT_OK;
}

QT_DEFINE_LAST_ERROR(attention_mma)
