// Memory-bound kernels of the step: embedding gather, residual add fused with RMSNorm,
// per-head q/k RMSNorm fused with rotary position encoding and the cache write, and the
// SiLU-gated product.  Norms, rotation and the residual sum are computed in float.
//
// Counterparts in luozoupi/Qwen-Triton: kernels/embedding.py:50-66, kernels/rmsnorm.py:100-133,
// kernels/residual_add.py:50-60, kernels/rope.py:99-120, csrc/rope_op_kernel.cu:12-39,
// kernels/cache.py:71-98, kernels/swiglu.py:84-92.
#include "common.cuh"

using namespace qt;

// ----------------------------------------------------------------------------- embedding
// residual[t, :] = table[ids[t], :] widened to float.  One block per token.
template <typename T>
__global__ void embedding_kernel(float* __restrict__ residual, const T* __restrict__ table,
                                 const int* __restrict__ ids, int hidden, int vocab) {
    const int t = blockIdx.x;
    int id = ids[t];
    const bool valid = id >= 0 && id < vocab;   // ids are range-checked on the host; never read outside the table
    const T* row = table + (size_t)(valid ? id : 0) * hidden;
    float* out = residual + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = valid ? to_float(row[i]) : 0.f;
}

extern "C" int qt_embedding(float* residual, const void* table, const int* ids, int n_tokens, int hidden, int vocab,
                            int table_dtype, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes T=%d H=%d V=%d", n_tokens, hidden, vocab);
    if (n_tokens == 0) return QT_OK;
    return QT_DISPATCH_DTYPE(table_dtype, "embedding", {
        embedding_kernel<T><<<n_tokens, 256, 0, (cudaStream_t)stream>>>(residual, (const T*)table, ids, hidden, vocab);
        QT_CHECK_LAUNCH("embedding");
        return QT_OK;
    });
}

// ----------------------------------------------------------------------------- residual add + RMSNorm
// One block per output row r.  src = rows ? rows[r] : r.
//   x = residual[src] + sum_s delta[s][src]            (float)
//   if (!rows) residual[src] = x                        (the stream is updated in place)
//   out[r] = x * rsqrt(mean(x^2) + eps) * weight       (rounded once to the output type)
// With `rows` the kernel norms only the listed rows (the positions whose logits are wanted) and
// leaves the stream untouched.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_splits,
                                   size_t split_stride, const float* __restrict__ weight, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows, int hidden) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* res = residual + (size_t)src * hidden;
    float sq = 0.f;
    // pass 1: form the new stream value; keep it in `res` (or, for listed rows, recompute in pass 2)
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float x = res[i];
        if (delta) x += load_sum(delta, (size_t)src * hidden + i, n_splits, split_stride);
        if (!rows) res[i] = x;
        sq += x * x;
    }
    const float total = block_sum(sq, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
    TO* o = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float x = res[i];   // each thread re-reads what it wrote itself
        if (rows && delta) x += load_sum(delta, (size_t)src * hidden + i, n_splits, split_stride);
        o[i] = from_float<TO>(x * inv * weight[i]);
    }
}

extern "C" int qt_add_rmsnorm(float* residual, const void* delta, int delta_dtype, int n_splits, long long split_stride,
                              const float* weight, float eps, void* out, int out_dtype, const int* rows, int n_rows,
                              int hidden, void* stream) {
    QT_REQUIRE(n_rows >= 0 && hidden > 0 && n_splits >= 1, "add_rmsnorm: bad sizes rows=%d H=%d splits=%d", n_rows, hidden, n_splits);
    QT_REQUIRE(eps > 0.f, "add_rmsnorm: eps must be positive");
    if (n_rows == 0) return QT_OK;
    const int threads = hidden >= 2048 ? 512 : 256;
    cudaStream_t s = (cudaStream_t)stream;
#define QT_LAUNCH_NORM(TD, TO)                                                                                   \
    add_rmsnorm_kernel<TD, TO><<<n_rows, threads, 0, s>>>(residual, (const TD*)delta, n_splits, (size_t)split_stride, \
                                                          weight, eps, (TO*)out, rows, hidden)
    if (delta_dtype == QT_F32 && out_dtype == QT_F32) QT_LAUNCH_NORM(float, float);
    else if (delta_dtype == QT_F32 && out_dtype == QT_BF16) QT_LAUNCH_NORM(float, __nv_bfloat16);
    else if (delta_dtype == QT_BF16 && out_dtype == QT_BF16) QT_LAUNCH_NORM(__nv_bfloat16, __nv_bfloat16);
    else if (delta_dtype == QT_BF16 && out_dtype == QT_F32) QT_LAUNCH_NORM(__nv_bfloat16, float);
    else QT_FAIL(QT_ERR_ARG, "add_rmsnorm: unknown element types %d/%d", delta_dtype, out_dtype);
#undef QT_LAUNCH_NORM
    QT_CHECK_LAUNCH("add_rmsnorm");
    return QT_OK;
}

// ----------------------------------------------------------------------------- q/k norm + rotary + cache write
// Input: the fused projection output qkv[t, (nq + 2 nkv) * d] (possibly split-K partial sums).
// One warp per (token, head):
//   q head:  RMSNorm over d with q_weight (if given), rotate, store to q_out[t, h, :]
//   k head:  RMSNorm with k_weight (if given), rotate, store into the key cache at the token's position
//   v head:  store into the value cache
// Rotation (rotate-half): the first rd dims are paired (i, i + rd/2); cos/sin come from the float
// table cos_sin[pos, 0:rd/2] = cos, [rd/2:rd] = sin.  rd = 0 means no position encoding.
// With kv_in_proj = 0 the projection holds query heads only; with write_kv = 0 the k and v heads
// are skipped (a call that reads the cache another call wrote).
struct QkvParams {
    const void* qkv; int n_splits; size_t split_stride;
    void* q_out; void* k_cache; void* v_cache;
    const int* token_seq; const int* token_pos; const int* block_table; int max_blocks;
    const float* q_weight; const float* k_weight; float eps;
    const float* cos_sin; int rotary_dim; int max_pos;
    int n_tokens, nq, nkv, d, page_tokens, ring_tokens, write_kv, kv_in_proj;
};

template <typename TI, typename TO>
__global__ void qk_norm_rope_write_kernel(const QkvParams p) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = p.nq + (p.kv_in_proj ? 2 * p.nkv : 0);
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long long)p.n_tokens * heads_total) return;
    const int t = (int)(item / heads_total);
    const int head = (int)(item % heads_total);
    const bool is_q = head < p.nq, is_k = !is_q && head < p.nq + p.nkv;
    if (!is_q && !p.write_kv) return;
    float* vec = smem + warp * p.d;
    const size_t in_base = (size_t)t * heads_total * p.d + (size_t)head * p.d;
    const TI* in = (const TI*)p.qkv;

    float sq = 0.f;
    for (int i = lane; i < p.d; i += 32) {
        const float x = load_sum(in, in_base + i, p.n_splits, p.split_stride);
        vec[i] = x;
        sq += x * x;
    }
    const float* w = is_q ? p.q_weight : (is_k ? p.k_weight : nullptr);
    if (w) {
        sq = warp_sum(sq);
        const float inv = rsqrtf(sq / (float)p.d + p.eps);
        for (int i = lane; i < p.d; i += 32) vec[i] = vec[i] * inv * w[i];
    }
    __syncwarp();

    TO* dst;
    const int pos = p.token_pos[t];
    if (is_q) {
        dst = (TO*)p.q_out + ((size_t)t * p.nq + head) * p.d;
    } else {
        const int kvh = is_k ? head - p.nq : head - p.nq - p.nkv;
        const int* table = p.block_table + (size_t)p.token_seq[t] * p.max_blocks;
        dst = (TO*)(is_k ? p.k_cache : p.v_cache) + cache_offset(table, pos, p.ring_tokens, p.page_tokens, p.nkv, kvh, p.d);
    }
    const int half = p.rotary_dim >> 1;
    const bool rotate = (is_q || is_k) && half > 0;
    const float* cs = p.cos_sin + (size_t)(pos < p.max_pos ? pos : p.max_pos - 1) * p.rotary_dim;
    for (int i = lane; i < p.d; i += 32) {
        float y = vec[i];
        if (rotate && i < p.rotary_dim) {
            if (i < half) y = vec[i] * cs[i] - vec[i + half] * cs[half + i];
            else y = vec[i] * cs[i - half] + vec[i - half] * cs[i];
        }
        dst[i] = from_float<TO>(y);
    }
}

extern "C" int qt_qk_norm_rope_write(const void* qkv, int in_dtype, int n_splits, long long split_stride, void* q_out,
                                     void* k_cache, void* v_cache, int out_dtype, const int* token_seq,
                                     const int* token_pos, const int* block_table, int max_blocks,
                                     const float* q_weight, const float* k_weight, float eps, const float* cos_sin,
                                     int rotary_dim, int max_pos, int n_tokens, int nq, int nkv, int d, int page_tokens,
                                     int ring_tokens, int write_kv, int kv_in_proj, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && nq > 0 && nkv > 0 && d > 0 && d <= 1024, "qk_norm_rope_write: bad sizes T=%d nq=%d nkv=%d d=%d", n_tokens, nq, nkv, d);
    QT_REQUIRE(rotary_dim >= 0 && rotary_dim <= d && rotary_dim % 2 == 0, "qk_norm_rope_write: rotary_dim=%d must be even and at most head_dim=%d", rotary_dim, d);
    QT_REQUIRE(rotary_dim == 0 || (cos_sin && max_pos > 0), "qk_norm_rope_write: rotation needs a cos/sin table");
    QT_REQUIRE(page_tokens > 0 && n_splits >= 1 && ring_tokens >= 0, "qk_norm_rope_write: bad cache geometry");
    QT_REQUIRE(!write_kv || (k_cache && v_cache && block_table), "qk_norm_rope_write: cache pointers missing");
    QT_REQUIRE(!write_kv || kv_in_proj, "qk_norm_rope_write: nothing to write without k and v in the projection");
    if (n_tokens == 0) return QT_OK;
    QkvParams p{qkv, n_splits, (size_t)split_stride, q_out, k_cache, v_cache, token_seq, token_pos, block_table, max_blocks,
                q_weight, k_weight, eps, cos_sin, rotary_dim, max_pos, n_tokens, nq, nkv, d, page_tokens, ring_tokens, write_kv, kv_in_proj};
    const int warps = 4;
    const long long items = (long long)n_tokens * (nq + (kv_in_proj ? 2 * nkv : 0));
    const unsigned grid = (unsigned)((items + warps - 1) / warps);
    const size_t smem = (size_t)warps * d * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == QT_F32 && out_dtype == QT_F32) qk_norm_rope_write_kernel<float, float><<<grid, warps * 32, smem, s>>>(p);
    else if (in_dtype == QT_F32 && out_dtype == QT_BF16) qk_norm_rope_write_kernel<float, __nv_bfloat16><<<grid, warps * 32, smem, s>>>(p);
    else if (in_dtype == QT_BF16 && out_dtype == QT_BF16) qk_norm_rope_write_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, warps * 32, smem, s>>>(p);
    else QT_FAIL(QT_ERR_ARG, "qk_norm_rope_write: unsupported element types %d -> %d", in_dtype, out_dtype);
    QT_CHECK_LAUNCH("qk_norm_rope_write");
    return QT_OK;
}

// ----------------------------------------------------------------------------- SiLU-gated product
// out[t, i] = silu(g) * u with g = gate_up[t, i], u = gate_up[t, inter + i]; float inside.
template <typename TI, typename TO>
__global__ void swiglu_kernel(const TI* __restrict__ gate_up, int n_splits, size_t split_stride, TO* __restrict__ out,
                              long long total, int inter) {
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / inter;
        const int i = (int)(idx % inter);
        const size_t base = (size_t)t * 2 * inter;
        const float g = load_sum(gate_up, base + i, n_splits, split_stride);
        const float u = load_sum(gate_up, base + inter + i, n_splits, split_stride);
        out[idx] = from_float<TO>(g / (1.f + expf(-g)) * u);
    }
}

extern "C" int qt_swiglu(const void* gate_up, int in_dtype, int n_splits, long long split_stride, void* out, int out_dtype,
                         int n_tokens, int inter, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && inter > 0 && n_splits >= 1, "swiglu: bad sizes T=%d I=%d", n_tokens, inter);
    if (n_tokens == 0) return QT_OK;
    const long long total = (long long)n_tokens * inter;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > 148LL * 32) blocks = 148LL * 32;
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == QT_F32 && out_dtype == QT_F32) swiglu_kernel<float, float><<<(unsigned)blocks, threads, 0, s>>>((const float*)gate_up, n_splits, (size_t)split_stride, (float*)out, total, inter);
    else if (in_dtype == QT_F32 && out_dtype == QT_BF16) swiglu_kernel<float, __nv_bfloat16><<<(unsigned)blocks, threads, 0, s>>>((const float*)gate_up, n_splits, (size_t)split_stride, (__nv_bfloat16*)out, total, inter);
    else if (in_dtype == QT_BF16 && out_dtype == QT_BF16) swiglu_kernel<__nv_bfloat16, __nv_bfloat16><<<(unsigned)blocks, threads, 0, s>>>((const __nv_bfloat16*)gate_up, n_splits, (size_t)split_stride, (__nv_bfloat16*)out, total, inter);
    else QT_FAIL(QT_ERR_ARG, "swiglu: unsupported element types %d -> %d", in_dtype, out_dtype);
    QT_CHECK_LAUNCH("swiglu");
    return QT_OK;
}

QT_DEFINE_LAST_ERROR(elementwise)
