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
    pdl_launch_dependents();
    pdl_wait();
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
        launch_kernel(embedding_kernel<T>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, residual, (const T*)table, ids, hidden, vocab);
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
    pdl_launch_dependents();
    pdl_wait();
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

// Vector form for widths that are multiples of 4: each thread owns up to NORM_CACHE chunks of four
// consecutive elements, sums the split-K partials with independent 16-byte loads and keeps the new
// stream values in registers between the two passes.
constexpr int NORM_CACHE = 4;

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TD, typename TO>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_splits,
                                       size_t split_stride, const float* __restrict__ weight, float eps,
                                       TO* __restrict__ out, const int* __restrict__ rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* res = residual + (size_t)src * hidden;
    const int chunks = hidden >> 2;
    float4 x[NORM_CACHE];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_CACHE; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            float4 v = load4(res + 4 * c);
            if (delta) {
                const TD* dp = delta + (size_t)src * hidden + 4 * c;
#pragma unroll 4
                for (int s = 0; s < n_splits; ++s) {
                    const float4 dv = load4(dp + (size_t)s * split_stride);
                    v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
                }
            }
            if (!rows) store4(res + 4 * c, v);
            x[i] = v;
            sq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    }
    const float total = block_sum(sq, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
    TO* o = out + (size_t)r * hidden;
#pragma unroll
    for (int i = 0; i < NORM_CACHE; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            const float4 w = load4(weight + 4 * c);
            store4(o + 4 * c, make_float4(x[i].x * inv * w.x, x[i].y * inv * w.y, x[i].z * inv * w.z, x[i].w * inv * w.w));
        }
    }
}

extern "C" int qt_add_rmsnorm(float* residual, const void* delta, int delta_dtype, int n_splits, long long split_stride,
                              const float* weight, float eps, void* out, int out_dtype, const int* rows, int n_rows,
                              int hidden, void* stream) {
    QT_REQUIRE(n_rows >= 0 && hidden > 0 && n_splits >= 1, "add_rmsnorm: bad sizes rows=%d H=%d splits=%d", n_rows, hidden, n_splits);
    QT_REQUIRE(eps > 0.f, "add_rmsnorm: eps must be positive");
    if (n_rows == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    // the vector kernel needs 16-byte aligned rows everywhere and at most NORM_CACHE chunks per thread
    const bool aligned = hidden % 4 == 0 && ((uintptr_t)residual % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
                         ((uintptr_t)weight % 16 == 0) && (!delta || ((uintptr_t)delta % 16 == 0 && split_stride % 4 == 0));
    if (aligned && hidden <= 4 * NORM_CACHE * 1024) {
        int vthreads = ((hidden / 4 + 31) / 32) * 32;
        if (vthreads > 1024) vthreads = 1024;
        if (vthreads < 64) vthreads = 64;
#define QT_LAUNCH_NORM_VEC(TD, TO)                                                                                      \
    launch_kernel(add_rmsnorm_vec_kernel<TD, TO>, dim3(n_rows), dim3(vthreads), 0, s, residual, (const TD*)delta, n_splits, (size_t)split_stride, \
                                                               weight, eps, (TO*)out, rows, hidden)
        if (delta_dtype == QT_F32 && out_dtype == QT_F32) QT_LAUNCH_NORM_VEC(float, float);
        else if (delta_dtype == QT_F32 && out_dtype == QT_BF16) QT_LAUNCH_NORM_VEC(float, __nv_bfloat16);
        else if (delta_dtype == QT_BF16 && out_dtype == QT_BF16) QT_LAUNCH_NORM_VEC(__nv_bfloat16, __nv_bfloat16);
        else if (delta_dtype == QT_BF16 && out_dtype == QT_F32) QT_LAUNCH_NORM_VEC(__nv_bfloat16, float);
        else QT_FAIL(QT_ERR_ARG, "add_rmsnorm: unknown element types %d/%d", delta_dtype, out_dtype);
#undef QT_LAUNCH_NORM_VEC
        QT_CHECK_LAUNCH("add_rmsnorm");
        return QT_OK;
    }
    const int threads = hidden >= 2048 ? 512 : 256;
#define QT_LAUNCH_NORM(TD, TO)                                                                                   \
    launch_kernel(add_rmsnorm_kernel<TD, TO>, dim3(n_rows), dim3(threads), 0, s, residual, (const TD*)delta, n_splits, (size_t)split_stride, \
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

template <typename TI, typename TO, bool VEC>
__global__ void qk_norm_rope_write_kernel(const QkvParams p) {
    pdl_launch_dependents();
    pdl_wait();
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
    const float* w = is_q ? p.q_weight : (is_k ? p.k_weight : nullptr);

    // 1. the head's vector in float (split-K partials added up), its sum of squares
    float sq = 0.f;
    if (VEC) {
        for (int c = lane; c < (p.d >> 2); c += 32) {
            float4 v = load4(in + in_base + 4 * c);
#pragma unroll 4
            for (int s = 1; s < p.n_splits; ++s) {
                const float4 dv = load4(in + in_base + 4 * c + (size_t)s * p.split_stride);
                v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
            }
            *reinterpret_cast<float4*>(vec + 4 * c) = v;
            sq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = lane; i < p.d; i += 32) {
            const float x = load_sum(in, in_base + i, p.n_splits, p.split_stride);
            vec[i] = x;
            sq += x * x;
        }
    }
    // 2. RMSNorm over the head (q and k heads with a weight)
    float inv = 1.f;
    if (w) inv = rsqrtf(warp_sum(sq) / (float)p.d + p.eps);
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
    // 3. rotate-half over the first rotary_dim dims with the normed values, store
    const int half = p.rotary_dim >> 1;
    const bool rotate = (is_q || is_k) && half > 0;
    const float* cs = p.cos_sin + (size_t)(pos < p.max_pos ? pos : p.max_pos - 1) * p.rotary_dim;
    auto value = [&](int i) { return w ? vec[i] * inv * w[i] : vec[i]; };
    auto rotated = [&](int i) {
        float y = value(i);
        if (rotate && i < p.rotary_dim) {
            if (i < half) y = y * cs[i] - value(i + half) * cs[half + i];
            else y = y * cs[i - half] + value(i - half) * cs[i];
        }
        return y;
    };
    if (VEC) {
        for (int c = lane; c < (p.d >> 2); c += 32)
            store4(dst + 4 * c, make_float4(rotated(4 * c), rotated(4 * c + 1), rotated(4 * c + 2), rotated(4 * c + 3)));
    } else {
        for (int i = lane; i < p.d; i += 32) dst[i] = from_float<TO>(rotated(i));
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
    // 16-byte loads and stores need head_dim % 8 == 0 (bfloat16 rows of the cache and of q) and aligned bases
    const bool vec = d % 8 == 0 && split_stride % 8 == 0 && ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)q_out % 16 == 0) &&
                     (!write_kv || (((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0)));
#define QT_LAUNCH_QKV(TI, TO)                                                                    \
    do {                                                                                         \
        if (vec) launch_kernel(qk_norm_rope_write_kernel<TI, TO, true>, dim3(grid), dim3(warps * 32), smem, s, p);      \
        else launch_kernel(qk_norm_rope_write_kernel<TI, TO, false>, dim3(grid), dim3(warps * 32), smem, s, p);         \
    } while (0)
    if (in_dtype == QT_F32 && out_dtype == QT_F32) QT_LAUNCH_QKV(float, float);
    else if (in_dtype == QT_F32 && out_dtype == QT_BF16) QT_LAUNCH_QKV(float, __nv_bfloat16);
    else if (in_dtype == QT_BF16 && out_dtype == QT_BF16) QT_LAUNCH_QKV(__nv_bfloat16, __nv_bfloat16);
    else QT_FAIL(QT_ERR_ARG, "qk_norm_rope_write: unsupported element types %d -> %d", in_dtype, out_dtype);
#undef QT_LAUNCH_QKV
    QT_CHECK_LAUNCH("qk_norm_rope_write");
    return QT_OK;
}

// ----------------------------------------------------------------------------- SiLU-gated product
// out[t, i] = silu(g) * u with g = gate_up[t, i], u = gate_up[t, inter + i]; float inside.
template <typename TI, typename TO>
__global__ void swiglu_kernel(const TI* __restrict__ gate_up, int n_splits, size_t split_stride, TO* __restrict__ out,
                              long long total, int inter) {
    pdl_launch_dependents();
    pdl_wait();
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

// Four elements per thread with 8- or 16-byte loads and stores (widths that are multiples of 4, aligned bases).
template <typename TI, typename TO>
__global__ void swiglu_vec_kernel(const TI* __restrict__ gate_up, int n_splits, size_t split_stride, TO* __restrict__ out,
                                  long long total4, int inter) {
    pdl_launch_dependents();
    pdl_wait();
    const int chunks = inter >> 2;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total4;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / chunks;
        const int i = (int)(idx % chunks) * 4;
        const TI* gp = gate_up + (size_t)t * 2 * inter + i;
        float4 g = load4(gp), u = load4(gp + inter);
#pragma unroll 4
        for (int s = 1; s < n_splits; ++s) {
            const float4 dg = load4(gp + (size_t)s * split_stride), du = load4(gp + inter + (size_t)s * split_stride);
            g.x += dg.x; g.y += dg.y; g.z += dg.z; g.w += dg.w;
            u.x += du.x; u.y += du.y; u.z += du.z; u.w += du.w;
        }
        store4(out + (size_t)t * inter + i, make_float4(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y,
                                                        g.z / (1.f + expf(-g.z)) * u.z, g.w / (1.f + expf(-g.w)) * u.w));
    }
}

extern "C" int qt_swiglu(const void* gate_up, int in_dtype, int n_splits, long long split_stride, void* out, int out_dtype,
                         int n_tokens, int inter, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && inter > 0 && n_splits >= 1, "swiglu: bad sizes T=%d I=%d", n_tokens, inter);
    if (n_tokens == 0) return QT_OK;
    const long long total = (long long)n_tokens * inter;
    const int threads = 256;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = inter % 4 == 0 && split_stride % 4 == 0 && ((uintptr_t)gate_up % 16 == 0) && ((uintptr_t)out % 16 == 0);
    const long long work = vec ? total / 4 : total;
    long long blocks = (work + threads - 1) / threads;
    if (blocks > 148LL * 16) blocks = 148LL * 16;
#define QT_LAUNCH_SWIGLU(TI, TO)                                                                                              \
    do {                                                                                                                      \
        if (vec) launch_kernel(swiglu_vec_kernel<TI, TO>, dim3((unsigned)blocks), dim3(threads), 0, s, (const TI*)gate_up,    \
                               n_splits, (size_t)split_stride, (TO*)out, work, inter);                                        \
        else launch_kernel(swiglu_kernel<TI, TO>, dim3((unsigned)blocks), dim3(threads), 0, s, (const TI*)gate_up, n_splits,  \
                           (size_t)split_stride, (TO*)out, work, inter);                                                      \
    } while (0)
    if (in_dtype == QT_F32 && out_dtype == QT_F32) QT_LAUNCH_SWIGLU(float, float);
    else if (in_dtype == QT_F32 && out_dtype == QT_BF16) QT_LAUNCH_SWIGLU(float, __nv_bfloat16);
    else if (in_dtype == QT_BF16 && out_dtype == QT_BF16) QT_LAUNCH_SWIGLU(__nv_bfloat16, __nv_bfloat16);
    else QT_FAIL(QT_ERR_ARG, "swiglu: unsupported element types %d -> %d", in_dtype, out_dtype);
#undef QT_LAUNCH_SWIGLU
    QT_CHECK_LAUNCH("swiglu");
    return QT_OK;
}

QT_DEFINE_LAST_ERROR(elementwise)
