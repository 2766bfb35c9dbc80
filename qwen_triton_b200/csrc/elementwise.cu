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

// ----------------------------------------------------------------------------- bias of a projection
// out[t, :] += bias, on the float sums of a product before anything rounds them (the first plane, where a product is
// split over K).  luozoupi/Qwen-Triton adds the bias of a linear layer with a kernel of its own as well
// (kernels/matmul.py:99-111, modules/linear.py:31).
__global__ void add_bias_kernel(float* __restrict__ out, const float* __restrict__ bias, int cols, size_t count) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
        out[i] += bias[i % (size_t)cols];
}

extern "C" int qt_add_bias(float* out, const float* bias, int rows, int cols, void* stream) {
    QT_REQUIRE(rows >= 0 && cols > 0, "add_bias: bad sizes rows=%d cols=%d", rows, cols);
    if (rows == 0) return QT_OK;
    const size_t count = (size_t)rows * cols;
    const size_t blocks = (count + 255) / 256;
    launch_kernel(add_bias_kernel, dim3((unsigned)(blocks < 4096 ? blocks : 4096)), dim3(256), 0, (cudaStream_t)stream, out, bias, cols, count);
    QT_CHECK_LAUNCH("add_bias");
    return QT_OK;
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

// v += sum over splits of the four elements at dp + s * split_stride, in the order of the splits.  Up to sixteen
// loads are issued before the first add: with one block per few hundred elements the kernel's time is the chain of
// L2 round trips, not the bytes.
template <int BATCH, typename TD>
__device__ __forceinline__ void add_splits4(float4& v, const TD* dp, int first, int n_splits, size_t split_stride) {
    for (int s0 = first; s0 < n_splits; s0 += BATCH) {
        float4 t[BATCH];
#pragma unroll
        for (int j = 0; j < BATCH; ++j)               // unconditional loads (the last split again beyond the end), so that they batch
            t[j] = load4(dp + (size_t)min(s0 + j, n_splits - 1) * split_stride);
#pragma unroll
        for (int j = 0; j < BATCH; ++j)
            if (s0 + j < n_splits) { v.x += t[j].x; v.y += t[j].y; v.z += t[j].z; v.w += t[j].w; }
    }
}

template <typename TD, typename TO, int BATCH, int MAX_THREADS, int MIN_BLOCKS>
__global__ void __launch_bounds__(MAX_THREADS, MIN_BLOCKS) add_rmsnorm_vec_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_splits,
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
            if (delta) add_splits4<BATCH>(v, delta + (size_t)src * hidden + 4 * c, 0, n_splits, split_stride);
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

// Few rows (a decode step): a cluster of NORM_CLUSTER blocks per row, one chunk of four elements per thread, so that
// 8 rows keep 64 SMs busy instead of 8.  Each block pushes its share of the sum of squares into every block of its
// cluster (distributed shared memory); after the cluster barrier each block adds the shares up in the same order.
constexpr int NORM_CLUSTER = 8;

template <typename TD, typename TO>
__global__ void __launch_bounds__(1024, 1) add_rmsnorm_cluster_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_splits,
                                                                   size_t split_stride, const float* __restrict__ weight, float eps,
                                                                   TO* __restrict__ out, const int* __restrict__ rows, int hidden) {
    pdl_launch_dependents();
    cluster_arrive_started();
    pdl_wait();
    __shared__ float scratch[32];
    __shared__ float shares[NORM_CLUSTER];
    const uint32_t rank = cluster_rank();
    const int r = blockIdx.x / NORM_CLUSTER;
    const int src = rows ? rows[r] : r;
    float* res = residual + (size_t)src * hidden;
    const int chunks = hidden >> 2;
    const int c = (int)rank * blockDim.x + threadIdx.x;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < chunks) {
        v = load4(res + 4 * c);
        if (delta) add_splits4<16>(v, delta + (size_t)src * hidden + 4 * c, 0, n_splits, split_stride);
        if (!rows) store4(res + 4 * c, v);
    }
    const float4 w = c < chunks ? load4(weight + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);   // in flight under the reductions
    const float share = block_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w, scratch);
    cluster_wait_started();                                    // every block of the cluster runs: its shared memory may be written
    if (threadIdx.x < NORM_CLUSTER) cluster_store_float(&shares[rank], threadIdx.x, share);
    cluster_barrier();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_CLUSTER; ++i) total += shares[i];
    const float inv = rsqrtf(total / (float)hidden + eps);
    if (c < chunks) {
        store4(out + (size_t)r * hidden + 4 * c, make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w));
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
    if (aligned && n_rows < 256 && hidden >= 4 * 32 * NORM_CLUSTER && hidden <= 4 * 1024 * NORM_CLUSTER) {
        const int per_block = (hidden / 4 + NORM_CLUSTER - 1) / NORM_CLUSTER;
        const int cthreads = ((per_block + 31) / 32) * 32;
#define QT_LAUNCH_NORM_CLUSTER(TD, TO)                                                                                  \
    launch_kernel_cluster(add_rmsnorm_cluster_kernel<TD, TO>, dim3(n_rows * NORM_CLUSTER), dim3(cthreads), 0, s, NORM_CLUSTER, residual, \
                          (const TD*)delta, n_splits, (size_t)split_stride, weight, eps, (TO*)out, rows, hidden)
        if (delta_dtype == QT_F32 && out_dtype == QT_F32) QT_LAUNCH_NORM_CLUSTER(float, float);
        else if (delta_dtype == QT_F32 && out_dtype == QT_BF16) QT_LAUNCH_NORM_CLUSTER(float, __nv_bfloat16);
        else if (delta_dtype == QT_BF16 && out_dtype == QT_BF16) QT_LAUNCH_NORM_CLUSTER(__nv_bfloat16, __nv_bfloat16);
        else if (delta_dtype == QT_BF16 && out_dtype == QT_F32) QT_LAUNCH_NORM_CLUSTER(__nv_bfloat16, float);
        else QT_FAIL(QT_ERR_ARG, "add_rmsnorm: unknown element types %d/%d", delta_dtype, out_dtype);
#undef QT_LAUNCH_NORM_CLUSTER
        QT_CHECK_LAUNCH("add_rmsnorm");
        return QT_OK;
    }
    if (aligned && hidden <= 4 * NORM_CACHE * 1024) {
        // few rows (decode): one chunk per thread, shortest critical path; many rows (prefill): up to NORM_CACHE
        // independent chunks per thread in smaller blocks, which keeps more loads in flight and more blocks resident
        const int per_thread = n_rows >= 256 ? NORM_CACHE : 1;
        int vthreads = ((hidden / 4 + 32 * per_thread - 1) / (32 * per_thread)) * 32;
        if (vthreads > 1024) vthreads = 1024;
        if (vthreads < 64) vthreads = 64;
        // many rows in blocks of up to 256 threads: few registers, five blocks per SM (partial sums of a split product
        // are rare there); otherwise up to 1,024 threads with eight loads of partial sums in flight
#define QT_NORM_VEC_ARGS residual, (const TD_*)delta, n_splits, (size_t)split_stride, weight, eps, (TO_*)out, rows, hidden
#define QT_LAUNCH_NORM_VEC(TD, TO)                                                                                      \
    do {                                                                                                                \
        using TD_ = TD; using TO_ = TO;                                                                                 \
        if (per_thread > 1 && vthreads <= 256)                                                                          \
            launch_kernel(add_rmsnorm_vec_kernel<TD, TO, 2, 256, 5>, dim3(n_rows), dim3(vthreads), 0, s, QT_NORM_VEC_ARGS); \
        else                                                                                                            \
            launch_kernel(add_rmsnorm_vec_kernel<TD, TO, 8, 1024, 1>, dim3(n_rows), dim3(vthreads), 0, s, QT_NORM_VEC_ARGS); \
    } while (0)
        if (delta_dtype == QT_F32 && out_dtype == QT_F32) QT_LAUNCH_NORM_VEC(float, float);
        else if (delta_dtype == QT_F32 && out_dtype == QT_BF16) QT_LAUNCH_NORM_VEC(float, __nv_bfloat16);
        else if (delta_dtype == QT_BF16 && out_dtype == QT_BF16) QT_LAUNCH_NORM_VEC(__nv_bfloat16, __nv_bfloat16);
        else if (delta_dtype == QT_BF16 && out_dtype == QT_F32) QT_LAUNCH_NORM_VEC(__nv_bfloat16, float);
        else QT_FAIL(QT_ERR_ARG, "add_rmsnorm: unknown element types %d/%d", delta_dtype, out_dtype);
#undef QT_LAUNCH_NORM_VEC
#undef QT_NORM_VEC_ARGS
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
// Rotation: the first rd dims are paired (i, i + rd/2) (rotate-half) or, with `interleaved`, (2i, 2i + 1); pair i
// turns by the angle whose cos/sin come from the float table cos_sin[pos, i] = cos, [pos, rd/2 + i] = sin.
// rd = 0 means no position encoding.
// With kv_in_proj = 0 the projection holds query heads only; with write_kv = 0 the k and v heads
// are skipped (a call that reads the cache another call wrote).
struct QkvParams {
    const void* qkv; int n_splits; size_t split_stride;
    void* q_out; void* k_cache; void* v_cache;
    const int* token_seq; const int* token_pos; const int* block_table; int max_blocks;
    const float* q_weight; const float* k_weight; float eps;
    const float* cos_sin; int rotary_dim; int max_pos;
    int n_tokens, nq, nkv, d, page_tokens, ring_tokens, write_kv, kv_in_proj;
    int interleaved;        // rotation pairs are (2i, 2i + 1) instead of (i, i + rd/2)
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
            add_splits4<16>(v, in + in_base + 4 * c, 1, p.n_splits, p.split_stride);
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
            if (p.interleaved) {
                const int j = i >> 1;
                y = (i & 1) ? y * cs[j] + value(i - 1) * cs[half + j] : y * cs[j] - value(i + 1) * cs[half + j];
            } else if (i < half) y = y * cs[i] - value(i + half) * cs[half + i];
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

// Fast form for many tokens: every dimension rotates (rotary_dim == d) and half a head is IT * 32 * E elements, so
// a lane holds the E-element pieces (j, j + d/2) of a rotation pair in registers and nothing passes through shared
// memory.  One warp takes HEADS_PER_WARP consecutive heads of one token, so that position, page and cos/sin are
// looked up once.  Same arithmetic as the kernel above: float norm, weight, then rotation.
constexpr int HEADS_PER_WARP = 4;

template <int E> struct Piece;
template <> struct Piece<1> { float v[1]; };
template <> struct Piece<2> { float v[2]; };

template <int E> __device__ __forceinline__ Piece<E> load_piece(const float* p) {
    Piece<E> r;
    if (E == 2) { const float2 t = *reinterpret_cast<const float2*>(p); r.v[0] = t.x; r.v[E - 1] = t.y; }
    else r.v[0] = p[0];
    return r;
}
template <int E> __device__ __forceinline__ Piece<E> load_piece(const __nv_bfloat16* p) {
    Piece<E> r;
    if (E == 2) { const __nv_bfloat162 t = *reinterpret_cast<const __nv_bfloat162*>(p); r.v[0] = __low2float(t); r.v[E - 1] = __high2float(t); }
    else r.v[0] = __bfloat162float(p[0]);
    return r;
}
template <int E> __device__ __forceinline__ void store_piece(float* p, const Piece<E>& r) {
    if (E == 2) *reinterpret_cast<float2*>(p) = make_float2(r.v[0], r.v[E - 1]);
    else p[0] = r.v[0];
}
template <int E> __device__ __forceinline__ void store_piece(__nv_bfloat16* p, const Piece<E>& r) {
    if (E == 2) *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(r.v[0], r.v[E - 1]);
    else p[0] = __float2bfloat16_rn(r.v[0]);
}

// blockIdx.x is the token, blockIdx.y * 4 + warp the run of heads.
template <typename TI, typename TO, int E, int IT>
__global__ void __launch_bounds__(128) qk_norm_rope_pairs_kernel(const QkvParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = p.nq + (p.kv_in_proj ? 2 * p.nkv : 0);
    const int t = blockIdx.x;
    const int head0 = (blockIdx.y * 4 + warp) * HEADS_PER_WARP;
    if (head0 >= heads_total || (head0 >= p.nq && !p.write_kv)) return;
    const int half = p.d >> 1;
    const TI* in = (const TI*)p.qkv + ((size_t)t * heads_total + head0) * p.d;

    // every load of the warp's heads is issued before the first store (the compiler cannot move loads across the
    // stores itself: it does not know that the projection and the outputs are different memory)
    Piece<E> lo[HEADS_PER_WARP][IT], hi[HEADS_PER_WARP][IT];
#pragma unroll
    for (int hh = 0; hh < HEADS_PER_WARP; ++hh) {
        const TI* src = in + (head0 + hh < heads_total ? hh : 0) * p.d;
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            const int j = (it * 32 + lane) * E;
            lo[hh][it] = load_piece<E>(src + j);
            hi[hh][it] = load_piece<E>(src + half + j);
        }
    }
    if (p.n_splits > 1) {
        for (int s = 1; s < p.n_splits; ++s) {
#pragma unroll
            for (int hh = 0; hh < HEADS_PER_WARP; ++hh) {
                const TI* src = in + (head0 + hh < heads_total ? hh : 0) * p.d + (size_t)s * p.split_stride;
#pragma unroll
                for (int it = 0; it < IT; ++it) {
                    const int j = (it * 32 + lane) * E;
                    const Piece<E> dl = load_piece<E>(src + j), dh = load_piece<E>(src + half + j);
#pragma unroll
                    for (int e = 0; e < E; ++e) { lo[hh][it].v[e] += dl.v[e]; hi[hh][it].v[e] += dh.v[e]; }
                }
            }
        }
    }
    // what all heads of the token share: position, cos and sin, the cache page, the norm weights
    const int pos = p.token_pos[t];
    const float* cs = p.cos_sin + (size_t)(pos < p.max_pos ? pos : p.max_pos - 1) * p.d;
    Piece<E> c[IT], sn[IT], wq_lo[IT], wq_hi[IT], wk_lo[IT], wk_hi[IT];
#pragma unroll
    for (int it = 0; it < IT; ++it) {
        const int j = (it * 32 + lane) * E;
        c[it] = load_piece<E>(cs + j);
        sn[it] = load_piece<E>(cs + half + j);
        if (p.q_weight) { wq_lo[it] = load_piece<E>(p.q_weight + j); wq_hi[it] = load_piece<E>(p.q_weight + half + j); }
        if (p.k_weight) { wk_lo[it] = load_piece<E>(p.k_weight + j); wk_hi[it] = load_piece<E>(p.k_weight + half + j); }
    }
    size_t cache_row = 0;    // element offset of (page, kv head 0, token) in the caches
    if (p.write_kv && head0 + HEADS_PER_WARP > p.nq) {
        const int slot_pos = p.ring_tokens > 0 ? pos % p.ring_tokens : pos;
        const int page = p.block_table[(size_t)p.token_seq[t] * p.max_blocks + slot_pos / p.page_tokens];
        cache_row = ((size_t)page * p.nkv * p.page_tokens + (slot_pos % p.page_tokens)) * (size_t)p.d;
    }
    const size_t head_stride = (size_t)p.page_tokens * p.d;
    const float inv_d = 1.f / (float)p.d;
#pragma unroll
    for (int hh = 0; hh < HEADS_PER_WARP; ++hh) {
        const int head = head0 + hh;
        if (head >= heads_total) break;
        const bool is_q = head < p.nq, is_k = !is_q && head < p.nq + p.nkv;
        if (!is_q && !p.write_kv) break;
        TO* dst;
        if (is_q) dst = (TO*)p.q_out + ((size_t)t * p.nq + head) * p.d;
        else if (is_k) dst = (TO*)p.k_cache + cache_row + (size_t)(head - p.nq) * head_stride;
        else dst = (TO*)p.v_cache + cache_row + (size_t)(head - p.nq - p.nkv) * head_stride;
        const bool normed = is_q ? p.q_weight != nullptr : (is_k && p.k_weight != nullptr);
        float inv = 1.f;
        if (normed) {
            float sq = 0.f;
#pragma unroll
            for (int it = 0; it < IT; ++it)
#pragma unroll
                for (int e = 0; e < E; ++e) sq += lo[hh][it].v[e] * lo[hh][it].v[e] + hi[hh][it].v[e] * hi[hh][it].v[e];
            inv = rsqrtf(warp_sum(sq) * inv_d + p.eps);
        }
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            const int j = (it * 32 + lane) * E;
            Piece<E> a = lo[hh][it], b = hi[hh][it];
            if (normed) {
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    a.v[e] = a.v[e] * inv * (is_q ? wq_lo[it].v[e] : wk_lo[it].v[e]);
                    b.v[e] = b.v[e] * inv * (is_q ? wq_hi[it].v[e] : wk_hi[it].v[e]);
                }
            }
            if (is_q || is_k) {
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const float ya = a.v[e] * c[it].v[e] - b.v[e] * sn[it].v[e];
                    const float yb = b.v[e] * c[it].v[e] + a.v[e] * sn[it].v[e];
                    a.v[e] = ya; b.v[e] = yb;
                }
            }
            store_piece<E>(dst + j, a);
            store_piece<E>(dst + half + j, b);
        }
    }
}

extern "C" int qt_qk_norm_rope_write(const void* qkv, int in_dtype, int n_splits, long long split_stride, void* q_out,
                                     void* k_cache, void* v_cache, int out_dtype, const int* token_seq,
                                     const int* token_pos, const int* block_table, int max_blocks,
                                     const float* q_weight, const float* k_weight, float eps, const float* cos_sin,
                                     int rotary_dim, int max_pos, int n_tokens, int nq, int nkv, int d, int page_tokens,
                                     int ring_tokens, int write_kv, int kv_in_proj, int interleaved, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && nq > 0 && nkv > 0 && d > 0 && d <= 1024, "qk_norm_rope_write: bad sizes T=%d nq=%d nkv=%d d=%d", n_tokens, nq, nkv, d);
    QT_REQUIRE(rotary_dim >= 0 && rotary_dim <= d && rotary_dim % 2 == 0, "qk_norm_rope_write: rotary_dim=%d must be even and at most head_dim=%d", rotary_dim, d);
    QT_REQUIRE(rotary_dim == 0 || (cos_sin && max_pos > 0), "qk_norm_rope_write: rotation needs a cos/sin table");
    QT_REQUIRE(page_tokens > 0 && n_splits >= 1 && ring_tokens >= 0, "qk_norm_rope_write: bad cache geometry");
    QT_REQUIRE(!write_kv || (k_cache && v_cache && block_table), "qk_norm_rope_write: cache pointers missing");
    QT_REQUIRE(!write_kv || kv_in_proj, "qk_norm_rope_write: nothing to write without k and v in the projection");
    if (n_tokens == 0) return QT_OK;
    QkvParams p{qkv, n_splits, (size_t)split_stride, q_out, k_cache, v_cache, token_seq, token_pos, block_table, max_blocks,
                q_weight, k_weight, eps, cos_sin, rotary_dim, max_pos, n_tokens, nq, nkv, d, page_tokens, ring_tokens, write_kv, kv_in_proj, interleaved};
    const int warps = 4;
    const long long items = (long long)n_tokens * (nq + (kv_in_proj ? 2 * nkv : 0));
    const unsigned grid = (unsigned)((items + warps - 1) / warps);
    const size_t smem = (size_t)warps * d * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    // 16-byte loads and stores need head_dim % 8 == 0 (bfloat16 rows of the cache and of q) and aligned bases
    const bool vec = d % 8 == 0 && split_stride % 8 == 0 && ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)q_out % 16 == 0) &&
                     (!write_kv || (((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0)));
    // the register form: all dimensions rotate, half a head is one or two rounds of 32 or 64 elements, enough tokens
    // to fill the machine with a few heads per warp
    const int half = d / 2;
    int pe = 0, pit = 0;
    if (interleaved) { pe = 0; }                     // the register form pairs (i, i + d/2)
    else if (rotary_dim == d && half % 64 == 0 && half / 64 <= 2) { pe = 2; pit = half / 64; }
    else if (rotary_dim == d && half == 32) { pe = 1; pit = 1; }
    const bool pair_aligned = split_stride % 2 == 0 && ((uintptr_t)qkv % 8 == 0) && ((uintptr_t)q_out % 8 == 0) && ((uintptr_t)cos_sin % 8 == 0) &&
                              (!q_weight || (uintptr_t)q_weight % 8 == 0) && (!k_weight || (uintptr_t)k_weight % 8 == 0) &&
                              (!write_kv || (((uintptr_t)k_cache % 8 == 0) && ((uintptr_t)v_cache % 8 == 0)));
    if (pe && pair_aligned && n_tokens >= 256 && nq + 2 * nkv <= 65535 * 16 && (in_dtype == QT_F32 || in_dtype == QT_BF16) && out_dtype == QT_BF16) {
        const int heads_total = nq + (kv_in_proj ? 2 * nkv : 0);
        const dim3 pgrid((unsigned)n_tokens, (unsigned)((heads_total + warps * HEADS_PER_WARP - 1) / (warps * HEADS_PER_WARP)));
#define QT_LAUNCH_PAIRS(TI, E, IT) launch_kernel(qk_norm_rope_pairs_kernel<TI, __nv_bfloat16, E, IT>, pgrid, dim3(warps * 32), 0, s, p)
        if (in_dtype == QT_BF16) {
            if (pe == 2 && pit == 1) QT_LAUNCH_PAIRS(__nv_bfloat16, 2, 1);
            else if (pe == 2) QT_LAUNCH_PAIRS(__nv_bfloat16, 2, 2);
            else QT_LAUNCH_PAIRS(__nv_bfloat16, 1, 1);
        } else {
            if (pe == 2 && pit == 1) QT_LAUNCH_PAIRS(float, 2, 1);
            else if (pe == 2) QT_LAUNCH_PAIRS(float, 2, 2);
            else QT_LAUNCH_PAIRS(float, 1, 1);
        }
#undef QT_LAUNCH_PAIRS
        QT_CHECK_LAUNCH("qk_norm_rope_write");
        return QT_OK;
    }
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

// ----------------------------------------------------------------------------- gated product
// out[t, i] = act(g) * u (act: SiLU or another of QT_ACT_*); float inside.  Plain layout (group 0): g = gate_up[t, i], u = gate_up[t, inter + i].
// Interleaved layout (group G, the fused weight's rows alternate G of gate and G of up, which is what lets a GEMM
// epilogue see both in one warp): g = gate_up[t, (i / G) * 2G + i % G], u = the element G further on.
__device__ __forceinline__ size_t gate_column(int i, int group) { return group ? (size_t)(i / group) * 2 * group + i % group : (size_t)i; }

template <typename TI, typename TO>
__global__ void swiglu_kernel(const TI* __restrict__ gate_up, int n_splits, size_t split_stride, TO* __restrict__ out,
                              long long total, int inter, int group, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int up_offset = group ? group : inter;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / inter;
        const int i = (int)(idx % inter);
        const size_t base = (size_t)t * 2 * inter + gate_column(i, group);
        const float g = load_sum(gate_up, base, n_splits, split_stride);
        const float u = load_sum(gate_up, base + up_offset, n_splits, split_stride);
        out[idx] = from_float<TO>(gate_activation<false>(g, act) * u);
    }
}

// Eight elements per thread with 16- or 32-byte loads and stores (widths that are multiples of 8, aligned bases).
// blockIdx.x is the token, blockIdx.y a run of chunks of its row.
struct Float8 { float4 a, b; };
__device__ __forceinline__ Float8 load8(const float* p) { return {load4(p), load4(p + 4)}; }
__device__ __forceinline__ Float8 load8(const __nv_bfloat16* p) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    return {make_float4(__low2float(h[0]), __high2float(h[0]), __low2float(h[1]), __high2float(h[1])),
            make_float4(__low2float(h[2]), __high2float(h[2]), __low2float(h[3]), __high2float(h[3]))};
}
__device__ __forceinline__ void store8(float* p, const Float8& v) { store4(p, v.a); store4(p + 4, v.b); }
__device__ __forceinline__ void store8(__nv_bfloat16* p, const Float8& v) {
    __nv_bfloat162 h[4] = {__floats2bfloat162_rn(v.a.x, v.a.y), __floats2bfloat162_rn(v.a.z, v.a.w),
                           __floats2bfloat162_rn(v.b.x, v.b.y), __floats2bfloat162_rn(v.b.z, v.b.w)};
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(h);
}
__device__ __forceinline__ void add4(float4& x, const float4& y) { x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w; }
// silu(g) * u.  For a float result the exponential and the division are the library's; for a bfloat16 result
// (8 bits of mantissa) the hardware approximations (2 ulp of float) are used: with the exact forms the kernel was
// bound by instruction issue, not by memory.
template <typename TO> __device__ __forceinline__ float silu_mul(float g, float u, int act) { return gate_activation<false>(g, act) * u; }
template <> __device__ __forceinline__ float silu_mul<__nv_bfloat16>(float g, float u, int act) { return gate_activation<true>(g, act) * u; }
template <typename TO> __device__ __forceinline__ float4 silu_mul4(const float4& g, const float4& u, int act) {
    return make_float4(silu_mul<TO>(g.x, u.x, act), silu_mul<TO>(g.y, u.y, act), silu_mul<TO>(g.z, u.z, act), silu_mul<TO>(g.w, u.w, act));
}

// PT chunks per thread, all loads issued before the first store.
template <typename TI, typename TO, int PT>
__global__ void swiglu_vec_kernel(const TI* __restrict__ gate_up, int n_splits, size_t split_stride, TO* __restrict__ out,
                                  int inter, int group, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int chunks = inter >> 3;
    const int up_offset = group ? group : inter;
    const TI* row = gate_up + (size_t)blockIdx.x * 2 * inter;
    TO* orow = out + (size_t)blockIdx.x * inter;
    for (int c0 = blockIdx.y * blockDim.x * PT + threadIdx.x; c0 < chunks; c0 += gridDim.y * blockDim.x * PT) {
        Float8 g[PT], u[PT];
#pragma unroll
        for (int i = 0; i < PT; ++i) {
            const int c = c0 + i * blockDim.x;
            if (c < chunks) { const size_t at = gate_column(8 * c, group); g[i] = load8(row + at); u[i] = load8(row + at + up_offset); }
        }
        for (int s = 1; s < n_splits; ++s) {
#pragma unroll
            for (int i = 0; i < PT; ++i) {
                const int c = c0 + i * blockDim.x;
                if (c < chunks) {
                    const size_t at = gate_column(8 * c, group) + (size_t)s * split_stride;
                    const Float8 dg = load8(row + at), du = load8(row + at + up_offset);
                    add4(g[i].a, dg.a); add4(g[i].b, dg.b); add4(u[i].a, du.a); add4(u[i].b, du.b);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < PT; ++i) {
            const int c = c0 + i * blockDim.x;
            if (c < chunks) store8(orow + 8 * c, Float8{silu_mul4<TO>(g[i].a, u[i].a, act), silu_mul4<TO>(g[i].b, u[i].b, act)});
        }
    }
}

extern "C" int qt_swiglu(const void* gate_up, int in_dtype, int n_splits, long long split_stride, void* out, int out_dtype,
                         int n_tokens, int inter, int group, int act, void* stream) {
    QT_REQUIRE(act >= 0 && act < QT_ACT_COUNT, "swiglu: unknown activation code %d", act);
    QT_REQUIRE(n_tokens >= 0 && inter > 0 && n_splits >= 1, "swiglu: bad sizes T=%d I=%d", n_tokens, inter);
    QT_REQUIRE(group >= 0 && (group == 0 || inter % group == 0), "swiglu: rows interleaved in groups of %d do not divide I=%d", group, inter);
    if (n_tokens == 0) return QT_OK;
    const long long total = (long long)n_tokens * inter;
    const int threads = 256;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = inter % 8 == 0 && group % 8 == 0 && split_stride % 8 == 0 && ((uintptr_t)gate_up % 16 == 0) && ((uintptr_t)out % 16 == 0);
    long long blocks = (total + threads - 1) / threads;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
    // few tokens (decode): one chunk per thread, most blocks; many tokens (prefill): two chunks per thread
    const int per_thread = n_tokens >= 256 ? 2 : 1;
    unsigned per_row = (unsigned)((inter / 8 + threads * per_thread - 1) / (threads * per_thread));
    if (per_row > 65535u) per_row = 65535u;
#define QT_LAUNCH_SWIGLU(TI, TO)                                                                                              \
    do {                                                                                                                      \
        if (vec && per_thread == 2) launch_kernel(swiglu_vec_kernel<TI, TO, 2>, dim3((unsigned)n_tokens, per_row), dim3(threads), 0, s, \
                               (const TI*)gate_up, n_splits, (size_t)split_stride, (TO*)out, inter, group, act);              \
        else if (vec) launch_kernel(swiglu_vec_kernel<TI, TO, 1>, dim3((unsigned)n_tokens, per_row), dim3(threads), 0, s,     \
                               (const TI*)gate_up, n_splits, (size_t)split_stride, (TO*)out, inter, group, act);              \
        else launch_kernel(swiglu_kernel<TI, TO>, dim3((unsigned)blocks), dim3(threads), 0, s, (const TI*)gate_up, n_splits,  \
                           (size_t)split_stride, (TO*)out, total, inter, group, act);                                         \
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
