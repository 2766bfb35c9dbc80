// Attention over the paged cache for any element type and head size: a tiled online-softmax
// kernel for steps with many tokens per sequence (prefill and continuation chunks), and a
// split-KV kernel with a combine pass for one token per sequence (decode).  Scores, softmax
// and the weighted sum are float.  Grouped-query attention: query head h reads kv head
// h / (nq / nkv).  Key j is visible to the query at absolute position p iff j <= p and, for a
// windowed group, j > p - window.
//
// Counterparts in luozoupi/Qwen-Triton: kernels/flash_attention.py:54-152 (one kernel for both
// cases, no split, no window) and the masked SDPA branch of modules/attention.py:110-123 with
// the mask of models/core.py:47-74.
#include "common.cuh"

#include <math.h>

using namespace qt;

struct AttnParams {
    const void* q;        // [T, nq, d]
    const void* k_cache;  // [pages, nkv, page_tokens, d]
    const void* v_cache;
    void* out;            // [T, nq, d]
    const int* block_table; int max_blocks;
    const int* seq_start;  // [B + 1] first token row of each sequence in this step
    const int* seq_past;   // [B] tokens already in the cache before this step
    int n_seqs, nq, nkv, d, page_tokens, ring_tokens, window;   // window <= 0: all keys
    float scale;
};

// ----------------------------------------------------------------------------- many tokens per sequence
constexpr int PF_BQ = 16;       // queries per block
constexpr int PF_BK = 32;       // keys per tile (one per lane)
constexpr int PF_WARPS = 4;     // warp w owns query rows w, w + 4, w + 8, w + 12
constexpr int PF_ROWS = PF_BQ / PF_WARPS;

template <typename T, int DMAX>
__global__ void __launch_bounds__(PF_WARPS * 32) attention_prefill_kernel(const AttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int d = p.d;
    const int kstride = d + 1;
    float* qs = smem;                         // [PF_BQ][d]
    float* ks = qs + PF_BQ * d;               // [PF_BK][d + 1]
    float* vs = ks + PF_BK * kstride;         // [PF_BK][d]
    float* ps = vs + PF_BK * d;               // [PF_BQ][PF_BK]

    const int seq = blockIdx.z, head = blockIdx.y;
    const int q_begin = p.seq_start[seq], q_len = p.seq_start[seq + 1] - q_begin;
    const int q0 = blockIdx.x * PF_BQ;
    if (q0 >= q_len) return;
    const int rows = min(PF_BQ, q_len - q0);
    const int past = p.seq_past[seq];
    const int kvh = head / (p.nq / p.nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* table = p.block_table + (size_t)seq * p.max_blocks;
    const T* q = (const T*)p.q;
    const T* kc = (const T*)p.k_cache;
    const T* vc = (const T*)p.v_cache;

    for (int r = warp; r < PF_BQ; r += PF_WARPS)
        for (int c = lane; c < d; c += 32)
            qs[r * d + c] = r < rows ? to_float(q[((size_t)(q_begin + q0 + r) * p.nq + head) * d + c]) * p.scale : 0.f;

    float m[PF_ROWS], l[PF_ROWS], acc[PF_ROWS][DMAX / 32];
#pragma unroll
    for (int i = 0; i < PF_ROWS; ++i) {
        m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
        for (int j = 0; j < DMAX / 32; ++j) acc[i][j] = 0.f;
    }

    const int p_first = past + q0, p_last = past + q0 + rows - 1;
    const int key_lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;
    for (int k0 = key_lo; k0 <= p_last; k0 += PF_BK) {
        __syncthreads();
        for (int r = warp; r < PF_BK; r += PF_WARPS) {
            const int key = k0 + r;
            if (key <= p_last) {
                const size_t off = cache_offset(table, key, p.ring_tokens, p.page_tokens, p.nkv, kvh, d);
                for (int c = lane; c < d; c += 32) {
                    ks[r * kstride + c] = to_float(kc[off + c]);
                    vs[r * d + c] = to_float(vc[off + c]);
                }
            } else {
                for (int c = lane; c < d; c += 32) { ks[r * kstride + c] = 0.f; vs[r * d + c] = 0.f; }
            }
        }
        __syncthreads();
        const int key = k0 + lane;
#pragma unroll
        for (int i = 0; i < PF_ROWS; ++i) {
            const int r = warp + i * PF_WARPS;
            const int pos = past + q0 + r;
            float s = 0.f;
            for (int c = 0; c < d; ++c) s += qs[r * d + c] * ks[lane * kstride + c];
            const bool visible = r < rows && key <= pos && (p.window <= 0 || key > pos - p.window);
            s = visible ? s : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(s));
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float e = visible ? expf(s - m_use) : 0.f;
            const float alpha = expf(m[i] - m_use);   // m[i] = -inf gives 0, and nothing is accumulated yet
            l[i] = l[i] * alpha + warp_sum(e);
            m[i] = m_new;
            ps[r * PF_BK + lane] = e;
#pragma unroll
            for (int j = 0; j < DMAX / 32; ++j) acc[i][j] *= alpha;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < PF_ROWS; ++i) {
            const int r = warp + i * PF_WARPS;
            for (int kk = 0; kk < PF_BK; ++kk) {
                const float w = ps[r * PF_BK + kk];
#pragma unroll
                for (int j = 0; j < DMAX / 32; ++j) {
                    const int c = lane + 32 * j;
                    if (c < d) acc[i][j] += w * vs[kk * d + c];
                }
            }
        }
    }
    T* out = (T*)p.out;
#pragma unroll
    for (int i = 0; i < PF_ROWS; ++i) {
        const int r = warp + i * PF_WARPS;
        if (r >= rows) continue;
        const float inv = 1.f / l[i];
#pragma unroll
        for (int j = 0; j < DMAX / 32; ++j) {
            const int c = lane + 32 * j;
            if (c < d) out[((size_t)(q_begin + q0 + r) * p.nq + head) * d + c] = from_float<T>(acc[i][j] * inv);
        }
    }
}

template <typename T, int DMAX>
static int launch_prefill(const AttnParams& p, int max_q_len, cudaStream_t stream) {
    const size_t smem = ((size_t)PF_BQ * p.d + (size_t)PF_BK * (p.d + 1) + (size_t)PF_BK * p.d + PF_BQ * PF_BK) * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(attention_prefill_kernel<T, DMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "attention_prefill: cannot raise shared memory: %s", cudaGetErrorString(err));
        configured = true;
    }
    dim3 grid((max_q_len + PF_BQ - 1) / PF_BQ, p.nq, p.n_seqs);
    launch_kernel(attention_prefill_kernel<T, DMAX>, dim3(grid), dim3(PF_WARPS * 32), smem, stream, p);
    QT_CHECK_LAUNCH("attention_prefill");
    return QT_OK;
}

static int check_common(const char* name, int n_seqs, int nq, int nkv, int d, int page_tokens, int ring_tokens, int window) {
    QT_REQUIRE(n_seqs > 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "%s: bad head counts nq=%d nkv=%d (B=%d)", name, nq, nkv, n_seqs);
    QT_REQUIRE(d > 0 && d <= 256, "%s: head_dim=%d is outside 1..256", name, d);
    QT_REQUIRE(page_tokens > 0 && ring_tokens >= 0, "%s: bad cache geometry", name);
    QT_REQUIRE(ring_tokens == 0 || (window > 0 && ring_tokens >= window), "%s: a ring of %d tokens cannot hold a window of %d", name, ring_tokens, window);
    return QT_OK;
}

extern "C" int qt_attention_prefill(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype,
                                    const int* block_table, int max_blocks, const int* seq_start, const int* seq_past,
                                    int n_seqs, int max_q_len, int nq, int nkv, int d, int page_tokens, int ring_tokens,
                                    int window, float scale, void* stream) {
    if (n_seqs == 0 || max_q_len == 0) return QT_OK;
    int rc = check_common("attention_prefill", n_seqs, nq, nkv, d, page_tokens, ring_tokens, window);
    if (rc) return rc;
    QT_REQUIRE(nq <= 65535 && n_seqs <= 65535, "attention_prefill: too many heads or sequences for one launch");
    AttnParams p{q, k_cache, v_cache, out, block_table, max_blocks, seq_start, seq_past, n_seqs, nq, nkv, d, page_tokens, ring_tokens, window, scale};
    cudaStream_t s = (cudaStream_t)stream;
    return QT_DISPATCH_DTYPE(dtype, "attention_prefill", {
        if (d <= 64) return launch_prefill<T, 64>(p, max_q_len, s);
        if (d <= 128) return launch_prefill<T, 128>(p, max_q_len, s);
        return launch_prefill<T, 256>(p, max_q_len, s);
    });
}

// ----------------------------------------------------------------------------- one token per sequence
// grid (split, kv head x head chunk, sequence).  A block handles up to DEC_HEADS (1, 2, 4 or 8) query heads of one
// kv head over the keys [lo + split * chunk, lo + (split + 1) * chunk) of its sequence, where
// [lo, len) is the visible range.  QK: one key per lane.  PV: one column group per lane.
// The partial result (max, sum, unnormalised accumulator) goes to scratch; the combine kernel
// merges the splits.  With one split the block writes the output itself.
constexpr int DEC_WARPS = 4;

struct DecodeParams {
    AttnParams a;
    const int* seq_len;   // [B] keys visible to the token of this step (its own included)
    int n_splits;
    float* part_acc;      // [B, nq, n_splits, d]
    float* part_ml;       // [B, nq, n_splits, 2]
};

template <typename T, int DMAX, int DEC_HEADS>
__global__ void __launch_bounds__(DEC_WARPS * 32) attention_decode_kernel(const DecodeParams dp) {
    pdl_launch_dependents();
    pdl_wait();
    const AttnParams& p = dp.a;
    extern __shared__ float smem[];
    const int d = p.d;
    const int group = p.nq / p.nkv;
    const int chunks_per_kv = (group + DEC_HEADS - 1) / DEC_HEADS;
    const int kvh = blockIdx.y / chunks_per_kv;
    const int h0 = (blockIdx.y % chunks_per_kv) * DEC_HEADS;          // first head of the chunk within the group
    const int nh = min(DEC_HEADS, group - h0);
    const int seq = blockIdx.z, split = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* qs = smem;                                   // [DEC_HEADS][d], scaled
    float* red_acc = qs + DEC_HEADS * d;                // [DEC_WARPS][DEC_HEADS][d]
    float* red_ml = red_acc + DEC_WARPS * DEC_HEADS * d; // [DEC_WARPS][DEC_HEADS][2]

    const int len = dp.seq_len[seq];
    const int lo = p.window > 0 ? max(0, len - p.window) : 0;
    const int span = len - lo;
    const int chunk = (span + dp.n_splits - 1) / dp.n_splits;
    const int k_begin = lo + split * chunk;
    const int k_end = min(len, k_begin + chunk);
    const int* table = p.block_table + (size_t)seq * p.max_blocks;
    const T* q = (const T*)p.q;
    const T* kc = (const T*)p.k_cache;
    const T* vc = (const T*)p.v_cache;
    const int head_base = kvh * group + h0;

    for (int i = threadIdx.x; i < DEC_HEADS * d; i += blockDim.x) {
        const int h = i / d, c = i % d;
        qs[i] = h < nh ? to_float(q[((size_t)seq * p.nq + head_base + h) * d + c]) * p.scale : 0.f;
    }
    __syncthreads();

    float m[DEC_HEADS], l[DEC_HEADS], acc[DEC_HEADS][DMAX / 32];
#pragma unroll
    for (int h = 0; h < DEC_HEADS; ++h) {
        m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
        for (int j = 0; j < DMAX / 32; ++j) acc[h][j] = 0.f;
    }

    for (int k0 = k_begin + warp * 32; k0 < k_end; k0 += DEC_WARPS * 32) {
        const int key = k0 + lane;
        const bool valid = key < k_end;
        float s[DEC_HEADS];
#pragma unroll
        for (int h = 0; h < DEC_HEADS; ++h) s[h] = 0.f;
        if (valid) {
            const T* krow = kc + cache_offset(table, key, p.ring_tokens, p.page_tokens, p.nkv, kvh, d);
            for (int c = 0; c < d; ++c) {
                const float kv = to_float(krow[c]);
#pragma unroll
                for (int h = 0; h < DEC_HEADS; ++h) s[h] += qs[h * d + c] * kv;
            }
        }
        float e[DEC_HEADS];
#pragma unroll
        for (int h = 0; h < DEC_HEADS; ++h) {
            const float sv = valid ? s[h] : -INFINITY;
            const float m_new = fmaxf(m[h], warp_max(sv));      // at least one key of the tile is valid
            e[h] = valid ? expf(sv - m_new) : 0.f;
            const float alpha = expf(m[h] - m_new);
            l[h] = l[h] * alpha + warp_sum(e[h]);
            m[h] = m_new;
#pragma unroll
            for (int j = 0; j < DMAX / 32; ++j) acc[h][j] *= alpha;
        }
        const int n_keys = min(32, k_end - k0);
        for (int kk = 0; kk < n_keys; ++kk) {
            const T* vrow = vc + cache_offset(table, k0 + kk, p.ring_tokens, p.page_tokens, p.nkv, kvh, d);
            float v[DMAX / 32];
#pragma unroll
            for (int j = 0; j < DMAX / 32; ++j) {
                const int c = lane + 32 * j;
                v[j] = c < d ? to_float(vrow[c]) : 0.f;
            }
#pragma unroll
            for (int h = 0; h < DEC_HEADS; ++h) {
                const float w = __shfl_sync(0xffffffffu, e[h], kk);
#pragma unroll
                for (int j = 0; j < DMAX / 32; ++j) acc[h][j] += w * v[j];
            }
        }
    }

    // merge the warps of the block
#pragma unroll
    for (int h = 0; h < DEC_HEADS; ++h) {
        if (lane == 0) { red_ml[(warp * DEC_HEADS + h) * 2] = m[h]; red_ml[(warp * DEC_HEADS + h) * 2 + 1] = l[h]; }
#pragma unroll
        for (int j = 0; j < DMAX / 32; ++j) {
            const int c = lane + 32 * j;
            if (c < d) red_acc[(warp * DEC_HEADS + h) * d + c] = acc[h][j];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nh * d; i += blockDim.x) {
        const int h = i / d, c = i % d;
        float m_all = -INFINITY;
        for (int w = 0; w < DEC_WARPS; ++w) m_all = fmaxf(m_all, red_ml[(w * DEC_HEADS + h) * 2]);
        float l_all = 0.f, a_all = 0.f;
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float mw = red_ml[(w * DEC_HEADS + h) * 2];
            const float f = mw == -INFINITY ? 0.f : expf(mw - m_all);
            l_all += red_ml[(w * DEC_HEADS + h) * 2 + 1] * f;
            a_all += red_acc[(w * DEC_HEADS + h) * d + c] * f;
        }
        const int head = head_base + h;
        if (dp.n_splits == 1) {
            ((T*)p.out)[((size_t)seq * p.nq + head) * d + c] = from_float<T>(a_all / l_all);
        } else {
            const size_t slot = ((size_t)seq * p.nq + head) * dp.n_splits + split;
            dp.part_acc[slot * d + c] = a_all;
            if (c == 0) { dp.part_ml[slot * 2] = m_all; dp.part_ml[slot * 2 + 1] = l_all; }
        }
    }
}

// One block per (sequence, head): out = sum_s acc_s e^{m_s - m} / sum_s l_s e^{m_s - m}; empty splits have m = -inf.
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                         T* __restrict__ out, int n_splits, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t item = blockIdx.x;   // seq * nq + head
    float m_all = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m_all = fmaxf(m_all, part_ml[(item * n_splits + s) * 2]);
    float l_all = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part_ml[(item * n_splits + s) * 2];
        l_all += ms == -INFINITY ? 0.f : part_ml[(item * n_splits + s) * 2 + 1] * expf(ms - m_all);
    }
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part_ml[(item * n_splits + s) * 2];
            if (ms != -INFINITY) a += part_acc[(item * n_splits + s) * d + c] * expf(ms - m_all);
        }
        out[item * d + c] = from_float<T>(a / l_all);
    }
}

template <typename T, int DMAX, int DEC_HEADS>
static int launch_decode_heads(const DecodeParams& dp, cudaStream_t stream) {
    const AttnParams& p = dp.a;
    const size_t smem = ((size_t)DEC_HEADS * p.d + (size_t)DEC_WARPS * DEC_HEADS * p.d + DEC_WARPS * DEC_HEADS * 2) * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(attention_decode_kernel<T, DMAX, DEC_HEADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "attention_decode: cannot raise shared memory: %s", cudaGetErrorString(err));
        configured = true;
    }
    const int group = p.nq / p.nkv;
    dim3 grid(dp.n_splits, p.nkv * ((group + DEC_HEADS - 1) / DEC_HEADS), p.n_seqs);
    launch_kernel(attention_decode_kernel<T, DMAX, DEC_HEADS>, dim3(grid), dim3(DEC_WARPS * 32), smem, stream, dp);
    QT_CHECK_LAUNCH("attention_decode");
    if (dp.n_splits > 1) {
        launch_kernel(attention_combine_kernel<T>, dim3(p.n_seqs * p.nq), dim3(128), 0, stream, dp.part_acc, dp.part_ml, (T*)p.out, dp.n_splits, p.d);
        QT_CHECK_LAUNCH("attention_combine");
    }
    return QT_OK;
}

template <typename T, int DMAX>
static int launch_decode(const DecodeParams& dp, cudaStream_t stream) {
    const int group = dp.a.nq / dp.a.nkv;
    if (group == 1) return launch_decode_heads<T, DMAX, 1>(dp, stream);
    if (group == 2) return launch_decode_heads<T, DMAX, 2>(dp, stream);
    if (group <= 4) return launch_decode_heads<T, DMAX, 4>(dp, stream);
    return launch_decode_heads<T, DMAX, 8>(dp, stream);
}

// Scratch the caller provides for n_splits > 1: part_acc of B * nq * n_splits * d floats and
// part_ml of B * nq * n_splits * 2 floats.
extern "C" int qt_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype,
                                   const int* block_table, int max_blocks, const int* seq_len, int n_seqs, int nq,
                                   int nkv, int d, int page_tokens, int ring_tokens, int window, float scale,
                                   int n_splits, float* part_acc, float* part_ml, void* stream) {
    if (n_seqs == 0) return QT_OK;
    int rc = check_common("attention_decode", n_seqs, nq, nkv, d, page_tokens, ring_tokens, window);
    if (rc) return rc;
    QT_REQUIRE(n_splits >= 1 && n_splits <= 65535, "attention_decode: n_splits=%d", n_splits);
    QT_REQUIRE(n_splits == 1 || (part_acc && part_ml), "attention_decode: split results need scratch memory");
    QT_REQUIRE(n_seqs <= 65535, "attention_decode: too many sequences for one launch");
    DecodeParams dp{{q, k_cache, v_cache, out, block_table, max_blocks, nullptr, nullptr, n_seqs, nq, nkv, d, page_tokens, ring_tokens, window, scale},
                    seq_len, n_splits, part_acc, part_ml};
    cudaStream_t s = (cudaStream_t)stream;
    return QT_DISPATCH_DTYPE(dtype, "attention_decode", {
        if (d <= 64) return launch_decode<T, 64>(dp, s);
        if (d <= 128) return launch_decode<T, 128>(dp, s);
        return launch_decode<T, 256>(dp, s);
    });
}

QT_DEFINE_LAST_ERROR(attention)
