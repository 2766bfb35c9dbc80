// What follows a decode step's product, as device functions shared by the kernels that run it in their epilogue
// (gemm_fused.cu: one launch per product; gemm_chain.cu: one persistent launch for a run of products).
//
//   STORE     out[m, n] = s_m * y                       float or bfloat16 (the output head)
//   RESIDUAL  r = residual[m, n] + y; residual[m, n] = r;  and, for the norm that follows, xw[m, n] = bf16(r * g[n])
//             and sq_out[tile, m] = sum over the tile's 128 columns of r^2
//   SWIGLU    act[m, f] = a(s_m * gate) * (s_m * up), a = SiLU or another QT_ACT_*, the weight's rows alternating 16 of gate and 16 of up
//   QKV       per head (head_dim divides 128): s_m * y, RMSNorm over the head with q or k weight, rotation by the
//             cos/sin table at the token's position (pairs (i, i + rd/2) or (2i, 2i + 1)), then q to q_out and k, v
//             into the paged cache
//
// s_m is the factor of an RMSNorm whose weight g was applied by the producer of X (X = bf16(r * g)):
// s_m = rsqrt(sum over tiles of sq_in[tile, m] / hidden + eps); the product is linear in X, so scaling the result
// equals normalising the input.  sq_in == nullptr means s_m = 1.  Partial sums of squares are kept per tile and added
// in a fixed order: results do not depend on scheduling.
//
// One warp finishes one (token, 128-column tile): lane l holds columns 4 l .. 4 l + 3 of the tile (for SWIGLU the
// gate and up values of features 2 l, 2 l + 1).
#pragma once

#include "common.cuh"

namespace qt_epi {

using namespace qt;

constexpr int TILE = 128;      // weight rows (output columns) per tile

enum Epilogue { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2, EPI_QKV = 3 };

struct EpilogueParams {
    int M, N;
    // the deferred factor of the norm in front of this product
    const float* sq_in; int sq_tiles; float inv_hidden; float eps;
    // STORE / SWIGLU
    void* out; int out_is_float; int act;      // act: the gate's activation, QT_ACT_*
    // RESIDUAL
    float* residual; const float* norm_w; __nv_bfloat16* xw; float* sq_out;
    // QKV
    __nv_bfloat16* q_out; __nv_bfloat16* k_cache; __nv_bfloat16* v_cache;
    const int* token_seq; const int* token_pos; const int* block_table; int max_blocks;
    const float* q_w; const float* k_w; float qk_eps;
    const float* cos_sin; int rotary_dim; int max_pos;
    int nq, nkv, d, page_tokens, ring_tokens, write_kv;
    int interleaved;        // QKV: rotation pairs are (2i, 2i + 1) instead of (i, i + rd/2)
};

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }

// The factor of the deferred norm for token m: every lane of the warp gets it.
__device__ __forceinline__ float row_scale(const EpilogueParams& p, int m, int lane) {
    if (p.sq_in == nullptr) return 1.f;
    float s = 0.f;
    for (int i = lane; i < p.sq_tiles; i += 32) s += p.sq_in[(size_t)i * p.M + m];
    return rsqrtf(warp_sum(s) * p.inv_hidden + p.eps);
}

// What the epilogue of one (token, tile) needs from global memory besides the product itself.  It depends only on
// what ran before the product, so it can be asked for ahead of the product's last sums.
struct Operands {
    float scale;            // the deferred norm factor of the token
    float4 a, b, c;         // RESIDUAL: stream piece, norm weight piece.  QKV: cos piece, sin piece, q/k norm weight piece
    int pos;                // QKV: the token's position
    long long cache_at;     // QKV: element offset of this lane's piece in the key or value cache
};

template <int EPI>
__device__ __forceinline__ Operands load_operands(const EpilogueParams& p, int m, int w0, int lane) {
    Operands o;
    o.scale = row_scale(p, m, lane);
    o.a = o.b = o.c = make_float4(0.f, 0.f, 0.f, 0.f);
    o.pos = 0;
    o.cache_at = 0;
    const int n = w0 + 4 * lane;
    if (EPI == EPI_RESIDUAL) {
        if (n < p.N) {
            o.a = ld4(p.residual + (size_t)m * p.N + n);
            if (p.norm_w) o.b = ld4(p.norm_w + n);
        }
    } else if (EPI == EPI_QKV) {
        const int d = p.d, head = n / d, c = n - head * d, half = p.rotary_dim >> 1;
        const bool valid = head < p.N / d, is_q = head < p.nq, is_k = !is_q && head < p.nq + p.nkv;
        const float* w = is_q ? p.q_w : (is_k ? p.k_w : nullptr);
        o.pos = p.token_pos[m];
        if (valid && w) o.c = ld4(w + c);
        if (valid && (is_q || is_k) && c < p.rotary_dim) {
            const float* row = p.cos_sin + (size_t)(o.pos < p.max_pos ? o.pos : p.max_pos - 1) * p.rotary_dim;
            if (p.interleaved) {                            // this lane's pairs c/2 and c/2 + 1
                const float2 co = *reinterpret_cast<const float2*>(row + (c >> 1)), si = *reinterpret_cast<const float2*>(row + half + (c >> 1));
                o.a = make_float4(co.x, co.y, 0.f, 0.f);
                o.b = make_float4(si.x, si.y, 0.f, 0.f);
            } else {
                const float* cs = row + (c < half ? c : c - half);
                o.a = ld4(cs);
                o.b = ld4(cs + half);
            }
        }
        if (valid && !is_q && p.write_kv) {
            const int kvh = is_k ? head - p.nq : head - p.nq - p.nkv;
            const int* table = p.block_table + (size_t)p.token_seq[m] * p.max_blocks;
            o.cache_at = (long long)cache_offset(table, o.pos, p.ring_tokens, p.page_tokens, p.nkv, kvh, d) + c;
        }
    }
    return o;
}

// SWIGLU: g and u are the gate and up sums of features 2 lane, 2 lane + 1 of tile w_tile (gate rows (f / 16) * 32 + f % 16
// of the tile, up rows 16 further).
__device__ __forceinline__ void finish_swiglu(const EpilogueParams& p, const Operands& ops, float2 g, float2 u, int m, int w_tile, int lane) {
    g.x *= ops.scale; g.y *= ops.scale; u.x *= ops.scale; u.y *= ops.scale;
    const int features = p.N >> 1, feature = w_tile * (TILE / 2) + 2 * lane;
    if (feature < features) {
        const float a0 = gate_activation<true>(g.x, p.act) * u.x, a1 = gate_activation<true>(g.y, p.act) * u.y;
        *reinterpret_cast<uint32_t*>((__nv_bfloat16*)p.out + (size_t)m * features + feature) = pack2(a0, a1);
    }
}
__device__ __forceinline__ int swiglu_gate_row(int lane) { const int f = 2 * lane; return (f >> 4) * 32 + (f & 15); }

// The other epilogues: v holds the sums of columns w_tile * 128 + 4 lane .. + 3 of token m.  The whole warp calls.
template <int EPI>
__device__ __forceinline__ void finish(const EpilogueParams& p, const Operands& ops, float4 v, int m, int w_tile, int lane) {
    const int n_rows = p.N, n = w_tile * TILE + 4 * lane;
    if (EPI == EPI_STORE) {
        v.x *= ops.scale; v.y *= ops.scale; v.z *= ops.scale; v.w *= ops.scale;
        const float e[4] = {v.x, v.y, v.z, v.w};
        if (p.out_is_float) {
            float* dst = (float*)p.out + (size_t)m * n_rows + n;
            if (n + 3 < n_rows && (n_rows & 3) == 0) *reinterpret_cast<float4*>(dst) = v;
            else for (int i = 0; i < 4; ++i) if (n + i < n_rows) dst[i] = e[i];
        } else {
            __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (size_t)m * n_rows + n;
            if (n + 3 < n_rows && (n_rows & 3) == 0) *reinterpret_cast<uint2*>(dst) = make_uint2(pack2(v.x, v.y), pack2(v.z, v.w));
            else for (int i = 0; i < 4; ++i) if (n + i < n_rows) dst[i] = __float2bfloat16_rn(e[i]);
        }
    } else if (EPI == EPI_RESIDUAL) {                       // N is a multiple of 4 (checked by the host)
        float sq = 0.f;
        if (n < n_rows) {
            v.x += ops.a.x; v.y += ops.a.y; v.z += ops.a.z; v.w += ops.a.w;
            *reinterpret_cast<float4*>(p.residual + (size_t)m * n_rows + n) = v;
            sq = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            if (p.norm_w)
                *reinterpret_cast<uint2*>(p.xw + (size_t)m * n_rows + n) =
                    make_uint2(pack2(v.x * ops.b.x, v.y * ops.b.y), pack2(v.z * ops.b.z, v.w * ops.b.w));
        }
        if (p.norm_w) {
            sq = warp_sum(sq);
            if (lane == 0) p.sq_out[(size_t)w_tile * p.M + m] = sq;
        }
    } else if (EPI == EPI_QKV) {
        const int d = p.d, lanes_per_head = d >> 2;
        v.x *= ops.scale; v.y *= ops.scale; v.z *= ops.scale; v.w *= ops.scale;
        const int head = n / d, c = n - head * d;
        const bool valid = head < n_rows / d;
        const bool is_q = head < p.nq, is_k = !is_q && head < p.nq + p.nkv;
        const bool normed = is_q ? p.q_w != nullptr : (is_k && p.k_w != nullptr);
        float sq = valid ? v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w : 0.f;
        for (int o = 1; o < lanes_per_head; o <<= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (valid && normed) {
            const float inv = rsqrtf(sq / (float)d + p.qk_eps);
            v.x *= inv * ops.c.x; v.y *= inv * ops.c.y; v.z *= inv * ops.c.z; v.w *= inv * ops.c.w;
        }
        const int half = p.rotary_dim >> 1;
        const bool rotates = valid && (is_q || is_k) && c < p.rotary_dim;
        const bool low = c < half;
        const int partner = rotates && !p.interleaved ? (low ? lane + (half >> 2) : lane - (half >> 2)) : lane;
        const float4 other = make_float4(__shfl_sync(0xffffffffu, v.x, partner), __shfl_sync(0xffffffffu, v.y, partner),
                                         __shfl_sync(0xffffffffu, v.z, partner), __shfl_sync(0xffffffffu, v.w, partner));
        if (rotates && p.interleaved) {                     // both elements of a pair sit in this lane
            const float x0 = v.x, x1 = v.y, x2 = v.z, x3 = v.w;
            v.x = x0 * ops.a.x - x1 * ops.b.x; v.y = x1 * ops.a.x + x0 * ops.b.x;
            v.z = x2 * ops.a.y - x3 * ops.b.y; v.w = x3 * ops.a.y + x2 * ops.b.y;
        } else if (rotates) {
            const float4 co = ops.a, si = ops.b;
            if (low) { v.x = v.x * co.x - other.x * si.x; v.y = v.y * co.y - other.y * si.y; v.z = v.z * co.z - other.z * si.z; v.w = v.w * co.w - other.w * si.w; }
            else { v.x = v.x * co.x + other.x * si.x; v.y = v.y * co.y + other.y * si.y; v.z = v.z * co.z + other.z * si.z; v.w = v.w * co.w + other.w * si.w; }
        }
        if (valid) {
            const uint2 packed = make_uint2(pack2(v.x, v.y), pack2(v.z, v.w));
            if (is_q) *reinterpret_cast<uint2*>(p.q_out + ((size_t)m * p.nq + head) * d + c) = packed;
            else if (p.write_kv) *reinterpret_cast<uint2*>((is_k ? p.k_cache : p.v_cache) + ops.cache_at) = packed;
        }
    }
}

// Host-side checks of one product's epilogue arguments; returns 0 or fails with a message (QT_FAIL).
inline int check_epilogue(const char* who, int epilogue, const EpilogueParams& p, int out_dtype) {
    switch (epilogue) {
        case EPI_STORE:
            QT_REQUIRE(p.out != nullptr && (out_dtype == QT_F32 || out_dtype == QT_BF16), "%s: the store epilogue needs a float or bfloat16 output", who);
            QT_REQUIRE((uintptr_t)p.out % 16 == 0, "%s: the output must be 16-byte aligned", who);
            break;
        case EPI_RESIDUAL:
            QT_REQUIRE(p.residual != nullptr && p.N % 4 == 0 && (uintptr_t)p.residual % 16 == 0, "%s: the residual epilogue needs an aligned stream whose width is a multiple of 4 (N=%d)", who, p.N);
            QT_REQUIRE(p.norm_w == nullptr || (p.xw != nullptr && p.sq_out != nullptr && (uintptr_t)p.norm_w % 16 == 0 && (uintptr_t)p.xw % 8 == 0),
                       "%s: preparing the next norm needs its weight, an output for the weighted stream and one for the sums of squares", who);
            break;
        case EPI_SWIGLU:
            QT_REQUIRE(p.out != nullptr && out_dtype == QT_BF16 && p.N % 32 == 0 && (uintptr_t)p.out % 4 == 0, "%s: the gated epilogue writes bfloat16 and needs gate and up rows in groups of 16 (N=%d)", who, p.N);
            QT_REQUIRE(p.act >= 0 && p.act < QT_ACT_COUNT, "%s: unknown activation code %d", who, p.act);
            break;
        case EPI_QKV:
            QT_REQUIRE(p.d >= 16 && TILE % p.d == 0 && p.d % 4 == 0 && p.N % p.d == 0, "%s: head_dim=%d must divide %d for the fused rotation (N=%d)", who, p.d, TILE, p.N);
            QT_REQUIRE(p.nq > 0 && p.nkv > 0 && (p.N == p.nq * p.d || p.N == (p.nq + 2 * p.nkv) * p.d), "%s: N=%d is neither nq*d nor (nq+2nkv)*d", who, p.N);
            QT_REQUIRE(p.rotary_dim >= 0 && p.rotary_dim <= p.d && p.rotary_dim % 8 == 0, "%s: rotary_dim=%d must be a multiple of 8 within head_dim=%d", who, p.rotary_dim, p.d);
            QT_REQUIRE(p.rotary_dim == 0 || (p.cos_sin && p.max_pos > 0 && (uintptr_t)p.cos_sin % 16 == 0), "%s: rotation needs an aligned cos/sin table", who);
            QT_REQUIRE(p.q_out && p.token_pos && (uintptr_t)p.q_out % 8 == 0, "%s: q output or positions missing", who);
            QT_REQUIRE((!p.q_w || (uintptr_t)p.q_w % 16 == 0) && (!p.k_w || (uintptr_t)p.k_w % 16 == 0), "%s: norm weights must be 16-byte aligned", who);
            QT_REQUIRE(!p.write_kv || (p.N == (p.nq + 2 * p.nkv) * p.d && p.k_cache && p.v_cache && p.block_table && p.token_seq && p.page_tokens > 0 && p.ring_tokens >= 0 &&
                                       (uintptr_t)p.k_cache % 8 == 0 && (uintptr_t)p.v_cache % 8 == 0),
                       "%s: writing keys and values needs them in the projection, the caches and the page table", who);
            break;
        default:
            QT_FAIL(QT_ERR_ARG, "%s: unknown epilogue %d", who, epilogue);
    }
    QT_REQUIRE(p.sq_in == nullptr || (p.sq_tiles > 0 && p.inv_hidden > 0.f && p.eps > 0.f), "%s: the deferred norm needs its tile count, width and eps", who);
    return QT_OK;
}

}  // namespace qt_epi
