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
#pragma once

#include "common.cuh"

#include <math.h>

namespace qt_mma {

using namespace qt;

constexpr int PAGE = 64;
constexpr int PAD = 8;              // elements of padding per shared-memory row: rows start 16 bytes apart modulo 128
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct MmaParams {
    const __nv_bfloat16* q;        // [T, nq, d]
    const __nv_bfloat16* k_cache;  // [pages, nkv, 64, d]
    const __nv_bfloat16* v_cache;
    __nv_bfloat16* out;            // [T, nq, d]
    const int* block_table; int max_blocks;
    const int* seq_start; const int* seq_past; const int* seq_len;
    int n_seqs, nq, nkv, d, ring_tokens, window;
    float scale;
    int n_splits; float* part_acc; float* part_ml;
    int stages;                    // decode: tiles in the shared-memory ring
    int cluster_merge;             // decode, one range per warp: the blocks of a (sequence, kv head) are a cluster and merge in shared memory
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// d[16x8] += a[16x16] * b[16x8]
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// The page of the cache that holds positions [64 * position_page, 64 * position_page + 64).
__device__ __forceinline__ int cache_page(const int* table, int position_page, int ring_tokens) {
    const int index = ring_tokens > 0 ? position_page % (ring_tokens / PAGE) : position_page;
    return table[index];
}

// Copy of a [64, d] tile (a page of one kv head) into padded shared-memory rows by a 128-thread block, 16 bytes
// per cp.async.  Where the chunks of a row divide the block size (head sizes 16, 32, 64, 128) a thread's chunks
// lie a fixed stride apart, so the loop is one add per chunk; other head sizes work the row and chunk out per
// piece (integer divisions by the runtime head size, which cost more than the copy itself).
struct TileCopy {
    int d, lds, chunks, pieces;          // pieces: 16-byte chunks of the tile
    bool linear;
    uint32_t dst0, dst_step;             // bytes
    int src0, src_step;                  // elements
    int tid;

    __device__ __forceinline__ TileCopy(int d_, int lds_, int tid_) : d(d_), lds(lds_), tid(tid_) {
        chunks = d >> 3;
        pieces = PAGE * chunks;
        linear = (128 % chunks) == 0;
        const int r = tid / chunks, c8 = (tid % chunks) * 8, rows_per_round = 128 / chunks;
        dst0 = (uint32_t)(r * lds + c8) * 2u;
        dst_step = (uint32_t)(rows_per_round * lds) * 2u;
        src0 = r * d + c8;
        src_step = rows_per_round * d;
    }
    __device__ __forceinline__ void start(uint32_t tile_smem, const __nv_bfloat16* tile_global) const {
        if (linear) {
            uint32_t dst = tile_smem + dst0;
            const __nv_bfloat16* src = tile_global + src0;
            for (int i = tid; i < pieces; i += 128, dst += dst_step, src += src_step) cp_async16(dst, src);
        } else {
            for (int i = tid; i < pieces; i += 128) {
                const int r = i / chunks, c8 = (i % chunks) * 8;
                cp_async16(tile_smem + (uint32_t)(r * lds + c8) * 2u, tile_global + r * d + c8);
            }
        }
    }
};

// Query fragments of a 16-row tile held in shared memory (row stride lds): qf[ks] covers dims 16 ks .. 16 ks + 15.
template <int DMAX>
__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[DMAX / 16][4], uint32_t q_smem, int lds, int dsteps, int lane) {
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8, col = (lane >> 4) * 8;
#pragma unroll
    for (int ks = 0; ks < DMAX / 16; ++ks)
        if (ks < dsteps) ldmatrix_x4(qf[ks], q_smem + (uint32_t)(row * lds + ks * 16 + col) * 2u);
}

// ----------------------------------------------------------------------------- decode
constexpr int DEC_MAX_STAGES = 3;     // depth of the key/value tile ring (2 or 3; fewer stages, more blocks per SM)

template <int DMAX>
__global__ void __launch_bounds__(128, 3) attention_decode_mma_kernel(const MmaParams p) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int d = p.d, lds = d + PAD, dsteps = d >> 4;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int group = p.nq / p.nkv;
    const int chunks_per_kv = (group + 15) / 16;
    const int kvh = blockIdx.y / chunks_per_kv;
    const int h0 = (blockIdx.y % chunks_per_kv) * 16;
    const int rows = min(16, group - h0);
    const int head_base = kvh * group + h0;
    const int seq = blockIdx.z, split = blockIdx.x;
    const int stages = p.stages;

    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [16][lds]
    const uint32_t tile_bytes = (uint32_t)PAGE * lds * 2u;
    const uint32_t q_bytes = 16u * lds * 2u;
    const uint32_t kv0 = smem_u32(smem_raw) + q_bytes;                               // stages of (K tile, V tile)

    const int len = p.seq_len[seq];
    const int lo = p.window > 0 ? max(0, len - p.window) : 0;
    const int first_page = lo / PAGE, last_page = (len - 1) / PAGE;
    const int n_pages = last_page - first_page + 1;
    const int per_split = (n_pages + p.n_splits - 1) / p.n_splits;
    const int page_begin = first_page + split * per_split;
    const int page_end = min(last_page + 1, page_begin + per_split);
    const int n_tiles = max(0, page_end - page_begin);
    const int* table = p.block_table + (size_t)seq * p.max_blocks;

    const TileCopy copy(d, lds, tid);
    auto issue = [&](int tile) {
        if (tile < n_tiles) {
            const int page = cache_page(table, page_begin + tile, p.ring_tokens);
            const size_t off = ((size_t)page * p.nkv + kvh) * PAGE * d;
            const uint32_t dst = kv0 + (uint32_t)(tile % stages) * 2u * tile_bytes;
            copy.start(dst, p.k_cache + off);
            copy.start(dst + tile_bytes, p.v_cache + off);
        }
        cp_async_commit();
    };
    // Keys and values of earlier positions do not depend on the kernel before this one (it writes only the new
    // token's row, which lies in the last page): their first tile is requested before waiting for that kernel.
    const bool early = n_tiles > 0 && page_begin < last_page;
    if (early) issue(0);
    pdl_wait();
    for (int i = tid; i < 16 * (d >> 3); i += 128) {                                 // query rows, zero beyond the group
        const int r = i / (d >> 3), c = i % (d >> 3);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)seq * p.nq + head_base + r) * d + c * 8);
        *reinterpret_cast<uint4*>(q_s + r * lds + c * 8) = v;
    }
    if (!early) issue(0);
    if (stages > 2) issue(1);
    __syncthreads();
    uint32_t qf[DMAX / 16][4];
    load_q_frags<DMAX>(qf, smem_u32(q_s), lds, dsteps, lane);

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    const float scale2 = p.scale * LOG2E;

    for (int tile = 0; tile < n_tiles; ++tile) {
        issue(tile + stages - 1);                                    // keeps stages - 1 tiles in flight behind this one
        if (stages > 2) cp_async_wait<2>(); else cp_async_wait<1>();
        __syncthreads();
        const uint32_t k_s = kv0 + (uint32_t)(tile % stages) * 2u * tile_bytes, v_s = k_s + tile_bytes;
        const int key0 = warp * 16;                                  // this warp's keys within the tile
        const int pos0 = (page_begin + tile) * PAGE + key0;
        if (pos0 < len && pos0 + 16 > lo) {                          // some key of this warp is visible
            float s[2][4] = {};
            {
                const int mi = lane >> 3;
                const int krow = key0 + (mi >> 1) * 8 + (lane & 7), kcol = (mi & 1) * 8;
#pragma unroll
                for (int ks = 0; ks < DMAX / 16; ++ks) {
                    if (ks < dsteps) {
                        uint32_t b[4];
                        ldmatrix_x4(b, k_s + (uint32_t)(krow * lds + ks * 16 + kcol) * 2u);
                        mma_bf16(s[0], qf[ks], b[0], b[1]);
                        mma_bf16(s[1], qf[ks], b[2], b[3]);
                    }
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int pos = pos0 + nt * 8 + 2 * t + (e & 1);
                    const bool visible = pos >= lo && pos < len;
                    s[nt][e] = visible ? s[nt][e] * scale2 : -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
                }
            float alpha[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m[r], mx[r]);
                const float m_use = m_new == -INFINITY ? 0.f : m_new;
                alpha[r] = fast_exp2(m[r] - m_use);
                m[r] = m_new;
                float sum = 0.f;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    s[nt][2 * r] = fast_exp2(s[nt][2 * r] - m_use);
                    s[nt][2 * r + 1] = fast_exp2(s[nt][2 * r + 1] - m_use);
                    sum += s[nt][2 * r] + s[nt][2 * r + 1];
                }
                l[r] = l[r] * alpha[r] + sum;                        // this thread's share of the row sum
            }
            uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                              pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
            const int mi = lane >> 3;
            const int vrow = key0 + (mi & 1) * 8 + (lane & 7), vcol = (mi >> 1) * 8;
#pragma unroll
            for (int nt2 = 0; nt2 < DMAX / 16; ++nt2) {
                if (nt2 < dsteps) {
                    o[2 * nt2][0] *= alpha[0]; o[2 * nt2][1] *= alpha[0]; o[2 * nt2][2] *= alpha[1]; o[2 * nt2][3] *= alpha[1];
                    o[2 * nt2 + 1][0] *= alpha[0]; o[2 * nt2 + 1][1] *= alpha[0]; o[2 * nt2 + 1][2] *= alpha[1]; o[2 * nt2 + 1][3] *= alpha[1];
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, v_s + (uint32_t)(vrow * lds + nt2 * 16 + vcol) * 2u);
                    mma_bf16(o[2 * nt2], pa, b[0], b[1]);
                    mma_bf16(o[2 * nt2 + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                             // the stage may be overwritten by the next issue
    }
    cp_async_wait<0>();
    __syncthreads();

    // merge the four warps through shared memory (the tile stages are free now)
    float* red_o = reinterpret_cast<float*>(smem_raw + q_bytes);     // [4][16][d]
    float* red_ml = red_o + 4 * 16 * d;                              // [4][16][2]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        if (t == 0) { red_ml[(warp * 16 + g + 8 * r) * 2] = m[r]; red_ml[(warp * 16 + g + 8 * r) * 2 + 1] = l[r]; }
    }
#pragma unroll
    for (int nt = 0; nt < DMAX / 8; ++nt) {
        if (nt < 2 * dsteps) {
            const int c = nt * 8 + 2 * t;
            red_o[(warp * 16 + g) * d + c] = o[nt][0]; red_o[(warp * 16 + g) * d + c + 1] = o[nt][1];
            red_o[(warp * 16 + g + 8) * d + c] = o[nt][2]; red_o[(warp * 16 + g + 8) * d + c + 1] = o[nt][3];
        }
    }
    __syncthreads();
    for (int i = tid; i < rows * d; i += 128) {
        const int r = i / d, c = i % d;
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m_all = fmaxf(m_all, red_ml[(w * 16 + r) * 2]);
        float l_all = 0.f, a_all = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = red_ml[(w * 16 + r) * 2];
            const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - m_all);
            l_all += red_ml[(w * 16 + r) * 2 + 1] * f;
            a_all += red_o[(w * 16 + r) * d + c] * f;
        }
        const int head = head_base + r;
        if (p.n_splits == 1) {
            p.out[((size_t)seq * p.nq + head) * d + c] = __float2bfloat16_rn(a_all / l_all);
        } else {
            const size_t slot = ((size_t)seq * p.nq + head) * p.n_splits + split;
            p.part_acc[slot * d + c] = a_all;
            if (c == 0) { p.part_ml[slot * 2] = m_all * LN2; p.part_ml[slot * 2 + 1] = l_all; }   // natural-log domain for the combine kernel
        }
    }
}

// ----------------------------------------------------------------------------- decode, one key range per warp
// The same work cut differently: every warp of a block walks a key range of its own, 32 keys (half a page) at a
// time, through a two-stage cp.async ring of its own, so that nothing in the loop waits for another warp.  A warp
// owns whole tiles: one online softmax and one accumulator rescale per 32 keys (the kernel above spends them per
// 16 keys in each of four warps), four independent QK^T accumulator chains, and no block barrier until the warps
// of a block merge their results at the end.  gridDim.x * warps ranges per (sequence, kv head); the block writes
// one partial result per gridDim.x.
constexpr int WS_TILE = 32;
constexpr int WS_MAX_WARPS = 6;

// Copy of a [32, d] tile by one warp, 16 bytes per cp.async (see TileCopy).
struct WarpTileCopy {
    int d, lds, chunks, pieces;
    bool linear;
    uint32_t dst0, dst_step;
    int src0, src_step;
    int lane;

    __device__ __forceinline__ WarpTileCopy(int d_, int lds_, int lane_) : d(d_), lds(lds_), lane(lane_) {
        chunks = d >> 3;
        pieces = WS_TILE * chunks;
        linear = (32 % chunks) == 0;
        const int r = lane / chunks, c8 = (lane % chunks) * 8, rows_per_round = 32 / chunks;
        dst0 = (uint32_t)(r * lds + c8) * 2u;
        dst_step = (uint32_t)(rows_per_round * lds) * 2u;
        src0 = r * d + c8;
        src_step = rows_per_round * d;
    }
    template <int DMAX, bool EXACT>
    __device__ __forceinline__ void start(uint32_t tile_smem, const __nv_bfloat16* tile_global) const {
        if (EXACT) {                                     // d == DMAX (64 or 128): a fixed number of pieces per lane
            uint32_t dst = tile_smem + dst0;
            const __nv_bfloat16* src = tile_global + src0;
#pragma unroll
            for (int i = 0; i < DMAX / 8; ++i, dst += dst_step, src += src_step) cp_async16(dst, src);
        } else if (linear) {
            uint32_t dst = tile_smem + dst0;
            const __nv_bfloat16* src = tile_global + src0;
            for (int i = lane; i < pieces; i += 32, dst += dst_step, src += src_step) cp_async16(dst, src);
        } else {
            for (int i = lane; i < pieces; i += 32) {
                const int r = i / chunks, c8 = (i % chunks) * 8;
                cp_async16(tile_smem + (uint32_t)(r * lds + c8) * 2u, tile_global + r * d + c8);
            }
        }
    }
};

template <int DMAX, bool EXACT>
__global__ void __launch_bounds__(32 * WS_MAX_WARPS) attention_decode_ws_kernel(const MmaParams p) {
    pdl_launch_dependents();
    const bool merges_in_cluster = p.cluster_merge && gridDim.x > 1;
    if (merges_in_cluster) cluster_arrive_started();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int d = EXACT ? DMAX : p.d, lds = d + PAD, dsteps = d >> 4;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int warps = blockDim.x >> 5;
    const int group = p.nq / p.nkv;
    const int chunks_per_kv = (group + 15) / 16;
    const int kvh = blockIdx.y / chunks_per_kv;
    const int h0 = (blockIdx.y % chunks_per_kv) * 16;
    const int rows = min(16, group - h0);
    const int head_base = kvh * group + h0;
    const int seq = blockIdx.z, split = blockIdx.x;
    const int stream = split * warps + warp, n_streams = gridDim.x * warps;

    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [16][lds]
    const uint32_t tile_bytes = (uint32_t)WS_TILE * lds * 2u;
    const uint32_t q_bytes = 16u * lds * 2u;
    const uint32_t ring0 = smem_u32(smem_raw) + q_bytes + (uint32_t)warp * 4u * tile_bytes;   // [stage][K tile, V tile]

    const int len = p.seq_len[seq];
    const int lo = p.window > 0 ? max(0, len - p.window) : 0;
    const int first_tile = lo / WS_TILE, last_tile = (len - 1) / WS_TILE;
    const int per_stream = (last_tile - first_tile + n_streams) / n_streams;
    const int tile_begin = first_tile + stream * per_stream;
    const int n_tiles = max(0, min(last_tile + 1, tile_begin + per_stream) - tile_begin);
    const int* table = p.block_table + (size_t)seq * p.max_blocks;

    const WarpTileCopy copy(d, lds, lane);
    // Page numbers of 32 tiles at a time, one per lane: a table lookup in front of every tile's copy would put an L2
    // round trip on each tile's path.
    int pages_from = -1, lane_page = 0;
    auto issue = [&](int tile) {
        if (tile < n_tiles) {
            if ((tile >> 5) != pages_from) {
                pages_from = tile >> 5;
                const int mine = min((pages_from << 5) + lane, n_tiles - 1);
                lane_page = cache_page(table, (tile_begin + mine) >> 1, p.ring_tokens);
            }
            const int t32 = tile_begin + tile;
            const int page = __shfl_sync(0xffffffffu, lane_page, tile & 31);
            const size_t off = (((size_t)page * p.nkv + kvh) * PAGE + (t32 & 1) * WS_TILE) * d;
            const uint32_t dst = ring0 + (uint32_t)(tile & 1) * 2u * tile_bytes;
            copy.template start<DMAX, EXACT>(dst, p.k_cache + off);
            copy.template start<DMAX, EXACT>(dst + tile_bytes, p.v_cache + off);
        }
        cp_async_commit();
    };
    // Keys and values of earlier positions do not depend on the kernel before this one (it writes only the new
    // token's row, which lies in the last tile): a first tile that is not the last is requested before the wait.
    const bool early = n_tiles > 0 && tile_begin < last_tile;
    if (early) issue(0);
    pdl_wait();
    for (int i = tid; i < 16 * (d >> 3); i += blockDim.x) {                          // query rows, zero beyond the group
        const int r = i / (d >> 3), c = i % (d >> 3);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)seq * p.nq + head_base + r) * d + c * 8);
        *reinterpret_cast<uint4*>(q_s + r * lds + c * 8) = v;
    }
    if (!early) issue(0);
    __syncthreads();
    uint32_t qf[DMAX / 16][4];
    load_q_frags<DMAX>(qf, smem_u32(q_s), lds, dsteps, lane);

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};          // m in the scaled base-2 domain
    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    const float scale2 = p.scale * LOG2E;                            // positive (checked by the host)
    const int mi = lane >> 3;
    const uint32_t k_lane = (uint32_t)(((mi >> 1) * 8 + (lane & 7)) * lds + (mi & 1) * 8) * 2u;
    const uint32_t v_lane = (uint32_t)(((mi & 1) * 8 + (lane & 7)) * lds + (mi >> 1) * 8) * 2u;
    const uint32_t half_tile = (uint32_t)(16 * lds) * 2u;            // 16 keys further down

    for (int tile = 0; tile < n_tiles; ++tile) {
        issue(tile + 1);                                             // into the stage that the tile before this one used
        cp_async_wait<1>();
        __syncwarp();
        const uint32_t k_s = ring0 + (uint32_t)(tile & 1) * 2u * tile_bytes, v_s = k_s + tile_bytes;
        const int pos0 = (tile_begin + tile) * WS_TILE;
        float s[4][4] = {};
#pragma unroll
        for (int ks = 0; ks < DMAX / 16; ++ks) {
            if (EXACT || ks < dsteps) {
                uint32_t b0[4], b1[4];
                ldmatrix_x4(b0, k_s + k_lane + (uint32_t)(ks * 32));
                ldmatrix_x4(b1, k_s + k_lane + half_tile + (uint32_t)(ks * 32));
                mma_bf16(s[0], qf[ks], b0[0], b0[1]);
                mma_bf16(s[1], qf[ks], b0[2], b0[3]);
                mma_bf16(s[2], qf[ks], b1[0], b1[1]);
                mma_bf16(s[3], qf[ks], b1[2], b1[3]);
            }
        }
        if (pos0 < lo || pos0 + WS_TILE > len) {                     // a tile at an edge of what the query sees
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int pos = pos0 + nt * 8 + 2 * t + (e & 1);
                    if (pos < lo || pos >= len) s[nt][e] = -INFINITY;
                }
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = fmaxf(fmaxf(s[0][2 * r], s[0][2 * r + 1]), fmaxf(s[1][2 * r], s[1][2 * r + 1]));
            mx = fmaxf(mx, fmaxf(fmaxf(s[2][2 * r], s[2][2 * r + 1]), fmaxf(s[3][2 * r], s[3][2 * r + 1])));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[r], mx * scale2);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            alpha[r] = fast_exp2(m[r] - m_use);
            m[r] = m_new;
            float sum = 0.f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                s[nt][2 * r] = fast_exp2(fmaf(s[nt][2 * r], scale2, -m_use));
                s[nt][2 * r + 1] = fast_exp2(fmaf(s[nt][2 * r + 1], scale2, -m_use));
                sum += s[nt][2 * r] + s[nt][2 * r + 1];
            }
            l[r] = l[r] * alpha[r] + sum;                            // this thread's share of the row sum
        }
        const uint32_t pa0[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                                 pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
        const uint32_t pa1[4] = {pack_bf16(s[2][0], s[2][1]), pack_bf16(s[2][2], s[2][3]),
                                 pack_bf16(s[3][0], s[3][1]), pack_bf16(s[3][2], s[3][3])};
#pragma unroll
        for (int nt2 = 0; nt2 < DMAX / 16; ++nt2) {
            if (EXACT || nt2 < dsteps) {
                o[2 * nt2][0] *= alpha[0]; o[2 * nt2][1] *= alpha[0]; o[2 * nt2][2] *= alpha[1]; o[2 * nt2][3] *= alpha[1];
                o[2 * nt2 + 1][0] *= alpha[0]; o[2 * nt2 + 1][1] *= alpha[0]; o[2 * nt2 + 1][2] *= alpha[1]; o[2 * nt2 + 1][3] *= alpha[1];
                uint32_t b0[4], b1[4];
                ldmatrix_x4_trans(b0, v_s + v_lane + (uint32_t)(nt2 * 32));
                ldmatrix_x4_trans(b1, v_s + v_lane + half_tile + (uint32_t)(nt2 * 32));
                mma_bf16(o[2 * nt2], pa0, b0[0], b0[1]);
                mma_bf16(o[2 * nt2 + 1], pa0, b0[2], b0[3]);
                mma_bf16(o[2 * nt2], pa1, b1[0], b1[1]);
                mma_bf16(o[2 * nt2 + 1], pa1, b1[2], b1[3]);
            }
        }
        __syncwarp();                                                // the stage may be overwritten by the next issue
    }
    cp_async_wait<0>();
    __syncthreads();

    // merge the warps through shared memory (the rings are free now)
    float* red_o = reinterpret_cast<float*>(smem_raw + q_bytes);     // [warps][16][d]
    float* red_ml = red_o + warps * 16 * d;                          // [warps][16][2]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        if (t == 0) { red_ml[(warp * 16 + g + 8 * r) * 2] = m[r]; red_ml[(warp * 16 + g + 8 * r) * 2 + 1] = l[r]; }
    }
#pragma unroll
    for (int nt = 0; nt < DMAX / 8; ++nt) {
        if (EXACT || nt < 2 * dsteps) {
            const int c = nt * 8 + 2 * t;
            *reinterpret_cast<float2*>(red_o + (warp * 16 + g) * d + c) = make_float2(o[nt][0], o[nt][1]);
            *reinterpret_cast<float2*>(red_o + (warp * 16 + g + 8) * d + c) = make_float2(o[nt][2], o[nt][3]);
        }
    }
    __syncthreads();
    // With cluster_merge the blocks of this (sequence, kv head) form a cluster: every block writes its merged rows
    // into the inbox of the first one (distributed shared memory, beyond that block's rings, which may still be in
    // use), and after the cluster barrier the first block merges the inboxes and stores the result.
    float* inbox = reinterpret_cast<float*>(smem_raw + q_bytes + (size_t)warps * 4 * tile_bytes);   // [blocks][rows * d + 2 * rows] in block 0
    const int inbox_stride = rows * d + 2 * rows;
    if (merges_in_cluster) cluster_wait_started();                   // the first block runs (a block with no keys gets here early)
    for (int i = tid; i < rows * d; i += blockDim.x) {
        const int r = i / d, c = i % d;
        float m_all = -INFINITY;
        for (int w = 0; w < warps; ++w) m_all = fmaxf(m_all, red_ml[(w * 16 + r) * 2]);
        float l_all = 0.f, a_all = 0.f;
        for (int w = 0; w < warps; ++w) {
            const float mw = red_ml[(w * 16 + r) * 2];
            const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - m_all);
            l_all += red_ml[(w * 16 + r) * 2 + 1] * f;
            a_all += red_o[(w * 16 + r) * d + c] * f;
        }
        const int head = head_base + r;
        if (gridDim.x == 1) {
            p.out[((size_t)seq * p.nq + head) * d + c] = __float2bfloat16_rn(a_all / l_all);
        } else if (p.cluster_merge) {
            float* slot = inbox + (size_t)split * inbox_stride;
            cluster_store_float(slot + i, 0, a_all);
            if (c == 0) { cluster_store_float(slot + rows * d + 2 * r, 0, m_all); cluster_store_float(slot + rows * d + 2 * r + 1, 0, l_all); }
        } else {
            const size_t slot = ((size_t)seq * p.nq + head) * gridDim.x + split;
            p.part_acc[slot * d + c] = a_all;
            if (c == 0) { p.part_ml[slot * 2] = m_all * LN2; p.part_ml[slot * 2 + 1] = l_all; }   // natural-log domain for the combine kernel
        }
    }
    if (merges_in_cluster) {
        cluster_barrier();
        if (split == 0) {
            const int blocks = gridDim.x;
            for (int i = tid; i < rows * d; i += blockDim.x) {
                const int r = i / d;
                float m_all = -INFINITY;
                for (int b = 0; b < blocks; ++b) m_all = fmaxf(m_all, inbox[(size_t)b * inbox_stride + rows * d + 2 * r]);
                float l_all = 0.f, a_all = 0.f;
                for (int b = 0; b < blocks; ++b) {
                    const float* slot = inbox + (size_t)b * inbox_stride;
                    const float mb = slot[rows * d + 2 * r];
                    const float f = mb == -INFINITY ? 0.f : fast_exp2(mb - m_all);
                    l_all += slot[rows * d + 2 * r + 1] * f;
                    a_all += slot[i] * f;
                }
                p.out[((size_t)seq * p.nq + head_base + r) * d + (i % d)] = __float2bfloat16_rn(a_all / l_all);
            }
        }
    }
}

// One block per (sequence, head): out = sum_s acc_s e^{m_s - m} / sum_s l_s e^{m_s - m}; empty splits have m = -inf.
__global__ void attention_combine_mma_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                             __nv_bfloat16* __restrict__ out, int n_splits, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t item = blockIdx.x;
    float m_all = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m_all = fmaxf(m_all, part_ml[(item * n_splits + s) * 2]);
    float l_all = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part_ml[(item * n_splits + s) * 2];
        l_all += ms == -INFINITY ? 0.f : part_ml[(item * n_splits + s) * 2 + 1] * __expf(ms - m_all);
    }
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part_ml[(item * n_splits + s) * 2];
            if (ms != -INFINITY) a += part_acc[(item * n_splits + s) * d + c] * __expf(ms - m_all);
        }
        out[item * d + c] = __float2bfloat16_rn(a / l_all);
    }
}

// ----------------------------------------------------------------------------- prefill
constexpr int PF_BQ = 64;

template <int DMAX>
__global__ void __launch_bounds__(128, 3) attention_prefill_mma_kernel(const MmaParams p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int d = p.d, lds = d + PAD, dsteps = d >> 4;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int q_begin = p.seq_start[seq], q_len = p.seq_start[seq + 1] - q_begin;
    const int q0 = blockIdx.x * PF_BQ;
    if (q0 >= q_len) return;
    const int rows = min(PF_BQ, q_len - q0);
    const int past = p.seq_past[seq];
    const int kvh = head / (p.nq / p.nkv);
    const int* table = p.block_table + (size_t)seq * p.max_blocks;

    const uint32_t tile_bytes = (uint32_t)PAGE * lds * 2u;
    const uint32_t kv0 = smem_u32(smem_raw);                                         // two stages of (K tile, V tile)
    // the query tile borrows the second stage's key tile until its fragments sit in registers
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw + 2 * tile_bytes);   // [64][lds]

    const int p_first = past + q0, p_last = past + q0 + rows - 1;
    const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;
    const int page_begin = lo / PAGE, n_tiles = p_last / PAGE - page_begin + 1;

    for (int i = tid; i < PF_BQ * (d >> 3); i += 128) {                              // query tile, rows beyond the sequence zero
        const int r = i / (d >> 3), c = i % (d >> 3);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)(q_begin + q0 + r) * p.nq + head) * d + c * 8);
        *reinterpret_cast<uint4*>(q_s + r * lds + c * 8) = v;
    }
    const TileCopy copy(d, lds, tid);
    auto issue = [&](int tile) {
        if (tile < n_tiles) {
            const int page = cache_page(table, page_begin + tile, p.ring_tokens);
            const size_t off = ((size_t)page * p.nkv + kvh) * PAGE * d;
            const uint32_t dst = kv0 + (uint32_t)(tile & 1) * 2u * tile_bytes;
            copy.start(dst, p.k_cache + off);
            copy.start(dst + tile_bytes, p.v_cache + off);
        }
        cp_async_commit();
    };
    issue(0);
    __syncthreads();
    uint32_t qf[DMAX / 16][4];
    load_q_frags<DMAX>(qf, smem_u32(q_s) + (uint32_t)(warp * 16 * lds) * 2u, lds, dsteps, lane);
    __syncthreads();                                                                 // before the second stage is filled

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    const float scale2 = p.scale * LOG2E;
    // absolute positions of this thread's two query rows; rows beyond the sequence act as its last row
    const int qpos[2] = {min(past + q0 + warp * 16 + g, p_last), min(past + q0 + warp * 16 + g + 8, p_last)};
    const int warp_pos_min = min(past + q0 + warp * 16, p_last), warp_pos_max = min(past + q0 + warp * 16 + 15, p_last);

    for (int tile = 0; tile < n_tiles; ++tile) {
        issue(tile + 1);
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t k_s = kv0 + (uint32_t)(tile & 1) * 2u * tile_bytes, v_s = k_s + tile_bytes;
        const int pos0 = (page_begin + tile) * PAGE;
        const bool any_visible = pos0 <= warp_pos_max && (p.window <= 0 || pos0 + PAGE - 1 > warp_pos_min - p.window);
        if (any_visible) {
            float s[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
            {
                const int mi = lane >> 3;
                const int krow = (mi >> 1) * 8 + (lane & 7), kcol = (mi & 1) * 8;
#pragma unroll
                for (int ks = 0; ks < DMAX / 16; ++ks) {
                    if (ks < dsteps) {
#pragma unroll
                        for (int np = 0; np < 4; ++np) {
                            uint32_t b[4];
                            ldmatrix_x4(b, k_s + (uint32_t)((np * 16 + krow) * lds + ks * 16 + kcol) * 2u);
                            mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
                            mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
                        }
                    }
                }
            }
            // Scores stay unscaled; the scale is folded into the exponent: p = 2^(s * scale2 - m * scale2), one FMA
            // and one ex2 per score.  Most tiles lie wholly below the diagonal (and inside the window) for every row
            // of the warp and need no mask.
            const bool all_visible = pos0 + PAGE - 1 <= warp_pos_min && (p.window <= 0 || pos0 > warp_pos_max - p.window);
            float mx[2] = {-INFINITY, -INFINITY};
            if (!all_visible) {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int pos = pos0 + nt * 8 + 2 * t + (e & 1);
                        const int qp = qpos[e >> 1];
                        const bool visible = pos <= qp && (p.window <= 0 || pos > qp - p.window);
                        if (!visible) s[nt][e] = -INFINITY;
                    }
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
            float alpha[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m[r], mx[r] * scale2);       // scale2 > 0: the max of the scaled scores
                const float m_use = m_new == -INFINITY ? 0.f : m_new;
                alpha[r] = fast_exp2(m[r] - m_use);
                m[r] = m_new;
                float sum = 0.f;
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    s[nt][2 * r] = fast_exp2(fmaf(s[nt][2 * r], scale2, -m_use));
                    s[nt][2 * r + 1] = fast_exp2(fmaf(s[nt][2 * r + 1], scale2, -m_use));
                    sum += s[nt][2 * r] + s[nt][2 * r + 1];
                }
                l[r] = l[r] * alpha[r] + sum;
            }
#pragma unroll
            for (int nt = 0; nt < DMAX / 8; ++nt) { o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0]; o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1]; }
            const int mi = lane >> 3;
            const int vrow = (mi & 1) * 8 + (lane & 7), vcol = (mi >> 1) * 8;
#pragma unroll
            for (int j = 0; j < 4; ++j) {                            // 16 keys at a time
                const uint32_t pa[4] = {pack_bf16(s[2 * j][0], s[2 * j][1]), pack_bf16(s[2 * j][2], s[2 * j][3]),
                                        pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]), pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3])};
#pragma unroll
                for (int nt2 = 0; nt2 < DMAX / 16; ++nt2) {
                    if (nt2 < dsteps) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, v_s + (uint32_t)((j * 16 + vrow) * lds + nt2 * 16 + vcol) * 2u);
                        mma_bf16(o[2 * nt2], pa, b[0], b[1]);
                        mma_bf16(o[2 * nt2 + 1], pa, b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        const int row = warp * 16 + g + 8 * r;
        if (row < rows) {
            const float inv = 1.f / l[r];
            __nv_bfloat16* dst = p.out + ((size_t)(q_begin + q0 + row) * p.nq + head) * d;
#pragma unroll
            for (int nt = 0; nt < DMAX / 8; ++nt)
                if (nt < 2 * dsteps)
                    *reinterpret_cast<uint32_t*>(dst + nt * 8 + 2 * t) = pack_bf16(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
        }
    }
}

}  // namespace qt_mma
