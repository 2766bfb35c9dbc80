// Causal attention for steps with many tokens per sequence on the fifth-generation tensor cores
// (bfloat16, head size 64 or 128, paged cache with 64-token pages).
//
// A block takes 128 query rows of one head and walks the keys in tiles of one page (64 keys; the kernel is written
// for tiles of one or two pages), two blocks per SM:
//
//   S = Q K^T        tcgen05.mma, Q and K tiles in shared memory (TMA, 128-byte swizzle), S in tensor memory
//   P = softmax(S)   four warps, one thread per query row: the row of S is read once with tcgen05.ld into
//                    registers, so the row maximum and sum need no shuffles and no exchange; P goes back into
//                    tensor memory as bfloat16 pairs (tcgen05.st) over the scores it came from
//   O += P V         tcgen05.mma with P as the A operand from tensor memory and V as an MN-major operand from
//                    shared memory (V is stored [key][dim]), accumulated in tensor memory over all tiles
//
// O stays in tensor memory, so the softmax threads touch it only when a row's maximum has to move: a row keeps
// the maximum it scaled by until the true one is more than 2^8 above it (P then holds values up to 2^8, which
// bfloat16 and the float accumulator carry; the row sum uses the same maximum, so the quotient is exact), and
// only then is that row of O read, scaled and written back (tcgen05.ld / tcgen05.st).  After the first tiles of
// a causal row this is rare.
//
// Warp roles (224 threads): warp 0 lane 0 = TMA producer of Q and of the K tiles, warp 6 lane 0 = TMA producer of
// the V tiles (two-stage rings each; separate producers so that a key tile is requested as soon as its stage is
// free, not behind a value tile), warp 1 = tensor-memory allocation and (lane 0) MMA issue, warps 2..5 = softmax
// and output.  S is double buffered: Q K^T of tile j+1 runs while the softmax of tile j is computed, and P V of
// tile j runs under the whole softmax of tile j+1 (P of tile j+1 goes to the other buffer; a softmax warp waits
// for P V only when it has to scale O, and at the end).  The buffer of tile j is overwritten by Q K^T of tile j+2,
// which the MMA thread issues after P V of tile j: the tensor pipe runs one thread's instructions in order.  Key j is visible to the query at
// absolute position p iff j <= p and, in a windowed group, j > p - window.  Every mbarrier wait is bounded and
// reports through a status word.
//
// Counterpart in luozoupi/Qwen-Triton: kernels/flash_attention.py:54-152 (32 x 32 tl.dot tiles) and the masked
// SDPA branch of modules/attention.py:110-123.
#include "tc_common.cuh"

#include <math.h>

using namespace qt;
using namespace qt_tc;

namespace {

constexpr int PAGE = 64;
constexpr int BQ = 128;            // query rows per block = MMA M
constexpr int THREADS = 224;        // warp 0: TMA of Q and K, warp 1: MMA + tensor-memory allocation, warps 2..5: softmax, warp 6: TMA of V
constexpr uint32_t ALIGN_SLACK = 1024;  // shared memory asked for beyond the tiles, to round their base up to 1,024 bytes (the
                                        // kernel refuses to run if the base ever needs more)
constexpr float RESCALE_STEP = 8.f; // a row's scaling maximum moves only when the true one is more than 2^8 above it
constexpr float LOG2E = 1.4426950408889634f;
constexpr uint32_t HALF_BYTES = 128 * 64 * 2;   // a [128 rows][64 columns] bfloat16 half tile: 16 KB

struct TcAttnParams {
    __nv_bfloat16* out;            // [T, nq, d]
    const int* block_table; int max_blocks;
    const int* seq_start; const int* seq_past;
    int nq, nkv, ring_tokens, window;
    float scale;
    int* status;
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// d[tmem] (+)= a[tmem] * b[smem]: the A operand comes from tensor memory, row i in lane i, K elements packed two to
// a 32-bit column (K-major), B from shared memory through its descriptor.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Three-input maximum and two-wide float arithmetic (sm_100): half the instructions of the softmax's maximum, scaling
// and row sum; every lane rounds as the one-wide form does.
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint64_t pair_f32(float lo, float hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ uint64_t pair_u32(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}
__device__ __forceinline__ void unpair_f32(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Operand descriptor of an MN-major tile stored as [64-element MN blocks][K rows][64 elements], 128-byte swizzle:
// groups of 8 K rows lie 1024 bytes apart (stride byte offset), MN blocks `mn_block_bytes` apart (leading byte offset).
__device__ __forceinline__ uint64_t operand_desc_mn(uint32_t saddr, uint32_t mn_block_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)((mn_block_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ int cache_page(const int* table, int max_blocks, int position_page, int ring_tokens) {
    int index = ring_tokens > 0 ? position_page % (ring_tokens / PAGE) : position_page;
    if (index >= max_blocks) index = max_blocks - 1;     // beyond the sequence: any valid page, its keys are masked
    return table[index];
}

// BKEY: keys per tile, one page or two.  One page: half the shared memory and tensor memory, so that two blocks share
// an SM and one's softmax runs under the other's MMAs.
template <int HD, int BKEY>
__global__ void __launch_bounds__(THREADS, BKEY == 64 ? 2 : 1) attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                       const __grid_constant__ CUtensorMap map_k,
                                                                       const __grid_constant__ CUtensorMap map_v,
                                                                       const TcAttnParams p) {
    constexpr int HALVES = HD / 64;                       // 64-column halves of a [*, HD] tile
    constexpr uint32_t Q_BYTES = HALVES * HALF_BYTES;     // [128 rows][HD]
    constexpr int PAGES = BKEY / PAGE;                    // pages per key tile
    constexpr uint32_t KEY_HALF_BYTES = BKEY * 64 * 2;    // a [BKEY keys][64 columns] half of a key or value tile
    constexpr uint32_t KV_BYTES = HALVES * KEY_HALF_BYTES;   // [BKEY keys][HD]
    constexpr uint32_t TMEM_COLS = BKEY == 64 ? 256 : 512;
    constexpr uint32_t S_COL0 = 0, S_COL1 = BKEY, O_COL = 2 * BKEY;
    // S = Q K^T: M 128, N 128 keys, both operands K-major.  O = P V: M 128, N HD, A K-major, B MN-major.
    constexpr uint32_t IDESC_QK = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BKEY >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);

    pdl_launch_dependents();
    const int seq = blockIdx.z, head = blockIdx.x;
    const int q_begin = p.seq_start[seq], q_len = p.seq_start[seq + 1] - q_begin;
    // Blocks are handed out in launch order, x fastest: every head's last query tile first (it walks the most keys),
    // every head's first tile last, so that the blocks still running at the end are the short ones; neighbours in x
    // are heads of one kv group and read the same keys.
    const int q0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * BQ;
    if (q0 >= q_len) return;                              // uniform for the block, before any barrier or allocation
    const int rows = min(BQ, q_len - q0);
    const int past = p.seq_past[seq];
    const int kvh = head / (p.nq / p.nkv);
    const int* table = p.block_table + (size_t)seq * p.max_blocks;
    const int p_first = past + q0, p_last = past + q0 + rows - 1;
    const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;
    const int tile_begin = lo / BKEY;
    const int n_tiles = p_last / BKEY - tile_begin + 1;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    if (base - raw > ALIGN_SLACK) {                       // the launch asked for less slack than this base needs: refuse, uniformly
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 5);
        return;
    }
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t q_s = base, k_s = q_s + Q_BYTES, v_s = k_s + 2 * KV_BYTES;
    const uint32_t bars = v_s + 2 * KV_BYTES;
    // barriers: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], pv_full[2]
    const uint32_t q_full = bars, k_full = bars + 8, k_empty = bars + 24, v_full = bars + 40, v_empty = bars + 56;
    const uint32_t s_full = bars + 72, p_full = bars + 88, pv_full = bars + 104;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + (bars - base) + 128);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int* status = p.status;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full + 8 * i, 1); mbar_init(k_empty + 8 * i, 1);
            mbar_init(v_full + 8 * i, 1); mbar_init(v_empty + 8 * i, 1);
            mbar_init(s_full + 8 * i, 1); mbar_init(p_full + 8 * i, 4);
            mbar_init(pv_full + 8 * i, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();                                   // queries and this step's keys come from the kernel before
            mbar_expect_tx(q_full, Q_BYTES);
            for (int h = 0; h < HALVES; ++h)
                tma_load_2d(q_s + h * HALF_BYTES, &map_q, q_full, head * HD + h * 64, q_begin + q0);
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j & 1;
                const uint32_t phase = (uint32_t)(j >> 1) & 1u;
                if (!mbar_wait(k_empty + 8 * s, phase ^ 1u, status, 1)) break;
                mbar_expect_tx(k_full + 8 * s, KV_BYTES);
                for (int pg = 0; pg < PAGES; ++pg) {
                    const int row0 = (cache_page(table, p.max_blocks, (tile_begin + j) * PAGES + pg, p.ring_tokens) * p.nkv + kvh) * PAGE;
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(k_s + s * KV_BYTES + h * KEY_HALF_BYTES + pg * (PAGE * 128), &map_k, k_full + 8 * s, h * 64, row0);
                }
            }
        }
    } else if (warp == 6) {
        if (lane == 0) {
            pdl_wait();
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j & 1;
                const uint32_t phase = (uint32_t)(j >> 1) & 1u;
                if (!mbar_wait(v_empty + 8 * s, phase ^ 1u, status, 1)) break;
                mbar_expect_tx(v_full + 8 * s, KV_BYTES);
                for (int pg = 0; pg < PAGES; ++pg) {
                    const int row0 = (cache_page(table, p.max_blocks, (tile_begin + j) * PAGES + pg, p.ring_tokens) * p.nkv + kvh) * PAGE;
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(v_s + s * KV_BYTES + h * KEY_HALF_BYTES + pg * (PAGE * 128), &map_v, v_full + 8 * s, h * 64, row0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // This thread's instructions are the tensor pipe's critical path: operand descriptors are formed once and
            // stepped by additions (their address field counts 16-byte units).
            const uint64_t q_desc0 = operand_desc(q_s), k_desc0 = operand_desc(k_s);
            const uint64_t v_desc0 = operand_desc_mn(v_s, KEY_HALF_BYTES);
            bool ok = mbar_wait(q_full, 0, status, 2);
            auto issue_qk = [&](int i) {
                const int s = i & 1;
                const uint32_t phase = (uint32_t)(i >> 1) & 1u;
                if (!mbar_wait(k_full + 8 * s, phase, status, 2)) return false;
                // this buffer held the scores and then P of tile i - 2: its P V was issued before this, and the tensor
                // pipe runs its instructions in order
                tc_fence_after();
                const uint32_t acc = tmem_base + (s ? S_COL1 : S_COL0);
                const uint64_t k_desc = k_desc0 + (uint64_t)(s * (KV_BYTES >> 4));
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {    // 16 dims per MMA; 4 MMAs per 64-column half
                    const uint32_t in_half = (uint32_t)(ks & 3) * 32u;
                    umma_bf16(acc, q_desc0 + (uint64_t)(((uint32_t)(ks >> 2) * HALF_BYTES + in_half) >> 4),
                              k_desc + (uint64_t)(((uint32_t)(ks >> 2) * KEY_HALF_BYTES + in_half) >> 4), IDESC_QK, ks > 0 ? 1u : 0u);
                }
                umma_commit(s_full + 8 * s);
                umma_commit(k_empty + 8 * s);
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) { ok = issue_qk(j + 1); if (!ok) break; }
                const int s = j & 1;
                if (!mbar_wait(p_full + 8 * s, (uint32_t)(j >> 1) & 1u, status, 2)) break;
                if (!mbar_wait(v_full + 8 * s, (uint32_t)(j >> 1) & 1u, status, 2)) break;
                tc_fence_after();
                const uint64_t v_desc = v_desc0 + (uint64_t)(s * (KV_BYTES >> 4));
                const uint32_t p_tmem = tmem_base + (s ? S_COL1 : S_COL0);     // P lies over the scores it came from
#pragma unroll
                for (int ks = 0; ks < BKEY / 16; ++ks) {  // 16 keys per MMA = 8 columns of packed pairs
                    const uint64_t b_desc = v_desc + (uint64_t)(((uint32_t)ks * (16 * 128)) >> 4);
                    umma_bf16_a_tmem(tmem_base + O_COL, p_tmem + (uint32_t)(ks * 8), b_desc, IDESC_PV, (j > 0 || ks > 0) ? 1u : 0u);    // O accumulates over the tiles
                }
                umma_commit(pv_full + 8 * s);
                umma_commit(v_empty + 8 * s);
            }
        }
    } else if (warp < 6) {
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                 // this thread's query row = its tensor-memory lane
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int qpos = min(past + q0 + r, p_last);       // rows beyond the sequence act as its last row
        const float scale2 = p.scale * LOG2E;
        float m_run = -INFINITY, l_run = 0.f;              // the maximum this row scales by (scaled base-2 domain) and its sum
        pdl_wait();                                        // the output may still be read by an earlier kernel
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int s = j & 1;
            if (!mbar_wait(s_full + 8 * s, (uint32_t)(j >> 1) & 1u, status, 3)) { ok = false; break; }
            tc_fence_after();
            const uint32_t s_addr = lane_addr + (s ? S_COL1 : S_COL0);
            const int pos0 = (tile_begin + j) * BKEY;
            // the whole row of scores, once
            constexpr int QUARTERS = BKEY / 32;            // 32-key pieces of the row
            uint32_t v[QUARTERS][32];
#pragma unroll
            for (int q = 0; q < QUARTERS; ++q) tmem_load32_start(s_addr + (uint32_t)(q * 32), v[q]);
            tmem_wait_ld();
            // mask only where some row of the block cannot see the whole tile
            const bool masked = pos0 + BKEY - 1 > p_first || (p.window > 0 && pos0 <= p_last - p.window);
            if (masked) {
#pragma unroll
                for (int q = 0; q < QUARTERS; ++q)
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int pos = pos0 + q * 32 + c;
                        if (!(pos <= qpos && (p.window <= 0 || pos > qpos - p.window))) v[q][c] = 0xff800000u;   // -inf
                    }
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int q = 0; q < QUARTERS; ++q)
#pragma unroll
                for (int c = 0; c < 32; c += 2) mx[(c >> 1) & 3] = max3(mx[(c >> 1) & 3], __uint_as_float(v[q][c]), __uint_as_float(v[q][c + 1]));
            const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale2;
            // the row's maximum moves only when the true one has run away from it
            const bool moves = m_tile > m_run + RESCALE_STEP;
            const float m_new = moves ? m_tile : m_run;
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = moves ? fast_exp2(m_run - m_use) : 1.f;
            if (j > 0 && __any_sync(0xffffffffu, moves)) {
                // O may be scaled once P V of the tile before is complete.  A softmax warp waits for P V only here and at
                // the end, so it can be behind: the barriers alternate by tile, and since the scores of tile j exist,
                // every P V up to tile j - 2 is complete, so the barrier of tile j - 1 is in that tile's phase or the next.
                if (!mbar_wait(pv_full + 8 * ((j - 1) & 1), (uint32_t)((j - 1) >> 1) & 1u, status, 3)) { ok = false; break; }
                tc_fence_after();
                {
#pragma unroll 1
                    for (int c0 = 0; c0 < HD; c0 += 32) {
                        uint32_t o[32];
                        tmem_load32(lane_addr + O_COL + (uint32_t)c0, o);
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                        tmem_store32(lane_addr + O_COL + (uint32_t)c0, o);
                    }
                    tmem_wait_st();
                }
            }
            // P = 2^(s * scale2 - m) as bfloat16, two keys to a 32-bit column, over this row's scores in tensor memory
            // (they are in registers); the row sum
            uint64_t sum2[2] = {0ull, 0ull};               // two pairs of partial sums
            const uint64_t scale22 = pair_f32(scale2, scale2), neg_m2 = pair_f32(-m_use, -m_use);
#pragma unroll
            for (int h = 0; h < QUARTERS / 2; ++h) {       // 64 keys = 32 columns per store
                uint32_t packed[32];
#pragma unroll
                for (int q = 0; q < 2; ++q)
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        float x0, x1;
                        unpair_f32(fma2(pair_u32(v[2 * h + q][c], v[2 * h + q][c + 1]), scale22, neg_m2), x0, x1);
                        const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
                        sum2[(c >> 1) & 1] = add2(sum2[(c >> 1) & 1], pair_f32(e0, e1));
                        packed[q * 16 + (c >> 1)] = pack_bf16(e0, e1);
                    }
                tmem_store32(s_addr + (uint32_t)(h * 32), packed);
            }
            tmem_wait_st();
            // P is written (and O scaled where it had to be): hand both to the MMA
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 8 * s);
            float sum[4];
            unpair_f32(sum2[0], sum[0], sum[2]);
            unpair_f32(sum2[1], sum[1], sum[3]);
            l_run = l_run * alpha + (sum[0] + sum[1]) + (sum[2] + sum[3]);
            m_run = m_new;
        }
        if (ok && mbar_wait(pv_full + 8 * ((n_tiles - 1) & 1), (uint32_t)((n_tiles - 1) >> 1) & 1u, status, 3)) {
            tc_fence_after();
            const float inv = 1.f / l_run;
            __nv_bfloat16* dst = p.out + ((size_t)(q_begin + q0 + r) * p.nq + head) * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t o[32];
                tmem_load32(lane_addr + O_COL + (uint32_t)c0, o);
                if (r < rows) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + c) = w;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*(volatile int*)status != 0) {                     // a wait gave up: let copies in flight land before the block leaves
        const unsigned long long t0 = global_timer();
        while (global_timer() - t0 < 2000000ull) __nanosleep(1000);
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <int HD, int BKEY>
int launch(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v, const TcAttnParams& p, int n_seqs,
           int max_q_len, cudaStream_t stream) {
    constexpr uint32_t HALVES = HD / 64;
    // Q, two key and two value tiles, alignment slack, barriers
    const size_t smem = (size_t)HALVES * HALF_BYTES + 4 * (size_t)HALVES * BKEY * 128 + ALIGN_SLACK + 128 + 64;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD, BKEY>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "attention_prefill_tc: cannot raise shared memory: %s", cudaGetErrorString(err));
        configured = true;
    }
    dim3 grid(p.nq, (max_q_len + BQ - 1) / BQ, n_seqs);
    launch_kernel(attention_prefill_tc_kernel<HD, BKEY>, grid, dim3(THREADS), smem, stream, map_q, map_k, map_v, p);
    QT_CHECK_LAUNCH("attention_prefill_tc");
    return QT_OK;
}

}  // namespace

// q [n_tokens, nq, d] bfloat16; caches [n_pages, nkv, 64, d] bfloat16 (they already hold this step's keys); out like q.
// `status` is a device int that stays 0 unless a wait inside the kernel ran out.
extern "C" int qt_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out, int n_tokens,
                                       int n_pages, const int* block_table, int max_blocks, const int* seq_start,
                                       const int* seq_past, int n_seqs, int max_q_len, int nq, int nkv, int d,
                                       int page_tokens, int ring_tokens, int window, float scale, int* status, void* stream) {
    if (n_seqs == 0 || max_q_len == 0) return QT_OK;
    QT_REQUIRE(n_seqs > 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention_prefill_tc: bad head counts nq=%d nkv=%d (B=%d)", nq, nkv, n_seqs);
    QT_REQUIRE(d == 64 || d == 128, "attention_prefill_tc: head_dim=%d (this kernel takes 64 or 128)", d);
    QT_REQUIRE(page_tokens == PAGE, "attention_prefill_tc: pages of %d tokens (this kernel walks pages of %d)", page_tokens, PAGE);
    QT_REQUIRE(ring_tokens >= 0 && ring_tokens % PAGE == 0, "attention_prefill_tc: the ring of %d tokens is not a whole number of pages", ring_tokens);
    QT_REQUIRE(ring_tokens == 0 || (window > 0 && ring_tokens >= window), "attention_prefill_tc: a ring of %d tokens cannot hold a window of %d", ring_tokens, window);
    QT_REQUIRE(n_seqs <= 65535 && (max_q_len + BQ - 1) / BQ <= 65535 && max_blocks > 0 && n_pages > 0 && n_tokens > 0, "attention_prefill_tc: bad sizes");
    QT_REQUIRE(status != nullptr, "attention_prefill_tc: a status word is required");
    QT_REQUIRE(((uintptr_t)q % 16 == 0) && ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0) && ((uintptr_t)out % 16 == 0),
               "attention_prefill_tc: operands must be 16-byte aligned");
    CUtensorMap map_q, map_k, map_v;
    int rc = tensor_map(&map_q, q, (uint64_t)n_tokens, (uint64_t)nq * d, BQ);
    if (rc) return rc;
    rc = tensor_map(&map_k, k_cache, (uint64_t)n_pages * nkv * PAGE, (uint64_t)d, PAGE);
    if (rc) return rc;
    rc = tensor_map(&map_v, v_cache, (uint64_t)n_pages * nkv * PAGE, (uint64_t)d, PAGE);
    if (rc) return rc;
    TcAttnParams p{(__nv_bfloat16*)out, block_table, max_blocks, seq_start, seq_past, nq, nkv, ring_tokens, window, scale, status};
    cudaStream_t s = (cudaStream_t)stream;
    // key tiles of one page, two blocks per SM: measured 12-22 % faster than tiles of two pages with one block per SM
    if (d == 64) return launch<64, 64>(map_q, map_k, map_v, p, n_seqs, max_q_len, s);
    return launch<128, 64>(map_q, map_k, map_v, p, n_seqs, max_q_len, s);
}

QT_DEFINE_LAST_ERROR(attention_tc)
