// bfloat16 matrix product on the fifth-generation tensor cores: Y[M, N] = X[M, K] * W[N, K]^T.
//
// The weight is the MMA's A operand (128 weight rows fill the instruction's M), the activations
// are its B operand (16 to 256 tokens on the instruction's N), so one kernel serves a decode step
// of a few tokens and a prefill of thousands.  Both operands are K-major in global memory, as the
// checkpoint stores them; TMA (cp.async.bulk.tensor, 128-byte swizzle; every block fetches its own tiles) stages
// 64-element K slices in shared memory, one elected thread issues tcgen05.mma with the float
// accumulator in tensor memory, and four warps read it back with tcgen05.ld and store Y
// (transposed back to [M, N]) as bfloat16 or float.  Split-K writes float partial sums
// [splits, M, N] that the consuming kernel adds up in a fixed order.
//
// Warp roles (192 threads): warp 0 lane 0 = TMA producer, warp 1 = tensor-memory allocation and
// (lane 0) MMA issue, warps 2..5 = epilogue, each on the 32 accumulator lanes its warp id allows.
// Every mbarrier wait is bounded: after about a second it records a code in `status` and the
// block winds down (waits briefly for copies in flight, frees its tensor memory, returns).
//
// Counterpart in luozoupi/Qwen-Triton: kernels/matmul.py:52-97 (tl.dot tiles, W transposed per call).
#include "tc_common.cuh"

using namespace qt;
using namespace qt_tc;

namespace {

constexpr int BW = 128;        // weight rows per tile = MMA M
constexpr int BK = 64;         // K elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;     // K per tcgen05.mma for 16-bit inputs
constexpr int THREADS = 192;
constexpr uint32_t W_BYTES = BW * BK * 2;

// Order of output tiles: groups of RASTER_W consecutive weight tiles, inside a group weight tiles fastest, then
// token tiles.  Blocks that run at the same time then cover a near-square patch of the output whose weight and
// activation tiles stay in L2, instead of one long row that streams a whole operand per token tile.
constexpr int RASTER_W = 16;
__device__ __forceinline__ void tile_coords(int t, int w_tiles, int x_tiles, int& w, int& x) {
    const int per_group = RASTER_W * x_tiles;
    const int group = t / per_group, r = t % per_group;
    const int first = group * RASTER_W;
    const int width = min(RASTER_W, w_tiles - first);
    w = first + r % width;
    x = r / width;
}

// GATED: the weight's rows alternate 16 of a gate projection and 16 of an up projection; the 32 accumulator lanes of
// an epilogue warp are then the gate rows (lanes 0..15) and the up rows (16..31) of the same 16 features, and the
// kernel stores act(gate) * up, [M, N / 2] (one K range only).  Of every two tokens the lower lanes finish the first
// and the upper lanes the second: one exchange gives each half the value it lacks, and all 32 lanes compute and store.
template <int BX, typename TO, bool GATED>
__global__ void __launch_bounds__(THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                          const __grid_constant__ CUtensorMap map_x, TO* __restrict__ out,
                                                          int M, int N, int kb_total, int kb_per_split,
                                                          size_t split_stride, int stages, int act, int* status) {
    constexpr uint32_t X_BYTES = BX * BK * 2;
    constexpr uint32_t STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr uint32_t TMEM_COLS = BX < 32 ? 32 : BX;
    // instruction descriptor: float accumulator, bfloat16 A and B, both K-major, N = BX, M = 128
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BX >> 3) << 17) | ((uint32_t)(BW >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                  // swizzled tiles need 1024-byte alignment
    uint8_t* smem = smem_raw + (base - raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * STAGE_BYTES);
    const uint32_t full0 = base + stages * STAGE_BYTES, empty0 = full0 + 8 * stages, tmem_full = empty0 + 8 * stages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * stages + 1);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int w_tile, x_tile;
    tile_coords(blockIdx.x, (N + BW - 1) / BW, (M + BX - 1) / BX, w_tile, x_tile);
    const int w0 = w_tile * BW, x0 = x_tile * BX, split = blockIdx.z;
    const int kb_begin = split * kb_per_split;
    const int nkb = min(kb_total, kb_begin + kb_per_split) - kb_begin;   // >= 1: the host sizes the splits so

    if (threadIdx.x == 0) {
        prefetch_tensor_map(&map_w);
        prefetch_tensor_map(&map_x);
        for (int s = 0; s < stages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(tmem_full, 1);
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
            // the weight depends on no earlier kernel: fill the ring with weight tiles first, then wait for
            // the kernel that produces the activations, then fetch their tiles
            const int ahead = min(nkb, stages);
            for (int i = 0; i < ahead; ++i) {
                mbar_expect_tx(full0 + 8 * i, STAGE_BYTES);
                tma_load_2d(base + i * STAGE_BYTES, &map_w, full0 + 8 * i, (kb_begin + i) * BK, w0);
            }
            pdl_wait();
            for (int i = 0; i < ahead; ++i)
                tma_load_2d(base + i * STAGE_BYTES + W_BYTES, &map_x, full0 + 8 * i, (kb_begin + i) * BK, x0);
            int s = ahead == stages ? 0 : ahead;            // stage and phase of K slice `ahead`, then counted on
            uint32_t phase = ahead == stages ? 1u : 0u;
            for (int i = ahead; i < nkb; ++i) {
                if (!mbar_wait(empty0 + 8 * s, phase ^ 1u, status, 1)) break;
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                const uint32_t dst = base + s * STAGE_BYTES;
                tma_load_2d(dst, &map_w, full0 + 8 * s, (kb_begin + i) * BK, w0);
                tma_load_2d(dst + W_BYTES, &map_x, full0 + 8 * s, (kb_begin + i) * BK, x0);
                if (++s == stages) { s = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // This thread's instructions are the tensor pipe's critical path: descriptors are formed once and
            // stepped by additions (the address field counts 16-byte units), stage and phase by counters.
            const uint64_t a_desc0 = operand_desc(base), b_desc0 = operand_desc(base + W_BYTES);
            int s = 0;
            uint32_t phase = 0;
            for (int i = 0; i < nkb; ++i) {
                if (!mbar_wait(full0 + 8 * s, phase, status, 2)) break;
                tc_fence_after();
                const uint64_t a_desc = a_desc0 + (uint64_t)(s * (STAGE_BYTES >> 4));
                const uint64_t b_desc = b_desc0 + (uint64_t)(s * (STAGE_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)      // 32 bytes further along K inside the swizzled row
                    umma_bf16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, IDESC, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);               // the stage is free once these MMAs have read it
                if (++s == stages) { s = 0; phase ^= 1u; }
            }
            umma_commit(tmem_full);                        // the accumulator is complete
        }
    } else {
        const int quarter = warp & 3;                      // the accumulator lanes this warp may read
        pdl_wait();                                        // the output may still be read by an earlier kernel
        const bool ready = mbar_wait(tmem_full, 0, status, 3);
        tc_fence_after();
        const int n = w0 + quarter * 32 + lane;
        TO* dst = out + (size_t)split * split_stride;
        if (ready) {
#pragma unroll 1
            for (int c = 0; c < BX; c += 16) {
                uint32_t v[16];
                tmem_load16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, v);
                if (GATED) {
                    const int features = N >> 1, feature = ((n - lane) >> 1) + (lane & 15);
                    const bool upper = (lane & 16) != 0;
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const float mine0 = __uint_as_float(v[j]), mine1 = __uint_as_float(v[j + 1]);
                        const float got = __shfl_xor_sync(0xffffffffu, upper ? mine0 : mine1, 16);
                        const float g = upper ? got : mine0;          // lower lanes: token j (their gate, the partner's up)
                        const float u = upper ? mine1 : got;          // upper lanes: token j + 1 (the partner's gate, their up)
                        const int m = x0 + c + j + (upper ? 1 : 0);
                        if (feature < features && m < M) dst[(size_t)m * features + feature] = from_float<TO>(gate_activation<true>(g, act) * u);
                    }
                } else if (n < N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = x0 + c + j;
                        if (m < M) dst[(size_t)m * N + n] = from_float<TO>(__uint_as_float(v[j]));
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


// ----------------------------------------------------------------------------- CTA pairs, for many tokens
// The same product with two blocks (a cluster on the two SMs of a TPC) per 256 x 256 output tile: each block stages
// 128 of the tile's tokens and 128 of its weight rows per K slice (32 KB instead of 48 KB for the same MMA work, so a
// third less traffic from L2 and a six-stage ring), and the even-ranked block issues tcgen05.mma.cta_group::2 with
// M = 256, N = 256.  Here the tokens are the MMA's rows and the weight rows its columns (the other way round than in
// the kernel above; both operands are K-major 128 x 64 tiles, so only their roles differ): a thread of the epilogue
// then holds consecutive output features of one token and stores them 16 bytes at a time, and the gate and up halves
// of a SwiGLU group arrive in the same thread.
//
// Split-K for a few hundred tokens, where the tiles alone do not fill the TPCs: a work item is (tile, K range), the
// items of one K range come first, and each range's sums go to a float plane of their own, out[split, M, N], which
// the consuming kernel adds up in a fixed order.
//
// One pair per TPC, persistent: a pair walks the tiles pair, pair + pairs, ... with two accumulators in tensor memory
// (all 512 columns), so that the epilogue of a tile runs under the MMAs of the next.  One block per SM is also what
// keeps the allocation safe: tcgen05.alloc.cta_group::2 takes columns on both SMs, and two pairs sharing a TPC that
// allocate at the same moment can each hold one SM's allocator while waiting for the other's (seen as a rare hang
// with two such blocks per SM); with 192 KB of shared memory per block no second pair fits beside this one.
//
// The last wave by K ranges (`tail_tiles` > 0, one plane): tiles seldom divide by the pairs, and a last wave that is
// half empty costs a whole tile's time.  With R tiles left for P pairs, the last R pairs each finish one of them and
// the first P - R pairs are helpers.  If there are fewer helpers than tiles, a helper takes the ends of the K ranges
// of n neighbouring tiles, a K range of 1 / (n + 1) of each, so that it has as much to do as the pair that finishes
// one of them; if there are more, the K range of a tile is cut into equal parts for its g helpers and its finisher.
// All cuts of neighbouring tiles lie at the same K blocks and the pairs of a kind walk them at the same time, so the
// operand tiles are shared in L2 as they are between whole tiles.  A helper writes its accumulator as float into a
// scratch slot and raises a flag per epilogue warp; the finishing pair's epilogue warps add up the slots of their
// tile, in slot order, and store the sum into the accumulator in tensor memory before the MMAs of the finishing piece
// start, which then accumulate on top of it.  Helpers do their pieces before anything else and finishers theirs
// last, and the sums are fetched one item ahead: slots are written and read under the MMAs of whole tiles, and the
// last epilogue is an ordinary one.  A helper never waits for another pair; all pairs are resident (one per TPC),
// and the finisher's wait is bounded like the others.  A flag is raised once and lowered once (by its reader) per
// launch, so the words are zero again when the kernel ends.
//
// Waits on mbarriers are bounded as above; every thread of both blocks reaches the cluster barriers at the start
// and at the end whatever happens in between, so no block waits for one that has left.
constexpr int PAIR_X = 256;                         // tokens per pair tile = MMA M
constexpr int PAIR_HALF = PAIR_X / 2;               // tokens staged by each block
constexpr int PAIR_W = 2 * BW;                      // weight rows per pair tile = MMA N
constexpr uint32_t PAIR_STAGE_BYTES = W_BYTES + PAIR_HALF * BK * 2;
constexpr int PAIR_STAGES = 6;
constexpr uint32_t PAIR_TMEM_COLS = 2 * PAIR_W;     // two accumulators

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// What a pair does, in order: a helper's pieces of last-wave tiles, the pair's `whole` items (a tile, or a tile's K
// range of one plane), and a finisher's piece of its last-wave tile.
enum { ITEM_WHOLE = 0, ITEM_PARTIAL = 1, ITEM_FINISH = 2 };
struct PairItem {
    int tile, split, kb0, nkb, kind, slot0, slot1;   // ITEM_PARTIAL writes slot0; ITEM_FINISH starts from slots slot0 .. slot1 - 1
};
__host__ __device__ __forceinline__ int part_begin(int index, int total, int parts) { return (int)((long long)index * total / parts); }
// the part that holds `element` when `total` elements are cut into `parts` (part i is part_begin(i) .. part_begin(i + 1))
__host__ __device__ __forceinline__ int part_of(int element, int total, int parts) {
    int i = (int)((long long)element * parts / total);
    while (part_begin(i + 1, total, parts) <= element) ++i;
    while (part_begin(i, total, parts) > element) --i;
    return i;
}
struct PairWork {
    int pair, n_pairs, n_tiles, splits, kb_total, kb_per_split, n_first, n_whole, n_last;
    int tile0, first_tile, small;                       // a helper of several tiles: its first tile and its K blocks of each
    PairItem single;                                 // a helper's only piece, or a finisher's piece

    __device__ PairWork(int pair_, int n_pairs_, int n_tiles_, int splits_, int kb_total_, int kb_per_split_, int tail_tiles)
        : pair(pair_), n_pairs(n_pairs_), n_tiles(n_tiles_), splits(splits_), kb_total(kb_total_), kb_per_split(kb_per_split_) {
        const int whole_items = (n_tiles - tail_tiles) * splits;
        n_whole = pair < whole_items ? (whole_items - pair + n_pairs - 1) / n_pairs : 0;
        n_first = n_last = 0;
        if (tail_tiles <= 0) return;
        const int R = tail_tiles, H = n_pairs - tail_tiles, kb = kb_total;
        tile0 = n_tiles - tail_tiles;
        single.split = 0;
        if (R >= H) {                                    // a helper per run of tiles, one slot per tile
            if (pair < H) {
                first_tile = part_begin(pair, R, H);
                n_first = part_begin(pair + 1, R, H) - first_tile;
                small = max(1, kb / (n_first + 1));
            } else {
                const int j = pair - H, h = part_of(j, R, H);
                const int n = part_begin(h + 1, R, H) - part_begin(h, R, H);
                single.tile = tile0 + j; single.kb0 = 0; single.nkb = kb - max(1, kb / (n + 1));
                single.kind = ITEM_FINISH; single.slot0 = j; single.slot1 = j + 1;
                n_last = 1;
            }
        } else {                                         // several helpers per tile, one slot per helper
            const int j = pair < H ? part_of(pair, H, R) : pair - H;
            const int h0 = part_begin(j, H, R), g = part_begin(j + 1, H, R) - h0;
            const int mine = pair < H ? pair - h0 + 1 : 0;   // which of the g + 1 parts of the tile's K range
            single.tile = tile0 + j;
            single.kb0 = part_begin(mine, kb, g + 1); single.nkb = part_begin(mine + 1, kb, g + 1) - single.kb0;
            if (pair < H) { single.kind = ITEM_PARTIAL; single.slot0 = single.slot1 = pair; n_first = 1; first_tile = -1; }
            else { single.kind = ITEM_FINISH; single.slot0 = h0; single.slot1 = h0 + g; n_last = 1; }
        }
    }
    __device__ __forceinline__ int count() const { return n_first + n_whole + n_last; }
    // the item (if any) that starts from other pairs' sums
    __device__ __forceinline__ int finish_at() const { return n_last ? n_first + n_whole : -1; }
    __device__ __forceinline__ PairItem item(int it) const {
        PairItem r;
        if (it < n_first) {
            if (first_tile < 0) return single;
            r.tile = tile0 + first_tile + it; r.split = 0; r.kb0 = kb_total - small; r.nkb = small;
            r.kind = ITEM_PARTIAL; r.slot0 = r.slot1 = first_tile + it;
            return r;
        }
        it -= n_first;
        if (it >= n_whole) return single;
        const int index = pair + it * n_pairs;
        r.split = splits == 1 ? 0 : index / n_tiles;
        r.tile = index - r.split * n_tiles;
        r.kb0 = r.split * kb_per_split;
        r.nkb = min(kb_total, r.kb0 + kb_per_split) - r.kb0;
        r.kind = ITEM_WHOLE; r.slot0 = r.slot1 = 0;
        return r;
    }
};
constexpr int PAIR_SLOT_FLOATS = PAIR_X * PAIR_W;    // one pair's accumulator tile in the scratch of the last wave
constexpr int PAIR_FLAGS = 8;                       // per pair: one word per epilogue warp of its two blocks

// SWIGLU: the weight's rows alternate 16 of a gate projection and 16 of an up projection (see swiglu in
// elementwise.cu); 32 accumulator columns of a token are then the gate and up values of 16 features, and the kernel
// stores act(gate) * up, [M, N / 2], instead of the product itself.
constexpr int SWIGLU_GROUP = 16;

template <typename TO> __device__ __forceinline__ void store8(TO* dst, const float (&f)[8]);
template <> __device__ __forceinline__ void store8<float>(float* dst, const float (&f)[8]) {
    reinterpret_cast<float4*>(dst)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(dst)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* dst, const float (&f)[8]) {
    uint4 packed;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(f[0], f[1]); packed.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(f[2], f[3]); packed.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(f[4], f[5]); packed.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(f[6], f[7]); packed.w = *reinterpret_cast<uint32_t*>(&h);
    *reinterpret_cast<uint4*>(dst) = packed;
}

template <typename TO, bool SWIGLU>
__global__ void __launch_bounds__(THREADS, 1) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                  const __grid_constant__ CUtensorMap map_x, TO* __restrict__ out,
                                                                  int M, int N, int kb_total, int kb_per_split, int splits,
                                                                  size_t split_stride, int act, int vector_stores, int tail_tiles,
                                                                  float* __restrict__ tail_scratch, int* tail_flags, int* status) {
    // instruction descriptor: float accumulator, bfloat16 A and B, both K-major, N = 256 weight rows, M = 256 tokens over the pair
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PAIR_W >> 3) << 17) | ((uint32_t)(PAIR_X >> 4) << 24);
    constexpr int S = PAIR_STAGES;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    // barriers: full[S], empty[S], acc_full[2], acc_empty[2], acc_seeded; then the tensor-memory address
    const uint32_t full0 = base + S * PAIR_STAGE_BYTES, empty0 = full0 + 8 * S, acc_full0 = empty0 + 8 * S, acc_empty0 = acc_full0 + 16;
    const uint32_t acc_seeded = acc_empty0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + (size_t)S * PAIR_STAGE_BYTES + 8 * (2 * S + 5));

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int w_tiles = (N + PAIR_W - 1) / PAIR_W, x_tiles = (M + PAIR_X - 1) / PAIR_X;
    const int n_tiles = w_tiles * x_tiles;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const PairWork work(pair, n_pairs, n_tiles, splits, kb_total, kb_per_split, tail_tiles);
    const int n_mine = work.count(), finish_at = work.finish_at();

    if (threadIdx.x == 0) {
        prefetch_tensor_map(&map_w);
        prefetch_tensor_map(&map_x);
        for (int s = 0; s < S; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 8); }   // four epilogue warps of each block
        mbar_init(acc_seeded, 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(PAIR_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();                                      // barriers of both blocks exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t leader_full0 = map_to_cta(full0, 0);
            int s = 0;                                       // stage and phase of the next K slice, over all tiles
            uint32_t phase = 0;
            bool ok = true;
            for (int it = 0; it < n_mine && ok; ++it) {
                const PairItem item = work.item(it);
                const int kb0 = item.kb0, nkb = item.nkb;
                int w_tile, x_tile;
                tile_coords(item.tile, w_tiles, x_tiles, w_tile, x_tile);
                const int w0 = w_tile * PAIR_W + (int)rank * BW, x_stage0 = x_tile * PAIR_X + (int)rank * PAIR_HALF;
                int kb = 0;
                if (it == 0) {
                    // the weight depends on no earlier kernel: fill the ring with weight tiles first, then wait for
                    // the kernel that produces the activations, then fetch their tiles
                    const int ahead = min(nkb, S);
                    for (int i = 0; i < ahead; ++i) {
                        if (leader) mbar_expect_tx(full0 + 8 * i, 2 * PAIR_STAGE_BYTES);
                        tma_load_2d_pair(base + i * PAIR_STAGE_BYTES, &map_w, leader_full0 + 8 * i, (kb0 + i) * BK, w0);
                    }
                    pdl_wait();
                    for (int i = 0; i < ahead; ++i)
                        tma_load_2d_pair(base + i * PAIR_STAGE_BYTES + W_BYTES, &map_x, leader_full0 + 8 * i, (kb0 + i) * BK, x_stage0);
                    kb = ahead;
                    if (ahead == S) phase = 1u; else s = ahead;
                }
                for (; kb < nkb; ++kb) {
                    if (!mbar_wait(empty0 + 8 * s, phase ^ 1u, status, 1)) { ok = false; break; }
                    if (leader) mbar_expect_tx(full0 + 8 * s, 2 * PAIR_STAGE_BYTES);
                    const uint32_t dst = base + s * PAIR_STAGE_BYTES;
                    tma_load_2d_pair(dst, &map_w, leader_full0 + 8 * s, (kb0 + kb) * BK, w0);
                    tma_load_2d_pair(dst + W_BYTES, &map_x, leader_full0 + 8 * s, (kb0 + kb) * BK, x_stage0);
                    if (++s == S) { s = 0; phase ^= 1u; }
                }
            }
            if (n_mine == 0) pdl_wait();
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // This thread's instructions are the tensor pipe's critical path (four MMAs of 128 cycles per K slice): the
            // descriptors are formed once and stepped by additions, stage and phase are counters, and a barrier that
            // is already complete costs one probe.  The token tiles are the MMA's A, the weight tiles its B.
            const uint64_t a_desc0 = operand_desc(base + W_BYTES), b_desc0 = operand_desc(base);
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int it = 0; it < n_mine && ok; ++it) {
                const int nkb = work.item(it).nkb;
                const int b = it & 1;
                // the epilogues of both blocks have read this accumulator's previous tile (passes at once the first time)
                if (!mbar_wait(acc_empty0 + 8 * b, (((uint32_t)it >> 1) & 1u) ^ 1u, status, 4)) break;
                // a finishing piece starts from the other pairs' sums, which the epilogue warps of both blocks put there
                const bool seeded = it == finish_at;
                if (seeded && !mbar_wait(acc_seeded, 0, status, 4)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(b * PAIR_W);
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait(full0 + 8 * s, phase, status, 2)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t a_desc = a_desc0 + (uint64_t)(s * (PAIR_STAGE_BYTES >> 4));
                    const uint64_t b_desc = b_desc0 + (uint64_t)(s * (PAIR_STAGE_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_pair(tmem_d, a_desc + 2 * k, b_desc + 2 * k, IDESC, (seeded || kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(empty0 + 8 * s);        // the stage is free in both blocks once these MMAs have read it
                    if (++s == S) { s = 0; phase ^= 1u; }
                }
                if (ok) umma_commit_pair(acc_full0 + 8 * b); // both halves of this accumulator are complete
            }
        }
    } else {
        // A thread of the epilogue owns one token of the tile (its accumulator lane) and walks the tile's 256 weight
        // rows 32 at a time.
        const int quarter = warp & 3;
        const uint32_t leader_acc_empty0 = map_to_cta(acc_empty0, 0);
        pdl_wait();                                          // the output may still be read by an earlier kernel
        const int slot_row = (int)rank * PAIR_HALF + quarter * 32 + lane;   // this thread's token within the tile
        const int my_flag = (int)rank * 4 + quarter;
        const int features = N >> 1;
        const uint32_t lanes = tmem_base + ((uint32_t)(quarter * 32) << 16);
        // The finishing piece's accumulator (this warp's tokens of it), seeded with the sums that the pairs before this
        // one left in their slots.  Called once this warp has read the accumulator's previous tile.
        auto seed = [&]() -> bool {
            const PairItem item = work.item(finish_at);
            int w_tile, x_tile;
            tile_coords(item.tile, w_tiles, x_tiles, w_tile, x_tile);
            bool peers_ready = true;
            for (int q = item.slot0; q < item.slot1 && peers_ready; ++q)
                peers_ready = __all_sync(0xffffffffu, flag_wait(tail_flags + q * PAIR_FLAGS + my_flag, status, 6));
            if (!peers_ready) return false;
            const uint32_t taddr = lanes + (uint32_t)((finish_at & 1) * PAIR_W);
#pragma unroll 1
            for (int c = 0; c < PAIR_W && w_tile * PAIR_W + c < N; c += 32) {
                float4 sum[8];
                for (int q = item.slot0; q < item.slot1; ++q) {
                    const float4* __restrict__ slot = reinterpret_cast<const float4*>(tail_scratch + (size_t)q * PAIR_SLOT_FLOATS) + slot_row;
                    float4 part[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) part[j] = __ldcg(slot + (size_t)(c / 4 + j) * PAIR_X);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (q == item.slot0) sum[j] = part[j];
                        else { sum[j].x += part[j].x; sum[j].y += part[j].y; sum[j].z += part[j].z; sum[j].w += part[j].w; }
                    }
                }
                uint32_t v[32];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[4 * j] = __float_as_uint(sum[j].x); v[4 * j + 1] = __float_as_uint(sum[j].y);
                    v[4 * j + 2] = __float_as_uint(sum[j].z); v[4 * j + 3] = __float_as_uint(sum[j].w);
                }
                tmem_store32(taddr + (uint32_t)c, v);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cluster(map_to_cta(acc_seeded, 0));
                for (int q = item.slot0; q < item.slot1; ++q) tail_flags[q * PAIR_FLAGS + my_flag] = 0;   // read: the flags go down again
            }
            return true;
        };
        // one item ahead of the finishing piece: the accumulator it will use is the one this warp read last
        const int seed_at = finish_at < 0 ? -1 : max(finish_at - 1, 0);
        for (int it = 0; it < n_mine; ++it) {
            if (it == seed_at && !seed()) break;
            const PairItem item = work.item(it);
            int w_tile, x_tile;
            tile_coords(item.tile, w_tiles, x_tiles, w_tile, x_tile);
            const int b = it & 1;
            if (!mbar_wait(acc_full0 + 8 * b, ((uint32_t)it >> 1) & 1u, status, 3)) break;
            tc_fence_after();
            const uint32_t taddr = lanes + (uint32_t)(b * PAIR_W);
            if (item.kind == ITEM_PARTIAL) {
                // not this pair's tile to finish: the accumulator goes to this pair's slot, laid out so that a warp
                // writes 512 consecutive bytes per instruction ([four columns][token]), and this warp's flag tells
                // the finishing pair's warp of the same tokens
                float4* __restrict__ slot = reinterpret_cast<float4*>(tail_scratch + (size_t)item.slot0 * PAIR_SLOT_FLOATS) + slot_row;
#pragma unroll 1
                for (int c = 0; c < PAIR_W; c += 32) {
                    uint32_t v[32];
                    tmem_load32(taddr + (uint32_t)c, v);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        slot[(size_t)(c / 4 + j) * PAIR_X] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                                         __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                }
                tc_fence_before();
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_cluster(leader_acc_empty0 + 8 * b);
                    st_release_gpu(tail_flags + item.slot0 * PAIR_FLAGS + my_flag, 1);
                }
                continue;
            }
            const int m = x_tile * PAIR_X + slot_row;
            const int n0 = w_tile * PAIR_W;
            TO* __restrict__ plane = out + (size_t)item.split * split_stride;
            TO* __restrict__ row = SWIGLU ? plane + (size_t)m * features + (n0 >> 1) : plane + (size_t)m * N + n0;
#pragma unroll 1
            for (int c = 0; c < PAIR_W; c += 32) {
                if (n0 + c >= N) break;
                uint32_t v[32];
                __syncwarp();                                // lanes beyond M skip the stores; the load wants the whole warp
                tmem_load32(taddr + (uint32_t)c, v);
                if (m >= M) continue;
                if (SWIGLU) {
                    // columns c .. c + 15 are the gate rows of 16 features, c + 16 .. c + 31 the up rows of the same
                    const int f0 = (n0 + c) >> 1;
                    TO* dst = row + (c >> 1);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float f[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            f[j] = gate_activation<true>(__uint_as_float(v[8 * h + j]), act) * __uint_as_float(v[16 + 8 * h + j]);
                        if (vector_stores && f0 + 8 * h + 8 <= features) {
                            store8<TO>(dst + 8 * h, f);
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (f0 + 8 * h + j < features) dst[8 * h + j] = from_float<TO>(f[j]);
                        }
                    }
                } else {
#pragma unroll
                    for (int h = 0; h < 4; ++h) {
                        float f[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[8 * h + j]);
                        if (vector_stores && n0 + c + 8 * h + 8 <= N) {
                            store8<TO>(row + c + 8 * h, f);
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (n0 + c + 8 * h + j < N) row[c + 8 * h + j] = from_float<TO>(f[j]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + 8 * b);   // this warp has read its tokens of the accumulator
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*(volatile int*)status != 0) {                       // a wait gave up: let copies in flight land before the blocks leave
        const unsigned long long t0 = global_timer();
        while (global_timer() - t0 < 2000000ull) __nanosleep(1000);
    }
    cluster_sync_all();                                      // the other block no longer reads this block's tiles or barriers
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(PAIR_TMEM_COLS) : "memory");
    }
}

// Tiles of the last wave to cut by K ranges (see the kernel): none if the tiles divide by the pairs, if a piece would
// be left without a K block, or if the caller gave no scratch for this many pairs; `tail` > 0 then forces it.
// Otherwise (`tail` < 0) by a model of the time saved, in microseconds, with figures measured on pair tiles in a
// prefill: a K block of a pair tile takes 0.35 us; a helper's epilogue (256 KB of float sums into its slot) 7 us, so a
// helper of several tiles is held up where its K ranges are shorter than that; a finisher reads a slot in 9 us, which
// hides under the whole tile before its piece and shows beyond it.  The cut is made where it saves 3 us or more
// and there is a whole wave before the last one.
int pick_tail_tiles(long long n_tiles, int pairs, int kb_total, int tail, int tail_pairs) {
    if (tail == 0 || tail_pairs < pairs || pairs < 2) return 0;
    const int rest = (int)(n_tiles % pairs), helpers = pairs - rest;
    if (rest == 0) return 0;
    const double block = 0.35, slot_write = 7.0, slot_read = 9.0, whole = kb_total * block;
    double last_wave;
    if (rest >= helpers) {
        const int most = (rest + helpers - 1) / helpers;     // tiles of the busiest helper
        if (kb_total < most + 1) return 0;
        const int small = kb_total / (most + 1);
        const double helper = most * (small * block > slot_write ? small * block : slot_write);
        const double finisher = (kb_total - small) * block;
        last_wave = (helper > finisher ? helper : finisher) + (slot_read > whole ? slot_read - whole : 0.0);
    } else {
        const int most = (helpers + rest - 1) / rest, fewest = helpers / rest;   // helpers per tile
        if (kb_total < most + 1) return 0;
        const int longest = (kb_total + fewest) / (fewest + 1);
        last_wave = longest * block + (most * slot_read > whole ? most * slot_read - whole : 0.0);
    }
    if (tail > 0) return rest;
    return (whole - last_wave >= 3.0 && n_tiles > pairs) ? rest : 0;
}

template <typename TO, bool SWIGLU>
int launch_pair(const CUtensorMap& map_w, const CUtensorMap& map_x, TO* out, int M, int N, int kb_total, int splits,
                size_t split_stride, int act, int tail, float* tail_scratch, int* tail_flags, int tail_pairs, int* status,
                cudaStream_t stream) {
    const size_t smem = (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + (2 * PAIR_STAGES + 5) * 8 + 16;
    static int resident_pairs = 0;                           // pairs the device runs at once (one per TPC that can host a cluster)
    if (resident_pairs == 0) {
        cudaError_t err = cudaFuncSetAttribute(gemm_tc_pair_kernel<TO, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "gemm_tc_pair: cannot raise shared memory: %s", cudaGetErrorString(err));
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(2 * (unsigned)sm_count());
        config.blockDim = dim3(THREADS);
        config.dynamicSmemBytes = smem;
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = 2;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        int clusters = 0;
        err = cudaOccupancyMaxActiveClusters(&clusters, gemm_tc_pair_kernel<TO, SWIGLU>, &config);
        if (err != cudaSuccess || clusters < 1)
            QT_FAIL(QT_ERR_LAUNCH, "gemm_tc_pair: no cluster of two blocks fits the device (%s)", cudaGetErrorString(err));
        resident_pairs = clusters;
    }
    const long long items = (long long)((N + 2 * BW - 1) / (2 * BW)) * ((M + PAIR_X - 1) / PAIR_X) * splits;
    unsigned pairs = (unsigned)(items < resident_pairs ? items : resident_pairs);
    const int kb_per_split = (kb_total + splits - 1) / splits;
    const int tail_tiles = splits == 1 && tail_scratch && tail_flags ? pick_tail_tiles(items, resident_pairs, kb_total, tail, tail_pairs) : 0;
    if (tail_tiles) pairs = (unsigned)resident_pairs;        // fewer tiles than pairs: all of them by K ranges over every pair
    // 16-byte stores need every output row (and plane) to start on a 16-byte boundary
    const int per16 = 16 / (int)sizeof(TO), row_elems = SWIGLU ? N / 2 : N;
    const int vector_stores = ((uintptr_t)out % 16 == 0 && row_elems % per16 == 0 && split_stride % per16 == 0) ? 1 : 0;
    launch_kernel_cluster(gemm_tc_pair_kernel<TO, SWIGLU>, dim3(2 * pairs), dim3(THREADS), smem, stream, 2, map_w, map_x, out, M, N, kb_total,
                          kb_per_split, splits, split_stride, act, vector_stores, tail_tiles, tail_scratch, tail_flags, status);
    QT_CHECK_LAUNCH("gemm_tc_pair");
    return QT_OK;
}

// ----------------------------------------------------------------------------- host side
template <int BX, typename TO, bool GATED>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, TO* out, int M, int N, int kb_total, int splits,
           size_t split_stride, int stages, int act, int* status, cudaStream_t stream) {
    constexpr uint32_t STAGE_BYTES = W_BYTES + BX * BK * 2;
    // Up to 16 tokens a block streams weights through a three-stage ring (54 KB), so that four blocks share an SM and
    // the next product's blocks can move in beside this one's last blocks and fetch their first weight tiles early
    // (measured 3-4 % on a decode step against two blocks with six stages).  Larger tiles: two blocks per SM with
    // rings of 110 KB, which overlap each other's epilogue and keep two MMA issuers feeding the tensor pipe.  (The
    // 32-token tile used to share the small budget, which is two stages of its 20 KB: a decode step at batch 20 / 32 of
    // the 8B shape took 4.91 / 5.40 ms with that, 4.50 / 4.99 ms with five stages and two blocks.)
    const int budget = (BX <= 16 ? 56 : 110) * 1024;
    const int most = (224 * 1024) / (int)STAGE_BYTES;
    if (stages <= 0) {
        stages = (budget - 2048) / (int)STAGE_BYTES;
        if (stages > 8) stages = 8;
    }
    if (stages > most) stages = most;
    if (stages < 2) stages = 2;
    const size_t smem = (size_t)stages * STAGE_BYTES + 1024 + (2 * stages + 1) * 8 + 16;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_tc_kernel<BX, TO, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "gemm_tc: cannot raise shared memory: %s", cudaGetErrorString(err));
        configured = true;
    }
    const int kb_per_split = (kb_total + splits - 1) / splits;
    dim3 grid(((N + BW - 1) / BW) * ((M + BX - 1) / BX), 1, splits);
    launch_kernel(gemm_tc_kernel<BX, TO, GATED>, dim3(grid), dim3(THREADS), smem, stream, map_w, map_x, out, M, N, kb_total, kb_per_split, split_stride, stages, act, status);
    QT_CHECK_LAUNCH("gemm_tc");
    return QT_OK;
}


template <typename TO, bool GATED>
int dispatch_tile(int bx, const CUtensorMap& map_w, const CUtensorMap& map_x, TO* out, int M, int N, int kb_total, int splits,
                  size_t split_stride, int stages, int act, int* status, cudaStream_t stream) {
    switch (bx) {
        case 16: return launch<16, TO, GATED>(map_w, map_x, out, M, N, kb_total, splits, split_stride, stages, act, status, stream);
        case 32: return launch<32, TO, GATED>(map_w, map_x, out, M, N, kb_total, splits, split_stride, stages, act, status, stream);
        case 64: return launch<64, TO, GATED>(map_w, map_x, out, M, N, kb_total, splits, split_stride, stages, act, status, stream);
        case 128: return launch<128, TO, GATED>(map_w, map_x, out, M, N, kb_total, splits, split_stride, stages, act, status, stream);
        case 256: return launch<256, TO, GATED>(map_w, map_x, out, M, N, kb_total, splits, split_stride, stages, act, status, stream);
    }
    QT_FAIL(QT_ERR_ARG, "gemm_tc: token tile %d is not one of 16, 32, 64, 128, 256", bx);
}

}  // namespace

// out[splits, M, N] (bfloat16 with splits == 1, or float) = x[M, K] * w[N, K]^T, bfloat16 inputs.
// `token_tile` is the number of tokens per block (16..256); `splits` must leave no split without K
// blocks: (splits - 1) * ceil(ceil(K/64) / splits) < ceil(K/64).  `status` is a device int that stays
// 0 unless a wait inside the kernel ran out (1 = producer, 2 = MMA issuer, 3 = epilogue).
// `stages` > 0 overrides the depth of the shared-memory ring (a tuning knob; 0 picks the default).
// With `gated` the weight's rows alternate 16 of a gate and 16 of an up projection and `out` is [M, N / 2] bfloat16 =
// act(gate) * up (`act`: one of QT_ACT_*; one K range only).
extern "C" int qt_gemm_tc(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int token_tile,
                          int splits, long long split_stride, int stages, int gated, int act, int* status, void* stream) {
    QT_REQUIRE(!gated || (splits == 1 && out_dtype == QT_BF16 && N % 32 == 0 && act >= 0 && act < QT_ACT_COUNT),
               "gemm_tc: the gated epilogue writes bfloat16 from one K range of gate and up rows in groups of 16 (N=%d, splits=%d)", N, splits);
    QT_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
    QT_REQUIRE(K % 8 == 0, "gemm_tc: K=%d must be a multiple of 8 (rows must start on 16-byte boundaries for TMA)", K);
    QT_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_tc: operands must be 16-byte aligned");
    QT_REQUIRE(status != nullptr, "gemm_tc: a status word is required");
    const int kb_total = (K + BK - 1) / BK;
    QT_REQUIRE(splits >= 1 && splits <= kb_total, "gemm_tc: splits=%d for %d K blocks", splits, kb_total);
    const int per = (kb_total + splits - 1) / splits;
    QT_REQUIRE((splits - 1) * per < kb_total, "gemm_tc: splits=%d would leave a split without K blocks (%d blocks)", splits, kb_total);
    QT_REQUIRE(out_dtype == QT_F32 || splits == 1, "gemm_tc: split-K partial sums are float");
    QT_REQUIRE((long long)((M + token_tile - 1) / token_tile) * ((N + BW - 1) / BW) < (1ll << 31), "gemm_tc: M=%d x N=%d is too large for one launch", M, N);
    CUtensorMap map_w, map_x;
    int rc = tensor_map(&map_w, w, (uint64_t)N, (uint64_t)K, BW);
    if (rc) return rc;
    rc = tensor_map(&map_x, x, (uint64_t)M, (uint64_t)K, (uint32_t)token_tile);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (gated)
        return dispatch_tile<__nv_bfloat16, true>(token_tile, map_w, map_x, (__nv_bfloat16*)out, M, N, kb_total, 1, 0, stages, act, status, s);
    if (out_dtype == QT_BF16)
        return dispatch_tile<__nv_bfloat16, false>(token_tile, map_w, map_x, (__nv_bfloat16*)out, M, N, kb_total, splits, (size_t)split_stride, stages, 0, status, s);
    if (out_dtype == QT_F32)
        return dispatch_tile<float, false>(token_tile, map_w, map_x, (float*)out, M, N, kb_total, splits, (size_t)split_stride, stages, 0, status, s);
    QT_FAIL(QT_ERR_ARG, "gemm_tc: unknown output type %d", out_dtype);
}

// The same product by pairs of blocks (see gemm_tc_pair_kernel): bfloat16 or float output, meant for many tokens (a
// pair covers 256 weight rows x 256 tokens); out[splits, M, N] in float when `splits` > 1, under the rule above.  With `swiglu` the weight's rows alternate 16 of a gate and
// 16 of an up projection and `out` is [M, N / 2] = act(gate) * up (`act`: one of QT_ACT_*).  Codes in `status`: as above, 4 = the MMA issuer
// waiting for the epilogues to free an accumulator.
// `tail`: 0 = every tile by one pair; -1 = the last wave's tiles by K ranges where that pays; 1 = wherever the tiles do
// not divide by the pairs.  It needs `tail_scratch` (tail_pairs x 256 x 256 floats) and `tail_flags` (tail_pairs x 8
// ints, zero before the first launch and left zero by every launch that ends without a fault); with fewer slots than
// resident pairs, or null pointers, every tile is walked whole.
extern "C" int qt_gemm_tc_pair_slots() { return PAIR_SLOT_FLOATS; }
extern "C" int qt_gemm_tc_pair(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int swiglu,
                               int act, int splits, long long split_stride, int tail, float* tail_scratch, int* tail_flags,
                               int tail_pairs, int* status, void* stream) {
    QT_REQUIRE(act >= 0 && act < QT_ACT_COUNT, "gemm_tc_pair: unknown activation code %d", act);
    QT_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc_pair: bad sizes M=%d N=%d K=%d", M, N, K);
    QT_REQUIRE(K % 8 == 0, "gemm_tc_pair: K=%d must be a multiple of 8 (rows must start on 16-byte boundaries for TMA)", K);
    QT_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_tc_pair: operands must be 16-byte aligned");
    QT_REQUIRE(status != nullptr, "gemm_tc_pair: a status word is required");
    QT_REQUIRE(!swiglu || N % (2 * SWIGLU_GROUP) == 0, "gemm_tc_pair: N=%d is not gate and up rows in groups of %d", N, SWIGLU_GROUP);
    const int kb_total = (K + BK - 1) / BK;
    QT_REQUIRE(splits >= 1 && splits <= kb_total, "gemm_tc_pair: splits=%d for %d K blocks", splits, kb_total);
    QT_REQUIRE((splits - 1) * ((kb_total + splits - 1) / splits) < kb_total, "gemm_tc_pair: splits=%d would leave a split without K blocks (%d blocks)", splits, kb_total);
    QT_REQUIRE(splits == 1 || (out_dtype == QT_F32 && !swiglu), "gemm_tc_pair: split-K partial sums are float and ungated");
    QT_REQUIRE((long long)((M + PAIR_X - 1) / PAIR_X) * ((N + 2 * BW - 1) / (2 * BW)) * splits < (1ll << 30), "gemm_tc_pair: M=%d x N=%d is too large for one launch", M, N);
    CUtensorMap map_w, map_x;
    int rc = tensor_map(&map_w, w, (uint64_t)N, (uint64_t)K, BW);
    if (rc) return rc;
    rc = tensor_map(&map_x, x, (uint64_t)M, (uint64_t)K, (uint32_t)PAIR_HALF);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == QT_BF16 && swiglu) return launch_pair<__nv_bfloat16, true>(map_w, map_x, (__nv_bfloat16*)out, M, N, kb_total, 1, 0, act, tail, tail_scratch, tail_flags, tail_pairs, status, s);
    if (out_dtype == QT_BF16) return launch_pair<__nv_bfloat16, false>(map_w, map_x, (__nv_bfloat16*)out, M, N, kb_total, 1, 0, 0, tail, tail_scratch, tail_flags, tail_pairs, status, s);
    if (out_dtype == QT_F32 && !swiglu) return launch_pair<float, false>(map_w, map_x, (float*)out, M, N, kb_total, splits, (size_t)split_stride, 0, tail, tail_scratch, tail_flags, tail_pairs, status, s);
    QT_FAIL(QT_ERR_ARG, "gemm_tc_pair: output type %d%s is not offered", out_dtype, swiglu ? " with the SiLU-gated epilogue" : "");
}

QT_DEFINE_LAST_ERROR(gemm_tc)
