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

template <int BX, typename TO>
__global__ void __launch_bounds__(THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                          const __grid_constant__ CUtensorMap map_x, TO* __restrict__ out,
                                                          int M, int N, int kb_total, int kb_per_split,
                                                          size_t split_stride, int stages, int* status) {
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
                if (n < N) {
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
// 128 weight rows and 128 of the tile's 256 tokens per K slice (32 KB instead of 48 KB for the same MMA work, so a
// third less traffic from L2 and a six-stage ring), the even-ranked block issues tcgen05.mma.cta_group::2 with
// M = 256, N = 256, and each block reads its own 128 accumulator rows back and stores them.
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
// Waits on mbarriers are bounded as above; every thread of both blocks reaches the cluster barriers at the start
// and at the end whatever happens in between, so no block waits for one that has left.
constexpr int PAIR_X = 256;                         // tokens per pair tile = MMA N
constexpr int PAIR_HALF = PAIR_X / 2;               // tokens staged by each block
constexpr uint32_t PAIR_STAGE_BYTES = W_BYTES + PAIR_HALF * BK * 2;
constexpr int PAIR_STAGES = 6;
constexpr uint32_t PAIR_TMEM_COLS = 2 * PAIR_X;     // two accumulators

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// SWIGLU: the weight's rows alternate 16 of a gate projection and 16 of an up projection (see swiglu in
// elementwise.cu); a warp of the epilogue then holds both halves of 16 features in its 32 accumulator lanes, and the
// kernel stores silu(gate) * up, [M, N / 2], instead of the product itself.
constexpr int SWIGLU_GROUP = 16;

template <typename TO, bool SWIGLU>
__global__ void __launch_bounds__(THREADS, 1) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                  const __grid_constant__ CUtensorMap map_x, TO* __restrict__ out,
                                                                  int M, int N, int kb_total, int kb_per_split, int splits,
                                                                  size_t split_stride, int act, int* status) {
    // instruction descriptor: float accumulator, bfloat16 A and B, both K-major, N = 256, M = 256 over the pair
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PAIR_X >> 3) << 17) | ((uint32_t)((2 * BW) >> 4) << 24);
    constexpr int S = PAIR_STAGES;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    // barriers: full[S], empty[S], acc_full[2], acc_empty[2]; then the tensor-memory address
    const uint32_t full0 = base + S * PAIR_STAGE_BYTES, empty0 = full0 + 8 * S, acc_full0 = empty0 + 8 * S, acc_empty0 = acc_full0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + (size_t)S * PAIR_STAGE_BYTES + 8 * (2 * S + 4));

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int w_tiles = (N + 2 * BW - 1) / (2 * BW), x_tiles = (M + PAIR_X - 1) / PAIR_X;
    const int n_tiles = w_tiles * x_tiles, n_items = n_tiles * splits;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    // work item -> its tile, the plane of its K range, the first K block and the number of K blocks
    auto item_range = [&](int item, int& tile, int& split, int& kb0, int& nkb) {
        split = splits == 1 ? 0 : item / n_tiles;
        tile = item - split * n_tiles;
        kb0 = split * kb_per_split;
        nkb = min(kb_total, kb0 + kb_per_split) - kb0;
    };

    if (threadIdx.x == 0) {
        prefetch_tensor_map(&map_w);
        prefetch_tensor_map(&map_x);
        for (int s = 0; s < S; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 8); }   // four epilogue warps of each block
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
            for (int item = pair; item < n_items && ok; item += n_pairs) {
                int tile, split, kb0, nkb, w_tile, x_tile;
                item_range(item, tile, split, kb0, nkb);
                tile_coords(tile, w_tiles, x_tiles, w_tile, x_tile);
                const int w0 = w_tile * 2 * BW + (int)rank * BW, x_stage0 = x_tile * PAIR_X + (int)rank * PAIR_HALF;
                int kb = 0;
                if (item == pair) {
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
            if (pair >= n_items) pdl_wait();
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // This thread's instructions are the tensor pipe's critical path (four MMAs of 128 cycles per K slice): the
            // descriptors are formed once and stepped by additions, stage and phase are counters, and a barrier that
            // is already complete costs one probe.
            const uint64_t a_desc0 = operand_desc(base), b_desc0 = operand_desc(base + W_BYTES);
            int it = 0, s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = pair; item < n_items && ok; item += n_pairs, ++it) {
                int tile, split, kb0, nkb;
                item_range(item, tile, split, kb0, nkb);
                const int b = it & 1;
                // the epilogues of both blocks have read this accumulator's previous tile (passes at once the first time)
                if (!mbar_wait(acc_empty0 + 8 * b, (((uint32_t)it >> 1) & 1u) ^ 1u, status, 4)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(b * PAIR_X);
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait(full0 + 8 * s, phase, status, 2)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t a_desc = a_desc0 + (uint64_t)(s * (PAIR_STAGE_BYTES >> 4));
                    const uint64_t b_desc = b_desc0 + (uint64_t)(s * (PAIR_STAGE_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_pair(tmem_d, a_desc + 2 * k, b_desc + 2 * k, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(empty0 + 8 * s);        // the stage is free in both blocks once these MMAs have read it
                    if (++s == S) { s = 0; phase ^= 1u; }
                }
                if (ok) umma_commit_pair(acc_full0 + 8 * b); // both halves of this accumulator are complete
            }
        }
    } else {
        const int quarter = warp & 3;
        const uint32_t leader_acc_empty0 = map_to_cta(acc_empty0, 0);
        pdl_wait();                                          // the output may still be read by an earlier kernel
        int it = 0;
        for (int item = pair; item < n_items; item += n_pairs, ++it) {
            int tile, split, kb0, nkb, w_tile, x_tile;
            item_range(item, tile, split, kb0, nkb);
            tile_coords(tile, w_tiles, x_tiles, w_tile, x_tile);
            TO* __restrict__ plane = out + (size_t)split * split_stride;
            const int b = it & 1;
            if (!mbar_wait(acc_full0 + 8 * b, ((uint32_t)it >> 1) & 1u, status, 3)) break;
            tc_fence_after();
            const int n = w_tile * 2 * BW + (int)rank * BW + quarter * 32 + lane;
            const int x0 = x_tile * PAIR_X;
            // SWIGLU: lanes 0..15 hold the gate rows of 16 features, lanes 16..31 the up rows of the same features.
            // Of every two tokens the lower lanes finish the first and the upper lanes the second: one exchange
            // gives each half the value it lacks, and all 32 lanes compute and store.
            const int feature = ((n - lane) >> 1) + (lane & 15), features = N >> 1;
            const bool upper = (lane & 16) != 0;
            const bool stores = SWIGLU ? feature < features : n < N;
#pragma unroll 1
            for (int c = 0; c < PAIR_X; c += 16) {
                uint32_t v[16];
                tmem_load16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * PAIR_X + c), v);
                if (SWIGLU) {
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const float mine0 = __uint_as_float(v[j]), mine1 = __uint_as_float(v[j + 1]);
                        const float got = __shfl_xor_sync(0xffffffffu, upper ? mine0 : mine1, 16);
                        const float g = upper ? got : mine0;          // lower lanes: token j (their gate, the partner's up)
                        const float u = upper ? mine1 : got;          // upper lanes: token j + 1 (the partner's gate, their up)
                        const int m = x0 + c + j + (upper ? 1 : 0);
                        if (stores && m < M) plane[(size_t)m * features + feature] = from_float<TO>(gate_activation<true>(g, act) * u);
                    }
                } else if (stores) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = x0 + c + j;
                        if (m < M) plane[(size_t)m * N + n] = from_float<TO>(__uint_as_float(v[j]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + 8 * b);    // this warp has read its rows of the accumulator
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

template <typename TO, bool SWIGLU>
int launch_pair(const CUtensorMap& map_w, const CUtensorMap& map_x, TO* out, int M, int N, int kb_total, int splits,
                size_t split_stride, int act, int* status, cudaStream_t stream) {
    const size_t smem = (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + (2 * PAIR_STAGES + 4) * 8 + 16;
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
    const unsigned pairs = (unsigned)(items < resident_pairs ? items : resident_pairs);
    const int kb_per_split = (kb_total + splits - 1) / splits;
    launch_kernel_cluster(gemm_tc_pair_kernel<TO, SWIGLU>, dim3(2 * pairs), dim3(THREADS), smem, stream, 2, map_w, map_x, out, M, N, kb_total,
                          kb_per_split, splits, split_stride, act, status);
    QT_CHECK_LAUNCH("gemm_tc_pair");
    return QT_OK;
}

// ----------------------------------------------------------------------------- host side
template <int BX, typename TO>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, TO* out, int M, int N, int kb_total, int splits,
           size_t split_stride, int stages, int* status, cudaStream_t stream) {
    constexpr uint32_t STAGE_BYTES = W_BYTES + BX * BK * 2;
    // Up to 32 tokens a block streams weights through a three-stage ring (54 KB), so that four blocks share an SM and
    // the next product's blocks can move in beside this one's last blocks and fetch their first weight tiles early
    // (measured 3-4 % on a decode step against two blocks with six stages).  Larger tiles: two blocks per SM, which
    // overlap each other's epilogue and keep two MMA issuers feeding the tensor pipe.
    const int budget = (BX <= 32 ? 56 : 110) * 1024;
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
        cudaError_t err = cudaFuncSetAttribute(gemm_tc_kernel<BX, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "gemm_tc: cannot raise shared memory: %s", cudaGetErrorString(err));
        configured = true;
    }
    const int kb_per_split = (kb_total + splits - 1) / splits;
    dim3 grid(((N + BW - 1) / BW) * ((M + BX - 1) / BX), 1, splits);
    launch_kernel(gemm_tc_kernel<BX, TO>, dim3(grid), dim3(THREADS), smem, stream, map_w, map_x, out, M, N, kb_total, kb_per_split, split_stride, stages, status);
    QT_CHECK_LAUNCH("gemm_tc");
    return QT_OK;
}


template <typename TO>
int dispatch_tile(int bx, const CUtensorMap& map_w, const CUtensorMap& map_x, TO* out, int M, int N, int kb_total, int splits,
                  size_t split_stride, int stages, int* status, cudaStream_t stream) {
    switch (bx) {
        case 16: return launch<16, TO>(map_w, map_x, out, M, N, kb_total, splits, split_stride, stages, status, stream);
        case 32: return launch<32, TO>(map_w, map_x, out, M, N, kb_total, splits, split_stride, stages, status, stream);
        case 64: return launch<64, TO>(map_w, map_x, out, M, N, kb_total, splits, split_stride, stages, status, stream);
        case 128: return launch<128, TO>(map_w, map_x, out, M, N, kb_total, splits, split_stride, stages, status, stream);
        case 256: return launch<256, TO>(map_w, map_x, out, M, N, kb_total, splits, split_stride, stages, status, stream);
    }
    QT_FAIL(QT_ERR_ARG, "gemm_tc: token tile %d is not one of 16, 32, 64, 128, 256", bx);
}

}  // namespace

// out[splits, M, N] (bfloat16 with splits == 1, or float) = x[M, K] * w[N, K]^T, bfloat16 inputs.
// `token_tile` is the number of tokens per block (16..256); `splits` must leave no split without K
// blocks: (splits - 1) * ceil(ceil(K/64) / splits) < ceil(K/64).  `status` is a device int that stays
// 0 unless a wait inside the kernel ran out (1 = producer, 2 = MMA issuer, 3 = epilogue).
// `stages` > 0 overrides the depth of the shared-memory ring (a tuning knob; 0 picks the default).
extern "C" int qt_gemm_tc(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int token_tile,
                          int splits, long long split_stride, int stages, int* status, void* stream) {
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
    if (out_dtype == QT_BF16)
        return dispatch_tile<__nv_bfloat16>(token_tile, map_w, map_x, (__nv_bfloat16*)out, M, N, kb_total, splits, (size_t)split_stride, stages, status, s);
    if (out_dtype == QT_F32)
        return dispatch_tile<float>(token_tile, map_w, map_x, (float*)out, M, N, kb_total, splits, (size_t)split_stride, stages, status, s);
    QT_FAIL(QT_ERR_ARG, "gemm_tc: unknown output type %d", out_dtype);
}

// The same product by pairs of blocks (see gemm_tc_pair_kernel): bfloat16 or float output, meant for many tokens (a
// pair covers 256 weight rows x 256 tokens); out[splits, M, N] in float when `splits` > 1, under the rule above.  With `swiglu` the weight's rows alternate 16 of a gate and
// 16 of an up projection and `out` is [M, N / 2] = act(gate) * up (`act`: one of QT_ACT_*).  Codes in `status`: as above, 4 = the MMA issuer
// waiting for the epilogues to free an accumulator.
extern "C" int qt_gemm_tc_pair(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int swiglu,
                               int act, int splits, long long split_stride, int* status, void* stream) {
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
    if (out_dtype == QT_BF16 && swiglu) return launch_pair<__nv_bfloat16, true>(map_w, map_x, (__nv_bfloat16*)out, M, N, kb_total, 1, 0, act, status, s);
    if (out_dtype == QT_BF16) return launch_pair<__nv_bfloat16, false>(map_w, map_x, (__nv_bfloat16*)out, M, N, kb_total, 1, 0, 0, status, s);
    if (out_dtype == QT_F32 && !swiglu) return launch_pair<float, false>(map_w, map_x, (float*)out, M, N, kb_total, splits, (size_t)split_stride, 0, status, s);
    QT_FAIL(QT_ERR_ARG, "gemm_tc_pair: output type %d%s is not offered", out_dtype, swiglu ? " with the SiLU-gated epilogue" : "");
}

QT_DEFINE_LAST_ERROR(gemm_tc)
