// bfloat16 matrix product for few tokens (a decode step) with what follows it done in the same launch.
//
// Y[M, N] = X[M, K] * W[N, K]^T as in gemm_tc.cu: the weight is the MMA's A operand (128 rows per tile), the tokens
// its B operand, TMA stages 64-element K slices, tcgen05.mma accumulates in tensor memory.  With few tokens the
// product is bound by reading the weight, so K is cut into `splits` ranges to have blocks on every SM; here the
// blocks of one weight tile form a thread-block cluster and add their partial sums through distributed shared
// memory (each block parks its accumulator tile in its own shared memory, and after a cluster barrier every block
// sums, in the fixed order of the ranks, a share of the tile's tokens from all of them).  No partial sums pass
// through global memory, and the kernel that used to add them up is not needed: its work is this kernel's epilogue.
//
// The epilogues (STORE, RESIDUAL, SWIGLU, QKV) and the deferred norm factor s_m are stated in fused_epilogue.cuh.
//
// Warp roles and bounded waits as in gemm_tc.cu.  Every thread of every block reaches both cluster barriers whatever
// happens before them, so no block waits for one that has left.  What a launch adds to the plain product is its
// tail, after the last MMA: park, barrier, the peers' sums, the epilogue; to keep it short the epilogue's operands
// are fetched under the main loop and the closing barrier is arrived at before the epilogue's own work.
//
// Counterparts in luozoupi/Qwen-Triton: kernels/matmul.py:52-97, kernels/rmsnorm.py:100-133, kernels/residual_add.py:50-60,
// kernels/swiglu.py:84-92, kernels/rope.py:99-120, kernels/cache.py:71-98 (one launch each, or two).
#include "fused_epilogue.cuh"
#include "tc_common.cuh"

using namespace qt;
using namespace qt_tc;
using namespace qt_epi;

namespace {

constexpr int BW = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr uint32_t W_BYTES = BW * BK * 2;
constexpr int MAX_SPLITS = 8;              // the portable cluster size (larger clusters measured much slower: 14 against 9 us)
constexpr int SPLIT_BATCH = 8;             // peer loads in flight at a time

struct FusedParams {
    int kb_total, kb_per_split, stages, splits;
    int* status;
    EpilogueParams e;
};

__device__ __forceinline__ float4 ld_cluster4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ float2 ld_cluster2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_arrive_all() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_all() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
template <int BX, int EPI>
__global__ void __launch_bounds__(THREADS, (BX <= 32 ? 4 : 2)) gemm_fused_kernel(const __grid_constant__ CUtensorMap map_w,
                                                             const __grid_constant__ CUtensorMap map_x,
                                                             const __grid_constant__ FusedParams p) {
    constexpr uint32_t X_BYTES = BX * BK * 2;
    constexpr uint32_t STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr uint32_t TMEM_COLS = BX < 32 ? 32 : BX;
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BX >> 3) << 17) | ((uint32_t)(BW >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const int stages = p.stages;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * STAGE_BYTES);
    const uint32_t full0 = base + stages * STAGE_BYTES, empty0 = full0 + 8 * stages, tmem_full = empty0 + 8 * stages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * stages + 1);
    // Once this block's MMAs are done its ring is free: the accumulator tile is parked there as float [token][row].
    float* park = reinterpret_cast<float*>(smem);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int splits = p.splits;
    const int rank = (int)(blockIdx.x % (unsigned)splits);          // = the block's rank in its cluster (clusters lie along x)
    const int w_tile = (int)(blockIdx.x / (unsigned)splits), x_tile = blockIdx.y;
    const int w0 = w_tile * BW, x0 = x_tile * BX;
    const EpilogueParams& ep = p.e;
    const int m_tile = min(BX, ep.M - x0);
    const int kb_begin = rank * p.kb_per_split;
    const int nkb = min(p.kb_total, kb_begin + p.kb_per_split) - kb_begin;
    int* status = p.status;

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
    Operands first;                                                 // of the first token this warp finishes (warps 2..5)

    if (warp == 0) {
        if (lane == 0) {
            // weights depend on no earlier kernel: they fill the ring before the wait for the producer of X
            const int ahead = min(nkb, stages);
            for (int i = 0; i < ahead; ++i) {
                mbar_expect_tx(full0 + 8 * i, STAGE_BYTES);
                tma_load_2d(base + i * STAGE_BYTES, &map_w, full0 + 8 * i, (kb_begin + i) * BK, w0);
            }
            pdl_wait();
            for (int i = 0; i < ahead; ++i)
                tma_load_2d(base + i * STAGE_BYTES + W_BYTES, &map_x, full0 + 8 * i, (kb_begin + i) * BK, x0);
            int s = ahead == stages ? 0 : ahead;
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
            const uint64_t a_desc0 = operand_desc(base), b_desc0 = operand_desc(base + W_BYTES);
            int s = 0;
            uint32_t phase = 0;
            for (int i = 0; i < nkb; ++i) {
                if (!mbar_wait(full0 + 8 * s, phase, status, 2)) break;
                tc_fence_after();
                const uint64_t a_desc = a_desc0 + (uint64_t)(s * (STAGE_BYTES >> 4));
                const uint64_t b_desc = b_desc0 + (uint64_t)(s * (STAGE_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    umma_bf16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, IDESC, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);
                if (++s == stages) { s = 0; phase ^= 1u; }
            }
            umma_commit(tmem_full);
        }
    } else {
        const int quarter = warp & 3;
        pdl_wait();
        if (rank * 4 + (warp - 2) < m_tile) first = load_operands<EPI>(ep, x0 + rank * 4 + (warp - 2), w0, lane);
        const bool ready = mbar_wait(tmem_full, 0, status, 3);      // every K slice has been read: the ring is free
        tc_fence_after();
        const int row = quarter * 32 + lane;
        if (ready) {
#pragma unroll 1
            for (int c = 0; c < m_tile; c += 16) {
                uint32_t v[16];
                tmem_load16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, v);
#pragma unroll
                for (int j = 0; j < 16; ++j) park[(c + j) * BW + row] = __uint_as_float(v[j]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                             // every block of the cluster has parked its tile

    // Every block sums a share of the tile's tokens from all parked tiles, in the order of the ranks.  A warp arrives at
    // the closing barrier as soon as it has read its last token's partial sums (its epilogue then runs under the
    // barrier), and nobody leaves before every warp of the cluster has done so: no tile is freed while it is read.
    bool arrived = false;
    if (warp >= 2 && *(volatile int*)status == 0) {
        const uint32_t park0 = smem_u32(park);
        const int t0 = rank * 4 + (warp - 2), stride = 4 * splits;
        for (int t = t0; t < m_tile; t += stride) {
            const int m = x0 + t;
            const Operands ops = t == t0 ? first : load_operands<EPI>(ep, m, w0, lane);
            const bool last = t + stride >= m_tile;
            if (EPI == EPI_SWIGLU) {
                const uint32_t off = (uint32_t)(t * BW + swiglu_gate_row(lane)) * 4u;
                float2 g = make_float2(0.f, 0.f), u = make_float2(0.f, 0.f);
                for (int r0 = 0; r0 < splits; r0 += SPLIT_BATCH) {
                    float2 gs[SPLIT_BATCH], us[SPLIT_BATCH];
#pragma unroll
                    for (int i = 0; i < SPLIT_BATCH; ++i)
                        if (r0 + i < splits) {
                            const uint32_t at = map_to_cta(park0, (uint32_t)(r0 + i)) + off;
                            gs[i] = ld_cluster2(at);
                            us[i] = ld_cluster2(at + 64u);
                        }
#pragma unroll
                    for (int i = 0; i < SPLIT_BATCH; ++i)
                        if (r0 + i < splits) { g.x += gs[i].x; g.y += gs[i].y; u.x += us[i].x; u.y += us[i].y; }
                }
                if (last) { cluster_arrive_all(); arrived = true; }
                finish_swiglu(ep, ops, g, u, m, w_tile, lane);
            } else {
                const uint32_t off = (uint32_t)(t * BW + 4 * lane) * 4u;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int r0 = 0; r0 < splits; r0 += SPLIT_BATCH) {
                    float4 parts[SPLIT_BATCH];
#pragma unroll
                    for (int i = 0; i < SPLIT_BATCH; ++i)
                        if (r0 + i < splits) parts[i] = ld_cluster4(map_to_cta(park0, (uint32_t)(r0 + i)) + off);
#pragma unroll
                    for (int i = 0; i < SPLIT_BATCH; ++i)
                        if (r0 + i < splits) { v.x += parts[i].x; v.y += parts[i].y; v.z += parts[i].z; v.w += parts[i].w; }
                }
                if (last) { cluster_arrive_all(); arrived = true; }
                finish<EPI>(ep, ops, v, m, w_tile, lane);
            }
        }
    }
    if (!arrived) cluster_arrive_all();
    cluster_wait_all();
    if (*(volatile int*)status != 0) {
        const unsigned long long t0 = global_timer();
        while (global_timer() - t0 < 2000000ull) __nanosleep(1000);
    }
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <int BX, int EPI>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, FusedParams p, int stages, cudaStream_t stream) {
    constexpr uint32_t STAGE_BYTES = W_BYTES + BX * BK * 2;
    const int most = (224 * 1024) / (int)STAGE_BYTES;
    if (stages <= 0) {
        // up to 32 tokens: three stages (54 KB), four blocks per SM; more: two blocks with deeper rings (as in gemm_tc.cu)
        stages = ((BX <= 32 ? 56 : 110) * 1024 - 2048) / (int)STAGE_BYTES;
        if (stages > 8) stages = 8;
    }
    if (stages > most) stages = most;
    // the ring also parks the accumulator tile, BX x 128 floats
    while ((size_t)stages * STAGE_BYTES < (size_t)BX * BW * 4) ++stages;
    if (stages < 2) stages = 2;
    p.stages = stages;
    const size_t smem = (size_t)stages * STAGE_BYTES + 1024 + (2 * stages + 1) * 8 + 16;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_fused_kernel<BX, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "gemm_fused: cannot raise shared memory: %s", cudaGetErrorString(err));
        configured = true;
    }
    dim3 grid(((p.e.N + BW - 1) / BW) * p.splits, (p.e.M + BX - 1) / BX, 1);
    launch_kernel_cluster(gemm_fused_kernel<BX, EPI>, grid, dim3(THREADS), smem, stream, (unsigned)p.splits, map_w, map_x, p);
    QT_CHECK_LAUNCH("gemm_fused");
    return QT_OK;
}

template <int EPI>
int dispatch_tile(int bx, const CUtensorMap& map_w, const CUtensorMap& map_x, const FusedParams& p, int stages, cudaStream_t stream) {
    switch (bx) {
        case 16: return launch<16, EPI>(map_w, map_x, p, stages, stream);
        case 32: return launch<32, EPI>(map_w, map_x, p, stages, stream);
        case 64: return launch<64, EPI>(map_w, map_x, p, stages, stream);
        case 128: return launch<128, EPI>(map_w, map_x, p, stages, stream);
    }
    QT_FAIL(QT_ERR_ARG, "gemm_fused: token tile %d is not one of 16, 32, 64, 128", bx);
}

}  // namespace

// x [M, K] bfloat16, w [N, K] bfloat16.  `epilogue` picks what is done with the product (see the top of the file) and
// which of the pointers are read; `splits` (1..8) is the size of the cluster that shares a weight tile and must leave
// no rank without K blocks: (splits - 1) * ceil(ceil(K / 64) / splits) < ceil(K / 64).  `status` as in qt_gemm_tc.
extern "C" int qt_gemm_fused(const void* x, const void* w, int M, int N, int K, int token_tile, int splits, int stages, int epilogue,
                             const float* sq_in, int sq_tiles, int norm_width, float eps,
                             void* out, int out_dtype, int act,
                             float* residual, const float* norm_w, void* xw, float* sq_out,
                             void* q_out, void* k_cache, void* v_cache, const int* token_seq, const int* token_pos,
                             const int* block_table, int max_blocks, const float* q_w, const float* k_w, float qk_eps,
                             const float* cos_sin, int rotary_dim, int max_pos, int nq, int nkv, int d, int page_tokens,
                             int ring_tokens, int write_kv, int interleaved, int* status, void* stream) {
    QT_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_fused: bad sizes M=%d N=%d K=%d", M, N, K);
    QT_REQUIRE(K % 8 == 0, "gemm_fused: K=%d must be a multiple of 8 (rows must start on 16-byte boundaries for TMA)", K);
    QT_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_fused: operands must be 16-byte aligned");
    QT_REQUIRE(status != nullptr, "gemm_fused: a status word is required");
    const int kb_total = (K + BK - 1) / BK;
    QT_REQUIRE(splits >= 1 && splits <= MAX_SPLITS && splits <= kb_total, "gemm_fused: splits=%d (1..%d) for %d K blocks", splits, MAX_SPLITS, kb_total);
    const int per = (kb_total + splits - 1) / splits;
    QT_REQUIRE((splits - 1) * per < kb_total, "gemm_fused: splits=%d would leave a rank without K blocks (%d blocks)", splits, kb_total);
    QT_REQUIRE((M + token_tile - 1) / token_tile <= 65535, "gemm_fused: M=%d is too many tokens for tiles of %d", M, token_tile);
    FusedParams p = {};
    p.kb_total = kb_total; p.kb_per_split = per; p.splits = splits; p.status = status;
    EpilogueParams& e = p.e;
    e.M = M; e.N = N;
    e.sq_in = sq_in; e.sq_tiles = sq_tiles; e.inv_hidden = norm_width > 0 ? 1.f / (float)norm_width : 0.f; e.eps = eps;
    e.out = out; e.out_is_float = out_dtype == QT_F32; e.act = act;
    e.residual = residual; e.norm_w = norm_w; e.xw = (__nv_bfloat16*)xw; e.sq_out = sq_out;
    e.q_out = (__nv_bfloat16*)q_out; e.k_cache = (__nv_bfloat16*)k_cache; e.v_cache = (__nv_bfloat16*)v_cache;
    e.token_seq = token_seq; e.token_pos = token_pos; e.block_table = block_table; e.max_blocks = max_blocks;
    e.q_w = q_w; e.k_w = k_w; e.qk_eps = qk_eps; e.cos_sin = cos_sin; e.rotary_dim = rotary_dim; e.max_pos = max_pos;
    e.nq = nq; e.nkv = nkv; e.d = d; e.page_tokens = page_tokens; e.ring_tokens = ring_tokens; e.write_kv = write_kv; e.interleaved = interleaved;
    int rc = check_epilogue("gemm_fused", epilogue, e, out_dtype);
    if (rc) return rc;
    CUtensorMap map_w, map_x;
    rc = tensor_map(&map_w, w, (uint64_t)N, (uint64_t)K, BW);
    if (rc) return rc;
    rc = tensor_map(&map_x, x, (uint64_t)M, (uint64_t)K, (uint32_t)token_tile);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    switch (epilogue) {
        case EPI_STORE: return dispatch_tile<EPI_STORE>(token_tile, map_w, map_x, p, stages, s);
        case EPI_RESIDUAL: return dispatch_tile<EPI_RESIDUAL>(token_tile, map_w, map_x, p, stages, s);
        case EPI_SWIGLU: return dispatch_tile<EPI_SWIGLU>(token_tile, map_w, map_x, p, stages, s);
        default: return dispatch_tile<EPI_QKV>(token_tile, map_w, map_x, p, stages, s);
    }
}

QT_DEFINE_LAST_ERROR(gemm_fused)
