// C[M, N] = A[M, K] * W[N, K]^T with float accumulation on the FMA pipe, for any sizes and for
// float or bfloat16 inputs.  This is the whole 32-bit path's matrix product (true float: no
// tensor cores, no reduced-precision mode; sums blocked over K in three levels) and the bfloat16 path's choice for shapes the
// tensor-core kernel refuses.  Counterpart in luozoupi/Qwen-Triton: kernels/matmul.py:52-97.
#include "common.cuh"

using namespace qt;

constexpr int GS_BM = 64, GS_BN = 64, GS_BK = 16, GS_THREADS = 256;

template <typename TI, typename TO>
__global__ void __launch_bounds__(GS_THREADS) gemm_simt_kernel(const TI* __restrict__ a, const TI* __restrict__ w,
                                                              TO* __restrict__ c, int M, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float as[GS_BK][GS_BM + 4];
    __shared__ float ws[GS_BK][GS_BN + 4];
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;   // thread computes rows ty*4.., cols tx*4..
    const int load_row = threadIdx.x / 4, load_k = (threadIdx.x % 4) * 4;
    // Three levels of float sums: the 16 products of a K tile, 16 tiles, and the groups of 16 tiles.  One running sum
    // over a K of thousands would lose about four times as many low-order bits as a blocked CPU product does.
    float acc[4][4] = {}, mid[4][4] = {};
    for (int k0 = 0, tile = 0; k0 < K; k0 += GS_BK, ++tile) {
        float part[4][4] = {};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + load_k + i;
            const int am = m0 + load_row, wn = n0 + load_row;
            as[load_k + i][load_row] = (am < M && k < K) ? to_float(a[(size_t)am * K + k]) : 0.f;
            ws[load_k + i][load_row] = (wn < N && k < K) ? to_float(w[(size_t)wn * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GS_BK; ++k) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = as[k][ty * 4 + i]; wv[i] = ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[i][j] = fmaf(av[i], wv[j], part[i][j]);
        }
        const bool flush = (tile & 15) == 15;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                mid[i][j] += part[i][j];
                if (flush) { acc[i][j] += mid[i][j]; mid[i][j] = 0.f; }
            }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += mid[i][j];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) c[(size_t)m * N + n] = from_float<TO>(acc[i][j]);
        }
    }
}

extern "C" int qt_gemm_simt(const void* a, const void* w, int in_dtype, void* c, int out_dtype, int M, int N, int K,
                            void* stream) {
    QT_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return QT_OK;
    dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM);
    QT_REQUIRE(grid.y <= 65535, "gemm_simt: M=%d is too large for one launch", M);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == QT_F32 && out_dtype == QT_F32) launch_kernel(gemm_simt_kernel<float, float>, dim3(grid), dim3(GS_THREADS), 0, s, (const float*)a, (const float*)w, (float*)c, M, N, K);
    else if (in_dtype == QT_BF16 && out_dtype == QT_BF16) launch_kernel(gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(grid), dim3(GS_THREADS), 0, s, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (__nv_bfloat16*)c, M, N, K);
    else if (in_dtype == QT_BF16 && out_dtype == QT_F32) launch_kernel(gemm_simt_kernel<__nv_bfloat16, float>, dim3(grid), dim3(GS_THREADS), 0, s, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (float*)c, M, N, K);
    else QT_FAIL(QT_ERR_ARG, "gemm_simt: unsupported element types %d -> %d", in_dtype, out_dtype);
    QT_CHECK_LAUNCH("gemm_simt");
    return QT_OK;
}

QT_DEFINE_LAST_ERROR(gemm_simt)
