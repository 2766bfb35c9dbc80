// Next-token choice from float logits [rows, vocab]: greedy argmax (ties go to the lowest id) and
// temperature sampling by inverse CDF in vocabulary order.  The reference only has
// argmax (luozoupi/Qwen-Triton models/core.py:405).
#include "common.cuh"

#include <math.h>

using namespace qt;

constexpr int SMP_THREADS = 1024;

// One block per row.
__global__ void __launch_bounds__(SMP_THREADS) argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = row[i];
        if (x > v || (x == v && i < idx)) { v = x; idx = i; }
    }
    auto better = [](float av, int ai, float bv, int bi) { return bv > av || (bv == av && bi < ai); };
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, off);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
        if (better(v, idx, ov, oi)) { v = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = v; best_i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = best_v[lane]; idx = best_i[lane];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, off);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
            if (better(v, idx, ov, oi)) { v = ov; idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
    }
}

extern "C" int qt_argmax(const float* logits, int* out, int rows, int vocab, void* stream) {
    QT_REQUIRE(rows >= 0 && vocab > 0, "argmax: bad sizes rows=%d vocab=%d", rows, vocab);
    if (rows == 0) return QT_OK;
    launch_kernel(argmax_kernel, dim3(rows), dim3(SMP_THREADS), 0, (cudaStream_t)stream, logits, out, vocab);
    QT_CHECK_LAUNCH("argmax");
    return QT_OK;
}

// One block per row: token = first index whose cumulative weight exceeds uniform * total, with
// weight_i = exp((logit_i - max) / T).  Thread t owns the contiguous ids [t * span, (t + 1) * span).
__device__ __forceinline__ int sample_row(const float* __restrict__ row, float inv_t, float uniform, int vocab) {
    __shared__ float scratch[32];
    __shared__ float sums[SMP_THREADS];
    __shared__ int chosen;
    const int span = (vocab + blockDim.x - 1) / blockDim.x;
    const int begin = min(vocab, (int)threadIdx.x * span), end = min(vocab, begin + span);

    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = scratch[threadIdx.x & 31];   // blockDim.x == 1024: all 32 entries are written
    mx = warp_max(mx);

    float local = 0.f;
    for (int i = begin; i < end; ++i) local += expf((row[i] - mx) * inv_t);
    sums[threadIdx.x] = local;
    if (threadIdx.x == 0) chosen = vocab - 1;
    __syncthreads();
    if (threadIdx.x == 0) {
        // serial scan over the 1024 partial sums: a fixed order, so the choice is reproducible
        float total = 0.f;
        for (int t = 0; t < SMP_THREADS; ++t) total += sums[t];
        const float target = uniform * total;
        float running = 0.f;
        int owner = -1;
        for (int t = 0; t < SMP_THREADS; ++t) {
            if (running + sums[t] > target) { owner = t; break; }
            running += sums[t];
        }
        if (owner >= 0) {
            const int b = min(vocab, owner * span), e = min(vocab, b + span);
            int pick = e - 1;
            for (int i = b; i < e; ++i) {
                running += expf((row[i] - mx) * inv_t);
                if (running > target) { pick = i; break; }
            }
            chosen = pick;
        }
    }
    __syncthreads();
    return chosen;
}

__global__ void __launch_bounds__(SMP_THREADS) sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                                                            const float* __restrict__ uniform, int* __restrict__ out, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int token = sample_row(logits + (size_t)blockIdx.x * vocab, 1.f / temperature[blockIdx.x], uniform[blockIdx.x], vocab);
    if (threadIdx.x == 0) out[blockIdx.x] = token;
}

extern "C" int qt_sample(const float* logits, const float* temperature, const float* uniform, int* out, int rows,
                         int vocab, void* stream) {
    QT_REQUIRE(rows >= 0 && vocab > 0, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
    if (rows == 0) return QT_OK;
    launch_kernel(sample_kernel, dim3(rows), dim3(SMP_THREADS), 0, (cudaStream_t)stream, logits, temperature, uniform, out, vocab);
    QT_CHECK_LAUNCH("sample");
    return QT_OK;
}

// The same choice with the uniform number made here: the counter-based stream of (seed, request, step), three rounds of
// the splitmix64 finaliser, its top 24 bits as a float in [0, 1).  keys[2 r] is row r's request number, keys[2 r + 1]
// its step number; nothing but these few integers has to come from the host for a step's sampling.
__device__ __forceinline__ unsigned long long mix64(unsigned long long v) {
    v += 0x9E3779B97F4A7C15ull;
    v = (v ^ (v >> 30)) * 0xBF58476D1CE4E5B9ull;
    v = (v ^ (v >> 27)) * 0x94D049BB133111EBull;
    return v ^ (v >> 31);
}

__global__ void __launch_bounds__(SMP_THREADS) sample_keyed_kernel(const float* __restrict__ logits, float inv_t, unsigned long long seed,
                                                                  const int* __restrict__ keys, int* __restrict__ out, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    unsigned long long state = mix64(seed);
    state = mix64(state ^ (unsigned long long)(long long)keys[2 * blockIdx.x]);
    state = mix64(state ^ (unsigned long long)(long long)keys[2 * blockIdx.x + 1]);
    const float uniform = (float)(state >> 40) * (1.f / 16777216.f);
    const int token = sample_row(logits + (size_t)blockIdx.x * vocab, inv_t, uniform, vocab);
    if (threadIdx.x == 0) out[blockIdx.x] = token;
}

extern "C" int qt_sample_keyed(const float* logits, float temperature, long long seed, const int* keys, int* out, int rows, int vocab,
                               void* stream) {
    QT_REQUIRE(rows >= 0 && vocab > 0, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
    QT_REQUIRE(temperature > 0.f, "sample: temperature must be positive (greedy choice is qt_argmax)");
    if (rows == 0) return QT_OK;
    launch_kernel(sample_keyed_kernel, dim3(rows), dim3(SMP_THREADS), 0, (cudaStream_t)stream, logits, 1.f / temperature,
                  (unsigned long long)seed, keys, out, vocab);
    QT_CHECK_LAUNCH("sample");
    return QT_OK;
}

// ----------------------------------------------------------------------------- chosen tokens as the next step's input
// ids[i] holds a row number of `chosen` (or a negative number); it is replaced by the token chosen for that row
// (0 for a negative number or a row that does not exist).  With this the next step can be launched before the host
// has seen the tokens.  Tokens outside the vocabulary (the sampling kernels produce none) are clamped into it.
__global__ void feed_tokens_kernel(int* __restrict__ ids, const int* __restrict__ chosen, int n, int n_chosen, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int row = ids[i];
    int token = (row >= 0 && row < n_chosen) ? chosen[row] : 0;
    token = token < 0 ? 0 : (token >= vocab ? vocab - 1 : token);
    ids[i] = token;
}

extern "C" int qt_feed_tokens(int* ids, const int* chosen, int n, int n_chosen, int vocab, void* stream) {
    QT_REQUIRE(n >= 0 && n_chosen >= 0 && vocab > 0, "feed_tokens: bad sizes n=%d rows=%d V=%d", n, n_chosen, vocab);
    if (n == 0) return QT_OK;
    launch_kernel(feed_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, (cudaStream_t)stream, ids, chosen, n, n_chosen, vocab);
    QT_CHECK_LAUNCH("feed_tokens");
    return QT_OK;
}

QT_DEFINE_LAST_ERROR(sampling)
