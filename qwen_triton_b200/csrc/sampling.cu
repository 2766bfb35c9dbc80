// Next-token choice from float logits [rows, vocab]: greedy argmax (ties go to the lowest id) and
// temperature sampling by inverse CDF in vocabulary order, over all tokens or over the most likely ones (top_k,
// top_p).  The reference only has argmax (luozoupi/Qwen-Triton models/core.py:405).
#include "common.cuh"

#include <math.h>

using namespace qt;

constexpr int SMP_THREADS = 1024;

// f(i, row[i]) for every id in [begin, end), shared among `threads` threads of which this is number `me`, in no
// particular order: 16-byte loads where the addresses allow them (single loads up to the first 16-byte boundary and
// after the last), four of them in flight per thread.  A block that walks its row one 4-byte load at a time waits a
// memory round trip per element.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ row, int begin, int end, int me, int threads, F f) {
    if (begin >= end) return;
    const int lead = min(end - begin, (int)(((16u - (unsigned int)((uintptr_t)(row + begin) & 15u)) & 15u) >> 2));
    if (me < lead) f(begin + me, row[begin + me]);
    const int body = begin + lead, quads = (end - body) >> 2;
    const float4* __restrict__ wide = reinterpret_cast<const float4*>(row + body);
    for (int base = me; base < quads; base += 4 * threads) {
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = base + j * threads < quads ? wide[base + j * threads] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (base + j * threads < quads) {
                const int i = body + 4 * (base + j * threads);
                f(i, v[j].x); f(i + 1, v[j].y); f(i + 2, v[j].z); f(i + 3, v[j].w);
            }
    }
    const int tail = body + 4 * quads;
    if (tail + me < end) f(tail + me, row[tail + me]);
}

// One block per row.
__global__ void __launch_bounds__(SMP_THREADS) argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for_each_logit(row, 0, vocab, threadIdx.x, blockDim.x, [&](int i, float x) {
        if (x > v || (x == v && i < idx)) { v = x; idx = i; }
    });
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

// Floats as unsigned integers of the same order (every key of a negative number below every key of a positive one;
// the two zeros, which compare equal, share the key of +0).
__device__ __forceinline__ unsigned int ordered_key(float x) {
    unsigned int bits = __float_as_uint(x);
    if (bits == 0x80000000u) bits = 0u;
    return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

// The largest logit of a row, known to every thread of the block (1,024 threads).
__device__ __forceinline__ float row_max(const float* __restrict__ row, int vocab) {
    __shared__ float scratch[32];
    float mx = -INFINITY;
    for_each_logit(row, 0, vocab, threadIdx.x, blockDim.x, [&](int, float x) { mx = fmaxf(mx, x); });
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = scratch[threadIdx.x & 31];   // blockDim.x == 1024: all 32 entries are written
    return warp_max(mx);
}

// One block per row: token = first index whose cumulative weight exceeds uniform * total, with
// weight_i = exp((logit_i - max) / T) for the logits whose key is at least `floor_key` and 0 for the others (0 keeps
// every token).  Warp w owns the contiguous ids [w * chunk, (w + 1) * chunk) and reads them 32 neighbours at a time:
// the 32 warps' sums are added in warp order, and the warp in whose ids the target falls walks them again with a
// prefix sum over its lanes.  Every sum has a fixed order, so a row and a uniform number give the same token always.
__device__ __forceinline__ int sample_row(const float* __restrict__ row, float inv_t, float uniform, int vocab, float mx,
                                          unsigned int floor_key) {
    __shared__ float warp_total[32];
    __shared__ int owner_warp, chosen;
    __shared__ float owner_base, owner_target;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunk = (((vocab + 31) / 32) + 31) & ~31;              // ids per warp, a multiple of 32
    const int begin = min(vocab, warp * chunk), end = min(vocab, begin + chunk);
    auto weight_of = [&](float x) { return ordered_key(x) >= floor_key ? expf((x - mx) * inv_t) : 0.f; };

    float local = 0.f;
    for_each_logit(row, begin, end, lane, 32, [&](int, float x) { local += weight_of(x); });
    local = warp_sum(local);
    if (lane == 0) warp_total[warp] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int w = 0; w < 32; ++w) total += warp_total[w];
        const float target = uniform * total;
        float running = 0.f;
        int owner = -1;
        for (int w = 0; w < 32; ++w) {
            if (running + warp_total[w] > target) { owner = w; break; }
            running += warp_total[w];
        }
        if (owner < 0) {                                   // rounding left the target at the total: the last warp with weight
            running = 0.f;
            for (int w = 0; w < 32; ++w)
                if (warp_total[w] > 0.f) owner = w;
            for (int w = 0; w < owner; ++w) running += warp_total[w];
        }
        owner_warp = owner; owner_base = running; owner_target = target;
        chosen = 0;
    }
    __syncthreads();
    if (warp == owner_warp) {
        float running = owner_base;
        const float target = owner_target;
        int pick = -1, last_kept = -1;
        for (int i8 = begin; i8 < end && pick < 0; i8 += 256) {
            float x[8];                                    // eight groups of 32 neighbours, their loads in flight together
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = i8 + 32 * j + lane < end ? row[i8 + 32 * j + lane] : 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i0 = i8 + 32 * j;
                if (pick >= 0 || i0 >= end) break;
                const float w = i0 + lane < end ? weight_of(x[j]) : 0.f;
                float prefix = w;                          // inclusive prefix sum over the lanes
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const float other = __shfl_up_sync(0xffffffffu, prefix, off);
                    if (lane >= off) prefix += other;
                }
                const unsigned int kept = __ballot_sync(0xffffffffu, w > 0.f);
                const unsigned int beyond = __ballot_sync(0xffffffffu, w > 0.f && running + prefix > target);
                if (beyond) pick = i0 + __ffs(beyond) - 1;
                if (kept) last_kept = i0 + 31 - __clz(kept);
                running += __shfl_sync(0xffffffffu, prefix, 31);
            }
        }
        // rounding can leave the target beyond the last kept token of these ids: the choice is a kept token
        if (lane == 0) chosen = pick >= 0 ? pick : max(last_kept, 0);
    }
    __syncthreads();
    return chosen;
}

__global__ void __launch_bounds__(SMP_THREADS) sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                                                            const float* __restrict__ uniform, int* __restrict__ out, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int token = sample_row(row, 1.f / temperature[blockIdx.x], uniform[blockIdx.x], vocab, row_max(row, vocab), 0u);
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

// ----------------------------------------------------------------------------- the most likely tokens only
// top_k: the k largest logits are kept (and every logit that ties with the k-th).  top_p: of what top_k keeps, the
// most likely tokens whose probabilities, renormalised over what top_k keeps, first sum to top_p (and every token that
// ties with the last of them).  Both are a threshold on the logit, found without sorting: the keys of the logits are
// cut into four digits of eight bits, and for one digit after the other a histogram over the tokens that share the
// digits found so far tells in which bin the running count (or mass), summed from the largest key down, reaches
// the wanted one.  Masses are integers, the weight exp((logit - max) / T) in units of 2^-30, so that the sums do
// not depend on the order in which the threads add them: the same row gives the same threshold every time.  (A
// token less likely than 2^-31 of the most likely one has mass 0 and is never what top_p stops at.)
// A mass bin is two 32-bit words: the low word takes the additions, and the thread whose addition wraps it adds one to
// the high word, so that a bin costs one native shared-memory atomic per token.
__device__ __forceinline__ void mass_add(unsigned int* lo, unsigned int* hi, unsigned int units) {
    const unsigned int before = atomicAdd(lo, units);
    if (before > 0xffffffffu - units) atomicAdd(hi, 1u);
}
__device__ __forceinline__ unsigned long long mass_of(unsigned int lo, unsigned int hi) { return ((unsigned long long)hi << 32) | lo; }

constexpr int TOP_BINS = 256;
constexpr int TOP_WARPS = SMP_THREADS / 32;
constexpr size_t TOP_SMEM = (size_t)TOP_WARPS * TOP_BINS * 3 * sizeof(unsigned int);      // per warp and bin: mass low, mass high, count

struct TopState {
    unsigned int key;              // the threshold found: tokens whose key is at least this are kept
    unsigned long long mass;       // their mass
};

// `by_mass`: stop where the mass reaches `target`, else where the count does.  Only keys >= floor_key take part.
__device__ TopState top_threshold(const float* __restrict__ row, int vocab, float mx, float inv_t, unsigned int floor_key,
                                  bool by_mass, unsigned long long target, unsigned int* warp_bins) {
    __shared__ unsigned long long bin_mass[TOP_BINS];
    __shared__ unsigned int bin_count[TOP_BINS];
    __shared__ unsigned int digit_found;
    __shared__ unsigned long long above_mass, above_count;       // of the keys above the digits found so far
    const int warp = threadIdx.x >> 5;
    unsigned int* my_bins = warp_bins + warp * 3 * TOP_BINS;       // [mass low | mass high | count][bin]
    if (threadIdx.x == 0) { above_mass = 0; above_count = 0; }
    unsigned int prefix = 0;
    for (int level = 0; level < 4; ++level) {
        const int shift = 24 - 8 * level;
        for (int i = threadIdx.x; i < TOP_WARPS * 3 * TOP_BINS; i += blockDim.x) warp_bins[i] = 0;
        __syncthreads();
        for_each_logit(row, 0, vocab, threadIdx.x, blockDim.x, [&](int, float x) {
            const unsigned int key = ordered_key(x);
            if (key < floor_key || (level > 0 && (key >> (shift + 8)) != (prefix >> (shift + 8)))) return;
            const unsigned int digit = (key >> shift) & 255u;
            const float w = expf((x - mx) * inv_t);
            atomicAdd(&my_bins[2 * TOP_BINS + digit], 1u);
            mass_add(&my_bins[digit], &my_bins[TOP_BINS + digit], (unsigned int)(w * 1073741824.f + 0.5f));
        });
        __syncthreads();
        if (threadIdx.x < TOP_BINS) {
            unsigned long long m = 0;
            unsigned int c = 0;
            for (int w = 0; w < TOP_WARPS; ++w) {
                const unsigned int* bins = warp_bins + w * 3 * TOP_BINS;
                m += mass_of(bins[threadIdx.x], bins[TOP_BINS + threadIdx.x]);
                c += bins[2 * TOP_BINS + threadIdx.x];
            }
            bin_mass[threadIdx.x] = m;
            bin_count[threadIdx.x] = c;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long m = above_mass, c = above_count;
            int digit = 0;
            for (int d = TOP_BINS - 1; d >= 0; --d) {
                const unsigned long long m_with = m + bin_mass[d], c_with = c + bin_count[d];
                if ((by_mass ? m_with : c_with) >= target || d == 0) {
                    digit = d;
                    if (level == 3) { m = m_with; c = c_with; }      // the last digit: the threshold's own tokens are kept
                    break;
                }
                m = m_with; c = c_with;
            }
            above_mass = m; above_count = c;
            digit_found = (unsigned int)digit;
        }
        __syncthreads();
        prefix |= digit_found << shift;
    }
    TopState state;
    state.key = prefix > floor_key ? prefix : floor_key;
    state.mass = above_mass;
    __syncthreads();
    return state;
}

// The quick way to the same thresholds, for rows whose tokens are not all alike.  One pass sorts every token into one
// of 256 bins by how far it lies below the largest, an eighth of a nat of log-probability per bin (the last bin
// takes everything 32 nats down and further).  The running count or mass over the bins tells in which bin the
// threshold lies; a second pass copies that bin's tokens (key and mass) into shared memory, and the four digits of the
// key are walked over that short list instead of over the row.  A bin with more tokens than the list holds (a row of
// nearly equal logits) sends the row the long way above; both ways find the same key.
constexpr int TOP_LIST = 8192;
constexpr size_t TOP_SMEM_ALL = TOP_SMEM + (size_t)TOP_LIST * 2 * sizeof(unsigned int);

__device__ __forceinline__ int depth_bin(float depth) { return min(TOP_BINS - 1, (int)(depth * 8.f)); }
__device__ __forceinline__ unsigned long long mass_units(float weight) { return (unsigned long long)(weight * 1073741824.f + 0.5f); }

__device__ void depth_histogram(const float* __restrict__ row, int vocab, float mx, float inv_t, unsigned int* warp_bins,
                                unsigned long long* bin_mass, unsigned int* bin_count) {
    unsigned int* my_bins = warp_bins + (threadIdx.x >> 5) * 3 * TOP_BINS;
    for (int i = threadIdx.x; i < TOP_WARPS * 3 * TOP_BINS; i += blockDim.x) warp_bins[i] = 0;
    __syncthreads();
    for_each_logit(row, 0, vocab, threadIdx.x, blockDim.x, [&](int, float x) {
        const float depth = (mx - x) * inv_t;
        const int bin = depth_bin(depth);
        atomicAdd(&my_bins[2 * TOP_BINS + bin], 1u);
        mass_add(&my_bins[bin], &my_bins[TOP_BINS + bin], (unsigned int)mass_units(expf(-depth)));
    });
    __syncthreads();
    if (threadIdx.x < TOP_BINS) {
        unsigned long long m = 0;
        unsigned int c = 0;
        for (int w = 0; w < TOP_WARPS; ++w) {
            const unsigned int* bins = warp_bins + w * 3 * TOP_BINS;
            m += mass_of(bins[threadIdx.x], bins[TOP_BINS + threadIdx.x]);
            c += bins[2 * TOP_BINS + threadIdx.x];
        }
        bin_mass[threadIdx.x] = m;
        bin_count[threadIdx.x] = c;
    }
    __syncthreads();
}

// The tokens of one bin whose key is at least floor_key, into the list.  False if they do not fit.
__device__ bool gather_bin(const float* __restrict__ row, int vocab, float mx, float inv_t, int bin, unsigned int floor_key,
                           unsigned int* list_key, unsigned int* list_mass, unsigned int* count) {
    __shared__ unsigned int n;
    if (threadIdx.x == 0) n = 0;
    __syncthreads();
    for_each_logit(row, 0, vocab, threadIdx.x, blockDim.x, [&](int, float x) {
        const float depth = (mx - x) * inv_t;
        const unsigned int key = ordered_key(x);
        if (key < floor_key || depth_bin(depth) != bin) return;
        const unsigned int slot = atomicAdd(&n, 1u);
        if (slot < (unsigned int)TOP_LIST) { list_key[slot] = key; list_mass[slot] = (unsigned int)mass_units(expf(-depth)); }
    });
    __syncthreads();
    *count = n;
    const bool fits = n <= (unsigned int)TOP_LIST;
    __syncthreads();
    return fits;
}

// top_threshold over a list in shared memory.
__device__ TopState list_threshold(const unsigned int* list_key, const unsigned int* list_mass, int n, unsigned int floor_key,
                                   bool by_mass, unsigned long long target) {
    __shared__ unsigned int digit_lo[TOP_BINS], digit_hi[TOP_BINS], digit_count[TOP_BINS];
    __shared__ unsigned int digit_found;
    __shared__ unsigned long long above_mass, above_count;
    if (threadIdx.x == 0) { above_mass = 0; above_count = 0; }
    unsigned int prefix = 0;
    for (int level = 0; level < 4; ++level) {
        const int shift = 24 - 8 * level;
        if (threadIdx.x < TOP_BINS) { digit_lo[threadIdx.x] = 0; digit_hi[threadIdx.x] = 0; digit_count[threadIdx.x] = 0; }
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const unsigned int key = list_key[i];
            if (key < floor_key || (level > 0 && (key >> (shift + 8)) != (prefix >> (shift + 8)))) continue;
            const unsigned int digit = (key >> shift) & 255u;
            atomicAdd(&digit_count[digit], 1u);
            mass_add(&digit_lo[digit], &digit_hi[digit], list_mass[i]);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long m = above_mass, c = above_count;
            int digit = 0;
            for (int d = TOP_BINS - 1; d >= 0; --d) {
                const unsigned long long m_with = m + mass_of(digit_lo[d], digit_hi[d]), c_with = c + digit_count[d];
                if ((by_mass ? m_with : c_with) >= target || d == 0) {
                    digit = d;
                    if (level == 3) { m = m_with; c = c_with; }
                    break;
                }
                m = m_with; c = c_with;
            }
            above_mass = m; above_count = c;
            digit_found = (unsigned int)digit;
        }
        __syncthreads();
        prefix |= digit_found << shift;
    }
    TopState state;
    state.key = prefix > floor_key ? prefix : floor_key;
    state.mass = above_mass;
    __syncthreads();
    return state;
}

template <bool TOP>
__global__ void __launch_bounds__(SMP_THREADS) sample_keyed_kernel(const float* __restrict__ logits, float inv_t, unsigned long long seed,
                                                                  const int* __restrict__ keys, int* __restrict__ out, int vocab,
                                                                  int top_k, float top_p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char top_smem[];
    unsigned long long state = mix64(seed);
    state = mix64(state ^ (unsigned long long)(long long)keys[2 * blockIdx.x]);
    state = mix64(state ^ (unsigned long long)(long long)keys[2 * blockIdx.x + 1]);
    const float uniform = (float)(state >> 40) * (1.f / 16777216.f);
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const float mx = row_max(row, vocab);
    unsigned int floor_key = 0;
    if (TOP) {
        __shared__ unsigned long long bin_mass[TOP_BINS];
        __shared__ unsigned int bin_count[TOP_BINS];
        unsigned int* warp_bins = reinterpret_cast<unsigned int*>(top_smem);
        unsigned int* list_key = warp_bins + TOP_WARPS * 3 * TOP_BINS;
        unsigned int* list_mass = list_key + TOP_LIST;
        const bool cut_k = top_k > 0 && top_k < vocab;
        depth_histogram(row, vocab, mx, inv_t, warp_bins, bin_mass, bin_count);
        // the first bin, from the likeliest down, in which the running count (or mass) reaches the target; every thread
        // walks the bins itself
        auto find_bin = [&](bool by_mass, unsigned long long target, int last, int& bin, unsigned long long& m_above,
                            unsigned long long& c_above) {
            unsigned long long m = 0, c = 0;
            for (int b = 0; b <= last; ++b) {
                const unsigned long long m_with = m + bin_mass[b], c_with = c + bin_count[b];
                if ((by_mass ? m_with : c_with) >= target) { bin = b; m_above = m; c_above = c; return true; }
                m = m_with; c = c_with;
            }
            m_above = m; c_above = c;
            return false;
        };
        bool long_way = false;                           // a bin did not fit the list: thresholds over the whole row
        int bin_k = TOP_BINS;
        unsigned int n_k = 0;
        unsigned long long kept_mass = 0, m_above_k = 0, c_above_k = 0;
        if (cut_k) {
            find_bin(false, (unsigned long long)top_k, TOP_BINS - 1, bin_k, m_above_k, c_above_k);   // the row has more than top_k tokens
            if (gather_bin(row, vocab, mx, inv_t, bin_k, 0u, list_key, list_mass, &n_k)) {
                const TopState kept = list_threshold(list_key, list_mass, (int)n_k, 0u, false, (unsigned long long)top_k - c_above_k);
                floor_key = kept.key;
                kept_mass = m_above_k + kept.mass;
            } else {
                const TopState kept = top_threshold(row, vocab, mx, inv_t, 0u, false, (unsigned long long)top_k, warp_bins);
                floor_key = kept.key;
                kept_mass = kept.mass;
                long_way = true;
            }
        } else {
            unsigned long long c_all;
            find_bin(true, ~0ull, TOP_BINS - 1, bin_k, kept_mass, c_all);                            // reaches nothing: the row's mass
            bin_k = TOP_BINS;
        }
        if (top_p < 1.f) {
            unsigned long long want = (unsigned long long)((double)top_p * (double)kept_mass);
            if (want == 0) want = 1;
            int bin_p = 0;
            unsigned long long m_above_p = 0, c_above_p = 0;
            if (long_way) {
                floor_key = top_threshold(row, vocab, mx, inv_t, floor_key, true, want, warp_bins).key;
            } else if (find_bin(true, want, min(bin_k, TOP_BINS) - 1, bin_p, m_above_p, c_above_p)) {
                // reached in a bin before the one top_k stops in (all of whose tokens top_k keeps)
                unsigned int n_p = 0;
                if (gather_bin(row, vocab, mx, inv_t, bin_p, floor_key, list_key, list_mass, &n_p))
                    floor_key = list_threshold(list_key, list_mass, (int)n_p, floor_key, true, want - m_above_p).key;
                else
                    floor_key = top_threshold(row, vocab, mx, inv_t, floor_key, true, want, warp_bins).key;
            } else if (cut_k) {
                // reached among the tokens that top_k keeps of its last bin: the list still holds that bin
                floor_key = list_threshold(list_key, list_mass, (int)n_k, floor_key, true, want - m_above_k).key;
            }                                            // else: rounding put the target at the row's whole mass: every token stays
        }
    }
    const int token = sample_row(row, inv_t, uniform, vocab, mx, floor_key);
    if (threadIdx.x == 0) out[blockIdx.x] = token;
}

// top_k <= 0 and top_p >= 1 keep every token.
extern "C" int qt_sample_keyed(const float* logits, float temperature, long long seed, const int* keys, int* out, int rows, int vocab,
                               int top_k, float top_p, void* stream) {
    QT_REQUIRE(rows >= 0 && vocab > 0, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
    QT_REQUIRE(temperature > 0.f, "sample: temperature must be positive (greedy choice is qt_argmax)");
    QT_REQUIRE(top_p > 0.f, "sample: top_p=%g must be positive", (double)top_p);
    if (rows == 0) return QT_OK;
    const bool top = (top_k > 0 && top_k < vocab) || top_p < 1.f;
    if (top) {
        static bool configured = false;
        if (!configured) {
            cudaError_t err = cudaFuncSetAttribute(sample_keyed_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TOP_SMEM_ALL);
            if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "sample: cannot raise shared memory: %s", cudaGetErrorString(err));
            configured = true;
        }
        launch_kernel(sample_keyed_kernel<true>, dim3(rows), dim3(SMP_THREADS), TOP_SMEM_ALL, (cudaStream_t)stream, logits, 1.f / temperature,
                      (unsigned long long)seed, keys, out, vocab, top_k, top_p);
    } else {
        launch_kernel(sample_keyed_kernel<false>, dim3(rows), dim3(SMP_THREADS), 0, (cudaStream_t)stream, logits, 1.f / temperature,
                      (unsigned long long)seed, keys, out, vocab, 0, 1.f);
    }
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
