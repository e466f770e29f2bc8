// Token selection on the device: greedy argmax and the sampled path
// (repetition penalty, temperature, min-p, top-p, categorical draw).
//
// Order of operations and meanings of the options are the reference host
// sampler's (src/sampler.rs:34-135).  One block works on one row of logits.
// Sorting is replaced by selection: "the smallest prefix of the descending
// order whose probability reaches a target" is found by a radix descent over
// the float bit patterns of the probabilities with integer (order-free,
// reproducible) mass histograms; ties at the cut are resolved by index, as a
// stable sort would.  The same routine finds the top-p cut and, with the
// target u * kept mass, the drawn token.
#include "common.cuh"
#include "ptx.cuh"

namespace mdma {

constexpr int kSampleThreads = 1024;
constexpr int kWarpHistBytes = (kSampleThreads / 32) * 256 * 3 * 4;     // a histogram of 256 digits (three limbs) per warp

struct ArgMax { float v; int i; };
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    // larger value wins; of equal values the lower index
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}
__device__ __forceinline__ ArgMax block_argmax(ArgMax a, ArgMax* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b{__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
        a = better(a, b);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = a;
    __syncthreads();
    ArgMax r = scratch[0];
    for (int w = 1; w < (blockDim.x + 31) / 32; ++w) r = better(r, scratch[w]);
    return r;
}

// tokens[r] = argmax(logits[r,:]); flags[r] = 1 if a logit of the row is not finite.
// Two stages so that a handful of rows still uses the whole device: each block
// of stage one scans a chunk of a row (four independent loads in flight per
// thread) and leaves its best (value, index) and flag; stage two reduces the
// chunks of a row.
constexpr int kArgmaxChunk = 4096;

__global__ void __launch_bounds__(256)
argmax_chunks_kernel(const float* __restrict__ logits, int vocab, int chunks, float* __restrict__ part_v,
                     int* __restrict__ part_i, int* __restrict__ part_bad) {
    chain_release();
    chain_wait();
    __shared__ ArgMax scratch[32];
    __shared__ int bad;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();
    const int r = blockIdx.y, c = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    const int lo = c * kArgmaxChunk, hi = min(vocab, lo + kArgmaxChunk);
    ArgMax a{-INFINITY, 0x7fffffff};
    bool nonfinite = false;
    for (int i = lo + threadIdx.x; i < hi; i += 4 * blockDim.x) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { const int e = i + j * blockDim.x; v[j] = e < hi ? row[e] : -INFINITY; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = i + j * blockDim.x;
            if (e < hi) { if (!isfinite(v[j])) nonfinite = true; a = better(a, ArgMax{v[j], e}); }
        }
    }
    if (nonfinite) bad = 1;
    a = block_argmax(a, scratch);
    if (threadIdx.x == 0) {
        part_v[(size_t)r * chunks + c] = a.v;
        part_i[(size_t)r * chunks + c] = a.i;
        part_bad[(size_t)r * chunks + c] = bad;
    }
}

__global__ void __launch_bounds__(128)
argmax_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                    const int* __restrict__ part_bad, int chunks, int* __restrict__ tokens, int* __restrict__ flags) {
    chain_release();
    chain_wait();
    __shared__ ArgMax scratch[32];
    __shared__ int bad;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();
    const int r = blockIdx.x;
    ArgMax a{-INFINITY, 0x7fffffff};
    bool any_bad = false;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        a = better(a, ArgMax{part_v[(size_t)r * chunks + c], part_i[(size_t)r * chunks + c]});
        if (part_bad[(size_t)r * chunks + c]) any_bad = true;
    }
    if (any_bad) bad = 1;
    a = block_argmax(a, scratch);
    if (threadIdx.x == 0) {
        tokens[r] = a.i == 0x7fffffff ? 0 : a.i;
        if (flags) flags[r] = bad;
    }
}

// ---- sampled path -----------------------------------------------------

// Mass is summed in fixed point so that the sum does not depend on the order
// in which threads add: 2^40 units per unit of probability.
constexpr float kMassScale = 1099511627776.0f;   // 2^40
__device__ __forceinline__ unsigned long long mass_of(float p) { return (unsigned long long)(p * kMassScale); }

// A pass over n floats of a row by the whole block: 16-byte loads, four in flight per thread, when the
// row allows it (a block alone on a row is bound by load latency, not bandwidth).  f(index, value).
template <typename F>
__device__ __forceinline__ void for_each(const float* __restrict__ v, int n, F f) {
    if ((reinterpret_cast<uintptr_t>(v) & 15) == 0) {
        const int n4 = n >> 2;
        const float4* v4 = reinterpret_cast<const float4*>(v);
        int i = threadIdx.x;
        for (; i + 3 * (int)blockDim.x < n4; i += 4 * blockDim.x) {
            const float4 a = v4[i], b = v4[i + blockDim.x], c = v4[i + 2 * blockDim.x], d = v4[i + 3 * blockDim.x];
            const int i0 = 4 * i, i1 = 4 * (i + blockDim.x), i2 = 4 * (i + 2 * blockDim.x), i3 = 4 * (i + 3 * blockDim.x);
            f(i0, a.x); f(i0 + 1, a.y); f(i0 + 2, a.z); f(i0 + 3, a.w);
            f(i1, b.x); f(i1 + 1, b.y); f(i1 + 2, b.z); f(i1 + 3, b.w);
            f(i2, c.x); f(i2 + 1, c.y); f(i2 + 2, c.z); f(i2 + 3, c.w);
            f(i3, d.x); f(i3 + 1, d.y); f(i3 + 2, d.z); f(i3 + 3, d.w);
        }
        for (; i < n4; i += blockDim.x) {
            const float4 a = v4[i];
            f(4 * i, a.x); f(4 * i + 1, a.y); f(4 * i + 2, a.z); f(4 * i + 3, a.w);
        }
        for (int j = 4 * n4 + threadIdx.x; j < n; j += blockDim.x) f(j, v[j]);
    } else {
        for (int j = threadIdx.x; j < n; j += blockDim.x) f(j, v[j]);
    }
}

// A histogram of masses over the 256 digits of a pass, one per warp, kept as three 32-bit limbs per
// digit (14 + 14 + the rest of a mass) so that it takes the native 32-bit shared-memory add: a 64-bit
// add that many threads aim at one word costs about 75 cycles each.  A warp adds at most 4096 masses of
// at most 2^47, so no limb overflows.
constexpr int kLimbWords = 256 * 3;
__device__ __forceinline__ void limb_add(unsigned* warp_hist, int digit, unsigned long long mass) {
    atomicAdd(&warp_hist[digit * 3], (unsigned)(mass & 0x3FFFull));
    atomicAdd(&warp_hist[digit * 3 + 1], (unsigned)((mass >> 14) & 0x3FFFull));
    atomicAdd(&warp_hist[digit * 3 + 2], (unsigned)(mass >> 28));
}
__device__ __forceinline__ unsigned long long limb_value(const unsigned* warp_hist, int digit) {
    return (unsigned long long)warp_hist[digit * 3] + ((unsigned long long)warp_hist[digit * 3 + 1] << 14) +
           ((unsigned long long)warp_hist[digit * 3 + 2] << 28);
}

// A thread's own two digits of a pass: most of a thread's elements share one or two digits, so they are
// summed in registers and reach the warp's histogram at the end of the pass; an element with a third
// digit goes there at once.
struct DigitPair {
    int d0 = -1, d1 = -1;
    unsigned long long m0 = 0ull, m1 = 0ull;
    __device__ __forceinline__ void add(unsigned* warp_hist, int digit, unsigned long long mass) {
        if (digit == d0) m0 += mass;
        else if (digit == d1) m1 += mass;
        else if (d0 < 0) { d0 = digit; m0 = mass; }
        else if (d1 < 0) { d1 = digit; m1 = mass; }
        else limb_add(warp_hist, digit, mass);
    }
    __device__ __forceinline__ void flush(unsigned* warp_hist) {
        if (d0 >= 0) limb_add(warp_hist, d0, m0);
        if (d1 >= 0) limb_add(warp_hist, d1, m1);
    }
};

// The sum of a 64-bit value over the block (order-free), through `slot`.
__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* slot) {
    const unsigned lo = __reduce_add_sync(0xffffffffu, (unsigned)(v & 0xFFFFFull));
    const unsigned mid = __reduce_add_sync(0xffffffffu, (unsigned)((v >> 20) & 0xFFFFFull));
    const unsigned hi = __reduce_add_sync(0xffffffffu, (unsigned)(v >> 40));
    if (threadIdx.x == 0) *slot = 0ull;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) atomicAdd(slot, ((unsigned long long)hi << 40) + ((unsigned long long)mid << 20) + lo);
    __syncthreads();
    const unsigned long long total = *slot;
    __syncthreads();
    return total;
}

// Given the masses of the 256 digits of a pass (`bins`) and the mass `above` them, the first digit from
// the top at which the running mass reaches `target`, and the mass above that digit.  If the target lies
// beyond the whole mass (rounding) it settles on the lowest populated digit.  Warp 0 computes, everyone
// gets the result; ends with a block barrier.
__device__ __forceinline__ void pick_digit(const unsigned long long* bins, unsigned long long above,
                                           unsigned long long target, int* misc, unsigned long long* out_above,
                                           int& digit, unsigned long long& new_above) {
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        unsigned long long mine = 0ull;
        int lowest = 256;
#pragma unroll
        for (int b = 7; b >= 0; --b) {
            const unsigned long long m = bins[lane * 8 + b];
            mine += m;
            if (m != 0ull) lowest = lane * 8 + b;
        }
        // mass of the lanes above this one
        unsigned long long higher = 0ull, all = 0ull;
        for (int l = 0; l < 32; ++l) {
            const unsigned long long m = __shfl_sync(0xffffffffu, mine, l);
            if (l > lane) higher += m;
            all += m;
        }
        unsigned long long run = above + higher;
        int found = -1;
        unsigned long long run_at = 0ull;
#pragma unroll
        for (int b = 7; b >= 0; --b) {
            const unsigned long long m = bins[lane * 8 + b];
            if (m == 0ull || found >= 0) continue;
            if (run + m >= target) { found = lane * 8 + b; run_at = run; }
            else run += m;
        }
        const unsigned who = __ballot_sync(0xffffffffu, found >= 0);
        int low_all = lowest;
        for (int o = 16; o > 0; o >>= 1) low_all = min(low_all, __shfl_xor_sync(0xffffffffu, low_all, o));
        if (who != 0u) {
            const int top = 31 - __clz(who);
            if (lane == top) { misc[0] = found; *out_above = run_at; }
        } else if (lane == 0) {
            const int d = low_all < 256 ? low_all : 0;
            misc[0] = d;
            *out_above = above + all - bins[d];
        }
    }
    __syncthreads();
    digit = misc[0];
    new_above = *out_above;
    __syncthreads();
}

// What a row's draw depends on besides its logits.  The uniform number is either given (`uniforms`) or
// made here from (seed, request, step) with the generator of the host side (three rounds of splitmix64,
// 24 bits).  The history is a ring of `history_stride` recent token ids per row with the count of
// tokens ever added; the repetition penalty looks at the last `penalty_window` of them (the order does
// not matter: a token is divided or multiplied once per occurrence).  With `advance` the kernel
// appends the token it selected to the ring and moves the row's step counter on, so that a decode loop
// replayed as a graph needs nothing from the host between steps.
// `dev_params`, when given, overrides the options passed by value with eight words read from device
// memory: temperature, top_p, min_p, penalty (floats), penalty window (int), one unused word, the seed's
// low and high halves.  A decode loop captured in a graph then serves every request's options and seed:
// the host rewrites the words between batches and replays the same graph.
struct SampleState {
    int* history; int* history_len; int history_stride;
    const float* uniforms;
    const int* requests; int* steps; unsigned long long seed;
    int advance;
    const unsigned* dev_params;
};
__device__ __forceinline__ void load_device_params(const SampleState& st, float& temperature, float& top_p,
                                                   float& min_p, float& penalty, int& penalty_window) {
    if (st.dev_params == nullptr) return;
    temperature = __uint_as_float(st.dev_params[0]);
    top_p = __uint_as_float(st.dev_params[1]);
    min_p = __uint_as_float(st.dev_params[2]);
    penalty = __uint_as_float(st.dev_params[3]);
    penalty_window = (int)st.dev_params[4];
}

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float row_uniform(const SampleState& st, int r) {
    if (st.uniforms != nullptr) return st.uniforms[r];
    const unsigned long long seed = st.dev_params ? (((unsigned long long)st.dev_params[7] << 32) | st.dev_params[6]) : st.seed;
    const unsigned long long z = mix64(mix64(mix64(seed) ^ (unsigned long long)st.requests[r]) ^ (unsigned long long)st.steps[r]);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}
// One thread: the row's result, and what the next step of the row starts from.
__device__ __forceinline__ void finish_row(const SampleState& st, int r, int token, int flag, int* tokens, int* flags) {
    tokens[r] = token;
    if (flags) flags[r] = flag;
    if (st.advance) {
        if (st.steps) st.steps[r] += 1;
        if (st.history) {
            const int c = st.history_len[r];
            st.history[(size_t)r * st.history_stride + (c % st.history_stride)] = token;
            st.history_len[r] = c + 1;
        }
    }
}

// ---- few candidates: sort them ------------------------------------------------------
// With the usual min-p a handful of tokens survive.  Up to 1024 candidates are sorted in shared memory
// (descending probability, ties by ascending token id: one 64-bit key each), their integer masses are
// summed in that order, and the top-p cut and the draw are read off the running sums.  The result is
// what the radix descent below gives.
constexpr int kSmallMax = 1024;

__device__ __forceinline__ unsigned long long small_key(float p, int id) {
    return ((unsigned long long)__float_as_uint(p) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)id);
}

// keys[kSmallMax] (zeros beyond n), cum[kSmallMax]: shared memory; blockDim.x == kSmallMax.
__device__ int small_select(unsigned long long* keys, unsigned long long* cum, int n, float top_p, float u,
                            int fallback_id, int* misc, unsigned long long* warp_totals /*32*/) {
    const int t = threadIdx.x;
    __syncthreads();
    for (int k = 2; k <= kSmallMax; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            const int partner = t ^ j;
            if (partner > t) {
                const unsigned long long a = keys[t], b = keys[partner];
                const bool descending = (t & k) == 0;
                if (descending ? a < b : a > b) { keys[t] = b; keys[partner] = a; }
            }
            __syncthreads();
        }
    }
    // running sums of the masses, in sorted order
    const unsigned long long key = keys[t];
    unsigned long long v = t < n ? mass_of(__uint_as_float((unsigned)(key >> 32))) : 0ull;
    const int lane = t & 31, warp = t >> 5;
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += up;
    }
    if (lane == 31) warp_totals[warp] = v;
    __syncthreads();
    unsigned long long base = 0ull;
    for (int w = 0; w < warp; ++w) base += warp_totals[w];
    v += base;
    cum[t] = v;
    if (t == 0) { misc[0] = n - 1; misc[1] = -1; }
    __syncthreads();
    // the top-p cut: the first position whose running sum reaches top_p (the last candidate if none does)
    const unsigned long long goal = top_p < 1.0f ? mass_of(top_p) : cum[n - 1];
    if (t < n && v >= goal && (t == 0 || cum[t - 1] < goal)) misc[0] = t;
    __syncthreads();
    const int cut = misc[0];
    const unsigned long long kept = cum[cut];
    unsigned long long target = (unsigned long long)((double)u * (double)kept);
    if (target < 1ull) target = 1ull;
    if (t <= cut && v >= target && (t == 0 || cum[t - 1] < target)) misc[1] = t;
    __syncthreads();
    const int drawn = misc[1] >= 0 ? misc[1] : cut;
    const int id = n > 0 ? (int)(0xFFFFFFFFu - (unsigned)(keys[drawn] & 0xFFFFFFFFull)) : fallback_id;
    __syncthreads();
    return id;
}

// Finds the element at which the running mass of the candidates, taken in descending order of
// probability (ties by ascending position), first reaches `target`.  If limit_pos >= 0, only candidates
// ranked at or before the one at limit_pos (whose bit pattern is limit_bits) take part.  Returns its
// position, bit pattern and the mass up to and including it.
struct Crossing { int pos; unsigned bits; unsigned long long mass; };

__device__ Crossing find_crossing(const float* __restrict__ probs, int n, unsigned long long target,
                                  unsigned limit_bits, int limit_pos,
                                  unsigned long long* hist /*256*/, int* misc /*8*/, int* warp_counts /*32*/,
                                  unsigned* warp_hists /*warps x 256 x 3 limbs*/) {
    auto takes_part = [&](int i, float p) -> bool {
        if (!(p > 0.f)) return false;
        if (limit_pos < 0) return true;
        const unsigned bits = __float_as_uint(p);
        return bits > limit_bits || (bits == limit_bits && i <= limit_pos);
    };
    const int warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    unsigned* my_hist = warp_hists + warp * kLimbWords;
    unsigned prefix = 0, prefix_mask = 0;
    unsigned long long above = 0;     // mass of elements with bit pattern above the current prefix range
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int b = threadIdx.x & 31; b < kLimbWords; b += 32) my_hist[b] = 0u;
        __syncwarp();
        DigitPair own;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float p = probs[i];
            const unsigned bits = __float_as_uint(p);
            if ((bits & prefix_mask) == prefix && takes_part(i, p)) own.add(my_hist, (int)((bits >> shift) & 255u), mass_of(p));
        }
        own.flush(my_hist);
        __syncthreads();
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            unsigned long long t = 0ull;
            for (int w = 0; w < n_warps; ++w) t += limb_value(warp_hists + w * kLimbWords, b);
            hist[b] = t;
        }
        __syncthreads();
        int digit;
        unsigned long long next_above;
        pick_digit(hist, above, target, misc, reinterpret_cast<unsigned long long*>(misc + 6), digit, next_above);
        above = next_above;
        prefix |= (unsigned)digit << shift;
        prefix_mask |= 255u << shift;
    }
    // All elements with bit pattern == prefix are tied; take them by ascending position.
    const float tie_p = __uint_as_float(prefix);
    const unsigned long long unit = mass_of(tie_p);
    unsigned long long need = target > above ? target - above : 1ull;
    long long kth = unit ? (long long)((need + unit - 1) / unit) : 1;   // how many tied elements are taken
    if (kth < 1) kth = 1;
    // the kth tied element by position: block-wide ordered count over chunks
    int* counter = misc + 1;     // running count of ties before the current chunk
    int* answer = misc + 2;
    int* last_index = misc + 3;      // the highest position among the ties
    if (threadIdx.x == 0) { *counter = 0; *answer = -1; *last_index = -1; }
    __syncthreads();
    int last_tie = -1;
    for (int base = 0; base < n; base += blockDim.x) {
        const int i = base + threadIdx.x;
        const float p = i < n ? probs[i] : 0.f;
        const bool tie = i < n && __float_as_uint(p) == prefix && takes_part(i, p);
        const unsigned ballot = __ballot_sync(0xffffffffu, tie);
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        if (lane == 0) warp_counts[warp] = __popc(ballot);
        __syncthreads();
        int before = *counter;
        for (int w = 0; w < warp; ++w) before += warp_counts[w];
        const int rank = before + __popc(ballot & ((1u << lane) - 1u)) + 1;   // 1-based among ties
        if (tie && rank == kth) *answer = i;
        if (tie) last_tie = i;
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
            for (int w = 0; w < (blockDim.x + 31) / 32; ++w) t += warp_counts[w];
            *counter += t;
        }
        __syncthreads();
        if (*answer >= 0) break;
    }
    // fewer ties than asked for (fixed-point rounding of the masses): take the last tied element,
    // and count only the ties that exist
    if (*answer < 0) {
        atomicMax(last_index, last_tie);
        __syncthreads();
        if (threadIdx.x == 0) *answer = *last_index;
        __syncthreads();
        kth = *counter > 0 ? *counter : 1;
    }
    Crossing c;
    c.pos = *answer;
    c.bits = prefix;
    c.mass = above + unit * (unsigned long long)kth;
    __syncthreads();
    return c;
}

// One row: adjusted logits -> probabilities -> min-p -> the surviving candidates, compacted in index
// order (probability and token id) -> top-p cut -> draw with the uniform number u[r].  With the usual
// min-p only a handful of tokens survive, and the selection passes run over those instead of the
// vocabulary.  `scratch` holds three words per vocabulary entry and row: exponentials, the candidates'
// probabilities, their token ids.
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int vocab, const SampleState st,
              float temperature, float top_p, float min_p, float penalty, int penalty_window,
              float* __restrict__ scratch, int* __restrict__ tokens, int* __restrict__ flags) {
    __shared__ float fscratch[32];
    __shared__ ArgMax ascratch[32];
    __shared__ unsigned long long hist[256];
    __shared__ __align__(8) int misc[8];
    __shared__ int warp_counts[32];
    __shared__ int bad;
    extern __shared__ __align__(16) unsigned warp_hists[];      // one histogram of 256 digits per warp
    load_device_params(st, temperature, top_p, min_p, penalty, penalty_window);
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    float* probs = scratch + (size_t)r * 3 * vocab;
    float* cand_p = probs + vocab;
    int* cand_id = reinterpret_cast<int*>(probs + 2 * (size_t)vocab);
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();

    // 1. copy, flag non-finite values, and the leader of the unadjusted row
    bool nonfinite = false;
    ArgMax a{-INFINITY, 0x7fffffff};
    for_each(row, vocab, [&](int i, float v) {
        if (!isfinite(v)) nonfinite = true;
        probs[i] = v;
        a = better(a, ArgMax{v, i});
    });
    if (nonfinite) bad = 1;
    __syncthreads();
    // 2. repetition penalty on the last `penalty_window` tokens of the history; a
    //    token that occurs several times is penalised once per occurrence, in order
    const bool penalised = penalty != 1.0f && st.history != nullptr && penalty_window > 0;
    if (penalised) {
        if (threadIdx.x == 0) {
            const int count = st.history_len[r];
            const int m = min(min(penalty_window, count), st.history_stride);
            const int* hrow = st.history + (size_t)r * st.history_stride;
            for (int e = 0; e < m; ++e) {
                const int id = hrow[(count - m + e) % st.history_stride];
                if (id >= 0 && id < vocab) {
                    const float l = probs[id];
                    probs[id] = l > 0.f ? l / penalty : l * penalty;
                }
            }
        }
        __syncthreads();
        a = ArgMax{-INFINITY, 0x7fffffff};
        for_each(probs, vocab, [&](int i, float v) { a = better(a, ArgMax{v, i}); });
    }
    // 3. greedy when temperature <= 0
    a = block_argmax(a, ascratch);
    if (temperature <= 0.f || bad) {
        if (threadIdx.x == 0) finish_row(st, r, a.i == 0x7fffffff ? 0 : a.i, bad, tokens, flags);
        return;
    }
    // 4. softmax of logits / temperature: the leader's exponential is exactly 1
    const float mx = a.v / temperature;
    float sum = 0.f;
    for_each(probs, vocab, [&](int i, float v) {
        const float e = expf(v / temperature - mx);
        probs[i] = e;
        sum += e;
    });
    sum = block_sum(sum, fscratch);
    __syncthreads();
    // 5. min-p: keep p >= p_max * min_p (p_max = 1 / sum).  Survivors are written in index order to a
    //    list of their own: every warp owns a run of the row, counts its survivors, and after one scan
    //    over the warps' counts writes them at its place (ballots give the order inside a warp).
    const float thr = min_p > 0.f ? (1.0f / sum) * min_p : 0.f;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int run_len = ((vocab + n_warps - 1) / n_warps + 31) / 32 * 32;
    const int run_lo = min(vocab, warp * run_len), run_hi = min(vocab, run_lo + run_len);
    auto survives = [&](int i, float& p) -> bool {
        p = i < run_hi ? probs[i] / sum : 0.f;
        return i < run_hi && p > 0.f && !(p < thr);
    };
    int count = 0;
    for (int i = run_lo + lane; i < run_hi + lane; i += 32) {        // whole warps: run_hi + lane keeps the lanes together
        if (i - lane >= run_hi) break;
        float p;
        count += __popc(__ballot_sync(0xffffffffu, survives(i, p)));
    }
    if (lane == 0) warp_counts[warp] = count;
    __syncthreads();
    int at = 0, n_all = 0;
    for (int w = 0; w < n_warps; ++w) { if (w < warp) at += warp_counts[w]; n_all += warp_counts[w]; }
    unsigned long long mine = 0ull;
    for (int i = run_lo + lane; i - lane < run_hi; i += 32) {
        float p;
        const bool keep = survives(i, p);
        const unsigned ballot = __ballot_sync(0xffffffffu, keep);
        if (keep) {
            const int pos = at + __popc(ballot & ((1u << lane) - 1u));
            cand_p[pos] = p; cand_id[pos] = i; mine += mass_of(p);
        }
        at += __popc(ballot);
    }
    __syncthreads();
    if (threadIdx.x == 0) misc[4] = n_all;
    __syncthreads();
    const int n_cand = misc[4];
    if (n_cand == 0) {                                      // cannot happen with finite logits; keep the leader
        if (threadIdx.x == 0) finish_row(st, r, a.i, 0, tokens, flags);
        return;
    }
    if (n_cand <= kSmallMax) {
        // few candidates: sort them (the warps' histograms are not needed: their room holds the keys)
        unsigned long long* keys = reinterpret_cast<unsigned long long*>(warp_hists);
        unsigned long long* cum = keys + kSmallMax;
        keys[threadIdx.x] = (int)threadIdx.x < n_cand ? small_key(cand_p[threadIdx.x], cand_id[threadIdx.x]) : 0ull;
        const int id = small_select(keys, cum, n_cand, top_p, row_uniform(st, r), a.i, misc, hist);
        if (threadIdx.x == 0) finish_row(st, r, id, 0, tokens, flags);
        return;
    }
    // 6. top-p: the smallest descending prefix whose mass reaches top_p
    unsigned long long kept = 0ull;
    unsigned limit_bits = 0;
    int limit_pos = -1;
    if (top_p < 1.0f) {
        const Crossing cut = find_crossing(cand_p, n_cand, mass_of(top_p), 0u, -1, hist, misc, warp_counts, warp_hists);
        kept = cut.mass;
        limit_bits = cut.bits;
        limit_pos = cut.pos;
    } else {
        kept = block_sum_u64(mine, &hist[0]);
    }
    // 7. draw: first element of the descending order whose running mass reaches u * kept
    const float u = row_uniform(st, r);
    unsigned long long target = (unsigned long long)((double)u * (double)kept);
    if (target < 1ull) target = 1ull;
    const Crossing drawn = find_crossing(cand_p, n_cand, target, limit_bits, limit_pos, hist, misc, warp_counts, warp_hists);
    if (threadIdx.x == 0) finish_row(st, r, drawn.pos >= 0 ? cand_id[drawn.pos] : a.i, 0, tokens, flags);
}

// ---- the same for a cluster of eight blocks per row ---------------------------------
// A block alone spends 60-100 us on every pass over a vocabulary of 128k (it is bound by its own
// instruction rate).  Here each block of a cluster keeps an eighth of the row in shared memory; maxima,
// sums, masses and the digit histograms of the selection are exchanged through distributed shared
// memory at cluster barriers.  Every block takes the same decisions, so the barriers match.  The
// order of every floating-point sum is fixed (threads of a block, then blocks by rank), and ties are
// taken by ascending token id as in the single-block kernel; the results are the same up to the
// rounding of the softmax denominator (a different order of addition).
constexpr int kSampleCluster = 8;

struct SampleExchange {          // one per block; the other blocks read it
    float max_v; int max_i; int bad; float sum;
    unsigned long long mass;
    int ties; int answer; int count; int pad;
    unsigned long long hist[2][256];
};

struct ClusterCrossing { int index; unsigned bits; unsigned long long mass; };

__device__ ClusterCrossing find_crossing_cluster(const float* slice, int n, int lo, unsigned long long target,
                                                 unsigned limit_bits, int limit_index, int fallback_index,
                                                 SampleExchange* xch, unsigned long long* total /*256*/, int* misc,
                                                 int* warp_counts, int& turn, unsigned* warp_hists) {
    const uint32_t xch_addr = ptx::smem_addr(xch);
    const int rank = (int)ptx::cluster_rank();
    auto takes_part = [&](int gi, float p) -> bool {
        if (!(p > 0.f)) return false;
        if (limit_index < 0) return true;
        const unsigned bits = __float_as_uint(p);
        return bits > limit_bits || (bits == limit_bits && gi <= limit_index);
    };
    const int warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    unsigned* my_hist = warp_hists + warp * kLimbWords;
    unsigned prefix = 0, prefix_mask = 0;
    unsigned long long above = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        unsigned long long* hist = xch->hist[turn & 1];
        for (int b = threadIdx.x & 31; b < kLimbWords; b += 32) my_hist[b] = 0u;
        __syncwarp();
        DigitPair own;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float p = slice[i];
            const unsigned bits = __float_as_uint(p);
            if ((bits & prefix_mask) == prefix && takes_part(lo + i, p)) own.add(my_hist, (int)((bits >> shift) & 255u), mass_of(p));
        }
        own.flush(my_hist);
        __syncthreads();
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            unsigned long long t = 0ull;
            for (int w = 0; w < n_warps; ++w) t += limb_value(warp_hists + w * kLimbWords, b);
            hist[b] = t;
        }
        ptx::cluster_sync();
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            unsigned long long t = 0ull;
            const uint32_t off = (uint32_t)(offsetof(SampleExchange, hist) + ((turn & 1) * 256 + b) * 8);
            for (int k = 0; k < kSampleCluster; ++k) t += ptx::cluster_load_u64(ptx::cluster_map(xch_addr + off, k));
            total[b] = t;
        }
        ++turn;
        __syncthreads();
        int digit;
        unsigned long long next_above;
        pick_digit(total, above, target, misc, reinterpret_cast<unsigned long long*>(misc + 6), digit, next_above);
        above = next_above;
        prefix |= (unsigned)digit << shift;
        prefix_mask |= 255u << shift;
    }
    // ties: the kth element with this bit pattern in ascending token id = blocks by rank, then position
    const float tie_p = __uint_as_float(prefix);
    const unsigned long long unit = mass_of(tie_p);
    const unsigned long long need = target > above ? target - above : 1ull;
    long long kth = unit ? (long long)((need + unit - 1) / unit) : 1;
    if (kth < 1) kth = 1;
    int mine = 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float p = slice[i];
        if (__float_as_uint(p) == prefix && takes_part(lo + i, p)) ++mine;
    }
    if (threadIdx.x == 0) { misc[1] = 0; xch->answer = -1; }
    __syncthreads();
    if (mine) atomicAdd(&misc[1], mine);
    __syncthreads();
    if (threadIdx.x == 0) xch->ties = misc[1];
    ptx::cluster_sync();
    int all_ties = 0, owner = -1;
    long long before_owner = 0;
    for (int k = 0; k < kSampleCluster; ++k)
        all_ties += (int)ptx::cluster_load_u32(ptx::cluster_map(xch_addr + (uint32_t)offsetof(SampleExchange, ties), k));
    if (all_ties > 0 && kth > all_ties) kth = all_ties;          // fewer ties than asked for (rounding): the last one
    {
        int run = 0;
        for (int k = 0; k < kSampleCluster; ++k) {
            const int t = (int)ptx::cluster_load_u32(ptx::cluster_map(xch_addr + (uint32_t)offsetof(SampleExchange, ties), k));
            if (owner < 0 && kth <= run + t) { owner = k; before_owner = run; }
            run += t;
        }
    }
    if (owner == rank) {
        // the (kth - before)-th tie of this block, by position: ordered count over chunks of the block
        const int want = (int)(kth - before_owner);
        if (threadIdx.x == 0) misc[2] = 0;
        __syncthreads();
        for (int base = 0; base < n; base += blockDim.x) {
            const int i = base + threadIdx.x;
            const float p = i < n ? slice[i] : 0.f;
            const bool tie = i < n && __float_as_uint(p) == prefix && takes_part(lo + i, p);
            const unsigned ballot = __ballot_sync(0xffffffffu, tie);
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            if (lane == 0) warp_counts[warp] = __popc(ballot);
            __syncthreads();
            int seen = misc[2];
            for (int w = 0; w < warp; ++w) seen += warp_counts[w];
            const int rank_in = seen + __popc(ballot & ((1u << lane) - 1u)) + 1;
            if (tie && rank_in == want) xch->answer = lo + i;
            __syncthreads();
            if (threadIdx.x == 0) {
                int t = 0;
                for (int w = 0; w < (blockDim.x + 31) / 32; ++w) t += warp_counts[w];
                misc[2] += t;
            }
            __syncthreads();
        }
    }
    ptx::cluster_sync();
    ClusterCrossing c;
    c.index = owner >= 0 ? (int)ptx::cluster_load_u32(ptx::cluster_map(xch_addr + (uint32_t)offsetof(SampleExchange, answer), owner))
                         : fallback_index;
    if (c.index < 0) c.index = fallback_index;
    c.bits = prefix;
    c.mass = above + unit * (unsigned long long)kth;
    ptx::cluster_sync();             // everyone has read the answer before the next use of the exchange words
    return c;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_cluster_kernel(const float* __restrict__ logits, int vocab, int per, const SampleState st,
                      float temperature, float top_p, float min_p, float penalty, int penalty_window,
                      int* __restrict__ tokens, int* __restrict__ flags) {
    extern __shared__ __align__(16) float slice[];          // `per` floats, then the warps' histograms
    unsigned* warp_hists = reinterpret_cast<unsigned*>(slice + per);
    unsigned long long* small_keys = reinterpret_cast<unsigned long long*>(warp_hists);
    __shared__ SampleExchange xch;
    __shared__ int window[64];
    __shared__ unsigned long long total[256];
    __shared__ float fscratch[32];
    __shared__ ArgMax ascratch[32];
    __shared__ __align__(8) int misc[8];
    __shared__ int warp_counts[32];
    __shared__ int bad;
    load_device_params(st, temperature, top_p, min_p, penalty, penalty_window);
    const int rank = (int)ptx::cluster_rank();
    const int r = blockIdx.y;
    const float* row = logits + (size_t)r * vocab;
    const int lo = rank * per;
    const int n = max(0, min(per, vocab - lo));
    const uint32_t xch_addr = ptx::smem_addr(&xch);
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();
    // 1. this block's part of the row -> shared memory; non-finite values
    bool nonfinite = false;
    for_each(row + lo, n, [&](int i, float v) {
        if (!isfinite(v)) nonfinite = true;
        slice[i] = v;
    });
    if (nonfinite) bad = 1;
    __syncthreads();
    // 2. repetition penalty: every block walks the window and changes the tokens it holds, in order
    if (penalty != 1.0f && st.history != nullptr && penalty_window > 0) {
        const int count = st.history_len[r];
        const int m_all = min(min(penalty_window, count), st.history_stride);
        const int* hrow = st.history + (size_t)r * st.history_stride;
        for (int base = 0; base < m_all; base += 64) {           // 64 ids at a time through shared memory
            const int m = min(64, m_all - base);
            if ((int)threadIdx.x < m) window[threadIdx.x] = hrow[(count - m_all + base + (int)threadIdx.x) % st.history_stride];
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int j = 0; j < m; ++j) {
                    const int id = window[j];
                    if (id >= lo && id < lo + n) {
                        const float l = slice[id - lo];
                        slice[id - lo] = l > 0.f ? l / penalty : l * penalty;
                    }
                }
            }
            __syncthreads();
        }
    }
    __syncthreads();
    // 3. the leader of the row
    ArgMax a{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < n; i += blockDim.x) a = better(a, ArgMax{slice[i], lo + i});
    a = block_argmax(a, ascratch);
    if (threadIdx.x == 0) { xch.max_v = a.v; xch.max_i = a.i; xch.bad = bad; }
    ptx::cluster_sync();
    // one thread reads the eight blocks' words (in rank order) and hands the result round
    if (threadIdx.x == 0) {
        ArgMax best{-INFINITY, 0x7fffffff};
        int any = 0;
        for (int k = 0; k < kSampleCluster; ++k) {
            ArgMax b;
            b.v = ptx::cluster_load_f32(ptx::cluster_map(xch_addr + (uint32_t)offsetof(SampleExchange, max_v), k));
            b.i = (int)ptx::cluster_load_u32(ptx::cluster_map(xch_addr + (uint32_t)offsetof(SampleExchange, max_i), k));
            any |= (int)ptx::cluster_load_u32(ptx::cluster_map(xch_addr + (uint32_t)offsetof(SampleExchange, bad), k));
            best = better(best, b);
        }
        ascratch[0] = best;
        misc[5] = any;
    }
    __syncthreads();
    a = ascratch[0];
    const int any_bad = misc[5];
    __syncthreads();
    if (temperature <= 0.f || any_bad) {
        if (rank == 0 && threadIdx.x == 0) finish_row(st, r, a.i == 0x7fffffff ? 0 : a.i, any_bad, tokens, flags);
        ptx::cluster_sync();          // nobody leaves while its words may still be read
        return;
    }
    // 4. softmax of logits / temperature
    const float mx = a.v / temperature;
    float sum = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float e = expf(slice[i] / temperature - mx);
        slice[i] = e;
        sum += e;
    }
    sum = block_sum(sum, fscratch);
    if (threadIdx.x == 0) xch.sum = sum;
    ptx::cluster_sync();
    if (threadIdx.x == 0) {
        float d = 0.f;
        for (int k = 0; k < kSampleCluster; ++k)
            d += ptx::cluster_load_f32(ptx::cluster_map(xch_addr + (uint32_t)offsetof(SampleExchange, sum), k));
        fscratch[0] = d;
    }
    __syncthreads();
    const float denom = fscratch[0];
    __syncthreads();
    // 5. probabilities; min-p: keep p >= p_max * min_p (p_max = 1 / sum: the leader's exponential is 1)
    const float thr = min_p > 0.f ? (1.0f / denom) * min_p : 0.f;
    unsigned long long mine = 0ull;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float p = slice[i] / denom;
        if (p < thr) p = 0.f;
        slice[i] = p;
        mine += mass_of(p);
    }
    int survivors = 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) survivors += slice[i] > 0.f ? 1 : 0;
    const unsigned long long block_mass = block_sum_u64(mine, &total[0]);
    const int block_count = (int)block_sum_u64((unsigned long long)survivors, &total[1]);
    if (threadIdx.x == 0) { xch.mass = block_mass; xch.count = block_count; }
    ptx::cluster_sync();
    if (threadIdx.x == 0) {
        int before = 0, all = 0;
        for (int k = 0; k < kSampleCluster; ++k) {
            const int c = (int)ptx::cluster_load_u32(ptx::cluster_map(xch_addr + (uint32_t)offsetof(SampleExchange, count), k));
            if (k < rank) before += c;
            all += c;
        }
        misc[3] = before; misc[4] = all;
    }
    __syncthreads();
    const int cand_before = misc[3], cand_all = misc[4];
    __syncthreads();
    if (cand_all <= kSmallMax) {
        // few candidates: every block sends its own to the first block, which sorts them
        // (their order of arrival does not matter); the keys live where the warps' histograms would
        const uint32_t keys0 = ptx::cluster_map(ptx::smem_addr(small_keys), 0);
        if (rank == 0) for (int i = threadIdx.x; i < 2 * kSmallMax; i += blockDim.x) small_keys[i] = 0ull;
        if (threadIdx.x == 0) misc[2] = 0;
        ptx::cluster_sync();                         // the first block's list is cleared
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float p = slice[i];
            if (p > 0.f) {
                const int at = cand_before + atomicAdd(&misc[2], 1);
                ptx::cluster_store_u64(keys0 + (uint32_t)at * 8u, small_key(p, lo + i));
            }
        }
        ptx::cluster_sync();                         // the list is complete
        if (rank == 0) {
            const int id = small_select(small_keys, small_keys + kSmallMax, cand_all, top_p, row_uniform(st, r), a.i, misc, total);
            if (threadIdx.x == 0) finish_row(st, r, id, 0, tokens, flags);
        }
        return;
    }
    if (threadIdx.x == 0) {
        unsigned long long m = 0ull;
        for (int k = 0; k < kSampleCluster; ++k)
            m += ptx::cluster_load_u64(ptx::cluster_map(xch_addr + (uint32_t)offsetof(SampleExchange, mass), k));
        total[0] = m;
    }
    __syncthreads();
    unsigned long long kept = total[0];
    __syncthreads();
    // 6. top-p: the smallest descending prefix whose mass reaches top_p
    int turn = 0;
    unsigned limit_bits = 0;
    int limit_index = -1;
    if (top_p < 1.0f) {
        const ClusterCrossing cut = find_crossing_cluster(slice, n, lo, mass_of(top_p), 0u, -1, a.i, &xch, total, misc,
                                                          warp_counts, turn, warp_hists);
        kept = cut.mass;
        limit_bits = cut.bits;
        limit_index = cut.index;
    }
    // 7. draw: first element of the descending order whose running mass reaches u * kept
    const float u = row_uniform(st, r);
    unsigned long long target = (unsigned long long)((double)u * (double)kept);
    if (target < 1ull) target = 1ull;
    const ClusterCrossing drawn = find_crossing_cluster(slice, n, lo, target, limit_bits, limit_index, a.i, &xch, total,
                                                        misc, warp_counts, turn, warp_hists);
    if (rank == 0 && threadIdx.x == 0) finish_row(st, r, drawn.index >= 0 ? drawn.index : a.i, 0, tokens, flags);
}

}  // namespace mdma

using namespace mdma;

// Floats (4-byte words) of scratch mdma_argmax needs for these sizes.
extern "C" long mdma_argmax_scratch(int n_rows, int vocab) {
    return 3l * n_rows * ((vocab + kArgmaxChunk - 1) / kArgmaxChunk);
}

extern "C" int mdma_argmax(const float* logits, int n_rows, int vocab, int* tokens, int* flags,
                           float* scratch, long scratch_words, cudaStream_t stream) {
    MDMA_REQUIRE(vocab > 0 && n_rows >= 0, "argmax: bad sizes");
    if (n_rows == 0) return 0;
    const int chunks = (vocab + kArgmaxChunk - 1) / kArgmaxChunk;
    MDMA_REQUIRE(n_rows <= 65535, "argmax: too many rows");
    MDMA_REQUIRE(scratch && scratch_words >= 3l * n_rows * chunks, "argmax: %ld words of scratch needed, %ld given", 3l * n_rows * chunks, scratch_words);
    float* part_v = scratch;
    int* part_i = reinterpret_cast<int*>(scratch + (size_t)n_rows * chunks);
    int* part_bad = part_i + (size_t)n_rows * chunks;
    launch_chained(argmax_chunks_kernel, dim3(chunks, n_rows), dim3(256), 0, stream, logits, vocab, chunks, part_v, part_i, part_bad);
    MDMA_LAUNCH_OK("argmax_chunks");
    launch_chained(argmax_final_kernel, dim3(n_rows), dim3(128), 0, stream, (const float*)part_v, (const int*)part_i, (const int*)part_bad, chunks, tokens, flags);
    MDMA_LAUNCH_OK("argmax_final");
    return 0;
}

// Floats (4-byte words) of scratch mdma_sample needs: three per vocabulary entry of every row.
extern "C" long mdma_sample_scratch(int n_rows, int vocab) { return 3l * n_rows * vocab; }

// Either `uniforms` (one number per row) or `requests`, `steps` and `seed` (the numbers are then made on
// the device); `advance`: append the selected tokens to the history rings and add one to the steps.
extern "C" int mdma_sample(const float* logits, int n_rows, int vocab, int* history,
                           int* history_len, int history_stride, const float* uniforms,
                           const int* requests, int* steps, unsigned long long seed, int advance,
                           float temperature, float top_p, float min_p, float penalty, int penalty_window,
                           float* probs_scratch, long scratch_words, int* tokens, int* flags, int impl,
                           const unsigned* dev_params, cudaStream_t stream) {
    MDMA_REQUIRE(vocab > 0 && n_rows >= 0, "sample: bad sizes");
    MDMA_REQUIRE(probs_scratch != nullptr, "sample: scratch is required");
    MDMA_REQUIRE(uniforms != nullptr || (requests != nullptr && steps != nullptr),
                 "sample: uniform numbers, or requests and steps to make them from, are required");
    MDMA_REQUIRE(history == nullptr || (history_len != nullptr && history_stride > 0), "sample: a history needs its lengths and a row length");
    MDMA_REQUIRE(penalty > 0.f, "sample: repetition penalty must be positive");
    SampleState st;
    st.history = history; st.history_len = history_len; st.history_stride = history_stride;
    st.uniforms = uniforms; st.requests = requests; st.steps = steps; st.seed = seed; st.advance = advance;
    st.dev_params = dev_params;
    MDMA_REQUIRE(scratch_words >= 3l * n_rows * vocab, "sample: %ld words of scratch needed, %ld given", 3l * n_rows * vocab, scratch_words);
    MDMA_REQUIRE(penalty > 0.f, "sample: repetition penalty must be positive");
    if (n_rows == 0) return 0;
    // A cluster of eight blocks per row when an eighth of the row fits a block's shared memory
    // (vocabularies up to about 250k); else, or if `impl` asks for it, one block per row.
    const int per = ((vocab + kSampleCluster - 1) / kSampleCluster + 3) / 4 * 4;
    const size_t slice_bytes = (size_t)per * sizeof(float) + kWarpHistBytes;
    if (impl != 1 && slice_bytes <= 220 * 1024 && n_rows <= 65535) {
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
            if (e != cudaSuccess) return fail("sample: cannot reserve shared memory: %s", cudaGetErrorString(e));
            configured = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(kSampleCluster, n_rows); cfg.blockDim = dim3(kSampleThreads);
        cfg.dynamicSmemBytes = slice_bytes; cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = kSampleCluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, sample_cluster_kernel, logits, vocab, per, st, temperature, top_p, min_p,
                                           penalty, penalty_window, tokens, flags);
        if (e == cudaSuccess) return 0;
        if (impl == 2) return fail("sample: the cluster launch failed: %s", cudaGetErrorString(e));
        (void)cudaGetLastError();          // the device cannot place the cluster: one block per row
    }
    MDMA_REQUIRE(impl != 2, "sample: a vocabulary of %d does not fit the cluster kernel", vocab);
    static bool configured_one = false;
    if (!configured_one) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWarpHistBytes);
        if (e != cudaSuccess) return fail("sample: cannot reserve shared memory: %s", cudaGetErrorString(e));
        configured_one = true;
    }
    sample_kernel<<<n_rows, kSampleThreads, kWarpHistBytes, stream>>>(logits, vocab, st, temperature, top_p, min_p, penalty,
                                                                      penalty_window, probs_scratch, tokens, flags);
    MDMA_LAUNCH_OK("sample");
    return 0;
}
