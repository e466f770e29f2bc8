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

namespace mdma {

constexpr int kSampleThreads = 1024;

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

// Finds the element at which the running mass of the row, taken in descending
// order of probability (ties by ascending index), first reaches `target`.
// Only elements with probability >= floor_p and, if limit_bits != 0, ranked at
// or before the element (limit_bits, limit_index) take part.  Returns its
// index, bit pattern and the mass up to and including it.
struct Crossing { int index; unsigned bits; unsigned long long mass; };

__device__ Crossing find_crossing(const float* __restrict__ probs, int vocab, unsigned long long target,
                                  unsigned long long* hist /*256*/, int* misc /*8*/) {
    unsigned prefix = 0, prefix_mask = 0;
    unsigned long long above = 0;     // mass of elements with bit pattern above the current prefix range
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0ull;
        __syncthreads();
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float p = probs[i];
            const unsigned bits = __float_as_uint(p);
            if (p > 0.f && (bits & prefix_mask) == prefix)
                atomicAdd(&hist[(bits >> shift) & 255u], mass_of(p));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long run = above;
            int digit = 0;
            bool found = false;
            for (int b = 255; b >= 0; --b) {
                if (hist[b] == 0ull) continue;
                digit = b;                       // the lowest populated digit so far: used if never reached
                if (run + hist[b] >= target) { found = true; break; }
                run += hist[b];
            }
            if (!found) {
                // target beyond the whole mass (rounding): settle on the smallest element
                run = above;
                for (int b = 255; b > digit; --b) run += hist[b];
            }
            misc[0] = digit;
            hist[0] = run;                       // reuse as the hand-over slot
        }
        __syncthreads();
        const int digit = misc[0];
        above = hist[0];
        __syncthreads();
        prefix |= (unsigned)digit << shift;
        prefix_mask |= 255u << shift;
    }
    // All elements with bit pattern == prefix are tied; take them by ascending index.
    const float tie_p = __uint_as_float(prefix);
    const unsigned long long unit = mass_of(tie_p);
    unsigned long long need = target > above ? target - above : 1ull;
    long long kth = unit ? (long long)((need + unit - 1) / unit) : 1;   // how many tied elements are taken
    if (kth < 1) kth = 1;
    // the kth tied element by index: block-wide ordered count over chunks
    int* counter = misc + 1;     // running count of ties before the current chunk
    int* answer = misc + 2;
    int* last_index = misc + 3;      // the highest index among the ties
    if (threadIdx.x == 0) { *counter = 0; *answer = -1; *last_index = 0; }
    __syncthreads();
    __shared__ int warp_counts[32];
    int last_tie = -1;
    for (int base = 0; base < vocab; base += blockDim.x) {
        const int i = base + threadIdx.x;
        const bool tie = i < vocab && __float_as_uint(probs[i]) == prefix;
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
            int s = 0;
            for (int w = 0; w < (blockDim.x + 31) / 32; ++w) s += warp_counts[w];
            *counter += s;
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
    c.index = *answer;
    c.bits = prefix;
    c.mass = above + unit * (unsigned long long)kth;
    __syncthreads();
    return c;
}

// One row: adjusted logits -> probabilities (in `probs`, scratch of vocab
// floats per row) -> min-p / top-p -> draw with the uniform number u[r].
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int vocab, const int* __restrict__ history,
              const int* __restrict__ history_len, int history_stride, const float* __restrict__ uniforms,
              float temperature, float top_p, float min_p, float penalty, int penalty_window,
              float* __restrict__ probs_all, int* __restrict__ tokens, int* __restrict__ flags) {
    __shared__ float fscratch[32];
    __shared__ ArgMax ascratch[32];
    __shared__ unsigned long long hist[256];
    __shared__ int misc[8];
    __shared__ int bad;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    float* probs = probs_all + (size_t)r * vocab;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();

    // 1. copy, flag non-finite values
    bool nonfinite = false;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (!isfinite(v)) nonfinite = true;
        probs[i] = v;
    }
    if (nonfinite) bad = 1;
    __syncthreads();
    // 2. repetition penalty on the last `penalty_window` tokens of the history; a
    //    token that occurs several times is penalised once per occurrence, in order
    if (penalty != 1.0f && history != nullptr && threadIdx.x == 0) {
        const int n = history_len[r];
        const int* hrow = history + (size_t)r * history_stride;
        for (int j = max(0, n - penalty_window); j < n; ++j) {
            const int id = hrow[j];
            if (id >= 0 && id < vocab) {
                const float l = probs[id];
                probs[id] = l > 0.f ? l / penalty : l * penalty;
            }
        }
    }
    __syncthreads();
    // 3. greedy when temperature <= 0
    ArgMax a{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) a = better(a, ArgMax{probs[i], i});
    a = block_argmax(a, ascratch);
    if (temperature <= 0.f || bad) {
        if (threadIdx.x == 0) { tokens[r] = a.i == 0x7fffffff ? 0 : a.i; if (flags) flags[r] = bad; }
        return;
    }
    // 4. softmax of logits / temperature
    const float mx = a.v / temperature;
    float sum = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float e = expf(probs[i] / temperature - mx);
        probs[i] = e;
        sum += e;
    }
    sum = block_sum(sum, fscratch);
    float pmax = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float p = probs[i] / sum;
        probs[i] = p;
        pmax = fmaxf(pmax, p);
    }
    // 5. min-p: keep p >= p_max * min_p
    __syncthreads();
    pmax = warp_max(pmax);
    if ((threadIdx.x & 31) == 0) fscratch[threadIdx.x >> 5] = pmax;
    __syncthreads();
    pmax = 0.f;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) pmax = fmaxf(pmax, fscratch[w]);
    __syncthreads();
    if (min_p > 0.f) {
        const float thr = pmax * min_p;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) if (probs[i] < thr) probs[i] = 0.f;
        __syncthreads();
    }
    // 6. top-p: the smallest descending prefix whose mass reaches top_p
    unsigned long long kept = 0ull;
    if (top_p < 1.0f) {
        const Crossing cut = find_crossing(probs, vocab, mass_of(top_p), hist, misc);
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const unsigned bits = __float_as_uint(probs[i]);
            const bool keep = bits > cut.bits || (bits == cut.bits && i <= cut.index);
            if (!keep) probs[i] = 0.f;
        }
        __syncthreads();
        kept = cut.mass;
    } else {
        for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0ull;
        __syncthreads();
        unsigned long long mine = 0ull;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) mine += mass_of(probs[i]);
        atomicAdd(&hist[0], mine);
        __syncthreads();
        kept = hist[0];
        __syncthreads();
    }
    // 7. draw: first element of the descending order whose running mass reaches u * kept
    const float u = uniforms[r];
    unsigned long long target = (unsigned long long)((double)u * (double)kept);
    if (target < 1ull) target = 1ull;
    const Crossing drawn = find_crossing(probs, vocab, target, hist, misc);
    if (threadIdx.x == 0) { tokens[r] = drawn.index >= 0 ? drawn.index : a.i; if (flags) flags[r] = 0; }
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

extern "C" int mdma_sample(const float* logits, int n_rows, int vocab, const int* history,
                           const int* history_len, int history_stride, const float* uniforms,
                           float temperature, float top_p, float min_p, float penalty, int penalty_window,
                           float* probs_scratch, int* tokens, int* flags, cudaStream_t stream) {
    MDMA_REQUIRE(vocab > 0 && n_rows >= 0, "sample: bad sizes");
    MDMA_REQUIRE(probs_scratch != nullptr && uniforms != nullptr, "sample: scratch and uniform numbers are required");
    MDMA_REQUIRE(penalty > 0.f, "sample: repetition penalty must be positive");
    if (n_rows == 0) return 0;
    sample_kernel<<<n_rows, kSampleThreads, 0, stream>>>(logits, vocab, history, history_len, history_stride,
                                                         uniforms, temperature, top_p, min_p, penalty,
                                                         penalty_window, probs_scratch, tokens, flags);
    MDMA_LAUNCH_OK("sample");
    return 0;
}
