// bfloat16 matrix products on the fifth-generation tensor cores.
//
//   out[t, f] (=, +=)  sum_k  X[t, k] * W[f, k]        X: tokens x K, W: features x K
//
// The weight matrix is the 128-row MMA operand (A) and the tokens are the MMA's
// N dimension, so that one kernel serves a prefill of thousands of tokens
// (N tile 256) and a decode step of a handful (N tile 16) while every tile
// still streams 128 weight rows.  Per block: one warp issues TMA loads of
// 128 x 64 weight boxes and N x 64 activation boxes (128-byte swizzle) into a
// ring of shared-memory stages, one thread issues tcgen05.mma into a float
// accumulator in tensor memory, four warps read the accumulator back
// (tcgen05.ld; lane = feature, column = token) and apply the ending:
//   store (bf16 or float), add into the float residual stream, SwiGLU of two
//   accumulators (gate and up share the activation tile), or float partial
//   sums of a K split, reduced afterwards in split order.
// Sizes: any token count, any feature count, K a multiple of 8 (16-byte rows
// for TMA); tails are zero-filled by TMA and masked at the store.
#include <unordered_map>
#include <mutex>
#include <string.h>

#include "common.cuh"
#include "ptx.cuh"

namespace mdma {

enum TcMode : int { kTcStore = 0, kTcAccumulate = 1, kTcSwiGLU = 2, kTcPartial = 3 };

constexpr int kBM = 128;        // features per tile (MMA M)
constexpr int kBK = 64;         // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kTcThreads = 192; // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
// Token tiles of 64 and more have eight epilogue warps, two per 32 rows, each with half of the columns: a block of such
// a tile has its SM to itself (or shares it with one other), so nothing else hides the time it takes to read the
// accumulators out.
template <int BN> constexpr int tc_epi_parts() { return BN >= 128 ? 4 : 2; }         // epilogue warps per 32 rows
template <int BN> constexpr int tc_threads() { return (2 + 4 * tc_epi_parts<BN>()) * 32; }
// block-pair kernel: warps 2 and up are the epilogue, two warps (column halves) per 32 lanes of tensor memory, four
// (column quarters) for the gated product, whose single accumulator buffer leaves the epilogue exposed
template <int MODE> constexpr int tc2_epi_warps() { return MODE == 2 ? 16 : 8; }
template <int MODE> constexpr int tc2_threads() { return (2 + tc2_epi_warps<MODE>()) * 32; }

struct TcParams {
    void* out; int ldo; int out_f32;
    int n_tokens, n_features, k_blocks, kb_per_split;
    float* partial;            // [splits, n_tokens, n_features] when MODE == kTcPartial
    int* status;               // device word set non-zero when a wait ran out
    int cluster;               // > 1: that many blocks of a cluster split K and reduce through shared memory
    Ending ending;             // bias vectors over the features and the gate's activation
    int pair_tokens;           // block-pair kernel: width of a token tile (a multiple of 32 up to 256)
    float* sk_partial;         // block-pair kernel: one partial tile per pair and block, for tiles shared by two pairs
    int* sk_flags;             // [pairs * 2] zero between launches; non-null switches the even K-block split on
};

template <int BN, int MODE>
struct TcSmem {
    static constexpr int kA = kBM * kBK * 2;
    static constexpr int kB = BN * kBK * 2;
    static constexpr int kStage = kA * (MODE == kTcSwiGLU ? 2 : 1) + (kB < 1024 ? 1024 : kB);
    // small token tiles leave room for two blocks per SM (decode: more blocks than SMs stay balanced);
    // 64 tokens with two weight matrices would have two stages only, so they get the whole SM
    static constexpr int kBudget = ((BN <= 32 || (BN == 64 && MODE != kTcSwiGLU)) ? 110 : 200) * 1024;
    static constexpr int kStages = (kBudget / kStage) < 8 ? (kBudget / kStage) : 8;
    static constexpr int kBytes = kStages * kStage + 1024 /*alignment*/ + 256 /*barriers*/;
    static constexpr int kTmemCols = (MODE == kTcSwiGLU ? 2 : 1) * BN < 32 ? 32 : (MODE == kTcSwiGLU ? 2 : 1) * BN;
};

template <int BN, int MODE>
__global__ void __launch_bounds__(tc_threads<BN>())
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
               const __grid_constant__ CUtensorMap map_x, const TcParams p) {
    using S = TcSmem<BN, MODE>;
    constexpr int kStages = S::kStages;
    constexpr bool kDual = MODE == kTcSwiGLU;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - ptx::smem_addr(smem_raw));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + kStages * S::kStage);
    const uint32_t bar0 = base + kStages * S::kStage;
    // barrier layout: full[kStages], empty[kStages], acc_full, then the TMEM base word and abort flag
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    const uint32_t acc_bar = bar0 + 8u * (2 * kStages);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * kStages + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kStages + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // With a cluster, the blocks of a cluster share one output tile and divide its K range by rank.
    const int rank = p.cluster > 1 ? (int)ptx::cluster_rank() : 0;
    const int f0 = (blockIdx.x / p.cluster) * kBM;
    const int t0 = blockIdx.y * BN;
    const int kb_begin = (p.cluster > 1 ? rank : (int)blockIdx.z) * p.kb_per_split;
    const int kb_end = min(p.k_blocks, kb_begin + p.kb_per_split);
    const int n_kb = kb_end - kb_begin;

    chain_release();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        ptx::mbar_init(acc_bar, 1);
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr((const void*)tmem_slot), S::kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- producer: TMA loads into the ring -------------------------------
        ptx::prefetch_tensormap(&map_w);
        ptx::prefetch_tensormap(&map_x);
        if (kDual) ptx::prefetch_tensormap(&map_w2);
        // Weights do not depend on earlier kernels: fill the ring with weight boxes first,
        // then wait for the kernel before this one and fetch the matching activation boxes.
        const int ahead = min(n_kb, kStages);
        for (int i = 0; i < ahead; ++i) {
            const uint32_t stage = base + i * S::kStage;
            ptx::mbar_expect_tx(full_bar(i), S::kA * (kDual ? 2 : 1) + S::kB);
            const int k = (kb_begin + i) * kBK;
            ptx::tma_load_2d(stage, &map_w, full_bar(i), k, f0);
            if (kDual) ptx::tma_load_2d(stage + S::kA, &map_w2, full_bar(i), k, f0);
        }
        chain_wait();
        for (int i = 0; i < ahead; ++i)
            ptx::tma_load_2d(base + i * S::kStage + S::kA * (kDual ? 2 : 1), &map_x, full_bar(i), (kb_begin + i) * kBK, t0);
        int issued = ahead;
        for (int i = ahead; i < n_kb; ++i) {
            const int s = i % kStages;
            if (!ptx::mbar_wait(empty_bar(s), ((i / kStages) & 1) ^ 1, abort_flag)) break;
            const uint32_t stage = base + s * S::kStage;
            ptx::mbar_expect_tx(full_bar(s), S::kA * (kDual ? 2 : 1) + S::kB);
            const int k = (kb_begin + i) * kBK;
            ptx::tma_load_2d(stage, &map_w, full_bar(s), k, f0);
            if (kDual) ptx::tma_load_2d(stage + S::kA, &map_w2, full_bar(s), k, f0);
            ptx::tma_load_2d(stage + S::kA * (kDual ? 2 : 1), &map_x, full_bar(s), k, t0);
            ++issued;
        }
        if (*abort_flag) {
            // let the copies in flight land before the block's shared memory is given up
            for (int i = max(0, issued - kStages); i < issued; ++i)
                ptx::mbar_wait(full_bar(i % kStages), (i / kStages) & 1, abort_flag);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer -------------------------------------------------------
        constexpr uint32_t idesc = ptx::idesc_bf16_f32(kBM, BN);
        bool ok = true;
        for (int i = 0; i < n_kb && ok; ++i) {
            const int s = i % kStages;
            ok = ptx::mbar_wait(full_bar(s), (i / kStages) & 1, abort_flag);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const uint32_t stage = base + s * S::kStage;
            const uint32_t a_addr = stage, b_addr = stage + S::kA * (kDual ? 2 : 1);
#pragma unroll
            for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
                const uint64_t b_desc = ptx::smem_desc_sw128(b_addr + kk * kUmmaK * 2);
                const uint32_t acc = (i > 0 || kk > 0) ? 1u : 0u;
                ptx::mma_bf16_ss(tmem_base, ptx::smem_desc_sw128(a_addr + kk * kUmmaK * 2), b_desc, idesc, acc);
                if (kDual)
                    ptx::mma_bf16_ss(tmem_base + BN, ptx::smem_desc_sw128(a_addr + S::kA + kk * kUmmaK * 2),
                                     b_desc, idesc, acc);
            }
            ptx::mma_commit(empty_bar(s));      // the stage is free once these MMAs have read it
        }
        ptx::mma_commit(acc_bar);               // the accumulator is complete
    }
    // ---- epilogue: TMEM -> registers -> (cluster reduction) -> global ------------------
    const int quad = warp & 3;                  // the TMEM lanes an epilogue warp may read
    const int f = f0 + quad * 32 + lane;
    constexpr int kColsPerWarp = BN / tc_epi_parts<BN>();                // eight epilogue warps: column halves (sixteen: quarters)
    constexpr int kStep = kColsPerWarp < 16 ? 8 : 16;                    // columns read out of tensor memory at a time
    const int c_lo = ((warp - 2) >> 2) * kColsPerWarp, c_hi = c_lo + kColsPerWarp;
    auto load_cols = [](uint32_t addr, float* dst) { if (kStep == 16) ptx::tmem_load_16(addr, dst); else ptx::tmem_load_8(addr, dst); };
    bool acc_ok = false;
    if (warp >= 2) {
        chain_wait();                           // the output may still be read by an earlier kernel
        acc_ok = ptx::mbar_wait(acc_bar, 0, abort_flag) && n_kb > 0;
        ptx::tc_fence_after_sync();
    }
    constexpr int kAccs = kDual ? 2 : 1;
    if (p.cluster > 1) {
        // Everyone's MMAs are done, so the leader's stage ring is free: the other ranks write their
        // accumulators there ([rank-1][accumulator][column][128 features] floats), the leader adds
        // them to its own in rank order.
        ptx::cluster_sync();
        if (warp >= 2 && rank > 0) {
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
            const uint32_t slot = ptx::cluster_map(base, 0) +
                                  (uint32_t)(((rank - 1) * kAccs * BN) * kBM + quad * 32 + lane) * 4u;
#pragma unroll 1
            for (int c = c_lo; c < c_hi; c += kStep) {
                if (t0 + c >= p.n_tokens) break;
                float v[16], u[16];
                if (acc_ok) {
                    load_cols(lane_addr + c, v);
                    if (kDual) load_cols(lane_addr + BN + c, u);
                } else {
#pragma unroll
                    for (int j = 0; j < kStep; ++j) { v[j] = 0.f; u[j] = 0.f; }
                }
#pragma unroll
                for (int j = 0; j < kStep; ++j) {
                    ptx::cluster_store_f32(slot + (uint32_t)((c + j) * kBM) * 4u, v[j]);
                    if (kDual) ptx::cluster_store_f32(slot + (uint32_t)((BN + c + j) * kBM) * 4u, u[j]);
                }
            }
        }
        ptx::cluster_sync();
    }
    if (warp >= 2 && rank == 0 && (acc_ok || p.cluster > 1)) {
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        const float* staged = reinterpret_cast<const float*>(base_ptr) + quad * 32 + lane;
        // the bias goes in once: with partial sums, into the first split's
        const bool biased = f < p.n_features && (MODE != kTcPartial || blockIdx.z == 0);
        const float b1 = biased ? ending_bias(p.ending.bias, p.ending.bias_dtype, f) : 0.f;
        const float b2 = kDual && biased ? ending_bias(p.ending.bias2, p.ending.bias_dtype, f) : 0.f;
#pragma unroll 1
        for (int c = c_lo; c < c_hi; c += kStep) {
            if (t0 + c >= p.n_tokens) break;           // uniform over the warp
            float v[16], u[16];
            if (acc_ok) {
                load_cols(lane_addr + c, v);
                if (kDual) load_cols(lane_addr + BN + c, u);
            } else {
#pragma unroll
                for (int j = 0; j < kStep; ++j) { v[j] = 0.f; u[j] = 0.f; }
            }
            for (int r = 1; r < p.cluster; ++r) {
#pragma unroll
                for (int j = 0; j < kStep; ++j) {
                    v[j] += staged[(size_t)(((r - 1) * kAccs * BN) + c + j) * kBM];
                    if (kDual) u[j] += staged[(size_t)(((r - 1) * kAccs * BN) + BN + c + j) * kBM];
                }
            }
            if (f < p.n_features) {
                const int valid = min(kStep, p.n_tokens - (t0 + c));
                if (MODE == kTcAccumulate) {
                    // read the 16 residual values first so the loads overlap, then add and store
                    float* o = reinterpret_cast<float*>(p.out) + (size_t)(t0 + c) * p.ldo + f;
                    float old[16];
#pragma unroll
                    for (int j = 0; j < kStep; ++j) old[j] = j < valid ? o[(size_t)j * p.ldo] : 0.f;
#pragma unroll
                    for (int j = 0; j < kStep; ++j) if (j < valid) o[(size_t)j * p.ldo] = old[j] + (v[j] + b1);
                } else {
#pragma unroll
                    for (int j = 0; j < kStep; ++j) {
                        if (j >= valid) break;
                        const int t = t0 + c + j;
                        float r = v[j] + b1;
                        if (MODE == kTcSwiGLU) r = gate_activation_fast(r, p.ending.act) * (u[j] + b2);
                        if (MODE == kTcPartial) {
                            p.partial[((size_t)blockIdx.z * p.n_tokens + t) * p.n_features + f] = r;
                        } else if (p.out_f32) {
                            reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + f] = r;
                        } else {
                            reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)t * p.ldo + f] = __float2bfloat16_rn(r);
                        }
                    }
                }
            }
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, S::kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
}

// ---------------------------------------------------------------------------------------
// The same product for many tokens with two blocks working as one (cta_group::2): a pair
// covers 256 features x 256 tokens.  Each block loads its own 128 weight rows and only HALF
// of the token tile (128 tokens) per stage; one tcgen05.mma issued by the leading block reads
// both blocks' shared memory and writes 128 accumulator rows into each block's tensor memory.
// Per block and K step that is 32 KB of operands instead of 48 KB (48 instead of 64 with two
// weight matrices), which is what the single-block kernel runs short of.
template <int MODE>
struct Tc2Smem {
    static constexpr int kA = kBM * kBK * 2, kB = 128 * kBK * 2;
    static constexpr int kStage = kA * (MODE == kTcSwiGLU ? 2 : 1) + kB;
    static constexpr int kStages = (200 * 1024) / kStage;
    static constexpr int kBytes = kStages * kStage + 1024 + 256;
    static constexpr int kTmemCols = MODE == kTcSwiGLU ? 512 : 256;
};

// Work of one pair: a list of segments (tile, K blocks [kb0, kb1), kind).  Without the even split a
// pair owns whole tiles (tile = pair, pair + pairs, ...).  With it, all K blocks of all tiles are
// divided evenly among the pairs, so that no pair idles in a last partial round; a tile that two pairs
// share is finished by the later pair: the earlier pair leaves its partial accumulators in global
// memory (its LAST segment but one), the later pair adds them at its LAST segment, so both reach the
// shared tile at about the same time and nobody waits long.
enum SegKind : int { kSegFull = 0, kSegHead = 1, kSegTail = 2 };
struct Segment { int tile, kb0, kb1, kind; };
struct PairWork {
    int n_round, n_pairs, pair;          // whole rounds: tile = pair + i * n_pairs
    int n_full, first_full;              // then consecutive whole tiles of the evenly split rest
    int head_tile, head_kb1;             // -1: none
    int tail_tile, tail_kb0;             // -1: none
    int n_kb;
    __device__ int count() const { return n_round + n_full + (head_tile >= 0) + (tail_tile >= 0); }
    __device__ Segment get(int i) const {
        if (i < n_round) return Segment{pair + i * n_pairs, 0, n_kb, kSegFull};
        i -= n_round;
        if (i < n_full) return Segment{first_full + i, 0, n_kb, kSegFull};
        if (head_tile >= 0 && i == n_full) return Segment{head_tile, 0, head_kb1, kSegHead};
        return Segment{tail_tile, tail_kb0, n_kb, kSegTail};
    }
};
// With the even split, all rounds but the last whole one run as without it (pairs that work at the
// same time then share weight and token tiles); the last whole round and the partial round after it
// are divided by K blocks.  Each pair's share is then at least one tile long, so a tile is shared by
// two pairs at most.
__device__ inline PairWork pair_work(int pair, int n_pairs, int n_tiles, int n_kb, bool even_split) {
    PairWork w;
    w.n_kb = n_kb; w.head_tile = w.tail_tile = -1; w.head_kb1 = w.tail_kb0 = 0;
    w.pair = pair; w.n_pairs = n_pairs; w.n_full = 0; w.first_full = 0;
    if (!even_split || n_tiles < n_pairs) {
        w.n_round = pair < n_tiles ? (n_tiles - pair + n_pairs - 1) / n_pairs : 0;
        return w;
    }
    w.n_round = n_tiles / n_pairs - 1;
    const int base = w.n_round * n_pairs;
    const long long units = (long long)(n_tiles - base) * n_kb;
    const long long lo = units * pair / n_pairs, hi = units * (pair + 1) / n_pairs;
    int first_tile = (int)(lo / n_kb), first_kb = (int)(lo % n_kb);
    int last_tile = (int)((hi - 1) / n_kb), last_end = (int)((hi - 1) % n_kb) + 1;
    if (first_kb > 0) { w.tail_tile = base + first_tile; w.tail_kb0 = first_kb; ++first_tile; }
    if (last_end < n_kb) { w.head_tile = base + last_tile; w.head_kb1 = last_end; --last_tile; }
    w.first_full = base + first_tile;
    w.n_full = last_tile >= first_tile ? last_tile - first_tile + 1 : 0;
    return w;
}

template <int MODE>
__global__ void __launch_bounds__(tc2_threads<MODE>())
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                const __grid_constant__ CUtensorMap map_x, const TcParams p) {
    // Persistent: the grid holds at most one pair per two SMs and every pair walks over its segments.
    // The shared-memory ring runs on across segments, and with one weight matrix the accumulator has
    // two buffers in tensor memory, so a tile's epilogue runs under the next tile's MMAs.
    using S = Tc2Smem<MODE>;
    constexpr int kStages = S::kStages;
    constexpr bool kDual = MODE == kTcSwiGLU;
    constexpr int BN = 256;                                // the widest token tile; accumulators and partial tiles are laid out for it
    const int bn = p.pair_tokens;                          // this launch's token tile: the tokens divided evenly over the fewest tiles
    constexpr int kAccs = kDual ? 2 : 1;
    constexpr int kBufs = kDual ? 1 : 2;                   // accumulator buffers of 256 (512) columns
    constexpr int kBufCols = kDual ? 512 : 256;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - ptx::smem_addr(smem_raw));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + kStages * S::kStage);
    const uint32_t bar0 = base + kStages * S::kStage;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto acc_full = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
    auto acc_empty = [&](int b) { return bar0 + 8u * (2 * kStages + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * kStages + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kStages + 5);
    const uint32_t ep_bar = bar0 + 8u * (2 * kStages + 6);      // this block's eight epilogue warps meet here (bounded)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)ptx::cluster_rank();
    const int n_pairs = gridDim.x / 2, pair = blockIdx.x / 2;
    const int f_tiles = (p.n_features + 255) / 256, t_tiles = (p.n_tokens + bn - 1) / bn;
    const PairWork work = pair_work(pair, n_pairs, f_tiles * t_tiles, p.k_blocks, p.sk_flags != nullptr);
    const int n_seg = work.count();

    // This kernel takes no part in programmatic dependent launch: launched early next to the tail of
    // another kernel it stalled now and then; it is used for many tokens, where a launch gap is
    // nothing against its run time.
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(acc_full(b), 1); ptx::mbar_init(acc_empty(b), 2 * tc2_epi_warps<MODE>()); }   // epilogue warps x 2 blocks
        ptx::mbar_init(ep_bar, 32 * tc2_epi_warps<MODE>());
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_addr((const void*)tmem_slot), 512);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before_sync();
    ptx::cluster_sync();                   // both blocks' barriers exist before either signals the other
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- producer: this block's halves; bytes are counted on the leading block's barrier ----
        ptx::prefetch_tensormap(&map_w);
        ptx::prefetch_tensormap(&map_x);
        if (kDual) ptx::prefetch_tensormap(&map_w2);
        int it = 0;                        // stage uses so far, across segments
        bool ok = true;
        for (int si = 0; si < n_seg && ok; ++si) {
            const Segment sg = work.get(si);
            const int f0 = (sg.tile / t_tiles) * 256 + rank * 128;      // token tiles of one feature tile run together
            const int t0 = (sg.tile % t_tiles) * bn + rank * (bn / 2);       // each block loads half of the token tile
            const uint32_t stage_bytes = (uint32_t)(S::kA * (kDual ? 2 : 1) + (bn / 2) * kBK * 2);
            for (int i = sg.kb0; i < sg.kb1; ++i, ++it) {
                const int s = it % kStages;
                if (!ptx::mbar_wait(empty_bar(s), ((it / kStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
                const uint32_t stage = base + s * S::kStage;
                const uint32_t lead_full = ptx::cluster_map(full_bar(s), 0);
                if (rank == 0) ptx::mbar_expect_tx(full_bar(s), 2 * stage_bytes);     // both blocks' bytes
                const int k = i * kBK;
                ptx::tma_load_2d_pair(stage, &map_w, lead_full, k, f0);
                if (kDual) ptx::tma_load_2d_pair(stage + S::kA, &map_w2, lead_full, k, f0);
                ptx::tma_load_2d_pair(stage + S::kA * (kDual ? 2 : 1), &map_x, lead_full, k, t0);
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---- MMA issuer (leading block only) ----------------------------------------------
        const uint32_t idesc = ptx::idesc_bf16_f32(256, bn);
        int it = 0;
        bool ok = true;
        for (int si = 0; si < n_seg && ok; ++si) {
            const Segment sg = work.get(si);
            const int buf = si % kBufs;
            // the buffer's previous tile must have been read out by both blocks' epilogues
            ok = ptx::mbar_wait(acc_empty(buf), (((si / kBufs) & 1) ^ 1), abort_flag);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const uint32_t acc_addr = tmem_base + buf * kBufCols;
            for (int i = sg.kb0; i < sg.kb1; ++i, ++it) {
                const int s = it % kStages;
                ok = ptx::mbar_wait(full_bar(s), (it / kStages) & 1, abort_flag);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t stage = base + s * S::kStage;
                const uint32_t a_addr = stage, b_addr = stage + S::kA * (kDual ? 2 : 1);
#pragma unroll
                for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
                    const uint64_t b_desc = ptx::smem_desc_sw128(b_addr + kk * kUmmaK * 2);
                    const uint32_t acc = (i > sg.kb0 || kk > 0) ? 1u : 0u;
                    ptx::mma_bf16_ss_pair(acc_addr, ptx::smem_desc_sw128(a_addr + kk * kUmmaK * 2), b_desc, idesc, acc);
                    if (kDual)
                        ptx::mma_bf16_ss_pair(acc_addr + BN, ptx::smem_desc_sw128(a_addr + S::kA + kk * kUmmaK * 2),
                                              b_desc, idesc, acc);
                }
                ptx::mma_commit_pair(empty_bar(s), 3);      // frees the stage in both blocks
            }
            ptx::mma_commit_pair(acc_full(buf), 3);         // both blocks' accumulators of this segment are complete
        }
    } else if (warp >= 2) {
        // ---- epilogue: each block handles its own 128 features x 256 tokens of every segment ------
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                   // feature row within this block's half
        constexpr int kParts = tc2_epi_warps<MODE>() / 4;                              // column parts: halves or quarters
        const int c_begin = ((warp - 2) >> 2) * (bn / kParts), c_end = c_begin + bn / kParts;     // this warp's columns
        const uint32_t lead_empty[2] = {ptx::cluster_map(acc_empty(0), 0), ptx::cluster_map(acc_empty(1), 0)};
        // partial tiles in global memory: [pair][block of the pair][accumulator][column][128 rows]
        const size_t part_stride = (size_t)kAccs * BN * 128;
        float* my_part = p.sk_partial ? p.sk_partial + ((size_t)pair * 2 + rank) * part_stride + row : nullptr;
        const float* prev_part = p.sk_partial && pair > 0 ? p.sk_partial + ((size_t)(pair - 1) * 2 + rank) * part_stride + row : nullptr;
        bool ok = true;
        uint32_t ep_phase = 0;
        for (int si = 0; si < n_seg && ok; ++si) {
            const Segment sg = work.get(si);
            const int buf = si % kBufs;
            const int f = (sg.tile / t_tiles) * 256 + rank * 128 + row;
            const int t0 = (sg.tile % t_tiles) * bn;
            const float b1 = f < p.n_features ? ending_bias(p.ending.bias, p.ending.bias_dtype, f) : 0.f;
            const float b2 = kDual && f < p.n_features ? ending_bias(p.ending.bias2, p.ending.bias_dtype, f) : 0.f;
            ok = __all_sync(0xffffffffu, ptx::mbar_wait(acc_full(buf), (si / kBufs) & 1, abort_flag));
            if (!ok) break;
            ptx::tc_fence_after_sync();
            if (sg.kind == kSegTail) {
                // the pair before this one did the first K blocks of this tile: wait for its partial sums
                const volatile int* flag = p.sk_flags + (size_t)(pair - 1) * 2 + rank;
                const bool there = ptx::flag_wait(flag, abort_flag);
                ok = __all_sync(0xffffffffu, there);
                if (!ok) { *abort_flag = 1; break; }
            }
            const uint32_t lane_addr = tmem_base + buf * kBufCols + ((uint32_t)(quad * 32) << 16);
            // the other pair's partial sums of the next 16 columns are fetched while these 16 are finished
            float pv[16], pu[16];
            auto fetch_partial = [&](int c) {
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    pv[q] = __ldcg(prev_part + (size_t)(c + q) * 128);
                    if (kDual) pu[q] = __ldcg(prev_part + (size_t)(BN + c + q) * 128);
                }
            };
            if (sg.kind == kSegTail) fetch_partial(c_begin);
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 16) {
                if (sg.kind != kSegHead && t0 + c >= p.n_tokens) break;      // a head part leaves all columns
                float v[16], u[16];
                ptx::tmem_load_16(lane_addr + c, v);
                if (kDual) ptx::tmem_load_16(lane_addr + BN + c, u);
                if (sg.kind == kSegHead) {
                    // leave the partial sums for the next pair (all 256 columns: it adds them all)
#pragma unroll
                    for (int q = 0; q < 16; ++q) {
                        my_part[(size_t)(c + q) * 128] = v[q];
                        if (kDual) my_part[(size_t)(BN + c + q) * 128] = u[q];
                    }
                    continue;
                }
                if (sg.kind == kSegTail) {
#pragma unroll
                    for (int q = 0; q < 16; ++q) {
                        v[q] += pv[q];
                        if (kDual) u[q] += pu[q];
                    }
                    if (c + 16 < c_end) fetch_partial(c + 16);
                }
                if (f < p.n_features) {
                    const int valid = min(16, p.n_tokens - (t0 + c));
                    if (MODE == kTcAccumulate) {
                        float* o = reinterpret_cast<float*>(p.out) + (size_t)(t0 + c) * p.ldo + f;
                        float old[16];
#pragma unroll
                        for (int q = 0; q < 16; ++q) old[q] = q < valid ? o[(size_t)q * p.ldo] : 0.f;
#pragma unroll
                        for (int q = 0; q < 16; ++q) if (q < valid) o[(size_t)q * p.ldo] = old[q] + (v[q] + b1);
                    } else {
#pragma unroll
                        for (int q = 0; q < 16; ++q) {
                            if (q >= valid) break;
                            const int t = t0 + c + q;
                            float r = v[q] + b1;
                            if (MODE == kTcSwiGLU) r = gate_activation_fast(r, p.ending.act) * (u[q] + b2);
                            if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + f] = r;
                            else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)t * p.ldo + f] = __float2bfloat16_rn(r);
                        }
                    }
                }
            }
            // this warp has read its part of the buffer: tell the leading block's MMA thread
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(lead_empty[buf]);
            if (sg.kind == kSegHead || sg.kind == kSegTail) {
                // the eight epilogue warps of this block: all partial rows written (read) before the flag moves
                // (an mbarrier, not bar.sync: a warp that gave up elsewhere must not leave the others waiting for ever)
                __threadfence();
                ptx::mbar_arrive(ep_bar);
                ok = __all_sync(0xffffffffu, ptx::mbar_wait(ep_bar, ep_phase & 1u, abort_flag));
                ++ep_phase;
                if (!ok) break;
                if (warp == 2 && lane == 0) {
                    int* flag = p.sk_flags + (size_t)(sg.kind == kSegHead ? pair : pair - 1) * 2 + rank;
                    const int v = sg.kind == kSegHead ? 1 : 0;          // set by the writer, cleared by the reader
                    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flag), "r"(v) : "memory");
                }
            }
        }
    }
    ptx::tc_fence_before_sync();
    ptx::cluster_sync();                   // neither block leaves (or frees tensor memory) while the other may still use it
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 3);
}

// out (=, +=) sum over splits of partial, in split order.
template <int MODE>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, int n_tokens, int n_features,
                                     void* __restrict__ out, int ldo, int out_f32) {
    chain_release();
    chain_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)n_tokens * n_features;
    if (i >= total) return;
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[(size_t)s * total + i];
    const size_t t = i / n_features, f = i % n_features;
    if (MODE == kTcAccumulate) reinterpret_cast<float*>(out)[t * ldo + f] += acc;
    else if (out_f32) reinterpret_cast<float*>(out)[t * ldo + f] = acc;
    else reinterpret_cast<__nv_bfloat16*>(out)[t * ldo + f] = __float2bfloat16_rn(acc);
}

// A kernel that does nothing but wait, with the waits of the kernels above: mode 0 on an mbarrier that
// nobody arrives on, mode 1 on a flag in global memory.  With a flag that nothing sets the wait runs out
// after the limit, the block raises its abort flag and reports through the status word, as a product
// kernel whose protocol broke would: this is how the tests see that path without breaking anything.
__global__ void wait_probe_kernel(int mode, const int* flag, int* status) {
    __shared__ uint64_t bar;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_addr(&bar), 1);
        abort_word = 0;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x < 32) {
        ok = mode == 0 ? ptx::mbar_wait(ptx::smem_addr(&bar), 0, abort_flag) : ptx::flag_wait(flag, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) *abort_flag = 1;
    }
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && status) atomicExch(status, 5);
}

// ---- tensor maps ----------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

struct MapKey {
    const void* ptr; uint64_t rows, cols, pitch; uint32_t box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && pitch == o.pitch && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ k.rows; h = h * 1000003u ^ k.cols; h = h * 1000003u ^ k.pitch; h = h * 1000003u ^ k.box_rows;
        return h;
    }
};

// A bf16 matrix [rows, cols] with `pitch` bytes per row, tiled in boxes of box_rows x 64.
static int make_map_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t pitch,
                       uint32_t box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    const MapKey key{ptr, rows, cols, pitch, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail("gemm_tc: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("gemm_tc: cuTensorMapEncodeTiled failed with %d (ptr %p rows %llu cols %llu pitch %llu)",
                                       (int)r, ptr, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)pitch);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

}  // namespace mdma

using namespace mdma;

template <int BN, int MODE>
static int run_tc(const void* x, int ldx, const void* w, const void* w2, int K, TcParams p, int splits,
                  cudaStream_t stream) {
    using S = TcSmem<BN, MODE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
        if (e != cudaSuccess) return fail("gemm_tc: cannot reserve %d bytes of shared memory: %s", S::kBytes, cudaGetErrorString(e));
        configured = true;
    }
    CUtensorMap mw, mw2, mx;
    if (int rc = make_map_2d(&mw, w, (uint64_t)p.n_features, (uint64_t)K, (uint64_t)K * 2, kBM)) return rc;
    mw2 = mw;
    if (MODE == kTcSwiGLU)
        if (int rc = make_map_2d(&mw2, w2, (uint64_t)p.n_features, (uint64_t)K, (uint64_t)K * 2, kBM)) return rc;
    if (int rc = make_map_2d(&mx, x, (uint64_t)p.n_tokens, (uint64_t)K, (uint64_t)ldx * 2, BN)) return rc;
    // the staging of the cluster reduction must fit the stage ring: shrink the cluster until it does
    while (p.cluster > 1 && (p.cluster - 1) * (MODE == kTcSwiGLU ? 2 : 1) * BN * kBM * 4 > S::kStages * S::kStage) {
        --p.cluster;
        p.kb_per_split = (p.k_blocks + p.cluster - 1) / p.cluster;
    }
    if (p.cluster > 1) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(((p.n_features + kBM - 1) / kBM) * p.cluster, (p.n_tokens + BN - 1) / BN, 1);
        cfg.blockDim = dim3(tc_threads<BN>()); cfg.dynamicSmemBytes = S::kBytes; cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = p.cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = chaining_enabled() ? 2 : 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, MODE>, mw, mw2, mx, p);
        if (e != cudaSuccess) return fail("gemm_tc: cluster launch failed: %s", cudaGetErrorString(e));
        return 0;
    }
    dim3 grid((p.n_features + kBM - 1) / kBM, (p.n_tokens + BN - 1) / BN, splits);
    launch_chained(gemm_tc_kernel<BN, MODE>, grid, dim3(tc_threads<BN>()), S::kBytes, stream, mw, mw2, mx, p);
    MDMA_LAUNCH_OK("gemm_tc");
    return 0;
}

template <int MODE>
static int run_tc2(const void* x, int ldx, const void* w, const void* w2, int K, TcParams p, cudaStream_t stream) {
    using S = Tc2Smem<MODE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
        if (e != cudaSuccess) return fail("gemm_tc2: cannot reserve %d bytes of shared memory: %s", S::kBytes, cudaGetErrorString(e));
        configured = true;
    }
    CUtensorMap mw, mw2, mx;
    if (int rc = make_map_2d(&mw, w, (uint64_t)p.n_features, (uint64_t)K, (uint64_t)K * 2, kBM)) return rc;
    mw2 = mw;
    if (MODE == kTcSwiGLU)
        if (int rc = make_map_2d(&mw2, w2, (uint64_t)p.n_features, (uint64_t)K, (uint64_t)K * 2, kBM)) return rc;
    // token tiles of up to 256, all of one width: the tokens divided evenly over the fewest tiles (320 tokens: two
    // tiles of 160, not one of 256 and one that is three quarters empty)
    const int t_tiles = (p.n_tokens + 255) / 256;
    // (a multiple of 16 columns for every epilogue warp: 32 with column halves, 64 with quarters)
    constexpr int kGrain = 16 * (tc2_epi_warps<MODE>() / 4);
    p.pair_tokens = (((p.n_tokens + t_tiles - 1) / t_tiles) + kGrain - 1) / kGrain * kGrain;
    if (int rc = make_map_2d(&mx, x, (uint64_t)p.n_tokens, (uint64_t)K, (uint64_t)ldx * 2, p.pair_tokens / 2)) return rc;
    p.cluster = 1;
    cudaLaunchConfig_t cfg = {};
    // persistent: one pair per two SMs at most
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count < 2) sm_count = 2;
    }
    const long tiles = (long)((p.n_features + 255) / 256) * ((p.n_tokens + p.pair_tokens - 1) / p.pair_tokens);
    const int pairs = (int)(tiles < sm_count / 2 ? tiles : sm_count / 2);
    cfg.gridDim = dim3(pairs * 2, 1, 1);
    cfg.blockDim = dim3(tc2_threads<MODE>()); cfg.dynamicSmemBytes = S::kBytes; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // The even split of K blocks pays when the tiles do not fill whole rounds of pairs, and only with
    // two weight matrices: with one, the product runs at the power limit of the device either way
    // (measured: 2048 tokens, gate+up 455 -> 425 us; QKV 79 -> 83 us, down 180 -> 192 us).
    // A pair that finishes a shared tile waits for the pair before it (a lower block index, so it has
    // been started no later), with a limit.  The split is only used when the device can hold all pairs
    // at once (asked once); the launch is an ordinary cluster launch, which profilers take.
    static int max_pairs = -1;
    if (max_pairs < 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel<MODE>, &cfg) != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
        max_pairs = n;
    }
    const bool uneven = MODE == kTcSwiGLU && tiles > pairs && tiles % pairs != 0;
    if (!(uneven && pairs <= max_pairs)) { p.sk_partial = nullptr; p.sk_flags = nullptr; }
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<MODE>, mw, mw2, mx, p);
    if (e != cudaSuccess) return fail("gemm_tc2: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

template <int MODE>
static int run_tc_bn(int bn, const void* x, int ldx, const void* w, const void* w2, int K, const TcParams& p,
                     int splits, cudaStream_t stream) {
    switch (bn) {
        case 16: return run_tc<16, MODE>(x, ldx, w, w2, K, p, splits, stream);
        case 32: return run_tc<32, MODE>(x, ldx, w, w2, K, p, splits, stream);
        case 64: return run_tc<64, MODE>(x, ldx, w, w2, K, p, splits, stream);
        case 128: return run_tc<128, MODE>(x, ldx, w, w2, K, p, splits, stream);
        case 256: return run_tc<256, MODE>(x, ldx, w, w2, K, p, splits, stream);
    }
    return fail("gemm_tc: no token tile of %d", bn);
}

extern "C" {

const char* mdma_last_error() { return error_buffer(); }

// The wall-clock limit of every bounded wait of the kernels in this source (2 s unless changed).
int mdma_set_wait_limit_ns(unsigned long long ns) {
    MDMA_REQUIRE(ns > 0, "set_wait_limit: the limit must be positive");
    cudaError_t e = cudaMemcpyToSymbol(ptx::g_wait_limit_ns, &ns, sizeof(ns));
    if (e != cudaSuccess) return fail("set_wait_limit: %s", cudaGetErrorString(e));
    return 0;
}

// Launches the kernel that only waits (see wait_probe_kernel): mode 0 an mbarrier, mode 1 the flag.
int mdma_wait_probe(int mode, const int* flag, int* status, cudaStream_t stream) {
    MDMA_REQUIRE((mode == 0 || mode == 1) && status && (mode == 0 || flag), "wait_probe: bad arguments");
    wait_probe_kernel<<<1, 64, 0, stream>>>(mode, flag, status);
    MDMA_LAUNCH_OK("wait_probe");
    return 0;
}

// Returns 1 if the tensor-core kernel takes this weight shape.
int mdma_gemm_tc_supported(int n_features, int K) { return (K % 8 == 0 && K >= 8 && n_features >= 1) ? 1 : 0; }

// Bytes of float scratch a call with these sizes needs (0 when it does not split K).
// `splits` <= 0 asks the library to choose.
// `splits_out` < 0 means: split K that many ways inside a cluster (no scratch, reduced in shared memory).
int mdma_gemm_tc_plan(int mode, int n_tokens, int n_features, int K, int sm_count, int* bn_out, int* splits_out) {
    if (n_tokens > 128) {
        // Many tokens: block pairs, 256 features x 256 tokens per pair (`bn` code 512).  But with few
        // feature tiles and 129-512 tokens the pairs leave most of the device idle (the down product of 256
        // tokens: 16 pairs for 74 SM pairs, 87.6 us; O: 32.2 us): the one-block kernel with token tiles of 128
        // and a K split that gives every SM a block takes 50.1 us and 24.8 us there (512 tokens: 79.9 against
        // 89.1 us and 29.5 against 32.9 us).  Two weight matrices (SwiGLU) stay with the pairs (61 against 95 us).
        const long pair_tiles = (long)((n_features + 255) / 256) * ((n_tokens + 255) / 256);
        if (mode != kTcSwiGLU && n_tokens <= 512 && pair_tiles * 10 < (long)(sm_count / 2) * 6) {
            // Token tiles of 128, or of 256 where that puts more blocks on the SMs at once (O and down of 384
            // tokens: 64 tiles of 256 x 2 splits against 96 tiles of 128).  Not for a product that is stored
            // (QKV): alone it gains (256 tokens: 20.7 against 24.7 us with 3 splits), but the kernel that
            // rotates and stores then reads three float partial sums per value and the step loses more.
            const int k_blocks = (K + kBK - 1) / kBK;
            int best_bn = 128, best_splits = 1;
            long best_blocks = 0;
            for (int bn = 128; bn <= (mode == kTcAccumulate ? 256 : 128); bn *= 2) {
                const long tiles = (long)((n_features + kBM - 1) / kBM) * ((n_tokens + bn - 1) / bn);
                int splits = (int)(sm_count / tiles);
                if (splits > k_blocks / 4) splits = k_blocks / 4;
                if (splits < 1) splits = 1;
                // (as many blocks either way: one token tile of 256 with more splits for up to 192 tokens or a long K.
                // 160 tokens: down 32.4 against 38.4 us, O 14.7 against 15.8 us; 256 tokens: down 37.1 against 38.8 us,
                // but O 17.7 against 16.2 us)
                const bool tie_for_wide = bn == 256 && tiles * splits == best_blocks && (n_tokens <= 192 || K >= 8192);
                if ((tiles * splits > best_blocks || tie_for_wide) && tiles * splits <= sm_count) { best_blocks = tiles * splits; best_bn = bn; best_splits = splits; }
            }
            *bn_out = best_bn; *splits_out = best_splits; return 0;
        }
        *bn_out = 512; *splits_out = 1; return 0;
    }
    if (mode == kTcSwiGLU && n_tokens > 96) {
        // the gated product of 97-128 tokens: block pairs with one token tile (50.4 against 54.3 us at 128 tokens, 48.2
        // against 50.6 us at 96; below that one block per tile is faster); a decode step of 128 sequences: 6.41
        // against 6.51 ms
        *bn_out = 512; *splits_out = 1; return 0;
    }
    int bn = 16;
    while (bn < 256 && bn < n_tokens) bn *= 2;
    const int k_blocks = (K + kBK - 1) / kBK;
    const long tiles = (long)((n_features + kBM - 1) / kBM) * ((n_tokens + bn - 1) / bn);
    int splits = 1;
    if (mode == kTcSwiGLU && bn <= 32 && tiles < sm_count && k_blocks >= 8) {
        // The SwiGLU ending needs complete sums, so its K split stays inside a cluster of two blocks
        // (measured at batch 8: 37.4 us against 41.8 us unsplit; larger clusters and cluster splits
        // of the other products were slower than partial sums through global memory).  With 64 tokens
        // the partial sums are four times as large and one block per SM with a deep ring is faster
        // (44.4 us against 48.4 us).
        *bn_out = bn; *splits_out = -2; return 0;
    }
    if (mode != kTcSwiGLU && tiles < sm_count) {
        // As many blocks as can be resident at once, not more: two per SM for token tiles up to 64
        // (measured at the 8B decode shapes, 288 blocks beat 192 and 160, and anything beyond 296 is
        // slower again), one per SM for larger tiles, which take the whole shared memory (128 tokens:
        // QKV 14.5 us with 3 splits against 21.8 us with 6, O 12.3 against 19.5, down 26.9 against 34.8).
        splits = (int)(((bn <= 64 ? 2 : 1) * sm_count) / tiles);
        // A product that is stored (QKV) is followed by a kernel on the critical path that adds its partial sums
        // up itself (the decode attention with the rotary encoding inside, or the rotary kernel): fewer, 5/4 blocks
        // per SM.  Measured in the layer chain at the 8B shape, 4 splits against 6: batch 1 88.8 against 90.3 us,
        // batch 4 91.7 against 94.1, batch 8 93.5 against 95.6, batch 16 97.6 against 100.0; batch 32 and 64 the same.
        if (mode == kTcStore && bn <= 64) splits = (int)((5L * sm_count / 4 + tiles - 1) / tiles);
        if (splits < 1) splits = 1;
        if (splits > 16) splits = 16;
        if (splits > k_blocks / 4) splits = k_blocks / 4 > 0 ? k_blocks / 4 : 1;
    }
    *bn_out = bn;
    *splits_out = splits;
    return 0;
}

// Sums the partial results of a K split into `out` (mode store) or adds them to it (mode accumulate),
// in split order.
int mdma_splitk_reduce(int mode, const float* partial, int splits, int n_tokens, int n_features, void* out,
                       int ldo, int out_f32, cudaStream_t stream) {
    MDMA_REQUIRE(splits >= 1 && partial && out, "splitk_reduce: nothing to reduce");
    MDMA_REQUIRE(mode == kTcStore || mode == kTcAccumulate, "splitk_reduce: unknown mode %d", mode);
    const size_t total = (size_t)n_tokens * n_features;
    if (total == 0) return 0;
    const int blocks = (int)((total + 255) / 256);
    if (mode == kTcAccumulate)
        launch_chained(splitk_reduce_kernel<kTcAccumulate>, dim3(blocks), dim3(256), 0, stream, partial, splits, n_tokens, n_features, out, ldo, out_f32);
    else
        launch_chained(splitk_reduce_kernel<kTcStore>, dim3(blocks), dim3(256), 0, stream, partial, splits, n_tokens, n_features, out, ldo, out_f32);
    MDMA_LAUNCH_OK("splitk_reduce");
    return 0;
}

// `defer_reduce`: with a K split, leave the partial sums [splits, n_tokens, n_features] in `scratch`
// for the caller's next kernel to add up; `splits_used` reports how many there are (1: `out` is complete).
int mdma_gemm_tc(int mode, const void* x, int ldx, const void* w, const void* w2, void* out, int out_f32,
                 int ldo, int n_tokens, int n_features, int K, int bn, int splits, float* scratch,
                 long scratch_floats, int* status, int defer_reduce, int* splits_used, int* sk_flags,
                 const void* bias, const void* bias2, int bias_dtype, int act, cudaStream_t stream) {
    if (splits_used) *splits_used = 1;
    MDMA_REQUIRE(n_tokens >= 0 && n_features > 0 && K > 0, "gemm_tc: bad sizes");
    MDMA_REQUIRE(K % 8 == 0, "gemm_tc: K=%d is not a multiple of 8 (rows must be 16-byte multiples for TMA)", K);
    MDMA_REQUIRE(ldx % 8 == 0 && ldx >= K, "gemm_tc: activation pitch %d must be a multiple of 8 and at least K", ldx);
    MDMA_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && (!w2 || ((uintptr_t)w2 & 15) == 0),
                 "gemm_tc: operands must be 16-byte aligned");
    MDMA_REQUIRE(mode != kTcSwiGLU || w2, "gemm_tc: SwiGLU needs two weights");
    MDMA_REQUIRE(act == kActSilu || act == kActGeluTanh, "gemm_tc: unknown activation %d", act);
    MDMA_REQUIRE(bias_dtype == kF32 || bias_dtype == kBF16, "gemm_tc: unknown bias dtype %d", bias_dtype);
    const Ending ending{bias, mode == kTcSwiGLU ? bias2 : nullptr, bias_dtype, act};
    MDMA_REQUIRE(mode != kTcAccumulate || out_f32, "gemm_tc: the residual stream is float");
    MDMA_REQUIRE(mode >= 0 && mode <= 2, "gemm_tc: unknown mode %d", mode);
    MDMA_REQUIRE(bn == 512 || (n_tokens + bn - 1) / bn <= 65535, "gemm_tc: too many token tiles");
    if (n_tokens == 0) return 0;
    const int k_blocks = (K + kBK - 1) / kBK;
    if (splits < -1) {
        // K split inside a cluster
        int c = -splits;
        MDMA_REQUIRE(c <= 8, "gemm_tc: clusters of more than 8 blocks are not portable");
        if (c > k_blocks) c = k_blocks;
        TcParams pc;
        pc.out = out; pc.ldo = ldo; pc.out_f32 = out_f32;
        pc.n_tokens = n_tokens; pc.n_features = n_features; pc.k_blocks = k_blocks;
        pc.kb_per_split = (k_blocks + c - 1) / c;
        pc.partial = nullptr; pc.status = status; pc.cluster = c; pc.sk_partial = nullptr; pc.sk_flags = nullptr;
        pc.ending = ending;
        if (mode == kTcStore) return run_tc_bn<kTcStore>(bn, x, ldx, w, w2, K, pc, 1, stream);
        if (mode == kTcAccumulate) return run_tc_bn<kTcAccumulate>(bn, x, ldx, w, w2, K, pc, 1, stream);
        return run_tc_bn<kTcSwiGLU>(bn, x, ldx, w, w2, K, pc, 1, stream);
    }
    if (splits < 1) splits = 1;
    if (splits > k_blocks) splits = k_blocks;
    if (mode == kTcSwiGLU) splits = 1;
    TcParams p;
    p.out = out; p.ldo = ldo; p.out_f32 = out_f32;
    p.n_tokens = n_tokens; p.n_features = n_features; p.k_blocks = k_blocks;
    p.kb_per_split = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + p.kb_per_split - 1) / p.kb_per_split;     // no empty split
    p.partial = nullptr; p.status = status; p.cluster = 1; p.sk_partial = nullptr; p.sk_flags = nullptr;
    p.ending = ending;
    if (bn == 512) {           // the two-block kernel (a pair covers 256 features x 256 tokens)
        // scratch: one partial tile per block of every pair (accumulators x 256 x 128 floats each); the flags,
        // one per block, are zero between launches
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long part_floats = (long)sms * (mode == kTcSwiGLU ? 2 : 1) * 256 * 128;
        p.sk_partial = nullptr; p.sk_flags = nullptr;
        if (sk_flags != nullptr && scratch != nullptr && scratch_floats >= part_floats) { p.sk_partial = scratch; p.sk_flags = sk_flags; }
        if (mode == kTcStore) return run_tc2<kTcStore>(x, ldx, w, w2, K, p, stream);
        if (mode == kTcAccumulate) return run_tc2<kTcAccumulate>(x, ldx, w, w2, K, p, stream);
        return run_tc2<kTcSwiGLU>(x, ldx, w, w2, K, p, stream);
    }
    if (splits == 1) {
        if (mode == kTcStore) return run_tc_bn<kTcStore>(bn, x, ldx, w, w2, K, p, 1, stream);
        if (mode == kTcAccumulate) return run_tc_bn<kTcAccumulate>(bn, x, ldx, w, w2, K, p, 1, stream);
        return run_tc_bn<kTcSwiGLU>(bn, x, ldx, w, w2, K, p, 1, stream);
    }
    const long need = (long)splits * n_tokens * n_features;
    MDMA_REQUIRE(scratch && scratch_floats >= need, "gemm_tc: a %d-way K split needs %ld floats of scratch, %ld given", splits, need, scratch_floats);
    p.partial = scratch;
    if (int rc = run_tc_bn<kTcPartial>(bn, x, ldx, w, w2, K, p, splits, stream)) return rc;
    if (splits_used) *splits_used = splits;
    if (defer_reduce) return 0;
    return mdma_splitk_reduce(mode, scratch, splits, n_tokens, n_features, out, ldo, out_f32, stream);
}

}  // extern "C"
