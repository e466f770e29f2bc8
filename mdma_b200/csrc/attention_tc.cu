// Prefill attention on the fifth-generation tensor cores (bfloat16, paged cache,
// causal, optional window, grouped-query).
//
// A block owns 128 query rows of one kv head of one sequence: the rows are
// (token, query head of the group) pairs, token-major, so the G heads that share
// a kv head share its key and value tiles.  Keys and values come in blocks of 64 (one cache page):
//     S = Q K^T        tcgen05.mma, M=128, for TWO key blocks at once (N=128; a product instruction costs
//                      about a hundred cycles to issue whatever its width), operands from shared memory
//                      (TMA, 128-byte swizzle), accumulator in tensor memory (128 columns)
//     softmax          256 threads, two per query row (32 keys of a block each; the row maximum is exchanged
//                      through shared memory): tcgen05.ld of the half row, mask, running maximum and sum in
//                      float, P rounded to bfloat16 and written to shared memory in the operand layout
//     O += P V         tcgen05.mma accumulating in tensor memory, M=128, N=head_dim, V taken MN-major
//                      straight from the cache tile
// The probabilities are taken against a reference maximum that is only moved when the row's true
// maximum has grown by more than 2^8 since; only then is the accumulator in tensor memory rescaled
// (read, multiplied, written back), which happens in the first blocks of a row and hardly after.
// Roles: warp 0 issues TMA loads (Q once, K and V through rings of their own: a key stage is free after
// its S product, a value stage after its P V product, so keys are fetched a block pair ahead), warp 1
// issues the S products as soon as the softmax has read the pair before out of tensor memory, warp 10
// the P V products (one thread alone would spend longer issuing than the tensor pipe works), warps 2-9
// are the softmax.  Two blocks fit an SM, so one block's softmax runs under the other's MMAs.
// Every wait is bounded.
// Limits: head_dim a multiple of 16 up to 128, group size up to 128, page size a multiple of 64.
#include <cuda_fp16.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "ptx.cuh"

namespace mdma {

constexpr int kTcRows = 128, kTcKeys = 64, kTcThreadsA = 352, kKvStages = 2;

struct AttnTcParams {
    const int* seq_start; const int* seq_pos0; const int* seq_slot;
    const int* page_table; int max_pages; int page_size;
    __nv_bfloat16* out;
    int n_heads, n_kv_heads, head_dim, group, tile_tokens, window, n_tokens;
    float scale_log2;
    int* status;
};

// shared memory map (bytes), all tiles 1024-aligned:
//   Q: 2 halves x [128 rows x 128 B]           32 KB
//   K ring: stages x 2 halves x [64 x 128 B]   stages x 16 KB
//   V ring: same
//   P: [128 rows x 128 B]                      16 KB
constexpr int kQHalf = kTcRows * 128, kKvHalf = kTcKeys * 128, kPBuf = kTcRows * 128;
constexpr int kSmemQ = 0, kSmemK = 2 * kQHalf, kSmemV = kSmemK + kKvStages * 2 * kKvHalf,
              kSmemP = kSmemV + kKvStages * 2 * kKvHalf, kSmemBars = kSmemP + kPBuf,
              kSmemXch = kSmemBars + 256,          // the two halves of a row exchange their maxima here: 2 x 128 halves (16-bit)
              kAttnTcSmem = kSmemXch + 512;        // 112.75 KB: two blocks per SM (113 KB each at most)

__global__ void __launch_bounds__(kTcThreadsA, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const AttnTcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = ptx::smem_addr(smem_raw);
    uint8_t* base_ptr = smem_raw;
    const uint32_t bars = base + kSmemBars;
    // barriers: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full, s_read, p_ready, pv_done, then the
    // tensor-memory base word, the abort flag and the four pair barriers of the softmax warps
    const uint32_t q_full = bars;
    auto k_full = [&](int s) { return bars + 8u * (1 + s); };
    auto k_empty = [&](int s) { return bars + 8u * (3 + s); };
    auto v_full = [&](int s) { return bars + 8u * (5 + s); };
    auto v_empty = [&](int s) { return bars + 8u * (7 + s); };
    const uint32_t s_full = bars + 8u * 9, s_read = bars + 8u * 10;
    const uint32_t p_ready = bars + 8u * 11, pv_done = bars + 8u * 12;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + kSmemBars + 8 * 13);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + kSmemBars + 8 * 14);
    const uint32_t pair_bars = bars + 8u * 15;

    chain_release();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = blockIdx.y, kvh = blockIdx.x;
    if (threadIdx.x == 0) {
        if (base & 1023u) *abort_flag = 1;          // the tiles need 1024-byte alignment (checked again below)
        ptx::mbar_init(q_full, 1);
        for (int s = 0; s < kKvStages; ++s) {
            ptx::mbar_init(k_full(s), 1); ptx::mbar_init(k_empty(s), 1);
            ptx::mbar_init(v_full(s), 1); ptx::mbar_init(v_empty(s), 1);
        }
        ptx::mbar_init(s_full, 1);
        ptx::mbar_init(s_read, 256);
        ptx::mbar_init(p_ready, 256);
        for (int q = 0; q < 4; ++q) ptx::mbar_init(pair_bars + 8u * q, 64);    // the two softmax warps of 32 rows
        ptx::mbar_init(pv_done, 1);
        if (!(base & 1023u)) *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) { ptx::tmem_alloc(ptx::smem_addr((const void*)tmem_slot), 256); ptx::tmem_relinquish(); }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;     // S: 2 x 64 columns, O: 128 columns

    chain_wait();
    const int row0_seq = p.seq_start[seq];
    const int n_new = p.seq_start[seq + 1] - row0_seq;
    // late tiles see the most keys: they are handed out first so that the short ones fill the tail.  The
    // kv heads (and sequences) run fastest in the grid: blocks that run side by side then read different
    // keys and values (with the tiles of ONE head side by side, all on the same lines of L2, the kernel
    // took 72 us instead of 54 us for 2,048 tokens)
    const int tok0 = (int)(gridDim.z - 1 - blockIdx.z) * p.tile_tokens;
    const bool active = tok0 < n_new && !(base & 1023u);      // uniform over the block
    const int n_tok = active ? min(p.tile_tokens, n_new - tok0) : 0;
    const int pos0 = p.seq_pos0[seq] + tok0;
    const int last_pos = pos0 + n_tok - 1;
    const int D = p.head_dim, G = p.group;
    const int first_key = p.window > 0 ? max(0, pos0 + 1 - p.window) : 0;
    const int b0 = first_key / kTcKeys, b1 = active ? last_pos / kTcKeys + 1 : b0;
    const int nb = b1 - b0;
    const int halves = (D + 63) / 64;

    if (active && warp == 0 && lane == 0) {
        // ---- TMA producer ---------------------------------------------------------
        const int* pages = p.page_table + (size_t)p.seq_slot[seq] * p.max_pages;
        ptx::mbar_expect_tx(q_full, halves * G * p.tile_tokens * 128);      // the box is G x tile_tokens rows of 128 bytes
        for (int h = 0; h < halves; ++h)
            ptx::tma_load_4d(base + kSmemQ + h * kQHalf, &map_q, q_full, h * 64, kvh * G, row0_seq + tok0, 0);
        // S is computed for two key blocks at once (below), so the two key stages are filled and freed
        // together; a value stage is free after its own P V product.  The loads are issued in the order in
        // which their stages come free: K0 K1 V0 V1 | K2 K3 (S of blocks 0,1 done) V2 (P V 0 done) |
        // K4 K5 (S 2,3) V3 (P V 1) V4 (P V 2) | K6 K7 V5 V6 | ...
        // Key tiles lie [half of head_dim][stage][64 keys x 128 bytes]: the two stages of a half are one
        // operand of 128 rows.
        auto load_k = [&](int i) -> bool {
            if (i >= nb) return true;
            const int s = i % kKvStages;
            if (!ptx::mbar_wait(k_empty(s), ((i / kKvStages) & 1) ^ 1, abort_flag)) return false;
            const int key0 = (b0 + i) * kTcKeys;
            const int page = pages[key0 / p.page_size], row = key0 % p.page_size;
            ptx::mbar_expect_tx(k_full(s), halves * kKvHalf);
            for (int h = 0; h < halves; ++h)
                ptx::tma_load_4d(base + kSmemK + (h * kKvStages + s) * kKvHalf, &map_k, k_full(s), h * 64, kvh, row, page);
            return true;
        };
        auto load_v = [&](int i) -> bool {
            if (i >= nb) return true;
            const int s = i % kKvStages;
            if (!ptx::mbar_wait(v_empty(s), ((i / kKvStages) & 1) ^ 1, abort_flag)) return false;
            const int key0 = (b0 + i) * kTcKeys;
            const int page = pages[key0 / p.page_size], row = key0 % p.page_size;
            ptx::mbar_expect_tx(v_full(s), halves * kKvHalf);
            for (int h = 0; h < halves; ++h)
                ptx::tma_load_4d(base + kSmemV + (s * 2 + h) * kKvHalf, &map_v, v_full(s), h * 64, kvh, row, page);
            return true;
        };
        bool fine = load_k(0) && load_k(1) && load_v(0) && load_v(1) && load_k(2) && load_k(3) && load_v(2);
        for (int jp = 1; fine && 2 * jp + 1 < nb; ++jp)
            fine = load_k(2 * jp + 2) && load_k(2 * jp + 3) && load_v(2 * jp + 1) && load_v(2 * jp + 2);
    } else if (active && warp == 1 && lane == 0) {
        // ---- MMA issuer -------------------------------------------------------------
        const uint32_t idesc_s = ptx::idesc_bf16_f32_ex(kTcRows, kTcKeys, 0);
        const uint32_t idesc_s2 = ptx::idesc_bf16_f32_ex(kTcRows, 2 * kTcKeys, 0);
        // S of the blocks 2 jp and 2 jp + 1 in one chain of products (N = 128; N = 64 for a last single
        // block): a product instruction costs about the same whatever its width, so fewer, wider ones.
        auto issue_s_pair = [&](int jp) {
            const bool both = 2 * jp + 1 < nb;
            for (int kd = 0; kd < D / 16; ++kd) {
                const uint32_t qa = base + kSmemQ + (kd / 4) * kQHalf + (kd % 4) * 32;
                const uint32_t kb = base + kSmemK + (kd / 4) * kKvStages * kKvHalf + (kd % 4) * 32;
                ptx::mma_bf16_ss(tmem_s, ptx::smem_desc_sw128(qa), ptx::smem_desc_sw128(kb), both ? idesc_s2 : idesc_s, kd > 0);
            }
            ptx::mma_commit(s_full);
            ptx::mma_commit(k_empty(0));                  // the key stages are free once these products are done
            if (both) ptx::mma_commit(k_empty(1));
        };
        // The next pair of S is issued as soon as the softmax has read the second block of this pair out of
        // tensor memory.  The P V products are issued by another warp (below): a product instruction
        // takes about a hundred cycles to issue from one thread whatever its size, and so does a wait, so one
        // thread alone would spend longer issuing than the tensor pipe works.
        bool ok = ptx::mbar_wait(q_full, 0, abort_flag);
        const int n_pairs = (nb + 1) / 2;
        for (int jp = 0; jp < n_pairs && ok; ++jp) {
            ok = ptx::mbar_wait(k_full(0), jp & 1, abort_flag) && (2 * jp + 1 >= nb || ptx::mbar_wait(k_full(1), jp & 1, abort_flag));
            if (ok && jp > 0) ok = ptx::mbar_wait(s_read, (jp - 1) & 1, abort_flag);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            issue_s_pair(jp);
        }
    } else if (active && warp == 10 && lane == 0) {
        // ---- second MMA issuer: O += P(i) V(i), K dimension = keys ----------------------
        const uint32_t idesc_o = ptx::idesc_bf16_f32_ex(kTcRows, D, 1);
        for (int i = 0; i < nb; ++i) {
            const int s = i % kKvStages;
            if (!(ptx::mbar_wait(v_full(s), (i / kKvStages) & 1, abort_flag) && ptx::mbar_wait(p_ready, i & 1, abort_flag))) break;
            ptx::tc_fence_after_sync();
            for (int kk = 0; kk < kTcKeys / 16; ++kk) {
                const uint32_t pa = base + kSmemP + kk * 32;
                const uint32_t vb = base + kSmemV + (s * 2) * kKvHalf + kk * 16 * 128;
                ptx::mma_bf16_ss(tmem_o, ptx::smem_desc_sw128(pa), ptx::smem_desc_sw128_mn(vb, kKvHalf), idesc_o,
                                 (i > 0 || kk > 0) ? 1u : 0u);
            }
            ptx::mma_commit(pv_done);
            ptx::mma_commit(v_empty(s));
        }
    } else if (active && warp >= 2 && warp < 10) {
        // ---- softmax: two threads per query row, 32 keys of a block each ------------------
        const int quad = warp & 3, half = (warp - 2) >> 2;
        const int r = quad * 32 + lane;                       // row of the tile = TMEM lane
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const int t = r / G, g = r % G;
        const bool row_valid = t < n_tok;
        const int pos = pos0 + (row_valid ? t : n_tok - 1);
        const int win = p.window > 0 ? pos + 1 - p.window : 0;
        float m_ref = -INFINITY, l = 0.f;                     // reference maximum (log2 domain), this half's running sum
        uint8_t* p_row = base_ptr + kSmemP + (size_t)r * 128;
        // The reference maximum need not be the exact maximum (it lags by up to 2^8 anyway), only the same
        // in both threads of a row: each rounds its own to 16 bits, both take the larger of the two.
        __half* xch = reinterpret_cast<__half*>(base_ptr + kSmemXch);    // [2 halves][128 rows]
        bool ok = true;
        // the two warps that share 32 rows meet on a barrier of their own (bounded like every wait here)
        const uint32_t pair_bar = pair_bars + 8u * quad;
        uint32_t pair_phase = 0;
        auto pair_sync = [&]() -> bool {
            ptx::mbar_arrive(pair_bar);
            const bool fine = __all_sync(0xffffffffu, ptx::mbar_wait(pair_bar, pair_phase & 1u, abort_flag));
            ++pair_phase;
            return fine;
        };
        for (int i = 0; i < nb && ok; ++i) {
            ok = __all_sync(0xffffffffu, ptx::mbar_wait(s_full, (i >> 1) & 1, abort_flag));   // whole warps go on or stop
            if (!ok) break;
            ptx::tc_fence_after_sync();
            float sv[32];
            ptx::tmem_load_32_nowait(tmem_s + (i & 1) * 64 + half * 32 + lane_base, sv);
            ptx::tmem_load_wait();
            ptx::tc_fence_before_sync();
            if (i & 1) ptx::mbar_arrive(s_read);              // both blocks of the pair are in registers: S may be overwritten
            const int key0 = (b0 + i) * kTcKeys + half * 32;
            const bool need_mask = key0 + 31 > pos || key0 < win;
            if (need_mask) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (key0 + j > pos || key0 + j < win) sv[j] = -INFINITY;
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 32; ++j) m4[j & 3] = fmaxf(m4[j & 3], sv[j]);
            const __half mine = __float2half_rn(fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2);   // scale > 0
            // the row's maximum over both halves (the first barrier: the other warp has read the last block's)
            if (!(ok = pair_sync())) break;
            xch[half * 128 + r] = mine;
            if (!(ok = pair_sync())) break;
            const float mx = fmaxf(__half2float(mine), __half2float(xch[(half ^ 1) * 128 + r]));
            // move the reference only when the maximum has grown by more than 2^8 (or at the first keys)
            float corr = 1.f;
            bool moved = false;
            if (mx > m_ref + 8.f) {
                corr = m_ref == -INFINITY ? 0.f : ptx::ex2_approx(m_ref - mx);
                m_ref = mx;
                moved = true;
            }
            const float ref = m_ref == -INFINITY ? 0.f : m_ref;
            float s4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float p0 = ptx::ex2_approx(fmaf(sv[2 * j], p.scale_log2, -ref));
                const float p1 = ptx::ex2_approx(fmaf(sv[2 * j + 1], p.scale_log2, -ref));
                s4[j & 3] += p0 + p1;
                __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
                pk[j] = *reinterpret_cast<uint32_t*>(&b2);
            }
            l = l * corr + ((s4[0] + s4[1]) + (s4[2] + s4[3]));
            // P(i-1) V(i-1) must be done before P is overwritten and before O is rescaled
            if (i > 0) {
                ok = __all_sync(0xffffffffu, ptx::mbar_wait(pv_done, (i - 1) & 1, abort_flag));
                if (!ok) break;
                ptx::tc_fence_after_sync();
                if (__any_sync(0xffffffffu, moved)) {          // rare: rescale this warp's rows of O (its column chunks)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        if ((c & 1) == half && c * 32 < D) {
                            float v[32];
                            ptx::tmem_load_32_nowait(tmem_o + lane_base + c * 32, v);
                            ptx::tmem_load_wait();
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] *= corr;
                            ptx::tmem_store_32_nowait(tmem_o + lane_base + c * 32, v);
                        }
                    }
                    ptx::tmem_store_wait();
                }
            }
            {
                // Value rows of keys that no row of this tile may see (beyond its last position, before its
                // window) belong to nobody: stale rows of an earlier sequence, possibly not finite.  Their
                // probabilities are zero, but 0 * NaN is NaN, so the rows are cleared in shared memory before
                // the product reads them.  Only the first and the last key block of a tile have any.
                const int kb0 = (b0 + i) * kTcKeys;
                if (kb0 + kTcKeys - 1 > last_pos || kb0 < first_key) {
                    const int vs = i % kKvStages;
                    ok = __all_sync(0xffffffffu, ptx::mbar_wait(v_full(vs), (i / kKvStages) & 1, abort_flag));
                    if (!ok) break;
                    const int tid = (warp - 2) * 32 + lane;
                    for (int e = tid; e < halves * kTcKeys * 8; e += 256) {
                        const int h = e / (kTcKeys * 8), kr = (e >> 3) % kTcKeys, c = e & 7;
                        if (kb0 + kr > last_pos || kb0 + kr < first_key)
                            *reinterpret_cast<uint4*>(base_ptr + kSmemV + (vs * 2 + h) * kKvHalf + kr * 128 + c * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {    // this half's 32 bf16 = 4 chunks of 16 bytes; chunk c of the row sits at c ^ (row & 7)
                const int cc = half * 4 + c;
                *reinterpret_cast<uint4*>(p_row + ((cc ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            }
            ptx::fence_proxy_async_shared();
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(p_ready);
        }
        if (ok && nb > 0) ok = __all_sync(0xffffffffu, ptx::mbar_wait(pv_done, (nb - 1) & 1, abort_flag));
        if (ok && nb > 0) {
            ptx::tc_fence_after_sync();
            // the row's sum over both halves, through the same words (128 floats: one a row)
            float* x = reinterpret_cast<float*>(xch);
            ok = pair_sync();                                  // the last maxima have been read
            if (half == 1) x[r] = l;
            ok = ok && pair_sync();
            float total = l;
            if (half == 0) { total = l + x[r]; x[r] = total; }
            ok = ok && pair_sync();
            if (half == 1) total = x[r];
            const float inv = 1.0f / total;
            __nv_bfloat16* dst = p.out + ((size_t)(row0_seq + tok0 + (row_valid ? t : 0)) * p.n_heads + kvh * G + g) * D;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if ((c & 1) == half && c * 32 < D) {
                    float v[32];
                    ptx::tmem_load_32_nowait(tmem_o + lane_base + c * 32, v);
                    ptx::tmem_load_wait();
                    if (row_valid) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (c * 32 + q * 8 < D) {
                                uint32_t w[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    __nv_bfloat162 b2 = __floats2bfloat162_rn(v[q * 8 + 2 * j] * inv, v[q * 8 + 2 * j + 1] * inv);
                                    w[j] = *reinterpret_cast<uint32_t*>(&b2);
                                }
                                *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        }
                    }
                }
            }
            ptx::tc_fence_before_sync();
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) { ptx::tc_fence_after_sync(); ptx::tmem_dealloc(tmem_base, 256); }
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 2);
}

// ---- tensor maps -----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn attn_encode_fn() {
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

// A bf16 tensor [d3][d2][d1][d0] (d0 innermost) with byte strides s1..s3, box (64, b1, b2, 1), 128-byte swizzle.
static int make_map_4d(CUtensorMap* out, const void* ptr, const uint64_t dims[4], const uint64_t strides[3],
                       const uint32_t box[4]) {
    EncodeTiledFn fn = attn_encode_fn();
    if (!fn) return fail("attention_tc: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
    cuuint64_t s[3] = {strides[0], strides[1], strides[2]};
    cuuint32_t b[4] = {box[0], box[1], box[2], box[3]};
    cuuint32_t e[4] = {1, 1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), d, s, b, e,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail("attention_tc: cuTensorMapEncodeTiled failed with %d (dims %llu %llu %llu %llu)", (int)r,
                    (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2], (unsigned long long)dims[3]);
    return 0;
}

}  // namespace mdma

using namespace mdma;

extern "C" {

int mdma_attention_tc_supported(int n_heads, int n_kv_heads, int head_dim, int page_size) {
    if (n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
    const int g = n_heads / n_kv_heads;
    return (head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 128 && g <= kTcRows && page_size % kTcKeys == 0) ? 1 : 0;
}

// q: rows of the fused projection [tokens_cap, row_width], queries first; caches [pages, page_size, kv_heads, head_dim].
int mdma_attention_tc(const void* q, int q_stride, int q_rows_cap, const void* k_cache, const void* v_cache,
                      int n_pages, const int* seq_start, const int* seq_pos0, const int* seq_slot,
                      const int* page_table, int max_pages, int page_size, void* out, int n_tokens, int n_seqs,
                      int max_new, int n_heads, int n_kv_heads, int head_dim, int window, float scale,
                      int* status, cudaStream_t stream) {
    MDMA_REQUIRE(mdma_attention_tc_supported(n_heads, n_kv_heads, head_dim, page_size),
                 "attention_tc: heads %d / kv heads %d / head_dim %d / page %d is outside its limits", n_heads, n_kv_heads, head_dim, page_size);
    MDMA_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0, "attention_tc: query rows must be 16-byte aligned");
    MDMA_REQUIRE(scale > 0.f, "attention_tc: the score scale must be positive");
    MDMA_REQUIRE(n_seqs <= 65535 && n_kv_heads <= 65535, "attention_tc: grid too large");
    if (n_tokens == 0 || n_seqs == 0) return 0;
    const int G = n_heads / n_kv_heads;
    AttnTcParams p;
    p.seq_start = seq_start; p.seq_pos0 = seq_pos0; p.seq_slot = seq_slot;
    p.page_table = page_table; p.max_pages = max_pages; p.page_size = page_size;
    p.out = (__nv_bfloat16*)out; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim;
    p.group = G; p.tile_tokens = kTcRows / G; p.window = window; p.n_tokens = n_tokens;
    p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    CUtensorMap mq, mk, mv;
    {   // queries: [tokens][heads][head_dim] inside rows of q_stride elements; box = 64 x G x tile_tokens
        const uint64_t dims[4] = {(uint64_t)head_dim, (uint64_t)n_heads, (uint64_t)n_tokens, 1};
        const uint64_t strides[3] = {(uint64_t)head_dim * 2, (uint64_t)q_stride * 2, (uint64_t)q_stride * 2 * (uint64_t)q_rows_cap};
        const uint32_t box[4] = {64, (uint32_t)G, (uint32_t)p.tile_tokens, 1};
        if (int rc = make_map_4d(&mq, q, dims, strides, box)) return rc;
    }
    {
        const uint64_t dims[4] = {(uint64_t)head_dim, (uint64_t)n_kv_heads, (uint64_t)page_size, (uint64_t)n_pages};
        const uint64_t strides[3] = {(uint64_t)head_dim * 2, (uint64_t)n_kv_heads * head_dim * 2,
                                     (uint64_t)page_size * n_kv_heads * head_dim * 2};
        const uint32_t box[4] = {64, 1, (uint32_t)kTcKeys, 1};
        if (int rc = make_map_4d(&mk, k_cache, dims, strides, box)) return rc;
        if (int rc = make_map_4d(&mv, v_cache, dims, strides, box)) return rc;
    }
    static bool once = false;
    if (!once) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnTcSmem);
        if (e != cudaSuccess) return fail("attention_tc: cannot reserve %d bytes of shared memory: %s", kAttnTcSmem, cudaGetErrorString(e));
        once = true;
    }
    dim3 grid(n_kv_heads, n_seqs, (max_new + p.tile_tokens - 1) / p.tile_tokens);
    cudaError_t e = launch_chained(attention_tc_kernel, grid, dim3(kTcThreadsA), kAttnTcSmem, stream, mq, mk, mv, p);
    if (e != cudaSuccess) return fail("attention_tc: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

}  // extern "C"
