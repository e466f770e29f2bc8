// Causal grouped-query attention over the paged cache on the tensor cores
// (bfloat16 in, float softmax and accumulation), for prefill and for decode.
//
// A block works on one tile of query rows of one kv head of one sequence.  The
// rows of a tile are (token, query head of the group) pairs, token-major, so
// the G query heads that share a kv head share its key and value loads: a
// prefill tile holds 64/G tokens, a decode tile one token.  Keys and values
// stream through shared memory in blocks of 64 (double-buffered cp.async,
// looked up page by page), scores and the running maximum and sum stay in
// registers in float, probabilities are rounded to bfloat16 for the P*V
// product, as is usual.  With `splits` > 1 the key blocks of a tile are divided
// among that many blocks of the grid; each writes its unnormalised output with
// its maximum and sum, and a second kernel merges them in split order, so the
// result does not depend on timing.
// Limits: head_dim a multiple of 16 up to 128; group size up to 64.
#pragma once
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace mdma {

constexpr int kRows = 64;        // query rows per block (4 warps x 16)
constexpr int kKeys = 64;        // keys per block of the stream
constexpr int kAttnThreads = 128;

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;       // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct AttnParams {
    const __nv_bfloat16* q; int q_stride;          // rows of the fused projection; queries first
    const __nv_bfloat16* k_cache; const __nv_bfloat16* v_cache;   // [pages, page_size, kv_heads, head_dim]
    const int* seq_start; const int* seq_pos0; const int* seq_slot;
    const int* page_table; int max_pages; int page_size;
    __nv_bfloat16* out;                             // [tokens, heads * head_dim]
    float* part_o; float* part_ml;                  // split partials: [tokens, heads, splits, head_dim], [.., 2]
    int n_heads, n_kv_heads, head_dim, group, tile_tokens, window, splits;
    float scale_log2;                               // scale * log2(e)
    int* status;                                    // optional device word, set non-zero if a wait ran out
    // Decode with the rotary encoding done here (`rot_inv_freq` not null): the step's projection rows are
    // `q` (bfloat16, not yet rotated) or, with `proj_splits` > 0, the sum of that many float partial rows
    // [split][token][proj_width]; the block rotates its query heads and its key head, rounds them to
    // bfloat16, writes the key and the value to the cache row of the token's position and uses them from
    // shared memory, so that no tile it fetches depends on the kernel before it.
    const float* rot_inv_freq; int rotary_dim; int rot_interleaved;
    const float* proj_partial; int proj_splits; long proj_split_stride; int proj_width;
    __nv_bfloat16* k_cache_w; __nv_bfloat16* v_cache_w;
};

// Tile shared-memory rows are DMAX elements wide; 16-byte chunk c of row r sits at chunk c ^ (r & 7).
template <int DMAX>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
    return (uint32_t)(row * DMAX * 2 + ((chunk ^ (row & 7)) << 4));
}

template <int DMAX>
__global__ void __launch_bounds__(kAttnThreads)
attention_mma_kernel(const AttnParams p) {
    constexpr int kChunks = DMAX / 8;              // 16-byte chunks per row
    constexpr int kTile = kRows * DMAX * 2;        // bytes of one 64-row tile
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t sK = sQ + kTile, sV = sK + 2 * kTile;

    chain_release();
    chain_wait();
    const int seq = blockIdx.y;
    const int kvh = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
    const int row0_seq = p.seq_start[seq];
    const int n_new = p.seq_start[seq + 1] - row0_seq;
    const int tok0 = blockIdx.x * p.tile_tokens;            // first token of this tile within the sequence's new tokens
    if (tok0 >= n_new) return;
    const int n_tok = min(p.tile_tokens, n_new - tok0);
    const int pos0 = p.seq_pos0[seq] + tok0;                // position of the tile's first token
    const int last_pos = pos0 + n_tok - 1;
    const int* pages = p.page_table + (size_t)p.seq_slot[seq] * p.max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = p.head_dim, G = p.group;
    const int d_chunks = D / 8;

    // key range of the tile, then of this split
    const int first_key = p.window > 0 ? max(0, pos0 + 1 - p.window) : 0;
    const int blk_lo = first_key / kKeys, blk_hi = last_pos / kKeys + 1;
    const int per = (blk_hi - blk_lo + p.splits - 1) / p.splits;
    const int b0 = blk_lo + split * per, b1 = min(blk_hi, b0 + per);

    // ---- Q tile -> shared -------------------------------------------------
    for (int i = threadIdx.x; i < kRows * kChunks; i += kAttnThreads) {
        const int r = i / kChunks, c = i % kChunks;
        const int t = r / G, g = r % G;
        const bool valid = t < n_tok && c < d_chunks;
        const __nv_bfloat16* src = p.q + (size_t)(row0_seq + tok0 + (valid ? t : 0)) * p.q_stride +
                                   (size_t)(kvh * G + g) * D + (valid ? c : 0) * 8;
        cp_async_16(sQ + tile_offset<DMAX>(r, c), src, valid);
    }
    auto load_kv = [&](int blk, int stage) {
        for (int i = threadIdx.x; i < kKeys * kChunks; i += kAttnThreads) {
            const int r = i / kChunks, c = i % kChunks;
            const int key = blk * kKeys + r;
            // keys outside [first_key, last_pos] are zero-filled, never read: their cache rows may be stale
            // (another sequence's, or not finite) and 0 * NaN would reach the output through P V
            const bool valid = key <= last_pos && key >= first_key && c < d_chunks;
            size_t off = 0;
            if (valid) {
                const int page = pages[key / p.page_size];
                off = (((size_t)page * p.page_size + key % p.page_size) * p.n_kv_heads + kvh) * D + c * 8;
            }
            cp_async_16(sK + stage * kTile + tile_offset<DMAX>(r, c), p.k_cache + off, valid);
            cp_async_16(sV + stage * kTile + tile_offset<DMAX>(r, c), p.v_cache + off, valid);
        }
    };
    if (b0 < b1) load_kv(b0, 0);
    cp_async_commit();

    // per-thread rows: r_lo = warp*16 + lane/4, r_hi = r_lo + 8
    const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
    const int pos_lo = pos0 + min(r_lo / G, n_tok - 1), pos_hi = pos0 + min(r_hi / G, n_tok - 1);
    const int win_lo = p.window > 0 ? pos_lo + 1 - p.window : 0, win_hi = p.window > 0 ? pos_hi + 1 - p.window : 0;

    float o[DMAX / 8][4];
#pragma unroll
    for (int n = 0; n < DMAX / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    for (int blk = b0; blk < b1; ++blk) {
        const int stage = (blk - b0) & 1;
        if (blk + 1 < b1) load_kv(blk + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        // ---- S = Q K^T for this warp's 16 rows x 64 keys ---------------------
        float s[kKeys / 8][4];
#pragma unroll
        for (int n = 0; n < kKeys / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
        for (int kd = 0; kd < DMAX / 16; ++kd) {
            if (kd * 16 < D) {
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4(sQ + tile_offset<DMAX>(warp * 16 + (lane & 15), kd * 2 + (lane >> 4)), a0, a1, a2, a3);
#pragma unroll
                for (int n2 = 0; n2 < kKeys / 16; ++n2) {
                    uint32_t k0, k1, k2, k3;
                    // matrices: (keys 0-7, d lo), (keys 0-7, d hi), (keys 8-15, d lo), (keys 8-15, d hi)
                    const int krow = n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
                    ldmatrix_x4(sK + stage * kTile + tile_offset<DMAX>(krow, kd * 2 + ((lane >> 3) & 1)), k0, k1, k2, k3);
                    mma_16816(s[n2 * 2], a0, a1, a2, a3, k0, k1);
                    mma_16816(s[n2 * 2 + 1], a0, a1, a2, a3, k2, k3);
                }
            }
        }
        // ---- mask, online softmax ---------------------------------------------
        const int key_base = blk * kKeys + (lane & 3) * 2;
        float mx_lo = m_lo, mx_hi = m_hi;
#pragma unroll
        for (int n = 0; n < kKeys / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key_base + n * 8 + e;
                const float v_lo = (key <= pos_lo && key >= win_lo) ? s[n][e] * p.scale_log2 : -INFINITY;
                const float v_hi = (key <= pos_hi && key >= win_hi) ? s[n][2 + e] * p.scale_log2 : -INFINITY;
                s[n][e] = v_lo; s[n][2 + e] = v_hi;
                mx_lo = fmaxf(mx_lo, v_lo); mx_hi = fmaxf(mx_hi, v_hi);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        // a row with no visible key yet keeps m = -inf; use 0 as its reference so that exp2(-inf - 0) = 0
        const float ref_lo = mx_lo == -INFINITY ? 0.f : mx_lo, ref_hi = mx_hi == -INFINITY ? 0.f : mx_hi;
        const float corr_lo = exp2f(m_lo - ref_lo), corr_hi = exp2f(m_hi - ref_hi);
        m_lo = mx_lo; m_hi = mx_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
        uint32_t pa[kKeys / 16][4];
#pragma unroll
        for (int n = 0; n < kKeys / 8; ++n) {
            const float p0 = exp2f(s[n][0] - ref_lo), p1 = exp2f(s[n][1] - ref_lo);
            const float p2 = exp2f(s[n][2] - ref_hi), p3 = exp2f(s[n][3] - ref_hi);
            sum_lo += p0 + p1; sum_hi += p2 + p3;
            pa[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
            pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_lo = l_lo * corr_lo + sum_lo; l_hi = l_hi * corr_hi + sum_hi;
#pragma unroll
        for (int n = 0; n < DMAX / 8; ++n) {
            o[n][0] *= corr_lo; o[n][1] *= corr_lo; o[n][2] *= corr_hi; o[n][3] *= corr_hi;
        }
        // ---- O += P V -----------------------------------------------------------
#pragma unroll
        for (int kk = 0; kk < kKeys / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < DMAX / 16; ++n2) {
                if (n2 * 16 < D) {
                    uint32_t v0, v1, v2, v3;
                    // transposed loads: (keys lo, d lo), (keys hi, d lo), (keys lo, d hi), (keys hi, d hi)
                    const int vrow = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    ldmatrix_x4_trans(sV + stage * kTile + tile_offset<DMAX>(vrow, n2 * 2 + (lane >> 4)), v0, v1, v2, v3);
                    mma_16816(o[n2 * 2], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], v0, v1);
                    mma_16816(o[n2 * 2 + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], v2, v3);
                }
            }
        }
        __syncthreads();        // the stage may be overwritten by the next iteration's loads
    }
    cp_async_wait<0>();

    // ---- finish: row sums across the quad, then write ----------------------------
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = half ? r_hi : r_lo;
        const int t = r / G, g = r % G;
        if (t >= n_tok) continue;
        const float l = half ? l_hi : l_lo, m = half ? m_hi : m_lo;
        const size_t token = (size_t)(row0_seq + tok0 + t);
        const int head = kvh * G + g;
        if (p.splits == 1) {
            const float inv = 1.0f / l;
            __nv_bfloat16* dst = p.out + (token * p.n_heads + head) * D;
#pragma unroll
            for (int n = 0; n < DMAX / 8; ++n) {
                const int d = n * 8 + (lane & 3) * 2;
                if (d < D)
                    *reinterpret_cast<__nv_bfloat162*>(dst + d) =
                        __floats2bfloat162_rn(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
            }
        } else {
            const size_t slot = (token * p.n_heads + head) * p.splits + split;
            float* dst = p.part_o + slot * D;
#pragma unroll
            for (int n = 0; n < DMAX / 8; ++n) {
                const int d = n * 8 + (lane & 3) * 2;
                if (d < D) { dst[d] = o[n][half * 2]; dst[d + 1] = o[n][half * 2 + 1]; }
            }
            if ((lane & 3) == 0) { p.part_ml[slot * 2] = m; p.part_ml[slot * 2 + 1] = l; }
        }
    }
}

// ---------------------------------------------------------------------------
// Decode: every sequence brings one token.  The G query heads of a kv head are
// the (up to 16) rows of one MMA tile, so nothing is computed for padding rows
// beyond that tile.  A block of four warps works on one (sequence, kv head,
// split); its warps take the key blocks of the split in turn (warp w: blocks
// w, w+4, ...), each with its own running maximum, sum and output, loading its
// keys and values into a private shared-memory buffer (K of the next block is
// fetched while P*V of this one runs).  At the end the four states are combined
// through shared memory in warp order and written as the final output or as
// this split's partial.  Tiles of 32 keys keep a block's shared memory small
// enough for three blocks per SM, which is what hides the load latency.
constexpr int kDecodeKeys = 32;
template <int DMAX, int KB>      // KB: keys per warp tile
__global__ void __launch_bounds__(kAttnThreads, 3)
attention_decode_kernel(const AttnParams p) {
    constexpr int kChunks = DMAX / 8;
    constexpr int kTile = KB * DMAX * 2;             // one 64-key K or V tile
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t s0 = (uint32_t)__cvta_generic_to_shared(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t sQ = s0;                              // 16 rows x DMAX
    const uint32_t sK = s0 + 16 * DMAX * 2 + warp * 2 * kTile, sV = sK + kTile;

    chain_release();
    chain_wait();
    const int seq = blockIdx.y;
    const int kvh = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
    const int token = p.seq_start[seq];
    const int pos = p.seq_pos0[seq];
    const int* pages = p.page_table + (size_t)p.seq_slot[seq] * p.max_pages;
    const int D = p.head_dim, G = p.group, d_chunks = D / 8;
    const int first_key = p.window > 0 ? max(0, pos + 1 - p.window) : 0;
    const int blk_lo = first_key / KB, blk_hi = pos / KB + 1;
    const int per = (blk_hi - blk_lo + p.splits - 1) / p.splits;
    const int b0 = blk_lo + split * per, b1 = min(blk_hi, b0 + per);
    const bool page_aligned = (p.page_size % KB) == 0;

    // Q rows (heads of the group) -> shared, zero beyond G and beyond D
    for (int i = threadIdx.x; i < 16 * kChunks; i += kAttnThreads) {
        const int r = i / kChunks, c = i % kChunks;
        const bool valid = r < G && c < d_chunks;
        const __nv_bfloat16* src = p.q + (size_t)token * p.q_stride + (size_t)(kvh * G + (valid ? r : 0)) * D + (valid ? c : 0) * 8;
        cp_async_16(sQ + tile_offset<DMAX>(r, c), src, valid);
    }
    auto load_tile = [&](const __nv_bfloat16* cache, uint32_t dst, int blk) {
        size_t base = 0;
        if (page_aligned) {
            const int key0 = blk * KB;
            base = ((size_t)pages[key0 / p.page_size] * p.page_size + key0 % p.page_size) * p.n_kv_heads;
        }
#pragma unroll 4
        for (int i = lane; i < KB * kChunks; i += 32) {
            const int r = i / kChunks, c = i % kChunks;
            const int key = blk * KB + r;
            const bool valid = key <= pos && key >= first_key && c < d_chunks;      // rows outside are zero-filled
            size_t off = 0;
            if (valid) {
                if (page_aligned) off = ((base + (size_t)r * p.n_kv_heads) + kvh) * D + c * 8;
                else off = (((size_t)pages[key / p.page_size] * p.page_size + key % p.page_size) * p.n_kv_heads + kvh) * D + c * 8;
            }
            cp_async_16(dst + tile_offset<DMAX>(r, c), cache + off, valid);
        }
    };
    int blk = b0 + warp;
    if (blk < b1) load_tile(p.k_cache, sK, blk);
    cp_async_commit();                                   // group: Q (+ first K)
    if (blk < b1) load_tile(p.v_cache, sV, blk);
    cp_async_commit();                                   // group: first V
    cp_async_wait<1>();
    __syncthreads();                                     // Q visible to all warps

    uint32_t qf[DMAX / 16][4];
#pragma unroll
    for (int kd = 0; kd < DMAX / 16; ++kd)
        ldmatrix_x4(sQ + tile_offset<DMAX>(lane & 15, kd * 2 + (lane >> 4)), qf[kd][0], qf[kd][1], qf[kd][2], qf[kd][3]);

    const int win = p.window > 0 ? pos + 1 - p.window : 0;
    float o[DMAX / 8][4];
#pragma unroll
    for (int n = 0; n < DMAX / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    for (; blk < b1; blk += 4) {
        cp_async_wait<1>();                              // this block's K has landed (its V may be in flight)
        __syncwarp();
        float s[KB / 8][4];
#pragma unroll
        for (int n = 0; n < KB / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
        for (int kd = 0; kd < DMAX / 16; ++kd) {
            if (kd * 16 < D) {
#pragma unroll
                for (int n2 = 0; n2 < KB / 16; ++n2) {
                    uint32_t k0, k1, k2, k3;
                    const int krow = n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
                    ldmatrix_x4(sK + tile_offset<DMAX>(krow, kd * 2 + ((lane >> 3) & 1)), k0, k1, k2, k3);
                    mma_16816(s[n2 * 2], qf[kd][0], qf[kd][1], qf[kd][2], qf[kd][3], k0, k1);
                    mma_16816(s[n2 * 2 + 1], qf[kd][0], qf[kd][1], qf[kd][2], qf[kd][3], k2, k3);
                }
            }
        }
        __syncwarp();
        const bool more = blk + 4 < b1;
        if (more) load_tile(p.k_cache, sK, blk + 4);     // K buffer is free: fetch the next block's keys
        cp_async_commit();
        const int key_base = blk * KB + (lane & 3) * 2;
        float mx_lo = m_lo, mx_hi = m_hi;
#pragma unroll
        for (int n = 0; n < KB / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key_base + n * 8 + e;
                const bool vis = key <= pos && key >= win;
                const float v_lo = vis ? s[n][e] * p.scale_log2 : -INFINITY;
                const float v_hi = vis ? s[n][2 + e] * p.scale_log2 : -INFINITY;
                s[n][e] = v_lo; s[n][2 + e] = v_hi;
                mx_lo = fmaxf(mx_lo, v_lo); mx_hi = fmaxf(mx_hi, v_hi);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float ref_lo = mx_lo == -INFINITY ? 0.f : mx_lo, ref_hi = mx_hi == -INFINITY ? 0.f : mx_hi;
        const float corr_lo = exp2f(m_lo - ref_lo), corr_hi = exp2f(m_hi - ref_hi);
        m_lo = mx_lo; m_hi = mx_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
        uint32_t pa[KB / 16][4];
#pragma unroll
        for (int n = 0; n < KB / 8; ++n) {
            const float p0 = exp2f(s[n][0] - ref_lo), p1 = exp2f(s[n][1] - ref_lo);
            const float p2 = exp2f(s[n][2] - ref_hi), p3 = exp2f(s[n][3] - ref_hi);
            sum_lo += p0 + p1; sum_hi += p2 + p3;
            pa[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
            pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_lo = l_lo * corr_lo + sum_lo; l_hi = l_hi * corr_hi + sum_hi;
#pragma unroll
        for (int n = 0; n < DMAX / 8; ++n) {
            o[n][0] *= corr_lo; o[n][1] *= corr_lo; o[n][2] *= corr_hi; o[n][3] *= corr_hi;
        }
        cp_async_wait<1>();                              // this block's V has landed (next K may be in flight)
        __syncwarp();
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < DMAX / 16; ++n2) {
                if (n2 * 16 < D) {
                    uint32_t v0, v1, v2, v3;
                    const int vrow = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    ldmatrix_x4_trans(sV + tile_offset<DMAX>(vrow, n2 * 2 + (lane >> 4)), v0, v1, v2, v3);
                    mma_16816(o[n2 * 2], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], v0, v1);
                    mma_16816(o[n2 * 2 + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], v2, v3);
                }
            }
        }
        __syncwarp();
        if (more) load_tile(p.v_cache, sV, blk + 4);
        cp_async_commit();
    }
    cp_async_wait<0>();
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    // ---- combine the four warps' states in warp order ---------------------------
    // layout in shared memory (reusing the tiles): per warp [16 rows][DMAX + 2] floats
    __syncthreads();
    float* comb = reinterpret_cast<float*>(smem);
    constexpr int kRowF = DMAX + 2;
    {
        float* mine = comb + (size_t)warp * 16 * kRowF;
        const int r_lo = lane >> 2, r_hi = r_lo + 8;
#pragma unroll
        for (int n = 0; n < DMAX / 8; ++n) {
            const int d = n * 8 + (lane & 3) * 2;
            mine[r_lo * kRowF + d] = o[n][0]; mine[r_lo * kRowF + d + 1] = o[n][1];
            mine[r_hi * kRowF + d] = o[n][2]; mine[r_hi * kRowF + d + 1] = o[n][3];
        }
        if ((lane & 3) == 0) {
            mine[r_lo * kRowF + DMAX] = m_lo; mine[r_lo * kRowF + DMAX + 1] = l_lo;
            mine[r_hi * kRowF + DMAX] = m_hi; mine[r_hi * kRowF + DMAX + 1] = l_hi;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * D; i += kAttnThreads) {
        const int r = i / D, d = i % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, comb[((size_t)w * 16 + r) * kRowF + DMAX]);
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = comb[((size_t)w * 16 + r) * kRowF + DMAX];
            if (mw != -INFINITY) {
                const float f = exp2f(mw - m);
                l += f * comb[((size_t)w * 16 + r) * kRowF + DMAX + 1];
                acc += f * comb[((size_t)w * 16 + r) * kRowF + d];
            }
        }
        const int head = kvh * G + r;
        if (p.splits == 1) {
            p.out[((size_t)token * p.n_heads + head) * D + d] = __float2bfloat16_rn(acc / l);
        } else {
            const size_t slot = ((size_t)token * p.n_heads + head) * p.splits + split;
            p.part_o[slot * D + d] = acc;
            if (d == 0) { p.part_ml[slot * 2] = m; p.part_ml[slot * 2 + 1] = l; }
        }
    }
}

// The same kernel with the key and value tiles fetched by TMA (one elected lane per warp issues a
// tile load, completion on the warp's own mbarrier) instead of 16-byte cp.async copies, whose address
// arithmetic was two thirds of the instructions.  Needs page_size to be a multiple of KB.  A tile is
// stored as halves of 64 head elements: [KB keys x 128 bytes] with the 128-byte swizzle.
// NW warps per block.  All blocks should run at once (a second, short round of blocks costs as
// much as the first): eight warps and one block per SM while the blocks are no more than the SMs, else
// four, three or two warps with three, four or five blocks per SM, or one warp with ten.
template <int DMAX, int KB, int NW>
__global__ void __launch_bounds__(NW * 32, NW == 8 ? 1 : NW == 4 ? 3 : NW == 3 ? 4 : NW == 2 ? 5 : 10)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const AttnParams p) {
    constexpr int kChunks = DMAX / 8;
    constexpr int kHalf = KB * 128;                      // one half tile: KB keys x 64 elements
    constexpr int kTile = KB * DMAX * 2;                 // a K or V tile (DMAX/64 halves)
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t s0 = (uint32_t)__cvta_generic_to_shared(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t sK = s0 + warp * 2 * kTile, sV = sK + kTile;      // tiles first: they need 1024-byte alignment
    const uint32_t sQ = s0 + NW * 2 * kTile;              // 16 rows x DMAX
    const uint32_t bars = sQ + 16 * DMAX * 2;
    const uint32_t kbar = bars + warp * 16, vbar = kbar + 8;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + NW * 2 * kTile + 16 * DMAX * 2 + NW * 16);
    // with the rotary encoding done here: this token's rotated key and its value (bfloat16), sines and cosines
    constexpr int kFreshOff = NW * 2 * kTile + 16 * DMAX * 2 + NW * 16 + 64;
    __nv_bfloat16* fresh_k = reinterpret_cast<__nv_bfloat16*>(smem + kFreshOff);
    __nv_bfloat16* fresh_v = fresh_k + DMAX;
    float* sincos = reinterpret_cast<float*>(smem + kFreshOff + 4 * DMAX);
    const bool fused = p.rot_inv_freq != nullptr;
    auto kv_offset = [](int row, int chunk) -> uint32_t {      // 16-byte chunk of a key row inside a tile
        return (uint32_t)((chunk >> 3) * kHalf + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
    };
    if (threadIdx.x == 0) {
        for (int w = 0; w < NW; ++w) { ptx::mbar_init(bars + w * 16, 1); ptx::mbar_init(bars + w * 16 + 8, 1); }
        *abort_flag = (s0 & 1023u) ? 1 : 0;
        ptx::fence_mbar_init();
    }

    chain_release();
    // Positions, slots and page tables were written before this step's kernels began, and the keys
    // and values of earlier positions before that: only the row of this step's own token (in the last
    // tile) and the queries come from the kernel before this one.  So every warp whose first tile
    // is not the last one asks for it before waiting for that kernel.
    __syncthreads();                                     // the barriers exist
    const int seq = blockIdx.y;
    const int kvh = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
    const int token = p.seq_start[seq];
    const int pos = p.seq_pos0[seq];
    const int* pages = p.page_table + (size_t)p.seq_slot[seq] * p.max_pages;
    const int D = p.head_dim, G = p.group, d_chunks = D / 8;
    const int first_key = p.window > 0 ? max(0, pos + 1 - p.window) : 0;
    const int blk_lo = first_key / KB, blk_hi = pos / KB + 1;
    const int per = (blk_hi - blk_lo + p.splits - 1) / p.splits;
    const int b0 = blk_lo + split * per, b1 = min(blk_hi, b0 + per);
    const int halves = (D + 63) / 64;

    auto load_tile = [&](const CUtensorMap* map, uint32_t dst, uint32_t bar, int blk) {      // one lane
        const int key0 = blk * KB;
        const int page = pages[key0 / p.page_size], row = key0 % p.page_size;
        ptx::fence_proxy_async_shared();
        ptx::mbar_expect_tx(bar, halves * kHalf);
        for (int h = 0; h < halves; ++h) ptx::tma_load_4d(dst + h * kHalf, map, bar, h * 64, kvh, row, page);
    };
    int blk = b0 + warp;
    if (*abort_flag != 0) blk = b1;
    // (with the rotary encoding done here the row of the own token is replaced in shared memory, so
    // the last tile does not depend on the kernel before either)
    const bool early = blk < b1 && (fused || blk != blk_hi - 1);
    if (early && lane == 0) { load_tile(&map_k, sK, kbar, blk); load_tile(&map_v, sV, vbar, blk); }
    if (fused) {
        // sines and cosines of this position (no dependence on the kernel before); the Q tile starts as zeros
        const int half = p.rotary_dim / 2;
        for (int i = threadIdx.x; i < half; i += NW * 32) {
            float sn, cs;
            sincosf((float)pos * p.rot_inv_freq[i], &sn, &cs);
            sincos[i] = sn; sincos[half + i] = cs;
        }
        for (int i = threadIdx.x; i < 16 * kChunks; i += NW * 32)
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(sQ + i * 16), "r"(0u) : "memory");
    }
    chain_wait();
    if (!early && blk < b1 && lane == 0) { load_tile(&map_k, sK, kbar, blk); load_tile(&map_v, sV, vbar, blk); }
    if (fused) {
        __syncthreads();                                 // sines, cosines and the zeroed tile are in place
        const int half = p.rotary_dim / 2, tail = D - p.rotary_dim;
        const __nv_bfloat16* row = p.q + (size_t)token * p.q_stride;
        const float* prow = p.proj_partial + (size_t)token * p.proj_width;
        auto load = [&](int col) -> float {              // the projection's value: as stored, or its partial sums in split order
            if (p.proj_splits == 0) return __bfloat162float(row[col]);
            float a = 0.f;
            int sidx = 0;
            for (; sidx + 4 <= p.proj_splits; sidx += 4) {       // four loads in flight, added in order
                const float* src = prow + (size_t)sidx * p.proj_split_stride + col;
                const float v0 = __ldcg(src), v1 = __ldcg(src + p.proj_split_stride),
                            v2 = __ldcg(src + 2 * p.proj_split_stride), v3 = __ldcg(src + 3 * p.proj_split_stride);
                a += v0; a += v1; a += v2; a += v3;
            }
            for (; sidx < p.proj_splits; ++sidx) a += __ldcg(prow + (size_t)sidx * p.proj_split_stride + col);
            return a;
        };
        uint8_t* q_tile = smem + NW * 2 * kTile;
        auto q_elem = [&](int r, int d) -> __nv_bfloat16* {
            return reinterpret_cast<__nv_bfloat16*>(q_tile + tile_offset<DMAX>(r, d >> 3) + (d & 7) * 2);
        };
        const int q_col0 = kvh * G * D, k_col0 = (p.n_heads + kvh) * D, v_col0 = (p.n_heads + p.n_kv_heads + kvh) * D;
        for (int i = threadIdx.x; i < (G + 1) * half; i += NW * 32) {        // the G query heads, then the key head
            const int r = i / half, pr = i % half;
            const int d0 = p.rot_interleaved ? 2 * pr : pr, d1 = p.rot_interleaved ? 2 * pr + 1 : pr + half;
            const int col = r < G ? q_col0 + r * D : k_col0;
            const float x0 = load(col + d0), x1 = load(col + d1);
            const float sn = sincos[pr], cs = sincos[half + pr];
            const __nv_bfloat16 y0 = __float2bfloat16_rn(x0 * cs - x1 * sn), y1 = __float2bfloat16_rn(x0 * sn + x1 * cs);
            if (r < G) { *q_elem(r, d0) = y0; *q_elem(r, d1) = y1; }
            else { fresh_k[d0] = y0; fresh_k[d1] = y1; }
        }
        for (int i = threadIdx.x; i < (G + 1) * tail; i += NW * 32) {        // beyond the rotated width: as it is
            const int r = i / tail, d = p.rotary_dim + i % tail;
            const __nv_bfloat16 y = __float2bfloat16_rn(load((r < G ? q_col0 + r * D : k_col0) + d));
            if (r < G) *q_elem(r, d) = y; else fresh_k[d] = y;
        }
        for (int i = threadIdx.x; i < D; i += NW * 32) fresh_v[i] = __float2bfloat16_rn(load(v_col0 + i));
        __syncthreads();
        // the block that holds the last tile keeps the token's key and value for later steps
        if (b1 == blk_hi && b0 < b1 && threadIdx.x < 2 * d_chunks) {
            const int which = threadIdx.x / d_chunks, c = threadIdx.x % d_chunks;
            const size_t cache_row = (((size_t)pages[pos / p.page_size] * p.page_size + pos % p.page_size) * p.n_kv_heads + kvh) * D;
            __nv_bfloat16* dst = (which ? p.v_cache_w : p.k_cache_w) + cache_row + c * 8;
            *reinterpret_cast<uint4*>(dst) = reinterpret_cast<const uint4*>(which ? fresh_v : fresh_k)[c];
        }
    } else {
        // Q rows (heads of the group) -> shared, zero beyond G and beyond D
        for (int i = threadIdx.x; i < 16 * kChunks; i += NW * 32) {
            const int r = i / kChunks, c = i % kChunks;
            const bool valid = r < G && c < d_chunks;
            const __nv_bfloat16* src = p.q + (size_t)token * p.q_stride + (size_t)(kvh * G + (valid ? r : 0)) * D + (valid ? c : 0) * 8;
            cp_async_16(sQ + tile_offset<DMAX>(r, c), src, valid);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();                                 // Q is visible to all warps
    }
    uint32_t phase = 0;

    uint32_t qf[DMAX / 16][4];
#pragma unroll
    for (int kd = 0; kd < DMAX / 16; ++kd)
        ldmatrix_x4(sQ + tile_offset<DMAX>(lane & 15, kd * 2 + (lane >> 4)), qf[kd][0], qf[kd][1], qf[kd][2], qf[kd][3]);

    const int win = p.window > 0 ? pos + 1 - p.window : 0;
    float o[DMAX / 8][4];
#pragma unroll
    for (int n = 0; n < DMAX / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    for (; blk < b1; blk += NW) {
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(kbar, phase, abort_flag))) break;     // this tile's K has landed
        const bool own_tile = fused && blk == blk_hi - 1;      // the tile of the token's own position
        if (own_tile) {
            if (lane < d_chunks)
                *reinterpret_cast<uint4*>(smem + (sK - s0) + kv_offset(pos - blk * KB, lane)) = reinterpret_cast<const uint4*>(fresh_k)[lane];
            __syncwarp();
        }
        float s[KB / 8][4];
#pragma unroll
        for (int n = 0; n < KB / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
        for (int kd = 0; kd < DMAX / 16; ++kd) {
            if (kd * 16 < D) {
#pragma unroll
                for (int n2 = 0; n2 < KB / 16; ++n2) {
                    uint32_t k0, k1, k2, k3;
                    const int krow = n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
                    ldmatrix_x4(sK + kv_offset(krow, kd * 2 + ((lane >> 3) & 1)), k0, k1, k2, k3);
                    mma_16816(s[n2 * 2], qf[kd][0], qf[kd][1], qf[kd][2], qf[kd][3], k0, k1);
                    mma_16816(s[n2 * 2 + 1], qf[kd][0], qf[kd][1], qf[kd][2], qf[kd][3], k2, k3);
                }
            }
        }
        __syncwarp();
        const bool more = blk + NW < b1;
        if (more && lane == 0) load_tile(&map_k, sK, kbar, blk + NW);     // K buffer is free: fetch the next tile's keys
        const int key_base = blk * KB + (lane & 3) * 2;
        float mx_lo = m_lo, mx_hi = m_hi;
#pragma unroll
        for (int n = 0; n < KB / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key_base + n * 8 + e;
                const bool vis = key <= pos && key >= win;
                const float v_lo = vis ? s[n][e] * p.scale_log2 : -INFINITY;
                const float v_hi = vis ? s[n][2 + e] * p.scale_log2 : -INFINITY;
                s[n][e] = v_lo; s[n][2 + e] = v_hi;
                mx_lo = fmaxf(mx_lo, v_lo); mx_hi = fmaxf(mx_hi, v_hi);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float ref_lo = mx_lo == -INFINITY ? 0.f : mx_lo, ref_hi = mx_hi == -INFINITY ? 0.f : mx_hi;
        const float corr_lo = exp2f(m_lo - ref_lo), corr_hi = exp2f(m_hi - ref_hi);
        m_lo = mx_lo; m_hi = mx_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
        uint32_t pa[KB / 16][4];
#pragma unroll
        for (int n = 0; n < KB / 8; ++n) {
            const float p0 = exp2f(s[n][0] - ref_lo), p1 = exp2f(s[n][1] - ref_lo);
            const float p2 = exp2f(s[n][2] - ref_hi), p3 = exp2f(s[n][3] - ref_hi);
            sum_lo += p0 + p1; sum_hi += p2 + p3;
            pa[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
            pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_lo = l_lo * corr_lo + sum_lo; l_hi = l_hi * corr_hi + sum_hi;
#pragma unroll
        for (int n = 0; n < DMAX / 8; ++n) {
            o[n][0] *= corr_lo; o[n][1] *= corr_lo; o[n][2] *= corr_hi; o[n][3] *= corr_hi;
        }
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(vbar, phase, abort_flag))) break;     // this tile's V has landed
        {
            // A tile is fetched whole.  Rows of keys outside [first_key, pos] belong to nobody (stale rows of
            // an earlier sequence, possibly not finite): their probabilities are zero, but 0 * NaN is NaN, so
            // their value rows are cleared before the product.  Only the first and the last tile have any.
            const int r_lo = first_key - blk * KB, r_hi = pos - blk * KB;      // rows [r_lo, r_hi] are real
            if (r_lo > 0 || r_hi < KB - 1) {
                for (int i = lane; i < halves * KB * 8; i += 32) {
                    const int h = i / (KB * 8), r = (i >> 3) % KB, c = i & 7;
                    if (r < r_lo || r > r_hi)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(sV + h * kHalf + r * 128 + c * 16), "r"(0u) : "memory");
                }
                __syncwarp();
            }
            if (own_tile) {
                if (lane < d_chunks)
                    *reinterpret_cast<uint4*>(smem + (sV - s0) + kv_offset(pos - blk * KB, lane)) = reinterpret_cast<const uint4*>(fresh_v)[lane];
                __syncwarp();
            }
        }
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < DMAX / 16; ++n2) {
                if (n2 * 16 < D) {
                    uint32_t v0, v1, v2, v3;
                    const int vrow = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    ldmatrix_x4_trans(sV + kv_offset(vrow, n2 * 2 + (lane >> 4)), v0, v1, v2, v3);
                    mma_16816(o[n2 * 2], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], v0, v1);
                    mma_16816(o[n2 * 2 + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], v2, v3);
                }
            }
        }
        __syncwarp();
        if (more && lane == 0) load_tile(&map_v, sV, vbar, blk + NW);
        phase ^= 1u;
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    // ---- combine the four warps' states in warp order ---------------------------
    // layout in shared memory (reusing the tiles): per warp [16 rows][DMAX + 2] floats
    __syncthreads();
    float* comb = reinterpret_cast<float*>(smem);
    constexpr int kRowF = DMAX + 2;
    {
        float* mine = comb + (size_t)warp * 16 * kRowF;
        const int r_lo = lane >> 2, r_hi = r_lo + 8;
#pragma unroll
        for (int n = 0; n < DMAX / 8; ++n) {
            const int d = n * 8 + (lane & 3) * 2;
            mine[r_lo * kRowF + d] = o[n][0]; mine[r_lo * kRowF + d + 1] = o[n][1];
            mine[r_hi * kRowF + d] = o[n][2]; mine[r_hi * kRowF + d + 1] = o[n][3];
        }
        if ((lane & 3) == 0) {
            mine[r_lo * kRowF + DMAX] = m_lo; mine[r_lo * kRowF + DMAX + 1] = l_lo;
            mine[r_hi * kRowF + DMAX] = m_hi; mine[r_hi * kRowF + DMAX + 1] = l_hi;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * D; i += NW * 32) {
        const int r = i / D, d = i % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) m = fmaxf(m, comb[((size_t)w * 16 + r) * kRowF + DMAX]);
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float mw = comb[((size_t)w * 16 + r) * kRowF + DMAX];
            if (mw != -INFINITY) {
                const float f = exp2f(mw - m);
                l += f * comb[((size_t)w * 16 + r) * kRowF + DMAX + 1];
                acc += f * comb[((size_t)w * 16 + r) * kRowF + d];
            }
        }
        const int head = kvh * G + r;
        if (p.splits == 1) {
            p.out[((size_t)token * p.n_heads + head) * D + d] = __float2bfloat16_rn(acc / l);
        } else {
            const size_t slot = ((size_t)token * p.n_heads + head) * p.splits + split;
            p.part_o[slot * D + d] = acc;
            if (d == 0) { p.part_ml[slot * 2] = m; p.part_ml[slot * 2 + 1] = l; }
        }
    }
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 4);
}

// out[token, head, :] = sum_s 2^(m_s - m) O_s / sum_s 2^(m_s - m) l_s, splits taken in order.
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       __nv_bfloat16* __restrict__ out, int splits, int head_dim) {
    chain_release();
    chain_wait();
    const size_t th = blockIdx.x;                   // token * heads + head
    const float* ml = part_ml + th * splits * 2;
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, ml[s * 2]);
    float l = 0.f;
    for (int s = 0; s < splits; ++s) if (ml[s * 2] != -INFINITY) l += exp2f(ml[s * 2] - m) * ml[s * 2 + 1];
    const float inv = 1.0f / l;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s)
            if (ml[s * 2] != -INFINITY) acc += exp2f(ml[s * 2] - m) * part_o[(th * splits + s) * head_dim + d];
        out[th * head_dim + d] = __float2bfloat16_rn(acc * inv);
    }
}


// Checks the geometry, launches the attention kernel and, for splits > 1, the merge.
// `scratch` holds the split partials; the caller owns it.
static inline int attention_mma_supported(int n_heads, int n_kv_heads, int head_dim) {
    if (n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
    const int g = n_heads / n_kv_heads;
    return (head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 128 && g <= kRows) ? 1 : 0;
}
static inline long attention_mma_scratch_floats(int n_tokens, int n_heads, int head_dim, int splits) {
    return splits > 1 ? (long)n_tokens * n_heads * splits * (head_dim + 2) : 0;
}

typedef CUresult (*AttnEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// A tensor map over a cache [pages, page_size, kv_heads, head_dim] with boxes of 64 elements x 1 head x
// `box_keys` keys x 1 page (128-byte swizzle).
static int make_cache_map(CUtensorMap* out, const void* cache, int n_pages, int page_size, int n_kv_heads,
                          int head_dim, int box_keys) {
    static AttnEncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<AttnEncodeTiledFn>(sym);
    });
    if (!fn) return fail("attention: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)n_kv_heads, (cuuint64_t)page_size, (cuuint64_t)n_pages};
    cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2, (cuuint64_t)n_kv_heads * head_dim * 2,
                             (cuuint64_t)page_size * n_kv_heads * head_dim * 2};
    cuuint32_t box[4] = {64, 1, (cuuint32_t)box_keys, 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(cache), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("attention: cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
}

// The rotary encoding and the cache write done inside the decode kernel (see AttnParams).
struct FusedRotary {
    const float* inv_freq; int rotary_dim; int interleaved;
    const float* partial; int splits; long split_stride; int width;      // K-split partial sums of the projection, or none
};
// Whether a decode step with these sizes can take the fused form (it needs the tile loads by TMA).
static inline int attention_fused_rotary_supported(int n_heads, int n_kv_heads, int head_dim, int page_size, int rotary_dim) {
    if (!attention_mma_supported(n_heads, n_kv_heads, head_dim)) return 0;
    return (n_heads / n_kv_heads <= 16 && page_size % 32 == 0 && rotary_dim % 2 == 0 && rotary_dim >= 2 &&
            rotary_dim <= head_dim && head_dim % 8 == 0) ? 1 : 0;
}

// `n_pages` > 0 tells how many pages the caches hold and lets the decode kernel fetch tiles by TMA.
static int launch_attention_mma(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                       const int* seq_start, const int* seq_pos0, const int* seq_slot, const int* page_table,
                       int max_pages, int page_size, void* out, int n_tokens, int n_seqs, int max_new,
                       int n_heads, int n_kv_heads, int head_dim, int window, float scale, int splits,
                       float* scratch, long scratch_floats, cudaStream_t stream, int n_pages = 0,
                       int* status = nullptr, const FusedRotary* fz = nullptr) {
    MDMA_REQUIRE(attention_mma_supported(n_heads, n_kv_heads, head_dim),
                 "attention_mma: heads %d / kv heads %d / head_dim %d is outside its limits (head_dim a multiple of 16 up to 128, group up to 64)",
                 n_heads, n_kv_heads, head_dim);
    MDMA_REQUIRE(page_table && page_size > 0 && max_pages > 0 && window >= 0, "attention_mma: bad cache geometry");
    MDMA_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0, "attention_mma: query rows must be 16-byte aligned");
    MDMA_REQUIRE(n_seqs <= 65535 && (long)n_kv_heads * splits <= 65535, "attention_mma: grid too large");
    if (n_tokens == 0 || n_seqs == 0) return 0;
    if (splits < 1) splits = 1;
    AttnParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
    p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
    p.seq_start = seq_start; p.seq_pos0 = seq_pos0; p.seq_slot = seq_slot;
    p.page_table = page_table; p.max_pages = max_pages; p.page_size = page_size;
    p.out = (__nv_bfloat16*)out;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim;
    p.group = n_heads / n_kv_heads; p.tile_tokens = kRows / p.group; p.window = window; p.splits = splits;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.part_o = nullptr; p.part_ml = nullptr; p.status = status;
    p.rot_inv_freq = nullptr; p.rotary_dim = 0; p.rot_interleaved = 0;
    p.proj_partial = nullptr; p.proj_splits = 0; p.proj_split_stride = 0; p.proj_width = 0;
    p.k_cache_w = nullptr; p.v_cache_w = nullptr;
    if (fz != nullptr) {
        MDMA_REQUIRE(max_new == 1 && n_pages > 0 && attention_fused_rotary_supported(n_heads, n_kv_heads, head_dim, page_size, fz->rotary_dim),
                     "attention: the rotary encoding can be done inside the kernel only for single tokens, page sizes that are multiples of 32 and groups up to 16");
        MDMA_REQUIRE(fz->inv_freq && (fz->splits == 0 || fz->partial), "attention: the fused rotary encoding needs its frequency table (and the partial sums it names)");
        p.rot_inv_freq = fz->inv_freq; p.rotary_dim = fz->rotary_dim; p.rot_interleaved = fz->interleaved;
        p.proj_partial = fz->partial; p.proj_splits = fz->partial ? fz->splits : 0;
        p.proj_split_stride = fz->split_stride; p.proj_width = fz->width;
        p.k_cache_w = (__nv_bfloat16*)const_cast<void*>(k_cache); p.v_cache_w = (__nv_bfloat16*)const_cast<void*>(v_cache);
    }
    if (splits > 1) {
        const long need = attention_mma_scratch_floats(n_tokens, n_heads, head_dim, splits);
        MDMA_REQUIRE(scratch && scratch_floats >= need, "attention_mma: %d splits need %ld floats of scratch, %ld given", splits, need, scratch_floats);
        p.part_o = scratch;
        p.part_ml = scratch + (long)n_tokens * n_heads * splits * head_dim;
    }
    dim3 grid((max_new + p.tile_tokens - 1) / p.tile_tokens, n_seqs, n_kv_heads * splits);
    const bool tma_ok = n_pages > 0 && page_size % kDecodeKeys == 0 && ((uintptr_t)k_cache & 15) == 0 &&
                        ((uintptr_t)v_cache & 15) == 0;
    MDMA_REQUIRE(fz == nullptr || tma_ok, "attention: the caches are not aligned for tile loads");
    if (max_new == 1 && p.group <= 16 && tma_ok) {
        // one token per sequence, tiles by TMA
        // heads of up to 64 elements take tiles of 64 keys when the pages allow: a tile of 32 such keys is
        // 4 KB, too little for what a tile costs (the same 8 KB per tile as for heads of 128 then)
        const int kb = (head_dim <= 64 && page_size % 64 == 0) ? 64 : kDecodeKeys;
        CUtensorMap mk, mv;
        if (int rc = make_cache_map(&mk, k_cache, n_pages, page_size, n_kv_heads, head_dim, kb)) return rc;
        if (int rc = make_cache_map(&mv, v_cache, n_pages, page_size, n_kv_heads, head_dim, kb)) return rc;
        auto launch = [&](auto kernel, int nw, int dmax) -> int {
            const int bytes = nw * 2 * kb * dmax * 2 + 16 * dmax * 2 + nw * 16 + 64 + 8 * dmax;
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
            if (e != cudaSuccess) return fail("attention: cannot reserve %d bytes of shared memory: %s", bytes, cudaGetErrorString(e));
            e = launch_chained(kernel, grid, dim3(nw * 32), bytes, stream, mk, mv, p);
            if (e != cudaSuccess) return fail("attention: launch failed: %s", cudaGetErrorString(e));
            return 0;
        };
        int rc;
        // few blocks: eight warps each (one block per SM); many: four warps and three blocks per SM
        int sm_count = 0, dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        // the most warps per block with which every block of the grid is resident at once
        const long blocks = (long)n_seqs * n_kv_heads * splits;
        // (up to ten blocks per SM: one warp each.  128 sequences x 8 kv heads at context 580, with the rotary kernel
        // before it: 64.0 us against 77.8 us in two and a bit rounds of four-warp blocks; 184 sequences 88.0 against
        // 98.8 us.  Beyond that, rounds of four-warp blocks: 192 sequences 99.0 us against 110.7 us with one warp)
        const int nw = blocks <= sm_count ? 8 : blocks <= 3l * sm_count ? 4 : blocks <= 4l * sm_count ? 3 :
                       blocks <= 5l * sm_count ? 2 : blocks <= 10l * sm_count ? 1 : 4;
        if (kb == 64) {
            rc = nw == 8 ? launch(attention_decode_tma_kernel<64, 64, 8>, 8, 64)
               : nw == 4 ? launch(attention_decode_tma_kernel<64, 64, 4>, 4, 64)
               : nw == 3 ? launch(attention_decode_tma_kernel<64, 64, 3>, 3, 64)
               : nw == 2 ? launch(attention_decode_tma_kernel<64, 64, 2>, 2, 64)
                         : launch(attention_decode_tma_kernel<64, 64, 1>, 1, 64);
        } else if (head_dim <= 64) {
            rc = nw == 8 ? launch(attention_decode_tma_kernel<64, kDecodeKeys, 8>, 8, 64)
               : nw == 4 ? launch(attention_decode_tma_kernel<64, kDecodeKeys, 4>, 4, 64)
               : nw == 3 ? launch(attention_decode_tma_kernel<64, kDecodeKeys, 3>, 3, 64)
               : nw == 2 ? launch(attention_decode_tma_kernel<64, kDecodeKeys, 2>, 2, 64)
                         : launch(attention_decode_tma_kernel<64, kDecodeKeys, 1>, 1, 64);
        } else {
            rc = nw == 8 ? launch(attention_decode_tma_kernel<128, kDecodeKeys, 8>, 8, 128)
               : nw == 4 ? launch(attention_decode_tma_kernel<128, kDecodeKeys, 4>, 4, 128)
               : nw == 3 ? launch(attention_decode_tma_kernel<128, kDecodeKeys, 3>, 3, 128)
               : nw == 2 ? launch(attention_decode_tma_kernel<128, kDecodeKeys, 2>, 2, 128)
                         : launch(attention_decode_tma_kernel<128, kDecodeKeys, 1>, 1, 128);
        }
        if (rc) return rc;
    } else if (max_new == 1 && p.group <= 16) {
        // one token per sequence: the decode kernel (no padding rows beyond one 16-row tile)
        if (head_dim <= 64) {
            constexpr int bytes = 16 * 64 * 2 + 4 * 2 * kDecodeKeys * 64 * 2;
            cudaFuncSetAttribute(attention_decode_kernel<64, kDecodeKeys>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);      // per launch: the attribute belongs to the current device
            launch_chained(attention_decode_kernel<64, kDecodeKeys>, grid, dim3(kAttnThreads), bytes, stream, p);
        } else {
            constexpr int bytes = 16 * 128 * 2 + 4 * 2 * kDecodeKeys * 128 * 2;
            cudaFuncSetAttribute(attention_decode_kernel<128, kDecodeKeys>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);      // per launch: the attribute belongs to the current device
            launch_chained(attention_decode_kernel<128, kDecodeKeys>, grid, dim3(kAttnThreads), bytes, stream, p);
        }
    } else if (head_dim <= 64) {
        constexpr int bytes = 5 * kRows * 64 * 2;
        cudaFuncSetAttribute(attention_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);      // per launch: the attribute belongs to the current device
        launch_chained(attention_mma_kernel<64>, grid, dim3(kAttnThreads), bytes, stream, p);
    } else {
        constexpr int bytes = 5 * kRows * 128 * 2;
        cudaFuncSetAttribute(attention_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);      // per launch: the attribute belongs to the current device
        launch_chained(attention_mma_kernel<128>, grid, dim3(kAttnThreads), bytes, stream, p);
    }
    MDMA_LAUNCH_OK("attention_mma");
    if (splits > 1) {
        launch_chained(attention_merge_kernel, dim3(n_tokens * n_heads), dim3(64), 0, stream, (const float*)p.part_o, (const float*)p.part_ml, p.out, splits, head_dim);
        MDMA_LAUNCH_OK("attention_merge");
    }
    return 0;
}

}  // namespace mdma
