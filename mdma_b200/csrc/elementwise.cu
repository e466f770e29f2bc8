// Embedding gather, RMSNorm, rotary position encoding fused with the cache
// write, and row gathers.  Every kernel is a template over the activation
// type (float for the true 32-bit engine, bfloat16 for the serving engine);
// sums of squares, rotation angles and their sines are always float.
#include "common.cuh"

namespace mdma {

// ---------------------------------------------------------------- embedding
// x[t,:] = float(table[ids[t],:]).  The residual stream is float in both engines.
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                  float* __restrict__ out, int width, int vocab) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * width;
    if (id < 0 || id >= vocab) {           // the host rejects such ids; never read out of range
        for (int e = threadIdx.x; e < width; e += blockDim.x) o[e] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x) o[e] = to_float(row[e]);
}

// ---------------------------------------------------------------- RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w, one block per row.  `rows` (optional)
// picks which rows of x are normed: y[i] = norm(x[rows[i]]).
// With `splits` > 0 the row is first completed: x += sum_s partial[s] (the
// K-split partial sums of the matrix product that feeds the residual stream,
// added in split order) and written back, so the product's reduction, the
// residual add and the norm are one pass over the row.
// PER > 0: each thread keeps PER elements of the row in registers (one read of
// x); PER == 0: rows of any width, read twice.
template <typename TO, typename TW, int PER>
__global__ void __launch_bounds__(1024)
rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ partial, int splits,
                               size_t split_stride, const TW* __restrict__ w, const int* __restrict__ rows,
                               TO* __restrict__ y, int width, float eps) {
    chain_release();
    chain_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * width;
    float* xr = x + src;
    TO* yr = y + (size_t)r * width;
    float ss = 0.f;
    if (PER > 0) {
        // All loads of the row are issued before anything is written back to x: a store in
        // between would order the loads behind it (same array) and serialise PER round trips.
        float v[PER > 0 ? PER : 1];
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            v[i] = e < width ? xr[e] : 0.f;
        }
        if (splits > 0) {
            for (int sidx = 0; sidx < splits; ++sidx) {
                const float* pr = partial + (size_t)sidx * split_stride + src;
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    const int e = i * blockDim.x + threadIdx.x;
                    if (e < width) v[i] += pr[e];
                }
            }
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int e = i * blockDim.x + threadIdx.x;
                if (e < width) xr[e] = v[i];
            }
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) ss += v[i] * v[i];
        ss = block_sum(ss, scratch);
        const float scale = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            if (e < width) yr[e] = from_float<TO>(v[i] * scale * to_float(w[e]));
        }
    } else {
        for (int e = threadIdx.x; e < width; e += blockDim.x) {
            float a = xr[e];
            for (int sidx = 0; sidx < splits; ++sidx) a += partial[(size_t)sidx * split_stride + src + e];
            if (splits > 0) xr[e] = a;
            ss += a * a;
        }
        ss = block_sum(ss, scratch);
        const float scale = 1.0f / sqrtf(ss / (float)width + eps);
        for (int e = threadIdx.x; e < width; e += blockDim.x)
            yr[e] = from_float<TO>(xr[e] * scale * to_float(w[e]));
    }
}

// The same for widths that are a multiple of 4: each thread keeps NV groups of four
// consecutive elements (16-byte loads of x and of the partial sums).
template <typename T> struct Pack4;
template <> struct Pack4<float> {
    static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) {
        *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    }
};
template <> struct Pack4<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo); u.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

template <typename TO, typename TW, int NV>
__global__ void __launch_bounds__(1024)
rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ partial, int splits, size_t split_stride,
                   const TW* __restrict__ w, const int* __restrict__ rows, TO* __restrict__ y, int width, float eps) {
    __shared__ float scratch[32];
    chain_release();
    chain_wait();
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * width;
    float4* xr = reinterpret_cast<float4*>(x + src);
    const int n4 = width / 4;
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int e = i * blockDim.x + threadIdx.x;
        v[i] = e < n4 ? xr[e] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (splits > 0) {
        for (int sidx = 0; sidx < splits; ++sidx) {
            const float4* pr = reinterpret_cast<const float4*>(partial + (size_t)sidx * split_stride + src);
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int e = i * blockDim.x + threadIdx.x;
                if (e < n4) { const float4 q = pr[e]; v[i].x += q.x; v[i].y += q.y; v[i].z += q.z; v[i].w += q.w; }
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            if (e < n4) xr[e] = v[i];
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TO* yr = y + (size_t)r * width;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int e = i * blockDim.x + threadIdx.x;
        if (e < n4) {
            const TW* wp = w + 4 * e;
            Pack4<TO>::store(yr + 4 * e, v[i].x * scale * to_float(wp[0]), v[i].y * scale * to_float(wp[1]),
                             v[i].z * scale * to_float(wp[2]), v[i].w * scale * to_float(wp[3]));
        }
    }
}

// ------------------------------------------------- rotary + cache write
// One block per token works on its fused projection row [q heads | k heads | v heads]:
// q is rotated in place; rotated k and raw v go to the cache row of (slot, position):
// page page_table[slot][pos / page_size], row pos % page_size of that page.
// With `splits` > 0 the projection row is read as the sum of that many float
// partial rows (the K-split partial sums of the projection, in split order)
// instead of from qkv; the rotated queries are still written to qkv.
template <typename T>
__global__ void rope_cache_write_kernel(T* __restrict__ qkv, int row_stride,
                                        const float* __restrict__ partial, int splits, size_t split_stride,
                                        int partial_width,
                                        const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                        const int* __restrict__ seq_slot,
                                        const float* __restrict__ inv_freq,
                                        T* __restrict__ k_cache, T* __restrict__ v_cache,
                                        const int* __restrict__ page_table, int max_pages, int page_size,
                                        int n_heads, int n_kv_heads, int head_dim, int rotary_dim,
                                        int interleaved, int write_kv) {
    // One block per token.  The angle of a pair depends on the position only, so its sine and
    // cosine are computed once and shared by every head of the row.
    extern __shared__ float sc[];                  // [rotary_dim/2] sines, then cosines
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int half = rotary_dim / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        sc[i] = s; sc[half + i] = c;
    }
    __syncthreads();
    T* row = qkv + (size_t)t * row_stride;
    const float* prow = partial + (size_t)t * partial_width;
    auto load = [&](int col) -> float {
        if (splits == 0) return to_float(row[col]);
        float a = 0.f;
        for (int sidx = 0; sidx < splits; ++sidx) a += prow[(size_t)sidx * split_stride + col];
        return a;
    };
    // two columns at once, the partial sums fetched four splits at a time before they are added (in split
    // order, as `load` adds them): the loads of a pair are in flight together instead of one after the other
    auto load2 = [&](int c0, int c1, float& x0, float& x1) {
        if (splits == 0) { x0 = to_float(row[c0]); x1 = to_float(row[c1]); return; }
        float a = 0.f, b = 0.f;
        int sidx = 0;
        for (; sidx + 4 <= splits; sidx += 4) {
            const float* q = prow + (size_t)sidx * split_stride;
            const float a0 = q[c0], a1 = q[split_stride + c0], a2 = q[2 * split_stride + c0], a3 = q[3 * split_stride + c0];
            const float b0 = q[c1], b1 = q[split_stride + c1], b2 = q[2 * split_stride + c1], b3 = q[3 * split_stride + c1];
            a += a0; a += a1; a += a2; a += a3;
            b += b0; b += b1; b += b2; b += b3;
        }
        for (; sidx < splits; ++sidx) { a += prow[(size_t)sidx * split_stride + c0]; b += prow[(size_t)sidx * split_stride + c1]; }
        x0 = a; x1 = b;
    };
    size_t cache_row = 0;
    if (write_kv) {
        const int slot = seq_slot[tok_seq[t]];
        const int page = page_table[(size_t)slot * max_pages + pos / page_size];
        cache_row = ((size_t)page * page_size + (size_t)(pos % page_size)) * n_kv_heads;
    }
    // blockIdx.y divides the heads of the row [q | k | v] among blocks (few tokens: many blocks per token)
    const int total_heads = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    const int per_block = (total_heads + gridDim.y - 1) / gridDim.y;
    const int h_lo = blockIdx.y * per_block, h_hi = min(total_heads, h_lo + per_block);
    const int rot_end = min(h_hi, n_heads + (write_kv ? n_kv_heads : 0));      // q and k rotate, v does not
    // rotated pairs
    for (int i = threadIdx.x; i < (rot_end - h_lo) * half; i += blockDim.x) {
        const int h = h_lo + i / half, pr = i % half;
        const int d0 = interleaved ? 2 * pr : pr, d1 = interleaved ? 2 * pr + 1 : pr + half;
        float x0, x1;
        load2(h * head_dim + d0, h * head_dim + d1, x0, x1);
        const float s = sc[pr], c = sc[half + pr];
        T* dst = h < n_heads ? row + (size_t)h * head_dim
                             : k_cache + (cache_row + (h - n_heads)) * head_dim;
        dst[d0] = from_float<T>(x0 * c - x1 * s);
        dst[d1] = from_float<T>(x0 * s + x1 * c);
    }
    // what is not rotated: the tail of q and k beyond rotary_dim, and v
    const int tail = head_dim - rotary_dim;
    if (tail > 0) {
        for (int i = threadIdx.x; i < (rot_end - h_lo) * tail; i += blockDim.x) {
            const int h = h_lo + i / tail, d = rotary_dim + i % tail;
            if (h < n_heads) { if (splits > 0) row[(size_t)h * head_dim + d] = from_float<T>(load(h * head_dim + d)); }
            else k_cache[(cache_row + (h - n_heads)) * head_dim + d] = from_float<T>(load(h * head_dim + d));
        }
    }
    const int v_lo = max(h_lo, n_heads + n_kv_heads);
    if (write_kv && h_hi > v_lo) {
        for (int i = threadIdx.x; i < (h_hi - v_lo) * head_dim; i += blockDim.x) {
            const int col = v_lo * head_dim + i;                       // column in the projection row
            v_cache[cache_row * head_dim + (col - (n_heads + n_kv_heads) * head_dim)] = from_float<T>(load(col));
        }
    }
}

// The same for 48 tokens or more of bfloat16 in the split-half layout, no partial sums: 16-byte accesses,
// eight pairs (d, d + rotary_dim/2) per thread and step.  One block per token (64 tokens: 3.2 us against 4.9 us
// with the kernel above, 160 tokens: 3.7 against 6.5 us).
__global__ void rope_cache_write_vec_kernel(__nv_bfloat16* __restrict__ qkv, int row_stride,
                                            const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                            const int* __restrict__ seq_slot, const float* __restrict__ inv_freq,
                                            __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                            const int* __restrict__ page_table, int max_pages, int page_size,
                                            int n_heads, int n_kv_heads, int head_dim, int rotary_dim, int write_kv) {
    extern __shared__ float sc[];                  // [rotary_dim/2] sines, then cosines
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int half = rotary_dim / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        sc[i] = s; sc[half + i] = c;
    }
    __syncthreads();
    __nv_bfloat16* row = qkv + (size_t)t * row_stride;
    size_t cache_row = 0;
    if (write_kv) {
        const int slot = seq_slot[tok_seq[t]];
        const int page = page_table[(size_t)slot * max_pages + pos / page_size];
        cache_row = ((size_t)page * page_size + (size_t)(pos % page_size)) * n_kv_heads;
    }
    const int rot_heads = n_heads + (write_kv ? n_kv_heads : 0);
    const int groups = half / 8;                   // groups of eight pairs per head
    for (int i = threadIdx.x; i < rot_heads * groups; i += blockDim.x) {
        const int h = i / groups, d = (i % groups) * 8;
        const __nv_bfloat16* src = row + (size_t)h * head_dim;
        __nv_bfloat16* dst = h < n_heads ? row + (size_t)h * head_dim : k_cache + (cache_row + (h - n_heads)) * head_dim;
        const uint4 lo = *reinterpret_cast<const uint4*>(src + d), hi = *reinterpret_cast<const uint4*>(src + d + half);
        const __nv_bfloat16* a = reinterpret_cast<const __nv_bfloat16*>(&lo);
        const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&hi);
        uint4 olo, ohi;
        __nv_bfloat16* oa = reinterpret_cast<__nv_bfloat16*>(&olo);
        __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&ohi);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float x0 = __bfloat162float(a[q]), x1 = __bfloat162float(b[q]);
            const float sn = sc[d + q], cs = sc[half + d + q];
            oa[q] = __float2bfloat16_rn(x0 * cs - x1 * sn);
            ob[q] = __float2bfloat16_rn(x0 * sn + x1 * cs);
        }
        *reinterpret_cast<uint4*>(dst + d) = olo;
        *reinterpret_cast<uint4*>(dst + d + half) = ohi;
    }
    if (!write_kv) return;
    // not rotated: k beyond rotary_dim, and v (q beyond rotary_dim stays where it is)
    const int tail8 = (head_dim - rotary_dim) / 8;
    for (int i = threadIdx.x; i < n_kv_heads * tail8; i += blockDim.x) {
        const int h = i / tail8, d = rotary_dim + (i % tail8) * 8;
        *reinterpret_cast<uint4*>(k_cache + (cache_row + h) * head_dim + d) =
            *reinterpret_cast<const uint4*>(row + (size_t)(n_heads + h) * head_dim + d);
    }
    const __nv_bfloat16* v_src = row + (size_t)(n_heads + n_kv_heads) * head_dim;
    for (int i = threadIdx.x; i < n_kv_heads * head_dim / 8; i += blockDim.x)
        *reinterpret_cast<uint4*>(v_cache + cache_row * head_dim + (size_t)i * 8) = *reinterpret_cast<const uint4*>(v_src + (size_t)i * 8);
}

// The same from K-split partial sums of the projection (bfloat16 out), with 16-byte loads (64 tokens, 6 splits: 4.6 us
// against 5.8 us with the scalar kernel; 160 tokens, 3 splits: 7.3 against 13.1 us): a thread takes four
// pairs of one head at a time (split-half layout: columns d..d+3 and d+half..d+half+3; interleaved: eight
// consecutive columns), adds the splits in order as the kernel above does, rotates, and stores 8 or 16 bytes.
// gridDim.y blocks share a token's work items (rotated groups of q and k, the columns beyond the rotated width,
// the value heads).
__global__ void __launch_bounds__(256)
rope_cache_write_partial_vec_kernel(__nv_bfloat16* __restrict__ qkv, int row_stride,
                                    const float* __restrict__ partial, int splits, size_t split_stride, int partial_width,
                                    const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                    const int* __restrict__ seq_slot, const float* __restrict__ inv_freq,
                                    __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                    const int* __restrict__ page_table, int max_pages, int page_size,
                                    int n_heads, int n_kv_heads, int head_dim, int rotary_dim, int interleaved, int write_kv) {
    extern __shared__ float sc[];                  // [rotary_dim/2] sines, then cosines
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int half = rotary_dim / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        sc[i] = s; sc[half + i] = c;
    }
    __syncthreads();
    __nv_bfloat16* row = qkv + (size_t)t * row_stride;
    const float* prow = partial + (size_t)t * partial_width;
    size_t cache_row = 0;
    if (write_kv) {
        const int slot = seq_slot[tok_seq[t]];
        const int page = page_table[(size_t)slot * max_pages + pos / page_size];
        cache_row = ((size_t)page * page_size + (size_t)(pos % page_size)) * n_kv_heads;
    }
    // the sum of the splits of four consecutive columns, four splits in flight at a time, added in split order
    auto load4 = [&](int col) -> float4 {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        int sidx = 0;
        for (; sidx + 4 <= splits; sidx += 4) {
            const float* q = prow + (size_t)sidx * split_stride + col;
            const float4 p0 = *reinterpret_cast<const float4*>(q), p1 = *reinterpret_cast<const float4*>(q + split_stride),
                         p2 = *reinterpret_cast<const float4*>(q + 2 * split_stride), p3 = *reinterpret_cast<const float4*>(q + 3 * split_stride);
            a.x += p0.x; a.y += p0.y; a.z += p0.z; a.w += p0.w;
            a.x += p1.x; a.y += p1.y; a.z += p1.z; a.w += p1.w;
            a.x += p2.x; a.y += p2.y; a.z += p2.z; a.w += p2.w;
            a.x += p3.x; a.y += p3.y; a.z += p3.z; a.w += p3.w;
        }
        for (; sidx < splits; ++sidx) {
            const float4 p0 = *reinterpret_cast<const float4*>(prow + (size_t)sidx * split_stride + col);
            a.x += p0.x; a.y += p0.y; a.z += p0.z; a.w += p0.w;
        }
        return a;
    };
    auto pack4 = [](float a, float b, float c, float d) -> uint2 {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo); u.y = *reinterpret_cast<uint32_t*>(&hi);
        return u;
    };
    const int rot_heads = n_heads + (write_kv ? n_kv_heads : 0);          // q and k rotate, v does not
    const int groups = half / 4;                                          // groups of four pairs per head
    const int tail4 = (head_dim - rotary_dim) / 4, v4 = write_kv ? head_dim / 4 : 0;
    const int n_rot = rot_heads * groups, n_tail = rot_heads * tail4, n_v = n_kv_heads * v4;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n_rot + n_tail + n_v; i += gridDim.y * blockDim.x) {
        if (i < n_rot) {
            const int h = i / groups, g = i % groups;
            const int col = h * head_dim;
            __nv_bfloat16* dst = h < n_heads ? row + (size_t)h * head_dim : k_cache + (cache_row + (h - n_heads)) * head_dim;
            if (!interleaved) {
                const int d0 = 4 * g;
                const float4 a = load4(col + d0), b = load4(col + d0 + half);
                const float x0[4] = {a.x, a.y, a.z, a.w}, x1[4] = {b.x, b.y, b.z, b.w};
                float y0[4], y1[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float sn = sc[d0 + j], cs = sc[half + d0 + j];
                    y0[j] = x0[j] * cs - x1[j] * sn;
                    y1[j] = x0[j] * sn + x1[j] * cs;
                }
                *reinterpret_cast<uint2*>(dst + d0) = pack4(y0[0], y0[1], y0[2], y0[3]);
                *reinterpret_cast<uint2*>(dst + d0 + half) = pack4(y1[0], y1[1], y1[2], y1[3]);
            } else {
                const int e0 = 8 * g;                                      // pairs 4g .. 4g+3 lie in columns e0 .. e0+7
                const float4 a = load4(col + e0), b = load4(col + e0 + 4);
                const float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                float y[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float sn = sc[4 * g + j], cs = sc[half + 4 * g + j];
                    y[2 * j] = x[2 * j] * cs - x[2 * j + 1] * sn;
                    y[2 * j + 1] = x[2 * j] * sn + x[2 * j + 1] * cs;
                }
                *reinterpret_cast<uint2*>(dst + e0) = pack4(y[0], y[1], y[2], y[3]);
                *reinterpret_cast<uint2*>(dst + e0 + 4) = pack4(y[4], y[5], y[6], y[7]);
            }
        } else if (i < n_rot + n_tail) {
            const int k = i - n_rot, h = k / tail4, d = rotary_dim + 4 * (k % tail4);
            const float4 a = load4(h * head_dim + d);
            __nv_bfloat16* dst = h < n_heads ? row + (size_t)h * head_dim : k_cache + (cache_row + (h - n_heads)) * head_dim;
            *reinterpret_cast<uint2*>(dst + d) = pack4(a.x, a.y, a.z, a.w);
        } else {
            const int k = i - n_rot - n_tail, h = k / v4, d = 4 * (k % v4);
            const float4 a = load4((n_heads + n_kv_heads + h) * head_dim + d);
            *reinterpret_cast<uint2*>(v_cache + (cache_row + h) * head_dim + d) = pack4(a.x, a.y, a.z, a.w);
        }
    }
}

// After a decode step: the sampled tokens become the next inputs and every
// position moves on by one.  With a ring, the step's result words (tokens, flags and
// what lies behind them: `out_words` integers) are also kept in row `*counter % ring_rows`
// of the ring and the counter moves on, so that several steps can run before the host
// reads their tokens in one copy.  One block.
__global__ void advance_decode_kernel(const int* __restrict__ tokens, int* __restrict__ ids,
                                      int* __restrict__ tok_pos, int* __restrict__ seq_pos0, int n,
                                      int out_words, int* __restrict__ ring, int ring_rows, int* __restrict__ counter) {
    chain_release();
    chain_wait();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        ids[i] = tokens[i];
        tok_pos[i] += 1;
        seq_pos0[i] += 1;
    }
    if (ring != nullptr) {
        const int row = *counter % ring_rows;
        for (int i = threadIdx.x; i < out_words; i += blockDim.x) ring[(size_t)row * out_words + i] = tokens[i];
        __syncthreads();                 // every thread has read the counter
        if (threadIdx.x == 0) *counter += 1;
    }
}

template <typename TO, typename TW>
static void launch_rmsnorm(float* x, const float* partial, int splits, size_t split_stride, const TW* w,
                           const int* rows, TO* y, int n_rows, int width, float eps, cudaStream_t stream) {
    auto threads_for = [&](int per) { int t = ((width + per - 1) / per + 31) / 32 * 32; return t < 64 ? 64 : t; };
    const bool aligned = width % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)partial & 15) == 0 &&
                         ((uintptr_t)y & 15) == 0 && split_stride % 4 == 0;
    if (aligned && width <= 16384) {
        // 16-byte accesses; many rows: few threads per row (more rows in flight), few rows: many threads
        if (n_rows >= 512 && width > 1024)
            launch_chained(rmsnorm_vec_kernel<TO, TW, 4>, dim3(n_rows), dim3(threads_for(16)), 0, stream, x, partial, splits, split_stride, w, rows, y, width, eps);
        else if (width <= 4096)
            launch_chained(rmsnorm_vec_kernel<TO, TW, 1>, dim3(n_rows), dim3(threads_for(4)), 0, stream, x, partial, splits, split_stride, w, rows, y, width, eps);
        else
            launch_chained(rmsnorm_vec_kernel<TO, TW, 4>, dim3(n_rows), dim3(threads_for(16)), 0, stream, x, partial, splits, split_stride, w, rows, y, width, eps);
        return;
    }
    if (n_rows >= 512 && width <= 16384 && width > 1024)
        // many rows: a quarter of the threads per row, four times the rows in flight per SM
        launch_chained(rmsnorm_kernel<TO, TW, 16>, dim3(n_rows), dim3(threads_for(16)), 0, stream, x, partial, splits, split_stride, w, rows, y, width, eps);
    else if (width <= 4096)
        launch_chained(rmsnorm_kernel<TO, TW, 4>, dim3(n_rows), dim3(threads_for(4)), 0, stream, x, partial, splits, split_stride, w, rows, y, width, eps);
    else if (width <= 8192)
        launch_chained(rmsnorm_kernel<TO, TW, 8>, dim3(n_rows), dim3(threads_for(8)), 0, stream, x, partial, splits, split_stride, w, rows, y, width, eps);
    else if (width <= 16384)
        launch_chained(rmsnorm_kernel<TO, TW, 16>, dim3(n_rows), dim3(threads_for(16)), 0, stream, x, partial, splits, split_stride, w, rows, y, width, eps);
    else
        launch_chained(rmsnorm_kernel<TO, TW, 0>, dim3(n_rows), dim3(1024), 0, stream, x, partial, splits, split_stride, w, rows, y, width, eps);
}

// Seeded normal numbers that the host can reproduce bit for bit: element i of a tensor takes 24 bits of
// a counter-based hash of (key, i) (two rounds of splitmix64); 16 of them pick an interval of a table
// of 65,537 normal quantiles that the host computed, 8 the place inside it.  Every floating-point step
// is a single correctly rounded operation (no fused multiply-add), as on the host.
__device__ __forceinline__ unsigned long long fill_mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, long n, unsigned long long key,
                                   const float* __restrict__ table, float std) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const unsigned long long z = fill_mix64(fill_mix64(key ^ (unsigned long long)i));
        const int j = (int)(z >> 48);
        const float f = (float)((z >> 40) & 0xFFull) * (1.0f / 256.0f);
        const float lo = table[j];
        const float v = __fadd_rn(lo, __fmul_rn(__fsub_rn(table[j + 1], lo), f));
        out[i] = from_float<T>(__fmul_rn(v, std));
    }
}

}  // namespace mdma

using namespace mdma;

extern "C" {

// out[i] = std * quantile(hash(key, i)) for i < n; `table` holds 65,537 floats on the device.
int mdma_fill_normal(void* out, int dtype, long n, unsigned long long key, const float* table, float std,
                     cudaStream_t stream) {
    MDMA_REQUIRE(out && table && n >= 0, "fill_normal: bad arguments");
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    MDMA_DISPATCH_DTYPE(dtype, T, (fill_normal_kernel<T><<<blocks, 256, 0, stream>>>((T*)out, n, key, table, std)));
    MDMA_LAUNCH_OK("fill_normal");
    return 0;
}

// `tokens` is the start of the sampler's result words (tokens first); `ring` (optional) has
// `ring_rows` rows of `out_words` integers, `counter` counts the steps kept so far.
int mdma_advance_decode(const int* tokens, int* ids, int* tok_pos, int* seq_pos0, int n, int out_words,
                        int* ring, int ring_rows, int* counter, cudaStream_t stream) {
    if (n <= 0) return 0;
    MDMA_REQUIRE(ring == nullptr || (ring_rows > 0 && counter != nullptr && out_words >= n), "advance_decode: bad ring");
    launch_chained(advance_decode_kernel, dim3(1), dim3(256), 0, stream, tokens, ids, tok_pos, seq_pos0, n,
                   out_words, ring, ring_rows, counter);
    MDMA_LAUNCH_OK("advance_decode");
    return 0;
}

const char* mdma_last_error() { return error_buffer(); }

int mdma_embed_rows(const void* table, int table_dtype, const int* ids, float* out,
                    int n_tokens, int width, int vocab, cudaStream_t stream) {
    MDMA_REQUIRE(n_tokens >= 0 && width > 0 && vocab > 0, "embed_rows: bad sizes");
    if (n_tokens == 0) return 0;
    MDMA_DISPATCH_DTYPE(table_dtype, T,
        launch_chained(embed_rows_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (const T*)table, ids, out, width, vocab));
    MDMA_LAUNCH_OK("embed_rows");
    return 0;
}

// partial/splits: optional K-split partial sums [splits, rows_total, width] to add into x first
// (not with `rows`).
int mdma_rmsnorm(float* x, const void* w, int w_dtype, const int* rows, void* y, int y_dtype,
                 int n_rows, int width, float eps, const float* partial, int splits, long split_stride,
                 cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0, "rmsnorm: bad sizes");
    MDMA_REQUIRE(splits >= 0 && (splits == 0 || (partial && !rows)), "rmsnorm: partial sums need a pointer and no row list");
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_DTYPE(y_dtype, TO,
        MDMA_DISPATCH_DTYPE(w_dtype, TW,
            launch_rmsnorm<TO, TW>(x, partial, splits, (size_t)split_stride, (const TW*)w, rows, (TO*)y, n_rows, width, eps, stream)));
    MDMA_LAUNCH_OK("rmsnorm");
    return 0;
}

int mdma_rope_cache_write(void* qkv, int dtype, int row_stride, const float* partial, int splits,
                          long split_stride, int partial_width, const int* tok_seq, const int* tok_pos,
                          const int* seq_slot, const float* inv_freq, void* k_cache, void* v_cache,
                          const int* page_table, int max_pages, int page_size,
                          int n_tokens, int n_heads, int n_kv_heads, int head_dim, int rotary_dim,
                          int interleaved, int write_kv, cudaStream_t stream) {
    MDMA_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads >= 0 && head_dim > 0, "rope_cache_write: bad sizes");
    MDMA_REQUIRE(rotary_dim % 2 == 0 && rotary_dim <= head_dim, "rope_cache_write: rotary_dim %d does not fit head_dim %d", rotary_dim, head_dim);
    MDMA_REQUIRE(!write_kv || (page_table && page_size > 0 && max_pages > 0), "rope_cache_write: no cache pages");
    MDMA_REQUIRE(splits >= 0 && (splits == 0 || partial), "rope_cache_write: partial sums need a pointer");
    if (n_tokens == 0) return 0;
    const bool aligned16 = ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0;
    if (n_tokens >= 48 && dtype == kBF16 && splits == 0 && !interleaved && rotary_dim % 16 == 0 && head_dim % 8 == 0 &&
        row_stride % 8 == 0 && aligned16) {
        using B = __nv_bfloat16;
        launch_chained(rope_cache_write_vec_kernel, dim3(n_tokens), dim3(256), (size_t)rotary_dim * sizeof(float), stream,
            (B*)qkv, row_stride, tok_seq, tok_pos, seq_slot, inv_freq, (B*)k_cache, (B*)v_cache,
            page_table, max_pages, page_size, n_heads, n_kv_heads, head_dim, rotary_dim, write_kv);
        MDMA_LAUNCH_OK("rope_cache_write");
        return 0;
    }
    // (from 65 tokens: alone it is faster from 32 on, but in a decode step's chain of kernels a layer of 32 or 64
    // sequences took 117.0 and 141.0 us with it against 113.5 and 137.1 us with the many small blocks of the scalar
    // kernel; 80 sequences 147.9 against 150.0 us, 128 sequences 176.5 against 179.0 us)
    if (n_tokens > 64 && splits > 0 && dtype == kBF16 && rotary_dim % 8 == 0 && head_dim % 8 == 0 && row_stride % 4 == 0 &&
        partial_width % 4 == 0 && split_stride % 4 == 0 && ((uintptr_t)partial & 15) == 0 && ((uintptr_t)qkv & 7) == 0 &&
        (!write_kv || (((uintptr_t)k_cache & 7) == 0 && ((uintptr_t)v_cache & 7) == 0))) {
        // partial sums with 16-byte loads; about two blocks per SM
        using B = __nv_bfloat16;
        int per_token = (300 + n_tokens - 1) / n_tokens;
        per_token = per_token < 1 ? 1 : per_token > 8 ? 8 : per_token;
        launch_chained(rope_cache_write_partial_vec_kernel, dim3(n_tokens, per_token), dim3(256), (size_t)rotary_dim * sizeof(float), stream,
            (B*)qkv, row_stride, partial, splits, (size_t)split_stride, partial_width, tok_seq, tok_pos, seq_slot, inv_freq,
            (B*)k_cache, (B*)v_cache, page_table, max_pages, page_size, n_heads, n_kv_heads, head_dim, rotary_dim, interleaved, write_kv);
        MDMA_LAUNCH_OK("rope_cache_write");
        return 0;
    }
    // about 300 blocks at least: few tokens get several blocks per row, many tokens one
    const int total_heads = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    int per_token = n_tokens >= 300 ? 1 : (n_tokens <= 128 ? total_heads : (300 + n_tokens - 1) / n_tokens);
    if (per_token > total_heads) per_token = total_heads;
    dim3 grid(n_tokens, per_token);
    const int work = ((total_heads + per_token - 1) / per_token) * head_dim / 2;
    const int threads = work >= 1024 ? 256 : (work >= 256 ? 128 : 64);
    const size_t smem = (size_t)rotary_dim * sizeof(float);
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(rope_cache_write_kernel<T>, grid, dim3(threads), smem, stream,
            (T*)qkv, row_stride, partial, splits, (size_t)split_stride, partial_width,
            tok_seq, tok_pos, seq_slot, inv_freq, (T*)k_cache, (T*)v_cache,
            page_table, max_pages, page_size, n_heads, n_kv_heads, head_dim, rotary_dim, interleaved, write_kv));
    MDMA_LAUNCH_OK("rope_cache_write");
    return 0;
}

}  // extern "C"
