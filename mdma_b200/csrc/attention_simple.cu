// Attention over the cache, one warp per (token, head), keys visited in order.
//
// This is the attention of the true 32-bit engine and the reference the fast
// kernels are checked against.  A query at position p of a sequence sees the
// keys [first, p] of its slot, first = 0 or p+1-window.  Scores, the running
// maximum, the normaliser and the output are float; because keys are visited
// in position order by one warp, the result for a token does not depend on
// how the tokens were cut into steps or on the rest of the batch.
#include "common.cuh"

namespace mdma {

constexpr int kMaxHeadDim = 256;

template <typename T>
__global__ void __launch_bounds__(128)
attention_simple_kernel(const T* __restrict__ q, int q_row_stride,
                        const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                        const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                        const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                        int max_pages, int page_size, T* __restrict__ out,
                        int n_heads, int n_kv_heads, int head_dim, int window, float scale) {
    const int t = blockIdx.x;
    const int h = blockIdx.y * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (h >= n_heads) return;
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    const int kvh = h / (n_heads / n_kv_heads);
    const int first = window > 0 ? max(0, pos + 1 - window) : 0;

    float qv[kMaxHeadDim / 32], acc[kMaxHeadDim / 32];
    const T* qp = q + (size_t)t * q_row_stride + (size_t)h * head_dim;
#pragma unroll
    for (int j = 0; j < kMaxHeadDim / 32; ++j) {
        const int d = lane + 32 * j;
        qv[j] = d < head_dim ? to_float(qp[d]) : 0.f;
        acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int* pages = page_table + (size_t)slot * max_pages;
    for (int p = first; p <= pos; ++p) {
        const size_t row = (((size_t)pages[p / page_size] * page_size + (size_t)(p % page_size)) * n_kv_heads + kvh) * head_dim;
        const T* kp = k_cache + row;
        const T* vp = v_cache + row;
        float part = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxHeadDim / 32; ++j) {
            const int d = lane + 32 * j;
            if (d < head_dim) part = fmaf(qv[j], to_float(kp[d]), part);
        }
        const float s = warp_sum(part) * scale;
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);     // exp(-inf) = 0 on the first key
        const float pe = expf(s - m_new);
        l = l * corr + pe;
#pragma unroll
        for (int j = 0; j < kMaxHeadDim / 32; ++j) {
            const int d = lane + 32 * j;
            if (d < head_dim) acc[j] = acc[j] * corr + pe * to_float(vp[d]);
        }
        m = m_new;
    }
    T* op = out + ((size_t)t * n_heads + h) * head_dim;
    const float inv = 1.0f / l;
#pragma unroll
    for (int j = 0; j < kMaxHeadDim / 32; ++j) {
        const int d = lane + 32 * j;
        if (d < head_dim) op[d] = from_float<T>(acc[j] * inv);
    }
}

}  // namespace mdma

using namespace mdma;

extern "C" int mdma_attention_simple(const void* q, int dtype, int q_row_stride, const void* k_cache,
                                     const void* v_cache, const int* tok_seq, const int* tok_pos,
                                     const int* seq_slot, const int* page_table, int max_pages,
                                     int page_size, void* out, int n_tokens, int n_heads,
                                     int n_kv_heads, int head_dim, int window, float scale,
                                     cudaStream_t stream) {
    MDMA_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention: %d heads over %d kv heads", n_heads, n_kv_heads);
    MDMA_REQUIRE(head_dim > 0 && head_dim <= kMaxHeadDim, "attention: head_dim %d is beyond the limit %d", head_dim, kMaxHeadDim);
    MDMA_REQUIRE(page_table && page_size > 0 && max_pages > 0 && window >= 0, "attention: bad cache geometry");
    if (n_tokens == 0) return 0;
    dim3 grid(n_tokens, (n_heads + 3) / 4);
    MDMA_DISPATCH_DTYPE(dtype, T,
        attention_simple_kernel<T><<<grid, 128, 0, stream>>>(
            (const T*)q, q_row_stride, (const T*)k_cache, (const T*)v_cache, tok_seq, tok_pos, seq_slot,
            page_table, max_pages, page_size, (T*)out, n_heads, n_kv_heads, head_dim, window, scale));
    MDMA_LAUNCH_OK("attention_simple");
    return 0;
}
