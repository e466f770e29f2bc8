// C entry points of the tensor-core attention (kernels in attention_mma.cuh).
#include "attention_mma.cuh"

using namespace mdma;

extern "C" {

// Whether the tensor-core attention takes this geometry.
int mdma_attention_mma_supported(int n_heads, int n_kv_heads, int head_dim) {
    return attention_mma_supported(n_heads, n_kv_heads, head_dim);
}

// Floats of scratch a call needs: n_tokens * n_heads * splits * (head_dim + 2); 0 for splits == 1.
long mdma_attention_mma_scratch(int n_tokens, int n_heads, int head_dim, int splits) {
    return attention_mma_scratch_floats(n_tokens, n_heads, head_dim, splits);
}

int mdma_attention_mma(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                       const int* seq_start, const int* seq_pos0, const int* seq_slot, const int* page_table,
                       int max_pages, int page_size, void* out, int n_tokens, int n_seqs, int max_new,
                       int n_heads, int n_kv_heads, int head_dim, int window, float scale, int splits,
                       float* scratch, long scratch_floats, cudaStream_t stream) {
    return launch_attention_mma(q, q_stride, k_cache, v_cache, seq_start, seq_pos0, seq_slot, page_table,
                                max_pages, page_size, out, n_tokens, n_seqs, max_new, n_heads, n_kv_heads,
                                head_dim, window, scale, splits, scratch, scratch_floats, stream);
}

// The same with the number of cache pages (lets the decode kernel fetch its tiles by TMA) and an
// optional status word that is set non-zero if a bounded wait ran out.
int mdma_attention_mma_paged(const void* q, int q_stride, const void* k_cache, const void* v_cache, int n_pages,
                             const int* seq_start, const int* seq_pos0, const int* seq_slot, const int* page_table,
                             int max_pages, int page_size, void* out, int n_tokens, int n_seqs, int max_new,
                             int n_heads, int n_kv_heads, int head_dim, int window, float scale, int splits,
                             float* scratch, long scratch_floats, int* status, cudaStream_t stream) {
    return launch_attention_mma(q, q_stride, k_cache, v_cache, seq_start, seq_pos0, seq_slot, page_table,
                                max_pages, page_size, out, n_tokens, n_seqs, max_new, n_heads, n_kv_heads,
                                head_dim, window, scale, splits, scratch, scratch_floats, stream, n_pages, status);
}

}  // extern "C"
