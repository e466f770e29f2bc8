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

// One token per sequence with the rotary encoding and the cache write inside the attention kernel:
// `qkv` holds the step's projection rows, not rotated; with `proj_splits` > 0 the rows are instead the sums
// of that many float partial rows at `proj_partial` (`proj_split_stride` floats apart).  The kernel writes
// the rotated key and the value of every token to the caches.
int mdma_attention_decode_rotary(const void* qkv, int q_stride, const float* proj_partial, int proj_splits,
                                 long proj_split_stride, const float* inv_freq, int rotary_dim, int interleaved,
                                 void* k_cache, void* v_cache, int n_pages, const int* seq_start, const int* seq_pos0,
                                 const int* seq_slot, const int* page_table, int max_pages, int page_size, void* out,
                                 int n_seqs, int n_heads, int n_kv_heads, int head_dim, int window, float scale,
                                 int splits, float* scratch, long scratch_floats, int* status, cudaStream_t stream) {
    FusedRotary fz;
    fz.inv_freq = inv_freq; fz.rotary_dim = rotary_dim; fz.interleaved = interleaved;
    fz.partial = proj_splits > 0 ? proj_partial : nullptr; fz.splits = proj_splits; fz.split_stride = proj_split_stride;
    fz.width = (n_heads + 2 * n_kv_heads) * head_dim;
    return launch_attention_mma(qkv, q_stride, k_cache, v_cache, seq_start, seq_pos0, seq_slot, page_table, max_pages,
                                page_size, out, n_seqs, n_seqs, 1, n_heads, n_kv_heads, head_dim, window, scale, splits,
                                scratch, scratch_floats, stream, n_pages, status, &fz);
}

int mdma_attention_fused_rotary_supported(int n_heads, int n_kv_heads, int head_dim, int page_size, int rotary_dim) {
    return attention_fused_rotary_supported(n_heads, n_kv_heads, head_dim, page_size, rotary_dim);
}

}  // extern "C"
