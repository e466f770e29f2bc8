// The allocation-free attention entry point: the kernels of attention_mma.cuh
// with their split scratch in an array that lives in this library's image.
// See attention_noalloc.h for who needs it, its limit and its rules.
#include <mutex>

#include "attention_mma.cuh"
#include "attention_noalloc.h"

namespace {

// The scratch itself.  In host code this name is a handle for the runtime, not
// a device address; the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_scratch[MDMA_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

// The device address of g_scratch on the current device, looked up once per device.
int scratch_for_current_device(float** out) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return mdma::fail("attention_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (device < 0 || device >= kMaxDevices) return mdma::fail("attention_noalloc: device %d is beyond the %d this table holds", device, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return mdma::fail("attention_noalloc: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
        g_scratch_address[device] = ptr;
    }
    *out = g_scratch_address[device];
    return 0;
}

}  // namespace

extern "C" {

const char* mdma_last_error() { return mdma::error_buffer(); }

int mdma_attention_mma_noalloc(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                               const int* seq_start, const int* seq_pos0, const int* seq_slot,
                               const int* page_table, int max_pages, int page_size, void* out,
                               int n_tokens, int n_seqs, int max_new, int n_heads, int n_kv_heads,
                               int head_dim, int window, float scale, int splits, cudaStream_t stream) {
    if (splits < 1) splits = 1;
    const long need = mdma::attention_mma_scratch_floats(n_tokens, n_heads, head_dim, splits);
    if (need > MDMA_NOALLOC_SCRATCH_FLOATS)
        return mdma::fail("attention_noalloc: %d tokens x %d heads x %d splits x (head_dim %d + 2) = %ld floats of "
                          "scratch, the fixed array holds %ld; use fewer splits or mdma_attention_mma with your own scratch",
                          n_tokens, n_heads, splits, head_dim, need, (long)MDMA_NOALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (int rc = scratch_for_current_device(&scratch)) return rc;
    return mdma::launch_attention_mma(q, q_stride, k_cache, v_cache, seq_start, seq_pos0, seq_slot, page_table,
                                      max_pages, page_size, out, n_tokens, n_seqs, max_new, n_heads, n_kv_heads,
                                      head_dim, window, scale, splits, scratch, MDMA_NOALLOC_SCRATCH_FLOATS, stream);
}

}  // extern "C"
