// Shared helpers for every kernel file of the library: element types, error
// reporting to the host, and fixed-order reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

namespace mdma {

// Element type codes shared with the Python side.
enum DType : int { kF32 = 0, kBF16 = 1 };

// The last error of this library, as text.  Every exported function returns 0
// on success and non-zero after storing a message here.
static inline char* error_buffer() {
    static char buf[1024] = {0};
    return buf;
}
static inline int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 1024, fmt, ap);
    va_end(ap);
    return 1;
}
// What a matrix product adds on its way out: a vector over the output features (for the second matrix of
// a gated product too), kept as float32 or bfloat16, and which activation a gated product applies to its gate.
enum Activation : int { kActSilu = 0, kActGeluTanh = 1 };
struct Ending {
    const void* bias;     // [n_features] or null
    const void* bias2;    // the second matrix's, or null
    int bias_dtype;       // DType of both
    int act;              // Activation, gated products only
};
__device__ __forceinline__ float ending_bias(const void* b, int dtype, int f) {
    if (b == nullptr) return 0.f;
    return dtype == kF32 ? reinterpret_cast<const float*>(b)[f] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(b)[f]);
}
// act(g) of a gated feed-forward in plain float arithmetic (the 32-bit engine) ...
__device__ __forceinline__ float gate_activation(float g, int act) {
    if (act == kActGeluTanh) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.0f + expf(-g));
}
// ... and with the fast exponential (the bfloat16 engine): 0.5 (1 + tanh t) = 1 / (1 + e^(-2t)).
__device__ __forceinline__ float gate_activation_fast(float g, int act) {
    if (act == kActGeluTanh) return g / (1.0f + __expf(-1.5957691216057308f * (g + 0.044715f * g * g * g)));
    return g / (1.0f + __expf(-g));
}

#define MDMA_REQUIRE(cond, ...) \
    do { if (!(cond)) return ::mdma::fail(__VA_ARGS__); } while (0)
#define MDMA_LAUNCH_OK(name) \
    do { cudaError_t e_ = cudaGetLastError(); \
         if (e_ != cudaSuccess) return ::mdma::fail("%s: launch failed: %s", name, cudaGetErrorString(e_)); } while (0)

// Programmatic dependent launch.  A kernel launched with `launch_chained` may start
// while the kernel before it in the stream is still running; it must call
// `chain_wait()` before it reads or writes anything that earlier kernels touch
// (reading weights before that is fine), and calls `chain_release()` early so the
// kernel after it can begin its own prologue.  Without the launch attribute both
// are no-ops.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool chaining_enabled() {
    static int on = -1;
    if (on < 0) { const char* e = getenv("MDMA_CHAIN"); on = (e && e[0] == '0') ? 0 : 1; }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = chaining_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Sum over a warp; every lane gets the same value, and the order of additions
// is fixed (butterfly), so the result does not depend on what else runs.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads, fixed order.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];
    return total;
}

}  // namespace mdma

// Dispatch on an element type code.
#define MDMA_DISPATCH_DTYPE(code, T, ...)                                  \
    do {                                                                   \
        if ((code) == ::mdma::kF32) { using T = float; __VA_ARGS__; }      \
        else if ((code) == ::mdma::kBF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else return ::mdma::fail("unknown dtype code %d", (int)(code));    \
    } while (0)
