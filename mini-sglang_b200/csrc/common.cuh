// Shared device helpers for the engine's sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define MSGL_API extern "C" __attribute__((visibility("default")))

// element type selector used by the C entry points: 0 = float32, 1 = bfloat16
enum { MSGL_F32 = 0, MSGL_BF16 = 1 };

// error codes returned by the C entry points (0 = launched)
enum {
    MSGL_OK = 0,
    MSGL_ERR_DTYPE = 1,       // element type not handled by this kernel
    MSGL_ERR_SIZE = 2,        // a size the kernel refuses (head size, row length, ...)
    MSGL_ERR_LAUNCH = 3,      // cudaGetLastError() after the launch was not cudaSuccess
    MSGL_ERR_ALIGN = 4,       // a pointer or stride not aligned as required
};

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// weight that may be stored as float32 or as bfloat16, chosen at run time
__device__ __forceinline__ float load_weight(const void* w, int i, int w_is_f32) {
    return w_is_f32 ? reinterpret_cast<const float*>(w)[i]
                    : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i]);
}

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

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats of shared memory.
// The order of the additions depends only on blockDim, never on the data or the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float r = (lane < nwarps) ? scratch[lane] : 0.f;
    r = warp_sum(r);
    return r;
}

// Programmatic dependent launch: a kernel launched with msgl_launch_pdl may start while the kernel
// before it in the stream is still running.  It must call pdl_wait() before it reads anything an
// earlier kernel wrote and before it writes anything at all; what comes before the wait (index
// arithmetic, fetching weights, which no kernel writes) overlaps the predecessor's tail.
// pdl_launch_dependents() lets the successor start as soon as every block of this grid has
// issued it.  Launched the ordinary way both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
// Where a kernel lets its successor start (griddepcontrol.launch_dependents takes effect once every
// block of the grid has issued it or exited).  MSGL_PDL_MODE: 0 = at pdl_late() (after the main loop of
// the long kernels, else at exit), 1 = right after the kernel's own pdl_wait() (so at most two kernels
// overlap), 2 = at the very start (successors of successors pile up on the SMs: measured slower).
#ifndef MSGL_PDL_MODE
#define MSGL_PDL_MODE 0
#endif
__device__ __forceinline__ void pdl_trigger_() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {          // at a kernel's start, before its wait
#if MSGL_PDL_MODE == 2
    pdl_trigger_();
#endif
}
__device__ __forceinline__ void pdl_after_wait() {
#if MSGL_PDL_MODE == 1
    pdl_trigger_();
#endif
}
// a short kernel (norm, rotation, merge) releases its successor as soon as it runs itself: the product that
// follows then launches and fetches its first weights beside it (MSGL_PDL_SMALL=0: at exit instead)
#ifndef MSGL_PDL_SMALL
#define MSGL_PDL_SMALL 1
#endif
__device__ __forceinline__ void pdl_small() {
#if MSGL_PDL_MODE == 0 && MSGL_PDL_SMALL
    pdl_trigger_();
#endif
}
__device__ __forceinline__ void pdl_late() {
#if MSGL_PDL_MODE == 0
    pdl_trigger_();
#endif
}

#include <stdlib.h>
static inline bool msgl_pdl_enabled() {
    static int on = -1;
    // on unless MSGL_PDL=0.  Measured on B200 (Qwen3-8B layer sizes, decode step in a CUDA graph): batch 8
    // 4.77 -> 4.57 ms, batch 1 3.77 -> 3.57 ms with the successor released after the main loop
    // (MSGL_PDL_MODE 0); released at a kernel's start the step was slower than without (4.89 ms).
    if (on < 0) { const char* e = getenv("MSGL_PDL"); on = (e && e[0] == '0') ? 0 : 1; }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline void msgl_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                   Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = msgl_pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// What a device needs once before a kernel's first launch there (function attributes, occupancy questions) is
// remembered per device: a process may drive several, and an attribute set while one device is current does not
// reach the others.
#define MSGL_MAX_DEVICES 64
static inline int msgl_device() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= MSGL_MAX_DEVICES) return 0;
    return d;
}
struct MsglOncePerDevice {
    bool done_[MSGL_MAX_DEVICES] = {};
    bool due() const { return !done_[msgl_device()]; }       // true until mark() was called with this device current
    void mark() { done_[msgl_device()] = true; }
};
static inline int msgl_sm_count() {
    static int n[MSGL_MAX_DEVICES] = {};
    const int d = msgl_device();
    if (n[d] == 0 && cudaDeviceGetAttribute(&n[d], cudaDevAttrMultiProcessorCount, d) != cudaSuccess) n[d] = 0;
    return n[d] > 0 ? n[d] : 1;
}

#include <stdio.h>
static inline int msgl_check_launch() {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return MSGL_OK;
    fprintf(stderr, "[mini_sglang_b200] kernel launch failed: %s\n", cudaGetErrorString(e));
    return MSGL_ERR_LAUNCH;
}
