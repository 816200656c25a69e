// Shared device helpers for the engine's sm_100a kernels.
//
// Conventions of every exported entry point (all `extern "C"`, called through ctypes):
//   * pointers are device pointers; `stream` is a cudaStream_t passed as an integer;
//   * the return value is 0 on success, a positive cudaError_t if the launch failed, or a
//     negative LLM_REFUSED_* code when the sizes are outside what the kernel was written
//     for (the Python wrapper turns that into an exception; nothing is launched);
//   * `dtype` arguments: 0 = float32, 1 = bfloat16.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLM_OK 0
#define LLM_REFUSED_SIZE (-1)      // a size the kernel does not take
#define LLM_REFUSED_DTYPE (-2)     // a dtype combination that is not instantiated
#define LLM_REFUSED_ALIGN (-3)     // a pointer or stride that breaks the kernel's alignment rule

#define LLM_DT_F32 0
#define LLM_DT_BF16 1

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads.  `scratch` holds 33 floats of shared memory.
// Every thread gets the total.  The order of additions depends only on blockDim.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                       // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = (lane < nwarps) ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Loads 8 consecutive elements (16 bytes of bfloat16, or two 16-byte float loads) as floats.
__device__ __forceinline__ void load8(const bf16* p, float (&o)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        o[2 * i] = f.x;
        o[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void load8(const float* p, float (&o)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
    o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// ---- programmatic dependent launch -----------------------------------------------------------
// Every kernel of the engine is launched with the "programmatic stream serialization" attribute
// and begins with `pdl_begin()`: it lets the NEXT kernel in the stream be scheduled onto SMs
// as they become free (instead of after this grid has completely drained) and then waits until
// the PREVIOUS kernel has finished and its writes are visible.  A kernel that has work that does
// not depend on its predecessor (the streaming product fetches weights) does that work between
// the two halves.  Big grids do not invite their successor early: its blocks would only take
// room from blocks of this grid that have not started yet.
// What a kernel may read BEFORE its wait: weights, the step's metadata (copied to the device
// before the step's first kernel) and the block tables (their scatter kernel invites nobody
// early), keys and values of earlier steps.  Never anything a kernel of this step writes: a
// chain of early invitations can keep several of them in flight at once.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_invite() {
    unsigned sms;
    asm("mov.u32 %0, %%nsmid;\n" : "=r"(sms));                 // this device's number of SMs
    if (gridDim.x * gridDim.y * gridDim.z <= 8u * sms) pdl_launch_dependents();     // a "big" grid: over 8 CTAs an SM
}
__device__ __forceinline__ void pdl_begin() {
    pdl_invite();
    pdl_wait();
}

#include <cstdlib>
#include <utility>

static inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("LLM_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}

static inline int launch_status() {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? LLM_OK : static_cast<int>(e);
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
