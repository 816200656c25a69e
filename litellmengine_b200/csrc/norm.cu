// RMSNorm over the last dimension, fused with the residual add that precedes it.
//
//   v   = x[row] (+ delta[row])                      32-bit sum: the residual stream is float32
//   out = v * rsqrt(mean(v^2) + eps) * w             sum of squares, rsqrt and products in 32-bit
//
// One block per output row.  `rows` (optional) picks which rows of x/delta are read, so the
// final norm can run only at the positions whose logits are wanted.  With `write_sum` the sum
// v is written back into x (the layer's residual update), which needs rows == nullptr.
// Formula and product order (x*inv)*w: src/layers/rms_norm.cu:77-93; the reference runs the
// add as its own kernel (src/ops/add.cu:16-27).
#include "common.cuh"

template <typename TX, typename TD, typename TO>
__global__ void rmsnorm_kernel(TX* __restrict__ x, const TD* __restrict__ delta,
                               const float* __restrict__ w, TO* __restrict__ out,
                               const int32_t* __restrict__ rows, int hidden, float eps,
                               int write_sum, int vec, int delta_parts, long long delta_part_stride) {
    // The norm weights are read before the wait for the kernel that produces x / delta.
    float g0[8];
    const bool one_trip = vec && hidden <= static_cast<int>(blockDim.x) * 8;
    if (one_trip && static_cast<int>(threadIdx.x) * 8 < hidden) load8(w + threadIdx.x * 8, g0);
    pdl_begin();
    extern __shared__ __align__(16) float smem[];   // hidden floats (padded to 8) + 33 for the reduction
    float* v = smem;
    float* scratch = smem + ((hidden + 7) & ~7);
    const size_t src = rows ? static_cast<size_t>(rows[blockIdx.x]) : blockIdx.x;
    TX* xr = x + src * hidden;
    const TD* dr = delta ? delta + src * hidden : nullptr;
    TO* orow = out + static_cast<size_t>(blockIdx.x) * hidden;
    float ss = 0.0f;
    if (vec) {                                      // 8 elements per thread per trip, 16-byte accesses
        for (int h = threadIdx.x * 8; h < hidden; h += blockDim.x * 8) {
            float a[8];
            load8(xr + h, a);
            if (dr) {
                for (int part = 0; part < delta_parts; ++part) {    // delta may come as the k-splits of a product
                    float b[8];
                    load8(dr + part * delta_part_stride + h, b);
#pragma unroll
                    for (int i = 0; i < 8; ++i) a[i] += b[i];
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += a[i] * a[i];
            store8(v + h, a);
            if (write_sum) store8(xr + h, a);
        }
    } else {
        for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
            float a = to_f32(xr[h]);
            if (dr)
                for (int part = 0; part < delta_parts; ++part) a += to_f32(dr[part * delta_part_stride + h]);
            v[h] = a;
            ss += a * a;
            if (write_sum) xr[h] = from_f32<TX>(a);
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
    if (one_trip) {
        const int h = threadIdx.x * 8;
        if (h < hidden) {
            float a[8];
            load8(v + h, a);
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = a[i] * inv * g0[i];
            store8(orow + h, a);
        }
    } else if (vec) {
        for (int h = threadIdx.x * 8; h < hidden; h += blockDim.x * 8) {
            float a[8], g[8];
            load8(v + h, a);
            load8(w + h, g);
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = a[i] * inv * g[i];
            store8(orow + h, a);
        }
    } else {
        for (int h = threadIdx.x; h < hidden; h += blockDim.x) orow[h] = from_f32<TO>(v[h] * inv * w[h]);
    }
}

template <typename TX, typename TD, typename TO>
static int launch_rmsnorm(void* x, const void* delta, const float* w, void* out, const int32_t* rows,
                          int num_rows, int hidden, float eps, int write_sum, int delta_parts,
                          long long delta_part_stride, cudaStream_t s) {
    const size_t smem = (static_cast<size_t>((hidden + 7) & ~7) + 33) * sizeof(float);
    const int vec = (hidden % 8 == 0) && aligned16(x) && aligned16(out) && aligned16(w) && (!delta || aligned16(delta));
    if (smem > 200 * 1024) return LLM_REFUSED_SIZE;
    auto kern = rmsnorm_kernel<TX, TD, TO>;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   static_cast<int>(smem));
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
    launch_pdl(kern, dim3(num_rows), dim3(threads), smem, s, static_cast<TX*>(x), static_cast<const TD*>(delta), w,
                                         static_cast<TO*>(out), rows, hidden, eps, write_sum, vec, delta_parts, delta_part_stride);
    return launch_status();
}

// x: [*, hidden] (x_dtype), delta: same shape or null (delta_dtype), w: float32 [hidden],
// out: [num_rows, hidden] (out_dtype), rows: int32 [num_rows] or null.  delta may be given as
// delta_parts tensors of x's shape, delta_part_stride elements apart, that are added up on the fly.
extern "C" int llm_rmsnorm(void* x, int x_dtype, const void* delta, int delta_dtype, const float* w,
                           void* out, int out_dtype, const int32_t* rows, int num_rows, int hidden,
                           float eps, int write_sum, int delta_parts, long long delta_part_stride,
                           uintptr_t stream) {
    if (num_rows <= 0) return LLM_OK;
    if (hidden <= 0) return LLM_REFUSED_SIZE;
    if (write_sum && rows) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (!delta) delta_dtype = x_dtype;
    const int key = x_dtype * 4 + delta_dtype * 2 + out_dtype;
#define CASE(k, TX, TD, TO)                                                                     \
    case k:                                                                                       \
        return launch_rmsnorm<TX, TD, TO>(x, delta, w, out, rows, num_rows, hidden, eps, write_sum,       \
                                          delta_parts < 1 ? 1 : delta_parts, delta_part_stride, s);
    switch (key) {
        CASE(0, float, float, float)
        CASE(1, float, float, bf16)
        CASE(2, float, bf16, float)
        CASE(3, float, bf16, bf16)
        CASE(4, bf16, float, float)
        CASE(5, bf16, float, bf16)
        CASE(6, bf16, bf16, float)
        CASE(7, bf16, bf16, bf16)
    }
#undef CASE
    return LLM_REFUSED_DTYPE;
}
