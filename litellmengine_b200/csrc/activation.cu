// SwiGLU's elementwise middle: out[t, i] = silu(gu[t, i]) * gu[t, inter + i], silu(g) = g / (1 + exp(-g))
// in 32-bit (src/ops/silu_and_mul.cu:44-46,76-79).  The gate and up projections are one fused
// matrix product, so both halves of a row sit side by side.
// Also the plain residual add h += delta in 32-bit (src/ops/add.cu:16-27).
#include "common.cuh"
#include <algorithm>

__device__ __forceinline__ float silu(float g) { return g / (1.0f + expf(-g)); }

// grid (blocks along the row, tokens): a thread takes 8 consecutive features of one token.
template <typename T>
__global__ void silu_and_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter) {
    pdl_begin();
    const size_t t = blockIdx.y;
    const T* g = gu + t * 2 * inter;
    const T* u = g + inter;
    T* o = out + t * inter;
    if ((inter & 7) == 0) {
        const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
        if (i < inter) {
            float a[8], b[8], r[8];
            load8(g + i, a);
            load8(u + i, b);
#pragma unroll
            for (int k = 0; k < 8; ++k) r[k] = silu(a[k]) * b[k];
            store8(o + i, r);
        }
    } else {
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < inter; i += gridDim.x * blockDim.x)
            o[i] = from_f32<T>(silu(to_f32(g[i])) * to_f32(u[i]));
    }
}

extern "C" int llm_silu_and_mul(const void* gu, void* out, int dtype, int num_tokens, int inter,
                                uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (inter <= 0 || num_tokens > 65535) return LLM_REFUSED_SIZE;
    if ((inter & 7) == 0 && (!aligned16(gu) || !aligned16(out))) return LLM_REFUSED_ALIGN;
    const int threads = 256;
    const int per_row = (inter & 7) == 0 ? inter / 8 : inter;
    const dim3 grid(std::min((per_row + threads - 1) / threads, 4096), num_tokens);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == LLM_DT_F32)
        launch_pdl((silu_and_mul_kernel<float>), grid, dim3(threads), 0, s, static_cast<const float*>(gu),
                   static_cast<float*>(out), inter);
    else if (dtype == LLM_DT_BF16)
        launch_pdl((silu_and_mul_kernel<bf16>), grid, dim3(threads), 0, s, static_cast<const bf16*>(gu),
                   static_cast<bf16*>(out), inter);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}

// The same over a product left as `slices` float32 partial sums [slices, tokens, 2*inter]: the
// slices are added in order and, for a bfloat16 result, rounded to bfloat16 first, which is
// what reading the finished bfloat16 product would have given.
template <typename T>
__global__ void silu_and_mul_parts_kernel(const float* __restrict__ parts, int slices, T* __restrict__ out, int inter,
                                          long long slice_stride) {
    pdl_begin();
    const size_t t = blockIdx.y;
    const float* g = parts + t * 2 * inter;
    T* o = out + t * inter;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < inter; i += gridDim.x * blockDim.x) {
        float a = 0.0f, b = 0.0f;
        for (int z = 0; z < slices; ++z) {
            a += g[z * slice_stride + i];
            b += g[z * slice_stride + inter + i];
        }
        o[i] = from_f32<T>(silu(to_f32(from_f32<T>(a))) * to_f32(from_f32<T>(b)));
    }
}

extern "C" int llm_silu_and_mul_parts(const float* parts, int slices, void* out, int dtype, int num_tokens, int inter,
                                      uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (inter <= 0 || num_tokens > 65535 || slices < 1) return LLM_REFUSED_SIZE;
    const int threads = 256;
    const dim3 grid(std::min((inter + threads - 1) / threads, 4096), num_tokens);
    const long long stride = static_cast<long long>(num_tokens) * 2 * inter;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == LLM_DT_F32)
        launch_pdl((silu_and_mul_parts_kernel<float>), grid, dim3(threads), 0, s, parts, slices, static_cast<float*>(out), inter, stride);
    else if (dtype == LLM_DT_BF16)
        launch_pdl((silu_and_mul_parts_kernel<bf16>), grid, dim3(threads), 0, s, parts, slices, static_cast<bf16*>(out), inter, stride);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}

template <typename T>
__global__ void residual_add_kernel(float* __restrict__ h, const T* __restrict__ delta, long long n) {
    pdl_begin();
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride)
        h[i] += to_f32(delta[i]);
}

extern "C" int llm_residual_add(float* h, const void* delta, int delta_dtype, long long n, uintptr_t stream) {
    if (n <= 0) return LLM_OK;
    const int threads = 256;
    const int blocks = static_cast<int>(std::min<long long>((n + threads - 1) / threads, 148LL * 16));
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (delta_dtype == LLM_DT_F32)
        launch_pdl((residual_add_kernel<float>), dim3(blocks), dim3(threads), 0, s, h, static_cast<const float*>(delta), n);
    else if (delta_dtype == LLM_DT_BF16)
        launch_pdl((residual_add_kernel<bf16>), dim3(blocks), dim3(threads), 0, s, h, static_cast<const bf16*>(delta), n);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}
