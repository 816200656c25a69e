// Token embedding: out[t, :] = table[ids[t], :], written as float32 (the residual stream is
// held in 32-bit).  An id outside [0, vocab) writes a zero row and records the first such
// token in `status` ({code, token index}); nothing traps.  The reference does the same gather
// with one element per thread and a blocking read of its error flag (src/layers/embedding.cu:91-158).
// A negative id -1-j stands for feedback[j]: the token that the previous step sampled into a
// device buffer, which the host has not read yet when it launches this step.
//
// Also here: the small scatter that applies a step's block-table changes on the device.
#include "common.cuh"

template <typename T>
__global__ void embedding_gather_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table,
                                        float* __restrict__ out, int hidden, int vocab,
                                        int32_t* __restrict__ status, const int32_t* __restrict__ feedback,
                                        int feedback_len) {
    pdl_begin();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 && feedback != nullptr && -1 - id < feedback_len) id = feedback[-1 - id];
    float* o = out + static_cast<size_t>(t) * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && atomicCAS(status, 0, 1) == 0) status[1] = t;
        for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = 0.0f;
        return;
    }
    const T* row = table + static_cast<size_t>(id) * hidden;
    if ((hidden & 7) == 0) {
        for (int h = threadIdx.x * 8; h < hidden; h += blockDim.x * 8) {
            float v[8];
            load8(row + h, v);
            store8(o + h, v);
        }
    } else {
        for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = to_f32(row[h]);
    }
}

extern "C" int llm_embedding_gather(const int32_t* ids, const void* table, int table_dtype, float* out,
                                    int num_tokens, int hidden, int vocab, int32_t* status,
                                    const int32_t* feedback, int feedback_len, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (hidden <= 0 || vocab <= 0) return LLM_REFUSED_SIZE;
    if ((hidden & 7) == 0 && (!aligned16(table) || !aligned16(out))) return LLM_REFUSED_ALIGN;
    const int threads = hidden >= 2048 ? 256 : 128;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (table_dtype == LLM_DT_F32)
        launch_pdl((embedding_gather_kernel<float>), dim3(num_tokens), dim3(threads), 0, s, 
            ids, static_cast<const float*>(table), out, hidden, vocab, status, feedback, feedback_len);
    else if (table_dtype == LLM_DT_BF16)
        launch_pdl((embedding_gather_kernel<bf16>), dim3(num_tokens), dim3(threads), 0, s, 
            ids, static_cast<const bf16*>(table), out, hidden, vocab, status, feedback, feedback_len);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}

// dst[index[i]] = value[i] for i < *count (count lives on the device so that a captured
// graph can replay with a different number of updates; a null count means max_count).  An index outside [0, dst_len)
// is skipped and recorded in status.
__global__ void scatter_int32_kernel(int32_t* __restrict__ dst, long long dst_len,
                                     const int32_t* __restrict__ index, const int32_t* __restrict__ value,
                                     const int32_t* __restrict__ count, int max_count,
                                     int32_t* __restrict__ status) {
    // No early invitation here: kernels later in the step read the tables before their own
    // griddepcontrol.wait (they only wait for the kernel just before them), which is safe
    // because nothing after this kernel starts until it has finished.
    pdl_wait();
    const int n = count ? min(*count, max_count) : max_count;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const long long at = index[i];
        if (at < 0 || at >= dst_len) {
            if (atomicCAS(status, 0, 2) == 0) status[1] = i;
            continue;
        }
        dst[at] = value[i];
    }
}

extern "C" int llm_scatter_int32(int32_t* dst, long long dst_len, const int32_t* index,
                                 const int32_t* value, const int32_t* count, int max_count,
                                 int32_t* status, uintptr_t stream) {
    if (max_count <= 0) return LLM_OK;
    const int threads = 256;
    const int blocks = min((max_count + threads - 1) / threads, 64);
    launch_pdl(scatter_int32_kernel, dim3(blocks), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream), 
        dst, dst_len, index, value, count, max_count, status);
    return launch_status();
}
