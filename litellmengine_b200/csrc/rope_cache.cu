// After the fused q/k/v projection: per-head RMSNorm of q and k, rotation by position, and
// the write of this step's keys and values into their cache pages, in one pass over the
// projection's output.
//
//   q, k:  x * rsqrt(mean_d(x^2) + eps) * w[d]            (one weight vector for all heads;
//                                                           src/model/qwen3.cpp:379-407)
//   rope:  pairs (i, i + r/2), i < r/2, angle = float(pos) * inv_freq[i] in 32-bit,
//          o[i] = x[i] cos - x[i+r/2] sin,  o[i+r/2] = x[i+r/2] cos + x[i] sin
//                                                          (src/layers/rotary.cu:85-117)
//   v:     written as projected (no norm, no rotation; src/model/qwen3.cpp:464-481)
//
// The cache of one stage is [num_pages, 2 (K,V), kv_heads, page_size, head_dim]; token at
// position p of the request in slot s goes to page table[s][p / page_size], row p % page_size
// (the address rule of src/engine/block_table_manager.cpp:91-122, with the tables on the device).
// A page number outside [0, num_pages) is recorded in `status` and the write is skipped.
//
// One warp handles one (token, head).  Norm weights and inv_freq may be null (no norm, no
// rotation); rotary_dim <= head_dim.  With has_kv == 0 the input holds only queries.
#include "common.cuh"

#define RC_WARPS 4

template <typename TI, typename T, typename TC>
__global__ void qk_norm_rope_kv_write_kernel(
    const TI* __restrict__ qkv, T* __restrict__ q_out, TC* __restrict__ cache,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_entry,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ block_table, int table_stride,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ inv_freq, int rotary_dim, int num_tokens, int nq, int nkv, int d,
    int page_size, int has_kv, int num_pages, int32_t* __restrict__ status, int qkv_parts,
    long long qkv_part_stride) {
    pdl_begin();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nq + (has_kv ? 2 * nkv : 0);
    const long long item = static_cast<long long>(blockIdx.x) * RC_WARPS + warp;
    if (item >= static_cast<long long>(num_tokens) * heads_total) return;
    const int t = static_cast<int>(item / heads_total);
    const int head = static_cast<int>(item - static_cast<long long>(t) * heads_total);
    float* x = smem + warp * d;
    const TI* src = qkv + static_cast<size_t>(t) * heads_total * d + static_cast<size_t>(head) * d;

    float ss = 0.0f;
    for (int i = lane; i < d; i += 32) {
        float v = to_f32(src[i]);
        for (int part = 1; part < qkv_parts; ++part) v += to_f32(src[part * qkv_part_stride + i]);   // k-splits of the product
        x[i] = v;
        ss += v * v;
    }
    __syncwarp();
    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    const float* nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
    if (nw) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / static_cast<float>(d) + eps);
        for (int i = lane; i < d; i += 32) x[i] = x[i] * inv * nw[i];
        __syncwarp();
    }
    const int pos = positions[t];
    if ((is_q || is_k) && inv_freq) {
        const int half = rotary_dim >> 1;
        for (int i = lane; i < half; i += 32) {
            const float ang = static_cast<float>(pos) * inv_freq[i];
            float s, c;
            sincosf(ang, &s, &c);
            const float x1 = x[i], x2 = x[i + half];
            x[i] = x1 * c - x2 * s;
            x[i + half] = x2 * c + x1 * s;
        }
        __syncwarp();
    }
    if (is_q) {
        T* dst = q_out + static_cast<size_t>(t) * nq * d + static_cast<size_t>(head) * d;
        for (int i = lane; i < d; i += 32) dst[i] = from_f32<T>(x[i]);
        return;
    }
    const int kv_head = is_k ? head - nq : head - nq - nkv;
    const int slot = entry_slot[token_entry[t]];
    const int logical = pos / page_size;
    const int page = (pos >= 0 && logical < table_stride)
                         ? block_table[static_cast<size_t>(slot) * table_stride + logical] : -1;
    if (page < 0 || page >= num_pages) {
        if (lane == 0 && atomicCAS(status, 0, 3) == 0) status[1] = t;
        return;
    }
    TC* dst = cache + ((static_cast<size_t>(page) * 2 + (is_k ? 0 : 1)) * nkv + kv_head) * page_size * d +
              static_cast<size_t>(pos % page_size) * d;
    for (int i = lane; i < d; i += 32) dst[i] = from_f32<TC>(x[i]);
}

// qkv: [T, heads_total * d] (qkv_dtype); q_out: [T, nq * d] (q_dtype); cache (cache_dtype).
extern "C" int llm_qk_norm_rope_kv_write(
    const void* qkv, int qkv_dtype, void* q_out, int q_dtype, void* cache, int cache_dtype,
    const int32_t* positions,
    const int32_t* token_entry, const int32_t* entry_slot, const int32_t* block_table, int table_stride,
    const float* q_norm_w, const float* k_norm_w, float eps, const float* inv_freq, int rotary_dim,
    int num_tokens, int nq, int nkv, int d, int page_size, int has_kv, int num_pages, int32_t* status,
    int qkv_parts, long long qkv_part_stride, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (nq <= 0 || nkv <= 0 || d <= 0 || page_size <= 0 || rotary_dim < 0 || rotary_dim > d ||
        (rotary_dim & 1))
        return LLM_REFUSED_SIZE;
    const size_t smem = static_cast<size_t>(RC_WARPS) * d * sizeof(float);
    if (smem > 48 * 1024) return LLM_REFUSED_SIZE;
    const int heads_total = nq + (has_kv ? 2 * nkv : 0);
    const long long items = static_cast<long long>(num_tokens) * heads_total;
    const unsigned blocks = static_cast<unsigned>((items + RC_WARPS - 1) / RC_WARPS);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define LAUNCH(TI, T, TC)                                                                           \
    launch_pdl((qk_norm_rope_kv_write_kernel<TI, T, TC>), dim3(blocks), dim3(RC_WARPS * 32), smem, s,                     \
        static_cast<const TI*>(qkv), static_cast<T*>(q_out), static_cast<TC*>(cache), positions,    \
        token_entry, entry_slot, block_table, table_stride, q_norm_w, k_norm_w, eps, inv_freq,      \
        rotary_dim, num_tokens, nq, nkv, d, page_size, has_kv, num_pages, status,                    \
        qkv_parts < 1 ? 1 : qkv_parts, qkv_part_stride)
    const int key = qkv_dtype * 4 + q_dtype * 2 + cache_dtype;
    if (key == 0) LAUNCH(float, float, float);
    else if (key == 3) LAUNCH(float, bf16, bf16);
    else if (key == 7) LAUNCH(bf16, bf16, bf16);
    else if (key == 1) LAUNCH(float, float, bf16);
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
    return launch_status();
}
