// Paged causal attention for any mix of tokens, any head size up to 256 in steps of 16, any
// head counts, float32 or bfloat16 — the kernel of the 32-bit path and the fallback of the
// bfloat16 path for sizes its tuned kernels do not take.
//
// For the query token t of the request in slot s at position p, head h (kv head h / group):
//     keys j in [lo, p],  lo = 0 or p - window + 1 with a window
//     s_j = (q . k_j) * scale;  softmax over j in 32-bit;  out = sum_j p_j v_j
// with the running-maximum form of src/ops/attention.cu:204-249 applied to tiles of 32 keys
// (the reference folds one key at a time; its paged kernel is src/ops/attention.cu:577-668).
// Keys and values are read straight from the pages through the device-resident block table,
// so prompt portions at any past length, single decoded tokens and mixed batches all take
// this one path; the step's own keys were written to the pages before this kernel runs.
//
// One thread block of AG_WARPS warps per (token, head).  The keys are cut into tiles of 32; warp w
// takes tiles w, w + AG_WARPS, ... : each lane scores one key of the tile (a 16-byte-vectorised dot
// product against q held in shared memory), the warp reduces max and sum, then every lane
// accumulates its output dimensions over the tile's values.  At the end the warps' running
// (maximum, sum, output) triples are merged through shared memory in warp order.  Which warp takes
// which tile depends only on (lo, p), never on the batch, so a position's result does not depend
// on how the work was cut.  (With one warp per (token, head) a decode step of 8 requests at a
// context of 4,096 kept two warps an SM busy: 5 ms a layer.)
#include "common.cuh"
#include <math_constants.h>

#define AG_WARPS 8
#define AG_MAX_D 256

template <typename T, typename TC>
__global__ void paged_attention_generic_kernel(
    const T* __restrict__ q, T* __restrict__ out, const TC* __restrict__ cache,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_entry,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ block_table, int table_stride,
    int num_tokens, int nq, int nkv, int d, int page_size, int window, float scale, int num_pages,
    int32_t* __restrict__ status) {
    pdl_begin();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = blockIdx.x;
    const int t = static_cast<int>(item / nq);
    const int h = static_cast<int>(item - static_cast<long long>(t) * nq);
    const int kvh = h / (nq / nkv);
    float* qs = smem;                                  // [d]
    float* merge = smem + d;                           // [AG_WARPS][d + 2]: output, maximum, sum of each warp
    const T* qrow = q + (static_cast<size_t>(t) * nq + h) * d;
    for (int i = threadIdx.x; i < d; i += AG_WARPS * 32) qs[i] = to_f32(qrow[i]) * scale;
    __syncthreads();

    const int pos = positions[t];
    const int slot = entry_slot[token_entry[t]];
    const int32_t* table = block_table + static_cast<size_t>(slot) * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const size_t head_stride = static_cast<size_t>(page_size) * d;       // one kv head inside a page
    const size_t page_stride = 2 * static_cast<size_t>(nkv) * head_stride;

    float m = -CUDART_INF_F, l = 0.0f;
    float acc[AG_MAX_D / 32];
#pragma unroll
    for (int r = 0; r < AG_MAX_D / 32; ++r) acc[r] = 0.0f;

    for (int base = lo + 32 * warp; base <= pos; base += 32 * AG_WARPS) {
        const int j = base + lane;
        const bool valid = j <= pos;
        long long koff = -1;
        float s = -CUDART_INF_F;
        if (valid) {
            const int logical = j / page_size;
            const int page = logical < table_stride ? table[logical] : -1;
            if (page < 0 || page >= num_pages) {
                if (atomicCAS(status, 0, 4) == 0) status[1] = t;
            } else {
                koff = static_cast<long long>(page) * page_stride + kvh * head_stride +
                       static_cast<size_t>(j % page_size) * d;
                const TC* kr = cache + koff;
                float dot = 0.0f;
                for (int i = 0; i < d; i += 8) {
                    float kv[8];
                    load8(kr + i, kv);
#pragma unroll
                    for (int u = 0; u < 8; ++u) dot += qs[i + u] * kv[u];
                }
                s = dot;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = (koff >= 0) ? expf(s - m_new) : 0.0f;
        const float alpha = (m == -CUDART_INF_F) ? 0.0f : expf(m - m_new);
        l = l * alpha + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int r = 0; r < AG_MAX_D / 32; ++r) acc[r] *= alpha;
        const int count = min(32, pos - base + 1);
        const long long voff = koff + static_cast<long long>(nkv) * head_stride;   // V follows K in a page
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long vo = __shfl_sync(0xffffffffu, voff, jj);
            if (pj == 0.0f) continue;                  // also skips keys whose page was refused
            const TC* vr = cache + vo;
#pragma unroll
            for (int r = 0; r < AG_MAX_D / 32; ++r) {
                const int i = lane + 32 * r;
                if (i < d) acc[r] += pj * to_f32(vr[i]);
            }
        }
    }
    // merge the warps' partial results, in warp order (a warp without tiles has m = -inf, l = 0)
    float* mine = merge + warp * (d + 2);
#pragma unroll
    for (int r = 0; r < AG_MAX_D / 32; ++r) {
        const int i = lane + 32 * r;
        if (i < d) mine[i] = acc[r];
    }
    if (lane == 0) { mine[d] = m; mine[d + 1] = l; }
    __syncthreads();
    float m_all = -CUDART_INF_F;
    for (int w2 = 0; w2 < AG_WARPS; ++w2) m_all = fmaxf(m_all, merge[w2 * (d + 2) + d]);
    float l_all = 0.0f;
    for (int w2 = 0; w2 < AG_WARPS; ++w2) {
        const float mw = merge[w2 * (d + 2) + d];
        if (mw != -CUDART_INF_F) l_all += merge[w2 * (d + 2) + d + 1] * expf(mw - m_all);
    }
    T* orow = out + (static_cast<size_t>(t) * nq + h) * d;
    const float inv = 1.0f / l_all;
    for (int i = threadIdx.x; i < d; i += AG_WARPS * 32) {
        float o = 0.0f;
        for (int w2 = 0; w2 < AG_WARPS; ++w2) {
            const float mw = merge[w2 * (d + 2) + d];
            if (mw != -CUDART_INF_F) o += merge[w2 * (d + 2) + i] * expf(mw - m_all);
        }
        orow[i] = from_f32<T>(o * inv);
    }
}

extern "C" int llm_paged_attention_generic(
    const void* q, void* out, int dtype, const void* cache, int cache_dtype, const int32_t* positions,
    const int32_t* token_entry, const int32_t* entry_slot, const int32_t* block_table, int table_stride,
    int num_tokens, int nq, int nkv, int d, int page_size, int window, float scale, int num_pages,
    int32_t* status, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || d <= 0 || d > AG_MAX_D || (d & 15) || page_size <= 0)
        return LLM_REFUSED_SIZE;
    if (!aligned16(cache)) return LLM_REFUSED_ALIGN;
    const size_t smem = (static_cast<size_t>(d) + static_cast<size_t>(AG_WARPS) * (d + 2)) * sizeof(float);
    const long long items = static_cast<long long>(num_tokens) * nq;
    if (items > 0x7fffffffLL) return LLM_REFUSED_SIZE;
    const unsigned blocks = static_cast<unsigned>(items);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define LAUNCH(T, TC)                                                                              \
    launch_pdl((paged_attention_generic_kernel<T, TC>), dim3(blocks), dim3(AG_WARPS * 32), smem, s,                      \
        static_cast<const T*>(q), static_cast<T*>(out), static_cast<const TC*>(cache), positions,  \
        token_entry, entry_slot, block_table, table_stride, num_tokens, nq, nkv, d, page_size,     \
        window, scale, num_pages, status)
    if (dtype == LLM_DT_F32 && cache_dtype == LLM_DT_F32) LAUNCH(float, float);
    else if (dtype == LLM_DT_BF16 && cache_dtype == LLM_DT_BF16) LAUNCH(bf16, bf16);
    else if (dtype == LLM_DT_F32 && cache_dtype == LLM_DT_BF16) LAUNCH(float, bf16);
    else if (dtype == LLM_DT_BF16 && cache_dtype == LLM_DT_F32) LAUNCH(bf16, float);
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
    return launch_status();
}
