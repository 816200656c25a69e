// Paged attention for single decoded tokens, bfloat16, split over the keys so that a small
// batch still fills the GPU.  Memory-bound by design: every key and value row of the request's
// kv head is read once, as 16-byte (keys) and 8-byte (values) loads, and serves all the query
// heads of the group.
//
// For the token in row r (request slot s, position p), kv head c, split i of n:
//     keys j in [lo + i*len, lo + (i+1)*len) ∩ [lo, p],  lo = 0 or p - window + 1
//     per query head h of the group: s_j = (q_h . k_j) * scale, running max m, sum l of
//     exp(s_j - m), acc = sum exp(s_j - m) v_j      -- all in 32-bit
// (the running-maximum form of src/ops/attention.cu:577-668, which walks the keys one by one
// with one block per query head).  The partial (m, l, acc) of each split go to scratch memory;
// `paged_decode_combine` merges them: out = sum_i acc_i e^{m_i - M} / sum_i l_i e^{m_i - M}.
//
// One CTA of 4 warps per (split, kv head, token).  A warp takes tiles of 32 keys: each lane
// scores one key against all G query heads (q sits in shared memory, pre-scaled), the warp
// reduces max and sum per head, then each lane accumulates its D/32 output dimensions over
// the tile's 32 value rows.  The 4 warps' states are merged through shared memory.
// Built for head sizes 64 and 128 and groups of 1 to 8; other sizes use the generic kernel.
#include "common.cuh"
#include <math_constants.h>

#define AD_WARPS 4
#define AD_THREADS (AD_WARPS * 32)

template <int D, int G>
__global__ void __launch_bounds__(AD_THREADS) paged_decode_attention_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ cache, const int32_t* __restrict__ rows,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_entry,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ block_table, int table_stride,
    float* __restrict__ part_acc, float* __restrict__ part_ml, bf16* __restrict__ out, int nq, int nkv,
    int page_size, int window, float scale, int num_pages, int num_splits, int32_t* __restrict__ status) {
    constexpr int DPL = D / 32;                     // output dims per lane
    constexpr int GP = (G <= 4) ? 4 : 8;            // heads padded so that p of one key is 1-2 float4
    __shared__ __align__(16) float q_s[G * D];
    __shared__ __align__(16) float p_s[AD_WARPS][32][GP];
    __shared__ long long voff_s[AD_WARPS][32];
    __shared__ float m_s[AD_WARPS][G], l_s[AD_WARPS][G];
    __shared__ __align__(16) float acc_s[AD_WARPS][G][D];

    const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = rows ? rows[r] : r;
    const int pos = positions[t];
    const int slot = entry_slot[token_entry[t]];
    const int32_t* table = block_table + static_cast<size_t>(slot) * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_keys = pos - lo + 1;
    int per_split = (n_keys + num_splits - 1) / num_splits;
    per_split = (per_split + 31) & ~31;
    const int k_begin = lo + split * per_split;
    const int k_end = min(pos + 1, k_begin + per_split);
    const int h0 = kvh * G;                          // first query head of the group

    for (int i = threadIdx.x; i < G * D; i += AD_THREADS)
        q_s[i] = to_f32(q[(static_cast<size_t>(t) * nq + h0) * D + i]) * scale;
    __syncthreads();

    const size_t head_stride = static_cast<size_t>(page_size) * D;
    const size_t page_stride = 2 * static_cast<size_t>(nkv) * head_stride;
    const long long v_shift = static_cast<long long>(nkv) * head_stride;

    float m[G], l[G], acc[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -CUDART_INF_F;
        l[g] = 0.0f;
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[g][e] = 0.0f;
    }

    for (int base = k_begin + warp * 32; base < k_end; base += AD_WARPS * 32) {
        const int j = base + lane;
        long long koff = -1;
        if (j < k_end) {
            const int logical = j / page_size;
            const int page = logical < table_stride ? table[logical] : -1;
            if (page < 0 || page >= num_pages) {
                if (atomicCAS(status, 0, 4) == 0) status[1] = t;
            } else {
                koff = static_cast<long long>(page) * page_stride + kvh * head_stride +
                       static_cast<long long>(j - logical * page_size) * D;
            }
        }
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) s[g] = 0.0f;
        if (koff >= 0) {
            const bf16* kr = cache + koff;
#pragma unroll 4
            for (int c = 0; c < D; c += 8) {
                float kf[8];
                load8(kr + c, kf);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float4 qa = *reinterpret_cast<const float4*>(q_s + g * D + c);
                    const float4 qb = *reinterpret_cast<const float4*>(q_s + g * D + c + 4);
                    s[g] += qa.x * kf[0] + qa.y * kf[1] + qa.z * kf[2] + qa.w * kf[3] + qb.x * kf[4] +
                            qb.y * kf[5] + qb.z * kf[6] + qb.w * kf[7];
                }
            }
        }
        voff_s[warp][lane] = koff + v_shift;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float sv = (koff >= 0) ? s[g] : -CUDART_INF_F;
            const float m_new = fmaxf(m[g], warp_max(sv));
            const float p = (koff >= 0) ? __expf(sv - m_new) : 0.0f;
            const float alpha = (m[g] == -CUDART_INF_F) ? 0.0f : __expf(m[g] - m_new);
            l[g] = l[g] * alpha + warp_sum(p);
            m[g] = m_new;
#pragma unroll
            for (int e = 0; e < DPL; ++e) acc[g][e] *= alpha;
            p_s[warp][lane][g] = p;
        }
        __syncwarp();
        const int count = min(32, k_end - base);
#pragma unroll 4
        for (int jj = 0; jj < count; ++jj) {
            float pv[GP];
            *reinterpret_cast<float4*>(pv) = *reinterpret_cast<const float4*>(&p_s[warp][jj][0]);
            if (GP == 8) *reinterpret_cast<float4*>(pv + 4) = *reinterpret_cast<const float4*>(&p_s[warp][jj][4]);
            const long long vo = voff_s[warp][jj];
            if (vo < v_shift) continue;              // the key's page was refused
            const bf16* vr = cache + vo + lane * DPL;
            float vf[DPL];
            if (DPL == 4) {
                const uint2 raw = *reinterpret_cast<const uint2*>(vr);
                const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                vf[0] = a.x; vf[1] = a.y; vf[2] = b.x; vf[3] = b.y;
            } else {
                const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vr));
                vf[0] = a.x; vf[1] = a.y;
            }
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int e = 0; e < DPL; ++e) acc[g][e] += pv[g] * vf[e];
        }
        __syncwarp();
    }

    // merge the warps' states
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) {
            m_s[warp][g] = m[g];
            l_s[warp][g] = l[g];
        }
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc_s[warp][g][lane * DPL + e] = acc[g][e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * D; i += AD_THREADS) {
        const int g = i / D, dim = i - g * D;
        float M = m_s[0][g];
#pragma unroll
        for (int w = 1; w < AD_WARPS; ++w) M = fmaxf(M, m_s[w][g]);
        float a = 0.0f, L = 0.0f;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) {
            const float f = (m_s[w][g] == -CUDART_INF_F) ? 0.0f : __expf(m_s[w][g] - M);
            a += acc_s[w][g][dim] * f;
            L += l_s[w][g] * f;
        }
        const size_t hrow = static_cast<size_t>(r) * nq + h0 + g;
        if (num_splits == 1) {
            out[(static_cast<size_t>(t) * nq + h0 + g) * D + dim] = __float2bfloat16_rn(a / L);
        } else {
            part_acc[(hrow * num_splits + split) * D + dim] = a;
            if (dim == 0) {
                part_ml[(hrow * num_splits + split) * 2] = M;
                part_ml[(hrow * num_splits + split) * 2 + 1] = L;
            }
        }
    }
}

// One block per (token row, query head): merge the splits.
template <int D>
__global__ void paged_decode_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                            const int32_t* __restrict__ rows, bf16* __restrict__ out, int nq,
                                            int num_splits) {
    const int r = blockIdx.x, h = blockIdx.y;
    const int t = rows ? rows[r] : r;
    const size_t hrow = static_cast<size_t>(r) * nq + h;
    float M = -CUDART_INF_F;
    for (int s = 0; s < num_splits; ++s)
        if (part_ml[(hrow * num_splits + s) * 2 + 1] > 0.0f) M = fmaxf(M, part_ml[(hrow * num_splits + s) * 2]);
    for (int dim = threadIdx.x; dim < D; dim += blockDim.x) {
        float a = 0.0f, L = 0.0f;
        for (int s = 0; s < num_splits; ++s) {
            const float ls = part_ml[(hrow * num_splits + s) * 2 + 1];
            if (ls > 0.0f) {                          // an empty split wrote no acc
                const float f = __expf(part_ml[(hrow * num_splits + s) * 2] - M);
                a += part_acc[(hrow * num_splits + s) * D + dim] * f;
                L += ls * f;
            }
        }
        out[(static_cast<size_t>(t) * nq + h) * D + dim] = __float2bfloat16_rn(a / L);
    }
}

template <int D, int G>
static int launch_decode(const bf16* q, const bf16* cache, const int32_t* rows, const int32_t* positions,
                         const int32_t* token_entry, const int32_t* entry_slot, const int32_t* block_table,
                         int table_stride, float* part_acc, float* part_ml, bf16* out, int n_rows, int nq, int nkv,
                         int page_size, int window, float scale, int num_pages, int num_splits, int32_t* status,
                         cudaStream_t s) {
    dim3 grid(num_splits, nkv, n_rows);
    paged_decode_attention_kernel<D, G><<<grid, AD_THREADS, 0, s>>>(
        q, cache, rows, positions, token_entry, entry_slot, block_table, table_stride, part_acc, part_ml, out, nq,
        nkv, page_size, window, scale, num_pages, num_splits, status);
    int rc = launch_status();
    if (rc != LLM_OK || num_splits == 1) return rc;
    dim3 cgrid(n_rows, nq);
    paged_decode_combine_kernel<D><<<cgrid, D <= 64 ? 64 : 128, 0, s>>>(part_acc, part_ml, rows, out, nq, num_splits);
    return launch_status();
}

// Whether (head_dim, group) has a tuned kernel; the Python side asks before choosing.
extern "C" int llm_paged_decode_supported(int d, int group) {
    return (d == 64 || d == 128) && group >= 1 && group <= 8;
}

// Floats of scratch the call needs: part_acc then part_ml.
extern "C" long long llm_paged_decode_scratch_floats(int n_rows, int nq, int d, int num_splits) {
    if (num_splits <= 1) return 0;
    return static_cast<long long>(n_rows) * nq * num_splits * (d + 2);
}

// q, out: bfloat16 [T, nq*d]; cache: bfloat16 [pages, 2, nkv, page_size, d]; rows: int32 [n_rows] token
// rows to attend for (null: rows 0..n_rows-1); scratch: float32, llm_paged_decode_scratch_floats long.
extern "C" int llm_paged_attention_decode(
    const void* q, void* out, const void* cache, const int32_t* rows, int n_rows, const int32_t* positions,
    const int32_t* token_entry, const int32_t* entry_slot, const int32_t* block_table, int table_stride, int nq,
    int nkv, int d, int page_size, int window, float scale, int num_pages, int num_splits, float* scratch,
    int32_t* status, uintptr_t stream) {
    if (n_rows <= 0) return LLM_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || num_splits < 1 || num_splits > 65535)
        return LLM_REFUSED_SIZE;
    const int group = nq / nkv;
    if (!llm_paged_decode_supported(d, group)) return LLM_REFUSED_SIZE;
    if (!aligned16(cache) || !aligned16(q) || (num_splits > 1 && (!scratch || !aligned16(scratch))))
        return LLM_REFUSED_ALIGN;
    float* part_acc = scratch;
    float* part_ml = scratch ? scratch + static_cast<size_t>(n_rows) * nq * num_splits * d : nullptr;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define CASE(DD, GG)                                                                                        \
    if (d == DD && group == GG)                                                                             \
        return launch_decode<DD, GG>(static_cast<const bf16*>(q), static_cast<const bf16*>(cache), rows,    \
                                     positions, token_entry, entry_slot, block_table, table_stride,         \
                                     part_acc, part_ml, static_cast<bf16*>(out), n_rows, nq, nkv,           \
                                     page_size, window, scale, num_pages, num_splits, status, s);
    CASE(64, 1) CASE(64, 2) CASE(64, 3) CASE(64, 4) CASE(64, 5) CASE(64, 6) CASE(64, 7) CASE(64, 8)
    CASE(128, 1) CASE(128, 2) CASE(128, 3) CASE(128, 4) CASE(128, 5) CASE(128, 6) CASE(128, 7) CASE(128, 8)
#undef CASE
    return LLM_REFUSED_SIZE;
}
