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
#include <type_traits>

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

// ---- head sizes 64 and 128, whole-head rotation: everything in registers -----------------------
// A lane holds D/32 consecutive elements of a head, so a head is one 8- or 16-byte access per
// lane, and element i's rotation partner i + D/2 sits in lane + 16 (one shuffle).  A warp takes
// HPW heads of one token at once: their loads are in flight together, and the token's sines and
// cosines are computed once for all of them.
template <int N> __device__ __forceinline__ void rc_load(const float* p, float (&v)[N]) {
    if constexpr (N == 4) { const float4 a = *reinterpret_cast<const float4*>(p); v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; }
    else { const float2 a = *reinterpret_cast<const float2*>(p); v[0] = a.x; v[1] = a.y; }
}
template <int N> __device__ __forceinline__ void rc_load(const bf16* p, float (&v)[N]) {
    if constexpr (N == 4) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    } else {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
        v[0] = a.x; v[1] = a.y;
    }
}
template <int N> __device__ __forceinline__ void rc_store(float* p, const float (&v)[N]) {
    if constexpr (N == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
}
template <int N> __device__ __forceinline__ void rc_store(bf16* p, const float (&v)[N]) {
    if constexpr (N == 4) {
        uint2 raw;
        *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v[0], v[1]);
        *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p) = raw;
    } else {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
    }
}

template <int D, int HPW, typename TI, typename T, typename TC>
__global__ void __launch_bounds__(RC_WARPS * 32) qk_norm_rope_kv_write_vec_kernel(
    const TI* __restrict__ qkv, T* __restrict__ q_out, TC* __restrict__ cache,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_entry,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ block_table, int table_stride,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ inv_freq, int num_tokens, int nq, int nkv, int page_size, int has_kv,
    int num_pages, int32_t* __restrict__ status, int qkv_parts, long long qkv_part_stride,
    const float4* __restrict__ angles) {
    constexpr int N = D / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nq + (has_kv ? 2 * nkv : 0);
    const int groups = (heads_total + HPW - 1) / HPW;
    const long long item = static_cast<long long>(blockIdx.x) * RC_WARPS + warp;
    if (item >= static_cast<long long>(num_tokens) * groups) return;
    const int t = static_cast<int>(item / groups);
    const int head0 = static_cast<int>(item - static_cast<long long>(t) * groups) * HPW;
    const int e0 = lane * N;                                             // this lane's first element of a head
    const TI* src = qkv + static_cast<size_t>(t) * heads_total * D + e0;

    // Before the wait for the projection: everything that comes from the step's metadata, the
    // block table and the weights (position, sines and cosines, norm weights, the page).
    const int pos = positions[t];
    float sn[N], cs[N], wq[N], wk[N];
    if (angles) {                                                        // the step's table: (sin, cos) pairs [T][D/2]
        const float4* a = angles + (static_cast<size_t>(t) * (D / 2) + (e0 & (D / 2 - 1))) / 2;
#pragma unroll
        for (int i = 0; i < N; i += 2) {
            const float4 v = a[i / 2];
            sn[i] = v.x; cs[i] = v.y; sn[i + 1] = v.z; cs[i + 1] = v.w;
        }
    } else if (inv_freq) {
#pragma unroll
        for (int i = 0; i < N; ++i) sincosf(static_cast<float>(pos) * inv_freq[(e0 + i) & (D / 2 - 1)], &sn[i], &cs[i]);
    }
    if (q_norm_w) rc_load<N>(q_norm_w + e0, wq);
    if (k_norm_w) rc_load<N>(k_norm_w + e0, wk);
    int page = -1;
    bool bad_page = false;
    if (head0 + HPW > nq && has_kv) {                                     // this warp holds a key or value head
        const int slot = entry_slot[token_entry[t]];
        const int logical = pos / page_size;
        page = (pos >= 0 && logical < table_stride) ? block_table[static_cast<size_t>(slot) * table_stride + logical] : -1;
        bad_page = page < 0 || page >= num_pages;
    }
    pdl_begin();
    if (bad_page) {
        if (lane == 0 && atomicCAS(status, 0, 3) == 0) status[1] = t;
        page = -1;
    }

    float x[HPW][N];
#pragma unroll
    for (int j = 0; j < HPW; ++j) {
        if (head0 + j < heads_total) {
            rc_load<N>(src + static_cast<size_t>(head0 + j) * D, x[j]);
            for (int part = 1; part < qkv_parts; ++part) {                // k-splits of the product
                float y[N];
                rc_load<N>(src + part * qkv_part_stride + static_cast<size_t>(head0 + j) * D, y);
#pragma unroll
                for (int i = 0; i < N; ++i) x[j][i] += y[i];
            }
        }
    }
    // second half of a head: x2 cos + x1 sin; first half: x1 cos - x2 sin
    if (inv_freq || angles) {
#pragma unroll
        for (int i = 0; i < N; ++i) sn[i] = lane < 16 ? -sn[i] : sn[i];
    }
    // A warp's heads are nearly always of one kind (queries, keys or values): the kind is then a
    // constant of the loop below instead of a choice per head.
    auto one = [&](auto kind_c, int j) {
        constexpr int KIND = decltype(kind_c)::value;                    // 0 q, 1 k, 2 v, 3 decide per head
        const int head = head0 + j;
        const bool is_q = KIND == 0 || (KIND == 3 && head < nq);
        const bool is_k = KIND == 1 || (KIND == 3 && !is_q && head < nq + nkv);
        const float* nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
        if (nw) {
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < N; ++i) ss += x[j][i] * x[j][i];
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
            for (int i = 0; i < N; ++i) x[j][i] = x[j][i] * inv * (is_q ? wq[i] : wk[i]);
        }
        if ((is_q || is_k) && (inv_freq || angles)) {
#pragma unroll
            for (int i = 0; i < N; ++i) {
                const float other = __shfl_xor_sync(0xffffffffu, x[j][i], 16);
                x[j][i] = x[j][i] * cs[i] + other * sn[i];
            }
        }
        if (is_q) {
            rc_store<N>(q_out + static_cast<size_t>(t) * nq * D + static_cast<size_t>(head) * D + e0, x[j]);
            return;
        }
        if (page < 0) return;
        const int kv_head = is_k ? head - nq : head - nq - nkv;
        TC* dst = cache + ((static_cast<size_t>(page) * 2 + (is_k ? 0 : 1)) * nkv + kv_head) * page_size * D +
                  static_cast<size_t>(pos % page_size) * D + e0;
        rc_store<N>(dst, x[j]);
    };
    const int last = min(head0 + HPW, heads_total) - 1;
#define RC_HEADS(KIND)                                                      \
    _Pragma("unroll") for (int j = 0; j < HPW; ++j) {                       \
        if (head0 + j >= heads_total) break;                                \
        one(std::integral_constant<int, KIND>{}, j);                        \
    }
    if (last < nq) { RC_HEADS(0) }
    else if (head0 >= nq && last < nq + nkv) { RC_HEADS(1) }
    else if (head0 >= nq + nkv) { RC_HEADS(2) }
    else { RC_HEADS(3) }
#undef RC_HEADS
}

template <int D, int HPW, typename TI, typename T, typename TC>
static void launch_rope_vec(const void* qkv, void* q_out, void* cache, const int32_t* positions,
                            const int32_t* token_entry, const int32_t* entry_slot, const int32_t* block_table,
                            int table_stride, const float* q_norm_w, const float* k_norm_w, float eps,
                            const float* inv_freq, int num_tokens, int nq, int nkv, int page_size, int has_kv,
                            int num_pages, int32_t* status, int qkv_parts, long long qkv_part_stride, const float* angles,
                            cudaStream_t s) {
    const int heads_total = nq + (has_kv ? 2 * nkv : 0);
    const long long items = static_cast<long long>(num_tokens) * ((heads_total + HPW - 1) / HPW);
    const unsigned blocks = static_cast<unsigned>((items + RC_WARPS - 1) / RC_WARPS);
    launch_pdl((qk_norm_rope_kv_write_vec_kernel<D, HPW, TI, T, TC>), dim3(blocks), dim3(RC_WARPS * 32), 0, s,
               static_cast<const TI*>(qkv), static_cast<T*>(q_out), static_cast<TC*>(cache), positions, token_entry,
               entry_slot, block_table, table_stride, q_norm_w, k_norm_w, eps, inv_freq, num_tokens, nq, nkv,
               page_size, has_kv, num_pages, status, qkv_parts < 1 ? 1 : qkv_parts, qkv_part_stride,
               reinterpret_cast<const float4*>(angles));
}

// The sines and cosines of a step, once for all its layers: out[t][i] = (sin, cos)(float(positions[t]) * inv_freq[i]),
// the same float32 expressions as inside the kernels above.  It does not let the next kernel start early:
// every later kernel of the step then starts after this one has finished and may read the table before its
// own griddepcontrol.wait.
__global__ void rope_angles_kernel(const int32_t* __restrict__ positions, const float* __restrict__ inv_freq,
                                   float2* __restrict__ out, int num_tokens, int half) {
    pdl_wait();
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= static_cast<long long>(num_tokens) * half) return;
    float sn, cs;
    sincosf(static_cast<float>(positions[i / half]) * inv_freq[i % half], &sn, &cs);
    out[i] = make_float2(sn, cs);
}

extern "C" int llm_rope_angles(const int32_t* positions, const float* inv_freq, float* out, int num_tokens, int half,
                               uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (half <= 0) return LLM_REFUSED_SIZE;
    const long long n = static_cast<long long>(num_tokens) * half;
    launch_pdl(rope_angles_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0,
               reinterpret_cast<cudaStream_t>(stream), positions, inv_freq, reinterpret_cast<float2*>(out), num_tokens, half);
    return launch_status();
}

// ---- the same work in two halves, for position encodings this file does not know ---------------
// A mixer whose position part is not a rotation runs `llm_qk_head_norm` (the per-head norms only:
// q and k leave as float32 [T, heads * d]), lets the part encode q and k in its own way, and then
// `llm_qk_store` (q rounded to the compute type, the encoded k and the projected v written into
// their pages by the same address rule as above).  One warp per (token, head) in both.
template <typename TI>
__global__ void qk_head_norm_kernel(const TI* __restrict__ qkv, float* __restrict__ q_out, float* __restrict__ k_out,
                                    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
                                    int num_tokens, int nq, int nkv, int d, int heads_total, int qkv_parts,
                                    long long qkv_part_stride) {
    pdl_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = nq + nkv;
    const long long item = static_cast<long long>(blockIdx.x) * RC_WARPS + warp;
    if (item >= static_cast<long long>(num_tokens) * heads) return;
    const int t = static_cast<int>(item / heads);
    const int head = static_cast<int>(item - static_cast<long long>(t) * heads);
    const bool is_q = head < nq;
    const TI* src = qkv + static_cast<size_t>(t) * heads_total * d + static_cast<size_t>(head) * d;
    float* dst = is_q ? q_out + (static_cast<size_t>(t) * nq + head) * d
                      : k_out + (static_cast<size_t>(t) * nkv + (head - nq)) * d;
    float ss = 0.0f;
    for (int i = lane; i < d; i += 32) {
        float v = to_f32(src[i]);
        for (int part = 1; part < qkv_parts; ++part) v += to_f32(src[part * qkv_part_stride + i]);
        dst[i] = v;
        ss += v * v;
    }
    const float* nw = is_q ? q_norm_w : k_norm_w;
    if (nw) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / static_cast<float>(d) + eps);
        for (int i = lane; i < d; i += 32) dst[i] = dst[i] * inv * nw[i];     // each lane rereads what it wrote
    }
}

extern "C" int llm_qk_head_norm(const void* qkv, int qkv_dtype, float* q_out, float* k_out, const float* q_norm_w,
                                const float* k_norm_w, float eps, int num_tokens, int nq, int nkv, int d, int has_kv,
                                int qkv_parts, long long qkv_part_stride, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (nq <= 0 || nkv <= 0 || d <= 0) return LLM_REFUSED_SIZE;
    const int heads_total = nq + (has_kv ? 2 * nkv : 0);
    const int heads = nq + (has_kv ? nkv : 0);
    const long long items = static_cast<long long>(num_tokens) * heads;
    const unsigned blocks = static_cast<unsigned>((items + RC_WARPS - 1) / RC_WARPS);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int parts = qkv_parts < 1 ? 1 : qkv_parts;
    if (qkv_dtype == LLM_DT_F32)
        launch_pdl(qk_head_norm_kernel<float>, dim3(blocks), dim3(RC_WARPS * 32), 0, s, static_cast<const float*>(qkv),
                   q_out, k_out, q_norm_w, k_norm_w, eps, num_tokens, nq, has_kv ? nkv : 0, d, heads_total, parts, qkv_part_stride);
    else
        launch_pdl(qk_head_norm_kernel<bf16>, dim3(blocks), dim3(RC_WARPS * 32), 0, s, static_cast<const bf16*>(qkv),
                   q_out, k_out, q_norm_w, k_norm_w, eps, num_tokens, nq, has_kv ? nkv : 0, d, heads_total, parts, qkv_part_stride);
    return launch_status();
}

template <typename TI, typename T, typename TC>
__global__ void qk_store_kernel(const float* __restrict__ q_in, const float* __restrict__ k_in, const TI* __restrict__ qkv,
                                T* __restrict__ q_out, TC* __restrict__ cache, const int32_t* __restrict__ positions,
                                const int32_t* __restrict__ token_entry, const int32_t* __restrict__ entry_slot,
                                const int32_t* __restrict__ block_table, int table_stride, int num_tokens, int nq, int nkv,
                                int d, int page_size, int has_kv, int num_pages, int32_t* __restrict__ status,
                                int qkv_parts, long long qkv_part_stride) {
    pdl_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nq + (has_kv ? 2 * nkv : 0);
    const long long item = static_cast<long long>(blockIdx.x) * RC_WARPS + warp;
    if (item >= static_cast<long long>(num_tokens) * heads_total) return;
    const int t = static_cast<int>(item / heads_total);
    const int head = static_cast<int>(item - static_cast<long long>(t) * heads_total);
    if (head < nq) {
        const float* src = q_in + (static_cast<size_t>(t) * nq + head) * d;
        T* dst = q_out + (static_cast<size_t>(t) * nq + head) * d;
        for (int i = lane; i < d; i += 32) dst[i] = from_f32<T>(src[i]);
        return;
    }
    const bool is_k = head < nq + nkv;
    const int kv_head = is_k ? head - nq : head - nq - nkv;
    const int pos = positions[t];
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
    if (is_k) {
        const float* src = k_in + (static_cast<size_t>(t) * nkv + kv_head) * d;
        for (int i = lane; i < d; i += 32) dst[i] = from_f32<TC>(src[i]);
    } else {
        const TI* src = qkv + static_cast<size_t>(t) * heads_total * d + static_cast<size_t>(head) * d;
        for (int i = lane; i < d; i += 32) {
            float v = to_f32(src[i]);
            for (int part = 1; part < qkv_parts; ++part) v += to_f32(src[part * qkv_part_stride + i]);
            dst[i] = from_f32<TC>(v);
        }
    }
}

// q_in, k_in: float32 [T, nq * d] and [T, nkv * d] as the position part left them; qkv: the projection
// (its v columns are read); q_out in q_dtype; cache in cache_dtype.
extern "C" int llm_qk_store(const float* q_in, const float* k_in, const void* qkv, int qkv_dtype, void* q_out, int q_dtype,
                            void* cache, int cache_dtype, const int32_t* positions, const int32_t* token_entry,
                            const int32_t* entry_slot, const int32_t* block_table, int table_stride, int num_tokens, int nq,
                            int nkv, int d, int page_size, int has_kv, int num_pages, int32_t* status, int qkv_parts,
                            long long qkv_part_stride, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (nq <= 0 || nkv <= 0 || d <= 0 || page_size <= 0) return LLM_REFUSED_SIZE;
    const int heads_total = nq + (has_kv ? 2 * nkv : 0);
    const long long items = static_cast<long long>(num_tokens) * heads_total;
    const unsigned blocks = static_cast<unsigned>((items + RC_WARPS - 1) / RC_WARPS);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define STORE(TI, T, TC)                                                                                          \
    launch_pdl((qk_store_kernel<TI, T, TC>), dim3(blocks), dim3(RC_WARPS * 32), 0, s, q_in, k_in,                 \
               static_cast<const TI*>(qkv), static_cast<T*>(q_out), static_cast<TC*>(cache), positions, token_entry, \
               entry_slot, block_table, table_stride, num_tokens, nq, nkv, d, page_size, has_kv, num_pages, status,  \
               qkv_parts < 1 ? 1 : qkv_parts, qkv_part_stride)
    const int key = qkv_dtype * 4 + q_dtype * 2 + cache_dtype;
    if (key == 0) STORE(float, float, float);
    else if (key == 3) STORE(float, bf16, bf16);
    else if (key == 7) STORE(bf16, bf16, bf16);
    else if (key == 1) STORE(float, float, bf16);
    else return LLM_REFUSED_DTYPE;
#undef STORE
    return launch_status();
}

// qkv: [T, heads_total * d] (qkv_dtype); q_out: [T, nq * d] (q_dtype); cache (cache_dtype).
// angles: nullptr, or the step's table from llm_rope_angles ([T][d/2] pairs; used when the whole head is rotated
// and the head size is 64 or 128, ignored otherwise).
extern "C" int llm_qk_norm_rope_kv_write(
    const void* qkv, int qkv_dtype, void* q_out, int q_dtype, void* cache, int cache_dtype,
    const int32_t* positions,
    const int32_t* token_entry, const int32_t* entry_slot, const int32_t* block_table, int table_stride,
    const float* q_norm_w, const float* k_norm_w, float eps, const float* inv_freq, int rotary_dim,
    int num_tokens, int nq, int nkv, int d, int page_size, int has_kv, int num_pages, int32_t* status,
    int qkv_parts, long long qkv_part_stride, const float* angles, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (inv_freq == nullptr) angles = nullptr;
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
    // the register kernel: head size 64 or 128 rotated whole, 16-byte aligned rows, float32 projection
    const bool whole = inv_freq == nullptr || rotary_dim == d;
    if ((d == 64 || d == 128) && whole && (key == 0 || key == 3) && aligned16(qkv) && aligned16(q_out) &&
        aligned16(cache) && (qkv_part_stride % 4) == 0 && aligned16(q_norm_w) && aligned16(k_norm_w) && aligned16(angles)) {
#define VEC(D, HPW)                                                                                           \
    do {                                                                                                      \
        if (key == 0) launch_rope_vec<D, HPW, float, float, float>(qkv, q_out, cache, positions, token_entry, entry_slot, block_table, table_stride, q_norm_w, k_norm_w, eps, inv_freq, num_tokens, nq, nkv, page_size, has_kv, num_pages, status, qkv_parts, qkv_part_stride, angles, s); \
        else launch_rope_vec<D, HPW, float, bf16, bf16>(qkv, q_out, cache, positions, token_entry, entry_slot, block_table, table_stride, q_norm_w, k_norm_w, eps, inv_freq, num_tokens, nq, nkv, page_size, has_kv, num_pages, status, qkv_parts, qkv_part_stride, angles, s); \
    } while (0)
        const bool many = num_tokens >= 64;                              // few tokens: one head per warp keeps more warps busy
        if (d == 128) { if (many) VEC(128, 4); else VEC(128, 1); }
        else { if (many) VEC(64, 4); else VEC(64, 1); }
#undef VEC
        return launch_status();
    }
    if (key == 0) LAUNCH(float, float, float);
    else if (key == 3) LAUNCH(float, bf16, bf16);
    else if (key == 7) LAUNCH(bf16, bf16, bf16);
    else if (key == 1) LAUNCH(float, float, bf16);
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
    return launch_status();
}
