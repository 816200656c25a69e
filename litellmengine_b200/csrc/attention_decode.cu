// Paged attention for single decoded tokens, bfloat16, on the tensor cores, split over the keys
// so that a small batch still fills the GPU.  Memory-bound by design: every key and value row
// of the request's kv head is read once (coalesced 16-byte cp.async into shared memory, three
// tiles deep) and serves all the query heads of the group, which sit in the 16 rows of
// one mma tile (rows past the group size are zero and never stored).
//
// For the token in row r (request slot s, position p), kv head c, split i of n:
//     keys j in [lo + i*len, lo + (i+1)*len) ∩ [lo, p],  lo = 0 or p - window + 1
//     per query head h of the group: s_j = (q_h . k_j) * scale, running max m, sum l of
//     exp(s_j - m), acc = sum exp(s_j - m) v_j      -- softmax state and accumulators in 32-bit
// (the running-maximum form of src/ops/attention.cu:577-668, which walks the keys one by one
// with one block per query head).  The partial (m, l, acc) of each split go to scratch memory;
// `paged_decode_combine` merges them: out = sum_i acc_i 2^{m_i - M} / sum_i l_i 2^{m_i - M}
// (m is kept in the base-2 domain: scores are multiplied by scale*log2(e) once).
//
// One CTA of 4 warps per (split, kv head, token).  The CTA loads tiles of 64 keys; warp w owns
// keys 16w..16w+15 of every tile: S = Q K^T (mma.sync m16n8k16), mask, online softmax, P rounded
// to bfloat16, O += P V.  The four warps' states are merged through shared memory at the end.
// Built for head sizes 64 and 128 and groups up to 16; other sizes use the generic kernel.
#include "common.cuh"
#include <math_constants.h>
#include <stdlib.h>

#define AD_BN 64
#define AD_THREADS 128

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    const int bytes = valid ? 16 : 0;                 // 0: nothing is read, the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}
// 16-byte chunk `chunk` of row `row` in a [rows][D] bfloat16 tile, XOR-swizzled against bank conflicts.
template <int D>
__device__ __forceinline__ bf16* tile_at(bf16* base, int row, int chunk) {
    return base + row * D + ((chunk ^ (row & 7)) << 3);
}

template <int D, int AD_STAGES>
__global__ void __launch_bounds__(AD_THREADS) paged_decode_attention_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ cache, const int32_t* __restrict__ rows,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_entry,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ block_table, int table_stride,
    float* __restrict__ part_acc, float* __restrict__ part_ml, bf16* __restrict__ out, int nq, int nkv,
    int page_size, int window, float scale_log2e, int num_pages, int num_splits, int32_t* __restrict__ status) {
    pdl_begin();
    constexpr int CH = D / 8, KB = D / 16;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);                 // [16][D]
    bf16* k_s = q_s + 16 * D;                                      // [STAGES][64][D]
    bf16* v_s = k_s + AD_STAGES * AD_BN * D;                       // [STAGES][64][D]
    __shared__ float m_s[4][16], l_s[4][16];

    const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = nq / nkv, h0 = kvh * G;
    const int t = rows ? rows[r] : r;
    if (t < 0) return;                                              // a padding entry of the row list: no work
    const int pos = positions[t];
    const int32_t* table = block_table + static_cast<size_t>(entry_slot[token_entry[t]]) * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_keys = pos - lo + 1;
    int per_split = (n_keys + num_splits - 1) / num_splits;
    per_split = (per_split + AD_BN - 1) / AD_BN * AD_BN;
    const int k_begin = lo + split * per_split;
    const int k_end = min(pos + 1, k_begin + per_split);
    const int n_tiles = k_end > k_begin ? (k_end - k_begin + AD_BN - 1) / AD_BN : 0;

    const size_t head_stride = static_cast<size_t>(page_size) * D;
    const size_t page_stride = 2 * static_cast<size_t>(nkv) * head_stride;
    const size_t v_shift = static_cast<size_t>(nkv) * head_stride;
    const int ld_row = tid >> 1, ld_half = tid & 1;                // a pair of threads copies one row

    // The page number of this thread's row is looked up one tile ahead of the copy that needs it,
    // so the table read's latency passes behind the arithmetic of a whole tile.
    auto lookup = [&](int kt) -> int {
        const int key = kt + ld_row;
        if (key >= k_end) return -2;                                // past the split: zero-fill
        const int logical = key / page_size;
        return logical < table_stride ? __ldg(table + logical) : -1;
    };
    auto load_kv = [&](int kt, int buf, int page) {
        const int key = kt + ld_row;
        bool valid = page >= 0;
        const bf16* src = cache;
        if (page == -1 || page >= num_pages) {
            if (atomicCAS(status, 0, 4) == 0) status[1] = t;
            valid = false;
        } else if (valid) {
            src = cache + static_cast<size_t>(page) * page_stride + kvh * head_stride +
                  static_cast<size_t>(key % page_size) * D;
        }
        bf16* kd = k_s + buf * AD_BN * D;
        bf16* vd = v_s + buf * AD_BN * D;
#pragma unroll
        for (int i = 0; i < CH / 2; ++i) {
            const int c = 2 * i + ld_half;
            cp_async16(tile_at<D>(kd, ld_row, c), src + c * 8, valid);
            cp_async16(tile_at<D>(vd, ld_row, c), src + v_shift + c * 8, valid);
        }
    };

    if (n_tiles > 0) {
        if (ld_row < 16) {                                          // the group's query heads, zero rows after them
            const bool valid = ld_row < G;
            const bf16* src = q + (static_cast<size_t>(t) * nq + h0 + (valid ? ld_row : 0)) * D;
#pragma unroll
            for (int i = 0; i < CH / 2; ++i) {
                const int c = 2 * i + ld_half;
                cp_async16(tile_at<D>(q_s, ld_row, c), src + c * 8, valid);
            }
        }
        load_kv(k_begin, 0, lookup(k_begin));
    }
    cp_async_commit();
#pragma unroll
    for (int st = 1; st < AD_STAGES - 1; ++st) {
        if (st < n_tiles) load_kv(k_begin + st * AD_BN, st, lookup(k_begin + st * AD_BN));
        cp_async_commit();
    }
    int page_ahead = (AD_STAGES - 1 < n_tiles) ? lookup(k_begin + (AD_STAGES - 1) * AD_BN) : -2;

    unsigned qf[KB][4];
    float o[D / 8][4];
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.0f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.0f, l1 = 0.0f;   // rows lane/4 and lane/4 + 8

    for (int it = 0; it < n_tiles; ++it) {
        const int kt = k_begin + it * AD_BN, buf = it % AD_STAGES;
        cp_async_wait<AD_STAGES - 2>();                             // tile `it` has landed; later ones may be in flight
        __syncthreads();                                            // and every warp is done with tile it-1's buffer
        if (it + AD_STAGES - 1 < n_tiles) load_kv(kt + (AD_STAGES - 1) * AD_BN, (it + AD_STAGES - 1) % AD_STAGES, page_ahead);
        cp_async_commit();
        page_ahead = (it + AD_STAGES < n_tiles) ? lookup(kt + AD_STAGES * AD_BN) : -2;
        if (it == 0) {
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
                ldmatrix_x4(qf[kb], tile_at<D>(q_s, (lane & 7) + ((lane >> 3) & 1) * 8, kb * 2 + (lane >> 4)));
        }
        const int key0 = kt + warp * 16;                            // this warp's 16 keys of the tile
        if (key0 >= k_end) continue;                                // warp-uniform: nothing of ours in this tile
        bf16* kd = k_s + buf * AD_BN * D;
        bf16* vd = v_s + buf * AD_BN * D;
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
            unsigned b[4];
            ldmatrix_x4(b, tile_at<D>(kd, warp * 16 + (lane & 7) + (lane >> 4) * 8, kb * 2 + ((lane >> 3) & 1)));
            mma_bf16(s[0], qf[kb], b[0], b[1]);
            mma_bf16(s[1], qf[kb], b[2], b[3]);
        }
        float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const bool vis = key0 + nb * 8 + (lane & 3) * 2 + c < k_end;
                s[nb][c] = vis ? s[nb][c] * scale_log2e : -CUDART_INF_F;
                s[nb][2 + c] = vis ? s[nb][2 + c] * scale_log2e : -CUDART_INF_F;
                mx0 = fmaxf(mx0, s[nb][c]);
                mx1 = fmaxf(mx1, s[nb][2 + c]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);     // finite: key0 < k_end, so one key is visible
        const float al0 = (m0 == -CUDART_INF_F) ? 0.0f : exp2f(m0 - mn0);
        const float al1 = (m1 == -CUDART_INF_F) ? 0.0f : exp2f(m1 - mn1);
        const float p00 = exp2f(s[0][0] - mn0), p01 = exp2f(s[0][1] - mn0), p02 = exp2f(s[1][0] - mn0),
                    p03 = exp2f(s[1][1] - mn0);
        const float p10 = exp2f(s[0][2] - mn1), p11 = exp2f(s[0][3] - mn1), p12 = exp2f(s[1][2] - mn1),
                    p13 = exp2f(s[1][3] - mn1);
        float sum0 = p00 + p01 + p02 + p03, sum1 = p10 + p11 + p12 + p13;
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        l0 = l0 * al0 + sum0;
        l1 = l1 * al1 + sum1;
        m0 = mn0;
        m1 = mn1;
        unsigned pf[4] = {pack_bf16(p00, p01), pack_bf16(p10, p11), pack_bf16(p02, p03), pack_bf16(p12, p13)};
#pragma unroll
        for (int nb = 0; nb < D / 8; ++nb) {
            o[nb][0] *= al0; o[nb][1] *= al0;
            o[nb][2] *= al1; o[nb][3] *= al1;
        }
#pragma unroll
        for (int np = 0; np < D / 16; ++np) {
            unsigned b[4];
            ldmatrix_x4_trans(b, tile_at<D>(vd, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, np * 2 + (lane >> 4)));
            mma_bf16(o[2 * np], pf, b[0], b[1]);
            mma_bf16(o[2 * np + 1], pf, b[2], b[3]);
        }
    }
    cp_async_wait_all();
    __syncthreads();                                                // tiles are done: reuse their memory

    constexpr int AS = D + 8;                                       // padded row: rows 0..3 hit different banks
    float* acc_s = reinterpret_cast<float*>(k_s);                   // [4 warps][16 rows][AS]; only rows < G are used
    {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
        float* a0 = acc_s + (warp * 16 + r0) * AS + c0;
        float* a1 = a0 + 8 * AS;
        if (r0 < G) {
#pragma unroll
            for (int nb = 0; nb < D / 8; ++nb)
                *reinterpret_cast<float2*>(a0 + nb * 8) = make_float2(o[nb][0], o[nb][1]);
        }
        if (r0 + 8 < G) {
#pragma unroll
            for (int nb = 0; nb < D / 8; ++nb)
                *reinterpret_cast<float2*>(a1 + nb * 8) = make_float2(o[nb][2], o[nb][3]);
        }
        if ((lane & 3) == 0) {
            m_s[warp][r0] = m0; l_s[warp][r0] = l0;
            m_s[warp][r0 + 8] = m1; l_s[warp][r0 + 8] = l1;
        }
    }
    __syncthreads();
    for (int i = tid; i < G * D; i += AD_THREADS) {
        const int g = i / D, dim = i - g * D;
        float M = fmaxf(fmaxf(m_s[0][g], m_s[1][g]), fmaxf(m_s[2][g], m_s[3][g]));
        float a = 0.0f, L = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = (m_s[w][g] == -CUDART_INF_F) ? 0.0f : exp2f(m_s[w][g] - M);
            a += acc_s[(w * 16 + g) * AS + dim] * f;
            L += l_s[w][g] * f;
        }
        if (num_splits == 1) {
            out[(static_cast<size_t>(t) * nq + h0 + g) * D + dim] = __float2bfloat16_rn(a / L);
        } else {
            const size_t hrow = static_cast<size_t>(r) * nq + h0 + g;
            part_acc[(hrow * num_splits + split) * D + dim] = a;
            if (dim == 0) {
                part_ml[(hrow * num_splits + split) * 2] = M;
                part_ml[(hrow * num_splits + split) * 2 + 1] = L;
            }
        }
    }
}

#include "attention_decode_tma.cuh"

// One block per (token row, query head): merge the splits (m in the base-2 domain).
template <int D>
__global__ void paged_decode_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                            const int32_t* __restrict__ rows, bf16* __restrict__ out, int nq,
                                            int num_splits) {
    pdl_begin();
    const int r = blockIdx.x, h = blockIdx.y;
    const int t = rows ? rows[r] : r;
    if (t < 0) return;                                              // a padding entry of the row list: no work
    const size_t hrow = static_cast<size_t>(r) * nq + h;
    float M = -CUDART_INF_F;
    for (int s = 0; s < num_splits; ++s)
        if (part_ml[(hrow * num_splits + s) * 2 + 1] > 0.0f) M = fmaxf(M, part_ml[(hrow * num_splits + s) * 2]);
    for (int dim = threadIdx.x; dim < D; dim += blockDim.x) {
        float a = 0.0f, L = 0.0f;
        for (int s = 0; s < num_splits; ++s) {
            const float ls = part_ml[(hrow * num_splits + s) * 2 + 1];
            if (ls > 0.0f) {                          // an empty split holds nothing to add
                const float f = exp2f(part_ml[(hrow * num_splits + s) * 2] - M);
                a += part_acc[(hrow * num_splits + s) * D + dim] * f;
                L += ls * f;
            }
        }
        out[(static_cast<size_t>(t) * nq + h) * D + dim] = __float2bfloat16_rn(a / L);
    }
}

template <int D, int AD_STAGES>
static int launch_decode(const bf16* q, const bf16* cache, const int32_t* rows, const int32_t* positions,
                         const int32_t* token_entry, const int32_t* entry_slot, const int32_t* block_table,
                         int table_stride, float* part_acc, float* part_ml, bf16* out, int n_rows, int nq, int nkv,
                         int page_size, int window, float scale, int num_pages, int num_splits, int32_t* status,
                         cudaStream_t s) {
    const size_t smem = static_cast<size_t>(16 + 2 * AD_STAGES * AD_BN) * D * sizeof(bf16);
    auto kern = paged_decode_attention_kernel<D, AD_STAGES>;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    dim3 grid(num_splits, nkv, n_rows);
    // pages of 8 to 64 tokens are boxes the copy engine fetches; other page sizes go through cp.async
    const CUtensorMap* map = decode_tma_page_ok(page_size) ? kv_tensor_map(cache, num_pages, nkv, page_size, D) : nullptr;
    if (map != nullptr) {
#define TMA_GO(TS)                                                                                                   \
    {                                                                                                                \
        const size_t tsmem = static_cast<size_t>(2 * TS * AD_BN + 16) * D * sizeof(bf16) + 1024;                     \
        auto tk = paged_decode_attention_tma_kernel<D, TS>;                                                          \
        const cudaError_t te = cudaFuncSetAttribute(tk, cudaFuncAttributeMaxDynamicSharedMemorySize,                 \
                                                    static_cast<int>(tsmem));                                        \
        if (te != cudaSuccess) return static_cast<int>(te);                                                          \
        launch_pdl(tk, dim3(grid), dim3(AD_THREADS + 32), tsmem, s, *map, q, rows, positions, token_entry, entry_slot, block_table,      \
                                                table_stride, part_acc, part_ml, out, nq, nkv, page_size, window,    \
                                                scale * 1.4426950408889634f, num_pages, num_splits, status);         \
    }
        TMA_GO(3)                                                   // three tiles in shared memory: one read, two in flight
#undef TMA_GO
    } else {
        launch_pdl(kern, dim3(grid), dim3(AD_THREADS), smem, s, q, cache, rows, positions, token_entry, entry_slot, block_table, table_stride,
                                            part_acc, part_ml, out, nq, nkv, page_size, window,
                                            scale * 1.4426950408889634f, num_pages, num_splits, status);
    }
    int rc = launch_status();
    if (rc != LLM_OK || num_splits == 1) return rc;
    dim3 cgrid(n_rows, nq);
    launch_pdl((paged_decode_combine_kernel<D>), cgrid, dim3(D <= 64 ? 64 : 128), 0, s, part_acc, part_ml, rows, out, nq, num_splits);
    return launch_status();
}

// Whether (head_dim, group) has a tuned kernel; the Python side asks before choosing.
extern "C" int llm_paged_decode_supported(int d, int group) {
    return (d == 64 || d == 128) && group >= 1 && group <= 16;
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
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || num_splits < 1 || num_splits > 65535 ||
        nkv > 65535 || n_rows > 65535)
        return LLM_REFUSED_SIZE;
    if (!llm_paged_decode_supported(d, nq / nkv)) return LLM_REFUSED_SIZE;
    if (!aligned16(cache) || !aligned16(q) || (num_splits > 1 && (!scratch || !aligned16(scratch))))
        return LLM_REFUSED_ALIGN;
    float* part_acc = scratch;
    float* part_ml = scratch ? scratch + static_cast<size_t>(n_rows) * nq * num_splits * d : nullptr;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    // Three tiles in shared memory: one being read, two in flight (more did not bring more bandwidth).
#define GO(DD, SS)                                                                                              \
    return launch_decode<DD, SS>(static_cast<const bf16*>(q), static_cast<const bf16*>(cache), rows, positions, \
                                 token_entry, entry_slot, block_table, table_stride, part_acc, part_ml,         \
                                 static_cast<bf16*>(out), n_rows, nq, nkv, page_size, window, scale, num_pages, \
                                 num_splits, status, s)
    if (d == 64) GO(64, 3);
    GO(128, 3);
#undef GO
}

// ---- the entry point that allocates nothing (declared and explained in attention_decode_noalloc.h) ----
#include "attention_decode_noalloc.h"

// The splits' partial results of llm_paged_attention_decode_noalloc live here, in the library image.
static __device__ __align__(256) float g_decode_noalloc_scratch[LLM_DECODE_NOALLOC_SCRATCH_FLOATS];

#define NOALLOC_MAX_DEVICES 64
static float* g_noalloc_scratch_ptr[NOALLOC_MAX_DEVICES];      // device address of the array, per device

extern "C" long long llm_paged_attention_decode_noalloc_needed(int n_rows, int nq, int d, int num_splits) {
    return llm_paged_decode_scratch_floats(n_rows, nq, d, num_splits);
}

extern "C" const char* llm_noalloc_strerror(int code) {
    switch (code) {
        case LLM_OK: return "ok";
        case LLM_REFUSED_SIZE: return "refused: head size, group or counts the decode attention kernel does not take";
        case LLM_REFUSED_DTYPE: return "refused: dtype";
        case LLM_REFUSED_ALIGN: return "refused: q, out or cache is not 16-byte aligned";
        case LLM_REFUSED_SCRATCH:
            return "refused: n_rows * nq * num_splits * (d + 2) exceeds the 4194304 floats of the static scratch; "
                   "use fewer splits or rows, or the allocating entry point";
        case LLM_SYMBOL_ADDRESS_FAILED: return "cudaGetSymbolAddress failed for the static scratch on this device";
        default: return code > 0 ? "CUDA error at launch (the value is the cudaError_t)" : "unknown code";
    }
}

extern "C" int llm_paged_attention_decode_noalloc(
    const void* q, void* out, const void* cache, const int32_t* rows, int n_rows, const int32_t* positions,
    const int32_t* token_entry, const int32_t* entry_slot, const int32_t* block_table, int table_stride, int nq,
    int nkv, int d, int page_size, int window, float scale, int num_pages, int num_splits, int32_t* status,
    uintptr_t stream) {
    if (n_rows <= 0) return LLM_OK;
    if (nq <= 0 || d <= 0 || num_splits < 1) return LLM_REFUSED_SIZE;
    if (llm_paged_decode_scratch_floats(n_rows, nq, d, num_splits) > LLM_DECODE_NOALLOC_SCRATCH_FLOATS)
        return LLM_REFUSED_SCRATCH;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= NOALLOC_MAX_DEVICES)
        return LLM_SYMBOL_ADDRESS_FAILED;
    float* scratch = g_noalloc_scratch_ptr[device];
    if (scratch == nullptr) {
        // Set-up, once per device, with that device current: the host-side name of a __device__
        // array is not a device address; the runtime hands out the real one.
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_decode_noalloc_scratch) != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return LLM_SYMBOL_ADDRESS_FAILED;
        }
        scratch = static_cast<float*>(p);
        g_noalloc_scratch_ptr[device] = scratch;
    }
    return llm_paged_attention_decode(q, out, cache, rows, n_rows, positions, token_entry, entry_slot, block_table,
                                      table_stride, nq, nkv, d, page_size, window, scale, num_pages, num_splits,
                                      scratch, status, stream);
}
