// Paged causal attention for prompt portions, bfloat16, on the tensor cores.
//
// A CTA takes 128 consecutive query rows of one request (a "tile" from the host-built tile
// list) for one query head and walks the request's keys in tiles of 64, reading keys and
// values straight from the cache pages (the step's own keys were written there first, so a
// portion at any past length takes the same path):
//     S = Q K^T (mma.sync m16n8k16, bfloat16 in, float32 out), scaled;
//     causal and window mask by absolute position: key j visible to the query at position p
//     iff lo(p) <= j <= p;
//     running maximum and sum per row in 32-bit (src/ops/attention.cu:204-249 folds one key at a
//     time; here a tile of 64), P rounded to bfloat16 for the second product, O += P V in 32-bit.
// K and V tiles are staged in shared memory with cp.async, double-buffered, XOR-swizzled in
// 16-byte chunks so that ldmatrix reads are conflict-free.  Eight warps, 16 query rows each; the
// host lists the tiles longest first (the last rows of a prompt see the most keys).
// Built for head sizes 64 and 128; other sizes use the generic kernel.
#include "common.cuh"
#include <math_constants.h>

#define AP_WARPS 8
#define AP_BM (16 * AP_WARPS)      // query rows per CTA
#define AP_BN 64                   // keys per tile
#define AP_THREADS (32 * AP_WARPS)

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    const int bytes = valid ? 16 : 0;                 // 0: nothing is read, the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::); }

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

// Address of 16-byte chunk `chunk` of row `row` in a [rows][D] bfloat16 tile, swizzled.
template <int D>
__device__ __forceinline__ bf16* tile_at(bf16* base, int row, int chunk) {
    return base + row * D + ((chunk ^ (row & 7)) << 3);
}

template <int D>
__global__ void __launch_bounds__(AP_THREADS) paged_prefill_attention_kernel(
    const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ cache,
    const int32_t* __restrict__ tiles,            // [n_tiles][2]: entry index, first query row of the tile in the entry
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ entry_q_start,
    const int32_t* __restrict__ entry_q_len, const int32_t* __restrict__ entry_kv_len,
    const int32_t* __restrict__ block_table, int table_stride, int nq, int nkv, int page_size, int window,
    float scale_log2e, int num_pages, int32_t* __restrict__ status) {
    pdl_begin();
    constexpr int CH = D / 8;                     // 16-byte chunks per row
    constexpr int KB = D / 16;                    // k-blocks of the first product
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);                    // [BM][D]
    bf16* k_s = q_s + AP_BM * D;                                      // [2][64][D]
    bf16* v_s = k_s + 2 * AP_BN * D;                                  // [2][64][D]

    const int tile = blockIdx.y, h = blockIdx.x;      // heads vary fastest: the tile list's expensive tiles start first
    const int kvh = h / (nq / nkv);
    const int e = tiles[2 * tile], q0 = tiles[2 * tile + 1];
    if (e < 0) return;                                            // a padding entry of the tile list: no work
    const int q_len = entry_q_len[e], kv_len = entry_kv_len[e];
    const int past = kv_len - q_len;
    const int row_base = entry_q_start[e] + q0;                       // batch row of the tile's first query
    const int rows_here = min(AP_BM, q_len - q0);
    const int32_t* table = block_table + static_cast<size_t>(entry_slot[e]) * table_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int pos_first = past + q0, pos_last = past + q0 + rows_here - 1;
    const int k_lo = (window > 0 && pos_first - window + 1 > 0) ? ((pos_first - window + 1) / AP_BN) * AP_BN : 0;
    const int n_tiles = (pos_last - k_lo) / AP_BN + 1;

    const size_t head_stride = static_cast<size_t>(page_size) * D;
    const size_t page_stride = 2 * static_cast<size_t>(nkv) * head_stride;
    const size_t v_shift = static_cast<size_t>(nkv) * head_stride;

    // a group of TPR threads copies one key row: thread (row, sub) takes chunks TPR*i + sub
    constexpr int TPR = AP_THREADS / AP_BN;
    const int ld_row = tid / TPR, ld_sub = tid % TPR;

    auto load_kv = [&](int kt, int buf) {
        const int key = kt + ld_row;
        bool valid = key <= pos_last;
        const bf16* src = cache;
        if (valid) {
            const int logical = key / page_size;
            const int page = logical < table_stride ? table[logical] : -1;
            if (page < 0 || page >= num_pages) {
                if (atomicCAS(status, 0, 4) == 0) status[1] = row_base;
                valid = false;
            } else {
                src = cache + static_cast<size_t>(page) * page_stride + kvh * head_stride +
                      static_cast<size_t>(key - logical * page_size) * D;
            }
        }
        bf16* kd = k_s + buf * AP_BN * D;
        bf16* vd = v_s + buf * AP_BN * D;
#pragma unroll
        for (int i = 0; i < CH / TPR; ++i) {
            const int c = TPR * i + ld_sub;
            cp_async16(tile_at<D>(kd, ld_row, c), src + c * 8, valid);
            cp_async16(tile_at<D>(vd, ld_row, c), src + v_shift + c * 8, valid);
        }
    };

    {   // Q tile: TPQ threads per query row
        constexpr int TPQ = AP_THREADS / AP_BM;
        const int qr = tid / TPQ, qsub = tid % TPQ;
        const bool valid = qr < rows_here;
        const bf16* src = q + (static_cast<size_t>(row_base + (valid ? qr : 0)) * nq + h) * D;
#pragma unroll
        for (int i = 0; i < CH / TPQ; ++i) {
            const int c = TPQ * i + qsub;
            cp_async16(tile_at<D>(q_s, qr, c), src + c * 8, valid);
        }
    }
    load_kv(k_lo, 0);
    cp_async_commit();

    unsigned qf[KB][4];
    float o[D / 8][4];
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.0f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.0f, l1 = 0.0f;      // rows lane/4 and lane/4 + 8
    const int r0 = warp * 16 + (lane >> 2);
    const int pos0 = past + q0 + r0, pos1 = pos0 + 8;
    const int lo0 = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int lo1 = (window > 0 && pos1 - window + 1 > 0) ? pos1 - window + 1 : 0;
    const bool live0 = r0 < rows_here, live1 = r0 + 8 < rows_here;

    for (int it = 0; it < n_tiles; ++it) {
        const int kt = k_lo + it * AP_BN, buf = it & 1;
        cp_async_wait_all();
        __syncthreads();
        if (it + 1 < n_tiles) load_kv(kt + AP_BN, buf ^ 1);
        cp_async_commit();
        if (it == 0) {
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
                ldmatrix_x4(qf[kb], tile_at<D>(q_s, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, kb * 2 + (lane >> 4)));
        }
        if (kt > past + q0 + warp * 16 + 15) continue;              // every key of the tile lies after this warp's rows
        const bf16* kd = k_s + buf * AP_BN * D;
        const bf16* vd = v_s + buf * AP_BN * D;

        float s[AP_BN / 8][4];
#pragma unroll
        for (int nb = 0; nb < AP_BN / 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
        {
            // S = Q K^T as KB * 4 steps of (one ldmatrix.x4 of K, two mma); fragments are fetched two
            // steps ahead of the mma that uses them, so the shared-memory latency hides behind the math.
            constexpr int NST = KB * (AP_BN / 16);
            unsigned kf[3][4];
            auto k_addr = [&](int st) {
                const int kb = st / (AP_BN / 16), np = st % (AP_BN / 16);
                return tile_at<D>(const_cast<bf16*>(kd), np * 16 + (lane & 7) + (lane >> 4) * 8, kb * 2 + ((lane >> 3) & 1));
            };
            ldmatrix_x4(kf[0], k_addr(0));
            ldmatrix_x4(kf[1], k_addr(1));
#pragma unroll
            for (int st = 0; st < NST; ++st) {
                if (st + 2 < NST) ldmatrix_x4(kf[(st + 2) % 3], k_addr(st + 2));
                const int kb = st / (AP_BN / 16), np = st % (AP_BN / 16);
                mma_bf16(s[2 * np], qf[kb], kf[st % 3][0], kf[st % 3][1]);
                mma_bf16(s[2 * np + 1], qf[kb], kf[st % 3][2], kf[st % 3][3]);
            }
        }
        // the first value fragments start their way now; the softmax arithmetic below covers them
        constexpr int VST = (AP_BN / 16) * (D / 16);
        unsigned vf[3][4];
        auto v_addr = [&](int st) {
            const int kb = st / (D / 16), np = st % (D / 16);
            return tile_at<D>(const_cast<bf16*>(vd), kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, np * 2 + (lane >> 4));
        };
        ldmatrix_x4_trans(vf[0], v_addr(0));
        ldmatrix_x4_trans(vf[1], v_addr(1));
        // mask, scale into the exp2 domain, running max
        const bool need_mask = (kt + AP_BN - 1 > pos_first) || (window > 0);
        float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
        for (int nb = 0; nb < AP_BN / 8; ++nb) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int key = kt + nb * 8 + (lane & 3) * 2 + c;
                float a = s[nb][c] * scale_log2e, b2 = s[nb][2 + c] * scale_log2e;
                if (need_mask) {
                    if (key > pos0 || key < lo0) a = -CUDART_INF_F;
                    if (key > pos1 || key < lo1) b2 = -CUDART_INF_F;
                }
                s[nb][c] = a;
                s[nb][2 + c] = b2;
                mx0 = fmaxf(mx0, a);
                mx1 = fmaxf(mx1, b2);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float al0 = (m0 == -CUDART_INF_F) ? 0.0f : exp2f(m0 - mn0);
        const float al1 = (m1 == -CUDART_INF_F) ? 0.0f : exp2f(m1 - mn1);
        const float sub0 = (mn0 == -CUDART_INF_F) ? 0.0f : mn0, sub1 = (mn1 == -CUDART_INF_F) ? 0.0f : mn1;
        float sum0 = 0.0f, sum1 = 0.0f;
        unsigned pf[AP_BN / 16][4];
#pragma unroll
        for (int nb = 0; nb < AP_BN / 8; ++nb) {
            const float p00 = exp2f(s[nb][0] - sub0), p01 = exp2f(s[nb][1] - sub0);
            const float p10 = exp2f(s[nb][2] - sub1), p11 = exp2f(s[nb][3] - sub1);
            sum0 += p00 + p01;
            sum1 += p10 + p11;
            pf[nb >> 1][(nb & 1) * 2] = pack_bf16(p00, p01);
            pf[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p10, p11);
        }
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        l0 = l0 * al0 + sum0;
        l1 = l1 * al1 + sum1;
        m0 = mn0;
        m1 = mn1;
#pragma unroll
        for (int nb = 0; nb < D / 8; ++nb) {
            o[nb][0] *= al0; o[nb][1] *= al0;
            o[nb][2] *= al1; o[nb][3] *= al1;
        }
        // O += P V, value fragments two steps ahead
#pragma unroll
        for (int st = 0; st < VST; ++st) {
            if (st + 2 < VST) ldmatrix_x4_trans(vf[(st + 2) % 3], v_addr(st + 2));
            const int kb = st / (D / 16), np = st % (D / 16);
            mma_bf16(o[2 * np], pf[kb], vf[st % 3][0], vf[st % 3][1]);
            mma_bf16(o[2 * np + 1], pf[kb], vf[st % 3][2], vf[st % 3][3]);
        }
    }
    cp_async_wait_all();

    const float inv0 = live0 && l0 > 0.0f ? 1.0f / l0 : 0.0f, inv1 = live1 && l1 > 0.0f ? 1.0f / l1 : 0.0f;
    bf16* orow0 = out + (static_cast<size_t>(row_base + r0) * nq + h) * D + (lane & 3) * 2;
    bf16* orow1 = orow0 + static_cast<size_t>(8) * nq * D;
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) {
        if (live0) *reinterpret_cast<unsigned*>(orow0 + nb * 8) = pack_bf16(o[nb][0] * inv0, o[nb][1] * inv0);
        if (live1) *reinterpret_cast<unsigned*>(orow1 + nb * 8) = pack_bf16(o[nb][2] * inv1, o[nb][3] * inv1);
    }
}

extern "C" int llm_paged_prefill_supported(int d) { return d == 64 || d == 128; }

extern "C" int llm_paged_prefill_tile_rows() { return AP_BM; }

// q, out: bfloat16 [T, nq*d]; cache: bfloat16 [pages, 2, nkv, page_size, d];
// tiles: int32 [n_tiles][2] = (entry, first query row of the tile inside the entry), each tile
// llm_paged_prefill_tile_rows() rows.
extern "C" int llm_paged_attention_prefill(
    const void* q, void* out, const void* cache, const int32_t* tiles, int n_tiles, const int32_t* entry_slot,
    const int32_t* entry_q_start, const int32_t* entry_q_len, const int32_t* entry_kv_len,
    const int32_t* block_table, int table_stride, int nq, int nkv, int d, int page_size, int window, float scale,
    int num_pages, int32_t* status, uintptr_t stream) {
    if (n_tiles <= 0) return LLM_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || !llm_paged_prefill_supported(d)) return LLM_REFUSED_SIZE;
    if (!aligned16(q) || !aligned16(out) || !aligned16(cache)) return LLM_REFUSED_ALIGN;
    const size_t smem = static_cast<size_t>(AP_BM + 4 * AP_BN) * d * sizeof(bf16);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    dim3 grid(nq, n_tiles);
    const float scale_log2e = scale * 1.4426950408889634f;
#define LAUNCH(DD)                                                                                             \
    {                                                                                                          \
        auto kern = paged_prefill_attention_kernel<DD>;                                                        \
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                                                   static_cast<int>(smem));                                    \
        if (e != cudaSuccess) return static_cast<int>(e);                                                      \
        launch_pdl(kern, dim3(grid), dim3(AP_THREADS), smem, s, static_cast<const bf16*>(q), static_cast<bf16*>(out),              \
                                            static_cast<const bf16*>(cache), tiles, entry_slot, entry_q_start, \
                                            entry_q_len, entry_kv_len, block_table, table_stride, nq, nkv,     \
                                            page_size, window, scale_log2e, num_pages, status);                \
    }
    if (d == 64) LAUNCH(64) else LAUNCH(128)
#undef LAUNCH
    return launch_status();
}
