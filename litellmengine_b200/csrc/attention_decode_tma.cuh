// The decode attention kernel with its key/value tiles fetched by TMA: a variant of
// paged_decode_attention_kernel (attention_decode.cu) for page sizes 8, 16, 32 and 64.
//
// What changes is who moves the data.  There, every thread issues sixteen 16-byte cp.async per
// tile and the memory-input queue is what the warps wait on.  Here a fifth warp asks for a tile
// with one warp-wide bulk tensor copy (a lane per box of [page_size rows x 64 columns]: one per
// page, 64-column half and K or V, 128-byte swizzled by the copy engine), arms an mbarrier with
// the byte count and runs up to STAGES-1 tiles ahead; the four compute warps wait on the tile's "full" barrier, do
// exactly the arithmetic of the cp.async kernel, and release the stage through its "empty"
// barrier.  A page is a box, so the copy engine does the address arithmetic that 128 threads did.
//
// Tile origin is aligned down to a multiple of 64 keys, so that tiles are whole pages; keys
// before the split's first key are masked like keys after its last.  A box past the last page of
// the split re-reads the last page (finite data, masked), so every stage carries the same bytes.
//
// Every wait on an mbarrier is bounded: after TMA_WAIT_LIMIT failed tries the thread raises the
// CTA's abort flag, records status code 5 and all loops wind down; before the CTA exits the
// producer makes a bounded wait for the copies it still has in flight.
#pragma once

#include <cuda.h>

#define TMA_WAIT_LIMIT (1 << 22)

__device__ __forceinline__ unsigned smem_u32(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  False: gave up (or someone else did); the abort flag is set and the caller leaves its loop.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag,
                                          int32_t* status, int where) {
    for (int i = 0; i < TMA_WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    if (atomicCAS(status, 0, 5) == 0) status[1] = where;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
            "r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// 16-byte chunk `chunk` (of D/8) of key row `row` (of 64) in a tile laid out by the copy engine:
// D/64 halves of [64 rows][128 bytes], each 8-row group swizzled (chunk ^= row % 8).
template <int D>
__device__ __forceinline__ bf16* tma_tile_at(bf16* base, int row, int chunk) {
    return base + (chunk >> 3) * (AD_BN * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
}

template <int D, int STAGES>
__global__ void __launch_bounds__(AD_THREADS + 32) paged_decode_attention_tma_kernel(
    const __grid_constant__ CUtensorMap kv_map, const bf16* __restrict__ q, const int32_t* __restrict__ rows,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_entry,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ block_table, int table_stride,
    float* __restrict__ part_acc, float* __restrict__ part_ml, bf16* __restrict__ out, int nq, int nkv,
    int page_size, int window, float scale_log2e, int num_pages, int num_splits, int32_t* __restrict__ status) {
    // The wait for the kernel before this one (which writes q and this step's key and value row)
    // comes late: keys and values of earlier steps, the block table and the step's metadata are
    // read first, so the first tiles are already on their way when q arrives.
    pdl_invite();
    constexpr int CH = D / 8, KB = D / 16;
    constexpr int TILE = AD_BN * D;                                  // elements of one K (or V) tile
    extern __shared__ unsigned char smem_dyn[];
    // the copy engine's swizzle works on 1024-byte atoms: align the tiles ourselves
    unsigned char* smem_al = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    bf16* k_s = reinterpret_cast<bf16*>(smem_al);                    // [STAGES][D/64][64][64]
    bf16* v_s = k_s + STAGES * TILE;
    bf16* q_s = v_s + STAGES * TILE;                                 // [16][D], layout of tile_at<D>
    __shared__ float m_s[4][16], l_s[4][16];
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES];
    __shared__ int abort_flag;

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
    const int k_origin = (k_begin / AD_BN) * AD_BN;                  // tiles are whole pages
    const int n_tiles = k_end > k_begin ? (k_end - k_origin + AD_BN - 1) / AD_BN : 0;

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();                                                 // the barriers exist

    if (warp == 4) {
        // ---- producer: every lane asks the copy engine for one box of the tile ----
        // A tile is (pages per tile) x (64-column halves) x (K, V) boxes, at most 32: lane l takes
        // box l, looks its page up one tile ahead, and the whole tile is requested by one warp-wide
        // instruction.  (One lane doing this box by box, each with its own table read, spent more
        // time per tile than the compute warps need for it.)
        const int boxes = AD_BN / page_size;                          // pages per tile
        constexpr int HALVES = D / 64;
        const int n_ops = boxes * HALVES * 2;
        const bool active = lane < n_ops;
        const int box = lane % boxes, half = (lane / boxes) % HALVES, kv = lane / (boxes * HALVES);
        const int last_logical = (k_end - 1) / page_size;
        const unsigned tile_bytes = 2u * TILE * sizeof(bf16);
        auto page_of = [&](int it) {                                  // this lane's page of tile `it` (checked)
            if (!active || it >= n_tiles) return 0;
            const int logical = min((k_origin + it * AD_BN) / page_size + box, last_logical);
            int page = logical < table_stride ? __ldg(table + logical) : -1;
            if (page < 0 || page >= num_pages) {
                if (atomicCAS(status, 0, 4) == 0) status[1] = t;
                page = 0;                                             // any page keeps the byte count; the result is flagged
            }
            return page;
        };
        int issued = 0;
        bool waited = false;
        int next_page = page_of(0);
        for (int it = 0; it < n_tiles; ++it) {
            const int st = it % STAGES;
            const int my_page = next_page;
            next_page = page_of(it + 1);
            if (!waited && (it >= STAGES || k_origin + (it + 1) * AD_BN > pos)) {
                pdl_wait();                                           // the tile with this step's own row, or a stage to be reused
                waited = true;
            }
            int go = 1;
            if (lane == 0) {
                if (it >= STAGES && !mbar_wait(&empty_bar[st], ((it / STAGES) - 1) & 1, &abort_flag, status, t)) go = 0;
                if (go) mbar_expect_tx(&full_bar[st], tile_bytes);
            }
            go = __shfl_sync(0xffffffffu, go, 0);
            if (!go) break;
            if (active) {
                const int row0 = ((my_page * 2 + kv) * nkv + kvh) * page_size;
                tma_load_2d((kv ? v_s : k_s) + st * TILE + half * (AD_BN * 64) + box * page_size * 64, &kv_map, half * 64, row0,
                            &full_bar[st]);
            }
            issued = it + 1;
        }
        if (lane == 0 && abort_flag) {                                // let what is in flight land before the CTA goes away
            for (int it = max(0, issued - STAGES); it < issued; ++it)
                for (int i = 0; i < TMA_WAIT_LIMIT && !mbar_try_wait(&full_bar[it % STAGES], (it / STAGES) & 1); ++i) {}
        }
        return;
    }

    // ---- consumers: warps 0..3, 16 keys of every tile each ----
    pdl_wait();
    if (n_tiles > 0 && tid < 16 * 2) {                               // the group's query heads, zero rows after them
        const int row = tid >> 1, half = tid & 1;
        const bool valid = row < G;
        const bf16* src = q + (static_cast<size_t>(t) * nq + h0 + (valid ? row : 0)) * D;
#pragma unroll
        for (int i = 0; i < CH / 2; ++i) {
            const int c = 2 * i + half;
            cp_async16(tile_at<D>(q_s, row, c), src + c * 8, valid);
        }
    }
    cp_async_commit();
    cp_async_wait_all();
    asm volatile("bar.sync 1, 128;\n" ::: "memory");                 // the four consumer warps
    unsigned qf[KB][4];
#pragma unroll
    for (int kb = 0; kb < KB; ++kb)
        ldmatrix_x4(qf[kb], tile_at<D>(q_s, (lane & 7) + ((lane >> 3) & 1) * 8, kb * 2 + (lane >> 4)));
    float o[D / 8][4];
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.0f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.0f, l1 = 0.0f;

    for (int it = 0; it < n_tiles; ++it) {
        const int st = it % STAGES;
        if (!mbar_wait(&full_bar[st], (it / STAGES) & 1, &abort_flag, status, t)) break;
        const int key0 = k_origin + it * AD_BN + warp * 16;
        if (key0 < k_end && key0 + 16 > k_begin) {
            bf16* kd = k_s + st * TILE;
            bf16* vd = v_s + st * TILE;
            float s[2][4];
            s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                unsigned b[4];
                ldmatrix_x4(b, tma_tile_at<D>(kd, warp * 16 + (lane & 7) + (lane >> 4) * 8, kb * 2 + ((lane >> 3) & 1)));
                mma_bf16(s[0], qf[kb], b[0], b[1]);
                mma_bf16(s[1], qf[kb], b[2], b[3]);
            }
            float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
            for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int key = key0 + nb * 8 + (lane & 3) * 2 + c;
                    const bool vis = key < k_end && key >= k_begin;
                    s[nb][c] = vis ? s[nb][c] * scale_log2e : -CUDART_INF_F;
                    s[nb][2 + c] = vis ? s[nb][2 + c] * scale_log2e : -CUDART_INF_F;
                    mx0 = fmaxf(mx0, s[nb][c]);
                    mx1 = fmaxf(mx1, s[nb][2 + c]);
                }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite: one key of ours is visible
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
                ldmatrix_x4_trans(b, tma_tile_at<D>(vd, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, np * 2 + (lane >> 4)));
                mma_bf16(o[2 * np], pf, b[0], b[1]);
                mma_bf16(o[2 * np + 1], pf, b[2], b[3]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[st]);                   // this warp is done with the stage
    }

    // merge the four warps' states (the tiles' memory is free once every warp is here)
    asm volatile("bar.sync 1, 128;\n" ::: "memory");                  // the four compute warps only
    constexpr int AS = D + 8;
    float* acc_s = reinterpret_cast<float*>(k_s);
    const bool tiles_idle = (abort_flag == 0);                        // after an abort copies may still land: skip the merge
    if (tiles_idle) {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
        float* a0 = acc_s + (warp * 16 + r0) * AS + c0;
        float* a1 = a0 + 8 * AS;
        if (r0 < G) {
#pragma unroll
            for (int nb = 0; nb < D / 8; ++nb) *reinterpret_cast<float2*>(a0 + nb * 8) = make_float2(o[nb][0], o[nb][1]);
        }
        if (r0 + 8 < G) {
#pragma unroll
            for (int nb = 0; nb < D / 8; ++nb) *reinterpret_cast<float2*>(a1 + nb * 8) = make_float2(o[nb][2], o[nb][3]);
        }
        if ((lane & 3) == 0) {
            m_s[warp][r0] = m0; l_s[warp][r0] = l0;
            m_s[warp][r0 + 8] = m1; l_s[warp][r0 + 8] = l1;
        }
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    if (!tiles_idle) return;
    for (int i = tid; i < G * D; i += AD_THREADS) {
        const int g = i / D, dim = i - g * D;
        const float M = fmaxf(fmaxf(m_s[0][g], m_s[1][g]), fmaxf(m_s[2][g], m_s[3][g]));
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

// ---- host side: the tensor map of a stage's cache, made once per (pointer, shape) ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct KvMapEntry {
    const void* ptr;
    long long rows;
    int d, page;
    CUtensorMap map;
};
#define KV_MAP_CACHE 512
static KvMapEntry g_kv_maps[KV_MAP_CACHE];
static int g_kv_map_count = 0;
static EncodeTiledFn g_encode_tiled = nullptr;
static int g_encode_state = 0;       // 0 unknown, 1 available, -1 not available

// The cache of one stage as a 2-D tensor [pages*2*kv_heads*page_size rows, d columns] with boxes of
// [page_size rows, 64 columns], 128-byte swizzle.  Null if the driver entry point is missing or refuses.
static const CUtensorMap* kv_tensor_map(const void* cache, int num_pages, int nkv, int page_size, int d) {
    if (g_encode_state == 0) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess && fn != nullptr) {
            g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
            g_encode_state = 1;
        } else {
            (void)cudaGetLastError();
            g_encode_state = -1;
        }
    }
    if (g_encode_state < 0) return nullptr;
    const long long rows = static_cast<long long>(num_pages) * 2 * nkv * page_size;
    for (int i = 0; i < g_kv_map_count; ++i)
        if (g_kv_maps[i].ptr == cache && g_kv_maps[i].rows == rows && g_kv_maps[i].d == d && g_kv_maps[i].page == page_size)
            return &g_kv_maps[i].map;
    if (g_kv_map_count >= KV_MAP_CACHE || rows >= (1LL << 31)) return nullptr;
    KvMapEntry& e = g_kv_maps[g_kv_map_count];
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(d) * sizeof(bf16)};
    const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(page_size)};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult rc = g_encode_tiled(&e.map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides,
                                       box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return nullptr;
    e.ptr = cache;
    e.rows = rows;
    e.d = d;
    e.page = page_size;
    ++g_kv_map_count;
    return &e.map;
}

static bool decode_tma_page_ok(int page_size) { return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64; }
