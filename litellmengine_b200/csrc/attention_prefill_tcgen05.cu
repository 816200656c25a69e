// Paged causal attention for prompt portions on the 5th-generation tensor cores: tcgen05.mma with
// accumulators in tensor memory (TMEM), operands fetched by TMA, bfloat16, head size 128.
//
// A CTA takes 128 consecutive query rows of one request for one query head (a tile of the same
// host-built list the mma.sync kernel uses) and walks the request's keys in tiles of 64, TWICE:
//   pass A:  S = Q K^T (tcgen05.mma, M 128 x N 64 x K 128 -> TMEM), row maxima m over visible keys;
//   pass B:  S again, P = exp2(S*scale*log2e - m) (exact softmax numerators: m is final, so the
//            output accumulator never has to be rescaled), l += row sums, P rounded to bfloat16
//            goes back into TMEM, O += P V (tcgen05.mma with A from TMEM, V as an MN-major
//            shared-memory operand), and at the end out = O / l.
// Running S twice costs half as much again in tensor work and removes the correction step of
// the running-maximum form (src/ops/attention.cu:204-249) from the critical path; the numbers
// are those of a two-pass softmax (src/ops/paged_attention.cpp:159-217).
//
// A CTA serves TWO query heads of the same kv head when the group size is even (one otherwise):
// they share every key/value tile in shared memory, which halves the L2 traffic and the number
// of copy-engine operations per unit of tensor work (with 16-token pages a tile is 4 pages x 2
// halves x K and V = 16 boxes of 2 KB, and the copy engine's time per box is what the first
// version of this kernel waited for).
// Roles: warp 0 feeds the copy engine (Q once, then K or K+V tiles, four stages); one lane of
// warp 1 issues the MMAs and owns the TMEM allocation; then four softmax warps per head: a
// thread owns one query row = one TMEM lane (a warp can only reach the 32 lanes of its quarter).
// Per head S is double-buffered in TMEM and P overwrites the first half of its own S in place
// (S0 S1 O = 64+64+128 = 256 columns per head), so the S of the next tile is computed while the
// softmax of this one runs.
// Every mbarrier wait is bounded; on a timeout the CTA raises an abort flag, records status
// code 6, lets its copies land (bounded) and frees its TMEM before it returns.
#include "common.cuh"
#include <cuda.h>
#include <math_constants.h>

#define T5_BM 128
#define T5_BN 64
#define T5_D 128
#define T5_WAIT_LIMIT 200000
#define T5_QHALF (T5_BM * 64)                 // elements of one 64-column half of the 128-row query tile
#define T5_HALF (T5_BN * 64)                  // elements of one 64-column half of a key or value tile
#define T5_TILE (2 * T5_HALF)


__device__ __forceinline__ unsigned t5_smem(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void t5_mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(t5_smem(bar)), "r"(count));
}
__device__ __forceinline__ void t5_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(t5_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void t5_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(t5_smem(bar)) : "memory");
}
__device__ __forceinline__ bool t5_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(t5_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool t5_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag,
                                        int32_t* status, int where) {
    for (int i = 0; i < T5_WAIT_LIMIT; ++i) {
        if (t5_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    if (atomicCAS(status, 0, 6) == 0) status[1] = where;
    return false;
}
__device__ __forceinline__ void t5_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
                     "r"(t5_smem(dst)), "l"(map), "r"(x), "r"(y), "r"(t5_smem(bar)) : "memory");
}

// ---- tcgen05 -------------------------------------------------------------------------------------
__device__ __forceinline__ void t5_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void t5_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void t5_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(t5_smem(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void t5_mma_ss(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                          unsigned idesc, unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::
                     "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void t5_mma_ts(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc, unsigned idesc,
                                          unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::
                     "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void t5_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void t5_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void t5_st16(unsigned taddr, const unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::
            "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void t5_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// Shared-memory operand descriptor, 128-byte swizzle, version 1.  lbo, sbo in bytes.
__device__ __forceinline__ unsigned long long t5_desc(const void* smem, unsigned lbo, unsigned sbo) {
    unsigned long long d = 0;
    d |= static_cast<unsigned long long>((t5_smem(smem) & 0x3FFFF) >> 4);
    d |= static_cast<unsigned long long>((lbo >> 4) & 0x3FFF) << 16;
    d |= static_cast<unsigned long long>((sbo >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;                      // descriptor version of this architecture
    d |= 2ull << 61;                      // SWIZZLE_128B
    return d;
}
// Instruction descriptor: bfloat16 x bfloat16 -> float32, M x N, A K-major, B K-major or MN-major.
__host__ __device__ constexpr unsigned t5_idesc(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<unsigned>(b_mn_major) << 16) |
           (static_cast<unsigned>(n >> 3) << 17) | (static_cast<unsigned>(m >> 4) << 24);
}
__device__ __forceinline__ float t5_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned t5_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// HEADS query heads of one kv head share every key/value tile (HEADS = 2 when the group size is
// even, else 1); STAGES key/value tiles sit in shared memory.
template <int HEADS, int STAGES>
__global__ void __launch_bounds__(64 + 128 * HEADS, 1) paged_prefill_attention_tcgen05_kernel(
    const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map, bf16* __restrict__ out,
    const int32_t* __restrict__ tiles, const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ entry_q_start,
    const int32_t* __restrict__ entry_q_len, const int32_t* __restrict__ entry_kv_len,
    const int32_t* __restrict__ block_table, int table_stride, int nq, int nkv, int page_size, int window,
    float scale_log2e, int num_pages, int32_t* __restrict__ status) {
    pdl_begin();
    constexpr int SOFTMAX_THREADS = 128 * HEADS;
    constexpr unsigned TMEM_COLS = 256 * HEADS;                   // per head: S0 S1 (64 each) and O (128)
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem_al = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    bf16* q_s = reinterpret_cast<bf16*>(smem_al);                 // [HEADS][2][128][64]
    bf16* k_s = q_s + HEADS * 2 * T5_QHALF;                       // [STAGES][2][BN][64]
    bf16* v_s = k_s + STAGES * T5_TILE;                           // [STAGES][2][BN][64]
    __shared__ __align__(8) unsigned long long q_full, kv_full[STAGES], kv_empty[STAGES], s_full[2], s_read[2],
        p_full[2], s_used[2], o_done;
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_flag;

    // Heads vary fastest: CTAs are handed to SMs in this order, and the tile list has the most
    // expensive tiles first, so those start first whatever the number of heads.
    const int tile = blockIdx.y;
    const int h0 = blockIdx.x * HEADS;                            // first query head of this CTA
    const int kvh = h0 / (nq / nkv);
    const int e = tiles[2 * tile], q0 = tiles[2 * tile + 1];
    if (e < 0) return;                                            // a padding entry of the tile list: no work
    const int q_len = entry_q_len[e], kv_len = entry_kv_len[e];
    const int past = kv_len - q_len;
    const int row_base = entry_q_start[e] + q0;
    const int rows_here = min(T5_BM, q_len - q0);
    const int32_t* table = block_table + static_cast<size_t>(entry_slot[e]) * table_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos_first = past + q0, pos_last = past + q0 + rows_here - 1;
    const int k_lo = (window > 0 && pos_first - window + 1 > 0) ? ((pos_first - window + 1) / T5_BN) * T5_BN : 0;
    const int n_tiles = (pos_last - k_lo) / T5_BN + 1;
    const int total = 2 * n_tiles;                                // pass A then pass B over the same tiles

    if (tid == 0) {
        abort_flag = 0;
        t5_mbar_init(&q_full, 1);
        for (int s = 0; s < STAGES; ++s) { t5_mbar_init(&kv_full[s], 1); t5_mbar_init(&kv_empty[s], 1); }
        for (int s = 0; s < 2; ++s) {
            t5_mbar_init(&s_full[s], 1);
            t5_mbar_init(&s_read[s], SOFTMAX_THREADS);   // pass A: every softmax thread has read its row of S
            t5_mbar_init(&p_full[s], SOFTMAX_THREADS);   // pass B: every softmax thread has put its row of P over S
            t5_mbar_init(&s_used[s], 1);                 // pass B: the P V products that read this buffer have finished
        }
        t5_mbar_init(&o_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {                                              // one warp allocates this CTA's TMEM columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(t5_smem(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    t5_fence_before();
    __syncthreads();
    t5_fence_after();
    const unsigned tmem = tmem_base_s;
    // columns of head g: S buffer b at g*256 + b*64, O at g*256 + 128; P lives in the first 32 columns of its S
    auto s_col = [](int g, int b) { return static_cast<unsigned>(g * 256 + b * 64); };
    auto o_col = [](int g) { return static_cast<unsigned>(g * 256 + 128); };

    if (warp == 0) {
        // ---- producer ----
        if (lane == 0) {
            t5_expect_tx(&q_full, HEADS * 2 * T5_QHALF * sizeof(bf16));
#pragma unroll
            for (int g = 0; g < HEADS; ++g) {
                t5_tma_2d(q_s + g * 2 * T5_QHALF, &q_map, (h0 + g) * T5_D, row_base, &q_full);
                t5_tma_2d(q_s + g * 2 * T5_QHALF + T5_QHALF, &q_map, (h0 + g) * T5_D + 64, row_base, &q_full);
            }
            const int boxes = T5_BN / page_size;
            const int last_logical = pos_last / page_size;
            int issued = 0;
            for (int u = 0; u < total; ++u) {
                const int st = u % STAGES, it = u % n_tiles;
                const bool with_v = u >= n_tiles;
                if (u >= STAGES && !t5_wait(&kv_empty[st], ((u / STAGES) - 1) & 1, &abort_flag, status, row_base)) break;
                t5_expect_tx(&kv_full[st], (with_v ? 2u : 1u) * T5_TILE * sizeof(bf16));
                const int first_logical = (k_lo + it * T5_BN) / page_size;
                for (int j = 0; j < boxes; ++j) {
                    const int logical = min(first_logical + j, last_logical);
                    int page = logical < table_stride ? __ldg(table + logical) : -1;
                    if (page < 0 || page >= num_pages) {
                        if (atomicCAS(status, 0, 4) == 0) status[1] = row_base;
                        page = 0;
                    }
                    const int k_row = ((page * 2) * nkv + kvh) * page_size;
                    const int v_row = ((page * 2 + 1) * nkv + kvh) * page_size;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        t5_tma_2d(k_s + st * T5_TILE + half * T5_HALF + j * page_size * 64, &kv_map, half * 64, k_row, &kv_full[st]);
                        if (with_v)
                            t5_tma_2d(v_s + st * T5_TILE + half * T5_HALF + j * page_size * 64, &kv_map, half * 64, v_row, &kv_full[st]);
                    }
                }
                issued = u + 1;
            }
            if (abort_flag)
                for (int u = max(0, issued - STAGES); u < issued; ++u)
                    for (int i = 0; i < T5_WAIT_LIMIT && !t5_try_wait(&kv_full[u % STAGES], (u / STAGES) & 1); ++i) {}
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            constexpr unsigned IDESC_QK = t5_idesc(T5_BM, T5_BN, 0);
            constexpr unsigned IDESC_PV = t5_idesc(T5_BM, T5_D, 1);
            bool ok = t5_wait(&q_full, 0, &abort_flag, status, row_base);
            // Descriptors are built once: a tile further on in shared memory is the same descriptor
            // plus its byte offset / 16 in the address field (one thread issues every product, so
            // what it computes per instruction is what limits the rate of issue).
            const unsigned long long qd0 = t5_desc(q_s, 16, 1024), kd0 = t5_desc(k_s, 16, 1024);
            const unsigned long long vd0 = t5_desc(v_s, T5_HALF * sizeof(bf16), 1024);
            constexpr unsigned long long STAGE_STEP = (T5_TILE * sizeof(bf16)) >> 4;
            auto issue_qk = [&](int u) -> bool {
                const int st = u % STAGES, sb = u & 1;
                if (!t5_wait(&kv_full[st], (u / STAGES) & 1, &abort_flag, status, row_base)) return false;
                if (u >= 2) {                                     // the buffer's previous tile must be done with it
                    const int prev = u - 2;
                    const bool a = prev < n_tiles;
                    if (!t5_wait(a ? &s_read[sb] : &s_used[sb], ((a ? prev : prev - n_tiles) >> 1) & 1, &abort_flag, status,
                                 row_base))
                        return false;
                }
                t5_fence_after();
#pragma unroll
                for (int g = 0; g < HEADS; ++g)
#pragma unroll
                    for (int k = 0; k < T5_D / 16; ++k) {
                        const unsigned long long qoff = ((g * 2 + (k >> 2)) * T5_QHALF + (k & 3) * 16) * sizeof(bf16) >> 4;
                        const unsigned long long koff = ((k >> 2) * T5_HALF + (k & 3) * 16) * sizeof(bf16) >> 4;
                        t5_mma_ss(tmem + s_col(g, sb), qd0 + qoff, kd0 + st * STAGE_STEP + koff, IDESC_QK, k > 0);
                    }
                t5_commit(&s_full[sb]);
                if (u < n_tiles) t5_commit(&kv_empty[st]);        // pass A: the keys are all this stage held
                return true;
            };
            if (ok && total > 0) ok = issue_qk(0);
            for (int u = 0; ok && u < total; ++u) {
                if (u + 1 < total) ok = issue_qk(u + 1);          // the next S while this tile's softmax runs
                if (!ok || u < n_tiles) continue;
                const int st = u % STAGES, sb = u & 1, v = u - n_tiles;
                if (!t5_wait(&p_full[sb], (v >> 1) & 1, &abort_flag, status, row_base)) { ok = false; break; }
                t5_fence_after();
#pragma unroll
                for (int g = 0; g < HEADS; ++g)
#pragma unroll
                    for (int k = 0; k < T5_BN / 16; ++k) {
                        const unsigned long long voff = (k * 16 * 64) * sizeof(bf16) >> 4;   // 16 keys further, both 64-column halves
                        t5_mma_ts(tmem + o_col(g), tmem + s_col(g, sb) + k * 8, vd0 + st * STAGE_STEP + voff,
                                  IDESC_PV, (v > 0 || k > 0) ? 1u : 0u);
                    }
                t5_commit(&kv_empty[st]);
                t5_commit(&s_used[sb]);
                if (u == total - 1) t5_commit(&o_done);
            }
        }
    } else {
        // ---- softmax: a thread owns one query row of one head = one TMEM lane, all 64 columns of a tile ----
        const int sw = warp - 2;
        const int g = sw >> 2;                                    // warps 2..5: head h0, warps 6..9: head h0 + 1
        const int quarter = warp & 3;                             // the TMEM lanes this warp may touch
        const int row = quarter * 32 + lane;
        const unsigned lane_addr = static_cast<unsigned>(quarter * 32) << 16;
        const int pos = (row < rows_here) ? past + q0 + row : -1;
        const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        float m = -CUDART_INF_F, l = 0.0f;
        bool ok = true;
        for (int u = 0; ok && u < n_tiles; ++u) {                 // pass A: maxima
            const int sb = u & 1, kt = k_lo + u * T5_BN;
            if (!t5_wait(&s_full[sb], (u >> 1) & 1, &abort_flag, status, row_base)) { ok = false; break; }
            t5_fence_after();
            const bool full_tile = (kt + T5_BN - 1 <= pos_first) && (window <= 0) && (rows_here == T5_BM);
            unsigned r[2][32];                                    // both halves of the row are requested at once
            t5_ld32(tmem + lane_addr + s_col(g, sb), r[0]);
            t5_ld32(tmem + lane_addr + s_col(g, sb) + 32, r[1]);
            t5_wait_ld();
            t5_fence_before();
            t5_arrive(&s_read[sb]);                               // S is in registers: the buffer may be overwritten
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                if (full_tile) {                                  // every row of the CTA sees every key of the tile
#pragma unroll
                    for (int i = 0; i < 32; ++i) m = fmaxf(m, __uint_as_float(r[cc][i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = kt + cc * 32 + i;
                        if (key <= pos && key >= lo) m = fmaxf(m, __uint_as_float(r[cc][i]));
                    }
                }
            }
        }
        const float msub = (m == -CUDART_INF_F) ? 0.0f : m * scale_log2e;
        for (int u = n_tiles; ok && u < total; ++u) {             // pass B: numerators with the final maximum
            const int sb = u & 1, v = u - n_tiles, kt = k_lo + v * T5_BN;
            if (!t5_wait(&s_full[sb], (u >> 1) & 1, &abort_flag, status, row_base)) { ok = false; break; }
            t5_fence_after();
            const bool full_tile = (kt + T5_BN - 1 <= pos_first) && (window <= 0) && (rows_here == T5_BM);
            unsigned pk[32], r[2][32];
            t5_ld32(tmem + lane_addr + s_col(g, sb), r[0]);
            t5_ld32(tmem + lane_addr + s_col(g, sb) + 32, r[1]);
            t5_wait_ld();
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                if (full_tile) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = t5_ex2(fmaf(__uint_as_float(r[cc][i]), scale_log2e, -msub));
                        const float p1 = t5_ex2(fmaf(__uint_as_float(r[cc][i + 1]), scale_log2e, -msub));
                        l += p0 + p1;
                        pk[(cc * 32 + i) >> 1] = t5_pack(p0, p1);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const int key = kt + cc * 32 + i;
                        const float p0 = (key <= pos && key >= lo) ? t5_ex2(fmaf(__uint_as_float(r[cc][i]), scale_log2e, -msub)) : 0.0f;
                        const float p1 = (key + 1 <= pos && key + 1 >= lo) ? t5_ex2(fmaf(__uint_as_float(r[cc][i + 1]), scale_log2e, -msub)) : 0.0f;
                        l += p0 + p1;
                        pk[(cc * 32 + i) >> 1] = t5_pack(p0, p1);
                    }
                }
            }
            // the whole row of S is in registers: P goes over its first 32 columns
            {
                unsigned a[16], b[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) { a[i] = pk[i]; b[i] = pk[16 + i]; }
                t5_st16(tmem + lane_addr + s_col(g, sb), a);
                t5_st16(tmem + lane_addr + s_col(g, sb) + 16, b);
            }
            t5_wait_st();
            t5_fence_before();
            t5_arrive(&p_full[sb]);
        }
        if (ok && t5_wait(&o_done, 0, &abort_flag, status, row_base)) {
            t5_fence_after();
            const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
            bf16* orow = out + (static_cast<size_t>(row_base + row) * nq + h0 + g) * T5_D;
#pragma unroll 1
            for (int c = 0; c < T5_D; c += 32) {
                unsigned r[32];
                t5_ld32(tmem + lane_addr + o_col(g) + c, r);
                t5_wait_ld();
                if (row < rows_here) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = t5_pack(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                        w.y = t5_pack(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                        w.z = t5_pack(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
                        w.w = t5_pack(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c + i) = w;
                    }
                }
            }
        }
    }
    t5_fence_before();
    __syncthreads();
    if (warp == 1) {
        t5_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ---- one pass with a running reference maximum, two heads in turns -------------------------------
// The same work in ONE pass over the keys, for the two query heads of a group that share a key/value
// tile (the kernel above stays for groups of odd size): 128 keys a tile, S = Q K^T of head 0 while
// the softmax threads of head 1 work and the other way round, so the tensor pipe has a product of
// one head to run while the other head's weights are being made.  Per head TMEM holds S (128
// columns of float32) and O (128 columns); P (bfloat16) lies over S, 32 columns at column 0 and 32
// at column 64, each over the columns of the thread that makes it.
// The weights are P = exp2(S*scale*log2e - m) with a reference m per row that trails the running
// maximum: m moves up only when the maximum has passed it by more than 8 (a factor 256, far
// inside what bfloat16 and the float32 sums hold), and only then O and the row sum l are
// multiplied by exp2(m_old - m_new) (the running-maximum form of src/ops/attention.cu:204-249 with
// the correction made rare).  The result sum(P V) / sum(P) does not depend on which m was used.
// Roles: warp 0 looks up pages and asks the copy engine for keys and values (rings of two tiles
// each); one lane of warp 1 issues every product; then eight softmax warps per head, two threads
// to a query row with 64 columns of S each.  What limited earlier forms, in the order found by
// reading the SM clock inside the kernel: the order of CTAs (long tiles must start
// first), one thread requesting the copies box by box (140 clocks a request), one thread per row in
// the softmax; what is left is the chain S -> weights -> P V of one head, about 4,000 clocks a
// tile against 2,050 of tensor work for both heads.
#define T5O_BN 128
#define T5O_HALF (T5O_BN * 64)                // elements of one 64-column half of a 128-key tile
#define T5O_TILE (2 * T5O_HALF)
#define T5O_STAGES 2
#define T5O_JUMP 8.0f
#define T5O_THREADS (64 + 2 * 256)             // producer warp, issuing warp, then 8 softmax warps per head

__device__ __forceinline__ void t5_st32(unsigned taddr, const unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::
            "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}

__global__ void __launch_bounds__(T5O_THREADS, 1) paged_prefill_attention_tcgen05_online_kernel(
    const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map, bf16* __restrict__ out,
    const int32_t* __restrict__ tiles, const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ entry_q_start,
    const int32_t* __restrict__ entry_q_len, const int32_t* __restrict__ entry_kv_len,
    const int32_t* __restrict__ block_table, int table_stride, int nq, int nkv, int page_size, int window,
    float scale_log2e, int num_pages, int32_t* __restrict__ status) {
    pdl_begin();
    constexpr int STAGES = T5O_STAGES;
    constexpr unsigned TMEM_COLS = 512;                           // S0 S1 O0 O1, 128 columns each
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem_al = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    bf16* q_s = reinterpret_cast<bf16*>(smem_al);                 // [2 heads][2 halves][128][64]
    bf16* k_s = q_s + 2 * 2 * T5_QHALF;                           // [STAGES][2][128][64]
    bf16* v_s = k_s + STAGES * T5O_TILE;                          // [STAGES][2][128][64]
    // keys and values have rings of their own: a key tile is free once both heads' S are made, a
    // value tile only after both heads' P V, half a tile's work later
    __shared__ __align__(8) unsigned long long q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES],
        s_full[2], p_full[2], pv_done[2];
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_flag;
    __shared__ float x_max[2][2][2][128];                         // [tile parity][head][column half][row]: the halves' maxima
    __shared__ float x_sum[2][2][128];                            // [head][column half][row]: the halves' row sums, at the end

    const int tile = blockIdx.y;
    const int h0 = blockIdx.x * 2;                                // first of this CTA's two query heads
    const int kvh = h0 / (nq / nkv);
    const int e = tiles[2 * tile], q0 = tiles[2 * tile + 1];
    if (e < 0) return;                                            // a padding entry of the tile list: no work
    const int q_len = entry_q_len[e], kv_len = entry_kv_len[e];
    const int past = kv_len - q_len;
    const int row_base = entry_q_start[e] + q0;
    const int rows_here = min(T5_BM, q_len - q0);
    const int32_t* table = block_table + static_cast<size_t>(entry_slot[e]) * table_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos_first = past + q0, pos_last = past + q0 + rows_here - 1;
    const int k_lo = (window > 0 && pos_first - window + 1 > 0) ? ((pos_first - window + 1) / T5O_BN) * T5O_BN : 0;
    const int n_tiles = (pos_last - k_lo) / T5O_BN + 1;

    if (tid == 0) {
        abort_flag = 0;
        t5_mbar_init(&q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            t5_mbar_init(&k_full[s], 1); t5_mbar_init(&k_empty[s], 1);
            t5_mbar_init(&v_full[s], 1); t5_mbar_init(&v_empty[s], 1);
        }
        for (int g = 0; g < 2; ++g) {
            t5_mbar_init(&s_full[g], 1);                 // the head's S of a tile is in TMEM
            t5_mbar_init(&p_full[g], 256);               // every softmax thread of the head has put its part of P over S
            t5_mbar_init(&pv_done[g], 1);                // the head's O holds the tile's P V
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(t5_smem(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    t5_fence_before();
    __syncthreads();
    t5_fence_after();
    const unsigned tmem = tmem_base_s;
    auto s_col = [](int g) { return static_cast<unsigned>(g * 128); };
    auto o_col = [](int g) { return static_cast<unsigned>(256 + g * 128); };

    if (warp == 0) {
        // ---- producer: lane b looks up the page of box b of a tile, one tile ahead, and asks the copy
        // engine for it ----
        // (One thread doing this box by box spent 140 clocks a copy, 4,500 a tile: longer than the
        // tile's products take.  A warp-wide copy instruction makes all boxes' requests at once.)
        if (lane == 0) {
            t5_expect_tx(&q_full, 2 * 2 * T5_QHALF * sizeof(bf16));
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                t5_tma_2d(q_s + g * 2 * T5_QHALF, &q_map, (h0 + g) * T5_D, row_base, &q_full);
                t5_tma_2d(q_s + g * 2 * T5_QHALF + T5_QHALF, &q_map, (h0 + g) * T5_D + 64, row_base, &q_full);
            }
        }
        const int boxes = T5O_BN / page_size;                     // at most 16
        const int last_logical = pos_last / page_size;
        auto page_of = [&](int j) {                               // lane b: the page of box b of tile j (checked)
            if (j >= n_tiles || lane >= boxes) return 0;
            const int logical = min((k_lo + j * T5O_BN) / page_size + lane, last_logical);
            int page = logical < table_stride ? __ldg(table + logical) : -1;
            if (page < 0 || page >= num_pages) {
                if (atomicCAS(status, 0, 4) == 0) status[1] = row_base;
                page = 0;
            }
            return page;
        };
        int issued_k = 0, issued_v = 0;
        int next_page = page_of(0);
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int st = j % STAGES;
            const int my_page = next_page;
            next_page = page_of(j + 1);
#pragma unroll 1
            for (int values = 0; values < 2; ++values) {
                unsigned long long* full = values ? &v_full[st] : &k_full[st];
                if (lane == 0) {
                    if (j >= STAGES && !t5_wait(values ? &v_empty[st] : &k_empty[st], ((j / STAGES) - 1) & 1, &abort_flag, status, row_base))
                        ok = false;
                    if (ok) t5_expect_tx(full, T5O_TILE * sizeof(bf16));
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                bf16* dst = (values ? v_s : k_s) + st * T5O_TILE;
                if (lane < boxes) {                               // every lane asks for its own box: one instruction, `boxes` copies
                    const int row0 = ((my_page * 2 + values) * nkv + kvh) * page_size;
                    t5_tma_2d(dst + lane * page_size * 64, &kv_map, 0, row0, full);
                    t5_tma_2d(dst + T5O_HALF + lane * page_size * 64, &kv_map, 64, row0, full);
                }
                if (values) issued_v = j + 1; else issued_k = j + 1;
            }
            if (!ok) break;
        }
        if (lane == 0 && abort_flag) {                            // let what is in flight land before the CTA goes away
            for (int j = max(0, issued_k - STAGES); j < issued_k; ++j)
                for (int i = 0; i < T5_WAIT_LIMIT && !t5_try_wait(&k_full[j % STAGES], (j / STAGES) & 1); ++i) {}
            for (int j = max(0, issued_v - STAGES); j < issued_v; ++j)
                for (int i = 0; i < T5_WAIT_LIMIT && !t5_try_wait(&v_full[j % STAGES], (j / STAGES) & 1); ++i) {}
        }
    } else if (warp == 1) {
        // ---- MMA issuer: S0(j), O1 += P1 V(j-1), S1(j), O0 += P0 V(j), ... ----
        if (lane == 0) {
            constexpr unsigned IDESC_QK = t5_idesc(T5_BM, T5O_BN, 0);
            constexpr unsigned IDESC_PV = t5_idesc(T5_BM, T5_D, 1);
            // One thread issues every product, and what it computes per instruction is what limits the
            // rate of issue: every operand descriptor is made once, here, and the loop over tiles is
            // unrolled by the two stages so that each product names its descriptors by constant index.
            unsigned long long qd[2][8], kd[2][8], vd[2][8];
            {
                const unsigned long long qd0 = t5_desc(q_s, 16, 1024), kd0 = t5_desc(k_s, 16, 1024);
                const unsigned long long vd0 = t5_desc(v_s, T5O_HALF * sizeof(bf16), 1024);
                constexpr unsigned long long STAGE_STEP = (T5O_TILE * sizeof(bf16)) >> 4;
#pragma unroll
                for (int a = 0; a < 2; ++a)
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        qd[a][k] = qd0 + (((a * 2 + (k >> 2)) * T5_QHALF + (k & 3) * 16) * sizeof(bf16) >> 4);
                        kd[a][k] = kd0 + a * STAGE_STEP + (((k >> 2) * T5O_HALF + (k & 3) * 16) * sizeof(bf16) >> 4);
                        vd[a][k] = vd0 + a * STAGE_STEP + ((k * 16 * 64) * sizeof(bf16) >> 4);   // 16 keys further, both 64-column halves
                    }
            }
            auto qk = [&](int g, int st) {                        // g, st: constants where this is inlined
#pragma unroll
                for (int k = 0; k < 8; ++k) t5_mma_ss(tmem + s_col(g), qd[g][k], kd[st][k], IDESC_QK, k > 0);
                t5_commit(&s_full[g]);
            };
            auto pv = [&](int g, int st, bool first) {
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    t5_mma_ts(tmem + o_col(g), tmem + s_col(g) + (k >> 2) * 64 + (k & 3) * 8, vd[st][k], IDESC_PV,
                              (!first || k > 0) ? 1u : 0u);      // P of keys 64..127 lies over S column 64
                t5_commit(&pv_done[g]);
            };
            bool ok = t5_wait(&q_full, 0, &abort_flag, status, row_base);
            auto one_tile = [&](int j, int st) -> bool {          // st = j % 2, a constant where this is inlined
                if (!t5_wait(&k_full[st], (j >> 1) & 1, &abort_flag, status, row_base)) return false;
                t5_fence_after();
                qk(0, st);
                if (j > 0) {
                    if (!t5_wait(&p_full[1], (j - 1) & 1, &abort_flag, status, row_base)) return false;
                    t5_fence_after();
                    pv(1, 1 - st, j == 1);
                    t5_commit(&v_empty[1 - st]);                       // the last reader of the values of tile j-1
                }
                qk(1, st);
                t5_commit(&k_empty[st]);                               // the last reader of the keys of tile j
                if (!t5_wait(&p_full[0], j & 1, &abort_flag, status, row_base)) return false;
                if (!t5_wait(&v_full[st], (j >> 1) & 1, &abort_flag, status, row_base)) return false;
                t5_fence_after();
                pv(0, st, j == 0);
                return true;
            };
            static_assert(T5O_STAGES == 2, "the issue loop is unrolled by the number of stages");
            for (int j = 0; ok && j < n_tiles; j += 2) {
                ok = one_tile(j, 0);
                if (ok && j + 1 < n_tiles) ok = one_tile(j + 1, 1);
            }
            if (ok && t5_wait(&p_full[1], (n_tiles - 1) & 1, &abort_flag, status, row_base)) {
                t5_fence_after();
                if ((n_tiles - 1) & 1) { pv(1, 1, n_tiles == 1); t5_commit(&v_empty[1]); }
                else { pv(1, 0, n_tiles == 1); t5_commit(&v_empty[0]); }
            }
        }
    } else {
        // ---- softmax: two threads share a query row of a head (one TMEM lane), 64 columns of S each ----
        // A warp reaches the 32 TMEM lanes of its quarter (warp index mod 4) only, so the two threads
        // of a row sit in two warps of the same quarter.  Each keeps its 64 values of S in registers,
        // the two exchange their maxima through shared memory, and each writes its 32 columns of P
        // over the first half of ITS OWN columns of S (so neither ever touches the other's columns).
        const int wl = warp - 2;
        const int g = wl >> 3;                                    // warps 2..9: head h0, warps 10..17: head h0 + 1
        const int half = (wl >> 2) & 1;                           // columns 64*half .. 64*half+63 of every tile
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const unsigned lane_addr = static_cast<unsigned>(quarter * 32) << 16;
        const unsigned my_s = tmem + lane_addr + s_col(g) + half * 64;
        const unsigned my_o = tmem + lane_addr + o_col(g) + half * 64;
        const int pos = (row < rows_here) ? past + q0 + row : -1;
        const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        float m = -CUDART_INF_F, l = 0.0f;                        // m: the reference maximum, in units of log2
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int kt = k_lo + j * T5O_BN + half * 64;         // this thread's first key of the tile
            // After a wait has run out (ok false) a thread still passes every barrier below, the same
            // number of times as the others, and touches nothing else.
            if (ok && !t5_wait(&s_full[g], j & 1, &abort_flag, status, row_base)) ok = false;
            t5_fence_after();
            const bool full_tile = (kt + 63 <= pos_first) && (window <= 0) && (rows_here == T5_BM);
            unsigned ra[32], rb[32];
            float mx = -CUDART_INF_F;
            if (ok) {
                t5_ld32(my_s, ra);
                t5_ld32(my_s + 32, rb);
                t5_wait_ld();
                if (full_tile) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(ra[i]), __uint_as_float(rb[i])));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (kt + i <= pos && kt + i >= lo) mx = fmaxf(mx, __uint_as_float(ra[i]));
                        if (kt + 32 + i <= pos && kt + 32 + i >= lo) mx = fmaxf(mx, __uint_as_float(rb[i]));
                    }
                }
                x_max[j & 1][g][half][row] = mx;
            }
            asm volatile("bar.sync %0, 256;\n" ::"r"(1 + g) : "memory");      // the 8 softmax warps of this head
            if (!ok) continue;
            mx = fmaxf(mx, x_max[j & 1][g][half ^ 1][row]) * scale_log2e;     // scale > 0; -inf stays -inf
            // move the reference up only when the maximum has run away from it (both threads of a row
            // see the same numbers and decide alike)
            const bool adopt = (m == -CUDART_INF_F) && (mx > m);  // nothing accumulated under the old reference
            const bool jump = (m != -CUDART_INF_F) && (mx > m + T5O_JUMP);
            if (__any_sync(0xffffffffu, jump)) {
                // O still receives the previous tile's product: wait for it, then scale this thread's half of its row
                if (!t5_wait(&pv_done[g], (j - 1) & 1, &abort_flag, status, row_base)) { ok = false; continue; }
                t5_fence_after();
                const float alpha = jump ? t5_ex2(m - mx) : 1.0f;
                l *= alpha;
#pragma unroll 1
                for (int c = 0; c < 64; c += 32) {                // through ra, which is read again below
                    t5_ld32(my_o + c, ra);
                    t5_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) ra[i] = __float_as_uint(__uint_as_float(ra[i]) * alpha);
                    t5_st32(my_o + c, ra);
                }
                t5_wait_st();
                t5_ld32(my_s, ra);
                t5_wait_ld();
            }
            if (adopt || jump) m = mx;
            const float msub = (m == -CUDART_INF_F) ? 0.0f : m;
            // the weights, rounded to bfloat16: 32 columns of P over the first half of this thread's 64 of S
            auto weights = [&](const unsigned (&r)[32], int c) {
                unsigned pk[16];
                if (full_tile) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float x0 = fmaf(__uint_as_float(r[i]), scale_log2e, -msub);
                        const float x1 = fmaf(__uint_as_float(r[i + 1]), scale_log2e, -msub);
                        const float p0 = t5_ex2(x0), p1 = t5_ex2(x1);     // (a cubic on the FMA pipe for a share of them: measured slower)
                        l += p0 + p1;
                        pk[i >> 1] = t5_pack(p0, p1);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const int key = kt + c + i;
                        const float p0 = (key <= pos && key >= lo) ? t5_ex2(fmaf(__uint_as_float(r[i]), scale_log2e, -msub)) : 0.0f;
                        const float p1 = (key + 1 <= pos && key + 1 >= lo) ? t5_ex2(fmaf(__uint_as_float(r[i + 1]), scale_log2e, -msub)) : 0.0f;
                        l += p0 + p1;
                        pk[i >> 1] = t5_pack(p0, p1);
                    }
                }
                t5_st16(my_s + (c >> 1), pk);
            };
            weights(ra, 0);
            weights(rb, 32);
            t5_wait_st();
            t5_fence_before();
            t5_arrive(&p_full[g]);
        }
        // the row sum is the two halves' sums
        x_sum[g][half][row] = l;
        asm volatile("bar.sync %0, 256;\n" ::"r"(1 + g) : "memory");
        l += x_sum[g][half ^ 1][row];
        if (ok && t5_wait(&pv_done[g], (n_tiles - 1) & 1, &abort_flag, status, row_base)) {
            t5_fence_after();
            const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
            bf16* orow = out + (static_cast<size_t>(row_base + row) * nq + h0 + g) * T5_D + half * 64;
#pragma unroll 1
            for (int c = 0; c < 64; c += 32) {
                unsigned r[32];
                t5_ld32(my_o + c, r);
                t5_wait_ld();
                if (row < rows_here) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = t5_pack(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                        w.y = t5_pack(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                        w.z = t5_pack(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
                        w.w = t5_pack(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c + i) = w;
                    }
                }
            }
        }
    }
    t5_fence_before();
    __syncthreads();
    if (warp == 1) {
        t5_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------------
typedef CUresult (*T5EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static T5EncodeFn g_t5_encode = nullptr;
static int g_t5_state = 0;

static bool t5_encode_2d(CUtensorMap* map, const void* base, long long cols, long long rows, int box_cols, int box_rows) {
    if (g_t5_state == 0) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess && fn != nullptr) {
            g_t5_encode = reinterpret_cast<T5EncodeFn>(fn);
            g_t5_state = 1;
        } else {
            (void)cudaGetLastError();
            g_t5_state = -1;
        }
    }
    if (g_t5_state < 0 || rows >= (1LL << 31)) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * sizeof(bf16)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1u, 1u};
    return g_t5_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

extern "C" int llm_paged_prefill_tcgen05_supported(int d, int page_size) {
    return d == T5_D && (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64);
}
extern "C" int llm_paged_prefill_tcgen05_tile_rows() { return T5_BM; }

// q, out: bfloat16 [num_tokens, nq*128]; cache: bfloat16 [pages, 2, nkv, page_size, 128];
// tiles: int32 [n_tiles][2] = (entry, first query row of the tile inside the entry), 128 rows each.
extern "C" int llm_paged_attention_prefill_tcgen05(
    const void* q, void* out, const void* cache, int num_tokens, const int32_t* tiles, int n_tiles,
    const int32_t* entry_slot, const int32_t* entry_q_start, const int32_t* entry_q_len, const int32_t* entry_kv_len,
    const int32_t* block_table, int table_stride, int nq, int nkv, int d, int page_size, int window, float scale,
    int num_pages, int32_t* status, uintptr_t stream) {
    if (n_tiles <= 0) return LLM_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || !llm_paged_prefill_tcgen05_supported(d, page_size) || nq > 65535 ||
        n_tiles > 65535)
        return LLM_REFUSED_SIZE;
    if (!aligned16(q) || !aligned16(out) || !aligned16(cache)) return LLM_REFUSED_ALIGN;
    CUtensorMap q_map, kv_map;
    if (!t5_encode_2d(&q_map, q, static_cast<long long>(nq) * d, num_tokens, 64, T5_BM)) return LLM_REFUSED_SIZE;
    if (!t5_encode_2d(&kv_map, cache, d, static_cast<long long>(num_pages) * 2 * nkv * page_size, 64, page_size))
        return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const float sl2 = scale * 1.4426950408889634f;
    const int group = nq / nkv;
#define T5_GO(HEADS, STAGES)                                                                                         \
    {                                                                                                                \
        const size_t smem = static_cast<size_t>(HEADS * 2 * T5_QHALF + 2 * STAGES * T5_TILE) * sizeof(bf16) + 1024;  \
        auto kern = paged_prefill_attention_tcgen05_kernel<HEADS, STAGES>;                                           \
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                \
                                                   static_cast<int>(smem));                                          \
        if (e != cudaSuccess) return static_cast<int>(e);                                                            \
        launch_pdl(kern, dim3(nq / HEADS, n_tiles), dim3(64 + 128 * HEADS), smem, s, q_map, kv_map,                  \
                   static_cast<bf16*>(out), tiles, entry_slot, entry_q_start, entry_q_len, entry_kv_len,             \
                   block_table, table_stride, nq, nkv, page_size, window, sl2, num_pages, status);                   \
    }
    if (group % 2 == 0) {                                           // two heads of a group share a CTA: the one-pass kernel
        const size_t smem = static_cast<size_t>(2 * 2 * T5_QHALF + 2 * T5O_STAGES * T5O_TILE) * sizeof(bf16) + 1024;
        auto kern = paged_prefill_attention_tcgen05_online_kernel;
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return static_cast<int>(e);
        launch_pdl(kern, dim3(nq / 2, n_tiles), dim3(T5O_THREADS), smem, s, q_map, kv_map, static_cast<bf16*>(out), tiles,
                   entry_slot, entry_q_start, entry_q_len, entry_kv_len, block_table, table_stride, nq, nkv, page_size,
                   window, sl2, num_pages, status);
        return launch_status();
    }
    T5_GO(1, 4)                                                     // odd groups: the two-pass kernel, one head per CTA
#undef T5_GO
    return launch_status();
}
