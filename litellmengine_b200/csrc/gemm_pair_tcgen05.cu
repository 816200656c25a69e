// y[T, N] = x[T, K] . w[N, K]^T for prompt portions (hundreds to thousands of rows): a product on the
// 5th-generation tensor cores that two CTAs of a cluster compute together (tcgen05.mma.cta_group::2),
// with the feed-forward's silu(gate) * up folded into its epilogue.
//
// A pair of CTAs owns a tile of 256 tokens x 256 output features.  Each CTA of the pair brings, per
// stage of 64 k-values, its own 128 tokens of x (operand A) and its own 128 rows of w (half of operand
// B) into shared memory by TMA (128-byte swizzle, K-major); one thread of the pair's first CTA issues
// the products M 256 x N 256 x K 16, which read A from each CTA's own shared memory and both halves of
// B, and leave rows 0..127 of the accumulator in the first CTA's tensor memory and rows 128..255 in
// the second's.  Against one CTA per tile this halves the bytes of w that an SM must fetch per product.
//   * warp 0, one lane: producer.  Both CTAs' copies report to the FIRST CTA's `full` barrier (the
//     loads carry .cta_group::2, which allows a barrier in the peer's shared memory); `empty` barriers
//     are signalled in both CTAs at once by tcgen05.commit with a CTA mask.
//   * warp 1, one lane, first CTA only: issues the products; two accumulators of 256 columns (all of
//     tensor memory), so that a tile's epilogue runs under the next tile's products.
//   * warps 2..5 of both CTAs: epilogue; a thread owns one token (one TMEM lane) and reads its 256 sums
//     32 at a time; the warp turns each 32 x 32 block through shared memory so that eight lanes write one
//     token's 32 columns side by side (a thread writing its own row costs 32 memory transactions an
//     instruction: 8 us of a tile's 25).  Plain mode writes float32 or bfloat16, or adds to the float32
//     that y already holds.  Gate/up mode: w is [gate; up]
//     (2 I rows); the first CTA's half of B is 128 gate rows, the second's the 128 up rows of the same
//     features, so a thread finds gate in columns 0..127 and up in columns 128..255 of its lane and
//     writes silu(bf16(gate)) * bf16(up) as bfloat16 [T, I]: what the product rounded to bfloat16
//     followed by the separate kernel gives, without writing and reading [T, 2 I].
// The kernel is persistent: cluster c takes tiles c, c + clusters, ...; tiles are numbered token tile
// fastest, so that the clusters running at one time share few rows of w and all of x stays in L2.  The
// tiles left over after the last full round are cut in two along the features when that ends sooner.
// Every mbarrier wait is bounded: a wait that runs out sets status code 9 and everyone winds down; the
// two CTAs meet at a cluster barrier before tensor memory is freed, so neither leaves while the other
// may still signal it.
// The reference calls cublasSgemm for every product (src/layers/linear.cu:169-215) and a separate
// kernel for silu(gate) * up (src/ops/silu_and_mul.cu:44-46).
#include "common.cuh"
#include <cuda.h>

#define GP_BM 128                 // tokens per CTA (rows of its half of the accumulator)
#define GP_BN 256                 // accumulator columns per tile (features; gate|up in gate/up mode)
#define GP_BK 64                  // k-values per stage: one 128-byte swizzled row
#define GP_STAGES 6
#define GP_THREADS 192            // producer warp, issuing warp, 4 epilogue warps
#define GP_WAIT_LIMIT 2000000
#define GP_STAGE_BYTES (2 * GP_BM * GP_BK * 2)      // one CTA's part of a stage: 128 rows of x and 128 rows of w

__device__ __forceinline__ unsigned gp_smem(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ unsigned gp_cta_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// The shared::cluster address of the same variable in CTA `rank` of this cluster.
__device__ __forceinline__ unsigned gp_map_to(unsigned smem_addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void gp_mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(gp_smem(bar)), "r"(count));
}
__device__ __forceinline__ void gp_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(gp_smem(bar)), "r"(bytes) : "memory");
}
// Arrival on a barrier anywhere in the cluster (address from gp_map_to).
__device__ __forceinline__ void gp_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool gp_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(gp_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// The same, ordered after arrivals from the other CTA of the cluster.
__device__ __forceinline__ bool gp_try_wait_cluster(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(gp_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
template <bool CLUSTER>
__device__ __forceinline__ bool gp_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag, int32_t* status) {
    for (int i = 0; i < GP_WAIT_LIMIT; ++i) {
        if (CLUSTER ? gp_try_wait_cluster(bar, parity) : gp_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    if (atomicCAS(status, 0, 9) == 0) status[1] = blockIdx.x;
    return false;
}
// A box of the tensor map into this CTA's shared memory; completion is counted on a barrier that may
// lie in the other CTA of the pair (cluster address).
__device__ __forceinline__ void gp_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
                     "r"(gp_smem(dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void gp_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void gp_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// Arrives, once the pair's products issued so far have run, on the barrier at this address in every CTA of `mask`.
__device__ __forceinline__ void gp_commit_pair(unsigned long long* bar, unsigned short mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::
                     "r"(gp_smem(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void gp_mma_pair(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc,
                                            unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::
                     "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void gp_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void gp_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
// Shared-memory operand descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long gp_desc(const void* smem) {
    unsigned long long d = 0;
    d |= static_cast<unsigned long long>((gp_smem(smem) & 0x3FFFF) >> 4);
    d |= static_cast<unsigned long long>(1) << 16;              // leading-dimension offset: unused for swizzled K-major
    d |= static_cast<unsigned long long>(1024 >> 4) << 32;      // stride between 8-row groups
    d |= 1ull << 46;                                            // descriptor version of this architecture
    d |= 2ull << 61;                                            // SWIZZLE_128B
    return d;
}
// Instruction descriptor: bfloat16 x bfloat16 -> float32, M x N (of the pair), both operands K-major.
__host__ __device__ constexpr unsigned gp_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<unsigned>(n >> 3) << 17) | (static_cast<unsigned>(m >> 4) << 24);
}
__device__ __forceinline__ void gp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float gp_silu(float g) { return g / (1.0f + expf(-g)); }

// The work of one cluster, in order: whole tiles c, c + C, ... below `whole` (a multiple of C), then the
// remaining tiles cut `cut` ways along the features (units of 256 / cut accumulator columns), dealt
// round-robin as well.  Tiles are numbered token tile fastest.
struct GpPlan {
    int tiles_m, tiles;      // token tiles; all tiles
    int whole, cut;          // tiles below `whole` are taken whole; the rest in `cut` parts (1 or 2)
};
struct GpUnit {
    int mt, nt, part, cut;
};
__device__ __forceinline__ bool gp_unit(const GpPlan& p, int i, int cluster, int clusters, GpUnit* u) {
    const int rounds = p.whole / clusters;
    int tile;
    if (i < rounds) {
        tile = i * clusters + cluster;
        u->part = 0;
        u->cut = 1;
    } else {
        const int j = (i - rounds) * clusters + cluster;
        if (j >= (p.tiles - p.whole) * p.cut) return false;
        tile = p.whole + j / p.cut;
        u->part = j % p.cut;
        u->cut = p.cut;
    }
    u->mt = tile % p.tiles_m;
    u->nt = tile / p.tiles_m;
    return true;
}

// MODE 0: y[T, N] = x . w^T.  MODE 1: w is [gate; up] of 2 * inter rows, y[T, inter] = silu(gate) * up.
// MODE 2: y[T, N] (float32) += x . w^T: the product joins the residual stream where it lies.
// w_map, w_map2: the same weights read in boxes of 128 and 64 rows (for whole tiles and for halves).
template <int MODE, typename TO>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GP_THREADS, 1) linear_pair_tcgen05_kernel(
    const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
    const __grid_constant__ CUtensorMap w_map2, TO* __restrict__ y,
    int T, int N, int K, int inter, GpPlan plan, int32_t* __restrict__ status) {
    pdl_invite();
    constexpr int TILE_ELEMS = GP_BM * GP_BK;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem_al = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    bf16* a_s = reinterpret_cast<bf16*>(smem_al);                 // [STAGES][128 tokens][64]
    bf16* b_s = a_s + GP_STAGES * TILE_ELEMS;                     // [STAGES][up to 128 rows of w][64]
    __shared__ __align__(8) unsigned long long full[GP_STAGES], empty[GP_STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const unsigned rank = gp_cta_rank();
    const int cluster = blockIdx.x >> 1, clusters = gridDim.x >> 1;
    const int nk = (K + GP_BK - 1) / GP_BK;

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < GP_STAGES; ++s) { gp_mbar_init(&full[s], 1); gp_mbar_init(&empty[s], 1); }
        for (int s = 0; s < 2; ++s) { gp_mbar_init(&acc_full[s], 1); gp_mbar_init(&acc_empty[s], 8); }   // 4 epilogue warps of 2 CTAs
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {                                              // the same warp of both CTAs, for the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(gp_smem(&tmem_base_s)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    gp_fence_before();
    __syncthreads();
    gp_cluster_sync();                                            // the other CTA's barriers exist before anyone signals them
    gp_fence_after();
    const unsigned tmem = tmem_base_s;
    pdl_wait();                                                   // x is the output of the kernel before this one

    if (warp == 0) {
        // ---- producer (both CTAs) ----
        if (lane == 0) {
            const unsigned full_first = gp_map_to(gp_smem(&full[0]), 0);       // the first CTA's barriers
            int it = 0;
            bool ok = true;
            GpUnit u;
            for (int i = 0; ok && gp_unit(plan, i, cluster, clusters, &u); ++i) {
                const int half = (GP_BN / 2) / u.cut;             // rows of w this CTA brings per stage
                const int row_x = u.mt * (2 * GP_BM) + static_cast<int>(rank) * GP_BM;
                const int row_w = MODE == 1 ? (rank == 0 ? 0 : inter) + u.nt * (GP_BN / 2) + u.part * half
                                            : u.nt * GP_BN + u.part * (2 * half) + static_cast<int>(rank) * half;
                const CUtensorMap* wm = u.cut == 1 ? &w_map : &w_map2;
                const unsigned bytes = 2u * (GP_BM + half) * GP_BK * sizeof(bf16);          // both CTAs' boxes
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % GP_STAGES;
                    if (it >= GP_STAGES && !gp_wait<false>(&empty[s], ((it / GP_STAGES) - 1) & 1, &abort_flag, status)) { ok = false; break; }
                    if (rank == 0) gp_arrive_expect_tx(&full[s], bytes);
                    gp_tma_2d(a_s + s * TILE_ELEMS, &x_map, kb * GP_BK, row_x, full_first + s * 8);
                    gp_tma_2d(b_s + s * TILE_ELEMS, wm, kb * GP_BK, row_w, full_first + s * 8);
                }
            }
            if (!ok)                                              // let what is in flight land before the CTA goes away
                for (int n = 0; n < 2000; ++n) __nanosleep(100);
        }
    } else if (warp == 1) {
        // ---- product issuer (first CTA of the pair) ----
        if (lane == 0 && rank == 0) {
            const unsigned long long ad0 = gp_desc(a_s), bd0 = gp_desc(b_s);
            int it = 0;
            bool ok = true;
            GpUnit u;
            for (int i = 0; ok && gp_unit(plan, i, cluster, clusters, &u); ++i) {
                const int buf = i & 1;
                const unsigned idesc = gp_idesc(2 * GP_BM, GP_BN / u.cut);
                if (i >= 2 && !gp_wait<true>(&acc_empty[buf], ((i >> 1) - 1) & 1, &abort_flag, status)) break;
                gp_fence_after();
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % GP_STAGES;
                    if (!gp_wait<false>(&full[s], (it / GP_STAGES) & 1, &abort_flag, status)) { ok = false; break; }
                    gp_fence_after();
                    const unsigned long long ad = ad0 + static_cast<unsigned long long>(s) * (TILE_ELEMS * sizeof(bf16) >> 4);
                    const unsigned long long bd = bd0 + static_cast<unsigned long long>(s) * (TILE_ELEMS * sizeof(bf16) >> 4);
#pragma unroll
                    for (int k = 0; k < GP_BK / 16; ++k)          // 16 k-values = 32 bytes further along the swizzled row
                        gp_mma_pair(tmem + buf * GP_BN, ad + 2 * k, bd + 2 * k, idesc, (kb | k) ? 1u : 0u);
                    gp_commit_pair(&empty[s], 3);                 // the stage is free in both CTAs when these have run
                }
                if (ok) gp_commit_pair(&acc_full[buf], 3);
            }
        }
    } else {
        // ---- epilogue: warps 2..5 of both CTAs.  A thread reads one token's sums (one TMEM lane), 32
        // columns at a time; the warp turns its 32 x 32 block through shared memory (16-byte chunks
        // XOR-swizzled by the row) so that eight lanes write one token's 32 columns side by side ----
        const int quarter = warp & 3;                             // the TMEM lanes this warp may touch
        const unsigned lane_addr = static_cast<unsigned>(quarter * 32) << 16;
        const unsigned acc_empty_first = gp_map_to(gp_smem(&acc_empty[0]), 0);
        float4* turn = reinterpret_cast<float4*>(b_s + GP_STAGES * TILE_ELEMS) + (warp - 2) * (32 * 8);    // [32 rows][8 chunks]
        const int out_n = MODE == 1 ? inter : N;
        GpUnit u;
        for (int i = 0; gp_unit(plan, i, cluster, clusters, &u); ++i) {
            const int buf = i & 1;
            if (!gp_wait<false>(&acc_full[buf], (i >> 1) & 1, &abort_flag, status)) break;
            gp_fence_after();
            const int tok0 = u.mt * (2 * GP_BM) + static_cast<int>(rank) * GP_BM + quarter * 32;       // the warp's first token
            const unsigned acc = tmem + lane_addr + buf * GP_BN;
            const int cols = GP_BN / u.cut;                       // accumulator columns of this unit
            const int out_cols = MODE == 1 ? cols / 2 : cols;     // columns it writes
            const int f0 = (MODE == 1 ? u.nt * (GP_BN / 2) : u.nt * GP_BN) + u.part * out_cols;
#pragma unroll 1
            for (int c = 0; c < out_cols; c += 32) {
                float v[32];
                float4 old[8];                                    // MODE 2: what y holds, asked for before anything waits
                if (MODE == 2) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const int tok = tok0 + k * 4 + (lane >> 3), col = f0 + c + (lane & 7) * 4;
                        old[k] = (tok < T && col < out_n)
                                     ? *reinterpret_cast<const float4*>(y + static_cast<size_t>(tok) * out_n + col)
                                     : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    }
                }
                if (MODE == 1) {
                    unsigned g[32], up[32];
                    gp_ld32(acc + c, g);
                    gp_ld32(acc + out_cols + c, up);
                    gp_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const float gate = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[e])));
                        const float upv = __bfloat162float(__float2bfloat16_rn(__uint_as_float(up[e])));
                        v[e] = gp_silu(gate) * upv;
                    }
                } else {
                    unsigned r[32];
                    gp_ld32(acc + c, r);
                    gp_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    turn[lane * 8 + (j ^ (lane & 7))] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                __syncwarp();
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int rl = k * 4 + (lane >> 3), q = lane & 7;
                    float4 val = turn[rl * 8 + (q ^ (rl & 7))];
                    const int tok = tok0 + rl, col = f0 + c + q * 4;
                    if (tok < T && col < out_n) {                 // out_n is a multiple of 8
                        TO* dst = y + static_cast<size_t>(tok) * out_n + col;
                        if constexpr (sizeof(TO) == 4) {
                            if (MODE == 2) { val.x += old[k].x; val.y += old[k].y; val.z += old[k].z; val.w += old[k].w; }
                            *reinterpret_cast<float4*>(dst) = val;
                        } else {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(val.x, val.y), hi = __floats2bfloat162_rn(val.z, val.w);
                            uint2 packed;
                            packed.x = *reinterpret_cast<unsigned*>(&lo);
                            packed.y = *reinterpret_cast<unsigned*>(&hi);
                            *reinterpret_cast<uint2*>(dst) = packed;
                        }
                    }
                }
                __syncwarp();
            }
            gp_fence_before();
            __syncwarp();
            if (lane == 0) gp_arrive_cluster(acc_empty_first + buf * 8);
        }
    }
    gp_fence_before();
    __syncthreads();
    gp_cluster_sync();                                            // nobody signals a CTA that has left
    if (warp == 1) {
        gp_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512) : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*GpEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static GpEncodeFn g_gp_encode = nullptr;
static int g_gp_state = 0;
static int g_gp_sms = 0;

static bool gp_ready() {
    if (g_gp_state == 0) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        int dev = 0;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess && fn != nullptr && cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&g_gp_sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && g_gp_sms >= 2) {
            g_gp_encode = reinterpret_cast<GpEncodeFn>(fn);
            g_gp_state = 1;
        } else {
            (void)cudaGetLastError();
            g_gp_state = -1;
        }
    }
    return g_gp_state > 0;
}

// A [rows, cols] bfloat16 matrix, row-major, read in boxes of box_rows rows x 64 columns (128-byte
// swizzle); rows and columns past the end read as zero.
static bool gp_encode(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * sizeof(bf16)};
    const cuuint32_t box[2] = {GP_BK, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1u, 1u};
    return g_gp_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Sizes this kernel takes: K and N multiples of 8 (16-byte rows for the copy engine and the stores).
extern "C" int llm_linear_pair_supported(int T, int N, int K) {
    return T >= 1 && N >= 8 && K >= 8 && (K % 8) == 0 && (N % 8) == 0;
}

// Whole tiles for as many full rounds of all clusters as there are; the tiles left over are taken whole or
// cut in two along the features, whichever ends sooner (a half counts as half a round).  Narrower units
// do not pay: 64 columns take 0.42 of a tile's time.
static void gp_make_plan(int tiles_m, int tiles_n, GpPlan* plan, int* clusters) {
    const int tiles = tiles_m * tiles_n, slots = g_gp_sms / 2;
    const int whole = tiles >= slots ? (tiles / slots) * slots : 0, rest = tiles - whole;
    const int cut = ((rest * 2 + slots - 1) / slots) < 2 * ((rest + slots - 1) / slots) ? 2 : 1;
    plan->tiles_m = tiles_m;
    plan->tiles = tiles;
    plan->whole = whole;
    plan->cut = cut;
    *clusters = whole > 0 ? slots : (rest * cut < slots ? rest * cut : slots);
}

// How full the clusters are kept by a product of T tokens and N output features (gate/up mode: N =
// inter), in thousandths: the tiles' share of the time that the rounds of the plan take.  0 if the
// device or the sizes are not taken.
extern "C" int llm_linear_pair_efficiency(int T, int N, int K, int gate_up) {
    if (!llm_linear_pair_supported(T, N, K) || !gp_ready()) return 0;
    const int tiles_m = (T + 2 * GP_BM - 1) / (2 * GP_BM);
    const int per_tile = gate_up ? GP_BN / 2 : GP_BN;
    const long long tiles_n = (N + per_tile - 1) / per_tile;
    if (tiles_m * tiles_n > (1LL << 28)) return 0;
    GpPlan plan;
    int clusters;
    gp_make_plan(tiles_m, static_cast<int>(tiles_n), &plan, &clusters);
    const int slots = g_gp_sms / 2, rest = plan.tiles - plan.whole;
    const double rounds = plan.whole / slots + static_cast<double>((rest * plan.cut + slots - 1) / slots) / plan.cut;
    const double work = static_cast<double>(T) * N / (2.0 * GP_BM * per_tile) / slots;
    return static_cast<int>(1000.0 * work / rounds);
}

template <int MODE, typename TO>
static int gp_launch(const bf16* x, const bf16* w, void* y, int T, int N, int K, int inter, long long w_rows, int32_t* status,
                     cudaStream_t s) {
    CUtensorMap x_map, w_map, w_map2;
    if (!gp_encode(&x_map, x, T, K, GP_BM) || !gp_encode(&w_map, w, w_rows, K, GP_BN / 2) ||
        !gp_encode(&w_map2, w, w_rows, K, GP_BN / 4))
        return LLM_REFUSED_SIZE;
    const int tiles_m = (T + 2 * GP_BM - 1) / (2 * GP_BM);
    const int tiles_n = MODE == 1 ? (inter + GP_BN / 2 - 1) / (GP_BN / 2) : (N + GP_BN - 1) / GP_BN;
    if (static_cast<long long>(tiles_m) * tiles_n > (1LL << 28)) return LLM_REFUSED_SIZE;
    GpPlan plan;
    int clusters;
    gp_make_plan(tiles_m, tiles_n, &plan, &clusters);
    const size_t smem = static_cast<size_t>(GP_STAGES) * GP_STAGE_BYTES + 4 * 32 * 32 * sizeof(float) + 1024;   // stages, the epilogue's four blocks, alignment
    auto kern = linear_pair_tcgen05_kernel<MODE, TO>;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    launch_pdl(kern, dim3(2 * clusters), dim3(GP_THREADS), smem, s, x_map, w_map, w_map2, static_cast<TO*>(y), T, N, K,
               inter, plan, status);
    return launch_status();
}

// x: bfloat16 [T, K]; w: bfloat16 [N, K]; y: [T, N] float32 (out_dtype 0) or bfloat16 (1).  accumulate: y (float32)
// holds a summand already and the product is added to it.
extern "C" int llm_linear_pair(const void* x, const void* w, void* y, int out_dtype, int accumulate, int T, int N, int K,
                               int32_t* status, uintptr_t stream) {
    if (!llm_linear_pair_supported(T, N, K)) return LLM_REFUSED_SIZE;
    if (!aligned16(x) || !aligned16(w) || !aligned16(y) || status == nullptr) return LLM_REFUSED_ALIGN;
    if (!gp_ready()) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bf16* xp = static_cast<const bf16*>(x);
    const bf16* wp = static_cast<const bf16*>(w);
    if (accumulate) {
        if (out_dtype != LLM_DT_F32) return LLM_REFUSED_DTYPE;
        return gp_launch<2, float>(xp, wp, y, T, N, K, 0, N, status, s);
    }
    if (out_dtype == LLM_DT_F32) return gp_launch<0, float>(xp, wp, y, T, N, K, 0, N, status, s);
    if (out_dtype == LLM_DT_BF16) return gp_launch<0, bf16>(xp, wp, y, T, N, K, 0, N, status, s);
    return LLM_REFUSED_DTYPE;
}

// x: bfloat16 [T, K]; w: bfloat16 [2 * inter, K] = [gate; up]; y: bfloat16 [T, inter] = silu(gate) * up, gate and up
// rounded to bfloat16 first.
extern "C" int llm_linear_pair_silu_mul(const void* x, const void* w, void* y, int T, int inter, int K, int32_t* status,
                                        uintptr_t stream) {
    if (!llm_linear_pair_supported(T, inter, K)) return LLM_REFUSED_SIZE;
    if (!aligned16(x) || !aligned16(w) || !aligned16(y) || status == nullptr) return LLM_REFUSED_ALIGN;
    if (!gp_ready()) return LLM_REFUSED_SIZE;
    return gp_launch<1, bf16>(static_cast<const bf16*>(x), static_cast<const bf16*>(w), y, T, inter, K, inter, 2LL * inter, status,
                              reinterpret_cast<cudaStream_t>(stream));
}
