// y[T, N] = x[T, K] . w[N, K]^T for 17..128 rows (decode steps of larger batches): a
// weight-streaming product on the 5th-generation tensor cores.
//
// With this few rows the product is still bound by reading w once (24576 x 4096 weights against
// 64 rows: 200 MB to read, 13 GFLOP to do), so the shape is that of the mma.sync kernel for up to
// 16 rows (gemm_skinny.cu), with the roles swapped for tcgen05: a tile of 128 output features of
// w is the M = 128 operand A, the tokens are the N operand B (padded to NT = 32, 64 or 128 by the
// copy engine's zero fill), and the accumulator D[128 features, NT tokens] lives in tensor memory.
//   * warp 0, one lane: producer.  The weights come from the copy stored tile by tile (ops.tile_weight:
//     [N/64][K/256] blocks of four [64 rows][64 k-values] sub-tiles in the 128-byte-swizzled K-major
//     order): a stage's operand A, 128 features x 64 k-values, is two contiguous 8 KB sub-tiles, each
//     one cp.async.bulk.  (Fetched by TMA boxes from the plain [N, K] layout the same kernel was bound
//     by DRAM's dislike of 128-byte pieces 8 KB apart: 54-98 us where the library takes 37-40.)  The
//     tokens x [NT x 64 k-values] come by one TMA box per stage.  w does not depend on the kernel
//     before this one, so its first stages are requested before griddepcontrol.wait, x after it.
//   * warp 1, one lane: issues tcgen05.mma (M 128 x N NT x K 16, four per stage) and owns the TMEM
//     allocation (two accumulators of NT columns, so that the epilogue of one segment runs while
//     the next segment's products are issued).
//   * warps 2..5: epilogue; a thread owns one feature (one TMEM lane) and writes its NT sums.
// Work is cut as in gemm_skinny.cu: items of 128 features x 64 k-values, numbered feature tile by
// feature tile; whole k-splits per tile when they fill the CTA slots well, otherwise one even run
// of items per CTA, with float32 partial sums in slices added by a second kernel or the consumer.
// Every mbarrier wait is bounded; a wait that runs out sets status code 7 and the CTA winds down.
// Measured (B200, chain of launches over weights larger than L2): 24576 x 4096 weights take 52 / 68 /
// 100 us for 32 / 64 / 128 rows against 37 / 40 / 40 us for the library's kernels, whichever way the
// operands are fetched (TMA boxes from the plain layout, bulk copies of the tiled copy; tokens by TMA
// or cp.async).  Taking the products out changes nothing; taking the epilogue's stores out gives 42 /
// 58 us: a thread writes its feature's NT sums one 4-byte store at a time at the end of the CTA's
// life, and the tokens' tile is read again from L2 for every 128 features (as many bytes as the
// weights at 128 rows).  The engine therefore keeps the library for these row counts unless
// LLM_STREAM=on; what this kernel needs next is 256 features per token tile and an epilogue that
// goes through shared memory.
// The reference calls cublasSgemm for every product (src/layers/linear.cu:169-215).
#include "common.cuh"
#include <cuda.h>

#define GT_BM 128                 // output features per tile (rows of A)
#define GT_BK 64                  // k-values per stage: one 128-byte swizzled row
#define GT_WAIT_LIMIT 400000
#define GT_THREADS 320                // producer warp, issuing warp, 4 epilogue warps, 4 warps that fetch the tokens

__device__ __forceinline__ unsigned gt_smem(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void gt_mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(gt_smem(bar)), "r"(count));
}
__device__ __forceinline__ void gt_expect_tx(unsigned long long* bar, unsigned bytes) {       // no arrival
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;\n" ::"r"(gt_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gt_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(gt_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gt_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(gt_smem(bar)) : "memory");
}
__device__ __forceinline__ bool gt_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(gt_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool gt_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag, int32_t* status) {
    for (int i = 0; i < GT_WAIT_LIMIT; ++i) {
        if (gt_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    if (atomicCAS(status, 0, 7) == 0) status[1] = blockIdx.x;
    return false;
}
__device__ __forceinline__ void gt_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
                     "r"(gt_smem(dst)), "l"(map), "r"(x), "r"(y), "r"(gt_smem(bar)) : "memory");
}
__device__ __forceinline__ void gt_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void gt_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void gt_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(gt_smem(bar)) : "memory");
}
__device__ __forceinline__ void gt_mma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::
                     "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void gt_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
// Shared-memory operand descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long gt_desc(const void* smem) {
    unsigned long long d = 0;
    d |= static_cast<unsigned long long>((gt_smem(smem) & 0x3FFFF) >> 4);
    d |= static_cast<unsigned long long>(1) << 16;              // leading-dimension offset: unused for swizzled K-major
    d |= static_cast<unsigned long long>(1024 >> 4) << 32;      // stride between 8-row groups
    d |= 1ull << 46;                                            // descriptor version of this architecture
    d |= 2ull << 61;                                            // SWIZZLE_128B
    return d;
}
// Instruction descriptor: bfloat16 x bfloat16 -> float32, M x N, both operands K-major.
__host__ __device__ constexpr unsigned gt_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<unsigned>(n >> 3) << 17) | (static_cast<unsigned>(m >> 4) << 24);
}
// Which CTA of `ctas` holds item `item` when CTA c takes items [c*total/ctas, (c+1)*total/ctas).
__host__ __device__ __forceinline__ long long gt_cta_of(long long item, long long total, long long ctas) {
    return ((item + 1) * ctas - 1) / total;
}

// NT: token tile (columns of the accumulator).  slices: float32 partial-sum slices of [T, N] in
// `partial` (1: none, y is written directly).  per_tile: CTAs that share a tile's k-values evenly
// (0: one even run of all items per CTA).
template <int NT, int STAGES, typename TO>
__global__ void __launch_bounds__(GT_THREADS) linear_stream_tcgen05_kernel(
    const bf16* __restrict__ w_tiled, const bf16* __restrict__ x, TO* __restrict__ y,
    float* __restrict__ partial, int T, int N, int K, int slices, int per_tile, int32_t* __restrict__ status) {
    pdl_invite();
    constexpr int A_ELEMS = GT_BM * GT_BK, B_ELEMS = NT * GT_BK;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem_al = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    bf16* a_s = reinterpret_cast<bf16*>(smem_al);                 // [STAGES][128][64]
    bf16* b_s = a_s + STAGES * A_ELEMS;                           // [STAGES][NT][64]
    __shared__ __align__(8) unsigned long long full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base_s;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nk = (K + GT_BK - 1) / GT_BK, tiles = (N + GT_BM - 1) / GT_BM;
    const long long total = static_cast<long long>(tiles) * nk, ctas = gridDim.x;
    long long begin;
    int count;
    if (per_tile) {
        const int t = blockIdx.x / per_tile, part = blockIdx.x % per_tile;
        const int k_begin = static_cast<int>(static_cast<long long>(part) * nk / per_tile);
        begin = static_cast<long long>(t) * nk + k_begin;
        count = static_cast<int>(static_cast<long long>(part + 1) * nk / per_tile) - k_begin;
    } else {
        begin = blockIdx.x * total / ctas;
        count = static_cast<int>((blockIdx.x + 1) * total / ctas - begin);
    }

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { gt_mbar_init(&full[s], 1 + 128); gt_mbar_init(&empty[s], 1); }   // weights + 128 token fetchers
        for (int s = 0; s < 2; ++s) { gt_mbar_init(&acc_full[s], 1); gt_mbar_init(&acc_empty[s], 128); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(gt_smem(&tmem_base_s)), "r"(2 * NT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    gt_fence_before();
    __syncthreads();
    gt_fence_after();
    const unsigned tmem = tmem_base_s;

    if (warp == 0) {
        // ---- producer ----
        if (lane == 0) {
            constexpr unsigned A_BYTES = A_ELEMS * sizeof(bf16);
            const int tiles64 = (N + 63) / 64;
            const long long nk256 = (K + 255) / 256;
            auto load_w = [&](int i) {                            // two sub-tiles: features 0..63 and 64..127 of the tile
                const long long item = begin + i;
                const int tile = static_cast<int>(item / nk), kc = static_cast<int>(item % nk);
                const bool two = 2 * tile + 1 < tiles64;          // the last tile may have one half only
                gt_arrive_expect_tx(&full[i % STAGES], two ? A_BYTES : A_BYTES / 2);
                for (int h = 0; h < (two ? 2 : 1); ++h) {
                    const bf16* src = w_tiled + ((static_cast<size_t>(2 * tile + h) * nk256 + (kc >> 2)) * 4 + (kc & 3)) * (64 * 64);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::
                                     "r"(gt_smem(a_s + (i % STAGES) * A_ELEMS + h * (64 * 64))), "l"(src), "r"(A_BYTES / 2),
                                 "r"(gt_smem(&full[i % STAGES])) : "memory");
                }
            };
            const int ahead = count < STAGES ? count : STAGES;
            for (int i = 0; i < ahead; ++i) load_w(i);            // weights: nobody in this step writes them
            int issued = ahead;
            for (int i = STAGES; i < count; ++i) {
                if (!gt_wait(&empty[i % STAGES], ((i / STAGES) - 1) & 1, &abort_flag, status)) break;
                load_w(i);
                issued = i + 1;
            }
            if (abort_flag)                                       // let what is in flight land before the CTA goes away
                for (int i = max(0, issued - STAGES); i < issued; ++i)
                    for (int n = 0; n < GT_WAIT_LIMIT && !gt_try_wait(&full[i % STAGES], (i / STAGES) & 1); ++n) {}
        }
    } else if (warp >= 6) {
        // ---- the tokens: warps 6..9 copy x[0..T) x 64 k-values of every stage with cp.async into the
        // 128-byte-swizzled K-major tile (rows of x are K values apart: a TMA box of such rows costs the
        // copy engine 21 clocks a row, which was this kernel's time) ----
        const int lt = tid - 6 * 32;                              // 0..127
        constexpr int LAG = 2;                                    // stages of x a thread keeps in flight
        constexpr int PER = NT * 8 / 128;                         // 16-byte chunks per thread and stage
        pdl_wait();                                               // x is the output of the kernel before this one
        auto arrive_after_copies = [&](int i) {
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");       // the tensor core reads through the async proxy
            gt_arrive(&full[i % STAGES]);
        };
        bool ok = true;
        int done = 0;                                             // stages whose arrival has been made
        for (int i = 0; i < count; ++i) {
            const int st = i % STAGES;
            if (i >= STAGES && !gt_wait(&empty[st], ((i / STAGES) - 1) & 1, &abort_flag, status)) { ok = false; break; }
            const int k0 = static_cast<int>((begin + i) % nk) * GT_BK;
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const int c = lt + 128 * j, row = c >> 3, ch = c & 7;
                const bool valid = row < T && k0 + ch * 8 < K;
                const unsigned dst = gt_smem(b_s + st * B_ELEMS + row * 64 + ((ch ^ (row & 7)) << 3));
                const bf16* src = x + (valid ? static_cast<size_t>(row) * K + k0 + ch * 8 : 0);
                const int bytes = valid ? 16 : 0;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
            }
            asm volatile("cp.async.commit_group;\n" ::);
            if (i >= LAG) {
                asm volatile("cp.async.wait_group %0;\n" ::"n"(LAG));
                arrive_after_copies(done++);
            }
        }
        asm volatile("cp.async.wait_group 0;\n" ::);
        if (ok)
            while (done < count) arrive_after_copies(done++);
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            constexpr unsigned IDESC = gt_idesc(GT_BM, NT);
            const unsigned long long ad0 = gt_desc(a_s), bd0 = gt_desc(b_s);
            int kt = static_cast<int>(begin % nk), seg = 0;
            bool fresh = true;                                    // the next product starts a segment's accumulator
            for (int i = 0; i < count; ++i) {
                const int st = i % STAGES, buf = seg & 1;
                if (fresh && seg >= 2 && !gt_wait(&acc_empty[buf], ((seg >> 1) - 1) & 1, &abort_flag, status)) break;
                if (!gt_wait(&full[st], (i / STAGES) & 1, &abort_flag, status)) break;
                gt_fence_after();
                const unsigned long long ad = ad0 + static_cast<unsigned long long>(st) * (A_ELEMS * sizeof(bf16) >> 4);
                const unsigned long long bd = bd0 + static_cast<unsigned long long>(st) * (B_ELEMS * sizeof(bf16) >> 4);
#pragma unroll
                for (int k = 0; k < GT_BK / 16; ++k)              // 16 k-values = 32 bytes further along the swizzled row
                    gt_mma(tmem + buf * NT, ad + 2 * k, bd + 2 * k, IDESC, (fresh && k == 0) ? 0u : 1u);
                gt_commit(&empty[st]);                            // the stage is free when these products have run
                fresh = false;
                if (kt == nk - 1 || i == count - 1) {             // the segment (this CTA's part of a tile) is complete
                    gt_commit(&acc_full[buf]);
                    fresh = true;
                    ++seg;
                }
                kt = (kt == nk - 1) ? 0 : kt + 1;
            }
        }
    } else {
        // ---- epilogue: warps 2..5, thread = one feature = one TMEM lane ----
        // (warps 6..9 were taken by the branch above)
        const int quarter = warp & 3;                             // the TMEM lanes this warp may touch
        const unsigned lane_addr = static_cast<unsigned>(quarter * 32) << 16;
        int tile = static_cast<int>(begin / nk), kt = static_cast<int>(begin % nk), seg = 0;
        for (int i = 0; i < count;) {
            const int left_in_tile = nk - kt;
            const int len = (count - i) < left_in_tile ? (count - i) : left_in_tile;     // items of this segment
            const bool tile_done = len == left_in_tile;
            const int buf = seg & 1;
            if (!gt_wait(&acc_full[buf], (seg >> 1) & 1, &abort_flag, status)) break;
            gt_fence_after();
            const int f = tile * GT_BM + quarter * 32 + lane;
            const int slice = per_tile ? static_cast<int>(blockIdx.x % per_tile)
                                       : static_cast<int>(blockIdx.x - gt_cta_of(static_cast<long long>(tile) * nk, total, ctas));
#pragma unroll 1
            for (int c = 0; c < NT; c += 32) {
                unsigned r[32];
                gt_ld32(tmem + lane_addr + buf * NT + c, r);
                if (f < N) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int tok = c + j;
                        if (tok < T) {
                            if (slices == 1) {
                                y[static_cast<size_t>(tok) * N + f] = from_f32<TO>(__uint_as_float(r[j]));
                            } else {
                                partial[(static_cast<size_t>(slice) * T + tok) * N + f] = __uint_as_float(r[j]);
                                if (tile_done && !per_tile)       // nobody else comes after: clear the unused slices
                                    for (int z = slice + 1; z < slices; ++z) partial[(static_cast<size_t>(z) * T + tok) * N + f] = 0.0f;
                            }
                        }
                    }
                }
            }
            gt_fence_before();
            gt_arrive(&acc_empty[buf]);
            i += len;
            ++seg;
            if (tile_done) { kt = 0; ++tile; } else kt += len;
        }
    }
    gt_fence_before();
    __syncthreads();
    if (warp == 1) {
        gt_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * NT) : "memory");
    }
}

// y[tok, f] = sum over slices of partial[slice, tok, f], in slice order.
template <typename TO>
__global__ void linear_stream_sum_kernel(const float* __restrict__ partial, TO* __restrict__ y, long long mn, int slices) {
    pdl_begin();
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= mn) return;
    float v = 0.0f;
    for (int s = 0; s < slices; ++s) v += partial[s * mn + i];
    y[i] = from_f32<TO>(v);
}

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*GtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static GtEncodeFn g_gt_encode = nullptr;
static int g_gt_state = 0;
static int g_gt_sms = 0;

static bool gt_ready() {
    if (g_gt_state == 0) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        int dev = 0;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess && fn != nullptr && cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&g_gt_sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && g_gt_sms > 0) {
            g_gt_encode = reinterpret_cast<GtEncodeFn>(fn);
            g_gt_state = 1;
        } else {
            (void)cudaGetLastError();
            g_gt_state = -1;
        }
    }
    return g_gt_state > 0;
}

extern "C" int llm_linear_stream_supported(int T, int N, int K) {
    return T >= 1 && T <= 128 && N >= 1 && K >= 8 && (K % 8) == 0;
}

// The grid for a product and the number of partial-sum slices it leaves (1 = none): two CTAs per
// SM; whole k-splits per tile when they fill at least 85 % of the slots, else one even run per slot.
static void gt_plan(int N, int K, int* ctas, int* slices, int* per_tile) {
    const long long slots = 2LL * g_gt_sms;
    const long long tiles = (N + GT_BM - 1) / GT_BM, nk = (K + GT_BK - 1) / GT_BK, total = tiles * nk;
    long long best = 0;
    for (long long s = 1; s <= 16 && s <= (nk >= 8 ? nk / 8 : 1); ++s)      // at least eight items per CTA
        if (tiles * s <= slots) best = s;
    if (best && tiles * best * 100 >= 85 * slots) {
        *ctas = static_cast<int>(tiles * best);
        *slices = *per_tile = static_cast<int>(best);
        return;
    }
    long long g = total / 8;
    if (g < 1) g = 1;
    if (g > slots) g = slots;
    int s = 1;
    if (!(total % g == 0 && (total / g) % nk == 0)) {
        s = 0;
        for (long long t = 0; t < tiles; ++t) {
            const int n = static_cast<int>(gt_cta_of((t + 1) * nk - 1, total, g) - gt_cta_of(t * nk, total, g)) + 1;
            if (n > s) s = n;
        }
    }
    *ctas = static_cast<int>(g);
    *slices = s;
    *per_tile = 0;
}

// The number of partial-sum slices a product of these sizes leaves on the current device.
extern "C" int llm_linear_stream_slices(int T, int N, int K) {
    (void)T;
    if (!gt_ready()) return 1;
    int ctas, slices, per_tile;
    gt_plan(N, K, &ctas, &slices, &per_tile);
    return slices;
}

template <int NT, typename TO>
static int gt_launch(const bf16* w_tiled, const bf16* x, void* y, float* scratch, int T, int N, int K, int ctas,
                     int slices, int per_tile, int32_t* status, cudaStream_t s) {
    constexpr int STAGES = NT <= 64 ? 4 : 3;                      // two CTAs per SM must fit
    const size_t smem = static_cast<size_t>(STAGES) * (GT_BM + NT) * GT_BK * sizeof(bf16) + 1024;
    auto kern = linear_stream_tcgen05_kernel<NT, STAGES, TO>;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    launch_pdl(kern, dim3(ctas), dim3(GT_THREADS), smem, s, w_tiled, x, static_cast<TO*>(y), scratch, T, N, K, slices, per_tile,
               status);
    return launch_status();
}

// x: bfloat16 [T, K]; w_tiled: the weights [N, K] stored tile by tile (ops.tile_weight); y: [T, N] float32
// (out_dtype 0) or bfloat16 (1);
// scratch: float32, slices * T * N elements when llm_linear_stream_slices says more than one.
// keep_partials: leave the partial sums in scratch as [slices, T, N] and write nothing to y.
extern "C" int llm_linear_stream(const void* x, const void* w_tiled, void* y, int out_dtype, float* scratch, long long scratch_floats,
                                 int T, int N, int K, int keep_partials, int32_t* status, uintptr_t stream) {
    if (!llm_linear_stream_supported(T, N, K)) return LLM_REFUSED_SIZE;
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(w_tiled) & 127u) != 0) return LLM_REFUSED_ALIGN;
    if (!gt_ready()) return LLM_REFUSED_SIZE;
    int ctas, slices, per_tile;
    gt_plan(N, K, &ctas, &slices, &per_tile);
    if (slices > 1 && (scratch == nullptr || scratch_floats < static_cast<long long>(slices) * T * N)) return LLM_REFUSED_SIZE;
    const int nt = T <= 32 ? 32 : (T <= 64 ? 64 : 128);
    const bf16* wt = static_cast<const bf16*>(w_tiled);
    const bf16* xp = static_cast<const bf16*>(x);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    int rc;
#define GO(NTV)                                                                                                         \
    rc = out_dtype == LLM_DT_F32 ? gt_launch<NTV, float>(wt, xp, y, scratch, T, N, K, ctas, slices, per_tile, status, s) \
                                 : gt_launch<NTV, bf16>(wt, xp, y, scratch, T, N, K, ctas, slices, per_tile, status, s)
    if (out_dtype != LLM_DT_F32 && out_dtype != LLM_DT_BF16) return LLM_REFUSED_DTYPE;
    if (nt == 32) GO(32); else if (nt == 64) GO(64); else GO(128);
#undef GO
    if (rc != LLM_OK || slices == 1 || keep_partials) return rc;
    const long long mn = static_cast<long long>(T) * N;
    if (out_dtype == LLM_DT_F32)
        launch_pdl((linear_stream_sum_kernel<float>), dim3(static_cast<unsigned>((mn + 255) / 256)), dim3(256), 0, s, scratch, static_cast<float*>(y), mn, slices);
    else
        launch_pdl((linear_stream_sum_kernel<bf16>), dim3(static_cast<unsigned>((mn + 255) / 256)), dim3(256), 0, s, scratch, static_cast<bf16*>(y), mn, slices);
    return launch_status();
}
