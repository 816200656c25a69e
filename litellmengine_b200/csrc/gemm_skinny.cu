// y[M, N] = x[M, K] . w[N, K]^T for a handful of rows (decode steps): a weight-streaming kernel.
//
// With few rows the product is bound by reading w once, and what decides the speed is how many
// bytes of w each SM keeps in flight and whether every SM is busy until the end.  The library's
// kernels for these shapes reach 40-60 % of the memory bandwidth when N is small (N = 4096 or 6144
// gives fewer thread blocks than the GPU has SMs).  Here the work is cut into items of 64 output
// features (one 16-row tensor-core tile per warp) by 256 k-values (128 for 16 tokens), numbered
// feature tile by feature tile, and the grid is persistent: two CTAs per SM, each taking one
// contiguous run of items of (nearly) the same length, whatever N and K are.  A CTA streams its
// items through three stages of shared memory (five for 16 tokens): 32 KB of w per stage, brought
// by the copy engine (one bulk copy of a stored tile, or four boxes of the plain weights; see
// below), and 4 KB of x by cp.async, without draining the pipeline between feature tiles.  A
// feature tile whose items lie in several CTAs gets one float32 partial sum from each, in a slice
// numbered by the CTA's place among them (the CTA that finishes the tile zeroes the slices nobody
// uses); a second small kernel, or the consumer, adds the slices in order (no atomics: the result
// does not depend on timing).  When every tile lies in one CTA the result is written directly.
// The product runs on the tensor cores with the roles swapped: w is the 16-row A operand of
// mma.sync m16n8k16 and the tokens are the 8 columns of B (8 tokens use a full instruction,
// 16 tokens two).  Accumulation is float32; the result is float32 or bfloat16.
// The reference calls cublasSgemm for every product (src/layers/linear.cu:169-215).
#include "common.cuh"
#include <cuda.h>
#include <unordered_map>

#define GS_ROWS 64          // output features per CTA (16 per warp)
// k-values per stage and stages, by token tile: two CTAs per SM must fit.  Three stages of weights (two
// for the 32-token tile, which only small, latency-bound products take) of
// 256 k-values (512 contiguous bytes of each weight row per request, which the memory system serves
// better than 256: 6.2 against 5.9 TB/s on the output head).  The tokens' rows of a stage come from L2:
// up to 8 tokens they are fetched two stages ahead like the weights; 16 tokens have room for two
// stages of rows only and fetch one stage ahead (five stages of 128 k-values, the layout before, paid
// a barrier round per 16 KB of weights: 39.4 us on a 24,576 x 4,096 product where this takes 36).
#define GS_BK_FOR(MT) 256
#define GS_STAGES_FOR(MT) ((MT) <= 16 ? 3 : 2)
#define GS_XSTAGES_FOR(MT) ((MT) <= 8 ? 3 : 2)
#define GS_THREADS 128

__device__ __forceinline__ void gs_cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void gs_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void gs_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void gs_ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void gs_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16-byte chunk `chunk` of row `row` in a [rows][BK] bfloat16 stage, XOR-swizzled.
template <int BK> __device__ __forceinline__ bf16* gs_at(bf16* base, int row, int chunk) {
    return base + row * BK + ((chunk ^ (row & 7)) << 3);
}

// Which CTA of `ctas` holds item `item` when CTA c takes items [c*total/ctas, (c+1)*total/ctas).
__host__ __device__ __forceinline__ long long gs_cta_of(long long item, long long total, long long ctas) {
    return ((item + 1) * ctas - 1) / total;
}

// ---- where a stage's weights come from ----------------------------------------------------------------
// Tiled: `w_tiled` holds the weights as the kernel wants them in shared memory: [feature tile][k-step]
// blocks of 64 x 256 values (32 KB), each block four sub-tiles of [64 rows][64 k-values] with 128-byte
// rows whose 16-byte chunks are XOR-swizzled by the row (chunk c of row r at position c ^ (r % 8):
// the layout the copy engine's 128-byte swizzle writes and tcgen05 reads as a K-major operand, so
// zero-padded at the edges.  A stage of weights is then ONE
// contiguous piece of memory (a block of 32 KB),
// fetched by one bulk copy (cp.async.bulk) of one thread instead of 2,048 sixteen-byte copies
// of 128 threads, and DRAM sees whole pages instead of 512-byte runs 8 KB apart (measured with
// the copy engine alone: 7.4 TB/s for contiguous pieces against 6.2 for the strided form; a whole
// decode step of the Qwen3-8B shape at batch 8: 3.60 ms from the stored tiles, 3.69 ms from boxes
// of the plain weights, 3.75 ms with sixteen-byte cp.async copies of the plain weights).  The
// tokens' rows come by cp.async.  The wait on a stage's mbarrier is bounded;
// when it runs out the kernel records status code 8 and goes on (its result is then flagged).
#define GS_TILED_BK 256          // k-values of a stored block
#define GS_TILED_WAIT_LIMIT 2000000

__device__ __forceinline__ unsigned gs_smem(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ bool gs_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(gs_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// 16-byte chunk `chunk` (of 32) of row `row` in a [4 sub-tiles][64 rows][64 k-values] block.
__device__ __forceinline__ bf16* gs_at_tiled(bf16* base, int row, int chunk) {
    return base + (chunk >> 3) * (GS_ROWS * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
}

// A stage is a whole 32 KB block; three stages of weights, and three (up to 8 tokens) or two (16) of the
// tokens' rows, so that two CTAs fit an SM.
//
// BOXES: the same stage fetched from the plain [N, K] weights instead, by the copy engine's tiled mode:
// a stage is GS_BK / 64 boxes of [64 rows][64 k-values] that the 128-byte swizzle lays down in exactly
// the order above (zeros beyond N and K), so that a model needs no second copy of its weights.
template <int MT, typename TO, bool BOXES>
__global__ void __launch_bounds__(GS_THREADS) linear_skinny_tiled_kernel(const bf16* __restrict__ x,
                                                                         const bf16* __restrict__ w_tiled, TO* __restrict__ y,
                                                                         float* __restrict__ partial, int M, int N, int K,
                                                                         int slices, int per_tile, int32_t* __restrict__ status,
                                                                         const __grid_constant__ CUtensorMap w_map) {
    constexpr int GS_STAGES = GS_STAGES_FOR(MT), GS_BK = GS_BK_FOR(MT), GS_XSTAGES = GS_XSTAGES_FOR(MT);
    constexpr unsigned W_BYTES = GS_ROWS * GS_BK * sizeof(bf16);
    const long long halves_per_tile = static_cast<long long>((K + 255) / 256) * (256 / GS_BK);   // stages of GS_BK in a tile's row of blocks
    extern __shared__ __align__(1024) unsigned char smem_raw[];          // the swizzle's pattern repeats every 1024 bytes
    bf16* w_s = reinterpret_cast<bf16*>(smem_raw);                       // [STAGES][64][BK], as stored in w_tiled
    bf16* x_s = w_s + GS_STAGES * GS_ROWS * GS_BK;                       // [XSTAGES][MT][BK]
    __shared__ __align__(8) unsigned long long full[GS_STAGES];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nk = (K + GS_BK - 1) / GS_BK, tiles = (N + GS_ROWS - 1) / GS_ROWS;
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
    constexpr int CPR = GS_BK / 8;

    auto load_w = [&](int i) {                                           // one thread, one copy: block (tile, k-step) = item
        if (tid == 0) {
            unsigned long long* bar = &full[i % GS_STAGES];
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // the stage was read through the generic proxy
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(gs_smem(bar)), "r"(W_BYTES) : "memory");
            if constexpr (BOXES) {
                const int n0 = static_cast<int>((begin + i) / nk) * GS_ROWS, k0 = static_cast<int>((begin + i) % nk) * GS_BK;
#pragma unroll
                for (int b = 0; b < GS_BK / 64; ++b)
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
                                     "r"(gs_smem(w_s + (i % GS_STAGES) * GS_ROWS * GS_BK + b * (GS_ROWS * 64))), "l"(&w_map),
                                 "r"(k0 + b * 64), "r"(n0), "r"(gs_smem(bar)) : "memory");
            } else {
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::
                                 "r"(gs_smem(w_s + (i % GS_STAGES) * GS_ROWS * GS_BK)),
                             "l"(w_tiled + (static_cast<size_t>((begin + i) / nk) * halves_per_tile + (begin + i) % nk) * (GS_ROWS * GS_BK)),
                             "r"(W_BYTES), "r"(gs_smem(bar)) : "memory");
            }
        }
    };
    auto load_x = [&](int i) {
        const int k0 = static_cast<int>((begin + i) % nk) * GS_BK;
        bf16* xs = x_s + (i % GS_XSTAGES) * MT * GS_BK;
#pragma unroll
        for (int j = 0; j < MT * CPR / GS_THREADS; ++j) {
            const int c = tid + GS_THREADS * j, row = c / CPR, ch = c % CPR;
            const bool valid = (row < M) && (k0 + ch * 8 < K);
            gs_cp_async16(gs_at<GS_BK>(xs, row, ch), x + (valid ? static_cast<size_t>(row) * K + k0 + ch * 8 : 0), valid);
        }
    };

    pdl_invite();
    if (tid == 0) {
        for (int s = 0; s < GS_STAGES; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(gs_smem(&full[s])));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
#pragma unroll
        for (int s = 0; s < GS_STAGES - 1; ++s)                           // the weights do not depend on the kernel before this one
            if (s < count) load_w(s);
    }
    pdl_wait();
#pragma unroll
    for (int s = 0; s < GS_XSTAGES - 1; ++s) {
        if (s < count) load_x(s);
        gs_commit();
    }
    __syncthreads();                                                     // the barriers exist for everyone
    // Two sums per output, over the even and the odd k-steps: consecutive products then never wait
    // for one another's accumulator.  They are added when a tile's k-range ends.
    float acc[MT / 8][4], acc2[MT / 8][4];
#pragma unroll
    for (int j = 0; j < MT / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = acc2[j][e] = 0.0f;
    int tile = static_cast<int>(begin / nk), kt = static_cast<int>(begin % nk);
    for (int i = 0; i < count; ++i) {
        gs_wait<GS_XSTAGES - 2>();                                       // this thread's copies of the tokens' rows
        {
            int n = 0;
            while (!gs_try_wait(&full[i % GS_STAGES], (i / GS_STAGES) & 1)) {
                if (++n > GS_TILED_WAIT_LIMIT) {
                    if (atomicCAS(status, 0, 8) == 0) status[1] = blockIdx.x;
                    break;
                }
            }
        }
        __syncthreads();                                                 // everyone's rows are there; stage i-1 is no longer read
        if (i + GS_STAGES - 1 < count) load_w(i + GS_STAGES - 1);
        if (i + GS_XSTAGES - 1 < count) load_x(i + GS_XSTAGES - 1);
        gs_commit();
        bf16* ws = w_s + (i % GS_STAGES) * GS_ROWS * GS_BK;
        bf16* xs = x_s + (i % GS_XSTAGES) * MT * GS_BK;
#pragma unroll
        for (int kp = 0; kp < GS_BK / 32; ++kp) {
            unsigned a0[4], a1[4];
            gs_ldmatrix_x4(a0, gs_at_tiled(ws, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, kp * 4 + (lane >> 4)));
            gs_ldmatrix_x4(a1, gs_at_tiled(ws, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, kp * 4 + 2 + (lane >> 4)));
            unsigned b[MT / 8][4];                                       // tokens 8j..8j+7, two k-steps
#pragma unroll
            for (int j = 0; j < MT / 8; ++j) gs_ldmatrix_x4(b[j], gs_at<GS_BK>(xs, j * 8 + (lane & 7), kp * 4 + (lane >> 3)));
#pragma unroll
            for (int j = 0; j < MT / 8; ++j) gs_mma(acc[j], a0, b[j][0], b[j][1]);
#pragma unroll
            for (int j = 0; j < MT / 8; ++j) gs_mma(acc2[j], a1, b[j][2], b[j][3]);
        }
        const bool tile_done = kt == nk - 1;
        if (tile_done || i == count - 1) {
            const int f0 = tile * GS_ROWS + warp * 16 + (lane >> 2), t0 = (lane & 3) * 2;
            const int slice = per_tile ? static_cast<int>(blockIdx.x % per_tile)
                                       : static_cast<int>(blockIdx.x - gs_cta_of(static_cast<long long>(tile) * nk, total, ctas));
#pragma unroll
            for (int j = 0; j < MT / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int f = f0 + (e >> 1) * 8, tok = j * 8 + t0 + (e & 1);
                    const float sum = acc[j][e] + acc2[j][e];
                    if (f < N && tok < M) {
                        if (slices == 1) {
                            y[static_cast<size_t>(tok) * N + f] = from_f32<TO>(sum);
                        } else {
                            partial[(static_cast<size_t>(slice) * M + tok) * N + f] = sum;
                            if (tile_done && !per_tile)
                                for (int z = slice + 1; z < slices; ++z) partial[(static_cast<size_t>(z) * M + tok) * N + f] = 0.0f;
                        }
                    }
                    acc[j][e] = acc2[j][e] = 0.0f;
                }
            }
        }
        if (tile_done) { kt = 0; ++tile; } else ++kt;
    }
    gs_wait<0>();
}

// y[tok, f] = sum over splits of partial[split, tok, f], in split order.
template <typename TO>
__global__ void linear_skinny_sum_kernel(const float* __restrict__ partial, TO* __restrict__ y, long long mn, int splits) {
    pdl_begin();
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= mn) return;
    float v = 0.0f;
    for (int s = 0; s < splits; ++s) v += partial[s * mn + i];
    y[i] = from_f32<TO>(v);
}

extern "C" int llm_linear_skinny_supported(int M, int N, int K) {
    return M >= 1 && M <= 32 && N >= 1 && K >= 8 && (K % 8) == 0;
}

static int g_skinny_slots = 0;     // CTAs the current device holds at once (two per SM), found at the first call

static bool skinny_device() {
    if (g_skinny_slots) return true;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        return false;
    g_skinny_slots = sms * 2;
    return true;
}

// The grid for a product and the number of partial-sum slices it leaves (1 = none).  When whole
// CTAs per feature tile fill at least 85 % of the GPU's CTA slots, each tile's k-values are shared
// evenly by `per_tile` CTAs (fewest slices); otherwise (more tiles than slots, or a poor fit) the
// items are cut into one even run per slot (per_tile = 0).
static void skinny_plan(int N, int K, int bk, int* ctas, int* slices, int* per_tile) {
    const long long tiles = (N + GS_ROWS - 1) / GS_ROWS, nk = (K + bk - 1) / bk, total = tiles * nk;
    long long best = 0;
    for (long long s = 1; s <= 16 && s <= (nk >= 4 ? nk / 4 : 1); ++s)   // at least four items per CTA
        if (tiles * s <= g_skinny_slots) best = s;
    if (best && tiles * best * 100 >= 85LL * g_skinny_slots) {
        *ctas = static_cast<int>(tiles * best);
        *slices = *per_tile = static_cast<int>(best);
        return;
    }
    // A small product (fewer items than would give every slot four) is bound by the latency of a CTA's
    // chain of stages, not by bytes: two items per CTA, so more CTAs and shorter chains (a decode step of
    // the 0.6B shape at batch 8: 0.83 ms instead of 0.94; one item per CTA: 0.90, its partial sums cost more).
    long long g = total / 2;
    if (g < 1) g = 1;
    if (g > g_skinny_slots) g = g_skinny_slots;
    int s = 1;
    if (!(total % g == 0 && (total / g) % nk == 0)) {                    // some tile is cut
        s = 0;
        for (long long t = 0; t < tiles; ++t) {                          // the most CTAs that meet in one tile
            const int n = static_cast<int>(gs_cta_of((t + 1) * nk - 1, total, g) - gs_cta_of(t * nk, total, g)) + 1;
            if (n > s) s = n;
        }
    }
    *ctas = static_cast<int>(g);
    *slices = s;
    *per_tile = 0;
}

// Whether a product is small in the sense above: fewer items than would give every CTA slot four.  Such
// products take this kernel up to 32 tokens: measured alone its 32-token tile is no faster than the
// library's kernels (6.9 against 5.4 us on 4,096 x 1,024), but inside a step it starts fetching weights
// while the kernel before it drains and hands its k-splits to the kernel after it (a decode step of the
// 0.6B shape at batch 32: 1.27 ms against 1.48).  On large products the 32-token tile loses (45.6 against
// 35.7 us on 24,576 x 4,096) and the library stays.
extern "C" int llm_linear_skinny_small(int N, int K) {
    if (!skinny_device()) return 0;
    int ctas, slices, per_tile;
    skinny_plan(N, K, GS_BK_FOR(8), &ctas, &slices, &per_tile);
    const long long tiles = (N + GS_ROWS - 1) / GS_ROWS, nk = (K + GS_BK_FOR(8) - 1) / GS_BK_FOR(8);
    return per_tile == 0 && tiles * nk < 4LL * g_skinny_slots ? 1 : 0;   // the plan took the two-items rule
}

// Floats of scratch a call needs for its partial sums.
extern "C" long long llm_linear_skinny_scratch_floats(int M, int N, int K) {
    if (!skinny_device()) return 0;
    int ctas, slices, per_tile;
    skinny_plan(N, K, GS_BK_FOR(M <= 8 ? 8 : 16), &ctas, &slices, &per_tile);
    return slices > 1 ? static_cast<long long>(slices) * M * N : 0;
}

// The number of partial-sum slices a product of these sizes leaves on the current device.
extern "C" int llm_linear_skinny_splits(int M, int N, int K) {
    if (!skinny_device()) return 1;
    int ctas, slices, per_tile;
    skinny_plan(N, K, GS_BK_FOR(M <= 8 ? 8 : 16), &ctas, &slices, &per_tile);
    return slices;
}

// The tiled form of llm_linear_skinny for M <= 8: w_tiled is what llm_linear_skinny_tiled_elems
// describes (blocks of 64 x 256 in the kernel's shared-memory order).  status: int32 [2].
extern "C" long long llm_linear_skinny_tiled_elems(int N, int K) {
    return static_cast<long long>((N + GS_ROWS - 1) / GS_ROWS) * ((K + GS_TILED_BK - 1) / GS_TILED_BK) * GS_ROWS * GS_TILED_BK;
}

// ---- tensor maps of plain weights: [N, K] bfloat16, boxes of 64 k-values x 64 rows, 128-byte swizzle ----
typedef CUresult (*GsEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static GsEncodeFn g_gs_encode = nullptr;
static int g_gs_encode_state = 0;
struct GsMapEntry { int n, k; CUtensorMap map; };
static std::unordered_map<const void*, GsMapEntry> g_gs_maps;     // by the weights' address

static const CUtensorMap* gs_weight_map(const void* w, int N, int K) {
    if (g_gs_encode_state == 0) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess && fn != nullptr) {
            g_gs_encode = reinterpret_cast<GsEncodeFn>(fn);
            g_gs_encode_state = 1;
        } else {
            (void)cudaGetLastError();
            g_gs_encode_state = -1;
        }
    }
    if (g_gs_encode_state < 0) return nullptr;
    auto it = g_gs_maps.find(w);
    if (it != g_gs_maps.end() && it->second.n == N && it->second.k == K) return &it->second.map;
    GsMapEntry e;
    e.n = N;
    e.k = K;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(N)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * sizeof(bf16)};
    const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(GS_ROWS)};
    const cuuint32_t estr[2] = {1u, 1u};
    if (g_gs_encode(&e.map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return nullptr;
    g_gs_maps[w] = e;
    return &g_gs_maps[w].map;
}

template <int MT, typename TO, bool BOXES>
static int launch_skinny_tiled(const bf16* x, const bf16* wt, void* y, float* scratch, long long scratch_floats, int M, int N,
                               int K, int keep_partials, int32_t* status, cudaStream_t s) {
    if (!skinny_device()) return LLM_REFUSED_SIZE;
    CUtensorMap map = {};
    if (BOXES) {
        const CUtensorMap* m = gs_weight_map(wt, N, K);
        if (m == nullptr) return LLM_REFUSED_ALIGN;                      // the driver refused the weights' address or strides
        map = *m;
    }
    const size_t smem = (static_cast<size_t>(GS_STAGES_FOR(MT)) * GS_ROWS + GS_XSTAGES_FOR(MT) * MT) * GS_BK_FOR(MT) * sizeof(bf16);
    auto kern = linear_skinny_tiled_kernel<MT, TO, BOXES>;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    int ctas, slices, per_tile;
    skinny_plan(N, K, GS_BK_FOR(MT), &ctas, &slices, &per_tile);
    if (slices > 1 && (scratch == nullptr || scratch_floats < static_cast<long long>(slices) * M * N)) return LLM_REFUSED_SIZE;
    launch_pdl(kern, dim3(ctas), dim3(GS_THREADS), smem, s, x, wt, static_cast<TO*>(y), scratch, M, N, K, slices, per_tile, status, map);
    int rc = launch_status();
    if (rc != LLM_OK || slices == 1 || keep_partials) return rc;
    const long long mn = static_cast<long long>(M) * N;
    launch_pdl((linear_skinny_sum_kernel<TO>), dim3(static_cast<unsigned>((mn + 255) / 256)), dim3(256), 0, s, scratch, static_cast<TO*>(y), mn, slices);
    return launch_status();
}

// The same product over the PLAIN weights [N, K], fetched box by box (one copy of the weights serves
// every kernel).  w must be 16-byte aligned and K a multiple of 8 (the copy engine's rule for strides).
extern "C" int llm_linear_skinny_boxes(const void* x, const void* w, void* y, int out_dtype, float* scratch,
                                       long long scratch_floats, int M, int N, int K, int keep_partials, int32_t* status,
                                       uintptr_t stream) {
    if (!llm_linear_skinny_supported(M, N, K)) return LLM_REFUSED_SIZE;
    if (!aligned16(x) || !aligned16(w) || status == nullptr) return LLM_REFUSED_ALIGN;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bf16* xp = static_cast<const bf16*>(x);
    const bf16* wp = static_cast<const bf16*>(w);
    if (out_dtype != LLM_DT_F32 && out_dtype != LLM_DT_BF16) return LLM_REFUSED_DTYPE;
    if (M <= 8)
        return out_dtype == LLM_DT_F32 ? launch_skinny_tiled<8, float, true>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, status, s)
                                       : launch_skinny_tiled<8, bf16, true>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, status, s);
    if (M <= 16)
        return out_dtype == LLM_DT_F32 ? launch_skinny_tiled<16, float, true>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, status, s)
                                       : launch_skinny_tiled<16, bf16, true>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, status, s);
    return out_dtype == LLM_DT_F32 ? launch_skinny_tiled<32, float, true>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, status, s)
                                   : launch_skinny_tiled<32, bf16, true>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, status, s);
}

extern "C" int llm_linear_skinny_tiled(const void* x, const void* w_tiled, void* y, int out_dtype, float* scratch,
                                       long long scratch_floats, int M, int N, int K, int keep_partials, int32_t* status,
                                       uintptr_t stream) {
    if (!llm_linear_skinny_supported(M, N, K)) return LLM_REFUSED_SIZE;
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(w_tiled) & 127u) != 0 || status == nullptr) return LLM_REFUSED_ALIGN;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bf16* xp = static_cast<const bf16*>(x);
    const bf16* wp = static_cast<const bf16*>(w_tiled);
    if (out_dtype != LLM_DT_F32 && out_dtype != LLM_DT_BF16) return LLM_REFUSED_DTYPE;
    if (M <= 8)
        return out_dtype == LLM_DT_F32 ? launch_skinny_tiled<8, float, false>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, status, s)
                                       : launch_skinny_tiled<8, bf16, false>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, status, s);
    if (M <= 16)
        return out_dtype == LLM_DT_F32 ? launch_skinny_tiled<16, float, false>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, status, s)
                                       : launch_skinny_tiled<16, bf16, false>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, status, s);
    return out_dtype == LLM_DT_F32 ? launch_skinny_tiled<32, float, false>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, status, s)
                                   : launch_skinny_tiled<32, bf16, false>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, status, s);
}

