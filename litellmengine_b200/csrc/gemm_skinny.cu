// y[M, N] = x[M, K] . w[N, K]^T for a handful of rows (decode steps): a weight-streaming kernel.
//
// With few rows the product is bound by reading w once.  The library's kernels for these shapes
// reach 40-60 % of the memory bandwidth when N is small (few thread blocks, little in flight per
// SM).  Here the work is cut into units of (16 output features) x (512 k-values): 16 KB of w each.
// A persistent grid of two CTAs per SM takes equal, contiguous runs of units (a run may start
// and end in the middle of a feature tile) and streams them through six shared-memory stages
// with cp.async, so about 160 KB per SM are in flight the whole time, whatever N is.
// The product runs on the tensor cores with the roles swapped: w is the 16-row A operand of
// mma.sync m16n8k16 and the tokens are the 8 columns of B (8 tokens use a full instruction,
// 16 tokens two).  The tokens' fragments come straight from global memory (x is small and
// lives in L2), prefetched one unit ahead.  The four warps split each unit along k and add
// their partial sums through shared memory when a tile ends.  A tile that one CTA covers
// entirely is written at once; the pieces of a tile shared by several CTAs go to scratch and a
// second small kernel adds them in a fixed order (no atomics: the result does not depend on
// timing).  Accumulation is float32; the result is float32 or bfloat16.
// The reference calls cublasSgemm for every product (src/layers/linear.cu:169-215).
#include "common.cuh"

#define GS_ROWS 16          // output features per tile
#define GS_BK 512           // k-values per unit
#define GS_STAGES 6
#define GS_THREADS 128
#define GS_KSTEPS (GS_BK / 16 / 4)   // k-steps of 16 per warp per unit

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
// 16-byte chunk `chunk` of row `row` in a [16][GS_BK] bfloat16 stage, XOR-swizzled.
__device__ __forceinline__ bf16* gs_at(bf16* base, int row, int chunk) {
    return base + row * GS_BK + ((chunk ^ (row & 7)) << 3);
}

// First unit of CTA c when `units` units are dealt to `ctas` CTAs in equal contiguous runs.
__host__ __device__ __forceinline__ long long gs_run_start(long long c, long long units, long long ctas) {
    return c * units / ctas;
}
__device__ __forceinline__ int gs_cta_of_unit(long long u, long long units, long long ctas) {
    long long c = u * ctas / units;
    while (c + 1 < ctas && gs_run_start(c + 1, units, ctas) <= u) ++c;
    while (c > 0 && gs_run_start(c, units, ctas) > u) --c;
    return static_cast<int>(c);
}

// MT: token tile (8 or 16).
template <int MT, typename TO>
__global__ void __launch_bounds__(GS_THREADS) linear_skinny_kernel(const bf16* __restrict__ x,
                                                                   const bf16* __restrict__ w, TO* __restrict__ y,
                                                                   float* __restrict__ partial, int M, int N, int K) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* w_s = reinterpret_cast<bf16*>(smem_raw);                       // [STAGES][16][BK]
    __shared__ float red[4][GS_ROWS][MT];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nk = (K + GS_BK - 1) / GS_BK;
    const long long tiles = (N + GS_ROWS - 1) / GS_ROWS;
    const long long units = tiles * nk;
    const long long u_begin = gs_run_start(blockIdx.x, units, gridDim.x);
    const long long u_end = gs_run_start(blockIdx.x + 1, units, gridDim.x);
    const int my_units = static_cast<int>(u_end - u_begin);
    constexpr int CPR = GS_BK / 8;                                       // chunks per row of a stage

    auto load_w = [&](int i) {                                           // unit i of this CTA's run into stage i % STAGES
        const long long u = u_begin + i;
        const int n0 = static_cast<int>(u / nk) * GS_ROWS, k0 = static_cast<int>(u % nk) * GS_BK;
        bf16* ws = w_s + (i % GS_STAGES) * GS_ROWS * GS_BK;
#pragma unroll
        for (int j = 0; j < GS_ROWS * CPR / GS_THREADS; ++j) {
            const int c = tid + GS_THREADS * j, row = c / CPR, ch = c % CPR;
            const bool valid = (n0 + row < N) && (k0 + ch * 8 < K);
            gs_cp_async16(gs_at(ws, row, ch), w + (valid ? static_cast<size_t>(n0 + row) * K + k0 + ch * 8 : 0), valid);
        }
    };
    // This thread's share of the tokens' B fragments for one unit: token j*8 + lane/4,
    // k = k0 + (warp*KSTEPS + ks)*16 + (lane%4)*2 (+8).
    auto load_x = [&](int i, unsigned (&xb)[MT / 8][GS_KSTEPS][2]) {
        const int k0 = static_cast<int>((u_begin + i) % nk) * GS_BK + warp * GS_KSTEPS * 16 + (lane & 3) * 2;
#pragma unroll
        for (int j = 0; j < MT / 8; ++j) {
            const int tok = j * 8 + (lane >> 2);
            const bf16* xr = x + static_cast<size_t>(tok) * K;
#pragma unroll
            for (int ks = 0; ks < GS_KSTEPS; ++ks) {
                const int k = k0 + ks * 16;
                xb[j][ks][0] = (tok < M && k < K) ? __ldg(reinterpret_cast<const unsigned*>(xr + k)) : 0u;
                xb[j][ks][1] = (tok < M && k + 8 < K) ? __ldg(reinterpret_cast<const unsigned*>(xr + k + 8)) : 0u;
            }
        }
    };

#pragma unroll
    for (int s = 0; s < GS_STAGES - 1; ++s) {
        if (s < my_units) load_w(s);
        gs_commit();
    }
    unsigned xcur[MT / 8][GS_KSTEPS][2], xnext[MT / 8][GS_KSTEPS][2];
    if (my_units > 0) load_x(0, xcur);
    float acc[MT / 8][4];
#pragma unroll
    for (int j = 0; j < MT / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
    const long long first_tile = my_units > 0 ? u_begin / nk : 0;

    for (int i = 0; i < my_units; ++i) {
        gs_wait<GS_STAGES - 2>();
        __syncthreads();
        if (i + GS_STAGES - 1 < my_units) load_w(i + GS_STAGES - 1);
        gs_commit();
        if (i + 1 < my_units) load_x(i + 1, xnext);
        bf16* ws = w_s + (i % GS_STAGES) * GS_ROWS * GS_BK;
#pragma unroll
        for (int ks = 0; ks < GS_KSTEPS; ++ks) {
            unsigned a[4];
            gs_ldmatrix_x4(a, gs_at(ws, (lane & 7) + ((lane >> 3) & 1) * 8, (warp * GS_KSTEPS + ks) * 2 + (lane >> 4)));
#pragma unroll
            for (int j = 0; j < MT / 8; ++j) gs_mma(acc[j], a, xcur[j][ks][0], xcur[j][ks][1]);
        }
#pragma unroll
        for (int j = 0; j < MT / 8; ++j)
#pragma unroll
            for (int ks = 0; ks < GS_KSTEPS; ++ks) {
                xcur[j][ks][0] = xnext[j][ks][0];
                xcur[j][ks][1] = xnext[j][ks][1];
            }
        const long long u = u_begin + i;
        const int kt = static_cast<int>(u % nk);
        if (kt == nk - 1 || i == my_units - 1) {                         // this CTA's share of the tile ends here
            const long long tile = u / nk;
            const int f0 = lane >> 2, t0 = (lane & 3) * 2;
#pragma unroll
            for (int j = 0; j < MT / 8; ++j) {
                red[warp][f0][j * 8 + t0] = acc[j][0];
                red[warp][f0][j * 8 + t0 + 1] = acc[j][1];
                red[warp][f0 + 8][j * 8 + t0] = acc[j][2];
                red[warp][f0 + 8][j * 8 + t0 + 1] = acc[j][3];
                acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
            }
            __syncthreads();
            // whole tile ours? (its first unit is in our run and so is its last)
            const bool whole = (tile * nk >= u_begin) && (kt == nk - 1);
            const int n0 = static_cast<int>(tile) * GS_ROWS;
            for (int e = tid; e < GS_ROWS * MT; e += GS_THREADS) {
                const int tok = e / GS_ROWS, f = e - tok * GS_ROWS;      // consecutive threads: consecutive features
                const float v = red[0][f][tok] + red[1][f][tok] + red[2][f][tok] + red[3][f][tok];
                if (whole) {
                    if (tok < M && n0 + f < N) y[static_cast<size_t>(tok) * N + n0 + f] = from_f32<TO>(v);
                } else {
                    const int slot = (tile == first_tile) ? 0 : 1;       // a run cuts at most its first and last tile
                    partial[(static_cast<size_t>(blockIdx.x) * 2 + slot) * GS_ROWS * MT + e] = v;
                }
            }
            __syncthreads();
        }
    }
    gs_wait<0>();
}

// One block per tile: if several CTAs of the main kernel shared the tile, add their pieces in
// CTA order and write the result.
template <int MT, typename TO>
__global__ void linear_skinny_fixup_kernel(const float* __restrict__ partial, TO* __restrict__ y, int M, int N, int K,
                                           int ctas) {
    const int nk = (K + GS_BK - 1) / GS_BK;
    const long long tiles = (N + GS_ROWS - 1) / GS_ROWS, units = tiles * nk;
    const long long tile = blockIdx.x;
    const int c_first = gs_cta_of_unit(tile * nk, units, ctas);
    const int c_last = gs_cta_of_unit(tile * nk + nk - 1, units, ctas);
    if (c_first == c_last) return;                                       // written whole by the main kernel
    const int n0 = static_cast<int>(tile) * GS_ROWS;
    for (int e = threadIdx.x; e < GS_ROWS * MT; e += blockDim.x) {
        const int tok = e / GS_ROWS, f = e - tok * GS_ROWS;
        float v = 0.0f;
        for (int c = c_first; c <= c_last; ++c) {
            const long long c_first_tile = gs_run_start(c, units, ctas) / nk;
            const int slot = (tile == c_first_tile) ? 0 : 1;
            v += partial[(static_cast<size_t>(c) * 2 + slot) * GS_ROWS * MT + e];
        }
        if (tok < M && n0 + f < N) y[static_cast<size_t>(tok) * N + n0 + f] = from_f32<TO>(v);
    }
}

extern "C" int llm_linear_skinny_supported(int M, int N, int K) {
    return M >= 1 && M <= 16 && N >= 1 && K >= 8 && (K % 8) == 0;
}

static int g_skinny_ctas = 0;      // two per SM of the current device, found at the first call

// Floats of scratch a call may need (pieces of tiles shared between CTAs).
extern "C" long long llm_linear_skinny_scratch_floats() { return 2LL * 1024 * GS_ROWS * 16; }

template <int MT, typename TO>
static int launch_skinny(const bf16* x, const bf16* w, void* y, float* scratch, int M, int N, int K, cudaStream_t s) {
    if (g_skinny_ctas == 0) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            return LLM_REFUSED_SIZE;
        g_skinny_ctas = sms * 2 > 1024 ? 1024 : sms * 2;
    }
    const size_t smem = static_cast<size_t>(GS_STAGES) * GS_ROWS * GS_BK * sizeof(bf16);
    auto kern = linear_skinny_kernel<MT, TO>;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    const long long tiles = (N + GS_ROWS - 1) / GS_ROWS, nk = (K + GS_BK - 1) / GS_BK, units = tiles * nk;
    const int ctas = static_cast<int>(units < g_skinny_ctas ? units : g_skinny_ctas);
    kern<<<ctas, GS_THREADS, smem, s>>>(x, w, static_cast<TO*>(y), scratch, M, N, K);
    int rc = launch_status();
    if (rc != LLM_OK) return rc;
    linear_skinny_fixup_kernel<MT, TO><<<static_cast<unsigned>(tiles), 128, 0, s>>>(scratch, static_cast<TO*>(y), M, N, K, ctas);
    return launch_status();
}

// x: bfloat16 [M, K]; w: bfloat16 [N, K]; y: [M, N] float32 (out_dtype 0) or bfloat16 (1);
// scratch: float32, llm_linear_skinny_scratch_floats() long.
extern "C" int llm_linear_skinny(const void* x, const void* w, void* y, int out_dtype, float* scratch, int M, int N,
                                 int K, uintptr_t stream) {
    if (!llm_linear_skinny_supported(M, N, K)) return LLM_REFUSED_SIZE;
    if (!aligned16(x) || !aligned16(w) || scratch == nullptr) return LLM_REFUSED_ALIGN;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bf16* xp = static_cast<const bf16*>(x);
    const bf16* wp = static_cast<const bf16*>(w);
    if (M <= 8) {
        if (out_dtype == LLM_DT_F32) return launch_skinny<8, float>(xp, wp, y, scratch, M, N, K, s);
        if (out_dtype == LLM_DT_BF16) return launch_skinny<8, bf16>(xp, wp, y, scratch, M, N, K, s);
    } else {
        if (out_dtype == LLM_DT_F32) return launch_skinny<16, float>(xp, wp, y, scratch, M, N, K, s);
        if (out_dtype == LLM_DT_BF16) return launch_skinny<16, bf16>(xp, wp, y, scratch, M, N, K, s);
    }
    return LLM_REFUSED_DTYPE;
}
