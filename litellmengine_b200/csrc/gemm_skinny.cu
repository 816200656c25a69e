// y[M, N] = x[M, K] . w[N, K]^T for a handful of rows (decode steps): a weight-streaming kernel.
//
// With few rows the product is bound by reading w once; the library's kernels for these shapes
// reach 40-60 % of the memory bandwidth when N is small (few thread blocks).  Here every CTA owns
// 16 output features (16 rows of w, each contiguous along K) and streams them through shared
// memory in stages of 512 k-values with cp.async (4 stages, so ~48 KB per CTA are in flight),
// while the rows of x for the same k-range come along (they are re-read from L2 by every CTA).
// The product runs on the tensor cores with the roles swapped: w is the 16-row A operand of
// mma.sync m16n8k16 and the tokens are the 8 columns of B, so 8 tokens use a full instruction and
// 16 tokens two.  The four warps split each stage along k and add their partial sums through
// shared memory at the end; accumulation is float32; the result is written as float32 or
// bfloat16.  The reference calls cublasSgemm for every product (src/layers/linear.cu:169-215).
#include "common.cuh"

#define GS_ROWS 16          // output features per CTA
#define GS_BK 512           // k-values per stage
#define GS_STAGES 4
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
// 16-byte chunk `chunk` of row `row` in a [rows][GS_BK] bfloat16 stage, XOR-swizzled.
__device__ __forceinline__ bf16* gs_at(bf16* base, int row, int chunk) {
    return base + row * GS_BK + ((chunk ^ (row & 7)) << 3);
}

// MT: token tile (8 or 16).
template <int MT, typename TO>
__global__ void __launch_bounds__(GS_THREADS) linear_skinny_kernel(const bf16* __restrict__ x,
                                                                   const bf16* __restrict__ w, TO* __restrict__ y,
                                                                   int M, int N, int K) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* w_s = reinterpret_cast<bf16*>(smem_raw);                       // [STAGES][16][BK]
    bf16* x_s = w_s + GS_STAGES * GS_ROWS * GS_BK;                       // [STAGES][MT][BK]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * GS_ROWS;
    const int nk = (K + GS_BK - 1) / GS_BK;
    constexpr int CPR = GS_BK / 8;                                       // chunks per row of a stage

    auto load_stage = [&](int kt, int buf) {
        const int k0 = kt * GS_BK;
        bf16* ws = w_s + buf * GS_ROWS * GS_BK;
        bf16* xs = x_s + buf * MT * GS_BK;
#pragma unroll
        for (int i = 0; i < GS_ROWS * CPR / GS_THREADS; ++i) {
            const int c = tid + GS_THREADS * i, row = c / CPR, ch = c % CPR;
            const bool valid = (n0 + row < N) && (k0 + ch * 8 < K);
            gs_cp_async16(gs_at(ws, row, ch), w + (valid ? static_cast<size_t>(n0 + row) * K + k0 + ch * 8 : 0), valid);
        }
#pragma unroll
        for (int i = 0; i < MT * CPR / GS_THREADS; ++i) {
            const int c = tid + GS_THREADS * i, row = c / CPR, ch = c % CPR;
            const bool valid = (row < M) && (k0 + ch * 8 < K);
            gs_cp_async16(gs_at(xs, row, ch), x + (valid ? static_cast<size_t>(row) * K + k0 + ch * 8 : 0), valid);
        }
    };

#pragma unroll
    for (int s = 0; s < GS_STAGES - 1; ++s) {
        if (s < nk) load_stage(s, s);
        gs_commit();
    }
    float acc[MT / 8][4];
#pragma unroll
    for (int j = 0; j < MT / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

    for (int kt = 0; kt < nk; ++kt) {
        gs_wait<GS_STAGES - 2>();
        __syncthreads();
        if (kt + GS_STAGES - 1 < nk) load_stage(kt + GS_STAGES - 1, (kt + GS_STAGES - 1) % GS_STAGES);
        gs_commit();
        bf16* ws = w_s + (kt % GS_STAGES) * GS_ROWS * GS_BK;
        bf16* xs = x_s + (kt % GS_STAGES) * MT * GS_BK;
        // this warp's quarter of the stage: k-steps [warp*8, warp*8+8)
#pragma unroll
        for (int kp = 0; kp < GS_BK / 16 / 4 / 2; ++kp) {               // pairs of k-steps
            const int ks = warp * (GS_BK / 16 / 4) + kp * 2;
            unsigned a0[4], a1[4];
            gs_ldmatrix_x4(a0, gs_at(ws, (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
            gs_ldmatrix_x4(a1, gs_at(ws, (lane & 7) + ((lane >> 3) & 1) * 8, (ks + 1) * 2 + (lane >> 4)));
#pragma unroll
            for (int j = 0; j < MT / 8; ++j) {
                unsigned b[4];                                           // tokens 8j..8j+7, two k-steps
                gs_ldmatrix_x4(b, gs_at(xs, j * 8 + (lane & 7), ks * 2 + (lane >> 3)));
                gs_mma(acc[j], a0, b[0], b[1]);
                gs_mma(acc[j], a1, b[2], b[3]);
            }
        }
    }
    gs_wait<0>();
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem_raw);                     // [4 warps][16 features][MT tokens]
    {
        const int f0 = lane >> 2, t0 = (lane & 3) * 2;
#pragma unroll
        for (int j = 0; j < MT / 8; ++j) {
            float* r = red + (warp * GS_ROWS + f0) * MT + j * 8 + t0;
            r[0] = acc[j][0]; r[1] = acc[j][1];
            r[8 * MT] = acc[j][2]; r[8 * MT + 1] = acc[j][3];
        }
    }
    __syncthreads();
    for (int i = tid; i < GS_ROWS * MT; i += GS_THREADS) {
        const int tok = i / GS_ROWS, f = i - tok * GS_ROWS;              // consecutive threads: consecutive features
        if (tok < M && n0 + f < N) {
            const float v = red[(0 * GS_ROWS + f) * MT + tok] + red[(1 * GS_ROWS + f) * MT + tok] +
                            red[(2 * GS_ROWS + f) * MT + tok] + red[(3 * GS_ROWS + f) * MT + tok];
            y[static_cast<size_t>(tok) * N + n0 + f] = from_f32<TO>(v);
        }
    }
}

extern "C" int llm_linear_skinny_supported(int M, int N, int K) {
    return M >= 1 && M <= 16 && N >= 1 && K >= 8 && (K % 8) == 0;
}

template <int MT, typename TO>
static int launch_skinny(const bf16* x, const bf16* w, void* y, int M, int N, int K, cudaStream_t s) {
    const size_t smem = static_cast<size_t>(GS_STAGES) * (GS_ROWS + MT) * GS_BK * sizeof(bf16);
    auto kern = linear_skinny_kernel<MT, TO>;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    kern<<<(N + GS_ROWS - 1) / GS_ROWS, GS_THREADS, smem, s>>>(x, w, static_cast<TO*>(y), M, N, K);
    return launch_status();
}

// x: bfloat16 [M, K]; w: bfloat16 [N, K]; y: [M, N] float32 (out_dtype 0) or bfloat16 (1).
extern "C" int llm_linear_skinny(const void* x, const void* w, void* y, int out_dtype, int M, int N, int K,
                                 uintptr_t stream) {
    if (!llm_linear_skinny_supported(M, N, K)) return LLM_REFUSED_SIZE;
    if (!aligned16(x) || !aligned16(w)) return LLM_REFUSED_ALIGN;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bf16* xp = static_cast<const bf16*>(x);
    const bf16* wp = static_cast<const bf16*>(w);
    if (M <= 8) {
        if (out_dtype == LLM_DT_F32) return launch_skinny<8, float>(xp, wp, y, M, N, K, s);
        if (out_dtype == LLM_DT_BF16) return launch_skinny<8, bf16>(xp, wp, y, M, N, K, s);
    } else {
        if (out_dtype == LLM_DT_F32) return launch_skinny<16, float>(xp, wp, y, M, N, K, s);
        if (out_dtype == LLM_DT_BF16) return launch_skinny<16, bf16>(xp, wp, y, M, N, K, s);
    }
    return LLM_REFUSED_DTYPE;
}
