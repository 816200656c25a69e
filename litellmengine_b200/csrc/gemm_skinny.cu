// y[M, N] = x[M, K] . w[N, K]^T for a handful of rows (decode steps): a weight-streaming kernel.
//
// With few rows the product is bound by reading w once, and what decides the speed is how many
// bytes of w each SM keeps in flight.  The library's kernels for these shapes do well when N is
// large and reach only 40-60 % of the memory bandwidth when N is small (N = 4096 or 6144 gives
// fewer thread blocks than the GPU has SMs).  Here a CTA owns 64 output features (one 16-row
// tensor-core tile per warp) and a slice of K, and streams its part of w through six (five for
// 16 tokens) shared-memory stages of 128 k-values with cp.async (16 KB of w and up to 4 KB of x per stage),
// two CTAs per SM.  The K dimension is split so that the grid fills the GPU once or twice
// exactly; each split writes float32 partial sums to scratch and a second small kernel adds them
// in a fixed order (no atomics: the result does not depend on timing).  With one split the
// result is written directly.
// The product runs on the tensor cores with the roles swapped: w is the 16-row A operand of
// mma.sync m16n8k16 and the tokens are the 8 columns of B (8 tokens use a full instruction,
// 16 tokens two).  Accumulation is float32; the result is float32 or bfloat16.
// The reference calls cublasSgemm for every product (src/layers/linear.cu:169-215).
#include "common.cuh"

#define GS_ROWS 64          // output features per CTA (16 per warp)
#define GS_BK 128           // k-values per stage
#define GS_STAGES_FOR(MT) ((MT) <= 8 ? 6 : 5)   // two CTAs per SM must fit: (64 + MT) rows * 256 B per stage
#define GS_THREADS 128
#define GS_MAX_SPLITS 16

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

// MT: token tile (8 or 16).  grid (feature tiles, k splits).
template <int MT, typename TO>
__global__ void __launch_bounds__(GS_THREADS) linear_skinny_kernel(const bf16* __restrict__ x,
                                                                   const bf16* __restrict__ w, TO* __restrict__ y,
                                                                   float* __restrict__ partial, int M, int N, int K) {
    constexpr int GS_STAGES = GS_STAGES_FOR(MT);
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* w_s = reinterpret_cast<bf16*>(smem_raw);                       // [STAGES][64][BK]
    bf16* x_s = w_s + GS_STAGES * GS_ROWS * GS_BK;                       // [STAGES][MT][BK]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * GS_ROWS;
    const int nk_all = (K + GS_BK - 1) / GS_BK, splits = gridDim.y;
    const int kt_begin = static_cast<int>(static_cast<long long>(blockIdx.y) * nk_all / splits);
    const int kt_end = static_cast<int>(static_cast<long long>(blockIdx.y + 1) * nk_all / splits);
    const int nk = kt_end - kt_begin;
    constexpr int CPR = GS_BK / 8;                                       // 16-byte chunks per row of a stage

    auto load_w = [&](int i) {                                           // weights of k-tile kt_begin + i into stage i % STAGES
        const int k0 = (kt_begin + i) * GS_BK;
        bf16* ws = w_s + (i % GS_STAGES) * GS_ROWS * GS_BK;
#pragma unroll
        for (int j = 0; j < GS_ROWS * CPR / GS_THREADS; ++j) {
            const int c = tid + GS_THREADS * j, row = c / CPR, ch = c % CPR;
            const bool valid = (n0 + row < N) && (k0 + ch * 8 < K);
            gs_cp_async16(gs_at(ws, row, ch), w + (valid ? static_cast<size_t>(n0 + row) * K + k0 + ch * 8 : 0), valid);
        }
    };
    auto load_x = [&](int i) {                                           // the tokens' rows for the same k-tile
        const int k0 = (kt_begin + i) * GS_BK;
        bf16* xs = x_s + (i % GS_STAGES) * MT * GS_BK;
#pragma unroll
        for (int j = 0; j < MT * CPR / GS_THREADS; ++j) {
            const int c = tid + GS_THREADS * j, row = c / CPR, ch = c % CPR;
            const bool valid = (row < M) && (k0 + ch * 8 < K);
            gs_cp_async16(gs_at(xs, row, ch), x + (valid ? static_cast<size_t>(row) * K + k0 + ch * 8 : 0), valid);
        }
    };

    // The weights do not depend on the kernel before this one: start streaming them at once, and
    // only then wait for that kernel (whose output is x) to finish.
    pdl_invite();
#pragma unroll
    for (int s = 0; s < GS_STAGES - 1; ++s)
        if (s < nk) load_w(s);
    pdl_wait();
#pragma unroll
    for (int s = 0; s < GS_STAGES - 1; ++s) {
        if (s < nk) load_x(s);
        gs_commit();                                                     // group 0 also holds every weight copy above
    }
    float acc[MT / 8][4];
#pragma unroll
    for (int j = 0; j < MT / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

    for (int i = 0; i < nk; ++i) {
        gs_wait<GS_STAGES - 2>();
        __syncthreads();
        if (i + GS_STAGES - 1 < nk) {
            load_w(i + GS_STAGES - 1);
            load_x(i + GS_STAGES - 1);
        }
        gs_commit();
        bf16* ws = w_s + (i % GS_STAGES) * GS_ROWS * GS_BK;
        bf16* xs = x_s + (i % GS_STAGES) * MT * GS_BK;
#pragma unroll
        for (int kp = 0; kp < GS_BK / 32; ++kp) {                        // pairs of k-steps
            unsigned a0[4], a1[4];
            gs_ldmatrix_x4(a0, gs_at(ws, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, kp * 4 + (lane >> 4)));
            gs_ldmatrix_x4(a1, gs_at(ws, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, kp * 4 + 2 + (lane >> 4)));
#pragma unroll
            for (int j = 0; j < MT / 8; ++j) {
                unsigned b[4];                                           // tokens 8j..8j+7, two k-steps
                gs_ldmatrix_x4(b, gs_at(xs, j * 8 + (lane & 7), kp * 4 + (lane >> 3)));
                gs_mma(acc[j], a0, b[0], b[1]);
                gs_mma(acc[j], a1, b[2], b[3]);
            }
        }
    }
    gs_wait<0>();
    // acc[j]: features warp*16 + lane/4 (+8), tokens j*8 + (lane%4)*2 (+1)
    const int f0 = n0 + warp * 16 + (lane >> 2), t0 = (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < MT / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int f = f0 + (e >> 1) * 8, tok = j * 8 + t0 + (e & 1);
            if (f < N && tok < M) {
                if (splits == 1) y[static_cast<size_t>(tok) * N + f] = from_f32<TO>(acc[j][e]);
                else partial[(static_cast<size_t>(blockIdx.y) * M + tok) * N + f] = acc[j][e];
            }
        }
    }
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
    return M >= 1 && M <= 16 && N >= 1 && K >= 8 && (K % 8) == 0;
}

static int g_skinny_slots = 0;     // CTAs the current device holds at once (two per SM), found at the first call

// How many k-splits a call uses: the grid should fill the GPU's CTA slots once or twice exactly.
static int skinny_splits(int N, int K) {
    const int tiles = (N + GS_ROWS - 1) / GS_ROWS, nk = (K + GS_BK - 1) / GS_BK;
    if (tiles >= g_skinny_slots) return 1;
    int best = 1;
    for (int s = 1; s <= GS_MAX_SPLITS && s <= nk / 4; ++s)             // at least 4 stages per split
        if (tiles * s <= g_skinny_slots) best = s;
    return best;
}

// Floats of scratch a call needs for its partial sums.
extern "C" long long llm_linear_skinny_scratch_floats(int M, int N, int K) {
    if (g_skinny_slots == 0) return static_cast<long long>(GS_MAX_SPLITS) * M * N;
    const int s = skinny_splits(N, K);
    return s > 1 ? static_cast<long long>(s) * M * N : 0;
}

// The number of k-splits a product of these sizes is cut into on the current device.
extern "C" int llm_linear_skinny_splits(int M, int N, int K) {
    if (g_skinny_slots == 0) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            return 1;
        g_skinny_slots = sms * 2;
    }
    (void)M;
    return skinny_splits(N, K);
}

template <int MT, typename TO>
static int launch_skinny(const bf16* x, const bf16* w, void* y, float* scratch, long long scratch_floats, int M, int N,
                         int K, int keep_partials, cudaStream_t s) {
    if (g_skinny_slots == 0) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            return LLM_REFUSED_SIZE;
        g_skinny_slots = sms * 2;
    }
    const size_t smem = static_cast<size_t>(GS_STAGES_FOR(MT)) * (GS_ROWS + MT) * GS_BK * sizeof(bf16);
    auto kern = linear_skinny_kernel<MT, TO>;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    int splits = skinny_splits(N, K);
    if (splits > 1 && (scratch == nullptr || scratch_floats < static_cast<long long>(splits) * M * N)) splits = 1;
    dim3 grid((N + GS_ROWS - 1) / GS_ROWS, splits);
    launch_pdl(kern, dim3(grid), dim3(GS_THREADS), smem, s, x, w, static_cast<TO*>(y), scratch, M, N, K);
    int rc = launch_status();
    if (rc != LLM_OK || splits == 1 || keep_partials) return rc;     // the caller's next kernel adds the splits itself
    const long long mn = static_cast<long long>(M) * N;
    launch_pdl((linear_skinny_sum_kernel<TO>), dim3(static_cast<unsigned>((mn + 255) / 256)), dim3(256), 0, s, scratch, static_cast<TO*>(y), mn, splits);
    return launch_status();
}

// x: bfloat16 [M, K]; w: bfloat16 [N, K]; y: [M, N] float32 (out_dtype 0) or bfloat16 (1);
// scratch: float32 of scratch_floats elements (without enough scratch K is not split).
// keep_partials: with more than one split, leave the splits' sums in scratch as [splits, M, N]
// and write nothing to y (llm_linear_skinny_splits tells the count beforehand).
extern "C" int llm_linear_skinny(const void* x, const void* w, void* y, int out_dtype, float* scratch,
                                 long long scratch_floats, int M, int N, int K, int keep_partials, uintptr_t stream) {
    if (!llm_linear_skinny_supported(M, N, K)) return LLM_REFUSED_SIZE;
    if (!aligned16(x) || !aligned16(w)) return LLM_REFUSED_ALIGN;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bf16* xp = static_cast<const bf16*>(x);
    const bf16* wp = static_cast<const bf16*>(w);
    if (M <= 8) {
        if (out_dtype == LLM_DT_F32) return launch_skinny<8, float>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, s);
        if (out_dtype == LLM_DT_BF16) return launch_skinny<8, bf16>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, s);
    } else {
        if (out_dtype == LLM_DT_F32) return launch_skinny<16, float>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, s);
        if (out_dtype == LLM_DT_BF16) return launch_skinny<16, bf16>(xp, wp, y, scratch, scratch_floats, M, N, K, keep_partials, s);
    }
    return LLM_REFUSED_DTYPE;
}
