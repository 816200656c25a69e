// Picking the next token on the device: greedy argmax and temperature sampling.
//
// argmax: largest logit, ties to the lowest index (src/ops/argmax.cu:41-62,98-114).
// sampling (the reference parses --temperature but only ever takes the argmax,
// src/main.cpp:175-178): p = softmax(logits / T) in 32-bit, u uniform in [0,1) from the
// request's own random stream, token = first index whose cumulative probability exceeds u.
//
// Each request's stream lives in its fixed-size state slot: {seed_lo, seed_hi, counter,
// temperature as float bits}.  u is a pure function of (seed, counter), so a request draws the
// same numbers whatever else is in the batch; the kernel advances the counter.
#include "common.cuh"
#include <math_constants.h>

#define SAMPLE_THREADS 1024

__host__ __device__ inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    uint64_t z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// 24 random bits -> [0, 1)
__host__ __device__ inline float uniform_from(uint64_t seed, uint32_t counter) {
    const uint64_t r = splitmix64(splitmix64(seed) + counter);
    return static_cast<float>(r >> 40) * (1.0f / 16777216.0f);
}

struct MaxIdx {
    float v;
    int i;
};
__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__device__ MaxIdx block_argmax(const float* __restrict__ row, int vocab, MaxIdx* sh) {
    MaxIdx best = {-CUDART_INF_F, 0x7fffffff};
    int i = threadIdx.x;
    const int step = blockDim.x;
    for (; i + 7 * step < vocab; i += 8 * step) {                        // eight loads in flight, then the comparisons in index order
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = row[i + k * step];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (v[k] > best.v || (v[k] == best.v && i + k * step < best.i)) best = {v[k], i + k * step};
    }
    for (; i < vocab; i += step) {
        const float v = row[i];
        if (v > best.v || (v == best.v && i < best.i)) best = {v, i};    // NaN never wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) sh[warp] = best;
    __syncthreads();
    if (warp == 0) {
        MaxIdx b = (lane < (blockDim.x >> 5)) ? sh[lane] : MaxIdx{-CUDART_INF_F, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            MaxIdx other = {__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
            b = better(b, other);
        }
        if (lane == 0) sh[32] = b;
    }
    __syncthreads();
    MaxIdx r = sh[32];
    if (r.i == 0x7fffffff) r.i = 0;            // a row of NaN or -inf: token 0, like a scan from index 0
    return r;
}

__global__ void argmax_rows_kernel(const float* __restrict__ logits, int vocab, int32_t* __restrict__ out) {
    pdl_begin();
    __shared__ MaxIdx sh[33];
    const MaxIdx r = block_argmax(logits + static_cast<size_t>(blockIdx.x) * vocab, vocab, sh);
    if (threadIdx.x == 0) out[blockIdx.x] = r.i;
}

// Two stages for long rows: every block takes a chunk of one row and leaves its best (value,
// index); a second launch picks the best chunk per row.  Ties still go to the lowest index,
// because `better` compares indices and chunks are index ranges.
__global__ void argmax_chunks_kernel(const float* __restrict__ logits, int vocab, int chunk,
                                     float* __restrict__ part_val, int32_t* __restrict__ part_idx) {
    pdl_begin();
    __shared__ MaxIdx sh[33];
    const int row = blockIdx.y, c0 = blockIdx.x * chunk, n = min(chunk, vocab - c0);
    MaxIdx r = block_argmax(logits + static_cast<size_t>(row) * vocab + c0, n, sh);
    if (threadIdx.x == 0) {
        part_val[row * gridDim.x + blockIdx.x] = r.v;
        part_idx[row * gridDim.x + blockIdx.x] = r.i + c0;
    }
}

__global__ void argmax_merge_kernel(const float* __restrict__ part_val, const int32_t* __restrict__ part_idx,
                                    int chunks, int32_t* __restrict__ out) {
    pdl_begin();
    MaxIdx best = {-CUDART_INF_F, 0x7fffffff};
    for (int c = threadIdx.x; c < chunks; c += 32)
        best = better(best, MaxIdx{part_val[blockIdx.x * chunks + c], part_idx[blockIdx.x * chunks + c]});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    if (threadIdx.x == 0) out[blockIdx.x] = best.i == 0x7fffffff ? 0 : best.i;
}

#define ARGMAX_CHUNK 8192
#define ARGMAX_MAX_CHUNKS 64

// scratch: room for num_rows * chunks floats and as many int32 (chunks = ceil(vocab / 8192), at most
// 64); may be null when vocab <= 8192.
extern "C" int llm_argmax_rows(const float* logits, int num_rows, int vocab, int32_t* out, void* scratch,
                               uintptr_t stream) {
    if (num_rows <= 0) return LLM_OK;
    if (vocab <= 0) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    int chunk = ARGMAX_CHUNK;
    int chunks = (vocab + chunk - 1) / chunk;
    if (chunks > ARGMAX_MAX_CHUNKS) {
        chunks = ARGMAX_MAX_CHUNKS;
        chunk = (vocab + chunks - 1) / chunks;
        chunks = (vocab + chunk - 1) / chunk;
    }
    if (chunks <= 1 || scratch == nullptr || num_rows > 65535) {
        launch_pdl(argmax_rows_kernel, dim3(num_rows), dim3(SAMPLE_THREADS), 0, s, logits, vocab, out);
        return launch_status();
    }
    float* part_val = static_cast<float*>(scratch);
    int32_t* part_idx = reinterpret_cast<int32_t*>(part_val + static_cast<size_t>(num_rows) * chunks);
    launch_pdl(argmax_chunks_kernel, dim3(dim3(chunks, num_rows)), dim3(256), 0, s, logits, vocab, chunk, part_val, part_idx);
    int rc = launch_status();
    if (rc != LLM_OK) return rc;
    launch_pdl(argmax_merge_kernel, dim3(num_rows), dim3(32), 0, s, part_val, part_idx, chunks, out);
    return launch_status();
}

__global__ void sample_rows_kernel(const float* __restrict__ logits, int vocab,
                                   const int32_t* __restrict__ row_slot, int32_t* __restrict__ sampler_state,
                                   int32_t* __restrict__ out) {
    pdl_begin();
    __shared__ MaxIdx sh[33];
    __shared__ float fs[33];
    __shared__ float warp_tot[32];
    __shared__ int result, owner;
    const float* row = logits + static_cast<size_t>(blockIdx.x) * vocab;
    int32_t* st = sampler_state + static_cast<size_t>(row_slot[blockIdx.x]) * 4;
    const float temperature = __int_as_float(st[3]);
    const MaxIdx top = block_argmax(row, vocab, sh);
    if (!(temperature > 0.0f)) {
        if (threadIdx.x == 0) out[blockIdx.x] = top.i;
        return;
    }
    const uint64_t seed = (static_cast<uint64_t>(static_cast<uint32_t>(st[1])) << 32) | static_cast<uint32_t>(st[0]);
    const uint32_t counter = static_cast<uint32_t>(st[2]);
    const float u = uniform_from(seed, counter);
    const float inv_t = 1.0f / temperature;

    // Each thread owns a contiguous run of the vocabulary, so cumulative order is index order.
    const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
    const int c0 = min(static_cast<int>(threadIdx.x) * chunk, vocab), c1 = min(c0 + chunk, vocab);
    float mine = 0.0f;
    for (int i = c0; i < c1; ++i) mine += expf((row[i] - top.v) * inv_t);
    const float total = block_sum(mine, fs);

    // Exclusive prefix of `mine` over threads: thread i owns the targets in [prefix[i], prefix[i+1]),
    // the last thread everything from its prefix on.  The prefixes come
    // out of a shuffle tree, so rounding may leave neighbours a few units in the last place out of
    // order; the owner is therefore the LAST thread whose prefix is not above the target, which is
    // one thread whatever the rounding did (prefix[0] is 0, so there always is one).
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    const float left = __shfl_up_sync(0xffffffffu, incl, 1);       // the inclusive sum of the lane before
    if (lane == 31) warp_tot[warp] = incl;
    if (threadIdx.x == 0) owner = 0;
    __syncthreads();
    float before = 0.0f;
    for (int wi = 0; wi < warp; ++wi) before += warp_tot[wi];
    const float excl = before + (lane > 0 ? left : 0.0f);
    const float target = u * total;
    if (excl <= target) atomicMax(&owner, static_cast<int>(threadIdx.x));
    __syncthreads();
    if (static_cast<int>(threadIdx.x) == owner) {
        float run = excl;
        int pick = -1;
        for (int i = c0; i < c1; ++i) {
            run += expf((row[i] - top.v) * inv_t);
            if (target < run) { pick = i; break; }
        }
        if (pick < 0) {
            // rounding left the target past this run (or the run is empty): the last token at or
            // before its end that has any weight
            for (int i = min(c1, vocab) - 1; i >= 0; --i)
                if (expf((row[i] - top.v) * inv_t) > 0.0f) { pick = i; break; }
            if (pick < 0) pick = top.i;
        }
        result = pick;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        out[blockIdx.x] = result;
        st[2] = static_cast<int32_t>(counter + 1u);
    }
}

extern "C" int llm_sample_rows(const float* logits, int num_rows, int vocab, const int32_t* row_slot,
                               int32_t* sampler_state, int32_t* out, uintptr_t stream) {
    if (num_rows <= 0) return LLM_OK;
    if (vocab <= 0) return LLM_REFUSED_SIZE;
    launch_pdl(sample_rows_kernel, dim3(num_rows), dim3(SAMPLE_THREADS), 0, reinterpret_cast<cudaStream_t>(stream), 
        logits, vocab, row_slot, sampler_state, out);
    return launch_status();
}

// Host copy of the stream function, so that tests and the scheduler can predict u.
extern "C" float llm_sampler_uniform(uint64_t seed, uint32_t counter) { return uniform_from(seed, counter); }
