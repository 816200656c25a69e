// Bench driver for the reference arm: times the UNMODIFIED reference engine (LiteLLMEngine's
// PagedGenerateEngine, float32, its own kernels and cuBLAS calls) on random weights of a given
// Qwen3 shape.  Built by reference_arm.py against the reference's own sources; nothing of this
// repository's package is compiled or linked in.
//
// The loop is the reference's own batch-decode benchmark loop (src/benchmark/generation_benchmark.cpp:
// 237-330): add the requests, prefill each alone, then decode_batch over all of them
// (src/engine/paged_generate_engine.cpp:99-149,182-341).  Only what the reference cannot do itself
// is new here: weights are random values written on the device (its loader wants a converted real
// checkpoint), and the decode steps are bracketed by CUDA events and a wall clock.
//
//   reference_arm --layers L --hidden H --heads NQ --kv-heads NKV --head-dim D --intermediate I
//                 --vocab V --theta T --eps E --batch B --context C --steps K --warmup W
//                 --page-size P --seed S [--prompt-min A --prompt-max Z --new-tokens N]
//
// Default mode: B requests whose prompts have C - (K + W) tokens; W untimed and K timed calls of
// decode_batch, the last of which reads a cache of C tokens.  With --new-tokens N the whole job is
// timed instead (prompts of uniform length in [A, Z], prefill included, N new tokens each), which is
// the reference's published measurement (readme.md:58-66).
// Prints one JSON object on the last line of standard output.
#include "engine/paged_generate_engine.hpp"
#include "model/qwen3.hpp"
#include "weights/weight_map.hpp"

#include <cuda_runtime.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

using namespace lite_llm;

namespace {

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// value[i] = mean + std * N(0, 1), a pure function of (key, i): Box-Muller over two hashed uniforms.
__global__ void fill_normal(float* out, int64_t n, uint64_t key, float mean, float std_dev) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t h = mix64(key ^ mix64(static_cast<uint64_t>(i)));
    const float u1 = (static_cast<float>(h >> 40) + 1.0f) * (1.0f / 16777217.0f);      // (0, 1)
    const float u2 = static_cast<float>((h >> 16) & 0xFFFFFF) * (1.0f / 16777216.0f);  // [0, 1)
    out[i] = mean + std_dev * sqrtf(-2.0f * logf(u1)) * cosf(6.283185307f * u2);
}

void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

struct Rng {            // host side, for token ids and prompt lengths
    uint64_t s;
    uint64_t next() {
        s += 0x9E3779B97F4A7C15ull;
        uint64_t z = s;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    int64_t below(int64_t n) { return static_cast<int64_t>(next() % static_cast<uint64_t>(n)); }
};

uint64_t g_tensor_index = 0;

void add_random(WeightMap& w, const std::string& name, std::vector<int64_t> shape, uint64_t seed, bool is_norm) {
    Tensor t(std::move(shape), DType::FP32, Device::CUDA);
    const int64_t n = static_cast<int64_t>(t.numel());
    const uint64_t key = seed * 0x100000001B3ull + (++g_tensor_index) * 0xD6E8FEB86659FD93ull;
    const int threads = 256;
    const unsigned blocks = static_cast<unsigned>((n + threads - 1) / threads);
    fill_normal<<<blocks, threads>>>(t.ptr<float>(), n, key, is_norm ? 1.0f : 0.0f, is_norm ? 0.01f : 0.02f);
    check(cudaGetLastError(), "fill_normal");
    w.add(name, std::move(t));
}

}  // namespace

int main(int argc, char** argv) {
    std::map<std::string, std::string> a;
    for (int i = 1; i + 1 < argc; i += 2) {
        if (std::strncmp(argv[i], "--", 2) != 0) { std::cerr << "bad argument " << argv[i] << "\n"; return 2; }
        a[argv[i] + 2] = argv[i + 1];
    }
    auto geti = [&](const char* k, long long dflt) { return a.count(k) ? std::atoll(a[k].c_str()) : dflt; };
    auto getf = [&](const char* k, double dflt) { return a.count(k) ? std::atof(a[k].c_str()) : dflt; };

    ModelConfig c;
    c.model_type = "qwen3";
    c.num_hidden_layers = static_cast<int>(geti("layers", 2));
    c.hidden_size = static_cast<int>(geti("hidden", 64));
    c.num_attention_heads = static_cast<int>(geti("heads", 4));
    c.num_key_value_heads = static_cast<int>(geti("kv-heads", 1));
    c.head_dim = static_cast<int>(geti("head-dim", 16));
    c.intermediate_size = static_cast<int>(geti("intermediate", 128));
    c.vocab_size = static_cast<int>(geti("vocab", 256));
    c.max_position_embeddings = 1 << 20;
    c.rope_theta = static_cast<float>(getf("theta", 10000.0));
    c.rms_norm_eps = static_cast<float>(getf("eps", 1e-6));
    c.tie_word_embeddings = false;          // the reference wants lm_head.weight in every case (src/model/qwen3.cpp:1413-1423)
    const int64_t B = geti("batch", 2), C = geti("context", 64), K = geti("steps", 4), W = geti("warmup", 3);
    const int64_t P = geti("page-size", 16);
    const uint64_t seed = static_cast<uint64_t>(geti("seed", 2));
    const int64_t job_new = geti("new-tokens", 0), pmin = geti("prompt-min", 0), pmax = geti("prompt-max", 0);

    try {
        check(cudaSetDevice(0), "cudaSetDevice");
        const int64_t H = c.hidden_size, D = c.head_dim, NQ = c.num_attention_heads, NKV = c.num_key_value_heads;
        const int64_t I = c.intermediate_size, V = c.vocab_size;
        WeightMap w;
        add_random(w, "model.embed_tokens.weight", {V, H}, seed, false);
        for (int l = 0; l < c.num_hidden_layers; ++l) {
            const std::string p = "model.layers." + std::to_string(l);
            add_random(w, p + ".input_layernorm.weight", {H}, seed, true);
            add_random(w, p + ".self_attn.q_proj.weight", {NQ * D, H}, seed, false);
            add_random(w, p + ".self_attn.k_proj.weight", {NKV * D, H}, seed, false);
            add_random(w, p + ".self_attn.v_proj.weight", {NKV * D, H}, seed, false);
            add_random(w, p + ".self_attn.o_proj.weight", {H, NQ * D}, seed, false);
            add_random(w, p + ".self_attn.q_norm.weight", {D}, seed, true);
            add_random(w, p + ".self_attn.k_norm.weight", {D}, seed, true);
            add_random(w, p + ".post_attention_layernorm.weight", {H}, seed, true);
            add_random(w, p + ".mlp.gate_proj.weight", {I, H}, seed, false);
            add_random(w, p + ".mlp.up_proj.weight", {I, H}, seed, false);
            add_random(w, p + ".mlp.down_proj.weight", {H, I}, seed, false);
        }
        add_random(w, "model.norm.weight", {H}, seed, true);
        add_random(w, "lm_head.weight", {V, H}, seed, false);
        check(cudaDeviceSynchronize(), "weights");

        Qwen3ForCausalLM model(c);
        model.load_weights(w);
        if (!w.empty()) throw std::runtime_error("some weights were not consumed");

        Rng rng{seed ^ 0xABCDEFull};
        const bool whole_job = job_new > 0;
        const int64_t new_tokens = whole_job ? job_new : K + W + 2;       // nobody finishes inside the timed steps
        std::vector<std::vector<int32_t>> prompts(B);
        int64_t longest = 0;
        for (auto& p : prompts) {
            const int64_t n = whole_job ? pmin + rng.below(pmax - pmin + 1) : C - (K + W);
            if (n <= 0) throw std::runtime_error("prompt length must be positive");
            p.resize(n);
            for (auto& t : p) t = static_cast<int32_t>(rng.below(V));
            longest = std::max(longest, n);
        }
        GreedyGenerateOptions opts;
        opts.max_new_tokens = new_tokens;
        opts.eos_token_id = -1;
        opts.verbose = false;
        opts.device = Device::CUDA;

        cudaEvent_t e0, e1;
        check(cudaEventCreate(&e0), "event");
        check(cudaEventCreate(&e1), "event");
        double prefill_s = 0.0, wall_s = 0.0;
        float dev_ms = 0.0f;
        int64_t produced = 0, steps_timed = 0;

        auto run_job = [&](bool timed) {
            // As the reference's benchmark does: an engine (and its pools) per run, requests added up
            // front, pool sized so that pages never run out (generation_benchmark.cpp:152-159).
            PagedGenerateEngine engine(model, opts, (longest + new_tokens + 16) * B, P);
            std::vector<int64_t> ids;
            for (auto& p : prompts) ids.push_back(engine.add_request(p, new_tokens, -1));
            const auto t0 = std::chrono::steady_clock::now();
            for (int64_t id : ids) if (!engine.finished(id)) engine.prefill(id);
            check(cudaDeviceSynchronize(), "prefill");
            const auto t1 = std::chrono::steady_clock::now();
            if (timed) prefill_s = std::chrono::duration<double>(t1 - t0).count();
            int64_t made = B;                                   // prefill sampled one token each
            bool all_finished = false;
            while (!all_finished) {
                all_finished = true;
                std::vector<int64_t> active;
                for (int64_t id : ids) if (!engine.finished(id)) { all_finished = false; active.push_back(id); }
                if (!active.empty()) made += static_cast<int64_t>(engine.decode_batch(active).size());
            }
            for (int64_t id : ids) engine.release_request(id);
            return made;
        };

        if (whole_job) {
            for (int64_t i = 0; i < std::min<int64_t>(W, 1); ++i) run_job(false);       // the reference's --benchmark-warmup 1
            check(cudaDeviceSynchronize(), "warmup");
            const auto t0 = std::chrono::steady_clock::now();
            check(cudaEventRecord(e0), "record");
            produced = run_job(true);
            check(cudaEventRecord(e1), "record");
            check(cudaDeviceSynchronize(), "job");
            wall_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            check(cudaEventElapsedTime(&dev_ms, e0, e1), "elapsed");
            steps_timed = new_tokens - 1;
        } else {
            PagedGenerateEngine engine(model, opts, (C + 16) * B, P);
            std::vector<int64_t> ids;
            for (auto& p : prompts) ids.push_back(engine.add_request(p, new_tokens, -1));
            const auto t0 = std::chrono::steady_clock::now();
            for (int64_t id : ids) engine.prefill(id);
            check(cudaDeviceSynchronize(), "prefill");
            prefill_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            for (int64_t i = 0; i < W; ++i) engine.decode_batch(ids);
            check(cudaDeviceSynchronize(), "warmup");
            const auto t1 = std::chrono::steady_clock::now();
            check(cudaEventRecord(e0), "record");
            for (int64_t i = 0; i < K; ++i) produced += static_cast<int64_t>(engine.decode_batch(ids).size());
            check(cudaEventRecord(e1), "record");
            check(cudaDeviceSynchronize(), "decode");
            wall_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t1).count();
            check(cudaEventElapsedTime(&dev_ms, e0, e1), "elapsed");
            steps_timed = K;
            if (produced != K * B) throw std::runtime_error("a request left the batch inside the timed steps");
            for (int64_t id : ids) engine.release_request(id);
        }
        // Host<->device bytes of one decode_batch call, from the reference's code: token ids and positions
        // (paged_generate_engine.cpp:252-262), then per layer a dense block table [B, blocks] and B lengths
        // (src/ops/attention.cu:959-1020); back come the embedding's error flag and B argmax results.
        const int64_t blocks = (C + P - 1) / P;
        const int64_t h2d = 2 * B * 4 + c.num_hidden_layers * (B * blocks * 4 + B * 4);
        const int64_t d2h = 4 + B * 4;
        std::printf("{\"tokens\": %lld, \"steps\": %lld, \"device_ms\": %.4f, \"wall_s\": %.6f, \"prefill_s\": %.4f, "
                    "\"h2d_bytes_per_step\": %lld, \"d2h_bytes_per_step\": %lld, \"batch\": %lld, \"longest_prompt\": %lld}\n",
                    static_cast<long long>(produced), static_cast<long long>(steps_timed), dev_ms, wall_s, prefill_s,
                    static_cast<long long>(h2d), static_cast<long long>(d2h), static_cast<long long>(B),
                    static_cast<long long>(longest));
    } catch (const std::exception& e) {
        std::cerr << "reference_arm: " << e.what() << "\n";
        return 1;
    }
    return 0;
}
