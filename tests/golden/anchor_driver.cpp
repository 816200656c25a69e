// Drives the reference's own CPU code (unmodified, compiled from its source tree) on a
// tiny random model and writes the float32 logits of every position.  Built and run by
// make_golden.py only; the tests read the committed outputs.
//
// argv: <bundle.bin> <tokens.i32> <out.f32> vocab hidden inter layers heads kv_heads head_dim eps theta
// bundle.bin: int32 count; per tensor int32 name_len, name, int32 ndim, int64 dims[ndim], float32 data.
#include "model/qwen3.hpp"
#include "weights/weight_map.hpp"
#include "runtime/forward_context.hpp"

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

using namespace lite_llm;

int main(int argc, char** argv) {
    if (argc != 13) { std::cerr << "usage error\n"; return 2; }
    ModelConfig c;
    c.model_type = "qwen3";
    c.vocab_size = std::atoi(argv[4]); c.hidden_size = std::atoi(argv[5]);
    c.intermediate_size = std::atoi(argv[6]); c.num_hidden_layers = std::atoi(argv[7]);
    c.num_attention_heads = std::atoi(argv[8]); c.num_key_value_heads = std::atoi(argv[9]);
    c.head_dim = std::atoi(argv[10]); c.max_position_embeddings = 4096;
    c.rms_norm_eps = std::strtof(argv[11], nullptr); c.rope_theta = std::strtof(argv[12], nullptr);
    c.tie_word_embeddings = false;

    WeightMap weights;
    std::ifstream in(argv[1], std::ios::binary);
    int32_t count = 0; in.read(reinterpret_cast<char*>(&count), 4);
    for (int32_t i = 0; i < count; ++i) {
        int32_t nl = 0; in.read(reinterpret_cast<char*>(&nl), 4);
        std::string name(nl, '\0'); in.read(name.data(), nl);
        int32_t nd = 0; in.read(reinterpret_cast<char*>(&nd), 4);
        std::vector<int64_t> shape(nd); in.read(reinterpret_cast<char*>(shape.data()), 8 * nd);
        Tensor t(shape, DType::FP32, Device::CPU);
        in.read(reinterpret_cast<char*>(t.data()), t.nbytes());
        if (!in) { std::cerr << "short bundle at " << name << "\n"; return 3; }
        weights.add(name, std::move(t));
    }
    std::ifstream tf(argv[2], std::ios::binary);
    std::vector<int32_t> ids; int32_t v;
    while (tf.read(reinterpret_cast<char*>(&v), 4)) ids.push_back(v);
    const int64_t T = static_cast<int64_t>(ids.size());
    std::vector<int32_t> pos(T); for (int64_t i = 0; i < T; ++i) pos[i] = static_cast<int32_t>(i);

    Qwen3ForCausalLM model(c);
    model.load_weights(weights);
    if (!weights.empty()) { std::cerr << "unconsumed weights\n"; return 4; }
    Tensor input_ids = Tensor::from_int32_vector(ids, Device::CPU);
    Tensor position_ids = Tensor::from_int32_vector(pos, Device::CPU);
    Tensor logits({T, c.vocab_size}, DType::FP32, Device::CPU);
    ForwardContext ctx;
    ctx.position_ids = &position_ids; ctx.seq_len = T; ctx.past_len = 0; ctx.use_cache = false;
    model.forward(input_ids, ctx, logits);
    std::ofstream out(argv[3], std::ios::binary);
    out.write(reinterpret_cast<const char*>(logits.data()), logits.nbytes());
    return 0;
}
