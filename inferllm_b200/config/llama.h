// Typed configuration of the LLaMA dense decoder, read from its config.json keys.
//
// The reference reads five integers from its own file header (n_embd, n_head, n_layer, n_mult,
// n_vocab, src/graph/llama_like.cpp:37-44) and fixes everything else in code: eps 1e-6 in the
// layers (src/graph/llama_like.cpp:77-78), rope base 10000 (src/kern/naive/naive.cpp:396),
// rotate-half over the whole head (:60, :82), no biases, BOS 1 (src/core/model_imp.cpp:124), EOS 2
// (application/llama/llama.cpp:175), context 2048 (application/llama/llama.cpp:25).  Here those
// constants are the defaults of the corresponding config.json keys and nothing else in the library
// repeats them.
#pragma once
#include "config/config.h"

namespace illm {

struct LlamaConfig : ArchConfig {
    long long hidden_size = 0, num_hidden_layers = 0, num_attention_heads = 0, intermediate_size = 0, vocab_size = 0;
    long long num_key_value_heads = 0, head_dim = 0;
    double rms_norm_eps = 1e-6, rope_theta = 10000.0;
    long long max_position_embeddings = 2048;
    bool tie_word_embeddings = false;
    bool has_bos = true;
    long long bos_token_id = 1;
    std::vector<long long> eos_token_id{2};
    std::string torch_dtype = "bfloat16";

    static std::unique_ptr<ArchConfig> from_json(const Json& d);
    std::string architecture() const override { return "LlamaForCausalLM"; }
    Json to_json() const override;
    // Layer stack of src/graph/llama_like.cpp:54-109: every layer is a pre-norm block of causal
    // attention with rotate-half position encoding and a gated feed-forward; the layers run once
    // each, in order, each with a cache entry of its own.
    ModelSpec model_spec() const override;
};

}  // namespace illm
