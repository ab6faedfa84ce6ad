#include "config/llama.h"

namespace illm {

std::unique_ptr<ArchConfig> LlamaConfig::from_json(const Json& d) {
    std::unique_ptr<LlamaConfig> c(new LlamaConfig);
    const long long nh = take_int(d, "num_attention_heads");
    const long long H = take_int(d, "hidden_size");
    const long long nkv = take_int(d, "num_key_value_heads", nh);
    if (nh <= 0 || nkv <= 0 || H <= 0) throw ConfigError("config.json: sizes must be positive");
    long long hd;
    if (d.has("head_dim") && !d.at("head_dim").is_null()) {
        hd = take_int(d, "head_dim");
    } else {
        if (H % nh)
            throw ConfigError("config.json: hidden_size " + std::to_string(H) + " is not a multiple of num_attention_heads " +
                              std::to_string(nh) + " and no head_dim is given");
        hd = H / nh;
    }
    if (nh % nkv)
        throw ConfigError("config.json: num_attention_heads " + std::to_string(nh) + " is not a multiple of num_key_value_heads " +
                          std::to_string(nkv));
    if (hd <= 0 || hd % 2) throw ConfigError("config.json: head_dim " + std::to_string(hd) + " must be even (rotary pairs)");
    const std::string act = take_string(d, "hidden_act", "silu");
    if (act != "silu") throw ConfigError("config.json: hidden_act '" + act + "' is not supported (only 'silu')");
    for (const char* key : {"attention_bias", "mlp_bias"})
        if (take_bool(d, key, false)) throw ConfigError(std::string("config.json: ") + key + "=true is not supported");
    if (d.has("rope_scaling") && !d.at("rope_scaling").is_null())
        throw ConfigError("config.json: rope_scaling is not supported (must be null)");
    c->eos_token_id = {2};
    if (d.has("eos_token_id") && !d.at("eos_token_id").is_null()) {
        const Json& eos = d.at("eos_token_id");
        c->eos_token_id.clear();
        if (eos.is_int()) {
            c->eos_token_id.push_back(eos.as_int());
        } else if (eos.is_array()) {
            for (const Json& e : eos.items()) {
                if (!e.is_int()) throw ConfigError("config.json: eos_token_id must be an int or a list of ints, found " + eos.repr());
                c->eos_token_id.push_back(e.as_int());
            }
        } else {
            throw ConfigError("config.json: eos_token_id must be an int or a list, found " + eos.repr());
        }
    }
    c->hidden_size = H;
    c->num_hidden_layers = take_int(d, "num_hidden_layers");
    c->num_attention_heads = nh;
    c->intermediate_size = take_int(d, "intermediate_size");
    c->vocab_size = take_int(d, "vocab_size");
    c->num_key_value_heads = nkv;
    c->head_dim = hd;
    c->rms_norm_eps = take_double(d, "rms_norm_eps", 1e-6);
    c->rope_theta = take_double(d, "rope_theta", 10000.0);
    c->max_position_embeddings = take_int(d, "max_position_embeddings", 2048);
    c->tie_word_embeddings = take_bool(d, "tie_word_embeddings", false);
    c->has_bos = true;
    c->bos_token_id = take_int(d, "bos_token_id", 1);
    c->torch_dtype = take_string(d, "torch_dtype", "bfloat16");
    for (auto kv : {std::make_pair("num_hidden_layers", c->num_hidden_layers), std::make_pair("intermediate_size", c->intermediate_size),
                    std::make_pair("vocab_size", c->vocab_size), std::make_pair("max_position_embeddings", c->max_position_embeddings)})
        if (kv.second <= 0) throw ConfigError(std::string("config.json: ") + kv.first + " must be positive");
    if (c->rms_norm_eps <= 0 || c->rope_theta <= 0) throw ConfigError("config.json: rms_norm_eps and rope_theta must be positive");
    return std::unique_ptr<ArchConfig>(c.release());
}

Json LlamaConfig::to_json() const {
    Json j = Json::object();
    Json archs = Json::array();
    archs.push(architecture());
    j.set("architectures", archs);
    j.set("model_type", "llama");
    j.set("hidden_size", hidden_size);
    j.set("num_hidden_layers", num_hidden_layers);
    j.set("num_attention_heads", num_attention_heads);
    j.set("num_key_value_heads", num_key_value_heads);
    j.set("head_dim", head_dim);
    j.set("intermediate_size", intermediate_size);
    j.set("vocab_size", vocab_size);
    j.set("rms_norm_eps", rms_norm_eps);
    j.set("rope_theta", rope_theta);
    j.set("max_position_embeddings", max_position_embeddings);
    j.set("tie_word_embeddings", tie_word_embeddings);
    j.set("hidden_act", "silu");
    j.set("attention_bias", false);
    j.set("mlp_bias", false);
    j.set("rope_scaling", Json());
    j.set("bos_token_id", bos_token_id);
    if (eos_token_id.size() == 1) {
        j.set("eos_token_id", eos_token_id[0]);
    } else {
        Json e = Json::array();
        for (long long t : eos_token_id) e.push(t);
        j.set("eos_token_id", e);
    }
    j.set("torch_dtype", torch_dtype);
    return j;
}

ModelSpec LlamaConfig::model_spec() const {
    auto obj = [](std::initializer_list<std::pair<const char*, Json>> kv) {
        Json o = Json::object();
        for (auto& p : kv) o.set(p.first, p.second);
        return o;
    };
    PartSpec norm("rmsnorm", obj({{"size", hidden_size}, {"eps", rms_norm_eps}}));
    PartSpec position("rope_half", obj({{"head_dim", head_dim}, {"rot_dim", head_dim}, {"theta", rope_theta},
                                        {"max_positions", max_position_embeddings}}));
    PartSpec mixer("attention", obj({{"hidden_size", hidden_size}, {"n_heads", num_attention_heads},
                                     {"n_kv_heads", num_key_value_heads}, {"head_dim", head_dim}, {"window", Json()},
                                     {"position", position.to_json()}}));
    PartSpec ffn("gated_mlp", obj({{"hidden_size", hidden_size}, {"intermediate_size", intermediate_size}, {"activation", "silu"}}));
    ModelSpec s;
    s.hidden_size = hidden_size;
    s.vocab_size = vocab_size;
    s.max_positions = max_position_embeddings;
    for (long long i = 0; i < num_hidden_layers; i++) {
        LayerSpec l;
        l.block = "prenorm";
        l.mixer = mixer;
        l.ffn = ffn;
        l.norms = {{"norm1", norm}, {"norm2", norm}};
        l.prefix = "model.layers." + std::to_string(i) + ".";
        l.names = {{"mixer", "self_attn."}, {"ffn", "mlp."}, {"norm1", "input_layernorm."}, {"norm2", "post_attention_layernorm."}};
        s.layers.push_back(l);
        s.schedule.push_back(ScheduleEntry{(int)i, (int)i, true});
    }
    s.embedding = PartSpec("embedding", obj({{"name", "model.embed_tokens."}, {"vocab_size", vocab_size}, {"hidden_size", hidden_size}}));
    s.final_norm = PartSpec("rmsnorm", obj({{"name", "model.norm."}, {"size", hidden_size}, {"eps", rms_norm_eps}}));
    s.head = PartSpec("lm_head", obj({{"name", "lm_head."}, {"tied", tie_word_embeddings}, {"vocab_size", vocab_size},
                                      {"hidden_size", hidden_size}}));
    s.has_bos = has_bos;
    s.bos_token_id = bos_token_id;
    s.eos_token_ids = eos_token_id;
    return s;
}

void register_llama_architecture() {
    register_architecture("LlamaForCausalLM", &LlamaConfig::from_json, {"llama", "llama2"});
}

}  // namespace illm
