// Architecture-neutral description of a decoder, the base of typed configurations, and the one
// registry from an architecture's name to its configuration class.
//
// A configuration class (one per architecture) reads the architecture's own config.json keys and
// turns them into a ModelSpec: a list of LayerSpecs (which mixer, feed-forward, norms and block
// arrangement each layer has, with all sizes and constants as parameters) and a schedule (the
// order in which layers run, as data).  Everything below the configuration (parts, cache, engine)
// sees only the ModelSpec.
//
// The reference keeps the same split between a per-model class that reads the hyper-parameters and
// builds the layer list (LlamaLikeGraph::load_param and construct_llm, src/graph/llama_like.cpp:26-109)
// and generic modules that take their sizes as constructor arguments (src/core/graph.h:84-205); its
// registry is an if-chain that aborts on an unknown name (Graph::make_graph, src/graph/graph_imp.cpp:6-21).
#pragma once
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "util/error.h"
#include "util/json.h"

namespace illm {

// Which implementation of a part (`kind`, a key of the part registries) and the sizes and
// constants it is built with.  A parameter may itself be a part (the attention mixer's position
// encoding): an object {"kind": ..., "params": {...}}.
struct PartSpec {
    std::string kind;
    Json params = Json::object();

    PartSpec() {}
    PartSpec(std::string k, Json p) : kind(std::move(k)), params(std::move(p)) {}
    bool has(const std::string& key) const { return params.has(key) && !params.at(key).is_null(); }
    // Typed reads; a missing or mistyped parameter is a ConfigError that names the part and the key.
    long long get_int(const std::string& key) const;
    long long get_int(const std::string& key, long long fallback) const;
    double get_double(const std::string& key) const;
    double get_double(const std::string& key, double fallback) const;
    bool get_bool(const std::string& key, bool fallback) const;
    std::string get_string(const std::string& key, const std::string& fallback) const;
    PartSpec get_part(const std::string& key) const;
    Json to_json() const;
    static PartSpec from_json(const Json& j, const std::string& where);
};

// One layer: a block arrangement around a mixer and a feed-forward.  `norms` gives each of the
// block's norm roles ("norm1", "norm2", ...) a spec of its own, so the norms of a block may differ in
// kind and constants.  `prefix` is the layer's tensor-name prefix in the weight file and `names`
// maps the block's roles ("mixer", "ffn" and the norm roles) to the sub-prefix below it; a part's
// own tensor names are appended to that.
struct LayerSpec {
    std::string block;
    PartSpec mixer, ffn;
    std::map<std::string, PartSpec> norms;
    std::string prefix;
    std::map<std::string, std::string> names;
};

// One execution of a layer.  `layer` indexes ModelSpec::layers (a layer may be named by several
// entries: its weights are then used several times).  `cache` is the number of the cache entry that
// the mixer uses: an entry with writes == true owns it and appends to it; one with writes == false
// only reads what an earlier entry of the same step wrote (a layer attending to another layer's
// keys and values).
struct ScheduleEntry {
    int layer = 0, cache = 0;
    bool writes = true;
};

struct ModelSpec {
    long long hidden_size = 0, vocab_size = 0, max_positions = 0;
    std::vector<LayerSpec> layers;
    std::vector<ScheduleEntry> schedule;
    PartSpec embedding;    // params: name (tensor-name prefix), vocab_size, hidden_size, ...
    PartSpec final_norm;   // params: name, size, eps, ...
    PartSpec head;         // params: name, tied, vocab_size, hidden_size, ...
    bool has_bos = false;
    long long bos_token_id = 0;
    std::vector<long long> eos_token_ids;

    void validate() const;   // ConfigError for a schedule that names no layer, writes an entry twice or reads before writing
    Json to_json() const;
    static ModelSpec from_json(const Json& j);
};

// Base of the typed configurations: the architecture's config.json keys as fields (with
// validation), back to those keys, and the ModelSpec.
class ArchConfig {
public:
    virtual ~ArchConfig() {}
    virtual std::string architecture() const = 0;
    virtual Json to_json() const = 0;
    virtual ModelSpec model_spec() const = 0;
};

using ConfigFactory = std::function<std::unique_ptr<ArchConfig>(const Json& config_json)>;

// Register (or replace) an architecture under `name` and aliases; the model is the generic decoder
// built from the configuration's ModelSpec.
void register_architecture(const std::string& name, ConfigFactory factory, const std::vector<std::string>& aliases = {});
void unregister_architecture(const std::string& name);
std::vector<std::string> registered_architectures();
// The canonical name behind a name or an alias; ConfigError listing what is registered otherwise.
std::string resolve_architecture(const std::string& name);

// Typed configuration of a config.json object; the class is chosen by architectures[0] unless
// `model_name` (not empty) overrides it.
std::unique_ptr<ArchConfig> config_from_json(const Json& d, const std::string& model_name = "");
std::unique_ptr<ArchConfig> config_from_folder(const std::string& folder, const std::string& model_name = "");
Json read_config_json(const std::string& folder);

// Typed readers used by the configuration classes: d[key] as the wanted type; a missing key without
// a fallback, or a value of another type, is a ConfigError naming the key.
long long take_int(const Json& d, const std::string& key);
long long take_int(const Json& d, const std::string& key, long long fallback);
double take_double(const Json& d, const std::string& key, double fallback);
bool take_bool(const Json& d, const std::string& key, bool fallback);
std::string take_string(const Json& d, const std::string& key, const std::string& fallback);

}  // namespace illm
