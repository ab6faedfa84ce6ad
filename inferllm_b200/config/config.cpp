#include "config/config.h"

#include <algorithm>
#include <fstream>
#include <set>
#include <sstream>

namespace illm {

// ---- PartSpec

static const Json& need_param(const PartSpec& s, const std::string& key) {
    if (!s.has(key)) throw ConfigError("part '" + s.kind + "': parameter '" + key + "' is missing");
    return s.params.at(key);
}
long long PartSpec::get_int(const std::string& key) const {
    const Json& v = need_param(*this, key);
    if (!v.is_int()) throw ConfigError("part '" + kind + "': parameter '" + key + "' must be an integer, found " + v.repr());
    return v.as_int();
}
long long PartSpec::get_int(const std::string& key, long long fallback) const { return has(key) ? get_int(key) : fallback; }
double PartSpec::get_double(const std::string& key) const {
    const Json& v = need_param(*this, key);
    if (!v.is_number()) throw ConfigError("part '" + kind + "': parameter '" + key + "' must be a number, found " + v.repr());
    return v.as_double();
}
double PartSpec::get_double(const std::string& key, double fallback) const { return has(key) ? get_double(key) : fallback; }
bool PartSpec::get_bool(const std::string& key, bool fallback) const {
    if (!has(key)) return fallback;
    const Json& v = params.at(key);
    if (!v.is_bool()) throw ConfigError("part '" + kind + "': parameter '" + key + "' must be true or false, found " + v.repr());
    return v.as_bool();
}
std::string PartSpec::get_string(const std::string& key, const std::string& fallback) const {
    if (!has(key)) return fallback;
    const Json& v = params.at(key);
    if (!v.is_string()) throw ConfigError("part '" + kind + "': parameter '" + key + "' must be a string, found " + v.repr());
    return v.as_string();
}
PartSpec PartSpec::get_part(const std::string& key) const {
    return from_json(need_param(*this, key), "part '" + kind + "', parameter '" + key + "'");
}
Json PartSpec::to_json() const {
    Json j = Json::object();
    j.set("kind", kind);
    j.set("params", params.is_object() ? params : Json::object());
    return j;
}
PartSpec PartSpec::from_json(const Json& j, const std::string& where) {
    if (!j.is_object() || !j.at("kind").is_string())
        throw ConfigError(where + ": a part is an object {\"kind\": ..., \"params\": {...}}, found " + j.repr());
    PartSpec s(j.at("kind").as_string(), j.has("params") && j.at("params").is_object() ? j.at("params") : Json::object());
    return s;
}

// ---- ModelSpec

void ModelSpec::validate() const {
    std::map<int, size_t> writer;
    for (size_t i = 0; i < schedule.size(); i++) {
        const ScheduleEntry& e = schedule[i];
        if (e.layer < 0 || e.layer >= (int)layers.size())
            throw ConfigError("schedule entry " + std::to_string(i) + " names layer " + std::to_string(e.layer) + ", but there are " +
                              std::to_string(layers.size()) + " layers");
        if (e.writes) {
            auto it = writer.find(e.cache);
            if (it != writer.end())
                throw ConfigError("schedule entries " + std::to_string(it->second) + " and " + std::to_string(i) +
                                  " both write cache entry " + std::to_string(e.cache));
            writer[e.cache] = i;
        } else if (!writer.count(e.cache)) {
            throw ConfigError("schedule entry " + std::to_string(i) + " reads cache entry " + std::to_string(e.cache) +
                              " before any entry has written it");
        }
    }
}

Json ModelSpec::to_json() const {
    Json j = Json::object();
    j.set("hidden_size", hidden_size);
    j.set("vocab_size", vocab_size);
    j.set("max_positions", max_positions);
    j.set("bos_token_id", has_bos ? Json(bos_token_id) : Json());
    Json eos = Json::array();
    for (long long t : eos_token_ids) eos.push(t);
    j.set("eos_token_ids", eos);
    j.set("embedding", embedding.to_json());
    j.set("final_norm", final_norm.to_json());
    j.set("head", head.to_json());
    Json ls = Json::array();
    for (const LayerSpec& l : layers) {
        Json o = Json::object();
        o.set("block", l.block);
        o.set("mixer", l.mixer.to_json());
        o.set("ffn", l.ffn.to_json());
        Json norms = Json::object();
        for (auto& n : l.norms) norms.set(n.first, n.second.to_json());
        o.set("norms", norms);
        o.set("prefix", l.prefix);
        Json names = Json::object();
        for (auto& n : l.names) names.set(n.first, n.second);
        o.set("names", names);
        ls.push(o);
    }
    j.set("layers", ls);
    Json sch = Json::array();
    for (const ScheduleEntry& e : schedule) {
        Json o = Json::object();
        o.set("layer", e.layer);
        o.set("cache", e.cache);
        o.set("writes", e.writes);
        sch.push(o);
    }
    j.set("schedule", sch);
    return j;
}

ModelSpec ModelSpec::from_json(const Json& j) {
    if (!j.is_object()) throw ConfigError("a model spec is a JSON object");
    ModelSpec s;
    s.hidden_size = take_int(j, "hidden_size");
    s.vocab_size = take_int(j, "vocab_size");
    s.max_positions = take_int(j, "max_positions");
    if (j.has("bos_token_id") && j.at("bos_token_id").is_int()) {
        s.has_bos = true;
        s.bos_token_id = j.at("bos_token_id").as_int();
    }
    for (const Json& t : j.at("eos_token_ids").items()) s.eos_token_ids.push_back(t.as_int());
    s.embedding = PartSpec::from_json(j.at("embedding"), "model spec, embedding");
    s.final_norm = PartSpec::from_json(j.at("final_norm"), "model spec, final_norm");
    s.head = PartSpec::from_json(j.at("head"), "model spec, head");
    size_t li = 0;
    for (const Json& o : j.at("layers").items()) {
        const std::string where = "model spec, layer " + std::to_string(li++);
        LayerSpec l;
        l.block = take_string(o, "block", "prenorm");
        l.mixer = PartSpec::from_json(o.at("mixer"), where + ", mixer");
        l.ffn = PartSpec::from_json(o.at("ffn"), where + ", ffn");
        if (o.at("norms").is_object())
            for (auto& m : o.at("norms").members()) l.norms[m.first] = PartSpec::from_json(m.second, where + ", norm " + m.first);
        l.prefix = take_string(o, "prefix", "");
        if (o.at("names").is_object())
            for (auto& m : o.at("names").members()) l.names[m.first] = m.second.as_string();
        s.layers.push_back(std::move(l));
    }
    for (const Json& o : j.at("schedule").items()) {
        ScheduleEntry e;
        e.layer = (int)take_int(o, "layer");
        e.cache = (int)take_int(o, "cache");
        e.writes = take_bool(o, "writes", true);
        s.schedule.push_back(e);
    }
    return s;
}

// ---- typed readers

static const Json* present(const Json& d, const std::string& key) {
    if (!d.is_object() || !d.has(key) || d.at(key).is_null()) return nullptr;
    return &d.at(key);
}
[[noreturn]] static void wrong_type(const std::string& key, const char* type, const Json& v) {
    throw ConfigError("config.json: key '" + key + "' must be " + type + ", found " + v.repr());
}
long long take_int(const Json& d, const std::string& key) {
    const Json* v = present(d, key);
    if (!v) throw ConfigError("config.json: required key '" + key + "' is missing");
    if (!v->is_int()) wrong_type(key, "int", *v);
    return v->as_int();
}
long long take_int(const Json& d, const std::string& key, long long fallback) {
    return present(d, key) ? take_int(d, key) : fallback;
}
double take_double(const Json& d, const std::string& key, double fallback) {
    const Json* v = present(d, key);
    if (!v) return fallback;
    if (!v->is_number()) wrong_type(key, "float", *v);
    return v->as_double();
}
bool take_bool(const Json& d, const std::string& key, bool fallback) {
    const Json* v = present(d, key);
    if (!v) return fallback;
    if (!v->is_bool()) wrong_type(key, "bool", *v);
    return v->as_bool();
}
std::string take_string(const Json& d, const std::string& key, const std::string& fallback) {
    const Json* v = present(d, key);
    if (!v) return fallback;
    if (!v->is_string()) wrong_type(key, "str", *v);
    return v->as_string();
}

// ---- registry

namespace {
struct Registry {
    std::map<std::string, ConfigFactory> archs;
    std::map<std::string, std::string> aliases;
};
Registry& registry() {
    static Registry r;
    return r;
}
}  // namespace

void register_llama_architecture();   // config/llama.cpp

static void ensure_builtin() {
    static bool done = false;
    if (!done) {
        done = true;
        register_llama_architecture();
    }
}

void register_architecture(const std::string& name, ConfigFactory factory, const std::vector<std::string>& aliases) {
    ensure_builtin();
    registry().archs[name] = std::move(factory);
    for (auto& a : aliases) registry().aliases[a] = name;
}
void unregister_architecture(const std::string& name) {
    ensure_builtin();
    registry().archs.erase(name);
    for (auto it = registry().aliases.begin(); it != registry().aliases.end();)
        it = it->second == name ? registry().aliases.erase(it) : std::next(it);
}
std::vector<std::string> registered_architectures() {
    ensure_builtin();
    std::vector<std::string> out;
    for (auto& a : registry().archs) out.push_back(a.first);
    return out;
}
std::string resolve_architecture(const std::string& name) {
    ensure_builtin();
    auto al = registry().aliases.find(name);
    const std::string key = al == registry().aliases.end() ? name : al->second;
    if (!registry().archs.count(key)) {
        std::string known;
        for (auto& a : registry().archs) known += (known.empty() ? "" : ", ") + a.first;
        for (auto& a : registry().aliases) known += ", " + a.first;
        throw ConfigError("unknown architecture '" + name + "'; registered: " + known);
    }
    return key;
}

std::unique_ptr<ArchConfig> config_from_json(const Json& d, const std::string& model_name) {
    if (!d.is_object()) throw ConfigError("config.json: expected a JSON object");
    std::string name = model_name;
    if (name.empty()) {
        const Json& archs = d.at("architectures");
        if (!archs.is_array() || archs.size() == 0 || !archs[0].is_string())
            throw ConfigError("config.json: required key 'architectures' (a list with the model class name) is missing");
        name = archs[0].as_string();
    }
    return registry().archs.at(resolve_architecture(name))(d);
}

Json read_config_json(const std::string& folder) {
    const std::string path = folder + "/config.json";
    std::ifstream f(path);
    if (!f) throw ConfigError(folder + ": no config.json in this model folder");
    std::stringstream ss;
    ss << f.rdbuf();
    Json d;
    try {
        d = Json::parse(ss.str());
    } catch (const std::runtime_error& e) {
        throw ConfigError(path + ": not valid JSON (" + e.what() + ")");
    }
    if (!d.is_object()) throw ConfigError(path + ": expected a JSON object");
    return d;
}

std::unique_ptr<ArchConfig> config_from_folder(const std::string& folder, const std::string& model_name) {
    return config_from_json(read_config_json(folder), model_name);
}

}  // namespace illm
