// Trace replay: feed given token ids through a model step by step and write logits.
//
//     trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
//
// Reads one JSON object per line from standard input:
//
//     {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
//
// `entries` gives each request's next tokens and the places among them whose logits are wanted; a
// request seen for the first time starts at its first token, any other goes on from what earlier
// steps left in the cache.  `end` names requests that are finished after the step; their slot and
// pages are given back.  For a step in which something is wanted the logits are written to
// OUT/<step>.f32 as little-endian float32 [wanted, vocab], in the order of the entries and of `want`.
// After every step a line `done <step>` is printed and flushed.
//
// It samples nothing and has no forward pass, cache or loader of its own: it drives illm::Engine::step,
// the function that generation uses.  --max-tokens is the number of tokens that live requests hold at
// any time, each request rounded up to a multiple of the page size (64); it sizes the cache.
#include <sys/stat.h>

#include <cstdio>
#include <cstring>
#include <iostream>
#include <map>
#include <string>
#include <vector>

#include "engine/engine.h"

using namespace illm;

static int usage(const char* msg) {
    fprintf(stderr, "trace_run: error: %s (usage: trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--device N])\n", msg);
    return 2;
}

static int run(int argc, char** argv) {
    std::string model, dtype, out;
    long long max_tokens = -1;
    int device = 0;
    for (int i = 1; i < argc; i++) {
        const std::string a = argv[i];
        auto value = [&](const char* name) -> std::string {
            if (i + 1 >= argc) throw EngineError(std::string(name) + " needs a value");
            return argv[++i];
        };
        if (a == "--model") model = value("--model");
        else if (a == "--dtype") dtype = value("--dtype");
        else if (a == "--out") out = value("--out");
        else if (a == "--max-tokens") max_tokens = atoll(value("--max-tokens").c_str());
        else if (a == "--device") device = atoi(value("--device").c_str());
        else if (a == "-h" || a == "--help") {
            printf("replay a trace of token ids through the engine\n"
                   "  trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--device N]\n");
            return 0;
        } else return usage(("unknown option " + a).c_str());
    }
    if (model.empty() || out.empty() || max_tokens <= 0) return usage("--model, --dtype, --out and --max-tokens are required");
    if (dtype != "bfloat16" && dtype != "float32") return usage("--dtype must be bfloat16 or float32");
    mkdir(out.c_str(), 0777);
    EngineOptions opt;
    opt.dtype = dtype;
    opt.device_id = device;
    opt.max_tokens = max_tokens;
    std::unique_ptr<Engine> engine = Engine::from_folder(model, opt);
    std::map<std::string, int> slots;
    std::string line;
    std::vector<float> host;
    while (std::getline(std::cin, line)) {
        size_t a = line.find_first_not_of(" \t\r\n");
        if (a == std::string::npos) continue;
        Json rec;
        try {
            rec = Json::parse(line);
        } catch (const std::runtime_error& e) {
            throw EngineError(std::string("a line of the trace is not valid JSON (") + e.what() + ")");
        }
        if (!rec.is_object() || !rec.has("step")) throw EngineError("a line of the trace lacks 'step'");
        const std::string step = rec.at("step").is_string() ? rec.at("step").as_string() : std::to_string(rec.at("step").as_int());
        std::vector<StepItem> items;
        const Json none = Json::parse("[]");       // a key that is left out means "nothing"
        const Json& entries = rec.has("entries") ? rec.at("entries") : none;
        const Json& ending = rec.has("end") ? rec.at("end") : none;
        if (!entries.is_array() || !ending.is_array()) throw EngineError("'entries' and 'end' of a trace line must be lists");
        for (const Json& e : entries.items()) {
            if (!e.is_object() || !e.has("id") || !e.at("tokens").is_array()) throw EngineError("an entry of the trace lacks 'id' or 'tokens'");
            const std::string id = e.at("id").is_string() ? e.at("id").as_string() : e.at("id").dump();
            auto it = slots.find(id);
            if (it == slots.end()) it = slots.emplace(id, engine->new_sequence()).first;
            StepItem item;
            item.slot = it->second;
            for (const Json& t : e.at("tokens").items()) item.tokens.push_back((int)t.as_int());
            if (e.has("want"))
                for (const Json& w : e.at("want").items()) item.want.push_back((int)w.as_int());
            items.push_back(std::move(item));
        }
        if (!items.empty()) {
            LogitsRef lg = engine->step(items);
            if (lg.rows > 0) {
                host.resize((size_t)lg.rows * lg.vocab);
                engine->read_logits(lg, host.data());
                const std::string path = out + "/" + step + ".f32";
                FILE* f = fopen(path.c_str(), "wb");
                if (!f || fwrite(host.data(), sizeof(float), host.size(), f) != host.size()) throw EngineError(path + ": cannot be written");
                fclose(f);
            }
        }
        for (const Json& id : ending.items()) {
            const std::string key = id.is_string() ? id.as_string() : id.dump();
            auto it = slots.find(key);
            if (it != slots.end()) {
                engine->end_sequence(it->second);
                slots.erase(it);
            }
        }
        engine->check_device_errors();
        printf("done %s\n", step.c_str());
        fflush(stdout);
    }
    return 0;
}

int main(int argc, char** argv) {
    try {
        return run(argc, argv);
    } catch (const std::exception& e) {
        std::string msg = e.what();
        for (char& c : msg)
            if (c == '\n') c = ' ';
        fprintf(stderr, "trace_run: error: %s\n", msg.c_str());
        return 1;
    }
}
