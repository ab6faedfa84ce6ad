// Command line in the manner of the reference's `llama` program.
//
// Options keep the reference's names and meanings where it has them (app_params_parse,
// application/llama/llama.cpp:88-128; defaults :20-41):
//   -m/--model, -g, -d/--dtype, -c/--ctx_size, -s/--seed, -t/--threads, --top_k, --top_p, --temp,
//   --repeat_penalty, --repeat_last_n, --mmap, -v/--version.
// What differs: -m names a model folder (config.json + safetensors) instead of a .bin file; -g takes
// "GPU" or a GPU ordinal ("CPU" is refused: there is no CPU path); -d takes bfloat16 or float32;
// prompts are token ids, since tokenisation is outside this library: --prompt-ids "1,5,9"
// (repeatable), --prompt-file FILE (one request per line) or --random-prompts "5,9,16" (lengths);
// -n is the reference's n_predict field (128, never parsed there).  --random-weights SEED with
// --config FILE writes nothing and runs a model with random weights; --write-random-model DIR writes
// such a model folder and exits.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <random>
#include <sstream>
#include <string>
#include <vector>

#include "engine/model_api.h"
#include "weights/loader.h"

using namespace illm;

static std::vector<int> ids_of(std::string text) {
    for (char& c : text)
        if (c == ',') c = ' ';
    std::istringstream is(text);
    std::vector<int> out;
    std::string tok;
    while (is >> tok) {
        char* end = nullptr;
        const long v = strtol(tok.c_str(), &end, 10);
        if (*end) throw EngineError("'" + tok + "' is not a token id");
        out.push_back((int)v);
    }
    return out;
}

static const char* kHelp =
    "usage: llama [options]\n"
    "  -m, --model DIR          model folder (config.json + model.safetensors)\n"
    "  -g DEVICE                GPU, or a GPU ordinal (default GPU = 0)\n"
    "  -d, --dtype TYPE         compute dtype: bfloat16 | float32 (default bfloat16)\n"
    "  -c, --ctx_size N         longest sequence (default 2048)\n"
    "  -s, --seed N             RNG seed (default -1: from the clock)\n"
    "  -t, --threads N          accepted for compatibility; no effect\n"
    "  -n, --n_predict N        new tokens per request (default 128)\n"
    "  --top_k N (40)  --top_p P (0.95)  --temp T (0.10; 0 = greedy)\n"
    "  --repeat_last_n N (64)  --repeat_penalty P (1.30)\n"
    "  --mmap, --color          accepted; no effect (weight files are always mapped)\n"
    "  -v, --version N          accepted; the model class comes from config.json\n"
    "  --prompt-ids IDS         comma-separated token ids (repeatable)\n"
    "  --prompt-file FILE       one request (comma- or space-separated ids) per line\n"
    "  --random-prompts LENS    comma-separated prompt lengths of random ids\n"
    "  --max-tokens N           tokens the cache holds (default: fits all requests at once, up to 64 Ki)\n"
    "  --config FILE            config.json for --random-weights / --write-random-model\n"
    "  --random-weights SEED    run a model with random weights made on the device\n"
    "  --write-random-model DIR write a model folder with random weights and exit\n"
    "  --no-stop                ignore the end token\n";

static int run(int argc, char** argv) {
    std::string model_dir, device = "GPU", dtype = "bfloat16", prompt_file, random_prompts, config_file, write_dir;
    long long ctx = 2048, seed = -1, n_predict = 128, max_tokens = 0, random_weights = 0;
    int top_k = 40, repeat_last_n = 64, threads = 4;
    float top_p = 0.95f, temp = 0.10f, repeat_penalty = 1.30f;
    bool has_random_weights = false, no_stop = false, mmap_flag = false;
    std::vector<std::string> prompt_ids;
    for (int i = 1; i < argc; i++) {
        const std::string a = argv[i];
        auto value = [&]() -> std::string {
            if (i + 1 >= argc) throw EngineError(a + " needs a value");
            return argv[++i];
        };
        if (a == "-m" || a == "--model") model_dir = value();
        else if (a == "-g") device = value();
        else if (a == "-d" || a == "--dtype") dtype = value();
        else if (a == "-c" || a == "--ctx_size") ctx = atoll(value().c_str());
        else if (a == "-s" || a == "--seed") seed = atoll(value().c_str());
        else if (a == "-t" || a == "--threads") threads = atoi(value().c_str());
        else if (a == "-n" || a == "--n_predict") n_predict = atoll(value().c_str());
        else if (a == "--top_k") top_k = atoi(value().c_str());
        else if (a == "--top_p") top_p = (float)atof(value().c_str());
        else if (a == "--temp") temp = (float)atof(value().c_str());
        else if (a == "--repeat_last_n") repeat_last_n = atoi(value().c_str());
        else if (a == "--repeat_penalty") repeat_penalty = (float)atof(value().c_str());
        else if (a == "--mmap") mmap_flag = true;
        else if (a == "--color") {}
        else if (a == "-v" || a == "--version") value();
        else if (a == "--prompt-ids") prompt_ids.push_back(value());
        else if (a == "--prompt-file") prompt_file = value();
        else if (a == "--random-prompts") random_prompts = value();
        else if (a == "--max-tokens") max_tokens = atoll(value().c_str());
        else if (a == "--config") config_file = value();
        else if (a == "--random-weights") { random_weights = atoll(value().c_str()); has_random_weights = true; }
        else if (a == "--write-random-model") write_dir = value();
        else if (a == "--no-stop") no_stop = true;
        else if (a == "-h" || a == "--help") { fputs(kHelp, stdout); return 0; }
        else { fprintf(stderr, "llama: unknown option %s\n%s", a.c_str(), kHelp); return 2; }
    }
    std::string dev_upper = device;
    for (char& c : dev_upper) c = (char)toupper((unsigned char)c);
    if (dev_upper == "CPU") {
        fprintf(stderr, "llama: -g CPU is not supported: this library runs on one CUDA GPU only\n");
        return 2;
    }
    const int device_id = dev_upper == "GPU" ? 0 : atoi(device.c_str());
    if (dtype == "bf16") dtype = "bfloat16";
    if (dtype == "fp32") dtype = "float32";

    std::unique_ptr<ArchConfig> cfg;
    Json cfg_json;
    if (!config_file.empty()) {
        std::ifstream f(config_file);
        if (!f) throw ConfigError(config_file + ": cannot be read");
        std::stringstream ss;
        ss << f.rdbuf();
        try {
            cfg_json = Json::parse(ss.str());
        } catch (const std::runtime_error& e) {
            throw ConfigError(config_file + ": not valid JSON (" + e.what() + ")");
        }
        cfg = config_from_json(cfg_json);
    }
    if (!write_dir.empty()) {
        if (!cfg) {
            fprintf(stderr, "llama: --write-random-model needs --config\n");
            return 2;
        }
        write_random_model(*cfg, write_dir, (unsigned long long)random_weights, dtype == "float32" ? DType::F32 : DType::BF16);
        printf("wrote %s\n", write_dir.c_str());
        return 0;
    }

    std::vector<std::vector<int>> prompts;
    for (auto& p : prompt_ids) prompts.push_back(ids_of(p));
    if (!prompt_file.empty()) {
        std::ifstream f(prompt_file);
        if (!f) throw EngineError(prompt_file + ": cannot be read");
        std::string line;
        while (std::getline(f, line))
            if (line.find_first_not_of(" \t\r\n") != std::string::npos) prompts.push_back(ids_of(line));
    }
    if (!random_prompts.empty()) {
        long long vocab = 0;
        if (cfg) vocab = cfg_json.at("vocab_size").as_int();
        else vocab = read_config_json(model_dir).at("vocab_size").as_int();
        if (vocab <= 0) throw ConfigError("config.json: vocab_size must be positive");
        std::mt19937_64 rng(seed >= 0 ? (unsigned long long)seed : std::random_device{}());
        for (int n : ids_of(random_prompts)) {
            std::vector<int> p;
            for (int i = 0; i < n; i++) p.push_back((int)(rng() % (unsigned long long)vocab));
            prompts.push_back(p);
        }
    }
    if (prompts.empty()) {
        fprintf(stderr, "llama: no prompt given (--prompt-ids, --prompt-file or --random-prompts)\n");
        return 2;
    }
    long long need = 0;
    for (auto& p : prompts) need += (std::min<long long>((long long)p.size() + n_predict, ctx) + 63) / 64 * 64;
    ModelConfig mc;
    mc.compt_type = dtype;
    mc.device_type = "gpu";
    mc.nr_thread = (unsigned)threads;
    mc.nr_ctx = (unsigned)ctx;
    mc.device_id = device_id;
    mc.enable_mmap = mmap_flag;
    mc.max_tokens = max_tokens > 0 ? max_tokens : std::min<long long>(need, 65536);
    Model model(mc);
    if (has_random_weights && cfg) {
        model.load_random(std::move(cfg), (unsigned long long)random_weights);
    } else if (!model_dir.empty()) {
        model.load(model_dir);
    } else {
        fprintf(stderr, "llama: give -m DIR, or --config FILE with --random-weights SEED\n");
        return 2;
    }
    const int end_token = model.has_end_token() ? model.end_token() : 2;
    model.init((unsigned)top_k, top_p, temp, repeat_penalty, repeat_last_n, seed, end_token);
    const std::vector<int> none;
    GenerationResult res = model.generate(prompts, n_predict, no_stop ? &none : nullptr);
    for (size_t i = 0; i < res.tokens.size(); i++) {
        std::string line = "[" + std::to_string(i) + "] " + res.finish[i] + ": ";
        for (size_t j = 0; j < res.tokens[i].size(); j++) line += (j ? "," : "") + std::to_string(res.tokens[i][j]);
        puts(line.c_str());
    }
    fprintf(stderr, "%s\n", res.summary().c_str());
    return 0;
}

int main(int argc, char** argv) {
    try {
        return run(argc, argv);
    } catch (const std::exception& e) {
        std::string msg = e.what();
        for (char& c : msg)
            if (c == '\n') c = ' ';
        fprintf(stderr, "llama: error: %s\n", msg.c_str());
        return 1;
    }
}
