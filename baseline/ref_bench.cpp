// Times MegEngine/InferLLM's own decode loop through its public API (include/model.h): the
// unmodified reference, linked as the static library its own CMake build makes.
//
//   ref_bench MODEL.bin cpu|gpu THREADS CTX CONTEXT_TOKENS WARMUP STEPS
//
// MODEL.bin is a LLaMA model in the reference's container whose vocabulary gives token i the
// four-letter word of `word_of(i)` below (reference_arm.py writes it), so that a prompt of chosen
// token ids can be handed to the reference's string API: all words have the same length, so its
// tokenizer (src/core/model_imp.cpp:82-131) can cut the text in one way only.
//
// What runs, in the manner of application/llama/llama.cpp:141-244: Model(config, "llama2"), load,
// init (the command line's default sampling settings), prefill of the first piece of the context,
// decode() of the further pieces, then decode_iter() WARMUP + STEPS times.  No call brings more
// than 100 tokens: the reference's KV storage grows by 100 rows once per call
// (src/core/kvstotage.cpp:53-70), which covers every call of at most 100 tokens and no longer one.
//
// Prints one JSON object: the wall time per decode_iter call over the last STEPS calls, the same by
// the reference's own timer (decode_summary's "Total Model Compute Time", which sums the execute
// calls of decode_iter, src/core/model_imp.cpp:55-64), the time the context took to feed, and the
// wall-clock times at which the timed calls began and ended.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "model.h"

static std::string word_of(int id) {
    std::string w(4, 'a');
    for (int i = 3; i >= 0; i--) {
        w[i] = (char)('a' + (id & 15));
        id >>= 4;
    }
    return w;
}

static double compute_seconds(const std::string& summary) {
    const char* key = "Total Model Compute Time:";
    size_t at = summary.find(key);
    return at == std::string::npos ? -1.0 : atof(summary.c_str() + at + strlen(key));
}

static double unix_s() {   // wall-clock time, so that the caller can pick the clock samples of the timed region
    return std::chrono::duration<double>(std::chrono::system_clock::now().time_since_epoch()).count();
}
static double now_s() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
    if (argc != 8) {
        fprintf(stderr, "usage: ref_bench MODEL.bin cpu|gpu THREADS CTX CONTEXT_TOKENS WARMUP STEPS\n");
        return 2;
    }
    const std::string path = argv[1], device = argv[2];
    const int threads = atoi(argv[3]), ctx = atoi(argv[4]), context_tokens = atoi(argv[5]);
    const int warmup = atoi(argv[6]), steps = atoi(argv[7]);
    const int vocab_draw = 16384;     // ids 1..16383 exist in every vocabulary this is used with
    if (context_tokens + warmup + steps + 2 >= ctx) {
        fprintf(stderr, "ref_bench: context %d + %d steps do not fit n_ctx %d\n", context_tokens, warmup + steps, ctx);
        return 2;
    }

    inferllm::ModelConfig config;
    config.compt_type = "float32";
    config.device_type = device;
    config.nr_thread = (uint32_t)threads;
    config.nr_ctx = (uint32_t)ctx;
    config.device_id = 0;
    config.enable_mmap = false;
    auto model = std::make_shared<inferllm::Model>(config, "llama2");
    model->load(path);
    // the command line's defaults (application/llama/llama.cpp:20-41); end token -1: never met
    model->init(40, 0.95f, 0.10f, 1.30f, 64, 1, -1);

    // the context: token ids from a small generator, never 0 (the reference's tokenizer reads id 0
    // as "no token found")
    unsigned long long state = 0x9E3779B97F4A7C15ull;
    auto next_id = [&]() {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        return 1 + (int)((state >> 33) % (unsigned)(vocab_draw - 1));
    };
    int fed = 0, token = 0;
    const double t_feed0 = now_s();
    while (fed < context_tokens) {
        const bool first = fed == 0;
        int n = context_tokens - fed;
        const int most = first ? 99 : 100;       // prefill() puts the begin token in front
        if (n > most) n = most;
        std::string text;
        for (int i = 0; i < n; i++) text += word_of(next_id());
        if (first) {
            model->prefill(text);
            fed += n + 1;
        } else {
            model->decode(text, token);
            fed += n;
        }
    }
    if (fed == context_tokens + 1 || token == 0) model->decode(word_of(next_id()), token);   // decode_iter needs a previous token
    const double t_feed = now_s() - t_feed0;

    for (int i = 0; i < warmup; i++) model->decode_iter(token);
    const double own0 = compute_seconds(model->decode_summary());
    const double unix0 = unix_s();
    const double t0 = now_s();
    for (int i = 0; i < steps; i++) model->decode_iter(token);
    const double wall = now_s() - t0;
    const double unix1 = unix_s();
    const double own = compute_seconds(model->decode_summary()) - own0;
    printf("{\"device\": \"%s\", \"threads\": %d, \"context_tokens\": %d, \"feed_s\": %.4f, \"steps\": %d, "
           "\"wall_ms_per_token\": %.4f, \"own_timer_ms_per_token\": %.4f, \"timed_begin_unix\": %.3f, \"timed_end_unix\": %.3f}\n",
           device.c_str(), threads, fed, t_feed, steps, wall * 1e3 / steps, own * 1e3 / steps, unix0, unix1);
    return 0;
}
