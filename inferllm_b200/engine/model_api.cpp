#include "engine/model_api.h"

#include <algorithm>
#include <chrono>
#include <ctime>

namespace illm {

static std::string lower(std::string s) {
    for (char& c : s) c = (char)tolower((unsigned char)c);
    return s;
}
static double now_s() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

Model::Model(const ModelConfig& config, const std::string& model_name) : config_(config), model_name_(model_name) {
    const std::string dev = lower(config.device_type);
    if (dev != "gpu" && dev != "cuda")
        throw EngineError("device_type '" + config.device_type + "' is not supported: this library runs on one CUDA GPU only");
}
Model::~Model() {
    single_sampler_.reset();
    engine_.reset();
}

EngineOptions Model::options() const {
    EngineOptions o;
    o.dtype = config_.compt_type;
    o.device_id = config_.device_id;
    o.max_tokens = config_.max_tokens > 0 ? config_.max_tokens : (long long)config_.nr_ctx;
    o.max_seq_len = config_.nr_ctx;
    o.max_batch = config_.max_batch;
    o.page_size = config_.page_size;
    o.cuda_graphs = config_.cuda_graphs;
    o.gemm = config_.gemm;
    o.poison_freed_pages = config_.poison_freed_pages;
    o.stream = config_.stream;
    return o;
}

Engine& Model::engine() {
    if (!engine_) throw EngineError("the model is not loaded yet");
    return *engine_;
}

void Model::take_end_tokens() {
    end_tokens_.clear();
    for (long long t : engine_->model().spec.eos_token_ids) end_tokens_.push_back((int)t);
    has_end_token_ = !end_tokens_.empty();
    end_token_ = has_end_token_ ? end_tokens_[0] : 0;
}

void Model::load(const std::string& model_path) {
    single_sampler_.reset();
    engine_ = Engine::from_folder(model_path, options(), model_name_);
    take_end_tokens();
}
void Model::load_random(std::unique_ptr<ArchConfig> config, unsigned long long seed) {
    single_sampler_.reset();
    engine_ = Engine::from_config(std::move(config), options(), seed);
    take_end_tokens();
}

void Model::init(unsigned top_k, float top_p, float temp, float repeat_penalty, int repeat_last_n, long long seed, int end_token) {
    if (seed < 0) seed = (long long)time(nullptr);
    SamplingParams p;
    p.temp = temp;
    p.top_k = (int)top_k;
    p.top_p = top_p;
    p.repeat_penalty = repeat_penalty;
    p.repeat_last_n = repeat_last_n;
    p.seed = seed;
    p.validate();
    sampling_ = p;
    single_sampler_.reset();
    has_end_token_ = true;
    end_token_ = end_token;
}

unsigned Model::get_remain_token() {
    const long long used = slot_ >= 0 ? engine().sequence_length(slot_) : 0;
    return (unsigned)(engine().limits().max_seq_len - used);
}

void Model::reset_token() {
    if (slot_ >= 0) engine().end_sequence(slot_);
    slot_ = -1;
    history_.clear();
    n_generated_ = 0;
    has_pre_token_ = false;
}

void Model::prefill(const std::vector<int>& prompt) {
    if (slot_ < 0) slot_ = engine().new_sequence();
    StepItem it;
    it.slot = slot_;
    it.tokens = prompt;
    engine().step({it});
    history_.insert(history_.end(), prompt.begin(), prompt.end());
}

int Model::sample(const LogitsRef& logits) {
    if (!single_sampler_) single_sampler_.reset(new Sampler(&engine().device(), sampling_));
    std::vector<std::vector<int>> hist{history_};
    TokensRef t = single_sampler_->choose(logits, {0}, {n_generated_}, &hist);
    const int tok = engine().finish_read(engine().read_tokens_async(t.p, 1))[0];
    n_generated_++;
    history_.push_back(tok);
    pre_token_ = tok;
    has_pre_token_ = true;
    return tok;
}

int Model::decode(const std::vector<int>& user_input) {
    if (slot_ < 0) slot_ = engine().new_sequence();
    StepItem it;
    it.slot = slot_;
    it.tokens = user_input;
    it.want = {(int)user_input.size() - 1};
    LogitsRef logits = engine().step({it});
    history_.insert(history_.end(), user_input.begin(), user_input.end());
    return sample(logits);
}

int Model::decode_iter() {
    if (!has_pre_token_) throw EngineError("decode_iter needs a previous token: call decode first");
    const double t0 = now_s();
    StepItem it;
    it.slot = slot_;
    it.tokens = {pre_token_};
    it.want = {0};
    LogitsRef logits = engine().step({it});
    const int tok = sample(logits);
    decode_s_ += now_s() - t0;
    decode_tokens_++;
    return tok;
}

std::string Model::decode_summary() const {
    const double per = decode_tokens_ ? decode_s_ * 1e3 / decode_tokens_ : 0.0, rate = decode_s_ > 0 ? decode_tokens_ / decode_s_ : 0.0;
    char buf[320];
    snprintf(buf, sizeof buf,
             "Run Model Summary:\nTotal Model Compute Time:   %.3fs\nTotal Model Compute Token:  %lld\n"
             "Average Token Compute Time: %.3fms\nAverage Token Generation Speed: %.3ftoken/s\n",
             decode_s_, decode_tokens_, per, rate);
    return buf;
}

void Model::warm_up(long long prompt_tokens, const std::vector<int>& batch_sizes) { engine().warm_up(prompt_tokens, batch_sizes); }

GenerationResult Model::generate(const std::vector<std::vector<int>>& prompts, long long max_new_tokens, const std::vector<int>* stop_ids,
                                 const TokenCallback& on_token) {
    std::vector<int> stop;
    if (stop_ids) {
        stop = *stop_ids;
    } else if (!has_end_token_ || std::find(end_tokens_.begin(), end_tokens_.end(), end_token_) != end_tokens_.end()) {
        stop = end_tokens_;
    } else {
        stop = {end_token_};
    }
    Engine& e = engine();
    Sampler sampler(&e.device(), sampling_);
    // the sampler keeps the windows of last tokens for the repetition penalty on the device
    SamplerChooser chooser(&sampler);
    EngineBackend backend(&e);
    GenerationResult res = illm::generate(backend, prompts, chooser, max_new_tokens, stop, on_token);
    e.check_device_errors();
    return res;
}

}  // namespace illm
