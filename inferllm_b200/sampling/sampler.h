// Sampling parameters and the per-batch sampler that drives the device kernels.
//
// Options and their meaning are the reference's (app_params, application/llama/llama.cpp:20-41;
// Model::init, include/model.h:38-39; algorithm llama_sample_top_p_top_k, src/utils.cpp:31-115):
// temperature, top_k, top_p, repeat_penalty over the last repeat_last_n tokens (prompt included,
// src/core/model_imp.cpp:25-28,72-73), seed.  Differences: temperature 0 means greedy (the reference
// would divide by zero); random numbers come from a counter-based generator keyed by (seed, request
// number, step), so a sequence's draws do not depend on what else is in its batch (the reference has
// one std::mt19937 for its one sequence).
#pragma once
#include <map>
#include <vector>

#include "device/device.h"
#include "engine/engine.h"

namespace illm {

struct SamplingParams {
    float temp = 0.0f;              // 0 = greedy
    int top_k = 0;                  // 0 = off
    float top_p = 1.0f;             // 1 = off
    float repeat_penalty = 1.0f;    // 1 = off
    int repeat_last_n = 64;
    long long seed = 0;
    void validate() const;          // ValueError for a parameter outside its range
    bool greedy() const { return temp == 0.0f; }
};

// A float32 uniform number in [0, 1) from (seed, request, step): splitmix64 of the mixed key.
float uniform_for(long long seed, long long request, long long step);

// Token ids on the device, int32 [n]; the memory belongs to whoever made it and stays valid for the
// next two steps (a small ring).
struct TokensRef {
    const int* p = nullptr;
    int n = 0;
};

// Chooses one token per row of logits.  requests[i] is the request number of row i, steps[i] how many
// tokens it has generated so far, histories[i] (if given) the tokens (prompt and generated) of its
// sequence.
//
// For the repetition penalty the sampler needs each sequence's last repeat_last_n tokens.  A loop
// that has them on the host passes `histories` with every call.  A loop that keeps the sampled tokens
// on the device passes the prompts as `histories` with the first call of a batch (all steps 0) and
// nullptr afterwards: the sampler then keeps the windows on the device itself, one row per request,
// and writes every token it samples into them (the sequences of a batch advance together, so the
// oldest entry of every row is at the same place).
class Sampler {
public:
    Sampler(Device* dev, const SamplingParams& params);
    ~Sampler();
    TokensRef choose(const LogitsRef& logits, const std::vector<int>& requests, const std::vector<int>& steps,
                     const std::vector<std::vector<int>>* histories);
    const SamplingParams& params() const { return params_; }

private:
    bool wants_history() const { return params_.repeat_penalty != 1.0f && params_.repeat_last_n > 0; }
    int* out_buffer(int n);
    const int* upload_ints(const std::vector<int>& v);
    Device* dev_;
    SamplingParams params_;
    int* window_ = nullptr;         // int32 [window_rows_, repeat_last_n] on the device
    int window_rows_ = 0, window_cap_ = 0;
    std::map<int, int> row_of_;     // request -> its row of the window
    int* ring_[4] = {nullptr, nullptr, nullptr, nullptr};
    int ring_cap_[4] = {0, 0, 0, 0};
    int ring_next_ = 0;
};

}  // namespace illm
