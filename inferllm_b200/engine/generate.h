// The generation loop above the step function.
//
// Requests (lists of token ids) are cut into batches that fit the cache; each batch starts together:
// all prompts in one step, then one token per live sequence and step.  A sequence ends at a stop token
// (which is kept in its output), at max_new_tokens, or when it has filled the longest sequence the
// cache allows; it leaves the batch at once and its slot and pages go back to the pools, where the
// next batch finds them.
//
// The host runs one step behind the device: the sampled tokens stay on the device and feed the next
// step directly; the host reads them only afterwards, while that next step already runs, so its own
// work (bookkeeping, packing and launching a step) does not add to the time per token.  A sequence
// that turns out to have sampled a stop token has then already been run one step too far: that step's
// result for it is dropped and its slot is freed, which changes nothing for the others (a sequence's
// logits do not depend on the rest of its batch).
//
// The reference's loop is the command line's `while (get_remain_token() > 0) decode_iter`
// (application/llama/llama.cpp:222-244) for its one sequence, ending a turn on token 2 (:237) and the
// run when the context is full (n_ctx - m_past, src/core/model_imp.h:93); its timing sums the wall
// time of the decode calls only (src/core/model_imp.cpp:56-59,133-142), as here.
//
// The loop needs only the few operations of GenBackend and a Chooser, so its decisions are tested on
// the CPU with stand-ins for both.
#pragma once
#include <functional>
#include <string>
#include <vector>

#include "engine/engine.h"
#include "sampling/sampler.h"

namespace illm {

struct GenerationResult {
    std::vector<std::vector<int>> tokens;       // generated ids per request (stop token included)
    std::vector<std::string> finish;            // "stop" | "length" | "context"
    std::vector<std::vector<int>> batches;      // which requests ran together
    long long prefill_tokens = 0, decode_tokens = 0, decode_steps = 0;
    double prefill_s = 0, decode_s = 0;
    std::vector<double> step_s;                 // wall time of every decode step, in order
    std::string summary() const;
    Json to_json() const;
};

class GenBackend {
public:
    virtual ~GenBackend() {}
    virtual Limits limits() = 0;
    virtual int new_sequence() = 0;
    virtual void end_sequence(int slot) = 0;
    // device_ids (may be nullptr): the step's tokens, one per item, as the chooser made them
    virtual LogitsRef step(const std::vector<StepItem>& items, const TokensRef* device_ids) = 0;
    virtual int read_tokens_async(const TokensRef& toks) = 0;        // a ticket
    virtual std::vector<int> finish_read(int ticket) = 0;
    virtual TokensRef select(const TokensRef& toks, const std::vector<int>& idx) = 0;   // toks[idx]
};

class Chooser {
public:
    virtual ~Chooser() {}
    virtual TokensRef choose(const LogitsRef& logits, const std::vector<int>& requests, const std::vector<int>& steps,
                             const std::vector<std::vector<int>>* histories) = 0;
};

// Cut the requests, in order, into batches: at most max_batch sequences, and pages for every
// sequence's worst case (prompt + new tokens, capped by the longest sequence), so that a batch that
// has started never runs out of cache.  RequestTooLong for a request that can never fit.
std::vector<std::vector<int>> plan_batches(const std::vector<int>& prompt_lens, long long max_new_tokens, const Limits& limits);

using TokenCallback = std::function<void(int request, int token)>;
GenerationResult generate(GenBackend& backend, const std::vector<std::vector<int>>& prompts, Chooser& chooser, long long max_new_tokens,
                          const std::vector<int>& stop_ids, const TokenCallback& on_token = nullptr,
                          const std::function<double()>& clock = nullptr);

// The engine and the sampler behind the loop's interfaces.
class EngineBackend : public GenBackend {
public:
    explicit EngineBackend(Engine* e) : e_(e) {}
    ~EngineBackend();
    Limits limits() override { return e_->limits(); }
    int new_sequence() override { return e_->new_sequence(); }
    void end_sequence(int slot) override { e_->end_sequence(slot); }
    LogitsRef step(const std::vector<StepItem>& items, const TokensRef* ids) override { return e_->step(items, ids ? ids->p : nullptr); }
    int read_tokens_async(const TokensRef& t) override { return e_->read_tokens_async(t.p, t.n); }
    std::vector<int> finish_read(int ticket) override { return e_->finish_read(ticket); }
    TokensRef select(const TokensRef& toks, const std::vector<int>& idx) override;

private:
    Engine* e_;
    int* ring_[4] = {nullptr, nullptr, nullptr, nullptr};
    int cap_[4] = {0, 0, 0, 0};
    int next_ = 0;
};

class SamplerChooser : public Chooser {
public:
    explicit SamplerChooser(Sampler* s) : s_(s) {}
    TokensRef choose(const LogitsRef& l, const std::vector<int>& r, const std::vector<int>& st,
                     const std::vector<std::vector<int>>* h) override {
        return s_->choose(l, r, st, h);
    }

private:
    Sampler* s_;
};

}  // namespace illm
