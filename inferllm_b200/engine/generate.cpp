#include "engine/generate.h"

#include <algorithm>
#include <chrono>
#include <map>
#include <set>

#include "csrc/kernels.h"

namespace illm {

std::string GenerationResult::summary() const {
    const double pf = prefill_s > 0 ? prefill_tokens / prefill_s : 0.0, dc = decode_s > 0 ? decode_tokens / decode_s : 0.0;
    char buf[256];
    snprintf(buf, sizeof buf, "prefill: %lld tokens in %.1f ms (%.1f tok/s); decode: %lld tokens in %lld steps, %.1f ms (%.1f tok/s)",
             prefill_tokens, prefill_s * 1e3, pf, decode_tokens, decode_steps, decode_s * 1e3, dc);
    return buf;
}

Json GenerationResult::to_json() const {
    Json j = Json::object(), toks = Json::array(), fin = Json::array(), bat = Json::array(), steps = Json::array();
    for (auto& t : tokens) {
        Json a = Json::array();
        for (int v : t) a.push(v);
        toks.push(a);
    }
    for (auto& f : finish) fin.push(f);
    for (auto& b : batches) {
        Json a = Json::array();
        for (int v : b) a.push(v);
        bat.push(a);
    }
    for (double s : step_s) steps.push(s);
    j.set("tokens", toks);
    j.set("finish", fin);
    j.set("batches", bat);
    j.set("prefill_tokens", prefill_tokens);
    j.set("prefill_s", prefill_s);
    j.set("decode_tokens", decode_tokens);
    j.set("decode_s", decode_s);
    j.set("decode_steps", decode_steps);
    j.set("step_s", steps);
    return j;
}

std::vector<std::vector<int>> plan_batches(const std::vector<int>& prompt_lens, long long max_new_tokens, const Limits& limits) {
    std::vector<std::vector<int>> batches;
    std::vector<int> cur;
    long long cur_pages = 0;
    for (size_t i = 0; i < prompt_lens.size(); i++) {
        const long long n = prompt_lens[i];
        if (n <= 0) throw RequestTooLong("request " + std::to_string(i) + ": the prompt is empty");
        if (n > limits.max_seq_len)
            throw RequestTooLong("request " + std::to_string(i) + ": prompt of " + std::to_string(n) + " tokens exceeds the longest sequence (" +
                                 std::to_string(limits.max_seq_len) + ")");
        const long long worst = std::min<long long>(n + std::max<long long>(max_new_tokens, 0), limits.max_seq_len);
        const long long pages = (worst + limits.page_size - 1) / limits.page_size;
        if (pages > limits.num_pages)
            throw RequestTooLong("request " + std::to_string(i) + ": " + std::to_string(worst) + " tokens need " + std::to_string(pages) +
                                 " pages, the cache has " + std::to_string(limits.num_pages));
        if (!cur.empty() && ((int)cur.size() >= limits.max_batch || cur_pages + pages > limits.num_pages)) {
            batches.push_back(cur);
            cur.clear();
            cur_pages = 0;
        }
        cur.push_back((int)i);
        cur_pages += pages;
    }
    if (!cur.empty()) batches.push_back(cur);
    return batches;
}

static double wall_clock() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

GenerationResult generate(GenBackend& backend, const std::vector<std::vector<int>>& prompts, Chooser& chooser, long long max_new_tokens,
                          const std::vector<int>& stop_ids, const TokenCallback& on_token, const std::function<double()>& clock_in) {
    const std::function<double()> clock = clock_in ? clock_in : std::function<double()>(wall_clock);
    const Limits limits = backend.limits();
    const std::set<int> stop(stop_ids.begin(), stop_ids.end());
    const size_t n = prompts.size();
    GenerationResult res;
    res.tokens.resize(n);
    res.finish.assign(n, "");
    std::vector<int> lens;
    for (auto& p : prompts) lens.push_back((int)p.size());
    res.batches = plan_batches(lens, max_new_tokens, limits);
    if (max_new_tokens <= 0) {
        res.finish.assign(n, "length");
        return res;
    }
    for (const std::vector<int>& batch : res.batches) {
        std::map<int, int> slots;
        std::map<int, long long> n_fed;         // tokens of a request that the cache holds
        try {
            for (int r : batch) {
                slots[r] = backend.new_sequence();
                n_fed[r] = (long long)prompts[(size_t)r].size();
            }
            double t0 = clock();
            // the requests of a batch are stepped longest prompt first (all grow by one token per step, so
            // the order holds): the attention kernels hand out their blocks in the order of the step's
            // sequences, and the blocks with the most keys should start first; results are kept by request
            std::vector<int> order = batch;
            std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return prompts[(size_t)a].size() > prompts[(size_t)b].size(); });
            std::vector<StepItem> items;
            std::vector<std::vector<int>> hist;
            for (int r : order) {
                StepItem it;
                it.slot = slots[r];
                it.tokens = prompts[(size_t)r];
                it.want = {(int)prompts[(size_t)r].size() - 1};
                items.push_back(std::move(it));
                hist.push_back(prompts[(size_t)r]);
            }
            LogitsRef logits = backend.step(items, nullptr);
            // (the prompts go with the first call: a sampler that penalises repetitions starts its windows
            // of last tokens from them and keeps them on the device from then on)
            std::vector<int> pending = order;
            TokensRef pending_toks = chooser.choose(logits, order, std::vector<int>(order.size(), 0), &hist);
            // the copy of the tokens to the host starts behind the sampling and is waited for by itself,
            // not by the stream (which by then holds the next step); pending_sel picks the sequences that
            // are still pending out of what was copied
            int pending_read = backend.read_tokens_async(pending_toks);
            std::vector<int> pending_sel;
            bool have_sel = false, first = true;
            while (!pending.empty()) {
                // who goes on if the token just sampled is no stop token: decided by counts alone
                std::map<int, int> n_tok;
                std::vector<int> cont, idx;
                for (size_t i = 0; i < pending.size(); i++) {
                    const int r = pending[i];
                    n_tok[r] = (int)res.tokens[(size_t)r].size() + 1;
                    if (n_tok[r] < max_new_tokens && n_fed[r] + 1 <= limits.max_seq_len) {
                        cont.push_back(r);
                        idx.push_back((int)i);
                    }
                }
                TokensRef nxt_toks;
                int nxt_read = -1;
                if (!cont.empty()) {
                    TokensRef feed = cont.size() == pending.size() ? pending_toks : backend.select(pending_toks, idx);
                    std::vector<StepItem> its;
                    std::vector<int> steps;
                    for (int r : cont) {
                        StepItem it;
                        it.slot = slots[r];
                        it.tokens = {0};
                        it.want = {0};
                        its.push_back(std::move(it));
                        steps.push_back(n_tok[r]);
                    }
                    logits = backend.step(its, &feed);
                    for (int r : cont) n_fed[r] += 1;
                    nxt_toks = chooser.choose(logits, cont, steps, nullptr);
                    nxt_read = backend.read_tokens_async(nxt_toks);
                }
                std::vector<int> toks = backend.finish_read(pending_read);      // waits for the sampling before the step above
                if (have_sel) {
                    std::vector<int> picked;
                    for (int i : pending_sel) picked.push_back(toks[(size_t)i]);
                    toks.swap(picked);
                }
                const double now = clock();
                if (first) {
                    res.prefill_s += now - t0;
                    for (int r : batch) res.prefill_tokens += (long long)prompts[(size_t)r].size();
                    first = false;
                } else {
                    res.step_s.push_back(now - t0);
                    res.decode_s += now - t0;
                    res.decode_tokens += (long long)pending.size();
                    res.decode_steps += 1;
                }
                t0 = now;
                std::set<int> stopped;
                const std::set<int> cont_set(cont.begin(), cont.end());
                for (size_t i = 0; i < pending.size(); i++) {
                    const int r = pending[i], tok = toks[i];
                    res.tokens[(size_t)r].push_back(tok);
                    if (on_token) on_token(r, tok);
                    if (stop.count(tok)) {
                        res.finish[(size_t)r] = "stop";
                        stopped.insert(r);
                    } else if ((long long)res.tokens[(size_t)r].size() >= max_new_tokens) {
                        res.finish[(size_t)r] = "length";
                    } else if (!cont_set.count(r)) {
                        res.finish[(size_t)r] = "context";
                    } else {
                        continue;
                    }
                    backend.end_sequence(slots[r]);
                    slots.erase(r);
                }
                std::vector<int> keep;
                bool any_stopped = false;
                for (size_t i = 0; i < cont.size(); i++) {
                    if (stopped.count(cont[i])) any_stopped = true;
                    else keep.push_back((int)i);
                }
                have_sel = false;
                pending_sel.clear();
                if (any_stopped) {
                    nxt_toks = keep.empty() ? TokensRef() : backend.select(nxt_toks, keep);
                    pending_sel = keep;
                    have_sel = true;
                    std::vector<int> kept;
                    for (int i : keep) kept.push_back(cont[(size_t)i]);
                    cont.swap(kept);
                }
                pending = cont;
                pending_toks = nxt_toks;
                pending_read = nxt_read;
            }
        } catch (...) {
            for (auto& s : slots) {
                try {
                    backend.end_sequence(s.second);
                } catch (...) {
                }
            }
            throw;
        }
        for (auto& s : slots) backend.end_sequence(s.second);
    }
    return res;
}

EngineBackend::~EngineBackend() {
    for (int* p : ring_)
        if (p) e_->device().free_persistent(p);
}

TokensRef EngineBackend::select(const TokensRef& toks, const std::vector<int>& idx) {
    Device& dev = e_->device();
    const int n = (int)idx.size(), i = next_;
    next_ = (next_ + 1) % 4;
    if (cap_[i] < n) {
        if (ring_[i]) dev.free_persistent(ring_[i]);
        cap_[i] = std::max(n, 256);
        ring_[i] = (int*)dev.alloc_persistent((size_t)cap_[i] * sizeof(int), "a buffer of selected tokens");
    }
    int* d_idx = dev.alloc_n<int>(std::max<size_t>(idx.size(), 1));
    dev.upload_small(d_idx, idx.data(), idx.size() * sizeof(int));
    check_kernel(illm_gather_i32(toks.p, d_idx, ring_[i], n, dev.stream()), "gather_i32");
    return TokensRef{ring_[i], n};
}

}  // namespace illm
