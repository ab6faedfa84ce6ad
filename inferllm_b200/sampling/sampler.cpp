#include "sampling/sampler.h"

#include <algorithm>

#include "csrc/kernels.h"

namespace illm {

void SamplingParams::validate() const {
    if (temp < 0) throw ValueError("temp must be >= 0");
    if (!(top_p > 0 && top_p <= 1)) throw ValueError("top_p must be in (0, 1]");
    if (!(repeat_penalty > 0)) throw ValueError("repeat_penalty must be > 0");
    if (top_k < 0 || repeat_last_n < 0) throw ValueError("top_k and repeat_last_n must be >= 0");
}

float uniform_for(long long seed, long long request, long long step) {
    unsigned long long x = (unsigned long long)seed * 0x9E3779B97F4A7C15ull + (unsigned long long)request * 0xBF58476D1CE4E5B9ull +
                           (unsigned long long)step * 0x94D049BB133111EBull + 0x2545F4914F6CDD1Dull;
    for (int i = 0; i < 2; i++) {
        x += 0x9E3779B97F4A7C15ull;
        unsigned long long z = x;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        x = z ^ (z >> 31);
    }
    return (float)((double)(x >> 40) / (double)(1 << 24));
}

Sampler::Sampler(Device* dev, const SamplingParams& params) : dev_(dev), params_(params) { params.validate(); }

Sampler::~Sampler() {
    if (window_) dev_->free_persistent(window_);
    for (int* p : ring_)
        if (p) dev_->free_persistent(p);
}

int* Sampler::out_buffer(int n) {
    const int i = ring_next_;
    ring_next_ = (ring_next_ + 1) % 4;
    if (ring_cap_[i] < n) {
        if (ring_[i]) dev_->free_persistent(ring_[i]);
        ring_cap_[i] = std::max(n, 256);
        ring_[i] = (int*)dev_->alloc_persistent((size_t)ring_cap_[i] * sizeof(int), "a buffer of sampled tokens");
    }
    return ring_[i];
}

const int* Sampler::upload_ints(const std::vector<int>& v) {
    int* d = dev_->alloc_n<int>(std::max<size_t>(v.size(), 1));
    dev_->upload_small(d, v.data(), v.size() * sizeof(int));
    return d;
}

TokensRef Sampler::choose(const LogitsRef& logits, const std::vector<int>& requests, const std::vector<int>& steps,
                          const std::vector<std::vector<int>>* histories) {
    const SamplingParams& p = params_;
    const int B = (int)logits.rows;
    dev_->make_current();
    if ((int)requests.size() != B || (int)steps.size() != B) throw ValueError("the sampler needs a request number and a step per row of logits");
    int* out = out_buffer(B);
    if (p.greedy() && p.repeat_penalty == 1.0f) {
        ops::argmax(*dev_, logits.p, B, logits.vocab, out);
        return TokensRef{out, B};
    }
    const int n_last = p.repeat_last_n;
    const int* last = nullptr;
    const int* rows = nullptr;
    bool on_device = false, all_known = true;
    if (wants_history()) {
        bool all_zero = true;
        for (int s : steps) all_zero = all_zero && s == 0;
        if (histories && all_zero) {
            // the windows start from the prompts (oldest first: entry 0 is the first to be replaced)
            std::vector<int> arr((size_t)B * n_last, -1);
            for (int i = 0; i < B; i++) {
                const std::vector<int>& h = (*histories)[(size_t)i];
                const int take = std::min<int>((int)h.size(), n_last);
                std::copy(h.end() - take, h.end(), arr.begin() + (size_t)i * n_last + (n_last - take));
            }
            if (window_cap_ < B) {
                if (window_) dev_->free_persistent(window_);
                window_cap_ = std::max(B, 64);
                window_ = (int*)dev_->alloc_persistent((size_t)window_cap_ * n_last * sizeof(int), "the windows of last tokens");
            }
            window_rows_ = B;
            dev_->upload_small(window_, arr.data(), arr.size() * sizeof(int));
            row_of_.clear();
            for (int i = 0; i < B; i++) row_of_[requests[(size_t)i]] = i;
        }
        for (int r : requests) all_known = all_known && row_of_.count(r);
        if (histories) {
            std::vector<int> arr((size_t)B * n_last, -1);
            for (int i = 0; i < B; i++) {
                const std::vector<int>& h = (*histories)[(size_t)i];
                const int take = std::min<int>((int)h.size(), n_last);
                std::copy(h.end() - take, h.end(), arr.begin() + (size_t)i * n_last);
            }
            last = upload_ints(arr);
        } else if (window_ && all_known) {
            std::vector<int> idx;
            bool identity = B == window_rows_;
            for (int i = 0; i < B; i++) {
                idx.push_back(row_of_[requests[(size_t)i]]);
                identity = identity && idx.back() == i;
            }
            if (identity) {
                last = window_;
            } else {
                rows = upload_ints(idx);
                int* gathered = dev_->alloc_n<int>((size_t)B * n_last);
                check_kernel(illm_window_gather(window_, n_last, rows, gathered, B, dev_->stream()), "window_gather");
                last = gathered;
            }
            on_device = true;
        }
    }
    float* u = dev_->alloc_n<float>((size_t)B);
    if (p.greedy()) {
        // greedy with a repetition penalty: the penalised maximum; top_k = 1 keeps exactly it
        check_cuda(cudaMemsetAsync(u, 0, (size_t)B * sizeof(float), dev_->stream()), "zeroing the uniform numbers");
        ops::sample(*dev_, logits.p, B, logits.vocab, u, 1.0f, 1, 1.0f, p.repeat_penalty, last, n_last, out);
    } else {
        std::vector<float> host((size_t)B);
        for (int i = 0; i < B; i++) host[(size_t)i] = uniform_for(p.seed, requests[(size_t)i], steps[(size_t)i]);
        dev_->upload_small(u, host.data(), host.size() * sizeof(float));
        ops::sample(*dev_, logits.p, B, logits.vocab, u, p.temp, p.top_k, p.top_p, p.repeat_penalty, last, n_last, out);
    }
    if (wants_history() && window_ && (on_device || histories) && all_known) {
        // the new token takes the place of the window's oldest entry
        const int col = steps[0] % n_last;
        if (!rows && B != window_rows_) {
            std::vector<int> idx;
            for (int r : requests) idx.push_back(row_of_[r]);
            rows = upload_ints(idx);
        } else if (!rows && histories) {
            std::vector<int> idx;
            bool identity = true;
            for (int i = 0; i < B; i++) {
                idx.push_back(row_of_[requests[(size_t)i]]);
                identity = identity && idx.back() == i;
            }
            if (!identity) rows = upload_ints(idx);
        }
        check_kernel(illm_window_put(window_, n_last, rows, col, out, B, dev_->stream()), "window_put");
    }
    return TokensRef{out, B};
}

}  // namespace illm
