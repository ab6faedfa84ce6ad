// Calls MegEngine/InferLLM's own grouped-head attention loops on the CPU (naive kernels) and dumps
// their results, for tests/golden/.  Links the reference's static library; compiled by make_golden.sh
// with -std=c++11.
//
//   ref_ops_harness OUT.f32
//
// Sizes: 6 query heads over 2 KV heads of size 24, 7 cached positions, 5 new tokens.  Inputs come from
// a small generator that tests/test_plain_and_golden.py repeats.  Written, as float32 in this order:
//   q [5, 6*24], k [12, 2*24], v [12, 2*24]                        (the inputs)
//   scores [6, 5, 12]   llm_matmul_compute_with_head_strideq_broadcastk_float (src/kern/naive/naive.cpp:576-604)
//   masked [6, 5, 12]   llm_scale_diag_mask_inf_float, scale 1/sqrt(24)       (:531-553)
//   probs  [6, 5, 12]   llm_softmax_compute_float over rows of 12              (:209-240)
//   out    [5, 6*24]    llm_head_batched_matmul_broadcastv_float              (:634-662)
#include <cmath>
#include <cstdio>
#include <vector>

#include "kern/naive/naive.h"

using namespace inferllm;

static void run(const TaskSet& tasks) {
    for (auto& t : tasks) t.first(TaskId{0, t.second, 0});
}

int main(int argc, char** argv) {
    if (argc != 2) {
        fprintf(stderr, "usage: ref_ops_harness OUT.f32\n");
        return 2;
    }
    const uint32_t nh = 6, nkv = 2, d = 24, past = 7, seqlen = 5, len = past + seqlen, embd = nh * d;
    unsigned long long state = 12345;
    auto next = [&]() {      // numbers in [-1, 1) with 16 bits: exact in float32 and float64
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        return (float)((double)((state >> 40) & 0xFFFF) / 32768.0 - 1.0);
    };
    std::vector<float> q(seqlen * embd), k(len * nkv * d), v(len * nkv * d);
    for (auto& x : q) x = next();
    for (auto& x : k) x = next();
    for (auto& x : v) x = next();
    std::vector<float> scores(nh * seqlen * len), masked(scores.size()), probs(scores.size()), out(seqlen * embd);
    run(naive::llm_matmul_compute_with_head_strideq_broadcastk_float(scores.data(), k.data(), q.data(), seqlen, embd, nh,
                                                                       nkv, past));
    run(naive::llm_scale_diag_mask_inf_float(masked.data(), scores.data(), 1.0f / sqrtf((float)d), past, seqlen, nh));
    run(naive::llm_softmax_compute_float(masked.data(), probs.data(), nh * seqlen, len));
    run(naive::llm_head_batched_matmul_broadcastv_float(out.data(), v.data(), probs.data(), seqlen, embd, nh, nkv, past));
    FILE* f = fopen(argv[1], "wb");
    for (auto* vec : {&q, &k, &v, &scores, &masked, &probs, &out}) fwrite(vec->data(), sizeof(float), vec->size(), f);
    fclose(f);
    return 0;
}
