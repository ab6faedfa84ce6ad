// Drives MegEngine/InferLLM's own LLaMA graph on the CPU (naive kernels, one thread) and dumps
// logits, for tests/golden/.  Links the reference's static library; compiled by make_golden.sh
// with -std=c++11 (the reference defines its own make_unique).
//
//   ref_harness MODEL.bin TOKENS.txt OUT.f32
//
// TOKENS.txt holds one request per line (token ids separated by blanks).  For every request it
// writes, as float32: the logits of each position obtained by feeding the tokens one at a time
// (n rows), then the logits of the last position obtained by feeding the whole request in one
// call (1 row).  The reference returns the last position's logits only
// (src/core/graph.cpp:166-197, src/core/op.cpp:230-247).
#include <cstdio>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "core/device.h"
#include "core/graph.h"
#include "file.h"
#include "utils.h"

using namespace inferllm;

int main(int argc, char** argv) {
    if (argc != 4) {
        fprintf(stderr, "usage: ref_harness MODEL.bin TOKENS.txt OUT.f32\n");
        return 2;
    }
    CPUDevice device(KernelType::Naive, 1);
    UserConfig uc;
    uc.compt_type = DType::Float32;
    auto graph = Graph::make_graph(uc, &device, "llama2");
    LlmParams param;
    param.n_ctx = 256;
    auto fin = std::make_shared<InputFile>(argv[1], false);
    auto vocab = std::make_shared<Vocab>();
    graph->load(fin, param, vocab);

    std::ifstream toks(argv[2]);
    FILE* out = fopen(argv[3], "wb");
    std::string line;
    while (std::getline(toks, line)) {
        std::istringstream is(line);
        std::vector<int32_t> ids;
        int32_t v;
        while (is >> v) ids.push_back(v);
        if (ids.empty()) continue;
        std::vector<float> logits(param.n_vocab);
        graph->reset_ctx();
        for (size_t i = 0; i < ids.size(); i++) {
            graph->execute({ids[i]}, logits, (uint32_t)i, false);
            fwrite(logits.data(), sizeof(float), logits.size(), out);
        }
        graph->reset_ctx();
        graph->execute(ids, logits, 0, false);
        fwrite(logits.data(), sizeof(float), logits.size(), out);
    }
    fclose(out);
    return 0;
}
