// The generic decoder: embedding, blocks run in the order of the schedule, final norm, head.
//
// It is built from a ModelSpec alone: each layer's block arrangement, mixer, feed-forward and norms,
// the embedding and the head are looked up by kind in the part registries and built with the spec's
// parameters, so layers of one model may differ, a layer may run twice, and a layer may read another
// layer's cache.  The reference builds its module list the same way from a per-model construct_llm
// (src/graph/llama_like.cpp:54-109) and runs it in Graph::execute (src/core/graph.cpp:166-197).
#pragma once
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "parts/parts.h"

namespace illm {

class SequenceCache;

class DecoderModel {
public:
    // runtime == nullptr: the parts only declare their tensors (for checking a folder or writing a
    // random one without a device).
    DecoderModel(const ModelSpec& spec, Runtime* runtime);

    // Every tensor the model reads from a weight file, by its name there, in a fixed order.
    std::vector<std::pair<std::string, TensorDecl>> tensor_decls() const;
    // `open(prefix)` gives the source of the tensors below a prefix; each part takes its own and packs
    // them, one part at a time.
    void load_tensors(const std::function<std::unique_ptr<TensorSource>(const std::string& prefix)>& open);
    // Cache entry number -> what its writing layer's mixer asks for.
    std::map<int, CacheRequest> cache_requests() const;
    // Run the tokens of one step; float32 logits [ctx.K, vocab] (rows == 0 when nothing is wanted).
    Mat forward(const StepContext& ctx, const SequenceCache& cache, const std::vector<const int*>& tables_dev);
    // true if a one-token-per-sequence step launches the same kernels every time, i.e. no part reads
    // host-side fields of the step context.
    bool graph_safe() const;
    // true if a single prompt may be run with tokens appended behind its own (see Mixer::pad_safe).
    bool pad_safe() const;

    ModelSpec spec;
    Runtime* rt;

private:
    struct Layer {
        std::unique_ptr<Block> block;
        std::unique_ptr<Mixer> mixer;
        std::unique_ptr<FeedForward> ffn;
        std::map<std::string, std::unique_ptr<Norm>> norms;
    };
    std::vector<std::pair<std::string, Part*>> owners() const;
    std::unique_ptr<EmbeddingPart> embedding_;
    std::vector<Layer> layers_;
    std::unique_ptr<Norm> final_norm_;
    std::unique_ptr<HeadPart> head_;
};

}  // namespace illm
