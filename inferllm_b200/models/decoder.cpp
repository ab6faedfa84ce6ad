#include "models/decoder.h"

#include "cache/cache.h"

namespace illm {

static std::string role_name(const LayerSpec& ls, const std::string& role) {
    auto it = ls.names.find(role);
    if (it == ls.names.end()) throw ConfigError("layer '" + ls.prefix + "': no tensor-name prefix for the role '" + role + "'");
    return it->second;
}

DecoderModel::DecoderModel(const ModelSpec& s, Runtime* runtime) : spec(s), rt(runtime) {
    spec.validate();
    embedding_ = build_embedding(spec.embedding, rt);
    for (const LayerSpec& ls : spec.layers) {
        const BlockKind& kind = lookup_block(ls.block);
        Layer l;
        l.mixer = build_mixer(ls.mixer, rt);
        l.ffn = build_feed_forward(ls.ffn, rt);
        l.block = kind.make();
        l.block->mixer = l.mixer.get();
        l.block->ffn = l.ffn.get();
        for (const std::string& role : kind.norm_roles) {
            auto it = ls.norms.find(role);
            if (it == ls.norms.end())
                throw ConfigError("layer '" + ls.prefix + "': the block arrangement '" + ls.block + "' needs a norm for the role '" + role + "'");
            l.norms[role] = build_norm(it->second, rt);
            l.block->norms[role] = l.norms[role].get();
        }
        layers_.push_back(std::move(l));
    }
    final_norm_ = build_norm(spec.final_norm, rt);
    head_ = build_head(spec.head, rt);
}

std::vector<std::pair<std::string, Part*>> DecoderModel::owners() const {
    std::vector<std::pair<std::string, Part*>> out;
    out.emplace_back(spec.embedding.get_string("name", ""), embedding_.get());
    for (size_t i = 0; i < layers_.size(); i++) {
        const LayerSpec& ls = spec.layers[i];
        out.emplace_back(ls.prefix + role_name(ls, "mixer"), layers_[i].mixer.get());
        out.emplace_back(ls.prefix + role_name(ls, "ffn"), layers_[i].ffn.get());
        for (auto& n : layers_[i].norms) out.emplace_back(ls.prefix + role_name(ls, n.first), n.second.get());
    }
    out.emplace_back(spec.final_norm.get_string("name", ""), final_norm_.get());
    out.emplace_back(spec.head.get_string("name", ""), head_.get());
    return out;
}

std::vector<std::pair<std::string, TensorDecl>> DecoderModel::tensor_decls() const {
    std::vector<std::pair<std::string, TensorDecl>> decls;
    for (auto& o : owners())
        for (auto& d : o.second->tensors()) decls.emplace_back(o.first + d.first, d.second);
    return decls;
}

void DecoderModel::load_tensors(const std::function<std::unique_ptr<TensorSource>(const std::string&)>& open) {
    for (auto& o : owners()) {
        if (o.second->tensors().empty()) continue;
        std::unique_ptr<TensorSource> src = open(o.first);
        o.second->load(*src);
    }
    if (head_->tied()) head_->tie(*embedding_);
}

std::map<int, CacheRequest> DecoderModel::cache_requests() const {
    std::map<int, CacheRequest> out;
    for (const ScheduleEntry& e : spec.schedule)
        if (e.writes) out[e.cache] = layers_[(size_t)e.layer].mixer->cache_request();
    return out;
}

Mat DecoderModel::forward(const StepContext& ctx, const SequenceCache& cache, const std::vector<const int*>& tables_dev) {
    Device& dev = *rt->dev;
    ResidualStream stream = embedding_->forward(ctx);
    int turn = 0;
    for (const ScheduleEntry& e : spec.schedule) {
        // the layers' activations take turns in two lanes of the step arena: what a layer leaves for the
        // next one (its last output, pending in the stream) is read before this lane's turn comes again
        dev.set_lane(1 + (turn++ & 1), true);
        CacheView view;
        switch (cache.kind_of(e.cache)) {
            case SequenceCache::KV:
                view.kind = CacheView::KV;
                view.kv = cache.kv_view(e.cache, tables_dev[(size_t)cache.group_of(e.cache)]);
                view.kv.writes = e.writes;
                break;
            case SequenceCache::State:
                view.kind = CacheView::State;
                view.st = cache.state_view(e.cache, ctx.slots);
                break;
            default: break;
        }
        layers_[(size_t)e.layer].block->forward(stream, ctx, view, e.writes);
    }
    dev.set_lane(0, false);
    if (ctx.K == 0) {
        Mat none;
        none.cols = spec.vocab_size;
        none.dtype = DType::F32;
        return none;
    }
    Mat y = final_norm_->forward(stream, ctx.want_rows, ctx.K);
    return head_->forward(y, ctx);
}

bool DecoderModel::graph_safe() const {
    for (const Layer& l : layers_)
        if (!l.mixer->graph_safe() || !l.ffn->graph_safe()) return false;
    return true;
}
bool DecoderModel::pad_safe() const {
    if (!graph_safe()) return false;
    for (const Layer& l : layers_)
        if (!l.mixer->pad_safe()) return false;
    return true;
}

}  // namespace illm
