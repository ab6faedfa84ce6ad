#include "cache/cache.h"

#include <algorithm>
#include <set>

extern "C" int illm_poison_pages(void* k, void* v, long long entry_stride_bytes, int n_entries, long long page_bytes,
                                 const int* pages, int n_pages, void* stream);

namespace illm {

// ---- requests

CacheRequest CacheRequest::paged(int n_kv_heads, int head_dim, int window) {
    CacheRequest r;
    r.kind = PagedKV;
    r.n_kv_heads = n_kv_heads;
    r.head_dim = head_dim;
    r.window = window;
    return r;
}
CacheRequest CacheRequest::state(std::vector<long long> shape, DType dtype) {
    CacheRequest r;
    r.kind = FixedState;
    r.shape = std::move(shape);
    r.dtype = dtype;
    return r;
}
bool CacheRequest::operator==(const CacheRequest& o) const {
    return kind == o.kind && n_kv_heads == o.n_kv_heads && head_dim == o.head_dim && window == o.window && shape == o.shape &&
           (kind != FixedState || dtype == o.dtype);
}
Json CacheRequest::to_json() const {
    if (kind == None) return Json();
    Json j = Json::object();
    if (kind == PagedKV) {
        j.set("kind", "kv");
        j.set("n_kv_heads", n_kv_heads);
        j.set("head_dim", head_dim);
        j.set("window", window ? Json(window) : Json());
    } else {
        j.set("kind", "state");
        Json s = Json::array();
        for (long long d : shape) s.push(d);
        j.set("shape", s);
        j.set("dtype", dtype_word(dtype));
    }
    return j;
}
CacheRequest CacheRequest::from_json(const Json& j) {
    if (j.is_null()) return CacheRequest();
    const std::string kind = j.at("kind").is_string() ? j.at("kind").as_string() : "";
    if (kind == "kv")
        return paged((int)j.at("n_kv_heads").as_int(), (int)j.at("head_dim").as_int(),
                     j.at("window").is_int() ? (int)j.at("window").as_int() : 0);
    if (kind == "state") {
        std::vector<long long> shape;
        for (const Json& d : j.at("shape").items()) shape.push_back(d.as_int());
        DType dt = DType::F32;
        const std::string w = j.at("dtype").is_string() ? j.at("dtype").as_string() : "float32";
        if (w == "bfloat16") dt = DType::BF16;
        else if (w == "int32") dt = DType::I32;
        else if (w != "float32") throw CacheError("fixed state of dtype '" + w + "' is not supported (float32, bfloat16, int32)");
        return state(shape, dt);
    }
    throw CacheError("unknown kind of cache request " + j.repr());
}

// ---- IndexPool

IndexPool::IndexPool(int n, std::string what) : n_(n), what_(std::move(what)), held_((size_t)std::max(n, 0), 0) {
    for (int i = n - 1; i >= 0; i--) free_.push_back(i);
}
std::vector<int> IndexPool::alloc(int count) {
    if (count > (int)free_.size())
        throw CacheFull(std::to_string(count) + " " + what_ + "(s) wanted, " + std::to_string(free_.size()) + " of " +
                        std::to_string(n_) + " free");
    std::vector<int> out;
    for (int c = 0; c < count; c++) {
        const int i = free_.back();
        free_.pop_back();
        if (held_[i]) throw CacheError(what_ + " " + std::to_string(i) + " was on the free list while held");
        held_[i] = 1;
        out.push_back(i);
    }
    return out;
}
void IndexPool::free(const std::vector<int>& items) {
    for (int i : items) {
        if (i < 0 || i >= n_) throw CacheError(what_ + " " + std::to_string(i) + " does not exist (0.." + std::to_string(n_ - 1) + ")");
        if (!held_[i]) throw CacheError(what_ + " " + std::to_string(i) + " freed twice (or never handed out)");
        held_[i] = 0;
        free_.push_back(i);
    }
    std::sort(free_.begin(), free_.end(), std::greater<int>());
}
void IndexPool::check() const {
    std::set<int> seen(free_.begin(), free_.end());
    if (seen.size() != free_.size()) throw CacheError("a " + what_ + " is on the free list twice");
    for (int i = 0; i < n_; i++)
        if ((held_[i] != 0) == (seen.count(i) != 0))
            throw CacheError(what_ + " " + std::to_string(i) + " is " + (held_[i] ? "both held and free" : "lost"));
}

// ---- PageLedger

PageLedger::PageLedger(int num_pages, int page_size_, int num_slots, int window_)
        : pool(num_pages, "page"), page_size(page_size_), window(window_), pages((size_t)num_slots), n_logical((size_t)num_slots, 0) {}

static long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }

int PageLedger::pages_needed(int slot, long long new_len) const {
    return (int)std::max<long long>(0, ceil_div(new_len, page_size) - n_logical[slot]);
}
void PageLedger::reserve(int slot, long long new_len) {
    const int want = (int)ceil_div(new_len, page_size), first = n_logical[slot];
    if (want > first) {
        std::vector<int> got = pool.alloc(want - first);
        for (int lp = first; lp < want; lp++) pages[slot][lp] = got[lp - first];
        n_logical[slot] = want;
    }
}
std::vector<int> PageLedger::release_outside_window(int slot, long long seq_len) {
    std::vector<int> gone;
    if (window <= 0) return gone;
    const long long first_needed_pos = seq_len - window + 1;     // oldest key the next token may see
    if (first_needed_pos <= 0) return gone;
    const int first_page = (int)(first_needed_pos / page_size);
    auto& have = pages[slot];
    for (auto it = have.begin(); it != have.end() && it->first < first_page;) {
        gone.push_back(it->second);
        it = have.erase(it);
    }
    pool.free(gone);
    return gone;
}
std::vector<int> PageLedger::release_all(int slot) {
    std::vector<int> gone;
    for (auto& p : pages[slot]) gone.push_back(p.second);
    pool.free(gone);
    pages[slot].clear();
    n_logical[slot] = 0;
    return gone;
}
std::vector<int> PageLedger::release_beyond(int slot, long long seq_len) {
    std::vector<int> gone;
    const int keep = (int)ceil_div(seq_len, page_size);
    auto& have = pages[slot];
    for (auto it = have.lower_bound(keep); it != have.end();) {
        gone.push_back(it->second);
        it = have.erase(it);
    }
    pool.free(gone);
    if (n_logical[slot] > keep) n_logical[slot] = keep;
    return gone;
}
void PageLedger::row(int slot, int width, int* out) const {
    for (int i = 0; i < width; i++) out[i] = -1;
    for (auto& p : pages[slot])
        if (p.first < width) out[p.first] = p.second;
}
void PageLedger::check() const {
    pool.check();
    std::set<int> held;
    size_t n = 0;
    for (auto& d : pages)
        for (auto& p : d) {
            held.insert(p.second);
            n++;
        }
    if (held.size() != n) throw CacheError("a page is held by two sequences");
    if ((int)n != pool.n_held())
        throw CacheError(std::to_string(pool.n_held()) + " pages are out of the pool but sequences hold " + std::to_string(n));
}

// ---- SequenceCache

size_t SequenceCache::bytes_per_token(const std::map<int, CacheRequest>& requests, DType dtype) {
    size_t n = 0;
    for (auto& r : requests)
        if (r.second.kind == CacheRequest::PagedKV) n += 2 * (size_t)r.second.n_kv_heads * r.second.head_dim * dtype_size(dtype);
    return n;
}

SequenceCache::SequenceCache(const std::map<int, CacheRequest>& requests, int num_slots_, int num_pages_, int page_size_,
                             long long max_seq_len_, Device* device, DType dtype, bool poison)
        : num_slots(num_slots_), num_pages(num_pages_), page_size(page_size_), width(0), max_seq_len(max_seq_len_),
          slots(num_slots_ > 0 ? num_slots_ : 0, "slot"), device_(device), dtype_(dtype), poison_(poison) {
    if (num_slots <= 0 || num_pages <= 0 || page_size <= 0) throw CacheError("num_slots, num_pages and page_size must be positive");
    width = (int)ceil_div(max_seq_len, page_size);
    seq_len.assign((size_t)num_slots, 0);
    for (auto& r : requests) {
        const CacheRequest& req = r.second;
        if (req.kind == CacheRequest::None) continue;
        if (req.kind == CacheRequest::PagedKV) {
            int gi = -1;
            for (size_t i = 0; i < paged.size(); i++)
                if (paged[i].request == req) gi = (int)i;
            if (gi < 0) {
                PagedGroup g;
                g.request = req;
                g.ledger.reset(new PageLedger(num_pages, page_size, num_slots, req.window));
                paged.push_back(std::move(g));
                gi = (int)paged.size() - 1;
            }
            where_[r.first] = Loc{KV, gi, (int)paged[gi].entries.size()};
            paged[gi].entries.push_back(r.first);
        } else {
            int gi = -1;
            for (size_t i = 0; i < states.size(); i++)
                if (states[i].request == req) gi = (int)i;
            if (gi < 0) {
                StateGroup g;
                g.request = req;
                states.push_back(std::move(g));
                gi = (int)states.size() - 1;
            }
            where_[r.first] = Loc{State, gi, (int)states[gi].entries.size()};
            states[gi].entries.push_back(r.first);
        }
    }
    for (PagedGroup& g : paged) {
        g.page_bytes = (size_t)g.request.n_kv_heads * page_size * g.request.head_dim * dtype_size(dtype);
        g.entry_bytes = g.page_bytes * num_pages;
    }
    for (StateGroup& g : states) g.entry_bytes = (size_t)num_slots * g.request.elements() * dtype_size(g.request.dtype);
    if (!device_) return;
    // refuse a cache that the device cannot hold, in words, before any allocation
    const size_t need = storage_bytes(), free_b = device_->mem_free();
    if (need > free_b) {
        char msg[256];
        snprintf(msg, sizeof msg, "a cache for %lld tokens needs %.1f GiB, the device has %.1f GiB free: ask for fewer tokens (max_tokens)",
                 (long long)num_pages * page_size, need / 1073741824.0, free_b / 1073741824.0);
        throw CacheError(msg);
    }
    for (PagedGroup& g : paged) {
        g.k = device_->alloc_persistent(g.entry_bytes * g.entries.size(), "the cache's keys", !poison);
        g.v = device_->alloc_persistent(g.entry_bytes * g.entries.size(), "the cache's values", !poison);
        if (poison) {
            check_cuda(cudaMemsetAsync(g.k, 0xFF, g.entry_bytes * g.entries.size(), device_->stream()), "poisoning the cache");
            check_cuda(cudaMemsetAsync(g.v, 0xFF, g.entry_bytes * g.entries.size(), device_->stream()), "poisoning the cache");
        }
    }
    for (StateGroup& g : states) g.state = device_->alloc_persistent(g.entry_bytes * g.entries.size(), "the per-sequence state", true);
}

SequenceCache::~SequenceCache() {
    if (!device_) return;
    for (PagedGroup& g : paged) {
        device_->free_persistent(g.k);
        device_->free_persistent(g.v);
    }
    for (StateGroup& g : states) device_->free_persistent(g.state);
    device_->free_persistent(poison_list_);
    device_->free_pinned(poison_host_);
}

void SequenceCache::poison_pages(PagedGroup& g, const std::vector<int>& pages) {
    if (!poison_ || !device_ || pages.empty() || !g.k) return;
    if ((int)pages.size() > poison_cap_) {
        device_->free_persistent(poison_list_);
        device_->free_pinned(poison_host_);
        poison_cap_ = std::max<int>((int)pages.size(), num_pages);
        poison_list_ = (int*)device_->alloc_persistent((size_t)poison_cap_ * 4, "the list of pages to poison");
        poison_host_ = (int*)device_->alloc_pinned((size_t)poison_cap_ * 4);
    }
    device_->synchronize();            // the staging list is reused: a check option, not a serving path
    std::copy(pages.begin(), pages.end(), poison_host_);
    check_cuda(cudaMemcpyAsync(poison_list_, poison_host_, pages.size() * 4, cudaMemcpyHostToDevice, device_->stream()),
               "uploading the pages to poison");
    check_kernel(illm_poison_pages(g.k, g.v, (long long)g.entry_bytes, (int)g.entries.size(), (long long)g.page_bytes, poison_list_,
                                   (int)pages.size(), device_->stream()),
                 "poison_pages");
}

int SequenceCache::alloc_slot() {
    const int slot = slots.alloc(1)[0];
    seq_len[slot] = 0;
    if (device_)
        for (StateGroup& g : states) {
            const size_t row = (size_t)g.request.elements() * dtype_size(g.request.dtype);
            for (size_t e = 0; e < g.entries.size(); e++)
                check_cuda(cudaMemsetAsync((char*)g.state + e * g.entry_bytes + (size_t)slot * row, 0, row, device_->stream()),
                           "zeroing a sequence's state");
        }
    return slot;
}

void SequenceCache::free_slot(int slot) {
    if (!slots.is_held(slot)) throw CacheError("slot " + std::to_string(slot) + " freed twice (or never handed out)");
    for (PagedGroup& g : paged) poison_pages(g, g.ledger->release_all(slot));
    seq_len[slot] = 0;
    slots.free({slot});
}

void SequenceCache::reset() {
    for (int s = 0; s < num_slots; s++)
        if (slots.is_held(s)) free_slot(s);
}

StepPlan SequenceCache::plan_step(const std::vector<int>& step_slots, const std::vector<int>& q_lens) {
    if (step_slots.size() != q_lens.size() || step_slots.empty())
        throw CacheError("a step needs as many lengths as slots, and at least one");
    if (std::set<int>(step_slots.begin(), step_slots.end()).size() != step_slots.size())
        throw CacheError("a slot appears twice in one step");
    for (size_t i = 0; i < step_slots.size(); i++) {
        const int s = step_slots[i], q = q_lens[i];
        if (!slots.is_held(s)) throw CacheError("slot " + std::to_string(s) + " is not live");
        if (q <= 0) throw CacheError("slot " + std::to_string(s) + ": a step must bring at least one token");
        if (seq_len[s] + q > max_seq_len)
            throw CacheError("slot " + std::to_string(s) + ": " + std::to_string(seq_len[s]) + " + " + std::to_string(q) +
                             " tokens exceed the maximum sequence length " + std::to_string(max_seq_len));
    }
    for (PagedGroup& g : paged) {
        long long need = 0;
        for (size_t i = 0; i < step_slots.size(); i++) need += g.ledger->pages_needed(step_slots[i], seq_len[step_slots[i]] + q_lens[i]);
        if (need > g.ledger->pool.n_free())
            throw CacheFull("the step needs " + std::to_string(need) + " more pages, " + std::to_string(g.ledger->pool.n_free()) +
                            " of " + std::to_string(g.ledger->pool.n()) + " are free");
    }
    StepPlan plan;
    plan.slots = step_slots;
    plan.q_lens = q_lens;
    for (int s : step_slots) plan.past.push_back(seq_len[s]);
    for (PagedGroup& g : paged) {
        std::vector<int> tab(step_slots.size() * (size_t)width);
        for (size_t i = 0; i < step_slots.size(); i++) {
            g.ledger->reserve(step_slots[i], seq_len[step_slots[i]] + q_lens[i]);
            g.ledger->row(step_slots[i], width, tab.data() + i * (size_t)width);
        }
        plan.tables.push_back(std::move(tab));
    }
    return plan;
}

void SequenceCache::commit_step(const StepPlan& plan) {
    for (size_t i = 0; i < plan.slots.size(); i++) {
        const int s = plan.slots[i];
        seq_len[s] += plan.q_lens[i];
        for (PagedGroup& g : paged) poison_pages(g, g.ledger->release_outside_window(s, seq_len[s]));
    }
}

void SequenceCache::abandon_step(const StepPlan& plan) {
    for (int s : plan.slots)
        if (slots.is_held(s))
            for (PagedGroup& g : paged) poison_pages(g, g.ledger->release_beyond(s, seq_len[s]));
}

void SequenceCache::check() const {
    slots.check();
    for (const PagedGroup& g : paged) {
        g.ledger->check();
        for (int s = 0; s < num_slots; s++)
            if (!slots.is_held(s) && !g.ledger->pages[s].empty()) throw CacheError("free slot " + std::to_string(s) + " still holds pages");
    }
}

SequenceCache::Where SequenceCache::kind_of(int entry) const {
    auto it = where_.find(entry);
    return it == where_.end() ? Absent : it->second.kind;
}
int SequenceCache::group_of(int entry) const {
    auto it = where_.find(entry);
    return it == where_.end() ? -1 : it->second.group;
}

KVView SequenceCache::kv_view(int entry, const int* table_dev) const {
    auto it = where_.find(entry);
    if (it == where_.end() || it->second.kind != KV)
        throw CacheError("cache entry " + std::to_string(entry) + " holds fixed state, not keys and values");
    const PagedGroup& g = paged[it->second.group];
    KVView v;
    v.k = g.k ? (char*)g.k + (size_t)it->second.index * g.entry_bytes : nullptr;
    v.v = g.v ? (char*)g.v + (size_t)it->second.index * g.entry_bytes : nullptr;
    v.block_table = table_dev;
    v.width = width;
    v.num_pages = num_pages;
    v.page_size = page_size;
    v.window = g.request.window;
    v.n_kv_heads = g.request.n_kv_heads;
    v.head_dim = g.request.head_dim;
    v.dtype = dtype_;
    return v;
}

StateView SequenceCache::state_view(int entry, const int* slots_dev) const {
    auto it = where_.find(entry);
    if (it == where_.end() || it->second.kind != State)
        throw CacheError("cache entry " + std::to_string(entry) + " holds keys and values, not fixed state");
    const StateGroup& g = states[it->second.group];
    StateView v;
    v.state = g.state ? (char*)g.state + (size_t)it->second.index * g.entry_bytes : nullptr;
    v.slots = slots_dev;
    v.num_slots = num_slots;
    v.elements = g.request.elements();
    v.dtype = g.request.dtype;
    return v;
}

std::vector<int> SequenceCache::pages_free() const {
    std::vector<int> out;
    for (const PagedGroup& g : paged) out.push_back(g.ledger->pool.n_free());
    return out;
}
size_t SequenceCache::storage_bytes() const {
    size_t n = 0;
    for (const PagedGroup& g : paged) n += 2 * g.entry_bytes * g.entries.size();
    return n;
}

}  // namespace illm
