// The cache of a model: a slot per sequence, paged keys and values per group of layers, and
// per-sequence state of fixed size.
//
// Layers ask for storage through their mixer's cache_request(): PagedKV(kv heads, head size,
// window) or FixedState(shape, dtype).  Cache entries (one per writing entry of the model's
// schedule) with equal requests form a group; every group has storage, a page pool and page tables
// of its own, so groups with different needs (all keys, a window of them, another head size) live
// side by side.  Device storage of a paged group: k, v : [entries, pages, kv heads, page_size,
// head_dim] in the engine's dtype; of a state group: [entries, slots, elements].
//
// Life of a sequence: alloc_slot() (state zeroed) -> plan_step() / commit_step() once per step
// (pages are reserved before the step runs and the length advances after it; abandon_step() gives
// back what a step that failed had reserved) -> free_slot() (pages and slot go back to the pools
// for the next sequence).  Nothing of the bookkeeping touches the device; its invariants (no slot
// or page lost, held twice or freed twice) are checked on every call.
//
// The reference has one implicit sequence per model: KvStorage keeps a single index of the tokens
// stored (m_store_id, src/core/kvstorage.h:40-49) in one growable float32 tensor per layer
// (src/core/kvstotage.cpp:53-76), checks it against the caller's nr_past (src/core/op.cpp:349-351),
// and reset_id rewinds it (src/core/kvstorage.h:43-46).  Here the length is the cache's own and the
// caller passes none.
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "device/device.h"
#include "util/error.h"
#include "util/json.h"

namespace illm {

// What a mixer may ask of the cache.
struct CacheRequest {
    enum Kind { None, PagedKV, FixedState } kind = None;
    // PagedKV: keys and values of every position (window 0) or of the last `window` positions
    int n_kv_heads = 0, head_dim = 0, window = 0;
    // FixedState: `elements` values of `dtype` per sequence, zeroed when a slot is handed out
    std::vector<long long> shape;
    DType dtype = DType::F32;

    static CacheRequest paged(int n_kv_heads, int head_dim, int window = 0);
    static CacheRequest state(std::vector<long long> shape, DType dtype = DType::F32);
    long long elements() const { long long n = 1; for (long long s : shape) n *= s; return n; }
    bool operator==(const CacheRequest& o) const;
    Json to_json() const;
    static CacheRequest from_json(const Json& j);
};

// A pool of the integers 0..n-1.  Lowest index first, so that reuse is deterministic.
class IndexPool {
public:
    IndexPool(int n, std::string what);
    int n() const { return n_; }
    int n_free() const { return (int)free_.size(); }
    int n_held() const { return n_ - (int)free_.size(); }
    std::vector<int> alloc(int count = 1);          // CacheFull if fewer are free
    void free(const std::vector<int>& items);       // CacheError for an index freed twice or unknown
    bool is_held(int i) const { return i >= 0 && i < n_ && held_[i]; }
    void check() const;                             // every index is either free exactly once or held

private:
    int n_;
    std::string what_;
    std::vector<int> free_;       // descending, so that pop_back gives the lowest
    std::vector<char> held_;
};

// The pages of one group of layers: a pool and, per slot, the pages it holds by logical page number.
// A windowed group gives pages back once every position in them has left the window of all future
// queries; their logical entry then reads -1.
class PageLedger {
public:
    PageLedger(int num_pages, int page_size, int num_slots, int window = 0);
    int pages_needed(int slot, long long new_len) const;
    void reserve(int slot, long long new_len);                        // pages for positions 0..new_len-1 (those not yet released)
    std::vector<int> release_outside_window(int slot, long long seq_len);   // after a step; returns the pages given back
    std::vector<int> release_all(int slot);
    std::vector<int> release_beyond(int slot, long long seq_len);     // pages reserved for positions >= seq_len (a step that failed)
    void row(int slot, int width, int* out) const;                    // logical -> physical table, -1 = no page
    void check() const;
    IndexPool pool;
    int page_size, window;
    std::vector<std::map<int, int>> pages;     // per slot: logical page -> physical page
    std::vector<int> n_logical;                // logical pages ever reserved by the slot's sequence
};

struct StepPlan {
    std::vector<int> slots, q_lens;
    std::vector<long long> past;                       // length of each sequence before the step
    std::vector<std::vector<int>> tables;              // per paged group: [B * width]
};

// What a mixer sees of its cache entry during one step.
struct KVView {
    void* k = nullptr;          // [pages, kv heads, page_size, head_dim] of this entry
    void* v = nullptr;
    const int* block_table = nullptr;   // int32 [B, width] on the device, rows in the order of the step's sequences
    int width = 0, num_pages = 0, page_size = 0, window = 0, n_kv_heads = 0, head_dim = 0;
    DType dtype = DType::BF16;
    bool writes = true;
};
struct StateView {
    void* state = nullptr;      // [slots, elements] of this entry
    const int* slots = nullptr; // int32 [B] on the device: the slots of the step's sequences
    int num_slots = 0;
    long long elements = 0;
    DType dtype = DType::F32;
};

class SequenceCache {
public:
    // `requests`: cache entry number -> request.  `device == nullptr` keeps the cache host-only
    // (bookkeeping without device storage).  `poison`: pages that go back to the pool, and pages that
    // nobody has held yet, are filled with NaN, so that a kernel that reads a page its sequence does
    // not hold shows it.
    SequenceCache(const std::map<int, CacheRequest>& requests, int num_slots, int num_pages, int page_size,
                  long long max_seq_len, Device* device, DType dtype, bool poison = false);
    ~SequenceCache();

    int alloc_slot();
    void free_slot(int slot);
    void reset();
    StepPlan plan_step(const std::vector<int>& slots, const std::vector<int>& q_lens);   // all or nothing
    void commit_step(const StepPlan& plan);
    void abandon_step(const StepPlan& plan);     // the step did not run: its reservations go back
    void check() const;

    struct PagedGroup {
        CacheRequest request;
        std::vector<int> entries;
        std::unique_ptr<PageLedger> ledger;
        void *k = nullptr, *v = nullptr;
        size_t entry_bytes = 0, page_bytes = 0;
    };
    struct StateGroup {
        CacheRequest request;
        std::vector<int> entries;
        void* state = nullptr;
        size_t entry_bytes = 0;
    };
    enum Where { Absent, KV, State };
    Where kind_of(int entry) const;
    int group_of(int entry) const;
    KVView kv_view(int entry, const int* table_dev) const;
    StateView state_view(int entry, const int* slots_dev) const;

    std::vector<int> pages_free() const;
    size_t storage_bytes() const;
    // bytes of cache that one token of a sequence takes (all paged groups)
    static size_t bytes_per_token(const std::map<int, CacheRequest>& requests, DType dtype);

    int num_slots, num_pages, page_size, width;
    long long max_seq_len;
    IndexPool slots;
    std::vector<long long> seq_len;
    std::vector<PagedGroup> paged;
    std::vector<StateGroup> states;

private:
    void poison_pages(PagedGroup& g, const std::vector<int>& pages);
    struct Loc { Where kind; int group, index; };
    std::map<int, Loc> where_;
    Device* device_;
    DType dtype_;
    bool poison_;
    int* poison_list_ = nullptr;      // device staging of page numbers to poison
    int* poison_host_ = nullptr;
    int poison_cap_ = 0;
};

}  // namespace illm
