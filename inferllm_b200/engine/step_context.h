// Building the device-side description of a step (StepContext) from the cache's plan: all index
// arrays go into one pinned staging buffer and one host-to-device copy.  Shared by the engine and by
// the sandbox in which single parts are run.
#pragma once
#include <vector>

#include "cache/cache.h"
#include "parts/parts.h"

namespace illm {

class StepContextBuilder {
public:
    StepContextBuilder(Device* dev, Runtime* rt);
    ~StepContextBuilder();
    // int32 elements of a step's buffer
    static size_t ints(int T, int B, int K, size_t n_groups, int width);
    // `into`: a device buffer of an earlier step of the same shape to fill again (the static input of
    // a captured graph); nullptr takes a fresh one from the step arena.  tables_dev gets, per paged
    // group of the cache, the device address of the step's page table [B, width].
    StepContext build(const SequenceCache& cache, const StepPlan& plan, const std::vector<int>& ids, const std::vector<int>& want_rows,
                      int* into, std::vector<const int*>* tables_dev);
    size_t last_upload_bytes = 0;

private:
    struct Stage { int* host = nullptr; size_t cap = 0; cudaEvent_t busy = nullptr; bool used = false; };
    Device* dev_;
    Runtime* rt_;
    Stage stages_[4];
    int next_ = 0;
};

}  // namespace illm
