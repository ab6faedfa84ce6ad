#include "engine/step_context.h"

#include <algorithm>

namespace illm {

StepContextBuilder::StepContextBuilder(Device* dev, Runtime* rt) : dev_(dev), rt_(rt) {
    for (Stage& s : stages_) check_cuda(cudaEventCreateWithFlags(&s.busy, cudaEventDisableTiming), "cudaEventCreate");
}
StepContextBuilder::~StepContextBuilder() {
    for (Stage& s : stages_) {
        if (s.host) dev_->free_pinned(s.host);
        if (s.busy) cudaEventDestroy(s.busy);
    }
}

static size_t pad4(size_t n) { return (n + 3) / 4 * 4; }      // keeps every array 16-byte aligned

size_t StepContextBuilder::ints(int T, int B, int K, size_t n_groups, int width) {
    return 3 * pad4((size_t)T) + pad4((size_t)K) + 2 * pad4((size_t)B) + pad4((size_t)B + 1) + n_groups * pad4((size_t)B * width);
}

StepContext StepContextBuilder::build(const SequenceCache& cache, const StepPlan& plan, const std::vector<int>& ids,
                                      const std::vector<int>& want_rows, int* into, std::vector<const int*>* tables_dev) {
    const int B = (int)plan.slots.size(), K = (int)want_rows.size();
    int T = 0, max_q = 0;
    long long max_len = 0;
    for (int i = 0; i < B; i++) {
        T += plan.q_lens[i];
        max_q = std::max(max_q, plan.q_lens[i]);
        max_len = std::max(max_len, plan.past[i] + plan.q_lens[i]);
    }
    const size_t total = ints(T, B, K, cache.paged.size(), cache.width);
    // one asynchronous copy for all of a step's index arrays, from a small ring of pinned staging
    // buffers: the host may prepare the next steps while the GPU still runs this one, and waits only
    // when it comes back to a buffer whose copy has not left yet
    Stage& st = stages_[next_];
    next_ = (next_ + 1) % 4;
    if (st.used) check_cuda(cudaEventSynchronize(st.busy), "waiting for a staging buffer");
    if (st.cap < total) {
        if (st.host) dev_->free_pinned(st.host);
        st.cap = std::max<size_t>(total, 4096);
        st.host = (int*)dev_->alloc_pinned(st.cap * sizeof(int));
    }
    int* h = st.host;
    size_t off = 0;
    const size_t o_ids = off;      off += pad4((size_t)T);
    const size_t o_pos = off;      off += pad4((size_t)T);
    const size_t o_seq = off;      off += pad4((size_t)T);
    const size_t o_want = off;     off += pad4((size_t)K);
    const size_t o_slots = off;    off += pad4((size_t)B);
    const size_t o_lens = off;     off += pad4((size_t)B);
    const size_t o_cu = off;       off += pad4((size_t)B + 1);
    std::copy(ids.begin(), ids.end(), h + o_ids);
    int t = 0;
    h[o_cu] = 0;
    for (int b = 0; b < B; b++) {
        for (int i = 0; i < plan.q_lens[b]; i++, t++) {
            h[o_pos + t] = (int)(plan.past[b] + i);
            h[o_seq + t] = b;
        }
        h[o_slots + b] = plan.slots[b];
        h[o_lens + b] = (int)(plan.past[b] + plan.q_lens[b]);
        h[o_cu + b + 1] = t;
    }
    std::copy(want_rows.begin(), want_rows.end(), h + o_want);
    std::vector<size_t> o_tab;
    for (const std::vector<int>& tab : plan.tables) {
        o_tab.push_back(off);
        std::copy(tab.begin(), tab.end(), h + off);
        off += pad4(tab.size());
    }
    int* buf = into ? into : dev_->alloc_n<int>(total);
    check_cuda(cudaMemcpyAsync(buf, h, total * sizeof(int), cudaMemcpyHostToDevice, dev_->stream()), "uploading a step's index arrays");
    check_cuda(cudaEventRecord(st.busy, dev_->stream()), "cudaEventRecord");
    st.used = true;
    last_upload_bytes = total * sizeof(int);

    StepContext ctx;
    ctx.ids = buf + o_ids;
    ctx.token_pos = buf + o_pos;
    ctx.token_seq = buf + o_seq;
    ctx.want_rows = buf + o_want;
    ctx.slots = buf + o_slots;
    ctx.seq_lens = buf + o_lens;
    ctx.cu_q = buf + o_cu;
    ctx.T = T;
    ctx.B = B;
    ctx.K = K;
    ctx.max_q = max_q;
    ctx.max_len = max_len;
    ctx.max_seq_len = cache.max_seq_len;
    ctx.is_decode = max_q == 1;
    ctx.err = dev_->step_error_word();
    ctx.dev = dev_;
    ctx.rt = rt_;
    ctx.q_lens = plan.q_lens;
    ctx.host_slots = plan.slots;
    ctx.past = plan.past;
    tables_dev->clear();
    for (size_t o : o_tab) tables_dev->push_back(buf + o);
    return ctx;
}

}  // namespace illm
