// A C face of the C++ cache manager and scheduler alone, without a device: tests drive it beside the Python
// scheduler with the same random workload and compare every decision.  Built into a small library of its
// own (cache.cpp + this file; no CUDA call is made).
#include <cstring>
#include <map>
#include <memory>
#include <string>

#include "host.hpp"

#define SIM_EXPORT extern "C" __attribute__((visibility("default")))

namespace {
using namespace vllm::host;
struct Sim {
    vllm::EngineConfig cfg;
    std::unique_ptr<CacheManager> cache;
    std::unique_ptr<Scheduler> sched;
    std::map<long long, std::unique_ptr<Sequence>> seqs;
};
thread_local std::string g_error;
}  // namespace

namespace vllm { namespace host {
void cuda_check(cudaError_t, const char*) {}          // cache.cpp needs neither; util.cpp is not linked here
void kernel_check(int, const char*) {}
} }

SIM_EXPORT const char* vcbs_last_error() { return g_error.c_str(); }

// windows: one entry per cache group (0: all keys).
SIM_EXPORT void* vcbs_create(const int* windows, int n_groups, int page_size, int num_pages, int max_num_seqs,
                             int max_num_batched_tokens, int max_tokens_per_step, int preempted_to_front) {
    auto* s = new Sim;
    s->cfg.max_num_seqs = (size_t)max_num_seqs;
    s->cfg.max_num_batched_tokens = (size_t)max_num_batched_tokens;
    s->cfg.max_tokens_per_step = (size_t)max_tokens_per_step;
    s->cfg.preempted_to_front = preempted_to_front != 0;
    s->cache.reset(new CacheManager(std::vector<int>(windows, windows + n_groups), page_size, num_pages, max_num_seqs));
    s->sched.reset(new Scheduler(*s->cache, s->cfg));
    return s;
}

SIM_EXPORT void vcbs_destroy(void* h) { delete static_cast<Sim*>(h); }

// 0, or -1 if the scheduler refuses the request (it can never fit).
SIM_EXPORT int vcbs_add_request(void* h, long long id, int prompt_len, int max_tokens) {
    Sim& s = *static_cast<Sim*>(h);
    std::unique_ptr<Sequence> q(new Sequence);
    q->seq_id = id;
    q->prompt.assign((size_t)prompt_len, 1);
    q->params.max_tokens = (size_t)max_tokens;
    try {
        s.sched->add_request(q.get());
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
    s.seqs[id] = std::move(q);
    return 0;
}

// One schedule() and what a step does with it: tokens committed, a token appended to every item that samples,
// requests that reach max_tokens finished.  Writes (id, start, count, samples) per item; returns their number.
SIM_EXPORT int vcbs_step(void* h, long long* ids, int* starts, int* counts, int* samples, int cap) {
    Sim& s = *static_cast<Sim*>(h);
    try {
        const std::vector<ScheduledItem> items = s.sched->schedule();
        int n = 0;
        for (const ScheduledItem& it : items) {
            if (n >= cap) throw Error("more items than room");
            ids[n] = it.seq->seq_id; starts[n] = it.start; counts[n] = it.count; samples[n] = it.samples ? 1 : 0;
            ++n;
        }
        for (const ScheduledItem& it : items) {
            s.cache->commit(it.seq->seq_id, it.count);
            it.seq->num_processed += it.count;
        }
        for (const ScheduledItem& it : items) {
            if (!it.samples) continue;
            it.seq->output.push_back(7);
            if (it.seq->output.size() >= it.seq->params.max_tokens) {
                const long long id = it.seq->seq_id;
                s.sched->finish(it.seq);
                s.seqs.erase(id);
            }
        }
        return n;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

SIM_EXPORT void vcbs_abort(void* h, long long id) {
    Sim& s = *static_cast<Sim*>(h);
    auto it = s.seqs.find(id);
    if (it == s.seqs.end()) return;
    s.sched->finish(it->second.get());
    s.seqs.erase(it);
}

SIM_EXPORT int vcbs_free_pages(void* h) { return static_cast<Sim*>(h)->cache->num_free_pages(); }
SIM_EXPORT long long vcbs_preemptions(void* h) { return (long long)static_cast<Sim*>(h)->sched->num_preemptions(); }
SIM_EXPORT int vcbs_pending(void* h) { return static_cast<Sim*>(h)->sched->has_pending_work() ? 1 : 0; }
// The block table of a live request in one group: writes up to cap entries, returns the table's length (-1: not live).
SIM_EXPORT int vcbs_table(void* h, long long id, int group, int* out, int cap) {
    Sim& s = *static_cast<Sim*>(h);
    if (!s.cache->live(id)) return -1;
    const std::vector<int>& t = s.cache->table(id, group);
    for (int i = 0; i < (int)t.size() && i < cap; ++i) out[i] = t[i];
    return (int)t.size();
}
