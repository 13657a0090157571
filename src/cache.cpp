// Page pools, block tables and the scheduler of the C++ host.  Decision for decision the same as
// vllm-cpp_b200/cache/manager.py and vllm-cpp_b200/engine/scheduler.py (whose headers say where and why they
// differ from src/core/block_manager.cpp and src/core/scheduler.cpp of the reference).
#include <algorithm>

#include "host.hpp"

namespace vllm {
namespace host {

static int cdiv(int a, int b) { return (a + b - 1) / b; }

// ------------------------------------------------------------------------------------------- BlockPool
BlockPool::BlockPool(int num_blocks) : refs_(num_blocks, 0) {
    if (num_blocks <= 0) throw Error("a page pool needs at least one page");
    for (int b = num_blocks - 1; b >= 0; --b) free_.push_back(b);      // page 0 is handed out first
}

int BlockPool::acquire() {
    if (free_.empty()) return -1;
    const int b = free_.back();
    free_.pop_back();
    refs_[b] = 1;
    return b;
}

void BlockPool::release(int block) {
    if (block < 0 || block >= (int)refs_.size()) throw Error("page id " + std::to_string(block) + " outside the pool");
    if (refs_[block] <= 0) throw Error("page " + std::to_string(block) + " released while not held (freed twice?)");
    if (--refs_[block] == 0) free_.push_back(block);                   // LIFO: the next one handed out
}

// ---------------------------------------------------------------------------------------- CacheManager
CacheManager::CacheManager(const std::vector<int>& group_windows, int page_size, int num_pages, int max_num_seqs)
    : windows_(group_windows), page_(page_size), num_pages_(num_pages) {
    if (page_size <= 0) throw Error("KV block size must be greater than zero");
    for (size_t g = 0; g < windows_.size(); ++g) pools_.emplace_back(num_pages);
    for (int s = max_num_seqs - 1; s >= 0; --s) free_slots_.push_back(s);
}

void CacheManager::add_request(int64_t id) {
    if (reqs_.count(id)) throw Error("request " + std::to_string(id) + " is already live");
    if (free_slots_.empty()) throw Error("all request slots are taken");
    Req r;
    r.tables.resize(windows_.size());
    r.released.assign(windows_.size(), 0);
    r.slot = free_slots_.back();
    free_slots_.pop_back();
    reqs_.emplace(id, std::move(r));
}

bool CacheManager::can_append(int64_t id, int n_new) const {
    const Req& r = reqs_.at(id);
    const int want = cdiv(r.num_tokens + n_new, page_);
    for (size_t g = 0; g < pools_.size(); ++g)
        if (pools_[g].num_free() < std::max(0, want - (int)r.tables[g].size())) return false;
    return true;
}

int CacheManager::max_appendable(int64_t id) const {
    const Req& r = reqs_.at(id);
    if (pools_.empty()) return 1 << 30;
    int best = 1 << 30;
    for (size_t g = 0; g < pools_.size(); ++g)
        best = std::min(best, ((int)r.tables[g].size() + pools_[g].num_free()) * page_);
    return best - r.num_tokens;
}

int CacheManager::max_appendable_new() const { return pools_.empty() ? 1 << 30 : num_free_pages() * page_; }

void CacheManager::reserve(int64_t id, int n_new) {
    Req& r = reqs_.at(id);
    if (!can_append(id, n_new))
        throw Error("request " + std::to_string(id) + " needs more pages for " + std::to_string(n_new) + " tokens than are free");
    const int want = cdiv(r.num_tokens + n_new, page_);
    for (size_t g = 0; g < pools_.size(); ++g)
        while ((int)r.tables[g].size() < want) r.tables[g].push_back(pools_[g].acquire());
}

void CacheManager::commit(int64_t id, int n_new) {
    Req& r = reqs_.at(id);
    r.num_tokens += n_new;
    for (size_t g = 0; g < pools_.size(); ++g) {
        if ((size_t)r.num_tokens > r.tables[g].size() * (size_t)page_) throw Error("a request holds more tokens than pages");
        const int w = windows_[g];
        if (w <= 0) continue;
        // keys at positions <= num_tokens - w are never read again
        const int dead = std::min<int>(std::max(0, (r.num_tokens - w + 1) / page_), (int)r.tables[g].size());
        for (int b = r.released[g]; b < dead; ++b) {
            pools_[g].release(r.tables[g][b]);
            r.tables[g][b] = RELEASED;
        }
        r.released[g] = std::max(r.released[g], dead);
    }
}

void CacheManager::free_request(int64_t id) {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) throw Error("request " + std::to_string(id) + " is not live");
    for (size_t g = 0; g < pools_.size(); ++g)
        for (auto b = it->second.tables[g].rbegin(); b != it->second.tables[g].rend(); ++b)
            if (*b != RELEASED) pools_[g].release(*b);
    free_slots_.push_back(it->second.slot);
    reqs_.erase(it);
}

int CacheManager::num_free_pages() const {
    int best = num_pages_;
    for (const auto& p : pools_) best = std::min(best, p.num_free());
    return best;
}

// ------------------------------------------------------------------------------------------- Scheduler
Scheduler::Scheduler(CacheManager& cache, const EngineConfig& cfg)
    : cache_(cache), max_seqs_(cfg.max_num_seqs), max_batched_(cfg.max_num_batched_tokens),
      max_portion_(cfg.max_tokens_per_step), to_front_(cfg.preempted_to_front) {}

void Scheduler::add_request(Sequence* seq) {
    if (seq->prompt.empty()) throw std::invalid_argument("prompt must contain at least one token");
    const size_t planned = seq->prompt.size() + seq->params.max_tokens;
    if ((planned + cache_.page_size() - 1) / cache_.page_size() > (size_t)cache_.num_pages())
        throw std::invalid_argument("request exceeds total KV cache block capacity");
    waiting_.push_back(seq);
}

void Scheduler::finish(Sequence* seq) {
    seq->finished = true;
    auto r = std::find(running_.begin(), running_.end(), seq);
    if (r != running_.end()) {
        running_.erase(r);
        cache_.free_request(seq->seq_id);
        return;
    }
    auto w = std::find(waiting_.begin(), waiting_.end(), seq);
    if (w != waiting_.end()) waiting_.erase(w);
}

Sequence* Scheduler::newest_running(const Sequence* newer_than) const {
    if (running_.empty() || running_.back() == newer_than) return nullptr;
    return running_.back();
}

int Scheduler::preempt(Sequence* victim, std::vector<ScheduledItem>& items) {
    int freed = 0;
    for (auto it = items.begin(); it != items.end();) {
        if (it->seq == victim) { freed += it->count; it = items.erase(it); }
        else ++it;
    }
    running_.erase(std::find(running_.begin(), running_.end(), victim));
    cache_.free_request(victim->seq_id);
    victim->num_processed = 0;
    victim->needs_recompute = true;
    ++victim->num_preemptions;
    ++preemptions_;
    if (to_front_) waiting_.push_front(victim);
    else waiting_.push_back(victim);
    return freed;
}

std::vector<ScheduledItem> Scheduler::schedule() {
    for (;;) {
        std::vector<ScheduledItem> items = schedule_once();
        if (!items.empty() || running_.empty()) return items;
        // requests are running but none got a token: take the newest one's pages so that the others can go on
        Sequence* victim = newest_running(nullptr);
        if (!victim || (running_.size() == 1 && cache_.max_appendable(victim->seq_id) <= 0)) return items;
        preempt(victim, items);
    }
}

std::vector<ScheduledItem> Scheduler::schedule_once() {
    std::vector<ScheduledItem> items;
    long budget = (long)max_batched_, portion_budget = (long)max_portion_;
    // 1. requests that decode: one token each, oldest first; may preempt the newest
    for (size_t i = 0; i < running_.size(); ++i) {
        Sequence* seq = running_[i];
        if (seq->remaining() != 1 || budget <= 0) continue;
        while (!cache_.can_append(seq->seq_id, 1)) {
            Sequence* victim = newest_running(seq);
            if (!victim) break;                       // nobody newer to take pages from: sit this step out
            budget += preempt(victim, items);
        }
        if (cache_.can_append(seq->seq_id, 1)) {
            cache_.reserve(seq->seq_id, 1);
            items.push_back({seq, seq->num_processed, 1, true});
            --budget;
        }
    }
    // 2. running requests still reading their prompt (or replaying), in arrival order
    for (Sequence* seq : running_) {
        if (seq->remaining() <= 1 || budget <= 0 || portion_budget <= 0) continue;
        const long n = std::min<long>({(long)seq->remaining(), budget, portion_budget, (long)cache_.max_appendable(seq->seq_id)});
        if (n <= 0) continue;
        cache_.reserve(seq->seq_id, (int)n);
        items.push_back({seq, seq->num_processed, (int)n, n == seq->remaining()});
        budget -= n;
        if (n > 1) portion_budget -= n;
    }
    // 3. admissions, strictly in queue order
    while (!waiting_.empty() && running_.size() < max_seqs_ && budget > 0 && cache_.has_free_slot()) {
        Sequence* seq = waiting_.front();
        const long n = std::min<long>({(long)seq->remaining(), budget, seq->remaining() > 1 ? portion_budget : 1L});
        if (n <= 0 || cache_.max_appendable_new() < n) break;
        waiting_.pop_front();
        cache_.add_request(seq->seq_id);
        cache_.reserve(seq->seq_id, (int)n);
        seq->needs_recompute = false;
        running_.push_back(seq);
        items.push_back({seq, 0, (int)n, n == seq->remaining()});
        budget -= n;
        if (n > 1) portion_budget -= n;
    }
    return items;
}

}  // namespace host
}  // namespace vllm
