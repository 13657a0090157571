// A plain C face of vllm::Engine for callers without a C++ compiler at hand (the tests drive it through
// ctypes).  Every function returns a negative number or null on failure and leaves the reason in
// vcbe_last_error().
#include <cstring>
#include <stdexcept>
#include <string>

#include "vllm/vllm.hpp"

#define VCBE_EXPORT extern "C" __attribute__((visibility("default")))

namespace {
thread_local std::string g_error;
template <typename F> auto guarded(F f, decltype(f()) on_error) -> decltype(f()) {
    try {
        return f();
    } catch (const std::exception& e) {
        g_error = e.what();
        return on_error;
    }
}
}  // namespace

VCBE_EXPORT const char* vcbe_last_error() { return g_error.c_str(); }

VCBE_EXPORT void* vcbe_create(const char* model_path, const char* model_arch, const char* dtype, int block_size, int num_gpu_blocks,
                              int max_num_seqs, int max_model_len, int max_num_batched_tokens, int max_tokens_per_step,
                              unsigned long long seed, int gpu_memory_utilization, int preempted_to_front, int fused_decode_tokens,
                              const char* load_format) {
    vllm::EngineConfig cfg;
    cfg.model_path = model_path ? model_path : "";
    cfg.model_arch = model_arch ? model_arch : "";
    cfg.dtype = dtype ? dtype : "bfloat16";
    cfg.block_size = (size_t)block_size;
    cfg.num_gpu_blocks = (size_t)num_gpu_blocks;
    cfg.max_num_seqs = (size_t)max_num_seqs;
    cfg.max_model_len = (size_t)max_model_len;
    cfg.max_num_batched_tokens = (size_t)max_num_batched_tokens;
    cfg.max_tokens_per_step = (size_t)max_tokens_per_step;
    cfg.seed = seed;
    cfg.gpu_memory_utilization = (size_t)gpu_memory_utilization;
    cfg.preempted_to_front = preempted_to_front != 0;
    cfg.fused_decode_tokens = (size_t)fused_decode_tokens;
    if (load_format && *load_format) cfg.load_format = load_format;
    auto* e = new vllm::Engine(cfg);
    if (!e->initialize()) {
        g_error = e->last_error();
        delete e;
        return nullptr;
    }
    return e;
}

VCBE_EXPORT void vcbe_destroy(void* h) { delete static_cast<vllm::Engine*>(h); }

// n_stop < 0: stop on the model's eos ids.  temperature, top_p, repetition_penalty < 0 and top_k == 0: the engine's default.
VCBE_EXPORT long long vcbe_add_request(void* h, const int* ids, int n, int max_tokens, float temperature, float top_p, int top_k,
                                       float repetition_penalty, int has_seed, unsigned long long seed, int ignore_eos,
                                       const int* stop_ids, int n_stop) {
    return guarded([&]() -> long long {
        vllm::SamplingParams sp;
        sp.max_tokens = (size_t)max_tokens;
        sp.temperature = temperature;
        sp.top_p = top_p;
        sp.top_k = top_k;
        sp.repetition_penalty = repetition_penalty;
        sp.has_seed = has_seed != 0;
        sp.seed = seed;
        sp.ignore_eos = ignore_eos != 0;
        if (n_stop >= 0) {
            sp.default_stop_ids = false;
            sp.stop_token_ids.assign(stop_ids, stop_ids + n_stop);
        }
        return static_cast<vllm::Engine*>(h)->add_request(std::vector<vllm::TokenId>(ids, ids + n), sp);
    }, -1);
}

// One step; up to `cap` outputs: the request, its new token, 0 / 1 (stop) / 2 (length).  Returns their number.
VCBE_EXPORT int vcbe_step(void* h, long long* seq_ids, int* tokens, int* finished, int cap) {
    return guarded([&]() -> int {
        const auto outs = static_cast<vllm::Engine*>(h)->step();
        int n = 0;
        for (const auto& o : outs) {
            if (n >= cap) throw std::runtime_error("more outputs than the caller has room for");
            seq_ids[n] = o.seq_id;
            tokens[n] = o.tokens[0];
            finished[n] = !o.finished ? 0 : o.finish_reason == "stop" ? 1 : 2;
            ++n;
        }
        return n;
    }, -1);
}

VCBE_EXPORT int vcbe_has_pending_work(void* h) { return static_cast<vllm::Engine*>(h)->has_pending_work() ? 1 : 0; }
VCBE_EXPORT void vcbe_abort_request(void* h, long long id) { static_cast<vllm::Engine*>(h)->abort_request(id); }
VCBE_EXPORT int vcbe_vocab_size(void* h) { return static_cast<vllm::Engine*>(h)->vocab_size(); }
VCBE_EXPORT long long vcbe_num_free_blocks(void* h) { return (long long)static_cast<vllm::Engine*>(h)->num_free_blocks(); }
VCBE_EXPORT long long vcbe_num_total_blocks(void* h) { return (long long)static_cast<vllm::Engine*>(h)->num_total_blocks(); }
VCBE_EXPORT long long vcbe_num_preemptions(void* h) { return (long long)static_cast<vllm::Engine*>(h)->num_preemptions(); }
VCBE_EXPORT long long vcbe_pool_total_bytes(void* h) { return (long long)static_cast<vllm::Engine*>(h)->pool_total_bytes(); }
VCBE_EXPORT long long vcbe_pool_used_bytes(void* h) { return (long long)static_cast<vllm::Engine*>(h)->pool_used_bytes(); }

// An explicit batch: entry i is request req_ids[i] with token_counts[i] tokens (taken in order from `tokens`) and
// want_counts[i] wanted places (from `want`).  Writes [rows, vocab] floats to `logits` (room for cap_floats) and
// returns the number of rows.
VCBE_EXPORT int vcbe_step_tokens(void* h, int n_entries, const long long* req_ids, const int* token_counts, const int* tokens,
                                 const int* want_counts, const int* want, float* logits, long long cap_floats) {
    return guarded([&]() -> int {
        std::vector<vllm::StepEntry> entries((size_t)n_entries);
        for (int i = 0; i < n_entries; ++i) {
            entries[i].request_id = req_ids[i];
            entries[i].tokens.assign(tokens, tokens + token_counts[i]);
            entries[i].want.assign(want, want + want_counts[i]);
            tokens += token_counts[i];
            want += want_counts[i];
        }
        const std::vector<float> out = static_cast<vllm::Engine*>(h)->step_tokens(entries);
        if ((long long)out.size() > cap_floats) throw std::runtime_error("more logits than the caller has room for");
        std::memcpy(logits, out.data(), out.size() * sizeof(float));
        const int vocab = static_cast<vllm::Engine*>(h)->vocab_size();
        return (int)(out.size() / (size_t)vocab);
    }, -1);
}

VCBE_EXPORT void vcbe_release(void* h, long long request_id) { static_cast<vllm::Engine*>(h)->release(request_id); }
