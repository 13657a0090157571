// The engine: requests in, tokens out, one step at a time.  API after the reference's Engine
// (include/vllm/core/engine.hpp:35-74): initialize, add_request, step, run, abort_request,
// pending_requests.  Requests are token ids (the reference tokenizes text inside add_request, and text is
// outside this engine); step_tokens runs an explicit batch without scheduler and sampler and returns
// logits, which is what the replay tool and the tests drive.
#pragma once

#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "vllm/core/config.hpp"

#define VLLM_API __attribute__((visibility("default")))

namespace vllm {

using TokenId = int32_t;

// Per-request options (include/vllm/core/engine.hpp:50-54 plus a seed, stop ids and ignore_eos).
// A negative temperature, top_p or repetition_penalty and top_k == 0 mean "the engine's default".
struct SamplingParams {
    size_t max_tokens = 64;
    float temperature = -1.0f;            // 0: greedy
    float top_p = -1.0f;
    int32_t top_k = 0;                    // -1: off
    float repetition_penalty = -1.0f;
    bool has_seed = false;
    uint64_t seed = 0;
    bool default_stop_ids = true;         // stop on the model's eos ids; false: on stop_token_ids
    std::vector<TokenId> stop_token_ids;
    bool ignore_eos = false;
};

// One request's news of one step (include/vllm/core/engine.hpp:22-28, without text).
struct GenerationOutput {
    int64_t seq_id = 0;
    std::vector<TokenId> tokens;
    bool finished = false;
    std::string finish_reason;            // "stop", "length", or empty
};

// One request's share of an explicit batch: its next tokens and the places among them whose logits are wanted.
struct StepEntry {
    int64_t request_id = 0;
    std::vector<TokenId> tokens;
    std::vector<int32_t> want;
};

using StreamCallback = std::function<void(const GenerationOutput&)>;

class VLLM_API Engine {
  public:
    explicit Engine(const EngineConfig& config);
    ~Engine();
    Engine(const Engine&) = delete;
    Engine& operator=(const Engine&) = delete;

    // Reads config.json, builds the model, loads the weights, sizes the pool and the cache.
    // False (with the reason in last_error()) if anything is refused.
    bool initialize();
    bool is_initialized() const;
    const std::string& last_error() const;

    // Queue a request; returns its id.  Throws std::invalid_argument on an empty prompt, an id outside the
    // vocabulary or a length that can never fit (src/core/engine.cpp:86-101).
    int64_t add_request(const std::vector<TokenId>& prompt_token_ids, const SamplingParams& params = SamplingParams());
    // One iteration: schedule, run the batch, sample, append, free what finished.
    std::vector<GenerationOutput> step();
    // Step until nothing is pending.
    void run(StreamCallback callback = nullptr);
    void abort_request(int64_t seq_id);
    size_t pending_requests() const;
    bool has_pending_work() const;
    const EngineConfig& config() const;

    // Explicit batches (no scheduler, no sampler): float32 logits [wanted places, vocab] in the order of the
    // entries and of each entry's `want`.  A request is created at its first entry and lives until release().
    std::vector<float> step_tokens(const std::vector<StepEntry>& entries);
    void release(int64_t request_id);

    int vocab_size() const;
    size_t num_free_blocks() const;
    size_t num_total_blocks() const;
    size_t num_preemptions() const;
    // Bytes of the one device allocation and how much of it is handed out.
    size_t pool_total_bytes() const;
    size_t pool_used_bytes() const;

  private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
};

}  // namespace vllm
