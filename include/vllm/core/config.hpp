// Engine configuration.  Field names and meanings follow the reference's EngineConfig
// (include/vllm/core/config.hpp:34-66); what it declares and never reads (min_p, the frequency and
// presence penalties, schedule_policy, enable_prefix_caching, port, quant_mode) is left out, and what this
// engine adds is marked.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

namespace vllm {

struct EngineConfig {
    // Model
    std::string model_path;               // a folder with config.json and model.safetensors
    std::string model_arch;               // "": config.json's architectures[0]; the reference takes it from --arch only
    std::string dtype = "bfloat16";       // added: "bfloat16" or "float32" (a true 32-bit path)
    int device = 0;                       // added: the CUDA device this engine runs on
    std::string load_format = "safetensors";   // added: "random" fills the weights from `seed` (model_path needs config.json only)

    // Memory
    size_t gpu_memory_utilization = 90;   // percentage (0-100] of the device's memory this engine may hold
    size_t block_size = 16;               // tokens per KV cache block; a multiple of 16, at most 256
    size_t num_gpu_blocks = 0;            // added: pages of the cache; 0 derives them from gpu_memory_utilization
    size_t max_num_seqs = 64;
    size_t max_model_len = 8192;
    size_t max_num_batched_tokens = 16384;   // most tokens in one step

    // Scheduling
    size_t max_tokens_per_step = 512;     // most prompt tokens in one step (the chunked-prefill budget)
    bool preempted_to_front = false;      // added: where a preempted request re-enters the waiting queue
    // added: bfloat16 steps of up to this many tokens (at most 64; 0: none) run with the layer's norms, residual
    // additions and SwiGLU inside the products' epilogues, on a second, pre-tiled copy of the weight matrices
    // (twice the weights' memory).  Measured at Qwen2.5-7B sizes, contexts of 2,048 to 4,096: 3.79 against 4.05 ms
    // a step at 16 tokens, 4.23 against 4.47 at 32, 5.30 against 5.59 at 64.
    size_t fused_decode_tokens = 64;

    // Sampling defaults (per-request values override them)
    float temperature = 1.0f;
    float top_p = 1.0f;
    int32_t top_k = -1;                   // -1 means disabled
    float repetition_penalty = 1.0f;
    uint64_t seed = 0;                    // added: requests without a seed of their own derive one from it; the random weights' seed
};

}  // namespace vllm
