// The C++ face of the engine: one include, as the reference's include/vllm/vllm.hpp:1-20 is.
//
//   #include "vllm/vllm.hpp"
//   vllm::EngineConfig cfg;  cfg.model_path = "...";
//   vllm::Engine engine(cfg);
//   if (!engine.initialize()) ...
//   auto id = engine.add_request({1, 2, 3}, vllm::SamplingParams{});
//   engine.run([](const vllm::GenerationOutput& o) { ... });
//
// The library (libvcb_engine.so) holds a host runtime written in C++ -- configuration, safetensors loader,
// one device pool, cache manager, scheduler, the decoder's forward pass, sampler front end -- over the same
// CUDA kernels (libvcb_kernels.so) that the Python host drives.  One GPU, one architecture
// (Qwen2ForCausalLM), token ids in and out.
#pragma once

#include "vllm/core/config.hpp"
#include "vllm/core/engine.hpp"
