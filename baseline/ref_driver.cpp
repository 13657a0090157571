// Drives the unmodified jiamumuzhao/vllm-cpp library (libvllm.a, built from its own CMake project)
// through its model interface, the way its engine does, so that its logits and its speed can be set
// beside this repository's engine.  Nothing of this repository's engine is linked here.
//
// What the reference's engine does per token (src/core/engine.cpp:176-187,198-211): copy one token id
// to the device, ModelBase::forward(logits, ids, 1, &ctx, block_table), copy V floats back, synchronise,
// Sampler::sample on the host.  A "step" of a batch of B sequences is B such calls, one after the other
// (engine.cpp:176: a loop over the decode sequences).  This driver repeats exactly that with
// QwenModel (src/model/qwen.cpp:291-328) and Sampler (src/sampler/sampler.cpp:27-47).
//
//   ref_driver logits --model DIR --tokens 5,17,3 --out FILE [--block-size 16] [--max-model-len 256]
//       feeds the tokens one by one from position 0 and writes the logits of every position,
//       float32 [tokens, vocab], to FILE
//   ref_driver bench --model DIR --batches 8,1,64 --contexts 2048,3072 --steps-per-context N --warmup W
//                    [--prefill T] [--max-model-len M] [--block-size 16] [--budget-s S]
//       decode: for every batch size B (in the order given; the prefill comes after the last) and
//       every context c, W untimed and N timed steps of B sequences whose caches hold c
//       tokens at the first timed step (the cache holds the zeros the model's pool was cleared to
//       plus what the steps themselves wrote; the work of a step does not depend on the values);
//       timed once on the device (CUDA events, ids copied in, no read-back) and once end to end
//       (wall clock, with the read-back and the host sampler).  prefill: T tokens of one sequence,
//       one forward per token from position 0, as Engine::prefill does.  Measurements that would begin
//       after S seconds are left out.  Prints one JSON line.
//
// Checks made before the first forward, because the reference checks none of them itself:
// the pool was created (a slice handed out by gpu_pool_alloc is device memory), the block tables
// fit the device buffer the attention layer copies them into (max_model_len / block_size entries,
// src/model/qwen.cpp:79,172-174), every page id is below num_kv_blocks(), every position is below
// max_position_embeddings (the rotation table's length, qwen.cpp:115-128).
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "vllm/core/config.hpp"
#include "vllm/model/qwen.hpp"
#include "vllm/sampler/sampler.hpp"
#include "vllm/utils/json_utils.hpp"

namespace {

[[noreturn]] void die(const std::string& why) {
    std::fprintf(stderr, "ref_driver: %s\n", why.c_str());
    std::printf("{\"error\": \"%s\"}\n", why.c_str());
    std::exit(3);
}

void cuda_ok(cudaError_t e, const char* what) {
    if (e != cudaSuccess) die(std::string(what) + ": " + cudaGetErrorString(e));
}

std::vector<int> parse_ints(const std::string& s) {
    std::vector<int> out;
    std::stringstream ss(s);
    std::string item;
    while (std::getline(ss, item, ',')) {
        if (!item.empty()) out.push_back(std::atoi(item.c_str()));
    }
    return out;
}

struct Args {
    std::string mode, model, tokens, out, contexts, batches = "1";
    int steps = 4, warmup = 3, prefill = 0, max_model_len = 0, block_size = 16;
    double budget_s = 1e9;
};

Args parse(int argc, char** argv) {
    Args a;
    if (argc < 2) die("usage: ref_driver logits|bench --model DIR ...");
    a.mode = argv[1];
    for (int i = 2; i + 1 < argc; i += 2) {
        std::string k = argv[i], v = argv[i + 1];
        if (k == "--model") a.model = v;
        else if (k == "--tokens") a.tokens = v;
        else if (k == "--out") a.out = v;
        else if (k == "--contexts") a.contexts = v;
        else if (k == "--batches") a.batches = v;
        else if (k == "--budget-s") a.budget_s = std::atof(v.c_str());
        else if (k == "--steps-per-context") a.steps = std::atoi(v.c_str());
        else if (k == "--warmup") a.warmup = std::atoi(v.c_str());
        else if (k == "--prefill") a.prefill = std::atoi(v.c_str());
        else if (k == "--max-model-len") a.max_model_len = std::atoi(v.c_str());
        else if (k == "--block-size") a.block_size = std::atoi(v.c_str());
        else die("unknown option " + k);
    }
    if (a.model.empty()) die("--model is required");
    return a;
}

double now_s() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// QwenModel::load_weights sizes one pool from an estimate (src/model/qwen.cpp:58-80,104) and then hands out
// slices that add up to something else (:108-161): the estimate counts one matrix where q and o (and k
// and v) are two, and 2 of the 3 feed-forward work buffers.  What the estimate lacks comes out of the
// cache's share, which is taken last; the cache's own constructor falls back to a cudaMalloc of its own
// when its slice is missing (src/memory/kv_cache.cpp:20-26, the "[POOL] OOM" line on stderr).  A slice
// BEFORE the cache that did not fit would come back as a null pointer, unchecked, and reach a kernel.
// This repeats both sums on the host and refuses such a configuration before anything is loaded.
void check_pool_arithmetic(const std::string& model_dir, const vllm::EngineConfig& cfg) {
    auto j = vllm::json::parse_file(model_dir + "/config.json");
    auto geti = [&](const char* k, long long dflt) { return j.contains(k) ? static_cast<long long>(j[k].get_int()) : dflt; };
    const size_t H = geti("hidden_size", 896), L = geti("num_hidden_layers", 24), nh = geti("num_attention_heads", 14),
                 nkv = geti("num_key_value_heads", 2), I = geti("intermediate_size", 4864),
                 P = geti("max_position_embeddings", 32768), V = geti("vocab_size", 151936);
    if (!H || !L || !nh || !nkv || !I || !P || !V || H % nh) die("config.json lacks a size the reference needs");
    const size_t d = H / nh, qkv = nh * d, kv = nkv * d, S = cfg.max_num_seqs, bs = cfg.block_size;
    const size_t blocks_per_seq = (cfg.max_model_len + bs - 1) / bs;
    size_t estimate = V * H * 2 + L * (H * qkv * 2 + H * kv * 2 + H * I * 3 * 2) + L * 3 * 4 * 1024 + L * P * d * 4 +
                      2 * S * H * 4 + 2 * L * I * 4 + L * (3 * I + 3 * qkv + 2 * kv + 2 * H) * 4 + H * 4 + (64u << 20) +
                      64 * 4 + 64 * V * 4 + L * (blocks_per_seq + 1) * 4;
    const size_t per_block = 2 * bs * nkv * d * 4 * L;
    size_t free_b = 0, total_b = 0;
    cuda_ok(cudaMemGetInfo(&free_b, &total_b), "cudaMemGetInfo");
    const size_t budget = static_cast<size_t>(static_cast<double>(free_b) * cfg.gpu_memory_utilization / 100.0);
    if (budget <= estimate) die("the device has too little free memory for the reference's pool");
    const size_t kv_blocks = std::min(blocks_per_seq * S, (budget - estimate) / per_block);
    const size_t pool = estimate + kv_blocks * per_block;
    const size_t before_cache = (V * H + L * (2 * H * qkv + 2 * H * kv + 3 * H * I)) * 2 + L * 3 * 1024 * 4 + L * P * d * 4 +
                                3 * L * I * 4 + L * (2 * qkv + 2 * kv) * 4 + L * qkv * 4 + L * (blocks_per_seq + 1) * 4 +
                                (2 * L + 1) * H * 4 + 2 * S * H * 4 + 16 * 256 /* alignment of the slices */;
    const size_t engine = 64 * 4 + V * 4 + 2 * 256;
    std::fprintf(stderr, "ref_driver: the reference's pool will be %zu bytes; its slices before the cache need %zu\n", pool, before_cache);
    if (before_cache + engine > pool)
        die("the reference's pool (src/model/qwen.cpp:58-104) is smaller than the slices it takes before the cache "
            "(:108-161) at these sizes; a null slice would reach a kernel, so this configuration is not run");
}

// The reference's model with the buffers its engine would hold (src/core/engine.cpp:68-76).
struct Reference {
    vllm::EngineConfig cfg;
    std::unique_ptr<vllm::QwenModel> model;
    int32_t* ids_d = nullptr;
    float* logits_d = nullptr;
    float* logits_host = nullptr;
    size_t blocks_per_seq = 0;
    double load_s = 0;

    Reference(const Args& a, size_t seqs, size_t max_model_len) {
        cfg.model_path = a.model;
        cfg.model_arch = "qwen";
        cfg.block_size = static_cast<size_t>(a.block_size);
        cfg.max_num_seqs = seqs;
        cfg.max_model_len = max_model_len;
        cfg.gpu_memory_utilization = 90;
        blocks_per_seq = (max_model_len + cfg.block_size - 1) / cfg.block_size;
        check_pool_arithmetic(a.model, cfg);
        const double t0 = now_s();
        model = std::make_unique<vllm::QwenModel>(cfg);
        if (!model->load_weights(a.model)) die("QwenModel::load_weights returned false");
        cuda_ok(cudaDeviceSynchronize(), "after load_weights");
        load_s = now_s() - t0;
        // engine buffers from the model's pool, as Engine::initialize takes them
        ids_d = static_cast<int32_t*>(model->gpu_pool_alloc(64 * sizeof(int32_t)));
        logits_d = static_cast<float*>(model->gpu_pool_alloc(static_cast<size_t>(model->vocab_size()) * sizeof(float)));
        if (!ids_d || !logits_d) die("the reference's pool has no room left for the engine buffers");
        cudaPointerAttributes at{};
        if (cudaPointerGetAttributes(&at, logits_d) != cudaSuccess || at.type != cudaMemoryTypeDevice)
            die("the reference's pool was not created (its slices are not device memory)");
        cuda_ok(cudaMallocHost(&logits_host, static_cast<size_t>(model->vocab_size()) * sizeof(float)), "cudaMallocHost");
        if (model->num_kv_blocks() < seqs * blocks_per_seq)
            die("the reference sized its cache at " + std::to_string(model->num_kv_blocks()) + " blocks, " +
                std::to_string(seqs * blocks_per_seq) + " are needed");
        if (max_model_len > static_cast<size_t>(model->max_seq_len()))
            die("positions would pass max_position_embeddings, the length of the reference's rotation table");
    }

    std::vector<int32_t> table_of(size_t seq) const {
        std::vector<int32_t> t(blocks_per_seq);
        for (size_t b = 0; b < blocks_per_seq; ++b) t[b] = static_cast<int32_t>(seq * blocks_per_seq + b);
        return t;
    }

    // one token of one sequence, as Engine::decode issues it; returns nothing, leaves logits on the device
    void forward_one(int32_t token, int ctx, const std::vector<int32_t>& table) {
        if (ctx < 0 || static_cast<size_t>(ctx) >= cfg.max_model_len) die("context outside max_model_len");
        if (token < 0 || token >= model->vocab_size()) die("token id outside the vocabulary");
        cuda_ok(cudaMemcpyAsync(ids_d, &token, sizeof(int32_t), cudaMemcpyHostToDevice, 0), "copy of the token id");
        int c = ctx;
        model->forward(logits_d, ids_d, 1, &c, table);
    }

    // ... and what Engine::sample_one does with the result
    int32_t read_and_sample(vllm::Sampler& sampler) {
        const int vocab = model->vocab_size();
        cuda_ok(cudaMemcpyAsync(logits_host, logits_d, static_cast<size_t>(vocab) * sizeof(float),
                                cudaMemcpyDeviceToHost, 0), "copy of the logits");
        cuda_ok(cudaDeviceSynchronize(), "synchronise");
        static const std::vector<vllm::TokenId> none;
        return sampler.sample(logits_host, vocab, 0.0f, 1.0f, -1, 1.0f, none).token;
    }
};

int run_logits(const Args& a) {
    const std::vector<int> toks = parse_ints(a.tokens);
    if (toks.empty() || a.out.empty()) die("logits mode needs --tokens and --out");
    const size_t len = a.max_model_len > 0 ? static_cast<size_t>(a.max_model_len) : toks.size();
    if (toks.size() > len) die("more tokens than max_model_len");
    Reference ref(a, 1, len);
    const auto table = ref.table_of(0);
    const size_t vocab = static_cast<size_t>(ref.model->vocab_size());
    std::vector<float> all(toks.size() * vocab);
    for (size_t t = 0; t < toks.size(); ++t) {
        ref.forward_one(toks[t], static_cast<int>(t), table);
        cuda_ok(cudaMemcpy(all.data() + t * vocab, ref.logits_d, vocab * sizeof(float), cudaMemcpyDeviceToHost),
                "copy of the logits");
    }
    std::ofstream f(a.out, std::ios::binary);
    f.write(reinterpret_cast<const char*>(all.data()), static_cast<std::streamsize>(all.size() * sizeof(float)));
    if (!f) die("cannot write " + a.out);
    std::printf("{\"tokens\": %zu, \"vocab\": %zu}\n", toks.size(), vocab);
    return 0;
}

int run_bench(const Args& a) {
    const std::vector<int> contexts = parse_ints(a.contexts), batches = parse_ints(a.batches);
    int most = 0;
    for (int b : batches) most = std::max(most, b);
    if (batches.empty() || most < 1 || most > 64 || a.steps < 1) die("bench mode needs --batches of 1..64 and --steps-per-context >= 1");
    int longest = a.prefill;
    for (int c : contexts) longest = std::max(longest, c + a.steps);
    const size_t len = a.max_model_len > 0 ? static_cast<size_t>(a.max_model_len) : static_cast<size_t>(longest);
    if (static_cast<size_t>(longest) > len) die("contexts pass max_model_len");
    const double started = now_s();
    Reference ref(a, static_cast<size_t>(most), len);
    vllm::Sampler sampler;
    std::vector<std::vector<int32_t>> tables;
    for (int s = 0; s < most; ++s) tables.push_back(ref.table_of(static_cast<size_t>(s)));
    const int vocab = ref.model->vocab_size();
    unsigned rng = 12345u;
    auto next_id = [&]() { rng = rng * 1664525u + 1013904223u; return static_cast<int32_t>((rng >> 8) % static_cast<unsigned>(vocab)); };
    cudaEvent_t e0, e1;
    cuda_ok(cudaEventCreate(&e0), "event");
    cuda_ok(cudaEventCreate(&e1), "event");

    int prefill_tokens = 0;
    auto time_prefill = [&]() {
        // one sequence from position 0; a first short pass warms the kernels up and is overwritten.
        // The prompt is cut short (and the count reported) if the time budget runs out on the way.
        for (int t = 0; t < std::min(8, a.prefill); ++t) ref.forward_one(next_id(), t, tables[0]);
        cuda_ok(cudaDeviceSynchronize(), "prefill warm-up");
        cuda_ok(cudaEventRecord(e0, 0), "record");
        int t = 0;
        for (; t < a.prefill; ++t) {
            ref.forward_one(next_id(), t, tables[0]);
            if ((t & 63) == 63) {
                cuda_ok(cudaDeviceSynchronize(), "prefill");
                if (now_s() - started > a.budget_s) { ++t; break; }
            }
        }
        prefill_tokens = t;
        cuda_ok(cudaEventRecord(e1, 0), "record");
        cuda_ok(cudaEventSynchronize(e1), "timed prefill");
        float ms = 0;
        cuda_ok(cudaEventElapsedTime(&ms, e0, e1), "elapsed");
        return static_cast<double>(ms);
    };

    std::fprintf(stderr, "ref_driver: model loaded in %.0f s\n", ref.load_s);
    std::string runs_json;
    double prefill_ms = 0;
    bool prefill_done = false, first_run = true;
    for (int batch : batches) {
        if (now_s() - started > a.budget_s) break;
        std::string decode_json;
        for (size_t ci = 0; ci < contexts.size(); ++ci) {
            const int c0 = contexts[ci];
            if (c0 - a.warmup < 0) die("a context is shorter than the warm-up");
            // device time: ids in, forward; nothing read back.  The full warm-up once per batch size; one
            // step before each later run (the kernels are the same, only the context differs).
            const int warm = ci == 0 ? a.warmup : 1;
            for (int k = 0; k < warm; ++k)
                for (int s = 0; s < batch; ++s) ref.forward_one(next_id(), c0 - warm + k, tables[static_cast<size_t>(s)]);
            cuda_ok(cudaDeviceSynchronize(), "warm-up");
            cuda_ok(cudaEventRecord(e0, 0), "record");
            for (int k = 0; k < a.steps; ++k)
                for (int s = 0; s < batch; ++s) ref.forward_one(next_id(), c0 + k, tables[static_cast<size_t>(s)]);
            cuda_ok(cudaEventRecord(e1, 0), "record");
            cuda_ok(cudaEventSynchronize(e1), "timed decode steps");
            float dev_ms = 0;
            cuda_ok(cudaEventElapsedTime(&dev_ms, e0, e1), "elapsed");
            // end to end: the same positions again, each token sampled on the host from logits read back
            std::vector<int32_t> last(static_cast<size_t>(batch));
            for (auto& t : last) t = next_id();
            const double t0 = now_s();
            for (int k = 0; k < a.steps; ++k)
                for (int s = 0; s < batch; ++s) {
                    ref.forward_one(last[static_cast<size_t>(s)], c0 + k, tables[static_cast<size_t>(s)]);
                    last[static_cast<size_t>(s)] = ref.read_and_sample(sampler);
                }
            const double e2e_ms = (now_s() - t0) * 1e3;
            std::fprintf(stderr, "ref_driver: batch %d context %d: %.1f ms a step on the device, %.1f end to end (%.0f s so far)\n",
                         batch, c0, dev_ms / a.steps, e2e_ms / a.steps, now_s() - started);
            char buf[256];
            std::snprintf(buf, sizeof(buf), "%s{\"context\": %d, \"device_ms_per_step\": %.4f, \"e2e_ms_per_step\": %.4f}",
                          ci ? ", " : "", c0, dev_ms / a.steps, e2e_ms / a.steps);
            decode_json += buf;
        }
        char head[64];
        std::snprintf(head, sizeof(head), "%s{\"batch\": %d, \"decode\": [", first_run ? "" : ", ", batch);
        runs_json += head + decode_json + "]}";
        first_run = false;
        if (!prefill_done && a.prefill > 0 && batch == batches.back() && now_s() - started <= a.budget_s) {
            prefill_ms = time_prefill();
            prefill_done = true;
            std::fprintf(stderr, "ref_driver: prefill of %d tokens: %.0f ms (%.0f s so far)\n", prefill_tokens, prefill_ms, now_s() - started);
        }
    }
    std::printf("{\"steps_per_context\": %d, \"warmup\": %d, \"runs\": [%s], "
                "\"prefill\": {\"tokens\": %d, \"ms\": %.3f}, \"load_s\": %.1f, \"kv_blocks\": %zu, "
                "\"blocks_per_seq\": %zu, \"layers\": %d, \"vocab\": %d, \"seconds\": %.1f}\n",
                a.steps, a.warmup, runs_json.c_str(), prefill_done ? prefill_tokens : 0, prefill_ms, ref.load_s,
                ref.model->num_kv_blocks(), ref.blocks_per_seq, ref.model->num_layers(), vocab, now_s() - started);
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    const Args a = parse(argc, argv);
    if (a.mode == "logits") return run_logits(a);
    if (a.mode == "bench") return run_bench(a);
    die("unknown mode " + a.mode);
}
