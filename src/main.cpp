// vllm_cli: the command line of the C++ host.  The reference's src/main.cpp:17-68 reads --model, --arch,
// --port and --quantization and starts an HTTP server; its run script feeds MODEL_PATH and MODEL_ARCH from the
// environment (scripts/run_server.sh:7-10,41-46).  This one keeps --model / --arch and the two environment
// variables, has no server, and generates from token ids: flags override the environment.
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <sstream>

#include "vllm/vllm.hpp"

namespace {
std::vector<vllm::TokenId> parse_ids(const std::string& s) {
    std::vector<vllm::TokenId> out;
    std::stringstream ss(s);
    std::string item;
    while (std::getline(ss, item, ','))
        if (!item.empty()) out.push_back((vllm::TokenId)std::stol(item));
    return out;
}
}  // namespace

int main(int argc, char** argv) {
    vllm::EngineConfig cfg;
    if (const char* p = std::getenv("MODEL_PATH")) cfg.model_path = p;
    if (const char* a = std::getenv("MODEL_ARCH")) cfg.model_arch = a;
    vllm::SamplingParams sp;
    sp.max_tokens = 16;
    sp.temperature = 0.0f;
    std::vector<std::vector<vllm::TokenId>> prompts;
    for (int i = 1; i < argc; ++i) {
        const std::string arg = argv[i];
        auto value = [&]() -> std::string {
            if (i + 1 >= argc) { std::cerr << arg << " needs a value\n"; std::exit(2); }
            return argv[++i];
        };
        if (arg == "--model") cfg.model_path = value();
        else if (arg == "--arch") cfg.model_arch = value();
        else if (arg == "--dtype") cfg.dtype = value();
        else if (arg == "--load-format") cfg.load_format = value();
        else if (arg == "--seed") cfg.seed = std::stoull(value());
        else if (arg == "--device") cfg.device = std::stoi(value());
        else if (arg == "--repetition-penalty") sp.repetition_penalty = std::stof(value());
        else if (arg == "--block-size") cfg.block_size = std::stoul(value());
        else if (arg == "--num-blocks") cfg.num_gpu_blocks = std::stoul(value());
        else if (arg == "--gpu-memory-utilization") cfg.gpu_memory_utilization = std::stoul(value());
        else if (arg == "--max-num-seqs") cfg.max_num_seqs = std::stoul(value());
        else if (arg == "--max-model-len") cfg.max_model_len = std::stoul(value());
        else if (arg == "--max-num-batched-tokens") cfg.max_num_batched_tokens = std::stoul(value());
        else if (arg == "--max-tokens-per-step") cfg.max_tokens_per_step = std::stoul(value());
        else if (arg == "--prompt-ids") prompts.push_back(parse_ids(value()));
        else if (arg == "--prompt-file") {
            std::ifstream f(value());
            std::string line;
            while (std::getline(f, line))
                if (!line.empty()) prompts.push_back(parse_ids(line));
        } else if (arg == "--max-tokens") sp.max_tokens = std::stoul(value());
        else if (arg == "--temperature") sp.temperature = std::stof(value());
        else if (arg == "--top-p") sp.top_p = std::stof(value());
        else if (arg == "--top-k") sp.top_k = std::stoi(value());
        else if (arg == "--sample-seed") { sp.has_seed = true; sp.seed = std::stoull(value()); }
        else if (arg == "--ignore-eos") sp.ignore_eos = true;
        else if (arg == "--quantization") { std::cerr << "quantized weights are not built\n"; return 2; }
        else { std::cerr << "unknown option " << arg << "\n"; return 2; }
    }
    if (prompts.empty()) { std::cerr << "give a prompt with --prompt-ids 1,2,3 or --prompt-file FILE (one prompt a line)\n"; return 2; }
    vllm::Engine engine(cfg);
    if (!engine.initialize()) {
        std::cerr << "Engine initialization failed: " << engine.last_error() << "\n";
        return 1;
    }
    std::vector<std::vector<vllm::TokenId>> outputs(prompts.size());
    try {
        for (const auto& p : prompts) engine.add_request(p, sp);
        engine.run([&](const vllm::GenerationOutput& o) {
            outputs[(size_t)o.seq_id].insert(outputs[(size_t)o.seq_id].end(), o.tokens.begin(), o.tokens.end());
        });
    } catch (const std::exception& e) {
        std::cerr << e.what() << "\n";
        return 1;
    }
    for (const auto& o : outputs) {
        for (size_t i = 0; i < o.size(); ++i) std::cout << (i ? "," : "") << o[i];
        std::cout << "\n";
    }
    return 0;
}
