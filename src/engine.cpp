// vllm::Engine: configuration -> model -> one device pool -> cache manager -> scheduler -> steps.
//
// Engine::initialize is the reference's Engine::initialize + QwenModel::load_weights (src/core/engine.cpp:25-81,
// src/model/qwen.cpp:25-289) without the tokenizer; Engine::step is schedule -> one mixed batch through the
// model -> sampling on the device for the rows that end a request's known tokens -> token ids to the host ->
// append, check stop, free (src/core/engine.cpp:106-127 runs prefill and decode per sequence and samples on
// the CPU).  The same steps, decisions and sampling keys as vllm-cpp_b200/engine/llm_engine.py, so a
// workload gives the same token ids on both hosts in float32.
#include <algorithm>
#include <cmath>
#include <numeric>

#include "model.hpp"

namespace vllm {

using namespace host;

namespace {

uint64_t splitmix64(uint64_t x) {
    uint64_t z = x + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// The uniform number in [0, 1) of draw `index` of a request with `seed`: 24 random bits, keyed so that a
// request's tokens do not depend on batching, cutting or preemption.
float uniform_for(uint64_t seed, uint64_t index) {
    const uint64_t h = splitmix64(splitmix64(seed) ^ ((index + 1) * 0xD1342543DE82EF95ull));
    return (float)(h >> 40) / (float)(1 << 24);
}

int cdiv(int a, int b) { return (a + b - 1) / b; }
size_t align4(size_t n) { return (n + 3) / 4 * 4; }

}  // namespace

struct Engine::Impl {
    EngineConfig cfg;
    bool initialized = false, bf16 = true;
    std::string error;
    Qwen2Config mc;
    std::unique_ptr<DevicePool> pool;
    std::unique_ptr<Qwen2Model> model;
    std::unique_ptr<CacheManager> cache;
    std::unique_ptr<Scheduler> scheduler;
    std::map<int64_t, std::unique_ptr<Sequence>> sequences;
    int64_t next_id = 0;
    int max_model_len = 0, max_blocks = 0, num_pages = 0;
    cudaStream_t stream = nullptr;
    // step metadata: one pinned buffer, one device buffer, copied once per step
    int *meta_host = nullptr, *meta_dev = nullptr;
    size_t meta_ints = 0;
    // sampler: options in, ids out
    float *samp_host = nullptr, *samp_dev = nullptr, *filter_scratch = nullptr;      // [4][max rows]: temperature, uniform, top_p, penalty
    int *topk_host = nullptr, *topk_dev = nullptr, *ids_host = nullptr, *ids_dev = nullptr;
    int *pen_ids_dev = nullptr, *pen_start_dev = nullptr;
    size_t pen_ids_cap = 0;
    int steps_since_check = 0;
    // Decode steps in which every request brings one token and wants its logits have a fixed shape for a given
    // number of requests and attention splits: the first such step runs directly, the second is captured as a
    // CUDA graph, later ones replay it.  The metadata copy and the sampling stay outside the graph.
    // At most kMaxGraphs are kept; the least recently launched goes first.
    struct CapturedStep { cudaGraphExec_t exec; uint64_t last_use; };
    static constexpr size_t kMaxGraphs = 256;
    std::map<std::vector<int>, CapturedStep> graphs;
    std::map<std::vector<int>, int> graph_seen;
    uint64_t graph_clock = 0;
    bool use_graphs = true;

    ~Impl() {
        for (auto& kv : graphs) cudaGraphExecDestroy(kv.second.exec);
        if (meta_host) cudaFreeHost(meta_host);
        if (samp_host) cudaFreeHost(samp_host);
        if (topk_host) cudaFreeHost(topk_host);
        if (ids_host) cudaFreeHost(ids_host);
        if (stream) cudaStreamDestroy(stream);
    }

    size_t max_rows() const { return model->max_logit_rows(); }

    void validate() const {
        auto need = [](bool ok, const std::string& msg) { if (!ok) throw Error(msg); };
        need(cfg.dtype == "bfloat16" || cfg.dtype == "float32", "dtype must be 'bfloat16' or 'float32', got '" + cfg.dtype + "'");
        need(cfg.load_format == "safetensors" || cfg.load_format == "random",
             "load_format must be 'safetensors' or 'random', got '" + cfg.load_format + "'");
        need(cfg.block_size > 0, "KV block size must be greater than zero");
        need(cfg.block_size % 16 == 0 && cfg.block_size <= 256, "block_size must be a multiple of 16 and at most 256");
        need(cfg.gpu_memory_utilization > 0 && cfg.gpu_memory_utilization <= 100, "gpu_memory_utilization is a percentage in (0, 100]");
        need(cfg.max_num_seqs > 0, "max_num_seqs must be positive");
        need(cfg.max_model_len > 0, "max_model_len must be positive");
        need(cfg.max_num_batched_tokens > 0, "max_num_batched_tokens must be positive");
        need(cfg.max_tokens_per_step > 0, "max_tokens_per_step must be positive");
        need(cfg.top_p > 0.0f && cfg.top_p <= 1.0f, "top_p must lie in (0, 1]");
        need(cfg.top_k == -1 || cfg.top_k > 0, "top_k is -1 (off) or positive");
        need(cfg.repetition_penalty > 0.0f, "repetition_penalty must be positive");
    }

    void initialize() {
        validate();
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
            throw Error("no CUDA device: this engine runs on a B200 (sm_100a) only; there is no CPU path");
        if (cfg.device < 0 || cfg.device >= count)
            throw Error("device " + std::to_string(cfg.device) + " does not exist (" + std::to_string(count) + " visible)");
        cuda_check(cudaSetDevice(cfg.device), "cudaSetDevice");
        if (cfg.model_path.empty()) throw Error("model_path is empty");
        const json::Value j = json::parse_file(cfg.model_path + "/config.json");
        if (j.kind != json::Value::Object) throw Error(cfg.model_path + "/config.json must hold a JSON object");
        // the registry: an architecture's name -> its model (src/model/model_registry.cpp:5-24, src/core/engine.cpp:26-44)
        std::string arch = cfg.model_arch;
        if (arch.empty()) {
            const json::Value* a = j.find("architectures");
            if (!a || a->kind != json::Value::Array || a->arr.empty() || a->arr[0].kind != json::Value::String)
                throw Error("config.json has no 'architectures' list and no model_arch was given; known architectures: Qwen2ForCausalLM, qwen");
            arch = a->arr[0].str;
        }
        if (arch != "Qwen2ForCausalLM" && arch != "qwen")
            throw Error("Unknown model architecture: '" + arch + "'; known: Qwen2ForCausalLM, qwen");
        mc = Qwen2Config::from_json(j);
        bf16 = cfg.dtype == "bfloat16";
        // every kernel of a step starts under the one before it (programmatic dependent launch, csrc/common.cuh)
        vcb_set_pdl(1);
        model.reset(new Qwen2Model(cfg, mc, bf16));
        max_model_len = (int)std::min<size_t>(cfg.max_model_len, (size_t)mc.max_pos);
        max_blocks = cdiv(max_model_len, (int)cfg.block_size);

        // The one pool: weights, step buffers and scratch are known from the configuration; the rest of the
        // budget is pages (src/model/qwen.cpp:84-104 does the same from an estimate).
        const size_t n = cfg.max_num_batched_tokens, r = cfg.max_num_seqs, rows = model->max_logit_rows();
        const size_t groups = model->group_windows().size();
        const size_t tiles_cap = n * (size_t)(mc.heads / mc.kv_heads) / 128 + r + 1;
        meta_ints = 3 * align4(n) + align4(r + 1) + align4(r) + align4(rows) + groups * align4(r * max_blocks) + 2 * align4(tiles_cap);
        const size_t sampler_bytes = DevicePool::rounded(4 * rows * 4) + 2 * DevicePool::rounded(rows * 4) +
                                     DevicePool::rounded(rows * (size_t)mc.vocab * 4) + DevicePool::rounded((r + 1) * 4) +
                                     DevicePool::rounded(penalty_ids_cap() * 4);
        const size_t fixed = model->weight_bytes() + model->step_bytes() + DevicePool::rounded(meta_ints * 4) + sampler_bytes +
                             (size_t)64 * 256 * (4 + mc.layers) /* alignment of the slices */;
        const size_t per_page = model->bytes_per_page();          // one page id in every group, over all layers
        size_t pages = cfg.num_gpu_blocks;
        if (pages == 0) {
            size_t free_b = 0, total_b = 0;
            cuda_check(cudaMemGetInfo(&free_b, &total_b), "cudaMemGetInfo");
            const size_t budget = total_b / 100 * cfg.gpu_memory_utilization;
            const size_t in_use = total_b - free_b, reserve = (size_t)384 << 20;      // libraries, context
            if (budget <= in_use + fixed + reserve) throw Error("GPU memory budget is insufficient for model buffers and KV cache");
            pages = std::min<size_t>((size_t)max_blocks * r, (budget - in_use - fixed - reserve) / per_page);
            if (pages < (size_t)max_blocks)
                throw Error("not enough device memory for one request of max_model_len " + std::to_string(max_model_len) + ": " +
                            std::to_string(pages) + " pages fit, " + std::to_string(max_blocks) + " are needed");
        }
        num_pages = (int)pages;
        pool.reset(new DevicePool(fixed + pages * per_page));
        model->place(*pool, num_pages);
        meta_dev = pool->alloc_n<int>(meta_ints, "the step's metadata");
        samp_dev = pool->alloc_n<float>(4 * rows, "the sampler's options");
        topk_dev = pool->alloc_n<int>(rows, "the sampler's options");
        ids_dev = pool->alloc_n<int>(rows, "the sampled ids");
        filter_scratch = pool->alloc_n<float>(rows * (size_t)mc.vocab, "the top-k/top-p scratch");
        pen_start_dev = pool->alloc_n<int>(r + 1, "the penalty's row starts");
        pen_ids_cap = penalty_ids_cap();
        pen_ids_dev = pool->alloc_n<int>(pen_ids_cap, "the penalty's ids");
        cuda_check(cudaMallocHost(&meta_host, meta_ints * 4), "pinned metadata");
        cuda_check(cudaMallocHost(&samp_host, 4 * rows * 4), "pinned sampler options");
        cuda_check(cudaMallocHost(&topk_host, rows * 4), "pinned sampler options");
        cuda_check(cudaMallocHost(&ids_host, rows * 4), "pinned ids");
        cuda_check(cudaStreamCreate(&stream), "cudaStreamCreate");
        if (cfg.load_format == "random") model->random_weights(cfg.seed);
        else model->load_weights(cfg.model_path);
        cache.reset(new CacheManager(model->group_windows(), (int)cfg.block_size, num_pages, (int)cfg.max_num_seqs));
        scheduler.reset(new Scheduler(*cache, cfg));
        initialized = true;
    }

    size_t penalty_ids_cap() const { return cfg.max_num_seqs * std::min<size_t>((size_t)std::max(1, max_model_len), 4096) + 16; }

    size_t max_context() const {          // min(max_model_len, max_position_embeddings, cache capacity) (src/core/engine.cpp:90-93)
        return std::min<size_t>((size_t)max_model_len, (size_t)num_pages * cfg.block_size);
    }

    // ------------------------------------------------------------------------------------------- a step
    // entries: (request, first position, tokens, wanted places).  Packs the metadata, copies it, runs the model.
    struct Item {
        int64_t id;
        std::vector<TokenId> tokens;
        std::vector<int32_t> want;
    };

    const float* run_batch(const std::vector<Item>& items, int* n_rows_out) {
        if (items.empty()) throw Error("a step needs at least one entry");
        const int r = (int)items.size();
        if ((size_t)r > cfg.max_num_seqs) throw Error(std::to_string(r) + " requests in one step; max_num_seqs is " + std::to_string(cfg.max_num_seqs));
        int n = 0, m = 0;
        std::vector<int> q_lens, ctx;
        for (const Item& it : items) {
            if (it.tokens.empty()) throw Error("a request brings no tokens");
            const int have = cache->num_tokens(it.id);
            if (have + (int)it.tokens.size() > max_model_len)
                throw Error("request " + std::to_string(it.id) + " would hold " + std::to_string(have + it.tokens.size()) +
                            " tokens; max_model_len is " + std::to_string(max_model_len));
            for (TokenId t : it.tokens)
                if (t < 0 || t >= mc.vocab) throw Error("a token id lies outside the vocabulary of " + std::to_string(mc.vocab));
            for (int w : it.want)
                if (w < 0 || w >= (int)it.tokens.size()) throw Error("a wanted place lies outside the request's tokens");
            q_lens.push_back((int)it.tokens.size());
            ctx.push_back(have);
            n += (int)it.tokens.size();
            m += (int)it.want.size();
        }
        if ((size_t)n > cfg.max_num_batched_tokens) throw Error(std::to_string(n) + " tokens in one step; max_num_batched_tokens is " + std::to_string(cfg.max_num_batched_tokens));
        if ((size_t)m > max_rows()) throw Error(std::to_string(m) + " logit rows wanted in one step; this engine returns at most " + std::to_string(max_rows()));
        for (const Item& it : items) cache->reserve(it.id, (int)it.tokens.size());

        // sections of the metadata buffer
        size_t off = 0;
        auto section = [&](size_t count) { int* p = meta_host + off; off += align4(count); return p; };
        int *tok = section(n), *pos = section(n), *rot = section(n), *qs = section(r + 1), *cl = section(r), *lr = section(m);
        std::vector<int*> tables;
        for (int g = 0; g < cache->num_groups(); ++g) tables.push_back(section((size_t)r * max_blocks));
        Batch b;
        int t0 = 0, mi = 0;
        qs[0] = 0;
        for (int i = 0; i < r; ++i) {
            const Item& it = items[i];
            for (int k = 0; k < q_lens[i]; ++k) { tok[t0 + k] = it.tokens[k]; pos[t0 + k] = ctx[i] + k; rot[t0 + k] = i; }
            for (int w : it.want) lr[mi++] = t0 + w;
            t0 += q_lens[i];
            qs[i + 1] = t0;
            cl[i] = ctx[i];
            for (int g = 0; g < cache->num_groups(); ++g) {
                const std::vector<int>& table = cache->table(it.id, g);
                int* row = tables[g] + (size_t)i * max_blocks;
                for (int k = 0; k < max_blocks; ++k) row[k] = k < (int)table.size() ? table[k] : CacheManager::RELEASED;
            }
            b.longest = std::max(b.longest, ctx[i] + q_lens[i]);
        }
        b.decode_only = *std::max_element(q_lens.begin(), q_lens.end()) == 1;
        // prefill attention's work list: per request its tiles of 128 packed rows (token x head in group), those
        // that see the most keys first
        const int group = mc.heads / mc.kv_heads;
        std::vector<int> tile_req, tile_row0, keys;
        if (!b.decode_only) {
            for (int i = 0; i < r; ++i)
                for (int k = 0; k < cdiv(q_lens[i] * group, 128); ++k) {
                    tile_req.push_back(i);
                    tile_row0.push_back(k * 128);
                    keys.push_back(ctx[i] + std::min(q_lens[i], ((k + 1) * 128 + group - 1) / group));
                }
            std::vector<int> order(tile_req.size());
            std::iota(order.begin(), order.end(), 0);
            std::stable_sort(order.begin(), order.end(), [&](int a, int c) { return keys[a] > keys[c]; });
            int *tr = section(order.size()), *t0s = section(order.size());
            for (size_t k = 0; k < order.size(); ++k) { tr[k] = tile_req[order[k]]; t0s[k] = tile_row0[order[k]]; }
            b.n_tiles = (int)order.size();
            b.tile_req = meta_dev + (tr - meta_host);
            b.tile_row0 = meta_dev + (t0s - meta_host);
        }
        if (off > meta_ints) throw Error("the step's metadata outgrew its buffer");
        cuda_check(cudaMemcpyAsync(meta_dev, meta_host, off * 4, cudaMemcpyHostToDevice, stream), "copy of the step's metadata");
        auto dev = [&](const int* host_ptr) { return meta_dev + (host_ptr - meta_host); };
        b.n_tokens = n; b.n_reqs = r; b.n_logit_rows = m; b.max_blocks = max_blocks;
        b.token_ids = dev(tok); b.positions = dev(pos); b.req_of_token = dev(rot); b.q_start = dev(qs); b.ctx_lens = dev(cl);
        b.logit_rows = dev(lr);
        for (int* t : tables) b.block_tables.push_back(dev(t));
        for (int g = 0; g < cache->num_groups(); ++g) b.decode_splits.push_back(model->decode_splits(g, r, b.longest));
        const float* logits = nullptr;
        if (use_graphs && bf16 && b.decode_only && m == r && r <= 128) {
            std::vector<int> key{r};
            key.insert(key.end(), b.decode_splits.begin(), b.decode_splits.end());
            auto it = graphs.find(key);
            if (it == graphs.end() && graph_seen[key]++ >= 1) {
                cudaGraph_t graph = nullptr;
                cuda_check(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
                try {
                    model->forward(b, stream);
                } catch (...) {
                    cudaStreamEndCapture(stream, &graph);
                    if (graph) cudaGraphDestroy(graph);
                    throw;
                }
                cuda_check(cudaStreamEndCapture(stream, &graph), "cudaStreamEndCapture");
                cudaGraphExec_t exec = nullptr;
                const cudaError_t err = cudaGraphInstantiate(&exec, graph, 0);
                cudaGraphDestroy(graph);
                cuda_check(err, "cudaGraphInstantiate");
                if (graphs.size() >= kMaxGraphs) {
                    auto oldest = graphs.begin();
                    for (auto g = graphs.begin(); g != graphs.end(); ++g)
                        if (g->second.last_use < oldest->second.last_use) oldest = g;
                    cudaGraphExecDestroy(oldest->second.exec);       // the driver frees it once its last launch is done
                    graph_seen.erase(oldest->first);
                    graphs.erase(oldest);
                }
                it = graphs.emplace(key, CapturedStep{exec, 0}).first;
            }
            if (it != graphs.end()) {
                it->second.last_use = ++graph_clock;
                cuda_check(cudaGraphLaunch(it->second.exec, stream), "cudaGraphLaunch");
                logits = model->logits();
            }
        }
        if (!logits) logits = model->forward(b, stream);
        for (const Item& it : items) cache->commit(it.id, (int)it.tokens.size());
        *n_rows_out = m;
        return logits;
    }

    // Sampling on the device for `rows` logits rows of `seqs` (penalty, greedy or temperature, top-k/top-p), as
    // the reference's order of operations (src/sampler/sampler.cpp:23-79); only the ids come back.
    std::vector<TokenId> sample(const float* logits, const std::vector<Sequence*>& seqs) {
        const int m = (int)seqs.size();
        if (m == 0) return {};
        const size_t cap = max_rows();
        bool any_filter = false, any_penalty = false;
        for (int i = 0; i < m; ++i) {
            const ResolvedParams& p = seqs[i]->params;
            samp_host[0 * cap + i] = p.temperature;
            samp_host[1 * cap + i] = uniform_for(p.seed, seqs[i]->output.size());
            samp_host[2 * cap + i] = p.top_p;
            samp_host[3 * cap + i] = p.repetition_penalty;
            topk_host[i] = p.top_k;
            any_filter |= p.temperature > 0 && (p.top_p < 1.0f || p.top_k > 0);
            any_penalty |= p.repetition_penalty != 1.0f && !seqs[i]->output.empty();
        }
        cuda_check(cudaMemcpyAsync(samp_dev, samp_host, 4 * cap * 4, cudaMemcpyHostToDevice, stream), "copy of the sampler's options");
        if (any_filter) cuda_check(cudaMemcpyAsync(topk_dev, topk_host, m * 4, cudaMemcpyHostToDevice, stream), "copy of top_k");
        float* lg = const_cast<float*>(logits);
        if (any_penalty) {
            std::vector<int> ids, start{0};
            for (Sequence* s : seqs) {
                if (s->params.repetition_penalty != 1.0f) {
                    std::vector<int> u(s->output.begin(), s->output.end());
                    std::sort(u.begin(), u.end());
                    u.erase(std::unique(u.begin(), u.end()), u.end());
                    ids.insert(ids.end(), u.begin(), u.end());
                }
                start.push_back((int)ids.size());
            }
            if (ids.size() > pen_ids_cap) throw Error("too many generated ids for the repetition penalty's buffer");
            if (ids.empty()) ids.push_back(0);
            cuda_check(cudaMemcpyAsync(pen_ids_dev, ids.data(), ids.size() * 4, cudaMemcpyHostToDevice, stream), "copy of the penalty's ids");
            cuda_check(cudaMemcpyAsync(pen_start_dev, start.data(), start.size() * 4, cudaMemcpyHostToDevice, stream), "copy of the penalty's rows");
            cuda_check(cudaStreamSynchronize(stream), "penalty inputs");        // the vectors go out of scope
            kernel_check(vcb_repetition_penalty(lg, mc.vocab, pen_ids_dev, pen_start_dev, samp_dev + 3 * cap, m, mc.vocab, stream),
                         "repetition_penalty");
        }
        kernel_check(vcb_sample(lg, mc.vocab, mc.vocab, samp_dev, samp_dev + cap, ids_dev, m, stream), "sample");
        if (any_filter)
            kernel_check(vcb_sample_filtered(lg, mc.vocab, mc.vocab, samp_dev, samp_dev + cap, samp_dev + 2 * cap, topk_dev, filter_scratch,
                                             ids_dev, m, stream), "sample_filtered");
        cuda_check(cudaMemcpyAsync(ids_host, ids_dev, m * 4, cudaMemcpyDeviceToHost, stream), "copy of the sampled ids");
        cuda_check(cudaStreamSynchronize(stream), "waiting for the step");
        if (++steps_since_check >= 64) {
            steps_since_check = 0;
            if (int code = model->read_status()) throw Error("a kernel left status " + std::to_string(code) + " (a bounded wait ran out, 11: a block table named a page that is not there, 12: a token id outside the vocabulary)");
        }
        return std::vector<TokenId>(ids_host, ids_host + m);
    }
};

// ------------------------------------------------------------------------------------------ public face
Engine::Engine(const EngineConfig& config) : impl_(new Impl) { impl_->cfg = config; }
Engine::~Engine() = default;

bool Engine::initialize() {
    try {
        impl_->initialize();
        return true;
    } catch (const std::exception& e) {
        impl_->error = e.what();
        impl_->initialized = false;
        return false;
    }
}

bool Engine::is_initialized() const { return impl_->initialized; }
const std::string& Engine::last_error() const { return impl_->error; }
const EngineConfig& Engine::config() const { return impl_->cfg; }
int Engine::vocab_size() const { return impl_->mc.vocab; }
size_t Engine::num_free_blocks() const { return impl_->cache ? (size_t)impl_->cache->num_free_pages() : 0; }
size_t Engine::num_total_blocks() const { return (size_t)impl_->num_pages; }
size_t Engine::num_preemptions() const { return impl_->scheduler ? impl_->scheduler->num_preemptions() : 0; }
size_t Engine::pool_total_bytes() const { return impl_->pool ? impl_->pool->total() : 0; }
size_t Engine::pool_used_bytes() const { return impl_->pool ? impl_->pool->used() : 0; }

int64_t Engine::add_request(const std::vector<TokenId>& prompt, const SamplingParams& sp) {
    Impl& e = *impl_;
    if (!e.initialized) throw std::logic_error("the engine is not initialized");
    ResolvedParams p;
    p.max_tokens = sp.max_tokens;
    p.temperature = sp.temperature < 0 ? e.cfg.temperature : sp.temperature;
    p.top_p = sp.top_p < 0 ? e.cfg.top_p : sp.top_p;
    p.top_k = sp.top_k == 0 ? e.cfg.top_k : sp.top_k;
    p.repetition_penalty = sp.repetition_penalty < 0 ? e.cfg.repetition_penalty : sp.repetition_penalty;
    p.stop_token_ids = sp.default_stop_ids ? e.mc.eos_ids : sp.stop_token_ids;
    p.ignore_eos = sp.ignore_eos;
    if (p.max_tokens == 0) throw std::invalid_argument("max_tokens must be positive");
    if (!(p.top_p > 0.0f && p.top_p <= 1.0f)) throw std::invalid_argument("top_p must lie in (0, 1]");
    if (!(p.top_k == -1 || p.top_k > 0)) throw std::invalid_argument("top_k is -1 (off) or positive");
    if (!(p.repetition_penalty > 0)) throw std::invalid_argument("repetition_penalty must be positive");
    if (prompt.empty()) throw std::invalid_argument("prompt must contain at least one token");
    for (TokenId t : prompt)
        if (t < 0 || t >= e.mc.vocab)
            throw std::invalid_argument("prompt holds token id " + std::to_string(t) + " outside the vocabulary of " + std::to_string(e.mc.vocab));
    const size_t max_context = e.max_context();
    if (prompt.size() > max_context)
        throw std::invalid_argument("prompt exceeds the available context length of " + std::to_string(max_context) + " tokens");
    if (p.max_tokens > max_context - prompt.size())
        throw std::invalid_argument("prompt tokens plus max_tokens exceeds the available context length of " + std::to_string(max_context) + " tokens");
    std::unique_ptr<Sequence> seq(new Sequence);
    seq->seq_id = e.next_id;
    seq->prompt = prompt;
    p.seed = sp.has_seed ? sp.seed : splitmix64((e.cfg.seed << 20) ^ (uint64_t)seq->seq_id);
    seq->params = p;
    e.scheduler->add_request(seq.get());
    e.sequences[seq->seq_id] = std::move(seq);
    return e.next_id++;
}

std::vector<GenerationOutput> Engine::step() {
    Impl& e = *impl_;
    if (!e.initialized) throw std::logic_error("the engine is not initialized");
    std::vector<GenerationOutput> outputs;
    const std::vector<ScheduledItem> items = e.scheduler->schedule();
    if (items.empty()) return outputs;
    std::vector<Impl::Item> batch;
    std::vector<Sequence*> sampled;
    for (const ScheduledItem& it : items) {
        Impl::Item b{it.seq->seq_id, {}, {}};
        for (int p = it.start; p < it.start + it.count; ++p) b.tokens.push_back(it.seq->token_at(p));
        if (it.samples) { b.want.push_back(it.count - 1); sampled.push_back(it.seq); }
        batch.push_back(std::move(b));
    }
    int rows = 0;
    const float* logits = e.run_batch(batch, &rows);
    const std::vector<TokenId> tokens = e.sample(logits, sampled);
    if (sampled.empty()) cuda_check(cudaStreamSynchronize(e.stream), "waiting for the step");
    for (const ScheduledItem& it : items) it.seq->num_processed += it.count;
    for (size_t i = 0; i < sampled.size(); ++i) {
        Sequence* seq = sampled[i];
        const TokenId tok = tokens[i];
        seq->output.push_back(tok);
        GenerationOutput out;
        out.seq_id = seq->seq_id;
        out.tokens = {tok};
        const auto& stops = seq->params.stop_token_ids;
        if (!seq->params.ignore_eos && std::find(stops.begin(), stops.end(), tok) != stops.end()) out.finish_reason = "stop";
        else if (seq->output.size() >= seq->params.max_tokens) out.finish_reason = "length";
        out.finished = !out.finish_reason.empty();
        outputs.push_back(out);
        if (out.finished) {
            e.scheduler->finish(seq);
            e.sequences.erase(seq->seq_id);
        }
    }
    return outputs;
}

void Engine::run(StreamCallback callback) {
    while (has_pending_work())
        for (const GenerationOutput& out : step())
            if (callback) callback(out);
}

void Engine::abort_request(int64_t seq_id) {
    auto it = impl_->sequences.find(seq_id);
    if (it == impl_->sequences.end()) return;
    impl_->scheduler->finish(it->second.get());
    impl_->sequences.erase(it);
}

size_t Engine::pending_requests() const {
    return impl_->scheduler ? impl_->scheduler->waiting().size() + impl_->scheduler->running().size() : 0;
}

bool Engine::has_pending_work() const { return impl_->scheduler && impl_->scheduler->has_pending_work(); }

std::vector<float> Engine::step_tokens(const std::vector<StepEntry>& entries) {
    Impl& e = *impl_;
    if (!e.initialized) throw std::logic_error("the engine is not initialized");
    std::vector<Impl::Item> batch;
    std::vector<int64_t> seen;
    for (const StepEntry& s : entries) {
        if (std::find(seen.begin(), seen.end(), s.request_id) != seen.end())
            throw Error("request " + std::to_string(s.request_id) + " appears twice in one step");
        seen.push_back(s.request_id);
        // explicit requests live beside the scheduler's: their ids are kept apart by the sign
        const int64_t id = -1 - s.request_id;
        if (s.request_id < 0) throw Error("explicit request ids must not be negative");
        if (!e.cache->live(id)) e.cache->add_request(id);
        batch.push_back({id, s.tokens, s.want});
    }
    int rows = 0;
    const float* logits = e.run_batch(batch, &rows);
    std::vector<float> out((size_t)rows * e.mc.vocab);
    if (rows) cuda_check(cudaMemcpyAsync(out.data(), logits, out.size() * 4, cudaMemcpyDeviceToHost, e.stream), "copy of the logits");
    cuda_check(cudaStreamSynchronize(e.stream), "waiting for the step");
    if (int code = e.model->read_status()) throw Error("a kernel left status " + std::to_string(code));
    return out;
}

void Engine::release(int64_t request_id) {
    const int64_t id = -1 - request_id;
    if (impl_->cache && impl_->cache->live(id)) impl_->cache->free_request(id);
}

}  // namespace vllm
