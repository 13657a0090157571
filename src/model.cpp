// The Qwen2 dense decoder of the C++ host: config.json, weights by tensor name, one forward pass over a
// mixed batch from the paged cache.
//
// Flow of a step as in the reference (src/model/qwen.cpp:291-328): ids -> embedding -> per layer
// [RMSNorm -> q/k/v with bias -> rotation -> cache write -> attention -> output projection -> residual;
// RMSNorm -> gate and up -> silu(gate) * up -> down -> residual] -> final RMSNorm -> lm_head; every formula
// is the kernels' (vllm-cpp_b200/csrc), which cite the reference's lines.  What differs from the reference is
// what differs in the Python host too: a batch holds portions of several requests, q/k/v and gate/up are one
// product each on matrices concatenated at load, residual additions happen inside the norm kernels, logits
// are computed at the wanted rows only, eps and the window come from config.json, an untied lm_head is a
// matrix of its own.  This host launches the plain sequence of kernels (a norm kernel before every product);
// the Python host's fused decode path and CUDA graphs are not repeated here.
#include <cublas_v2.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>
#include <numeric>
#include <set>

#include "model.hpp"

namespace vllm {
namespace host {

// ---------------------------------------------------------------------------------------------- config
Qwen2Config Qwen2Config::from_json(const json::Value& j) {
    std::vector<std::string> problems;
    auto get_int = [&](const char* key, bool required, int dflt) {
        const json::Value* v = j.find(key);
        if (!v || v->kind == json::Value::Null) {
            if (required) problems.push_back(std::string("missing required key '") + key + "'");
            return dflt;
        }
        if (v->kind != json::Value::Number || !v->integral) {
            problems.push_back(std::string("'") + key + "' must be an integer");
            return dflt;
        }
        return (int)v->num;
    };
    Qwen2Config c;
    c.hidden = get_int("hidden_size", true, 0);
    c.layers = get_int("num_hidden_layers", true, 0);
    c.heads = get_int("num_attention_heads", true, 0);
    c.kv_heads = get_int("num_key_value_heads", true, 0);
    c.inter = get_int("intermediate_size", true, 0);
    c.max_pos = get_int("max_position_embeddings", true, 0);
    c.vocab = get_int("vocab_size", true, 0);
    const json::Value* theta = j.find("rope_theta");
    if (!theta || theta->kind != json::Value::Number) problems.push_back("missing required key 'rope_theta'");
    else c.rope_theta = theta->num;
    auto stop_if_faulty = [&]() {
        if (problems.empty()) return;
        std::string msg = "Qwen2 config.json: ";
        for (size_t i = 0; i < problems.size(); ++i) msg += (i ? "; " : "") + problems[i];
        throw Error(msg);
    };
    stop_if_faulty();
    for (auto kv : {std::make_pair("hidden_size", c.hidden), std::make_pair("num_hidden_layers", c.layers),
                    std::make_pair("num_attention_heads", c.heads), std::make_pair("num_key_value_heads", c.kv_heads),
                    std::make_pair("intermediate_size", c.inter), std::make_pair("max_position_embeddings", c.max_pos),
                    std::make_pair("vocab_size", c.vocab)})
        if (kv.second <= 0) problems.push_back(std::string("'") + kv.first + "' must be positive");
    if (!(c.rope_theta > 0)) problems.push_back("'rope_theta' must be positive");
    stop_if_faulty();
    c.head_dim = get_int("head_dim", false, 0);
    if (c.head_dim == 0) {
        if (c.hidden % c.heads) problems.push_back("hidden_size is not a multiple of num_attention_heads and no 'head_dim' is given");
        else c.head_dim = c.hidden / c.heads;             // src/model/qwen.cpp:47
    }
    if (c.head_dim % 2) problems.push_back("head_dim must be even (rotary pairs)");
    if (c.head_dim > 256) problems.push_back("head_dim exceeds 256, the largest the kernels take");
    if (c.heads % c.kv_heads) problems.push_back("num_attention_heads is not a multiple of num_key_value_heads");
    if (const json::Value* e = j.find("rms_norm_eps")) {
        if (e->kind != json::Value::Number || !(e->num > 0)) problems.push_back("'rms_norm_eps' must be a positive number");
        else c.eps = e->num;
    }
    if (const json::Value* r = j.find("initializer_range")) {
        if (r->kind != json::Value::Number || !(r->num >= 0)) problems.push_back("'initializer_range' must be a non-negative number");
        else c.init_range = r->num;
    }
    if (const json::Value* a = j.find("hidden_act"))
        if (a->kind != json::Value::String || a->str != "silu") problems.push_back("hidden_act is not supported (only 'silu')");
    if (const json::Value* rs = j.find("rope_scaling"))
        if (rs->kind != json::Value::Null) problems.push_back("rope_scaling is not supported (must be null)");
    if (const json::Value* t = j.find("tie_word_embeddings")) {
        if (t->kind != json::Value::Bool) problems.push_back("'tie_word_embeddings' must be true or false");
        else c.tie = t->b;
    }
    if (const json::Value* u = j.find("use_sliding_window")) {
        if (u->kind != json::Value::Bool) problems.push_back("'use_sliding_window' must be true or false");
        else c.use_window = u->b;
    }
    if (c.use_window) {
        c.window = get_int("sliding_window", false, 0);
        c.max_window_layers = get_int("max_window_layers", false, 0);
        if (c.window <= 0) problems.push_back("use_sliding_window is true but 'sliding_window' is not a positive integer");
        if (c.max_window_layers < 0) problems.push_back("'max_window_layers' must not be negative");
    }
    if (const json::Value* e = j.find("eos_token_id")) {
        if (e->kind == json::Value::Number && e->integral) c.eos_ids.push_back((TokenId)e->num);
        else if (e->kind == json::Value::Array) {
            for (const auto& x : e->arr) {
                if (x.kind != json::Value::Number || !x.integral) { problems.push_back("'eos_token_id' must be an integer or a list of integers"); break; }
                c.eos_ids.push_back((TokenId)x.num);
            }
        } else if (e->kind != json::Value::Null) problems.push_back("'eos_token_id' must be an integer or a list of integers");
        for (TokenId id : c.eos_ids)
            if (id < 0 || id >= c.vocab) problems.push_back("eos_token_id " + std::to_string(id) + " lies outside the vocabulary");
    }
    stop_if_faulty();
    return c;
}

// ------------------------------------------------------------------------------------------- the model
static uint16_t f32_to_bf16(float f) {                       // round to nearest even
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x7FFFFFu)) return (uint16_t)((u >> 16) | 0x40);   // NaN stays NaN
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h >> 15) << 31, exp = (h >> 10) & 0x1F, mant = h & 0x3FF;
    float out;
    if (exp == 0) out = std::ldexp((float)mant, -24);
    else if (exp == 31) out = mant ? NAN : INFINITY;
    else out = std::ldexp((float)(mant | 0x400), (int)exp - 25);
    uint32_t u;
    std::memcpy(&u, &out, 4);
    u |= sign;
    std::memcpy(&out, &u, 4);
    return out;
}

Qwen2Model::Qwen2Model(const EngineConfig& cfg, const Qwen2Config& mc, bool bf16)
    : cfg_(cfg), mc_(mc), bf16_(bf16), el_(bf16 ? 2 : 4), dt_(bf16 ? DT_BF16 : DT_F32) {
    // cache groups: layers with the same window share pages and block tables
    for (int l = 0; l < mc.layers; ++l) {
        const int w = mc.layer_window(l);
        auto it = std::find(group_windows_.begin(), group_windows_.end(), w);
        if (it == group_windows_.end()) { group_windows_.push_back(w); it = group_windows_.end() - 1; }
        layer_group_.push_back((int)(it - group_windows_.begin()));
        layer_index_in_group_.push_back((int)std::count(layer_group_.begin(), layer_group_.end() - 1, layer_group_.back()));
    }
    int dev = 0;
    cuda_check(cudaGetDevice(&dev), "cudaGetDevice");
    cuda_check(cudaDeviceGetAttribute(&sms_, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute");
}

Qwen2Model::~Qwen2Model() {
    if (cublas_) cublasDestroy((cublasHandle_t)cublas_);
}

std::map<std::string, std::vector<int64_t>> Qwen2Model::expected_tensors() const {
    const int64_t H = mc_.hidden, q = (int64_t)mc_.heads * mc_.head_dim, kv = (int64_t)mc_.kv_heads * mc_.head_dim, I = mc_.inter, V = mc_.vocab;
    std::map<std::string, std::vector<int64_t>> t{{"model.embed_tokens.weight", {V, H}}, {"model.norm.weight", {H}}};
    if (!mc_.tie) t["lm_head.weight"] = {V, H};
    for (int l = 0; l < mc_.layers; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        t[p + "self_attn.q_proj.weight"] = {q, H};  t[p + "self_attn.q_proj.bias"] = {q};
        t[p + "self_attn.k_proj.weight"] = {kv, H}; t[p + "self_attn.k_proj.bias"] = {kv};
        t[p + "self_attn.v_proj.weight"] = {kv, H}; t[p + "self_attn.v_proj.bias"] = {kv};
        t[p + "self_attn.o_proj.weight"] = {H, q};
        t[p + "mlp.gate_proj.weight"] = {I, H}; t[p + "mlp.up_proj.weight"] = {I, H}; t[p + "mlp.down_proj.weight"] = {H, I};
        t[p + "input_layernorm.weight"] = {H}; t[p + "post_attention_layernorm.weight"] = {H};
    }
    return t;
}

size_t Qwen2Model::weight_bytes() const {
    const size_t H = mc_.hidden, q = (size_t)mc_.heads * mc_.head_dim, kv = (size_t)mc_.kv_heads * mc_.head_dim, I = mc_.inter, V = mc_.vocab;
    auto r = DevicePool::rounded;
    size_t n = r(V * H * el_) + (mc_.tie ? 0 : r(V * H * el_)) + r(H * 4) + r((size_t)mc_.head_dim / 2 * 4);
    n += (size_t)mc_.layers * (r((q + 2 * kv) * H * el_) + r((q + 2 * kv) * 4) + r(H * q * el_) + r(2 * I * H * el_) + r(H * I * el_) + 2 * r(H * 4));
    return n + image_bytes();
}

bool Qwen2Model::fuses(int n_tokens) const {
    const int H = mc_.hidden, q = mc_.heads * mc_.head_dim, I = mc_.inter;
    return bf16_ && n_tokens <= (int)std::min<size_t>(cfg_.fused_decode_tokens, 64) && H % 8 == 0 && q % 8 == 0 && I % 8 == 0;
}

size_t Qwen2Model::image_bytes() const {
    if (!bf16_ || cfg_.fused_decode_tokens == 0 || mc_.hidden % 8 || (mc_.heads * mc_.head_dim) % 8 || mc_.inter % 8) return 0;
    const int H = mc_.hidden, q = mc_.heads * mc_.head_dim, kv = mc_.kv_heads * mc_.head_dim, I = mc_.inter;
    auto r = DevicePool::rounded;
    size_t per_layer = r((size_t)vcb_tiled_weight_bytes(q + 2 * kv, H, 0)) + r((size_t)vcb_tiled_weight_bytes(H, q, 0)) +
                       r((size_t)vcb_tiled_weight_bytes(2 * I, H, I)) + r((size_t)vcb_tiled_weight_bytes(H, I, 0));
    return (size_t)mc_.layers * per_layer + r((size_t)vcb_tiled_weight_bytes(mc_.vocab, H, 0)) +
           r((size_t)2 * sumsq_parts(H) * 64 * 4) + r((size_t)sumsq_parts(H) * 64 * 4);
}

size_t Qwen2Model::bytes_per_page() const {
    return (size_t)mc_.layers * 2 * mc_.kv_heads * cfg_.block_size * mc_.head_dim * el_;
}

size_t Qwen2Model::step_bytes() const {
    // every buffer of a step at max_num_batched_tokens tokens and max_num_seqs wanted rows, plus the kernels' scratch
    const size_t n = cfg_.max_num_batched_tokens, rows = max_logit_rows(), H = mc_.hidden,
                 q = (size_t)mc_.heads * mc_.head_dim, kv = (size_t)mc_.kv_heads * mc_.head_dim, I = mc_.inter;
    auto r = DevicePool::rounded;
    size_t b = r(n * H * 4) + 3 * r(n * H * el_) + r(n * (q + 2 * kv) * el_) + 2 * r(n * q * el_) + r(n * 2 * I * el_) + r(n * I * el_) +
               r(rows * H * el_) + r(max_logit_rows() * (size_t)mc_.vocab * 4);
    b += r((size_t)sms_ * 2 * 256 * 128 * 4) + r(16384 * 4) + r(4);                                  // products' partial tiles, tickets; status
    b += r(cfg_.max_num_seqs * (size_t)mc_.heads * 32 * mc_.head_dim * 4) + r(cfg_.max_num_seqs * (size_t)mc_.heads * 32 * 2 * 4) +
         r(std::max<size_t>(1024, cfg_.max_num_seqs * (size_t)mc_.kv_heads) * 4);                      // decode attention's split merge
    return b;
}

void Qwen2Model::place(DevicePool& pool, int num_pages) {
    const size_t H = mc_.hidden, q = (size_t)mc_.heads * mc_.head_dim, kv = (size_t)mc_.kv_heads * mc_.head_dim, I = mc_.inter, V = mc_.vocab;
    num_pages_ = num_pages;
    embed_ = pool.alloc(V * H * el_, "the embedding table");
    lm_head_ = mc_.tie ? embed_ : pool.alloc(V * H * el_, "the output matrix");
    final_gain_ = pool.alloc_n<float>(H, "the final norm's gain");
    denom_ = pool.alloc_n<float>(mc_.head_dim / 2, "the rotation's divisors");
    layers_.resize(mc_.layers);
    for (auto& L : layers_) {
        L.w_qkv = pool.alloc((q + 2 * kv) * H * el_, "a q/k/v matrix");
        L.b_qkv = pool.alloc_n<float>(q + 2 * kv, "a q/k/v bias");
        L.w_o = pool.alloc(H * q * el_, "an output projection");
        L.w_gate_up = pool.alloc(2 * I * H * el_, "a gate-and-up matrix");
        L.w_down = pool.alloc(H * I * el_, "a down projection");
        L.gain_in = pool.alloc_n<float>(H, "a norm's gain");
        L.gain_post = pool.alloc_n<float>(H, "a norm's gain");
    }
    if (image_bytes()) {
        for (auto& L : layers_) {
            L.t_qkv = pool.alloc((size_t)vcb_tiled_weight_bytes((int)(q + 2 * kv), (int)H, 0), "a tiled q/k/v matrix");
            L.t_o = pool.alloc((size_t)vcb_tiled_weight_bytes((int)H, (int)q, 0), "a tiled output projection");
            L.t_gate_up = pool.alloc((size_t)vcb_tiled_weight_bytes((int)(2 * I), (int)H, (int)I), "a tiled gate-and-up matrix");
            L.t_down = pool.alloc((size_t)vcb_tiled_weight_bytes((int)H, (int)I, 0), "a tiled down projection");
        }
        t_lm_head_ = pool.alloc((size_t)vcb_tiled_weight_bytes((int)V, (int)H, 0), "the tiled output matrix");
        carry_ = pool.alloc_n<float>((size_t)2 * sumsq_parts((int)H) * 64, "sums of squares");
        ss_inner_ = pool.alloc_n<float>((size_t)sumsq_parts((int)H) * 64, "sums of squares");
    }
    // pages: per group [layers of the group][page][k|v][kv head][page x head size]
    for (size_t g = 0; g < group_windows_.size(); ++g) {
        const size_t n_layers = std::count(layer_group_.begin(), layer_group_.end(), (int)g);
        const size_t bytes = n_layers * num_pages * 2 * kv * cfg_.block_size * el_;
        void* p = pool.alloc(bytes, "the cache's pages");
        cuda_check(cudaMemset(p, 0, bytes), "clearing the pages");
        pages_.push_back(p);
    }
    const size_t n = cfg_.max_num_batched_tokens, rows = max_logit_rows();
    residual_ = pool.alloc_n<float>(n * H, "the residual stream");
    delta_ = pool.alloc(n * H * el_, "a step buffer");
    h_ = pool.alloc(n * H * el_, "a step buffer");
    mixed_ = pool.alloc(n * H * el_, "a step buffer");
    qkv_ = pool.alloc(n * (q + 2 * kv) * el_, "a step buffer");
    q_ = pool.alloc(n * q * el_, "a step buffer");
    attn_ = pool.alloc(n * q * el_, "a step buffer");
    gate_up_ = pool.alloc(n * 2 * I * el_, "a step buffer");
    act_ = pool.alloc(n * I * el_, "a step buffer");
    normed_ = pool.alloc(rows * H * el_, "a step buffer");
    logits_ = pool.alloc_n<float>(max_logit_rows() * V, "the logits");
    gemm_partial_ = pool.alloc_n<float>((size_t)sms_ * 2 * 256 * 128, "the products' partial tiles");
    gemm_tickets_ = pool.alloc_n<int>(16384, "the products' tickets");
    status_ = pool.alloc_n<int>(1, "the status word");
    part_o_ = pool.alloc_n<float>(cfg_.max_num_seqs * (size_t)mc_.heads * 32 * mc_.head_dim, "decode attention's partial outputs");
    part_ml_ = pool.alloc_n<float>(cfg_.max_num_seqs * (size_t)mc_.heads * 32 * 2, "decode attention's partial sums");
    attn_tickets_ = pool.alloc_n<int>(std::max<size_t>(1024, cfg_.max_num_seqs * (size_t)mc_.kv_heads), "decode attention's tickets");
    cuda_check(cudaMemset(gemm_tickets_, 0, 16384 * 4), "clearing tickets");
    cuda_check(cudaMemset(status_, 0, 4), "clearing the status word");
    cuda_check(cudaMemset(attn_tickets_, 0, std::max<size_t>(1024, cfg_.max_num_seqs * (size_t)mc_.kv_heads) * 4), "clearing tickets");
    // divisors of the rotation: theta and the exponent 2j/d in float as src/model/qwen.cpp:124 has them, the power in
    // double and then rounded, which is the same float on every host (parts/position.py does the same)
    std::vector<float> denom(mc_.head_dim / 2);
    for (int j = 0; j < mc_.head_dim / 2; ++j)
        denom[j] = (float)pow((double)(float)mc_.rope_theta, (double)((2.0f * (float)j) / (float)mc_.head_dim));
    cuda_check(cudaMemcpy(denom_, denom.data(), denom.size() * 4, cudaMemcpyHostToDevice), "copy of the divisors");
    scale_ = 1.0f / sqrtf((float)mc_.head_dim);                     // src/layers/attention.cpp:126
}

// One tensor to the device: matrices in the compute type, biases and gains in float32.
void Qwen2Model::upload(const TensorInfo& t, void* dst, bool as_float32) {
    const size_t n = (size_t)t.numel();
    const bool to_bf16 = bf16_ && !as_float32;
    if ((t.dtype == "F32" && !to_bf16) || (t.dtype == "BF16" && to_bf16)) {
        cuda_check(cudaMemcpy(dst, t.data, t.nbytes, cudaMemcpyHostToDevice), "copy of a tensor");
        return;
    }
    std::vector<float> f(n);
    if (t.dtype == "F32") std::memcpy(f.data(), t.data, n * 4);
    else {
        const uint16_t* src = reinterpret_cast<const uint16_t*>(t.data);
        for (size_t i = 0; i < n; ++i) {
            if (t.dtype == "BF16") { uint32_t u = (uint32_t)src[i] << 16; std::memcpy(&f[i], &u, 4); }
            else f[i] = f16_to_f32(src[i]);
        }
    }
    if (!to_bf16) {
        cuda_check(cudaMemcpy(dst, f.data(), n * 4, cudaMemcpyHostToDevice), "copy of a tensor");
        return;
    }
    std::vector<uint16_t> b(n);
    for (size_t i = 0; i < n; ++i) b[i] = f32_to_bf16(f[i]);
    cuda_check(cudaMemcpy(dst, b.data(), n * 2, cudaMemcpyHostToDevice), "copy of a tensor");
}

void Qwen2Model::load_weights(const std::string& model_path) {
    // single file or index + shards; every expected tensor must be there with its shape, and nothing else
    std::vector<std::unique_ptr<SafetensorsFile>> files;
    std::map<std::string, const TensorInfo*> present;
    const std::string single = model_path + "/model.safetensors", index = model_path + "/model.safetensors.index.json";
    if (std::ifstream(single).good()) {
        files.emplace_back(new SafetensorsFile(single));
        for (const auto& kv : files.back()->tensors()) present[kv.first] = &kv.second;
    } else if (std::ifstream(index).good()) {
        const json::Value idx = json::parse_file(index);
        const json::Value* wm = idx.find("weight_map");
        if (!wm || wm->kind != json::Value::Object) throw Error(index + ": not a safetensors index (no 'weight_map')");
        std::map<std::string, SafetensorsFile*> by_name;
        for (const auto& kv : wm->obj) {
            if (!by_name.count(kv.second.str)) {
                files.emplace_back(new SafetensorsFile(model_path + "/" + kv.second.str));
                by_name[kv.second.str] = files.back().get();
            }
            auto it = by_name[kv.second.str]->tensors().find(kv.first);
            if (it == by_name[kv.second.str]->tensors().end())
                throw Error(index + " places '" + kv.first + "' in " + kv.second.str + ", which does not hold it");
            present[kv.first] = &it->second;
        }
    } else {
        throw Error("no weights in " + model_path + ": neither model.safetensors nor model.safetensors.index.json");
    }
    const auto expected = expected_tensors();
    std::string missing, unexpected, wrong;
    int n_missing = 0, n_unexpected = 0, n_wrong = 0;
    for (const auto& kv : expected) {
        auto it = present.find(kv.first);
        if (it == present.end()) { missing += (n_missing++ ? ", " : "") + kv.first; continue; }
        if (it->second->shape != kv.second) wrong += (n_wrong++ ? ", " : "") + kv.first;
    }
    for (const auto& kv : present) {
        const std::string& n = kv.first;
        const bool ignored = n.size() >= 19 && n.compare(n.size() - 19, 19, "rotary_emb.inv_freq") == 0;
        if (!expected.count(n) && !ignored && !(mc_.tie && n == "lm_head.weight")) unexpected += (n_unexpected++ ? ", " : "") + n;
    }
    if (n_missing || n_unexpected || n_wrong) {
        std::string msg = "checkpoint does not match the model:";
        if (n_missing) msg += "\n  missing tensors (" + std::to_string(n_missing) + "): " + missing;
        if (n_unexpected) msg += "\n  unexpected tensors (" + std::to_string(n_unexpected) + "): " + unexpected;
        if (n_wrong) msg += "\n  wrong shapes (" + std::to_string(n_wrong) + "): " + wrong;
        throw Error(msg);
    }
    const size_t H = mc_.hidden, q = (size_t)mc_.heads * mc_.head_dim, kv = (size_t)mc_.kv_heads * mc_.head_dim, I = mc_.inter;
    auto at = [&](const std::string& name) -> const TensorInfo& { return *present.at(name); };
    auto offset = [&](void* base, size_t elems, size_t elem_bytes) { return static_cast<void*>(static_cast<uint8_t*>(base) + elems * elem_bytes); };
    upload(at("model.embed_tokens.weight"), embed_, false);
    if (!mc_.tie) upload(at("lm_head.weight"), lm_head_, false);
    upload(at("model.norm.weight"), final_gain_, true);
    for (int l = 0; l < mc_.layers; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        Layer& L = layers_[l];
        // [Wq; Wk; Wv] and [bq; bk; bv] row after row, [W_gate; W_up] likewise
        upload(at(p + "self_attn.q_proj.weight"), L.w_qkv, false);
        upload(at(p + "self_attn.k_proj.weight"), offset(L.w_qkv, q * H, el_), false);
        upload(at(p + "self_attn.v_proj.weight"), offset(L.w_qkv, (q + kv) * H, el_), false);
        upload(at(p + "self_attn.q_proj.bias"), L.b_qkv, true);
        upload(at(p + "self_attn.k_proj.bias"), L.b_qkv + q, true);
        upload(at(p + "self_attn.v_proj.bias"), L.b_qkv + q + kv, true);
        upload(at(p + "self_attn.o_proj.weight"), L.w_o, false);
        upload(at(p + "mlp.gate_proj.weight"), L.w_gate_up, false);
        upload(at(p + "mlp.up_proj.weight"), offset(L.w_gate_up, I * H, el_), false);
        upload(at(p + "mlp.down_proj.weight"), L.w_down, false);
        upload(at(p + "input_layernorm.weight"), L.gain_in, true);
        upload(at(p + "post_attention_layernorm.weight"), L.gain_post, true);
    }
    make_images();
}

// Random weights from a seed, the values weights/random_init.py gives every tensor for the same seed (element i of
// a tensor is a function of the seed, the tensor's name and i; csrc/random_init.cu): matrices and biases
// N(0, initializer_range), gains 1 + N(0, initializer_range).  Biases and gains of a bfloat16 model take the value
// a bfloat16 checkpoint would hold.
void Qwen2Model::random_weights(uint64_t seed) {
    const size_t H = mc_.hidden, q = (size_t)mc_.heads * mc_.head_dim, kv = (size_t)mc_.kv_heads * mc_.head_dim, I = mc_.inter;
    const float std_ = (float)mc_.init_range;
    const auto shapes = expected_tensors();
    auto numel = [&](const std::string& name) {
        size_t n = 1;
        for (int64_t d : shapes.at(name)) n *= (size_t)d;
        return n;
    };
    auto matrix = [&](const std::string& name, void* dst) {
        kernel_check(vcb_random_normal(dst, numel(name), 0, tensor_key(seed, name), 0.0f, std_, bf16_ ? DT_BF16 : DT_F32, nullptr), "random_normal");
    };
    std::vector<uint16_t> rounded;
    std::vector<float> widened;
    auto vector32 = [&](const std::string& name, float* dst, float mean) {
        const size_t n = numel(name);
        if (!bf16_) {
            kernel_check(vcb_random_normal(dst, n, 0, tensor_key(seed, name), mean, std_, DT_F32, nullptr), "random_normal");
            return;
        }
        // through bfloat16: generated into the (larger) float32 destination, read back, widened, stored again
        kernel_check(vcb_random_normal(dst, n, 0, tensor_key(seed, name), mean, std_, DT_BF16, nullptr), "random_normal");
        rounded.resize(n);
        widened.resize(n);
        cuda_check(cudaMemcpy(rounded.data(), dst, n * 2, cudaMemcpyDeviceToHost), "copy of a tensor");
        for (size_t i = 0; i < n; ++i) { const uint32_t u = (uint32_t)rounded[i] << 16; std::memcpy(&widened[i], &u, 4); }
        cuda_check(cudaMemcpy(dst, widened.data(), n * 4, cudaMemcpyHostToDevice), "copy of a tensor");
    };
    auto offset = [&](void* base, size_t elems) { return static_cast<void*>(static_cast<uint8_t*>(base) + elems * el_); };
    matrix("model.embed_tokens.weight", embed_);
    if (!mc_.tie) matrix("lm_head.weight", lm_head_);
    vector32("model.norm.weight", final_gain_, 1.0f);
    for (int l = 0; l < mc_.layers; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        Layer& L = layers_[l];
        matrix(p + "self_attn.q_proj.weight", L.w_qkv);
        matrix(p + "self_attn.k_proj.weight", offset(L.w_qkv, q * H));
        matrix(p + "self_attn.v_proj.weight", offset(L.w_qkv, (q + kv) * H));
        vector32(p + "self_attn.q_proj.bias", L.b_qkv, 0.0f);
        vector32(p + "self_attn.k_proj.bias", L.b_qkv + q, 0.0f);
        vector32(p + "self_attn.v_proj.bias", L.b_qkv + q + kv, 0.0f);
        matrix(p + "self_attn.o_proj.weight", L.w_o);
        matrix(p + "mlp.gate_proj.weight", L.w_gate_up);
        matrix(p + "mlp.up_proj.weight", offset(L.w_gate_up, I * H));
        matrix(p + "mlp.down_proj.weight", L.w_down);
        vector32(p + "input_layernorm.weight", L.gain_in, 1.0f);
        vector32(p + "post_attention_layernorm.weight", L.gain_post, 1.0f);
    }
    cuda_check(cudaDeviceSynchronize(), "random weights");
    make_images();
}

// The second copy of the matrices for steps of few tokens: cut into 128 x 64 tiles, each stored as the tensor
// core reads it from shared memory, gate rows paired with their up rows (csrc/gemm_tcgen05.cu tile_weights_kernel).
void Qwen2Model::make_images() {
    if (!t_lm_head_) return;
    const int H = mc_.hidden, q = mc_.heads * mc_.head_dim, kv = mc_.kv_heads * mc_.head_dim, I = mc_.inter;
    for (auto& L : layers_) {
        kernel_check(vcb_tile_weights(L.w_qkv, q + 2 * kv, H, H, 0, L.t_qkv, nullptr), "tile_weights");
        kernel_check(vcb_tile_weights(L.w_o, H, q, q, 0, L.t_o, nullptr), "tile_weights");
        kernel_check(vcb_tile_weights(L.w_gate_up, 2 * I, H, H, I, L.t_gate_up, nullptr), "tile_weights");
        kernel_check(vcb_tile_weights(L.w_down, H, I, I, 0, L.t_down, nullptr), "tile_weights");
    }
    kernel_check(vcb_tile_weights(lm_head_, mc_.vocab, H, H, 0, t_lm_head_, nullptr), "tile_weights");
    cuda_check(cudaDeviceSynchronize(), "tiling the weights");
    tune_grids();
}

int Qwen2Model::grid_for(int n, int k, int gated, int bn) const {
    auto it = grids_.find({n, k, gated, bn});
    return it == grids_.end() ? (bn == 16 ? sms_ : 2 * sms_) : it->second;
}

// columns of the tensor-core tile for a step of m tokens
static int tile_columns(int m) { return m <= 16 ? 16 : m <= 32 ? 32 : 64; }

// The grid of each few-token product, measured once at load as the Python host does (ops.choose_ctas): one
// CTA per SM, two per SM, and in between the counts that cut every 128-row tile into the same number of whole
// runs of k slabs.  Timed with CUDA events over the layers' matrices in turn, so that the L2 cache serves none.
void Qwen2Model::tune_grids() {
    const int H = mc_.hidden, q = mc_.heads * mc_.head_dim, kv = mc_.kv_heads * mc_.head_dim, I = mc_.inter;
    struct Shape { int n, k, gated; };
    cudaEvent_t e0, e1;
    cuda_check(cudaEventCreate(&e0), "cudaEventCreate");
    cuda_check(cudaEventCreate(&e1), "cudaEventCreate");
    // inputs and outputs of the trial products: a transient allocation of its own, given back below
    const int limit = (int)std::min<size_t>(cfg_.fused_decode_tokens, 64);
    const size_t x_bytes = (size_t)64 * std::max({H, q, I}) * 2, out_bytes = (size_t)64 * std::max({q + 2 * kv, H, 2 * I}) * 2;
    void *x = nullptr, *out = nullptr;
    cuda_check(cudaMalloc(&x, x_bytes), "cudaMalloc");
    cuda_check(cudaMalloc(&out, out_bytes), "cudaMalloc");
    cuda_check(cudaMemset(x, 0, x_bytes), "clearing a buffer");
    // one measurement per width of the tensor-core tile (16, 32, 64 columns), at a token count that takes it
    for (int m : {8, 32, 64}) {
        if (m > std::max(limit, 8)) break;
        const int bn = tile_columns(m);
        for (const Shape& sh : {Shape{q + 2 * kv, H, 0}, Shape{H, q, 0}, Shape{2 * I, H, I}, Shape{H, I, 0}}) {
            const int tiles = sh.gated ? (sh.gated + 63) / 64 : (sh.n + 127) / 128, slabs = (sh.k + 63) / 64;
            std::set<int> candidates{sms_, 2 * sms_};
            for (int per_tile = 1; per_tile <= slabs / 4; ++per_tile)
                if (slabs % per_tile == 0 && tiles * per_tile >= sms_ * 3 / 4 && tiles * per_tile <= 2 * sms_) candidates.insert(tiles * per_tile);
            const std::vector<int> key{sh.n, sh.k, sh.gated, bn};
            int best_ctas = sms_;
            float best_ms = 0;
            for (int ctas : candidates) {
                grids_[key] = ctas;
                float ms = 0;
                for (int rep = 0; rep < 2; ++rep) {                   // the second pass is the one that counts
                    cuda_check(cudaEventRecord(e0, nullptr), "cudaEventRecord");
                    for (const Layer& L : layers_) {
                        const void *w = sh.gated ? L.w_gate_up : sh.n == q + 2 * kv && sh.k == H ? L.w_qkv : sh.k == I ? L.w_down : L.w_o;
                        const void *t = sh.gated ? L.t_gate_up : sh.n == q + 2 * kv && sh.k == H ? L.t_qkv : sh.k == I ? L.t_down : L.t_o;
                        fused_product(x, w, t, out, m, sh.n, sh.k, false, RowScale(), nullptr, nullptr, sh.gated, nullptr);
                    }
                    cuda_check(cudaEventRecord(e1, nullptr), "cudaEventRecord");
                    cuda_check(cudaEventSynchronize(e1), "cudaEventSynchronize");
                    cuda_check(cudaEventElapsedTime(&ms, e0, e1), "cudaEventElapsedTime");
                }
                if (best_ms == 0 || ms < best_ms * 0.98f) {           // a larger grid must win by more than the noise
                    best_ms = ms;
                    best_ctas = ctas;
                }
            }
            grids_[key] = best_ctas;
        }
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(x);
    cudaFree(out);
}

void Qwen2Model::fused_product(const void* x, const void* w, const void* tiled, void* out, int m, int n, int k, bool out_f32,
                               RowScale scale, const float* gain, float* sumsq_out, int gated, cudaStream_t s) {
    const int bn = tile_columns(m);
    const int ctas = grid_for(n, k, gated, bn);
    // swapped form: the weights are the 128-row operand; a gated product writes [m, gated] columns
    kernel_check(vcb_gemm_bf16_tcgen05_fused(w, n, k, tiled, x, m, k, k, out, gated ? gated : n, out_f32 ? 1 : 0, 1, bn, ctas,
                                             gemm_partial_, gemm_tickets_, 16384, status_, scale.sumsq, scale.parts, 64,
                                             mc_.hidden, (float)mc_.eps, gain ? residual_ : nullptr, mc_.hidden, gain, sumsq_out, 64,
                                             gated, s), "gemm_bf16_tcgen05_fused");
}

// A step of few tokens with no norm, activation or addition kernel inside a layer: norm(x) W^T =
// rsqrt(mean(x^2) + eps) * ((x * gain) W^T), so the product that ends a residual branch adds its result into the
// float32 residual stream, stores residual * (the next norm's gain) as the next product's input and leaves the
// rows' sums of squares; the next product multiplies its rows by the factor.  (parts/block.py in the Python host.)
const float* Qwen2Model::forward_fused(const Batch& b, cudaStream_t s) {
    const int n = b.n_tokens, H = mc_.hidden, q = mc_.heads * mc_.head_dim, kv = mc_.kv_heads * mc_.head_dim, I = mc_.inter;
    const float eps = (float)mc_.eps;
    const int parts = sumsq_parts(H);
    kernel_check(vcb_embedding(embed_, b.token_ids, residual_, n, H, mc_.vocab, status_, dt_, s), "embedding");
    RowScale incoming;                                   // set: delta holds residual * gain_in of this layer, factor pending
    int cur = 0;
    for (int l = 0; l < mc_.layers; ++l) {
        const Layer& L = layers_[l];
        const int g = layer_group_[l];
        void* pages = static_cast<uint8_t*>(pages_[g]) + (size_t)layer_index_in_group_[l] * num_pages_ * (size_t)kv * cfg_.block_size * el_ * 2;
        const void* x = delta_;
        if (!incoming.sumsq) {
            kernel_check(vcb_add_rmsnorm(residual_, nullptr, L.gain_in, h_, nullptr, n, H, eps, dt_, s), "add_rmsnorm");
            x = h_;
        }
        fused_product(x, L.w_qkv, L.t_qkv, qkv_, n, q + 2 * kv, H, false, incoming, nullptr, nullptr, 0, s);
        kernel_check(vcb_rope_cache_write(qkv_, L.b_qkv, b.positions, b.req_of_token, b.block_tables[g], b.max_blocks, denom_, q_, pages,
                                          n, mc_.heads, mc_.kv_heads, mc_.head_dim, mc_.head_dim, 0, (int)cfg_.block_size, 1, num_pages_,
                                          status_, dt_, s), "rope_cache_write");
        attend(b, l, s);
        // the output projection ends the attention branch and prepares the feed-forward's norm
        fused_product(attn_, L.w_o, L.t_o, mixed_, n, H, q, false, RowScale(), L.gain_post, ss_inner_, 0, s);
        fused_product(mixed_, L.w_gate_up, L.t_gate_up, act_, n, 2 * I, H, false, RowScale{ss_inner_, parts}, nullptr, nullptr, I, s);
        if (l + 1 < mc_.layers) {
            // the down projection ends the feed-forward branch and prepares the next layer's first norm
            float* out_ss = carry_ + (size_t)cur * parts * 64;
            fused_product(act_, L.w_down, L.t_down, delta_, n, H, I, false, RowScale(), layers_[l + 1].gain_in, out_ss, 0, s);
            incoming = RowScale{out_ss, parts};
            cur ^= 1;
        } else {
            fused_product(act_, L.w_down, L.t_down, delta_, n, H, I, false, RowScale(), nullptr, nullptr, 0, s);
            incoming = RowScale();
        }
    }
    if (b.n_logit_rows == 0) return logits_;
    kernel_check(vcb_add_rmsnorm(residual_, delta_, final_gain_, normed_, b.logit_rows, b.n_logit_rows, H, eps, dt_, s), "add_rmsnorm");
    if (b.n_logit_rows <= 64)
        fused_product(normed_, lm_head_, t_lm_head_, logits_, b.n_logit_rows, mc_.vocab, H, true, RowScale(), nullptr, nullptr, 0, s);
    else
        linear(normed_, lm_head_, logits_, b.n_logit_rows, mc_.vocab, H, true, s);
    return logits_;
}

// out [m, n] = x [m, k] @ w [n, k]^T.  float32: the engine's FMA product.  bfloat16 with up to 128 rows: the
// engine's tcgen05 product with the weights on the 128-row side; more rows: cuBLAS with float accumulation
// (src/layers/linear.cpp:70-77 is the same call with half-precision operands).
void Qwen2Model::linear(const void* x, const void* w, void* out, int m, int n, int k, bool out_f32, cudaStream_t s) {
    if (!bf16_) {
        kernel_check(vcb_gemm_f32((const float*)x, (const float*)w, (float*)out, m, n, k, k, k, n, s), "gemm_f32");
        return;
    }
    // Up to 64 tokens the weights are streamed once by this library's product; from 65 on the library's is the
    // faster one (at Qwen2.5-7B sizes and 128 tokens 108 against 126 us for a layer's four products: tiles of 128
    // columns leave partial tiles of 64 KB to merge).
    if (m <= 64 && k % 8 == 0 && (n + 127) / 128 <= 16384) {
        const int bn = tile_columns(m);
        const int ctas = (bn == 32 || bn == 64) ? 2 * sms_ : sms_;
        kernel_check(vcb_gemm_bf16_tcgen05(w, n, k, nullptr, x, m, k, k, out, n, out_f32 ? 1 : 0, 1, bn, ctas, gemm_partial_,
                                           gemm_tickets_, 16384, status_, s), "gemm_bf16_tcgen05");
        return;
    }
    if (!cublas_) {
        cublasHandle_t h;
        if (cublasCreate(&h) != CUBLAS_STATUS_SUCCESS) throw Error("cublasCreate failed");
        cublas_ = h;
    }
    cublasSetStream((cublasHandle_t)cublas_, s);
    const float alpha = 1.0f, beta = 0.0f;
    const cublasStatus_t st = cublasGemmEx((cublasHandle_t)cublas_, CUBLAS_OP_T, CUBLAS_OP_N, n, m, k, &alpha, w, CUDA_R_16BF, k, x,
                                           CUDA_R_16BF, k, &beta, out, out_f32 ? CUDA_R_32F : CUDA_R_16BF, n, CUBLAS_COMPUTE_32F,
                                           CUBLAS_GEMM_DEFAULT);
    if (st != CUBLAS_STATUS_SUCCESS) throw Error("cublasGemmEx failed with status " + std::to_string((int)st));
}

void Qwen2Model::attend(const Batch& b, int layer, cudaStream_t s) {
    const int g = layer_group_[layer], window = group_windows_[g];
    const size_t kv = (size_t)mc_.kv_heads * mc_.head_dim;
    void* pages = static_cast<uint8_t*>(pages_[g]) + (size_t)layer_index_in_group_[layer] * num_pages_ * 2 * kv * cfg_.block_size * el_;
    const int* bt = b.block_tables[g];
    const int page = (int)cfg_.block_size, d = mc_.head_dim;
    if (bf16_ && (d == 64 || d == 128)) {
        if (b.decode_only) {
            const int nsplit = b.decode_splits[g];
            kernel_check(vcb_attention_decode_mma(q_, pages, attn_, b.q_start, b.ctx_lens, bt, b.max_blocks, nullptr, b.n_reqs, nsplit,
                                                  part_o_, part_ml_, attn_tickets_, nullptr, mc_.heads, mc_.kv_heads, d, page, window,
                                                  scale_, num_pages_, status_, s), "attention_decode_mma");
        } else {
            kernel_check(vcb_attention_prefill_tc(q_, pages, attn_, b.q_start, b.ctx_lens, bt, b.max_blocks, b.tile_req, b.tile_row0,
                                                  b.n_tiles, mc_.heads, mc_.kv_heads, d, page, window, scale_, num_pages_, status_, s),
                         "attention_prefill_tc");
        }
        return;
    }
    kernel_check(vcb_attention_simt(q_, pages, attn_, b.positions, b.req_of_token, bt, b.max_blocks, b.n_tokens, mc_.heads,
                                    mc_.kv_heads, d, page, window, scale_, num_pages_, status_, dt_, s), "attention_simt");
}

int Qwen2Model::decode_splits(int group, int n_reqs, int longest) const {
    const int window = group_windows_[group];
    if (window > 0) longest = std::min(longest, window + 64);
    return std::max(1, std::min({(longest + 63) / 64, 2 * sms_ / std::max(1, n_reqs * mc_.kv_heads), 32}));
}

const float* Qwen2Model::forward(const Batch& b, cudaStream_t s) {
    if (t_lm_head_ && fuses(b.n_tokens)) return forward_fused(b, s);
    const int n = b.n_tokens, H = mc_.hidden, q = mc_.heads * mc_.head_dim, kv = mc_.kv_heads * mc_.head_dim, I = mc_.inter;
    const float eps = (float)mc_.eps;
    kernel_check(vcb_embedding(embed_, b.token_ids, residual_, n, H, mc_.vocab, status_, dt_, s), "embedding");
    bool pending = false;                                 // delta holds an addition to the residual stream not made yet
    for (int l = 0; l < mc_.layers; ++l) {
        const Layer& L = layers_[l];
        const int g = layer_group_[l];
        const size_t kvb = (size_t)kv * cfg_.block_size * el_ * 2;
        void* pages = static_cast<uint8_t*>(pages_[g]) + (size_t)layer_index_in_group_[l] * num_pages_ * kvb;
        kernel_check(vcb_add_rmsnorm(residual_, pending ? delta_ : nullptr, L.gain_in, h_, nullptr, n, H, eps, dt_, s), "add_rmsnorm");
        linear(h_, L.w_qkv, qkv_, n, q + 2 * kv, H, false, s);
        kernel_check(vcb_rope_cache_write(qkv_, L.b_qkv, b.positions, b.req_of_token, b.block_tables[g], b.max_blocks, denom_, q_, pages,
                                          n, mc_.heads, mc_.kv_heads, mc_.head_dim, mc_.head_dim, 0, (int)cfg_.block_size, 1, num_pages_,
                                          status_, dt_, s), "rope_cache_write");
        attend(b, l, s);
        linear(attn_, L.w_o, mixed_, n, H, q, false, s);
        kernel_check(vcb_add_rmsnorm(residual_, mixed_, L.gain_post, h_, nullptr, n, H, eps, dt_, s), "add_rmsnorm");
        linear(h_, L.w_gate_up, gate_up_, n, 2 * I, H, false, s);
        kernel_check(vcb_silu_mul(gate_up_, act_, n, I, dt_, s), "silu_mul");
        linear(act_, L.w_down, delta_, n, H, I, false, s);
        pending = true;
    }
    if (b.n_logit_rows == 0) return logits_;
    // only the rows whose logits are wanted go through the final norm and the output product
    kernel_check(vcb_add_rmsnorm(residual_, pending ? delta_ : nullptr, final_gain_, normed_, b.logit_rows, b.n_logit_rows, H, eps, dt_, s),
                 "add_rmsnorm");
    linear(normed_, lm_head_, logits_, b.n_logit_rows, mc_.vocab, H, true, s);
    return logits_;
}

int Qwen2Model::read_status() {
    int code = 0;
    cuda_check(cudaMemcpy(&code, status_, 4, cudaMemcpyDeviceToHost), "reading the status word");
    if (code) cuda_check(cudaMemset(status_, 0, 4), "clearing the status word");
    return code;
}

}  // namespace host
}  // namespace vllm
