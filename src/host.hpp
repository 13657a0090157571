// Internals of the C++ host runtime (libvcb_engine.so): what engine.cpp, model.cpp, cache.cpp and
// scheduler.cpp share.  Nothing here is part of the public interface (include/vllm/).
//
// Map to the reference: json::Value ~ include/vllm/utils/json_utils.hpp; SafetensorsFile ~
// src/model/model_loader.cpp:14-107 (here memory-mapped, with byte counts checked); DevicePool ~
// include/vllm/memory/gpu_pool.hpp:12-41; BlockPool / CacheManager ~ src/core/block_manager.cpp;
// Sequence ~ include/vllm/core/sequence.hpp; Scheduler ~ src/core/scheduler.cpp; Qwen2Model ~
// src/model/qwen.cpp.  The Python host (vllm-cpp_b200/engine, cache) has the same semantics step for
// step; tests run one workload through both and compare the token ids.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "vllm/core/config.hpp"
#include "vllm/core/engine.hpp"

// ---------------------------------------------------------------------------- the kernels' C interface
// (vllm-cpp_b200/csrc/*.cu; every launcher takes raw device pointers and a stream and returns 0, a
// cudaError_t value or 10001 "bad argument" / 10002 "size not supported")
extern "C" {
void vcb_set_pdl(int on);
int vcb_embedding(const void* table, const int* ids, float* residual, int n_tokens, int hidden, int vocab, int* status, int dtype,
                  void* stream);
int vcb_add_rmsnorm(float* residual, const void* delta, const float* gain, void* out, const int* row_index, int n_rows,
                    int hidden, float eps, int dtype, void* stream);
int vcb_silu_mul(const void* gu, void* out, int n_tokens, int inter, int dtype, void* stream);
int vcb_rope_cache_write(const void* qkv, const float* bias, const int* positions, const int* req_of_token,
                         const int* block_table, int bt_stride, const float* denom, void* q_out, void* cache, int n_tokens,
                         int nh, int nkv, int d, int rot, int pairing, int page, int write_kv, int num_pages, int* status,
                         int dtype, void* stream);
int vcb_attention_simt(const void* q, const void* cache, void* out, const int* positions, const int* req_of_token,
                       const int* block_table, int bt_stride, int n_tokens, int nh, int nkv, int d, int page, int window,
                       float scale, int num_pages, int* status, int dtype, void* stream);
int vcb_attention_decode_mma(const void* q, const void* cache, void* out, const int* q_start, const int* ctx_lens,
                             const int* block_table, int bt_stride, const int* req_list, int n_list, int nsplit,
                             float* part_o, float* part_ml, int* counters, const int* split_tiles, int nh, int nkv, int d,
                             int page, int window, float scale, int num_pages, int* status, void* stream);
int vcb_attention_prefill_tc(const void* q, const void* cache, void* out, const int* q_start, const int* ctx_lens,
                             const int* block_table, int bt_stride, const int* tile_req, const int* tile_row0, int n_tiles,
                             int nh, int nkv, int d, int page, int window, float scale, int num_pages, int* status,
                             void* stream);
int vcb_gemm_f32(const float* a, const float* w, float* c, int m, int n, int k, int lda, int ldw, int ldc, void* stream);
int vcb_gemm_bf16_tcgen05(const void* p, int rows_p, int ldp, const void* p_tiled, const void* q, int rows_q, int ldq, int k,
                          void* out, int ldc, int out_f32, int swapped, int bn, int max_ctas, float* partial, int* tickets,
                          int n_tickets, int* status, void* stream);
int vcb_gemm_bf16_tcgen05_fused(const void* p, int rows_p, int ldp, const void* p_tiled, const void* q, int rows_q, int ldq, int k,
                                void* out, int ldc, int out_f32, int swapped, int bn, int max_ctas, float* partial, int* tickets,
                                int n_tickets, int* status, const float* scale_sumsq, int scale_parts, int scale_ld, int scale_width,
                                float scale_eps, float* residual, int ldr, const float* gain, float* sumsq_out, int sumsq_ld,
                                int gated, void* stream);
long long vcb_tiled_weight_bytes(int rows, int k, int gated);
int vcb_tile_weights(const void* w, int rows, int k, int ld, int gated, void* out, void* stream);
int vcb_random_normal(void* out, unsigned long long n, unsigned long long first, unsigned long long key, float mean,
                      float std_, int dtype, void* stream);
int vcb_repetition_penalty(float* logits, int ld, const int* ids, const int* row_start, const float* penalty, int n_rows,
                           int vocab, void* stream);
int vcb_sample(const float* logits, int ld, int vocab, const float* temperature, const float* uniform, int* out, int n_rows,
               void* stream);
int vcb_sample_filtered(const float* logits, int ld, int vocab, const float* temperature, const float* uniform,
                        const float* top_p, const int* top_k, float* scratch, int* out, int n_rows, void* stream);
}

namespace vllm {
namespace host {

enum { DT_F32 = 0, DT_BF16 = 1 };      // the kernels' dtype codes

// The key of a tensor's stream of random values: the first eight bytes (little-endian) of SHA-256 of
// "<seed>:<name>", as weights/random_init.py computes it.
uint64_t tensor_key(uint64_t seed, const std::string& name);

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

void cuda_check(cudaError_t e, const char* what);
void kernel_check(int code, const char* what);

// ------------------------------------------------------------------------------------------------ JSON
namespace json {
struct Value {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0;
    bool integral = false;
    std::string str;
    std::vector<Value> arr;
    std::vector<std::pair<std::string, Value>> obj;
    const Value* find(const std::string& key) const;
};
Value parse(const std::string& text);     // throws Error with the offset of what it cannot read
Value parse_file(const std::string& path);
}  // namespace json

// ------------------------------------------------------------------------------------------ safetensors
// 8-byte little-endian header length, JSON header, raw data; data_offsets count from the end of the header
// (the layout src/model/model_loader.cpp:21-64 parses).  The file is mapped, not read; every tensor's byte
// count is checked against its shape and type when the header is parsed.
struct TensorInfo {
    std::string dtype;                  // "F32", "BF16", "F16"
    std::vector<int64_t> shape;
    const uint8_t* data = nullptr;
    size_t nbytes = 0;
    int64_t numel() const;
};
class SafetensorsFile {
  public:
    explicit SafetensorsFile(const std::string& path);
    ~SafetensorsFile();
    SafetensorsFile(const SafetensorsFile&) = delete;
    const std::map<std::string, TensorInfo>& tensors() const { return tensors_; }
    const std::string& path() const { return path_; }

  private:
    std::string path_;
    void* map_ = nullptr;
    size_t size_ = 0;
    std::map<std::string, TensorInfo> tensors_;
};

// ------------------------------------------------------------------------------------------------ pool
// One cudaMalloc for everything the engine holds on the device; slices of it, 256-byte aligned, never given
// back (include/vllm/memory/gpu_pool.hpp:12-41).  A slice that does not fit throws: no null slice ever
// leaves here (the reference returns nullptr unchecked, :24-28).
class DevicePool {
  public:
    explicit DevicePool(size_t bytes);
    ~DevicePool();
    DevicePool(const DevicePool&) = delete;
    void* alloc(size_t bytes, const char* what);
    template <typename T> T* alloc_n(size_t n, const char* what) { return static_cast<T*>(alloc(n * sizeof(T), what)); }
    size_t used() const { return offset_; }
    size_t total() const { return total_; }
    static size_t rounded(size_t bytes) { return (bytes + 255) / 256 * 256; }

  private:
    uint8_t* base_ = nullptr;
    size_t total_ = 0, offset_ = 0;
};

// ---------------------------------------------------------------------------------------- cache manager
class BlockPool {                        // LIFO free list with reference counts (src/core/block_manager.cpp:20-53)
  public:
    explicit BlockPool(int num_blocks);
    int num_free() const { return static_cast<int>(free_.size()); }
    int acquire();                       // -1 if none is free
    void release(int block);             // throws if the page is not held
  private:
    std::vector<int> free_, refs_;
};

// Keys and values in pages with a block table per request.  A windowed model's layers would form groups of
// their own; Qwen2 with use_sliding_window has two kinds of layer (all keys, the last W keys), so there are
// up to two groups, each with its own pool of page ids, and a request holds one table per group.
class CacheManager {
  public:
    static constexpr int RELEASED = -1;
    CacheManager(const std::vector<int>& group_windows, int page_size, int num_pages, int max_num_seqs);
    int page_size() const { return page_; }
    int num_pages() const { return num_pages_; }
    int num_groups() const { return static_cast<int>(windows_.size()); }
    bool has_free_slot() const { return !free_slots_.empty(); }
    bool live(int64_t id) const { return reqs_.count(id) != 0; }
    void add_request(int64_t id);
    bool can_append(int64_t id, int n_new) const;
    int max_appendable(int64_t id) const;        // for a live request
    int max_appendable_new() const;              // for a request that is not admitted yet
    void reserve(int64_t id, int n_new);         // pages for the next n_new tokens in every group, or throws
    void commit(int64_t id, int n_new);          // the request now holds n_new more tokens; windows give pages back
    void free_request(int64_t id);
    int num_tokens(int64_t id) const { return reqs_.at(id).num_tokens; }
    int slot(int64_t id) const { return reqs_.at(id).slot; }
    const std::vector<int>& table(int64_t id, int group) const { return reqs_.at(id).tables[group]; }
    int num_free_pages() const;
    size_t live_requests() const { return reqs_.size(); }

  private:
    struct Req {
        std::vector<std::vector<int>> tables;
        std::vector<int> released;
        int num_tokens = 0, slot = -1;
    };
    std::vector<int> windows_;
    int page_, num_pages_;
    std::vector<BlockPool> pools_;
    std::vector<int> free_slots_;
    std::unordered_map<int64_t, Req> reqs_;
};

// ------------------------------------------------------------------------------------------- sequences
struct ResolvedParams {                  // SamplingParams with the engine's defaults filled in
    size_t max_tokens = 64;
    float temperature = 1.0f, top_p = 1.0f, repetition_penalty = 1.0f;
    int32_t top_k = -1;
    uint64_t seed = 0;
    std::vector<TokenId> stop_token_ids;
    bool ignore_eos = false;
};

struct Sequence {                        // include/vllm/core/sequence.hpp:11-94
    int64_t seq_id = 0;
    std::vector<TokenId> prompt, output;
    ResolvedParams params;
    int num_processed = 0;               // tokens whose keys and values are in the cache
    bool finished = false, needs_recompute = false;
    int num_preemptions = 0;
    int total_len() const { return static_cast<int>(prompt.size() + output.size()); }
    int remaining() const { return total_len() - num_processed; }      // 1 for a request that decodes
    TokenId token_at(int pos) const { return pos < static_cast<int>(prompt.size()) ? prompt[pos] : output[pos - prompt.size()]; }
};

struct ScheduledItem {
    Sequence* seq;
    int start, count;
    bool samples;                        // the portion reaches the last known token: a token is sampled
};

// Continuous batching with token-budgeted portions of prompts and recompute preemption; the decisions are
// those of vllm-cpp_b200/engine/scheduler.py, whose header says how they differ from src/core/scheduler.cpp.
class Scheduler {
  public:
    Scheduler(CacheManager& cache, const EngineConfig& cfg);
    void add_request(Sequence* seq);     // throws std::invalid_argument if it can never fit
    bool has_pending_work() const { return !waiting_.empty() || !running_.empty(); }
    std::vector<ScheduledItem> schedule();
    void finish(Sequence* seq);          // leaves the lists, gives its pages back
    const std::deque<Sequence*>& waiting() const { return waiting_; }
    const std::vector<Sequence*>& running() const { return running_; }
    size_t num_preemptions() const { return preemptions_; }

  private:
    std::vector<ScheduledItem> schedule_once();
    Sequence* newest_running(const Sequence* newer_than) const;
    int preempt(Sequence* victim, std::vector<ScheduledItem>& items);
    CacheManager& cache_;
    size_t max_seqs_, max_batched_, max_portion_;
    bool to_front_;
    std::deque<Sequence*> waiting_;
    std::vector<Sequence*> running_;
    size_t preemptions_ = 0;
};

// ----------------------------------------------------------------------------------------------- model
struct Qwen2Config {                     // the config.json keys of Qwen2ForCausalLM (src/model/qwen.cpp:33-47 reads eight of them)
    int hidden = 0, layers = 0, heads = 0, kv_heads = 0, head_dim = 0, inter = 0, vocab = 0, max_pos = 0;
    double rope_theta = 0, eps = 1e-6, init_range = 0.02;    // init_range: 'initializer_range', the random weights' spread
    bool tie = false, use_window = false;
    int window = 0, max_window_layers = 0;
    std::vector<TokenId> eos_ids;
    static Qwen2Config from_json(const json::Value& j);      // throws Error listing every fault
    int layer_window(int layer) const { return use_window && layer >= max_window_layers ? window : 0; }
};

// One step's batch as the model sees it: device arrays (slices of the step's metadata buffer) and a few host facts.
struct Batch {
    int n_tokens = 0, n_reqs = 0, n_logit_rows = 0, max_blocks = 0;
    const int *token_ids = nullptr, *positions = nullptr, *req_of_token = nullptr, *q_start = nullptr, *ctx_lens = nullptr,
              *logit_rows = nullptr;
    std::vector<const int*> block_tables;                    // per cache group: [n_reqs, max_blocks]
    const int *tile_req = nullptr, *tile_row0 = nullptr;     // prefill attention's work list
    int n_tiles = 0;
    bool decode_only = false;
    int longest = 0;                                         // longest context after this step
    std::vector<int> decode_splits;                          // per cache group: context splits of the decode attention
};

class Qwen2Model;                        // model.cpp
std::unique_ptr<Qwen2Model> make_model(const EngineConfig& cfg, const Qwen2Config& mc, bool bf16);

}  // namespace host
}  // namespace vllm
