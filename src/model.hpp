// The Qwen2 model of the C++ host (see model.cpp).
#pragma once

#include <fstream>

#include "host.hpp"

namespace vllm {
namespace host {

class Qwen2Model {
  public:
    Qwen2Model(const EngineConfig& cfg, const Qwen2Config& mc, bool bf16);
    ~Qwen2Model();

    // Sizes, known from the configuration alone, from which the engine sizes the one pool.
    size_t weight_bytes() const;
    size_t step_bytes() const;                  // buffers of a step at the token budget, logits, kernels' scratch
    size_t bytes_per_page() const;              // one page id over all layers
    size_t max_logit_rows() const { return std::max<size_t>(cfg_.max_num_seqs, std::min<size_t>(cfg_.max_num_batched_tokens, 1024)); }
    const std::vector<int>& group_windows() const { return group_windows_; }
    const Qwen2Config& config() const { return mc_; }

    void place(DevicePool& pool, int num_pages);          // takes every slice: weights, pages, step buffers, scratch
    void load_weights(const std::string& model_path);     // by tensor name; one error lists all faults
    void random_weights(uint64_t seed);                   // the tensors weights/random_init.py makes for this seed
    // Runs the batch's tokens from the cache; returns the float32 logits [n_logit_rows, vocab] on the device.
    const float* forward(const Batch& b, cudaStream_t s);
    // Context splits per (request, kv head) of the split-KV decode attention in cache group `group`, for a
    // decode-only step of n_reqs requests whose longest context is `longest`: enough to fill the device once.
    int decode_splits(int group, int n_reqs, int longest) const;
    const float* logits() const { return logits_; }
    int read_status();                                    // what a kernel noted (0: nothing); synchronises

  private:
    struct Layer {
        void *w_qkv = nullptr, *w_o = nullptr, *w_gate_up = nullptr, *w_down = nullptr;
        void *t_qkv = nullptr, *t_o = nullptr, *t_gate_up = nullptr, *t_down = nullptr;     // pre-tiled images (fused decode)
        float *b_qkv = nullptr, *gain_in = nullptr, *gain_post = nullptr;
    };
    std::map<std::string, std::vector<int64_t>> expected_tensors() const;
    void upload(const TensorInfo& t, void* dst, bool as_float32);
    void linear(const void* x, const void* w, void* out, int m, int n, int k, bool out_f32, cudaStream_t s);
    // the few-token product with what it can take over: the rows' norm factor on its input (scale), the end of a
    // residual branch (residual, gain, sumsq_out), silu(gate) * up (gated > 0); see csrc/gemm_tcgen05.cu
    struct RowScale { const float* sumsq = nullptr; int parts = 0; };
    void fused_product(const void* x, const void* w, const void* tiled, void* out, int m, int n, int k, bool out_f32, RowScale scale,
                       const float* gain, float* sumsq_out, int gated, cudaStream_t s);
    bool fuses(int n_tokens) const;
    const float* forward_fused(const Batch& b, cudaStream_t s);
    void make_images();
    void tune_grids();                           // measures, per product shape, the grid of the few-token product
    int grid_for(int n, int k, int gated, int bn) const;
    size_t image_bytes() const;
    int sumsq_parts(int features) const { return 4 * ((features + 127) / 128); }
    void attend(const Batch& b, int layer, cudaStream_t s);

    EngineConfig cfg_;
    Qwen2Config mc_;
    bool bf16_;
    size_t el_;
    int dt_, sms_ = 148, num_pages_ = 0;
    float scale_ = 1.0f;
    std::vector<int> group_windows_, layer_group_, layer_index_in_group_;
    std::vector<Layer> layers_;
    std::vector<void*> pages_;
    void *embed_ = nullptr, *lm_head_ = nullptr;
    float *final_gain_ = nullptr, *denom_ = nullptr;
    float* residual_ = nullptr;
    void *delta_ = nullptr, *h_ = nullptr, *mixed_ = nullptr, *qkv_ = nullptr, *q_ = nullptr, *attn_ = nullptr, *gate_up_ = nullptr,
         *act_ = nullptr, *normed_ = nullptr;
    float *logits_ = nullptr, *gemm_partial_ = nullptr, *part_o_ = nullptr, *part_ml_ = nullptr;
    int *gemm_tickets_ = nullptr, *status_ = nullptr, *attn_tickets_ = nullptr;
    void* cublas_ = nullptr;
    void* t_lm_head_ = nullptr;
    std::map<std::vector<int>, int> grids_;      // (features, k, gated, tile columns) -> persistent CTAs
    float *carry_ = nullptr, *ss_inner_ = nullptr;       // sums of squares handed from product to product
};

}  // namespace host
}  // namespace vllm
