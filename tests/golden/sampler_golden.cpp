// Runs the reference's own host-side sampler code (src/sampler/sampler.cpp,
// src/sampler/topk_topp.cpp of jiamumuzhao/vllm-cpp, compiled from the reference checkout
// given on the command line of make_sampler_golden.sh) on a few small seeded inputs and prints
// what it returns as JSON.  The reference draws its uniform number from an unseeded generator
// inside Sampler::sample, so the draw is reproduced here with the same helper functions in the
// same order (sampler.cpp:27-71) and a uniform number chosen by this program.
#include <cstdint>
#include <cstdio>
#include <random>
#include <vector>

#include "vllm/sampler/sampler.hpp"
#include "vllm/sampler/topk_topp.hpp"

using namespace vllm;

static int draw(std::vector<float> probs, float temperature, float top_p, int top_k, float u) {
    const int vocab = (int)probs.size();
    if (temperature > 0.0f && temperature != 1.0f) {
        const float inv = 1.0f / temperature;                    // sampler.cpp:94-99
        for (auto& x : probs) x *= inv;
    }
    if (temperature <= 0.0f) return Sampler::greedy(probs.data(), vocab);
    sampler::softmax(probs.data(), vocab);
    std::vector<int32_t> idx(vocab);
    for (int i = 0; i < vocab; i++) idx[i] = i;
    int kept = vocab;
    if (top_k > 0 && top_k < vocab) kept = sampler::top_k_filter(probs.data(), idx.data(), vocab, top_k);
    if (top_p < 1.0f || top_k > 0) kept = sampler::top_p_filter(probs.data(), idx.data(), kept, top_p);
    std::vector<float> sel(kept);
    float total = 0.0f;
    for (int i = 0; i < kept; ++i) { sel[i] = probs[idx[i]]; total += sel[i]; }
    for (auto& p : sel) p /= total;
    return idx[sampler::random_sample(sel.data(), kept, u)];
}

int main() {
    std::mt19937 rng(1234);
    std::normal_distribution<float> normal(0.0f, 2.0f);
    std::uniform_real_distribution<float> uni(0.0f, 1.0f);
    printf("{\"cases\": [\n");
    const int vocab = 50;
    const float temps[] = {0.0f, 1.0f, 0.7f, 1.5f};
    const float tps[] = {1.0f, 0.9f, 0.5f};
    const int tks[] = {-1, 1, 5, 50};
    bool first = true;
    for (int c = 0; c < 48; ++c) {
        std::vector<float> logits(vocab);
        for (auto& x : logits) x = normal(rng);
        if (c % 5 == 0) logits[7] = logits[31];                  // a tie
        const float t = temps[c % 4], tp = tps[c % 3];
        const int tk = tks[(c / 3) % 4];
        const float u = uni(rng);
        const int tok = draw(logits, t, tp, tk, u);
        printf("%s{\"logits\": [", first ? "" : ",\n");
        first = false;
        for (int i = 0; i < vocab; ++i) printf("%s%.9g", i ? ", " : "", logits[i]);
        printf("], \"temperature\": %.9g, \"top_p\": %.9g, \"top_k\": %d, \"u\": %.9g, \"token\": %d}", t, tp, tk, u, tok);
    }
    printf("\n]}\n");
    return 0;
}
