// Sampling weights of the reference's generate(): what sample_step builds from a row of logits before it hands the
// weights to its random generator (crates/autodiff/src/generate/mod.rs:331-369 greedy_argmax, softmax_weights_f64,
// top_k_indices; :382-455 sample_step, sampling_weights_f32).  The reference computes them on the host in f64 so that
// they do not depend on the backend; so does this file.  The draw itself (Generator::multinomial over the weights)
// stays with the caller's generator: the sampled ids go back into the decoder through b200_decoder_step.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <numeric>
#include <string>
#include <vector>

#include "backend.h"

namespace b200 {
namespace {

// first index of the maximum (mod.rs:331-343)
int64_t greedy_argmax(const float* row, int64_t n) {
    int64_t best = 0;
    float best_val = row[0];
    for (int64_t i = 1; i < n; ++i)
        if (row[i] > best_val) {
            best_val = row[i];
            best = i;
        }
    return best;
}

// softmax((x - max) / t) in f64, summed in index order, narrowed to f32 at the end (mod.rs:347-355)
void softmax_weights_f64(const float* row, int64_t n, float temperature, float* out) {
    double mx = -std::numeric_limits<double>::infinity();
    for (int64_t i = 0; i < n; ++i) mx = std::max(mx, static_cast<double>(row[i]));
    const double t = static_cast<double>(temperature);
    std::vector<double> e(static_cast<size_t>(n));
    double sum = 0.0;
    for (int64_t i = 0; i < n; ++i) {
        e[size_t(i)] = std::exp((static_cast<double>(row[i]) - mx) / t);
        sum += e[size_t(i)];
    }
    for (int64_t i = 0; i < n; ++i) out[i] = static_cast<float>(e[size_t(i)] / sum);
}

// the k largest values, by value descending and index ascending (mod.rs:359-369)
std::vector<int64_t> top_k_indices(const float* row, int64_t n, int64_t k) {
    std::vector<int64_t> idx(static_cast<size_t>(n));
    std::iota(idx.begin(), idx.end(), int64_t(0));
    std::partial_sort(idx.begin(), idx.begin() + k, idx.end(), [row](int64_t a, int64_t b) {
        if (row[a] != row[b]) return row[a] > row[b];
        return a < b;
    });
    idx.resize(static_cast<size_t>(k));
    return idx;
}

int32_t weights_impl(const float* logits, int64_t rows, int64_t vocab, int32_t strategy, int32_t k, float temperature, float* out) {
    // GenerateConfig::validate (mod.rs:179-250)
    if (!logits || !out || rows <= 0 || vocab <= 0) return fail(B200_INVALID_ARGUMENT, "sampling_weights: bad argument");
    if (!std::isfinite(temperature) || temperature <= 0.0f)
        return fail(B200_INVALID_ARGUMENT, "sampling_weights: temperature must be finite and positive");
    switch (strategy) {
        case B200_SAMPLE_GREEDY:
            if (temperature != 1.0f || k != 0) return fail(B200_INVALID_ARGUMENT, "sampling_weights: greedy takes temperature 1 and no k");
            break;
        case B200_SAMPLE_TEMPERATURE:
            if (k != 0) return fail(B200_INVALID_ARGUMENT, "sampling_weights: the temperature strategy takes no k");
            break;
        case B200_SAMPLE_TOP_K:
            if (k < 1) return fail(B200_INVALID_ARGUMENT, "sampling_weights: top-k needs k >= 1");
            if (k > vocab) return fail(B200_INVALID_ARGUMENT, "sampling_weights: k exceeds the vocabulary");
            break;
        default:
            return fail(B200_INVALID_ARGUMENT, "sampling_weights: unknown strategy");
    }
    // sample_step rejects rows with non-finite logits before anything is drawn (mod.rs:401-407)
    for (int64_t i = 0; i < rows * vocab; ++i)
        if (!std::isfinite(logits[i])) return fail(B200_INVALID_ARGUMENT, "sampling_weights: the logits contain a non-finite value");
    for (int64_t r = 0; r < rows; ++r) {
        const float* row = logits + r * vocab;
        float* w = out + r * vocab;
        if (strategy == B200_SAMPLE_TEMPERATURE) {
            softmax_weights_f64(row, vocab, temperature, w);
            continue;
        }
        std::fill(w, w + vocab, 0.0f);
        if (strategy == B200_SAMPLE_GREEDY) {
            w[greedy_argmax(row, vocab)] = 1.0f;
            continue;
        }
        const std::vector<int64_t> top = top_k_indices(row, vocab, k);
        std::vector<float> vals(top.size()), tw(top.size());
        for (size_t i = 0; i < top.size(); ++i) vals[i] = row[top[i]];
        softmax_weights_f64(vals.data(), int64_t(vals.size()), temperature, tw.data());
        for (size_t i = 0; i < top.size(); ++i) w[top[i]] = tw[i];
    }
    return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int32_t b200_sampling_weights(const float* logits, int64_t rows, int64_t vocab, int32_t strategy, int32_t k, float temperature,
                              float* weights_out) {
    return weights_impl(logits, rows, vocab, strategy, k, temperature, weights_out);
}

int32_t b200_decoder_sampling_weights(b200_decoder* dec, int32_t strategy, int32_t k, float temperature, float* weights_out,
                                      uint64_t capacity_elems) {
    if (!dec || !weights_out) return fail(B200_INVALID_ARGUMENT, "decoder_sampling_weights: null pointer");
    const int32_t batch = b200_decoder_batch(dec), vocab = b200_decoder_vocab(dec);
    if (batch <= 0 || vocab <= 0) return fail(B200_INVALID_ARGUMENT, "decoder_sampling_weights: no step has run");
    const uint64_t n = uint64_t(batch) * uint64_t(vocab);
    if (capacity_elems < n) return fail(B200_INVALID_ARGUMENT, "decoder_sampling_weights: host buffer too small");
    std::vector<float> logits(static_cast<size_t>(n));
    if (int32_t st = b200_decoder_logits(dec, logits.data(), n)) return st;
    return weights_impl(logits.data(), batch, vocab, strategy, k, temperature, weights_out);
}

}  // extern "C"
