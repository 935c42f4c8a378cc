// Test infrastructure, not part of the shipped library: the C++ standard library's own std::mt19937 and
// std::normal_distribution<float> behind C names, so that a Python test can draw exactly the stream a C++ test
// draws.  MIInfer's quantized-attention test builds its inputs that way (tests/qwen3_quant_kv_attention_test.cpp:79-80:
// mt19937(42), normal(0, 0.5)), and its experiment record quotes the errors it measured on them
// (experiments/EXP-V2-0024-quantized-prefix-kv.md:122-126); tests/test_statistical_pin.py repeats the recipe through
// the oracle and compares with those figures.
#include <cstddef>
#include <random>

namespace {
struct Stream {
    std::mt19937 rng;
    std::normal_distribution<float> dist;
    Stream(unsigned seed, float mean, float stddev) : rng(seed), dist(mean, stddev) {}
};
}  // namespace

extern "C" {
__attribute__((visibility("default"))) void* std_stream_new(unsigned seed, float mean, float stddev) { return new Stream(seed, mean, stddev); }
__attribute__((visibility("default"))) void std_stream_fill(void* stream, float* out, size_t count) {
    Stream* s = static_cast<Stream*>(stream);
    for (size_t i = 0; i < count; ++i) out[i] = s->dist(s->rng);
}
__attribute__((visibility("default"))) void std_stream_free(void* stream) { delete static_cast<Stream*>(stream); }
}
