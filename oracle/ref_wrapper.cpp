// C names for the reference's own host primitives (test infrastructure only).
// Compiled together with the reference's src/qwen3_primitives.cpp, in place,
// into oracle/_ref/libmiinfer_host_ref.so; used to check oracle/kv_oracle.c and
// to generate tests/golden/ref_host_primitives.npz.
#include "miinfer/qwen3_primitives.hpp"

#include <cstddef>
#include <cstdint>
#include <span>

extern "C" {

// miinfer::fp16_bits_to_float, src/qwen3_primitives.cpp:67
float ref_fp16_bits_to_float(std::uint16_t bits) { return miinfer::fp16_bits_to_float(bits); }

// miinfer::rope_qwen3_reference, src/qwen3_primitives.cpp:109
int ref_rope_qwen3(const float* in, float* out, std::size_t heads, std::size_t head_dim,
                   std::size_t position, float theta) {
    try {
        miinfer::rope_qwen3_reference({in, heads * head_dim}, {out, heads * head_dim}, heads, head_dim,
                                      position, theta);
    } catch (...) { return -1; }
    return 0;
}

// miinfer::softmax_reference, src/qwen3_primitives.cpp:137
int ref_softmax(const float* in, float* out, std::size_t n) {
    try { miinfer::softmax_reference({in, n}, {out, n}); } catch (...) { return -1; }
    return 0;
}

// miinfer::rms_norm_reference, src/qwen3_primitives.cpp:93
int ref_rms_norm(const float* in, const float* w, float* out, std::size_t n, float eps) {
    try { miinfer::rms_norm_reference({in, n}, {w, n}, {out, n}, eps); } catch (...) { return -1; }
    return 0;
}

}  // extern "C"
