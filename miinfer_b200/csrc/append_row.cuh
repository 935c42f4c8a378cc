// One cache row (one token of one kv head) through the append arithmetic, with the row spread over a warp:
// lane L holds elements L, L+32, L+64, ...  Shared by the append kernel and by the decode kernel's fused
// single-token append, so both write bit-identical rows.  Arithmetic follows MIInfer's store kernel
// (gfx906/kernels/qwen3_primitives.hip:7257-7300): K RMSNorm -> RoPE -> amax/127 scale -> round-half-even
// int8, every step with explicit IEEE operations (no fused contraction) so a host restatement reproduces the bits.
#pragma once

#include "kv_common.cuh"

namespace b200kv {

// K side before quantization: optional RMSNorm * weight, then RoPE at `position`.
template <int D>
__device__ __forceinline__ void transform_k_row(float (&k)[D / 32], int lane, uint32_t position, const float* k_norm_weight,
                                                float epsilon, int rope_mode, const float* inv_freq, float sectioned_step) {
    constexpr int NJ = D / 32;
    if (k_norm_weight != nullptr) {
        // the reference's shared-memory tree (stride D/2 .. 1) as register adds + a shuffle-down tree over the same pairs
        float sq[NJ];
#pragma unroll
        for (int j = 0; j < NJ; ++j) sq[j] = __fmul_rn(k[j], k[j]);
#pragma unroll
        for (int half = NJ / 2; half >= 1; half >>= 1)
#pragma unroll
            for (int j = 0; j < half; ++j) sq[j] = __fadd_rn(sq[j], sq[j + half]);
        float ss = sq[0];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, o));
        ss = __shfl_sync(0xffffffffu, ss, 0);
        const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(D)), epsilon)));
#pragma unroll
        for (int j = 0; j < NJ; ++j) k[j] = __fmul_rn(__fmul_rn(k[j], r), k_norm_weight[lane + 32 * j]);
    }
    if (rope_mode == B200KV_ROPE_NEOX_FULL) {
#pragma unroll
        for (int j = 0; j < NJ / 2; ++j) {
            const float angle = __fmul_rn(static_cast<float>(position), inv_freq[lane + 32 * j]);
            float s, c;
            sincos_pinned(angle, &s, &c);
            const float x0 = k[j], x1 = k[j + NJ / 2];
            k[j] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
            k[j + NJ / 2] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
        }
    } else if (rope_mode == B200KV_ROPE_SECTIONED64) {
        float angle = static_cast<float>(position);
        for (int i = 0; i < lane; ++i) angle = __fmul_rn(angle, sectioned_step);
        float s, c;
        sincos_pinned(angle, &s, &c);
        const float x0 = k[0], x1 = k[1];
        k[0] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        k[1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
}

// Quantizer: q[j] is this lane's byte of block j (or of the row), scale[j] the fp32 scale of that block as every
// lane sees it (row_scale: all equal).  The cache stores __float2half_rn(scale[j]).
template <int NJ>
__device__ __forceinline__ void quantize_row(const float (&x)[NJ], bool row_scale, int8_t (&q)[NJ], float (&scale)[NJ]) {
    if (row_scale) {
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) amax = fmaxf(amax, fabsf(x[j]));
        amax = warp_max(amax);
        const float s = (amax > 0.0f) ? __fdiv_rn(amax, 127.0f) : 1.0f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) scale[j] = s;
    } else {
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const float amax = warp_max(fabsf(x[j]));
            scale[j] = (amax > 0.0f) ? __fdiv_rn(amax, 127.0f) : 1.0f;
        }
    }
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const float inv = (scale[j] > 0.0f) ? __fdiv_rn(1.0f, scale[j]) : 1.0f;
        int v = __float2int_rn(__fmul_rn(x[j], inv));
        v = max(-128, min(127, v));
        q[j] = static_cast<int8_t>(v);
    }
}

}  // namespace b200kv
