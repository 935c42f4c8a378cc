// int8 -> fp16 dequantisation shared by the prefill kernels.
#pragma once

#include "kv_common.cuh"

namespace b200kv {

// 16 int8 values (one 16-byte load) times `scale` -> 16 fp16 in two 16-byte stores.
__device__ __forceinline__ void dequant16(const uint4& raw, __half scale, uint4* lo, uint4* hi) {
    const __half2 s2 = __half2half2(scale);
    const __half2 off = __float2half2_rn(-1152.0f);   // -(1024 + 128): the sum below is an exact small integer
    const uint32_t w[4] = {raw.x ^ 0x80808080u, raw.y ^ 0x80808080u, raw.z ^ 0x80808080u, raw.w ^ 0x80808080u};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t p01 = __byte_perm(w[i], 0x64646464u, 0x4140);   // halves 0x64b0, 0x64b1: 1024 + u
        const uint32_t p23 = __byte_perm(w[i], 0x64646464u, 0x4342);
        const __half2 a = __hmul2(__hadd2(*reinterpret_cast<const __half2*>(&p01), off), s2);
        const __half2 b = __hmul2(__hadd2(*reinterpret_cast<const __half2*>(&p23), off), s2);
        o[2 * i] = *reinterpret_cast<const uint32_t*>(&a);
        o[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&b);
    }
    *lo = make_uint4(o[0], o[1], o[2], o[3]);
    *hi = make_uint4(o[4], o[5], o[6], o[7]);
}

}  // namespace b200kv
