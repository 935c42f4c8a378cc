// Fused KV append: (optional K RMSNorm) -> RoPE on K -> int8 quantization with
// fp16 block scales (or fp16 passthrough) -> cache write, for K and V of every
// (token, kv_head) row in one launch.
//
// Behaviour follows MIInfer's store kernel
// (gfx906/kernels/qwen3_primitives.hip:7213-7326): same operation order, same
// quantizer, positions optionally read from device-resident state.  The mapping
// is new: one warp owns one row, lane L holds elements L, L+32, L+64, ... so
//   - a q8_0 block (32 consecutive dims) is one register index across the warp
//     and its amax is a single warp reduction;
//   - both RoPE pairings (i, i+d/2) and (i, i+32) pair two registers of the SAME
//     lane, so the rotation needs no exchange;
//   - the reference's shared-memory binary tree for the sum of squares (stride
//     d/2 .. 1) becomes register adds followed by a shuffle-down tree that adds
//     exactly the same pairs in the same order (bit-identical sum).
// Input rows are fetched with 16-byte loads, two rows per warp, all in flight at once, and re-read from a
// per-warp staging area in the lane-strided order; output rows are staged through shared memory so the cache is
// written with one 4- or 8-byte store per lane (a full 128/256-byte line per row).
#include "append_row.cuh"

#include <cmath>
#include <type_traits>

namespace b200kv {

struct AppendParams {
    b200kv_view view;
    const void* key;
    const void* value;
    const float* k_norm_weight;
    const b200kv_prefill_state* prefill_state;
    const b200kv_decode_state* decode_state;
    uint32_t token_count;
    uint32_t base_position;
    int rope_mode;
    float epsilon;
    float sectioned_step;    // powf(theta, -2/64)
    float inv_freq[128];     // NeoX: powf(theta, -2i/d), i < d/2
};

constexpr int kAppendWarps = 4;

template <int NJ>
__device__ __forceinline__ void quantize_and_stage(const float (&x)[NJ], uint32_t qblock_is_row, int lane,
                                                   int8_t* stage, __half* scale_dst) {
    int8_t q[NJ];
    float scale[NJ];
    quantize_row<NJ>(x, qblock_is_row != 0, q, scale);
    if (qblock_is_row) {
        if (lane == 0) scale_dst[0] = __float2half_rn(scale[0]);
    } else {
        // lane j stores the scale of block j (NJ <= 8 lanes take part)
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (lane == j) scale_dst[j] = __float2half_rn(scale[j]);
    }
#pragma unroll
    for (int j = 0; j < NJ; ++j) stage[lane + 32 * j] = q[j];
}

// One warp takes TWO consecutive input rows (a row = one token of one kv head; consecutive rows are contiguous in the
// [token][kv_heads * D] inputs), fetches them with 16-byte loads -- all loads of both rows and both sides in flight
// before anything is used -- into a per-warp staging area, and then runs each row through the warp with lane L holding
// elements L, L + 32, ...  (VEC = false: element-wise loads, for inputs that are not 16-byte aligned.)
template <int D, bool IN_F16, bool VEC>
__global__ void __launch_bounds__(kAppendWarps * 32)
append_kernel(const __grid_constant__ AppendParams p) {
    constexpr int NJ = D / 32;
    constexpr int kEsize = IN_F16 ? 2 : 4;
    constexpr int kRowBytes = D * kEsize;
    __shared__ __align__(16) int8_t stage[kAppendWarps][2][D];
    __shared__ __align__(16) uint8_t in_stage[VEC ? kAppendWarps : 1][2][VEC ? 2 * kRowBytes : 16];   // [warp][K | V][two rows]
    // Let the next kernel of the stream become resident now (it orders itself against this one), then wait
    // for everything before us: K/V inputs and the device-side position come from preceding kernels.
    pdl_launch_dependents();
    pdl_wait();

    uint32_t base_position = p.base_position;
    uint32_t token_count = p.token_count;
    uint64_t capacity = p.view.capacity;
    if (p.prefill_state != nullptr) {
        base_position = p.prefill_state->base_position;
        token_count = min(token_count, p.prefill_state->token_count);
        if (p.prefill_state->kv_capacity > 0) capacity = p.prefill_state->kv_capacity;
    } else if (p.decode_state != nullptr) {
        base_position = p.decode_state->position;
        token_count = min(token_count, 1u);
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t H = p.view.kv_heads;
    const uint64_t total_rows = static_cast<uint64_t>(token_count) * H;
    const uint64_t row0 = (static_cast<uint64_t>(blockIdx.x) * kAppendWarps + warp) * 2;
    if (row0 >= total_rows) return;
    const int rows_here = row0 + 1 < total_rows ? 2 : 1;

    if constexpr (VEC) {
        const uint8_t* ksrc = static_cast<const uint8_t*>(p.key) + row0 * kRowBytes;
        const uint8_t* vsrc = static_cast<const uint8_t*>(p.value) + row0 * kRowBytes;
        const int bytes = rows_here * kRowBytes;
        constexpr int kIters = (2 * kRowBytes + 511) / 512;
        uint4 kr[kIters], vr[kIters];
#pragma unroll
        for (int it = 0; it < kIters; ++it) {
            const int off = it * 512 + lane * 16;
            if (off < bytes) {
                kr[it] = *reinterpret_cast<const uint4*>(ksrc + off);
                vr[it] = *reinterpret_cast<const uint4*>(vsrc + off);
            }
        }
#pragma unroll
        for (int it = 0; it < kIters; ++it) {
            const int off = it * 512 + lane * 16;
            if (off < bytes) {
                *reinterpret_cast<uint4*>(&in_stage[warp][0][off]) = kr[it];
                *reinterpret_cast<uint4*>(&in_stage[warp][1][off]) = vr[it];
            }
        }
        __syncwarp();
    }

    const uint32_t mode = p.view.quant_mode;
    const bool k_q8 = (mode == B200KV_Q8_F16 || mode == B200KV_Q8_Q8);
    const bool v_q8 = (mode == B200KV_F16_Q8 || mode == B200KV_Q8_Q8);
    const uint32_t nblk = D / p.view.qblock;

    for (int r = 0; r < rows_here; ++r) {
        const uint64_t row = row0 + r;
        const uint32_t token = static_cast<uint32_t>(row / H), head = static_cast<uint32_t>(row % H);
        const uint64_t position = static_cast<uint64_t>(base_position) + token;
        if (position >= capacity) continue;  // never write outside the cache

        float k[NJ], v[NJ];
        if constexpr (VEC) {
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                if (IN_F16) {
                    k[j] = __half2float(reinterpret_cast<const __half*>(&in_stage[warp][0][r * kRowBytes])[lane + 32 * j]);
                    v[j] = __half2float(reinterpret_cast<const __half*>(&in_stage[warp][1][r * kRowBytes])[lane + 32 * j]);
                } else {
                    k[j] = reinterpret_cast<const float*>(&in_stage[warp][0][r * kRowBytes])[lane + 32 * j];
                    v[j] = reinterpret_cast<const float*>(&in_stage[warp][1][r * kRowBytes])[lane + 32 * j];
                }
            }
        } else {
            const size_t in_base = static_cast<size_t>(row) * D;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                if (IN_F16) {
                    k[j] = __half2float(static_cast<const __half*>(p.key)[in_base + lane + 32 * j]);
                    v[j] = __half2float(static_cast<const __half*>(p.value)[in_base + lane + 32 * j]);
                } else {
                    k[j] = static_cast<const float*>(p.key)[in_base + lane + 32 * j];
                    v[j] = static_cast<const float*>(p.value)[in_base + lane + 32 * j];
                }
            }
        }

        transform_k_row<D>(k, lane, static_cast<uint32_t>(position), p.k_norm_weight, p.epsilon, p.rope_mode, p.inv_freq, p.sectioned_step);

        const size_t row_index = static_cast<size_t>(head) * capacity + position;
        if (k_q8) quantize_and_stage<NJ>(k, nblk == 1, lane, stage[warp][0],
                                         static_cast<__half*>(p.view.key_scales) + row_index * nblk);
        if (v_q8) quantize_and_stage<NJ>(v, nblk == 1, lane, stage[warp][1],
                                         static_cast<__half*>(p.view.value_scales) + row_index * nblk);
        __syncwarp();
        using word_t = typename std::conditional<D == 128, uint32_t, uint2>::type;
        if (k_q8) {
            reinterpret_cast<word_t*>(p.view.key_q8 + row_index * D)[lane] = reinterpret_cast<const word_t*>(stage[warp][0])[lane];
        } else {
            __half* dst = static_cast<__half*>(p.view.key_f16) + row_index * D;
#pragma unroll
            for (int j = 0; j < NJ; ++j) dst[lane + 32 * j] = __float2half_rn(k[j]);
        }
        if (v_q8) {
            reinterpret_cast<word_t*>(p.view.value_q8 + row_index * D)[lane] = reinterpret_cast<const word_t*>(stage[warp][1])[lane];
        } else {
            __half* dst = static_cast<__half*>(p.view.value_f16) + row_index * D;
#pragma unroll
            for (int j = 0; j < NJ; ++j) dst[lane + 32 * j] = __float2half_rn(v[j]);
        }
        __syncwarp();   // the staging rows are reused by the warp's second row
    }
}

}  // namespace b200kv

using namespace b200kv;

extern "C" int b200kv_append(const b200kv_view* view, const void* key, const void* value, int dtype,
                             const float* k_norm_weight, int rope_mode, float theta, float epsilon,
                             uint32_t token_count, uint32_t base_position,
                             const b200kv_prefill_state* prefill_state, const b200kv_decode_state* decode_state,
                             void* stream) {
    int rc = validate_view(view);
    if (rc != B200KV_OK) return rc;
    if (key == nullptr || value == nullptr || (dtype != B200KV_F16 && dtype != B200KV_F32)) return B200KV_ERR_INVALID;
    if (rope_mode < B200KV_ROPE_NONE || rope_mode > B200KV_ROPE_SECTIONED64) return B200KV_ERR_INVALID;
    if (!std::isfinite(theta) || !std::isfinite(epsilon)) return B200KV_ERR_INVALID;
    if (rope_mode != B200KV_ROPE_NONE && !(theta > 0.0f)) return B200KV_ERR_INVALID;
    if (token_count == 0) return B200KV_OK;
    if (prefill_state == nullptr && decode_state == nullptr &&
        static_cast<uint64_t>(base_position) + token_count > view->capacity)
        return B200KV_ERR_RANGE;
    rc = ensure_device();
    if (rc != B200KV_OK) return rc;

    AppendParams p{};
    p.view = *view;
    p.key = key;
    p.value = value;
    p.k_norm_weight = k_norm_weight;
    p.prefill_state = prefill_state;
    p.decode_state = decode_state;
    p.token_count = token_count;
    p.base_position = base_position;
    p.rope_mode = rope_mode;
    p.epsilon = epsilon;
    if (rope_mode == B200KV_ROPE_NEOX_FULL) {
        const uint32_t d = view->head_dim;
        for (uint32_t i = 0; i < d / 2; ++i)
            p.inv_freq[i] = std::pow(theta, -static_cast<float>(2 * i) / static_cast<float>(d));
    } else if (rope_mode == B200KV_ROPE_SECTIONED64) {
        p.sectioned_step = std::pow(theta, -2.0f / 64.0f);
    }

    const uint64_t rows = static_cast<uint64_t>(token_count) * view->kv_heads;
    const unsigned grid = static_cast<unsigned>((rows + 2 * kAppendWarps - 1) / (2 * kAppendWarps));   // two rows per warp
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool f16 = (dtype == B200KV_F16);
    const bool vec = ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value)) & 15u) == 0;   // 16-byte loads need aligned inputs
    const dim3 block(kAppendWarps * 32);
    cudaError_t err;
    auto launch = [&](auto kernel) { return launch_kernel(kernel, grid, block, 0, s, true, p); };
    if (view->head_dim == 128) {
        if (vec) err = f16 ? launch(append_kernel<128, true, true>) : launch(append_kernel<128, false, true>);
        else err = f16 ? launch(append_kernel<128, true, false>) : launch(append_kernel<128, false, false>);
    } else {
        if (vec) err = f16 ? launch(append_kernel<256, true, true>) : launch(append_kernel<256, false, true>);
        else err = f16 ? launch(append_kernel<256, true, false>) : launch(append_kernel<256, false, false>);
    }
    B200KV_CUDA_TRY(err);
    return B200KV_OK;
}
