// The two small operators next to the KV path in a decode or prefill step:
//
//  * the query side of an attention layer -- de-interleave the projection output [token][heads][q | gate], RMSNorm x
//    weight on q, RoPE at the token's position, write q and gate -- MIInfer's
//    qwen35_decoupled_q_split_norm_rope_batch_kernel (gfx906/kernels/qwen3_primitives.hip:994-1045) and its
//    single-token twin qwen35_fused_q_split_norm_rope_kernel (.hip:661-717).  The row arithmetic is the append
//    kernel's (append_row.cuh), so a query and the key appended at the same position are rotated by identical bits;
//  * the device-side step bookkeeping of a replayed decode graph, qwen35_decode_state_advance_kernel (.hip:4417-4428).
#include "append_row.cuh"

#include <cmath>

namespace b200kv {

struct QSideParams {
    const void* qfull;       // [token][heads][2 * D] of fp16 or fp32
    const float* q_norm_weight;
    void* query;             // [token][heads][D] of fp16 or fp32
    float* gate;             // [token][heads][D] fp32, or null
    const b200kv_prefill_state* prefill_state;
    const b200kv_decode_state* decode_state;
    uint32_t token_count, base_position, heads;
    int rope_mode;
    float epsilon, sectioned_step;
    float inv_freq[128];
};

constexpr int kQSideWarps = 4;

// One warp per (token, head) row; lane L holds elements L, L + 32, ...
template <int D, bool IN_F16, bool OUT_F16>
__global__ void __launch_bounds__(kQSideWarps * 32) q_split_norm_rope_kernel(const __grid_constant__ QSideParams p) {
    constexpr int NJ = D / 32;
    pdl_launch_dependents();
    pdl_wait();   // the projection output and the device-side position come from preceding kernels
    uint32_t base_position = p.base_position, token_count = p.token_count;
    if (p.prefill_state != nullptr) {
        base_position = p.prefill_state->base_position;
        token_count = min(token_count, p.prefill_state->token_count);
    } else if (p.decode_state != nullptr) {
        base_position = p.decode_state->position;
        token_count = min(token_count, 1u);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * kQSideWarps + warp;
    if (row >= static_cast<uint64_t>(token_count) * p.heads) return;
    const uint32_t token = static_cast<uint32_t>(row / p.heads);
    const size_t in_base = static_cast<size_t>(row) * 2 * D, out_base = static_cast<size_t>(row) * D;
    float q[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        float g;
        if (IN_F16) {
            q[j] = __half2float(static_cast<const __half*>(p.qfull)[in_base + lane + 32 * j]);
            g = __half2float(static_cast<const __half*>(p.qfull)[in_base + D + lane + 32 * j]);
        } else {
            q[j] = static_cast<const float*>(p.qfull)[in_base + lane + 32 * j];
            g = static_cast<const float*>(p.qfull)[in_base + D + lane + 32 * j];
        }
        if (p.gate != nullptr) p.gate[out_base + lane + 32 * j] = g;
    }
    transform_k_row<D>(q, lane, base_position + token, p.q_norm_weight, p.epsilon, p.rope_mode, p.inv_freq, p.sectioned_step);
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        if (OUT_F16) static_cast<__half*>(p.query)[out_base + lane + 32 * j] = __float2half_rn(q[j]);
        else static_cast<float*>(p.query)[out_base + lane + 32 * j] = q[j];
    }
}

__global__ void decode_state_advance_kernel(b200kv_decode_state* state, uint32_t* token_output, uint32_t capacity) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    pdl_wait();
    const uint32_t generated = state->generated;
    if (generated < capacity) token_output[generated] = state->current_token;
    state->stop = (state->stop || state->current_token == 151643u || state->current_token == 151645u ||
                   generated + 1 >= state->max_generated) ? 1u : 0u;
    state->position += 1;
    state->generated = generated + 1;
}

template <int D>
static cudaError_t launch_qside(const QSideParams& p, bool in_f16, bool out_f16, unsigned grid, cudaStream_t s) {
    const dim3 block(kQSideWarps * 32);
    if (in_f16) return out_f16 ? launch_kernel(q_split_norm_rope_kernel<D, true, true>, grid, block, 0, s, true, p)
                               : launch_kernel(q_split_norm_rope_kernel<D, true, false>, grid, block, 0, s, true, p);
    return out_f16 ? launch_kernel(q_split_norm_rope_kernel<D, false, true>, grid, block, 0, s, true, p)
                   : launch_kernel(q_split_norm_rope_kernel<D, false, false>, grid, block, 0, s, true, p);
}

}  // namespace b200kv

using namespace b200kv;

extern "C" {

int b200kv_q_split_norm_rope(const void* qfull, int in_dtype, const float* q_norm_weight, void* query, int out_dtype, float* gate,
                             uint32_t token_count, uint32_t base_position, uint32_t heads, uint32_t head_dim, int rope_mode,
                             float theta, float epsilon, const b200kv_prefill_state* prefill_state,
                             const b200kv_decode_state* decode_state, void* stream) {
    if (qfull == nullptr || query == nullptr || heads == 0) return B200KV_ERR_INVALID;
    if ((in_dtype != B200KV_F16 && in_dtype != B200KV_F32) || (out_dtype != B200KV_F16 && out_dtype != B200KV_F32)) return B200KV_ERR_INVALID;
    if (head_dim != 128 && head_dim != 256) return B200KV_ERR_UNSUPPORTED;
    if (rope_mode < B200KV_ROPE_NONE || rope_mode > B200KV_ROPE_SECTIONED64) return B200KV_ERR_INVALID;
    if (!std::isfinite(theta) || !std::isfinite(epsilon) || (rope_mode != B200KV_ROPE_NONE && !(theta > 0.0f))) return B200KV_ERR_INVALID;
    if (token_count == 0) return B200KV_OK;
    int rc = ensure_device();
    if (rc != B200KV_OK) return rc;
    QSideParams p{};
    p.qfull = qfull;
    p.q_norm_weight = q_norm_weight;
    p.query = query;
    p.gate = gate;
    p.prefill_state = prefill_state;
    p.decode_state = decode_state;
    p.token_count = token_count;
    p.base_position = base_position;
    p.heads = heads;
    p.rope_mode = rope_mode;
    p.epsilon = epsilon;
    rope_constants(rope_mode, theta, head_dim, p.inv_freq, &p.sectioned_step);
    const uint64_t rows = static_cast<uint64_t>(token_count) * heads;
    const unsigned grid = static_cast<unsigned>((rows + kQSideWarps - 1) / kQSideWarps);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const cudaError_t err = head_dim == 128 ? launch_qside<128>(p, in_dtype == B200KV_F16, out_dtype == B200KV_F16, grid, s)
                                            : launch_qside<256>(p, in_dtype == B200KV_F16, out_dtype == B200KV_F16, grid, s);
    B200KV_CUDA_TRY(err);
    return B200KV_OK;
}

int b200kv_decode_state_advance(b200kv_decode_state* state, uint32_t* token_output, uint32_t capacity, void* stream) {
    // the reference launcher aborts on these (gfx906/kernels/qwen3_primitives.hip:5981-5983)
    if (state == nullptr || token_output == nullptr || capacity == 0) return B200KV_ERR_INVALID;
    int rc = ensure_device();
    if (rc != B200KV_OK) return rc;
    B200KV_CUDA_TRY(launch_kernel(decode_state_advance_kernel, dim3(1), dim3(1), 0, static_cast<cudaStream_t>(stream), true, state,
                                  token_output, capacity));
    return B200KV_OK;
}

}  // extern "C"
