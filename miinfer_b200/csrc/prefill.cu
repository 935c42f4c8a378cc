// Suffix / prefill cross-query attention over a quantized prefix: entry point.
//
// Replaces launch_qwen35_splitk_suffix_attention_quant
// (include/miinfer/qwen3_gpu_primitives.hpp:670-692).  Query token t attends
// cache positions [0, base_position + t + 1) -- the chunk has been appended
// before this call (src/prefill_v2/attention_layer.cpp:297-343), so causality
// inside the chunk is just the per-token length (.hip:6829).
#include "decode_common.cuh"

#include <cmath>

using namespace b200kv;

extern "C" {

size_t b200kv_prefill_workspace_bytes(uint32_t token_count, uint32_t query_heads, uint32_t head_dim) {
    return b200kv_decode_workspace_bytes(query_heads, head_dim, token_count ? token_count : 1);
}

int b200kv_prefill_attn(const b200kv_view* view, const void* q, int q_dtype, const float* gate,
                        float* gated_output, uint32_t token_count, uint32_t base_position,
                        uint32_t query_heads, float scale, const b200kv_prefill_state* prefill_state,
                        void* workspace, size_t workspace_bytes, void* stream) {
    int rc = validate_view(view);
    if (rc != B200KV_OK) return rc;
    if (q == nullptr || gated_output == nullptr || token_count == 0) return B200KV_ERR_INVALID;
    if (q_dtype != B200KV_F16 && q_dtype != B200KV_F32) return B200KV_ERR_INVALID;
    if (query_heads == 0 || query_heads % view->kv_heads != 0 || !std::isfinite(scale)) return B200KV_ERR_INVALID;
    if (query_heads / view->kv_heads > 8 || token_count > 65535) return B200KV_ERR_UNSUPPORTED;
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    DecodeParams p{};
    p.view = *view;
    p.causal = 1;
    p.causal_base = base_position;
    p.prefill_state = prefill_state;
    p.sessions = token_count;
    p.q = q;
    p.q_is_f16 = (q_dtype == B200KV_F16);
    p.query_heads = query_heads;
    p.scale = scale;
    uint64_t max_length = prefill_state ? view->capacity : static_cast<uint64_t>(base_position) + token_count;
    if (max_length > view->capacity) max_length = view->capacity;
    MergeParams mp{};
    mp.query_heads = query_heads;
    mp.head_dim = view->head_dim;
    mp.gate = gate;
    mp.gated_output = gated_output;
    return run_decode(p, *view, static_cast<uint32_t>(max_length), workspace, workspace_bytes, B200KV_SPLITS_FORCE_GENERIC, mp,
                      token_count, s);
}

}  // extern "C"
