// Suffix / prefill cross-query attention over a quantized prefix: entry point.
//
// Replaces launch_qwen35_splitk_suffix_attention_quant
// (include/miinfer/qwen3_gpu_primitives.hpp:670-692).  Query token t attends
// cache positions [0, base_position + t + 1) -- the chunk has been appended
// before this call (src/prefill_v2/attention_layer.cpp:297-343), so causality
// inside the chunk is just the per-token length (.hip:6829).  Two kernels:
// prefill_tc5.cu (tcgen05/TMEM/TMA; needs an fp16 scratch of the visible prefix
// in the caller's workspace, b200kv_prefill_scratch_bytes) and prefill_mma.cu
// (mma.sync, running state in registers, no workspace at all).  The reference
// needs 405.8 MB of split partials at 512 tokens (src/prefill_v2/workspace.cpp:67-70).
#include "decode_common.cuh"

#include <cmath>

namespace b200kv {
size_t prefill_tc5_workspace_bytes(uint32_t rows, uint32_t kv_heads, uint32_t head_dim);
size_t prefill_tc5_split_bytes(uint32_t token_count, uint32_t query_heads, uint32_t kv_heads, uint32_t head_dim, uint32_t splits);
int launch_prefill_tc5(const b200kv_view& view, const void* q, int q_is_f16, const float* gate, float* out,
                       uint32_t token_count, uint32_t base_position, const b200kv_prefill_state* prefill_state,
                       uint32_t query_heads, float scale, void* workspace, size_t workspace_bytes, uint32_t prepared_rows,
                       cudaStream_t stream);
int launch_prefill_tc5_prepare(const b200kv_view& view, uint32_t prepared_rows, uint64_t rows, void* workspace, size_t workspace_bytes,
                               cudaStream_t stream);
int launch_prefill_mma(const b200kv_view& view, const void* q, int q_is_f16, const float* gate, float* out,
                       uint32_t token_count, uint32_t base_position, const b200kv_prefill_state* prefill_state,
                       uint32_t query_heads, float scale, cudaStream_t stream);
}

using namespace b200kv;

extern "C" {

size_t b200kv_prefill_workspace_bytes(uint32_t, uint32_t, uint32_t) { return 0; }

size_t b200kv_prefill_scratch_bytes(uint64_t rows, uint32_t kv_heads, uint32_t head_dim) {
    return prefill_tc5_workspace_bytes(static_cast<uint32_t>(rows), kv_heads, head_dim);
}

size_t b200kv_prefill_split_bytes(uint32_t token_count, uint32_t query_heads, uint32_t kv_heads, uint32_t head_dim) {
    return prefill_tc5_split_bytes(token_count, query_heads, kv_heads, head_dim, 8) + 2048;   // up to 8 splits, alignment slack
}

int b200kv_prefill_prepare(const b200kv_view* view, uint32_t prepared_rows, uint64_t rows, void* workspace, size_t workspace_bytes,
                           void* stream) {
    int rc = validate_view(view);
    if (rc != B200KV_OK) return rc;
    if (view->head_dim != 128 && view->head_dim != 256) return B200KV_ERR_UNSUPPORTED;
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    return launch_prefill_tc5_prepare(*view, prepared_rows, rows, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int b200kv_prefill_attn(const b200kv_view* view, const void* q, int q_dtype, const float* gate,
                        float* gated_output, uint32_t token_count, uint32_t base_position,
                        uint32_t query_heads, float scale, const b200kv_prefill_state* prefill_state,
                        void* workspace, size_t workspace_bytes, void* stream) {
    return b200kv_prefill_attn_prepared(view, q, q_dtype, gate, gated_output, token_count, base_position, query_heads, scale,
                                        prefill_state, workspace, workspace_bytes, 0, stream);
}

int b200kv_prefill_attn_prepared(const b200kv_view* view, const void* q, int q_dtype, const float* gate,
                                 float* gated_output, uint32_t token_count, uint32_t base_position,
                                 uint32_t query_heads, float scale, const b200kv_prefill_state* prefill_state,
                                 void* workspace, size_t workspace_bytes, uint32_t prepared_rows, void* stream) {
    int rc = validate_view(view);
    if (rc != B200KV_OK) return rc;
    if (q == nullptr || gated_output == nullptr || token_count == 0) return B200KV_ERR_INVALID;
    if (q_dtype != B200KV_F16 && q_dtype != B200KV_F32) return B200KV_ERR_INVALID;
    if (query_heads == 0 || query_heads % view->kv_heads != 0 || !std::isfinite(scale)) return B200KV_ERR_INVALID;
    if (static_cast<uint64_t>(token_count) * (query_heads / view->kv_heads) > 0x7fffffffull) return B200KV_ERR_UNSUPPORTED;
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    // tcgen05 path when the caller provides the fp16 scratch; otherwise the register-resident mma.sync kernel
    rc = launch_prefill_tc5(*view, q, q_dtype == B200KV_F16, gate, gated_output, token_count, base_position, prefill_state, query_heads,
                            scale, workspace, workspace_bytes, prepared_rows, static_cast<cudaStream_t>(stream));
    if (rc != B200KV_ERR_UNSUPPORTED) return rc;
    return launch_prefill_mma(*view, q, q_dtype == B200KV_F16, gate, gated_output, token_count, base_position, prefill_state,
                              query_heads, scale, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
