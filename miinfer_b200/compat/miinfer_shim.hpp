// miinfer_shim.hpp -- the reference's operator names over the B200 C ABI.
//
// A MIInfer build that includes this header instead of the HIP declarations of
// include/miinfer/qwen3_gpu_primitives.hpp:670-739 and
// include/miinfer/prefill_v2/kv_cache.hpp keeps its call sites
// (src/prefill_v2/attention_layer.cpp:297,333,599,613,634) unchanged: same
// function names, same argument order and meaning, `hipStream_t` spelled
// `cudaStream_t`.  Differences a caller can observe:
//   * a bad argument throws std::runtime_error (the reference aborts the process);
//   * head_dim 128 and 256, any kv_heads, and q8_0 blocks (kQBlock) are accepted;
//   * the decode launcher takes a caller-owned workspace through
//     set_decode_workspace() instead of file-scope device arrays;
//   * k_norm_weight may be null; gate may be null.
// Header-only; link with libb200kv.so.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "b200kv.h"

namespace miinfer {

using DeviceDecodeState = b200kv_decode_state;    // qwen3_gpu_primitives.hpp:30-37
using DevicePrefillState = b200kv_prefill_state;  // qwen3_gpu_primitives.hpp:39-45

namespace shim_detail {
inline void check(int status, const char* where) {
    if (status != B200KV_OK)
        throw std::runtime_error(std::string(where) + ": " + b200kv_status_string(status) + " " + b200kv_last_cuda_error());
}
struct Workspace { void* ptr = nullptr; std::size_t bytes = 0; };
inline Workspace& decode_workspace() { static thread_local Workspace w; return w; }
inline b200kv_view make_view(const __half* kf, const __half* vf, const int8_t* kq, const __half* ks, const int8_t* vq,
                             const __half* vs, std::uint32_t capacity, std::uint32_t kv_heads, std::uint32_t head_dim,
                             std::uint32_t qblock, bool is_k_q8, bool is_v_q8) {
    b200kv_view v{};
    v.key_f16 = const_cast<__half*>(kf); v.value_f16 = const_cast<__half*>(vf);
    v.key_q8 = const_cast<int8_t*>(kq); v.key_scales = const_cast<__half*>(ks);
    v.value_q8 = const_cast<int8_t*>(vq); v.value_scales = const_cast<__half*>(vs);
    v.capacity = capacity; v.kv_heads = kv_heads; v.head_dim = head_dim; v.qblock = qblock ? qblock : head_dim;
    v.quant_mode = (is_k_q8 ? 1u : 0u) | (is_v_q8 ? 2u : 0u);
    return v;
}
}  // namespace shim_detail

// Scale-block width used by the launchers below: 0 = one scale per head row (the reference's format), 32 = q8_0.
inline std::uint32_t& kv_qblock() { static thread_local std::uint32_t qb = 0; return qb; }

// The decode launcher needs split-K scratch; the reference hides it in file-scope device arrays
// (gfx906/kernels/qwen3_primitives.hip:2111-2113).  Size it with b200kv_decode_workspace_bytes and zero it once.
inline void set_decode_workspace(void* device_ptr, std::size_t bytes) { shim_detail::decode_workspace() = {device_ptr, bytes}; }

// qwen3_gpu_primitives.hpp:695-716
inline void launch_qwen35_decoupled_k_norm_rope_kv_store_batch_quant(
    const float* key, const float* value, const float* k_norm_weight, __half* key_cache_f16, __half* value_cache_f16,
    int8_t* key_cache_q8, __half* key_scales, int8_t* value_cache_q8, __half* value_scales, std::uint32_t token_count,
    std::uint32_t base_position, std::uint32_t cache_capacity, std::uint32_t kv_heads, std::uint32_t head_dim, float theta,
    float epsilon, bool is_k_q8, bool is_v_q8, cudaStream_t stream = nullptr, const DevicePrefillState* prefill_state = nullptr,
    const DeviceDecodeState* decode_state = nullptr) {
    const b200kv_view v = shim_detail::make_view(key_cache_f16, value_cache_f16, key_cache_q8, key_scales, value_cache_q8,
                                                 value_scales, cache_capacity, kv_heads, head_dim, kv_qblock(), is_k_q8, is_v_q8);
    shim_detail::check(b200kv_append(&v, key, value, B200KV_F32, k_norm_weight, B200KV_ROPE_SECTIONED64, theta, epsilon, token_count,
                                     base_position, prefill_state, decode_state, stream),
                       "launch_qwen35_decoupled_k_norm_rope_kv_store_batch_quant");
}

// Q8_1Block (include/miinfer/q4_q8_gemv.hpp:23-27): the 36-byte activation block the projections consume
using Q8_1Block = b200kv_q8_1_block;

// qwen3_gpu_primitives.hpp:719-739
inline void launch_qwen35_tiled_online_attention_quant_dynamic(
    const float* q, const __half* key_cache_f16, const __half* value_cache_f16, const int8_t* key_cache_q8, const __half* key_scales,
    const int8_t* value_cache_q8, const __half* value_scales, const DeviceDecodeState* decode_state, std::uint32_t cache_capacity,
    float* output, const float* gate, float* gated_output, std::uint32_t query_heads, std::uint32_t kv_heads, std::uint32_t head_dim,
    float scale, bool is_k_q8, bool is_v_q8, cudaStream_t stream = nullptr, Q8_1Block* gated_output_q8 = nullptr) {
    if (decode_state == nullptr) shim_detail::check(B200KV_ERR_INVALID, "launch_qwen35_tiled_online_attention_quant_dynamic");
    const b200kv_view v = shim_detail::make_view(key_cache_f16, value_cache_f16, key_cache_q8, key_scales, value_cache_q8,
                                                 value_scales, cache_capacity, kv_heads, head_dim, kv_qblock(), is_k_q8, is_v_q8);
    const auto& ws = shim_detail::decode_workspace();
    shim_detail::check(b200kv_decode_attn(&v, q, B200KV_F32, gate, output, gated_output, gated_output_q8, query_heads, scale, 0,
                                          decode_state, ws.ptr, ws.bytes, 0, stream),
                       "launch_qwen35_tiled_online_attention_quant_dynamic");
}

// qwen3_gpu_primitives.hpp:670-692.  d_split_workspace is sized by the reference's contract,
// num_splits * token_count * query_heads * (2 + head_dim) floats (gfx906/kernels/qwen3_primitives.hip:7154-7157); when
// that is enough for the fp16 scratch of the visible prefix the tcgen05 kernel uses it, otherwise (or when it is null)
// the register-resident kernel runs.
inline void launch_qwen35_splitk_suffix_attention_quant(
    const float* q, const __half* key_cache_f16, const __half* value_cache_f16, const int8_t* key_cache_q8, const __half* key_scales,
    const int8_t* value_cache_q8, const __half* value_scales, const float* gate, float* gated_output, float* d_split_workspace,
    std::uint32_t token_count, std::uint32_t base_position, std::uint32_t cache_capacity, std::uint32_t query_heads,
    std::uint32_t kv_heads, std::uint32_t head_dim, float scale, bool is_k_q8, bool is_v_q8, std::uint32_t num_splits = 64,
    cudaStream_t stream = nullptr, const DevicePrefillState* prefill_state = nullptr) {
    const b200kv_view v = shim_detail::make_view(key_cache_f16, value_cache_f16, key_cache_q8, key_scales, value_cache_q8,
                                                 value_scales, cache_capacity, kv_heads, head_dim, kv_qblock(), is_k_q8, is_v_q8);
    shim_detail::check(b200kv_prefill_attn(&v, q, B200KV_F32, gate, gated_output, token_count, base_position, query_heads, scale,
                                           prefill_state, d_split_workspace,
                                           d_split_workspace ? static_cast<std::size_t>(num_splits ? (num_splits > 64 ? 64 : num_splits) : 64) * token_count *
                                                                   query_heads * (2 + head_dim) * sizeof(float)
                                                             : 0,
                                           stream),
                       "launch_qwen35_splitk_suffix_attention_quant");
}

// qwen3_gpu_primitives.hpp:869-881: the query side of a prefill chunk (sectioned RoPE on the first 64 dims)
inline void launch_qwen35_decoupled_q_split_norm_rope_batch(
    const float* qfull, const float* q_norm_weight, float* query_rope, float* gate, std::uint32_t token_count, std::uint32_t base_position,
    std::uint32_t heads, std::uint32_t head_dim, float theta, float epsilon, cudaStream_t stream = nullptr,
    const DevicePrefillState* prefill_state = nullptr) {
    shim_detail::check(b200kv_q_split_norm_rope(qfull, B200KV_F32, q_norm_weight, query_rope, B200KV_F32, gate, token_count, base_position, heads,
                                                head_dim, B200KV_ROPE_SECTIONED64, theta, epsilon, prefill_state, nullptr, stream),
                       "launch_qwen35_decoupled_q_split_norm_rope_batch");
}

// qwen3_gpu_primitives.hpp:934-938: the query side of a decode step, position read from the device state
inline void launch_qwen35_fused_q_split_norm_rope_dynamic(
    const float* qfull, const float* q_norm_weight, float* query_rope, float* gate, std::uint32_t heads, std::uint32_t head_dim,
    const DeviceDecodeState* decode_state, float theta, float epsilon, cudaStream_t stream = nullptr) {
    if (decode_state == nullptr) shim_detail::check(B200KV_ERR_INVALID, "launch_qwen35_fused_q_split_norm_rope_dynamic");
    shim_detail::check(b200kv_q_split_norm_rope(qfull, B200KV_F32, q_norm_weight, query_rope, B200KV_F32, gate, 1, 0, heads, head_dim,
                                                B200KV_ROPE_SECTIONED64, theta, epsilon, nullptr, decode_state, stream),
                       "launch_qwen35_fused_q_split_norm_rope_dynamic");
}

// qwen3_gpu_primitives.hpp:1248-1250
inline void launch_qwen35_decode_state_advance(DeviceDecodeState* state, std::uint32_t* token_output, std::uint32_t capacity,
                                               cudaStream_t stream = nullptr) {
    shim_detail::check(b200kv_decode_state_advance(state, token_output, capacity, stream), "launch_qwen35_decode_state_advance");
}

namespace prefill_v2 {

enum class KvCacheQuantMode : std::uint8_t { kFp16Fp16 = 0, kQ8Fp16 = 1, kFp16Q8 = 2, kQ8Q8 = 3 };   // kv_cache.hpp:16-21

struct AttentionKvCacheView {   // kv_cache.hpp:24-46
    __half* key_cache = nullptr;
    __half* value_cache = nullptr;
    int8_t* key_cache_q8 = nullptr;
    __half* key_scales = nullptr;
    int8_t* value_cache_q8 = nullptr;
    __half* value_scales = nullptr;
    std::size_t capacity = 0;
    std::size_t head_count_kv = 4;
    std::size_t head_dim = 256;
    KvCacheQuantMode quant_mode = KvCacheQuantMode::kFp16Fp16;
    std::size_t qblock = 256;   // not in the reference: 32 selects q8_0 blocks
    [[nodiscard]] bool is_k_q8() const noexcept { return quant_mode == KvCacheQuantMode::kQ8Fp16 || quant_mode == KvCacheQuantMode::kQ8Q8; }
    [[nodiscard]] bool is_v_q8() const noexcept { return quant_mode == KvCacheQuantMode::kFp16Q8 || quant_mode == KvCacheQuantMode::kQ8Q8; }
};

class AttentionLayerKvCacheStorage {   // kv_cache.hpp:49-122
public:
    explicit AttentionLayerKvCacheStorage(std::size_t capacity = 8192, KvCacheQuantMode quant_mode = KvCacheQuantMode::kFp16Fp16,
                                          std::size_t kv_heads = 4, std::size_t head_dim = 256, std::size_t qblock = 0) {
        if (capacity == 0) throw std::runtime_error("AttentionLayerKvCacheStorage: capacity must be > 0");
        shim_detail::check(b200kv_cache_create(&cache_, capacity, static_cast<std::uint32_t>(kv_heads), static_cast<std::uint32_t>(head_dim),
                                               static_cast<std::uint32_t>(qblock ? qblock : head_dim), static_cast<std::uint32_t>(quant_mode)),
                           "AttentionLayerKvCacheStorage");
        b200kv_cache_view(cache_, &view_);
    }
    ~AttentionLayerKvCacheStorage() { b200kv_cache_destroy(cache_); }
    AttentionLayerKvCacheStorage(const AttentionLayerKvCacheStorage&) = delete;
    AttentionLayerKvCacheStorage& operator=(const AttentionLayerKvCacheStorage&) = delete;
    AttentionLayerKvCacheStorage(AttentionLayerKvCacheStorage&& o) noexcept : cache_(std::exchange(o.cache_, nullptr)), view_(o.view_) {}
    AttentionLayerKvCacheStorage& operator=(AttentionLayerKvCacheStorage&& o) noexcept {
        if (this != &o) { b200kv_cache_destroy(cache_); cache_ = std::exchange(o.cache_, nullptr); view_ = o.view_; }
        return *this;
    }
    void reset(cudaStream_t stream = nullptr) { shim_detail::check(b200kv_cache_reset(cache_, stream), "reset"); }
    [[nodiscard]] std::size_t raw_tokens_bytes(std::size_t tokens) const noexcept { return b200kv_snapshot_bytes(&view_, tokens); }
    void download_raw(void* host_dst, std::size_t tokens, cudaStream_t stream = nullptr) const {
        if (tokens > view_.capacity) throw std::runtime_error("AttentionLayerKvCacheStorage::download_raw: tokens exceeds capacity");
        shim_detail::check(b200kv_snapshot_save(&view_, tokens, host_dst, stream), "download_raw");
        if (stream == nullptr) cudaStreamSynchronize(nullptr);   // the reference's null-stream path is blocking
    }
    void upload_raw(const void* host_src, std::size_t tokens, cudaStream_t stream = nullptr) {
        if (tokens > view_.capacity) throw std::runtime_error("AttentionLayerKvCacheStorage::upload_raw: tokens exceeds capacity");
        shim_detail::check(b200kv_snapshot_restore(&view_, tokens, host_src, stream), "upload_raw");
        if (stream == nullptr) cudaStreamSynchronize(nullptr);
    }
    // kv_cache.cpp:132-212: dequantising downloads to fp32 host vectors [kv_head][tokens][head_dim]
    void download_key(std::vector<float>& host_key, std::size_t tokens) const {
        if (tokens > view_.capacity) throw std::runtime_error("AttentionLayerKvCacheStorage: tokens exceeds capacity");
        host_key.resize(static_cast<std::size_t>(view_.kv_heads) * tokens * view_.head_dim);
        shim_detail::check(b200kv_download_key(&view_, tokens, host_key.data(), nullptr), "download_key");
    }
    void download_value(std::vector<float>& host_value, std::size_t tokens) const {
        if (tokens > view_.capacity) throw std::runtime_error("AttentionLayerKvCacheStorage: tokens exceeds capacity");
        host_value.resize(static_cast<std::size_t>(view_.kv_heads) * tokens * view_.head_dim);
        shim_detail::check(b200kv_download_value(&view_, tokens, host_value.data(), nullptr), "download_value");
    }
    [[nodiscard]] AttentionKvCacheView view() const noexcept {
        AttentionKvCacheView v;
        v.key_cache = static_cast<__half*>(view_.key_f16); v.value_cache = static_cast<__half*>(view_.value_f16);
        v.key_cache_q8 = view_.key_q8; v.key_scales = static_cast<__half*>(view_.key_scales);
        v.value_cache_q8 = view_.value_q8; v.value_scales = static_cast<__half*>(view_.value_scales);
        v.capacity = view_.capacity; v.head_count_kv = view_.kv_heads; v.head_dim = view_.head_dim;
        v.quant_mode = static_cast<KvCacheQuantMode>(view_.quant_mode); v.qblock = view_.qblock;
        return v;
    }
    [[nodiscard]] std::size_t capacity() const noexcept { return view_.capacity; }
    [[nodiscard]] KvCacheQuantMode quant_mode() const noexcept { return static_cast<KvCacheQuantMode>(view_.quant_mode); }
    [[nodiscard]] std::size_t total_bytes() const noexcept {
        return b200kv_cache_bytes(view_.capacity, view_.kv_heads, view_.head_dim, view_.qblock, view_.quant_mode);
    }
    [[nodiscard]] const b200kv_view& raw_view() const noexcept { return view_; }

private:
    b200kv_cache* cache_ = nullptr;
    b200kv_view view_{};
};


// Steps 3-5 of PrefillV2AttentionLayer::forward and ::decode (src/prefill_v2/attention_layer.cpp:291-349, 587-656): the
// query-side split / norm / RoPE, the KV store, and the attention over the cache -- the part of the layer executor that
// is the KV path.  The projections before (steps 1-2) and after (step 6 on) stay with the caller.  Buffers are the
// caller's, named as in PrefillV2Workspace (src/prefill_v2/workspace.hpp:15-60).
struct AttentionKvPathBuffers {
    const float* attn_qfull = nullptr;       // [token][q_heads][q | gate] from the Q projection
    const float* attn_k = nullptr;           // [token][kv_heads * head_dim]
    const float* attn_v = nullptr;
    float* attn_q_rope = nullptr;            // [token][q_heads][head_dim]
    float* gate = nullptr;
    float* attn_gated_output = nullptr;
    Q8_1Block* attn_gated_output_q8 = nullptr;   // decode only, optional: the input format of the output projection
    float* splitk_attn_workspace = nullptr;  // optional scratch of the suffix kernel (b200kv_prefill_scratch_bytes)
    std::size_t splitk_attn_workspace_bytes = 0;
};

class AttentionLayerKvPath {
public:
    AttentionLayerKvPath(const float* d_q_norm, const float* d_k_norm, std::uint32_t q_heads = 24, std::uint32_t kv_heads = 4,
                         std::uint32_t head_dim = 256, float rope_theta = 1.0e6f, float rms_epsilon = 1.0e-6f)
        : q_norm_(d_q_norm), k_norm_(d_k_norm), q_heads_(q_heads), kv_heads_(kv_heads), head_dim_(head_dim), theta_(rope_theta), eps_(rms_epsilon) {}

    // attention_layer.cpp:291-349.  The chunk is stored first and attended second; causality inside the chunk is the
    // per-token length.  The reference picks between three attention kernels here (a query-tiled fp16 kernel, the
    // split-K suffix kernel when token_count <= 512 behind a prefix or under a device-side state, a cold-prefill fp16
    // kernel otherwise); this library has one entry point for all of those cases and picks its kernel by the workspace.
    void forward(const AttentionKvCacheView& kv_cache, const AttentionKvPathBuffers& ws, std::uint32_t token_count, std::uint32_t base_position,
                 cudaStream_t stream = nullptr, const DevicePrefillState* prefill_state = nullptr) const {
        launch_qwen35_decoupled_q_split_norm_rope_batch(ws.attn_qfull, q_norm_, ws.attn_q_rope, ws.gate, token_count, base_position, q_heads_,
                                                        head_dim_, theta_, eps_, stream, prefill_state);
        store(kv_cache, ws, token_count, base_position, stream, prefill_state, nullptr);
        const b200kv_view v = raw(kv_cache);
        shim_detail::check(b200kv_prefill_attn(&v, ws.attn_q_rope, B200KV_F32, ws.gate, ws.attn_gated_output, token_count, base_position, q_heads_,
                                               scale(), prefill_state, ws.splitk_attn_workspace, ws.splitk_attn_workspace_bytes, stream),
                           "AttentionLayerKvPath::forward");
    }

    // attention_layer.cpp:587-656.  With a device-side state (graph replay) the query side, the store and the attention
    // all read the position on the device; the attention covers positions [0, position], i.e. position + 1 entries
    // (the reference's host-position branch passes position + 1 as the BASE of a one-token suffix call and so attends
    // one slot too many, :646; that is not reproduced).
    void decode(const AttentionKvCacheView& kv_cache, const AttentionKvPathBuffers& ws, std::uint32_t position, cudaStream_t stream = nullptr,
                const DeviceDecodeState* decode_state = nullptr) const {
        if (decode_state != nullptr)
            launch_qwen35_fused_q_split_norm_rope_dynamic(ws.attn_qfull, q_norm_, ws.attn_q_rope, ws.gate, q_heads_, head_dim_, decode_state, theta_,
                                                          eps_, stream);
        else
            launch_qwen35_decoupled_q_split_norm_rope_batch(ws.attn_qfull, q_norm_, ws.attn_q_rope, ws.gate, 1, position, q_heads_, head_dim_, theta_,
                                                            eps_, stream);
        const b200kv_view v = raw(kv_cache);
        const auto& dws = shim_detail::decode_workspace();
        // store + attention as ONE launch where the cache takes the streaming kernel, as two otherwise (b200kv_decode_step decides)
        shim_detail::check(b200kv_decode_step(&v, ws.attn_k, ws.attn_v, B200KV_F32, k_norm_, B200KV_ROPE_SECTIONED64, theta_, eps_, ws.attn_q_rope,
                                              B200KV_F32, ws.gate, nullptr, ws.attn_gated_output, ws.attn_gated_output_q8, q_heads_, scale(), position,
                                              decode_state, dws.ptr, dws.bytes, 0, stream),
                           "AttentionLayerKvPath::decode");
    }

private:
    void store(const AttentionKvCacheView& c, const AttentionKvPathBuffers& ws, std::uint32_t token_count, std::uint32_t base_position,
               cudaStream_t stream, const DevicePrefillState* ps, const DeviceDecodeState* ds) const {
        const b200kv_view v = raw(c);   // launch_qwen35_decoupled_k_norm_rope_kv_store_batch_quant with the view's own scale-block width
        shim_detail::check(b200kv_append(&v, ws.attn_k, ws.attn_v, B200KV_F32, k_norm_, B200KV_ROPE_SECTIONED64, theta_, eps_, token_count, base_position,
                                         ps, ds, stream),
                           "AttentionLayerKvPath::store");
    }
    b200kv_view raw(const AttentionKvCacheView& c) const {
        return shim_detail::make_view(c.key_cache, c.value_cache, c.key_cache_q8, c.key_scales, c.value_cache_q8, c.value_scales,
                                      static_cast<std::uint32_t>(c.capacity), kv_heads_, head_dim_, static_cast<std::uint32_t>(c.qblock), c.is_k_q8(),
                                      c.is_v_q8());
    }
    float scale() const { return 1.0f / std::sqrt(static_cast<float>(head_dim_)); }
    const float* q_norm_;
    const float* k_norm_;
    std::uint32_t q_heads_, kv_heads_, head_dim_;
    float theta_, eps_;
};

}  // namespace prefill_v2
}  // namespace miinfer
