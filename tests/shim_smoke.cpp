// Compiled and run by tests/test_shim_gpu.py: a reference-style call sequence (the names and argument order of
// src/prefill_v2/attention_layer.cpp:297-343, 599-632) through miinfer_shim.hpp on a real device.
// Prints "shim ok <checksum>"; the Python test checks the numbers against the oracle.
#include <cmath>
#include <cstdio>
#include <vector>

#include "miinfer_shim.hpp"

template <class T>
static T* dalloc(std::size_t count) {
    void* p = nullptr;
    cudaMalloc(&p, count * sizeof(T));
    return static_cast<T*>(p);
}

int main() {
    using namespace miinfer;
    using namespace miinfer::prefill_v2;
    constexpr std::uint32_t kQ = 24, kKv = 4, kD = 256, kPrefix = 96, kChunk = 8, kCap = 128;
    AttentionLayerKvCacheStorage cache(kCap, KvCacheQuantMode::kQ8Q8);   // reference defaults: 4 kv heads, d=256, row scales
    const AttentionKvCacheView v = cache.view();
    std::vector<float> k((kPrefix + kChunk) * kKv * kD), val(k.size()), w(kD, 1.0f), q(kChunk * kQ * kD), gate(q.size());
    unsigned s = 12345u;
    auto rnd = [&]() { s = s * 1664525u + 1013904223u; return (static_cast<float>(s >> 8) / 8388608.0f - 1.0f); };
    for (auto& x : k) x = rnd();
    for (auto& x : val) x = rnd();
    for (auto& x : q) x = rnd();
    for (auto& x : gate) x = rnd();
    float *dk = dalloc<float>(k.size()), *dv = dalloc<float>(val.size()), *dw = dalloc<float>(kD), *dq = dalloc<float>(q.size());
    float *dg = dalloc<float>(gate.size()), *dout = dalloc<float>(q.size()), *ddec = dalloc<float>(kQ * kD);
    cudaMemcpy(dk, k.data(), k.size() * 4, cudaMemcpyHostToDevice); cudaMemcpy(dv, val.data(), val.size() * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(dw, w.data(), kD * 4, cudaMemcpyHostToDevice); cudaMemcpy(dq, q.data(), q.size() * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(dg, gate.data(), gate.size() * 4, cudaMemcpyHostToDevice);
    // prefix, then the chunk (store first, attend second -- attention_layer.cpp:297-343)
    launch_qwen35_decoupled_k_norm_rope_kv_store_batch_quant(dk, dv, dw, v.key_cache, v.value_cache, v.key_cache_q8, v.key_scales,
        v.value_cache_q8, v.value_scales, kPrefix + kChunk, 0, kCap, kKv, kD, 1.0e6f, 1.0e-6f, v.is_k_q8(), v.is_v_q8());
    launch_qwen35_splitk_suffix_attention_quant(dq, v.key_cache, v.value_cache, v.key_cache_q8, v.key_scales, v.value_cache_q8,
        v.value_scales, dg, dout, nullptr, kChunk, kPrefix, kCap, kQ, kKv, kD, 1.0f / 16.0f, v.is_k_q8(), v.is_v_q8(), 32);
    // one decode step with the device-side position (attention_layer.cpp:613-632)
    DeviceDecodeState st{}; st.position = kPrefix + kChunk - 1;
    DeviceDecodeState* dst = dalloc<DeviceDecodeState>(1); cudaMemcpy(dst, &st, sizeof st, cudaMemcpyHostToDevice);
    const std::size_t ws_bytes = b200kv_decode_workspace_bytes(kQ, kD, 1);
    void* ws = dalloc<unsigned char>(ws_bytes); cudaMemset(ws, 0, ws_bytes);
    set_decode_workspace(ws, ws_bytes);
    launch_qwen35_tiled_online_attention_quant_dynamic(dq + (kChunk - 1) * kQ * kD, v.key_cache, v.value_cache, v.key_cache_q8, v.key_scales,
        v.value_cache_q8, v.value_scales, dst, kCap, ddec, nullptr, nullptr, kQ, kKv, kD, 1.0f / 16.0f, v.is_k_q8(), v.is_v_q8());
    if (cudaDeviceSynchronize() != cudaSuccess) { std::printf("shim FAILED: %s\n", cudaGetErrorString(cudaGetLastError())); return 1; }
    std::vector<float> out(q.size()), dec(kQ * kD);
    cudaMemcpy(out.data(), dout, out.size() * 4, cudaMemcpyDeviceToHost); cudaMemcpy(dec.data(), ddec, dec.size() * 4, cudaMemcpyDeviceToHost);
    // the last chunk token's ungated decode output must equal its suffix output divided by sigmoid(gate)
    double worst = 0.0, checksum = 0.0;
    for (std::uint32_t i = 0; i < kQ * kD; ++i) {
        const std::size_t j = static_cast<std::size_t>(kChunk - 1) * kQ * kD + i;
        const double gated = dec[i] / (1.0 + std::exp(-static_cast<double>(gate[j])));
        worst = std::fmax(worst, std::fabs(gated - out[j]));
        checksum += out[j];
    }
    bool threw = false;
    try { cache.download_raw(out.data(), kCap + 1); } catch (const std::runtime_error&) { threw = true; }
    // the operators either side of the KV path, with the reference's names: query-side split / norm / RoPE from the device
    // state (attention_layer.cpp:589), the Q8_1 form of the gated output for the projection that follows (:659-662), the
    // step advance (model.cpp:1136-1197), and the dequantising download (kv_cache.cpp:132-170)
    std::vector<float> qfull(kQ * 2 * kD);
    for (auto& x : qfull) x = rnd();
    float *dqfull = dalloc<float>(qfull.size()), *dqr = dalloc<float>(kQ * kD), *dgate1 = dalloc<float>(kQ * kD), *dgated = dalloc<float>(kQ * kD);
    Q8_1Block* dq8 = dalloc<Q8_1Block>(kQ * kD / 32);
    std::uint32_t* dtok = dalloc<std::uint32_t>(4);
    cudaMemcpy(dqfull, qfull.data(), qfull.size() * 4, cudaMemcpyHostToDevice);
    launch_qwen35_fused_q_split_norm_rope_dynamic(dqfull, dw, dqr, dgate1, kQ, kD, dst, 1.0e6f, 1.0e-6f);
    launch_qwen35_tiled_online_attention_quant_dynamic(dqr, v.key_cache, v.value_cache, v.key_cache_q8, v.key_scales, v.value_cache_q8,
        v.value_scales, dst, kCap, nullptr, dgate1, dgated, kQ, kKv, kD, 1.0f / 16.0f, v.is_k_q8(), v.is_v_q8(), nullptr, dq8);
    launch_qwen35_decode_state_advance(dst, dtok, 4);
    if (cudaDeviceSynchronize() != cudaSuccess) { std::printf("shim FAILED: %s\n", cudaGetErrorString(cudaGetLastError())); return 1; }
    std::vector<float> gated(kQ * kD), key_rows;
    std::vector<Q8_1Block> q8(kQ * kD / 32);
    DeviceDecodeState after{};
    cudaMemcpy(gated.data(), dgated, gated.size() * 4, cudaMemcpyDeviceToHost);
    cudaMemcpy(q8.data(), dq8, q8.size() * sizeof(Q8_1Block), cudaMemcpyDeviceToHost);
    cudaMemcpy(&after, dst, sizeof after, cudaMemcpyDeviceToHost);
    cache.download_key(key_rows, kPrefix);
    // every Q8_1 block reproduces its 32 gated outputs to within half a quantisation step (plus what the fp16 rounding of
    // the stored scale adds: at most 127 * 2^-11 of a step)
    double q8_worst = 0.0;
    for (std::size_t b = 0; b < q8.size(); ++b) {
        const float d = __half2float(*reinterpret_cast<const __half*>(&q8[b].d));
        for (int i = 0; i < 32; ++i) q8_worst = std::fmax(q8_worst, std::fabs(static_cast<double>(q8[b].qs[i]) * d - gated[b * 32 + i]) - 0.57 * d);
    }
    const bool extras_ok = q8_worst <= 1e-6 && after.position == kPrefix + kChunk && after.generated == 1 &&
                           key_rows.size() == static_cast<std::size_t>(kKv) * kPrefix * kD && std::isfinite(key_rows[5]);
    // the same chunk and the same decode step through the layer object (attention_layer.cpp:291-349, 587-656) on a second
    // cache: its outputs must equal what the individual launchers gave above
    AttentionLayerKvCacheStorage cache2(kCap, KvCacheQuantMode::kQ8Q8);
    std::vector<float> chunk_qfull((kPrefix + kChunk) * kQ * 2 * kD, 0.0f);
    float *dq2 = dalloc<float>(chunk_qfull.size()), *dqr2 = dalloc<float>((kPrefix + kChunk) * kQ * kD), *dg2 = dalloc<float>((kPrefix + kChunk) * kQ * kD);
    float* dout2 = dalloc<float>((kPrefix + kChunk) * kQ * kD);
    AttentionLayerKvPath layer(dw, dw);
    AttentionKvPathBuffers bufs;
    bufs.attn_qfull = dq2; bufs.attn_k = dk; bufs.attn_v = dv; bufs.attn_q_rope = dqr2; bufs.gate = dg2; bufs.attn_gated_output = dout2;
    // prefix through forward() with zero queries (only the store matters), then one decode step with the query of above
    cudaMemset(dq2, 0, chunk_qfull.size() * 4);
    layer.forward(cache2.view(), bufs, kPrefix + kChunk - 1, 0);
    DeviceDecodeState st2{}; st2.position = kPrefix + kChunk - 1;
    cudaMemcpy(dst, &st2, sizeof st2, cudaMemcpyHostToDevice);
    AttentionKvPathBuffers step = bufs;
    step.attn_qfull = dqfull; step.attn_k = dk + static_cast<std::size_t>(kPrefix + kChunk - 1) * kKv * kD; step.attn_v = dv + static_cast<std::size_t>(kPrefix + kChunk - 1) * kKv * kD;
    step.attn_q_rope = dqr; step.gate = dgate1; step.attn_gated_output = dout2;
    layer.decode(cache2.view(), step, 0, nullptr, dst);
    if (cudaDeviceSynchronize() != cudaSuccess) { std::printf("shim FAILED (layer): %s\n", cudaGetErrorString(cudaGetLastError())); return 1; }
    std::vector<float> gated2(kQ * kD);
    cudaMemcpy(gated2.data(), dout2, gated2.size() * 4, cudaMemcpyDeviceToHost);
    double layer_worst = 0.0;
    for (std::size_t i = 0; i < gated2.size(); ++i) layer_worst = std::fmax(layer_worst, std::fabs(static_cast<double>(gated2[i]) - gated[i]));
    const bool ok = worst < 2e-3 && threw && extras_ok && layer_worst < 1e-5;
    std::printf("shim %s worst=%.3e checksum=%.6f bytes=%zu q8=%.2e pos=%u layer=%.2e\n", ok ? "ok" : "MISMATCH", worst, checksum,
                cache.raw_tokens_bytes(kPrefix), q8_worst, after.position, layer_worst);
    return ok ? 0 : 2;
}
