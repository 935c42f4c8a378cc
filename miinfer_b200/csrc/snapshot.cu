// Prefix snapshot / restore of one layer's KV cache.
//
// The blob layout is the raw compact layout of MIInfer's
// AttentionLayerKvCacheStorage::download_raw / upload_raw
// (src/prefill_v2/kv_cache.cpp:214-369): K first, per kv head the int8 slice of
// `tokens` rows followed by that head's scale slice (or one fp16 slice), then V
// the same way.  The reference issues 2-4 memcpys per kv head; here every plane
// is ONE strided 2D copy (row = one head's `tokens` positions, source pitch =
// capacity, destination pitch = the per-head record), and the device-to-device
// clone is a single kernel over all planes.
#include "kv_common.cuh"

namespace b200kv {

struct PlaneCopy {
    const uint8_t* src;
    uint8_t* dst;
    size_t span;       // contiguous bytes per head
    size_t src_pitch;  // bytes between heads
    size_t dst_pitch;
};

struct CloneParams {
    PlaneCopy plane[4];
    int planes;
    uint32_t heads;
};

__global__ void __launch_bounds__(256) clone_kernel(const __grid_constant__ CloneParams p) {
    const int plane = blockIdx.z;
    const uint32_t head = blockIdx.y;
    const PlaneCopy& c = p.plane[plane];
    const uint8_t* src = c.src + head * c.src_pitch;
    uint8_t* dst = c.dst + head * c.dst_pitch;
    const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    if (vec) {
        const size_t n16 = c.span / 16;
        for (size_t i = tid; i < n16; i += stride)
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
        for (size_t i = n16 * 16 + tid; i < c.span; i += stride) dst[i] = src[i];
    } else {
        const size_t n2 = c.span / 2;  // every plane holds 2-byte or wider units
        for (size_t i = tid; i < n2; i += stride)
            reinterpret_cast<uint16_t*>(dst)[i] = reinterpret_cast<const uint16_t*>(src)[i];
    }
}

struct SidePlanes {
    bool q8;
    uint8_t* data;    // int8 plane or fp16 plane
    uint8_t* scales;  // fp16 scale plane (q8 only)
};

static SidePlanes k_side(const b200kv_view& v) {
    return is_k_q8(v.quant_mode) ? SidePlanes{true, reinterpret_cast<uint8_t*>(v.key_q8), static_cast<uint8_t*>(v.key_scales)}
                                 : SidePlanes{false, static_cast<uint8_t*>(v.key_f16), nullptr};
}
static SidePlanes v_side(const b200kv_view& v) {
    return is_v_q8(v.quant_mode) ? SidePlanes{true, reinterpret_cast<uint8_t*>(v.value_q8), static_cast<uint8_t*>(v.value_scales)}
                                 : SidePlanes{false, static_cast<uint8_t*>(v.value_f16), nullptr};
}

static size_t side_record_bytes(const b200kv_view& v, bool q8, uint64_t tokens) {
    const size_t d = v.head_dim, nblk = d / v.qblock;
    return q8 ? tokens * (d + 2 * nblk) : tokens * d * 2;
}

// One side (K or V) between the cache and the blob; to_blob selects direction.
static int copy_side(const b200kv_view& v, const SidePlanes& side, uint64_t tokens, uint8_t* blob, bool to_blob,
                     cudaStream_t s) {
    const size_t d = v.head_dim, nblk = d / v.qblock;
    const size_t record = side_record_bytes(v, side.q8, tokens);
    auto copy2d = [&](uint8_t* cache_plane, size_t bytes_per_pos, size_t blob_offset) -> cudaError_t {
        const size_t width = tokens * bytes_per_pos, cache_pitch = static_cast<size_t>(v.capacity) * bytes_per_pos;
        return to_blob ? cudaMemcpy2DAsync(blob + blob_offset, record, cache_plane, cache_pitch, width, v.kv_heads, cudaMemcpyDefault, s)
                       : cudaMemcpy2DAsync(cache_plane, cache_pitch, blob + blob_offset, record, width, v.kv_heads, cudaMemcpyDefault, s);
    };
    if (side.q8) {
        B200KV_CUDA_TRY(copy2d(side.data, d, 0));
        B200KV_CUDA_TRY(copy2d(side.scales, nblk * 2, tokens * d));
    } else {
        B200KV_CUDA_TRY(copy2d(side.data, d * 2, 0));
    }
    return B200KV_OK;
}

static int snapshot_copy(const b200kv_view* view, uint64_t tokens, void* blob, bool to_blob, void* stream) {
    int rc = validate_view(view);
    if (rc != B200KV_OK) return rc;
    if (tokens > view->capacity) return B200KV_ERR_RANGE;  // the reference throws here (kv_cache.cpp:228-230)
    if (tokens == 0 || blob == nullptr) return B200KV_OK;  // the reference returns silently (kv_cache.cpp:231)
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint8_t* bytes = static_cast<uint8_t*>(blob);
    const SidePlanes ks = k_side(*view), vs = v_side(*view);
    if ((rc = copy_side(*view, ks, tokens, bytes, to_blob, s)) != B200KV_OK) return rc;
    const size_t k_bytes = side_record_bytes(*view, ks.q8, tokens) * view->kv_heads;
    return copy_side(*view, vs, tokens, bytes + k_bytes, to_blob, s);
}

}  // namespace b200kv

using namespace b200kv;

extern "C" {

size_t b200kv_snapshot_bytes(const b200kv_view* view, uint64_t tokens) {
    if (view == nullptr || view->qblock == 0) return 0;
    return (side_record_bytes(*view, is_k_q8(view->quant_mode), tokens) +
            side_record_bytes(*view, is_v_q8(view->quant_mode), tokens)) * view->kv_heads;
}

int b200kv_snapshot_save(const b200kv_view* view, uint64_t tokens, void* dst, void* stream) {
    return snapshot_copy(view, tokens, dst, true, stream);
}

int b200kv_snapshot_restore(const b200kv_view* view, uint64_t tokens, const void* src, void* stream) {
    return snapshot_copy(view, tokens, const_cast<void*>(src), false, stream);
}

int b200kv_snapshot_clone(const b200kv_view* dst, const b200kv_view* src, uint64_t tokens, void* stream) {
    int rc;
    if ((rc = validate_view(dst)) != B200KV_OK || (rc = validate_view(src)) != B200KV_OK) return rc;
    if (dst->head_dim != src->head_dim || dst->kv_heads != src->kv_heads || dst->qblock != src->qblock ||
        dst->quant_mode != src->quant_mode)
        return B200KV_ERR_INVALID;
    if (tokens > dst->capacity || tokens > src->capacity) return B200KV_ERR_RANGE;
    if (tokens == 0) return B200KV_OK;
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    const size_t d = src->head_dim, nblk = d / src->qblock;
    CloneParams p{};
    p.heads = src->kv_heads;
    auto add = [&](const uint8_t* s, uint8_t* t, size_t bytes_per_pos) {
        p.plane[p.planes++] = PlaneCopy{s, t, tokens * bytes_per_pos, static_cast<size_t>(src->capacity) * bytes_per_pos,
                                        static_cast<size_t>(dst->capacity) * bytes_per_pos};
    };
    const SidePlanes sk = k_side(*src), dk = k_side(*dst), sv = v_side(*src), dv = v_side(*dst);
    if (sk.q8) { add(sk.data, dk.data, d); add(sk.scales, dk.scales, nblk * 2); } else add(sk.data, dk.data, d * 2);
    if (sv.q8) { add(sv.data, dv.data, d); add(sv.scales, dv.scales, nblk * 2); } else add(sv.data, dv.data, d * 2);
    // enough CTAs to cover the widest plane with 16-byte units, capped at ~4 waves
    size_t widest = 0;
    for (int i = 0; i < p.planes; ++i) widest = p.plane[i].span > widest ? p.plane[i].span : widest;
    size_t blocks = (widest / 16 + 255) / 256;
    const size_t cap = (148u * 8u + p.heads * p.planes - 1) / (p.heads * p.planes);
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    clone_kernel<<<dim3(static_cast<unsigned>(blocks), p.heads, p.planes), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    B200KV_CUDA_TRY(cudaGetLastError());
    return B200KV_OK;
}

}  // extern "C"

// ---- dequantising download (inspection and tests) ----------------------------------------------------------------
// AttentionLayerKvCacheStorage::download_key / download_value, src/prefill_v2/kv_cache.cpp:132-212: the first `tokens`
// positions of one side as fp32 [kv_head][tokens][head_dim] in HOST memory, int8 values multiplied by their fp16
// scale (here: the scale of their block), fp16 values widened.  Like the reference's it is a blocking host routine
// (it stages the raw planes in host memory and converts there); it is not part of the per-token path.
#include <vector>

namespace {
int download_side(const b200kv_view* view, uint64_t tokens, float* host_dst, bool key, cudaStream_t stream) {
    using namespace b200kv;
    int rc = validate_view(view);
    if (rc != B200KV_OK) return rc;
    if (host_dst == nullptr && tokens > 0) return B200KV_ERR_INVALID;
    if (tokens > view->capacity) return B200KV_ERR_RANGE;   // the reference throws (kv_cache.cpp:133-135)
    if (tokens == 0) return B200KV_OK;
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    const uint32_t H = view->kv_heads, d = view->head_dim, nblk = d / view->qblock;
    const bool q8 = key ? is_k_q8(view->quant_mode) : is_v_q8(view->quant_mode);
    try {
        if (q8) {
            std::vector<int8_t> q(static_cast<size_t>(H) * tokens * d);
            std::vector<uint16_t> sc(static_cast<size_t>(H) * tokens * nblk);
            const int8_t* src_q = key ? view->key_q8 : view->value_q8;
            const uint8_t* src_s = static_cast<const uint8_t*>(key ? view->key_scales : view->value_scales);
            B200KV_CUDA_TRY(cudaMemcpy2DAsync(q.data(), tokens * d, src_q, view->capacity * d, tokens * d, H, cudaMemcpyDeviceToHost, stream));
            B200KV_CUDA_TRY(cudaMemcpy2DAsync(sc.data(), tokens * nblk * 2, src_s, view->capacity * nblk * 2, tokens * nblk * 2, H,
                                              cudaMemcpyDeviceToHost, stream));
            B200KV_CUDA_TRY(cudaStreamSynchronize(stream));
            for (size_t row = 0; row < static_cast<size_t>(H) * tokens; ++row)
                for (uint32_t b = 0; b < nblk; ++b) {
                    const float scale = __half2float(__ushort_as_half(sc[row * nblk + b]));
                    for (uint32_t i = 0; i < view->qblock; ++i) {
                        const size_t idx = row * d + b * view->qblock + i;
                        host_dst[idx] = static_cast<float>(q[idx]) * scale;
                    }
                }
        } else {
            std::vector<uint16_t> h(static_cast<size_t>(H) * tokens * d);
            const void* src = key ? view->key_f16 : view->value_f16;
            B200KV_CUDA_TRY(cudaMemcpy2DAsync(h.data(), tokens * d * 2, src, view->capacity * d * 2, tokens * d * 2, H, cudaMemcpyDeviceToHost, stream));
            B200KV_CUDA_TRY(cudaStreamSynchronize(stream));
            for (size_t i = 0; i < h.size(); ++i) host_dst[i] = __half2float(__ushort_as_half(h[i]));
        }
    } catch (const std::exception&) {
        return B200KV_ERR_CUDA;
    }
    return B200KV_OK;
}
}  // namespace

extern "C" int b200kv_download_key(const b200kv_view* view, uint64_t tokens, float* host_dst, void* stream) {
    return download_side(view, tokens, host_dst, true, static_cast<cudaStream_t>(stream));
}
extern "C" int b200kv_download_value(const b200kv_view* view, uint64_t tokens, float* host_dst, void* stream) {
    return download_side(view, tokens, host_dst, false, static_cast<cudaStream_t>(stream));
}
