// Library plumbing: status strings, device guard, view validation and the
// owning cache storage object (the counterpart of MIInfer's
// AttentionLayerKvCacheStorage, src/prefill_v2/kv_cache.cpp:10-130).
#include "decode_common.cuh"

#include <atomic>
#include <cmath>
#include <mutex>
#include <cstdio>
#include <cstring>
#include <new>

namespace b200kv {

static thread_local char g_last_error[256] = "";
static std::atomic<uint32_t> g_overlap_tail{0};

uint32_t launch_overlap_tail() { return g_overlap_tail.load(std::memory_order_relaxed); }

static std::atomic<uint32_t> g_launch_tag{0};
uint32_t next_launch_tag() {
    uint32_t t = g_launch_tag.fetch_add(1, std::memory_order_relaxed) + 1;
    if (t == 0) t = g_launch_tag.fetch_add(1, std::memory_order_relaxed) + 1;   // the counter wrapped: 0 means "no word"
    return t;
}

constexpr int kMaxDevices = 64;
static std::atomic<uint32_t*> g_status_word[kMaxDevices] = {};
namespace {
struct TensorMapSlot {
    TensorMapKey key;
    CUtensorMap map;
    bool used;
};
TensorMapSlot* tensor_map_slot(const TensorMapKey& key) {
    static thread_local TensorMapSlot slots[256] = {};
    const uint64_t a = reinterpret_cast<uintptr_t>(key.base);
    return &slots[((a >> 8) ^ (a >> 16) ^ (a >> 24) ^ key.box_rows ^ key.kind) & 255u];
}
}  // namespace

bool tensor_map_lookup(const TensorMapKey& key, CUtensorMap* out) {
    const TensorMapSlot* s = tensor_map_slot(key);
    if (!s->used || !(s->key == key)) return false;
    *out = s->map;
    return true;
}

void tensor_map_remember(const TensorMapKey& key, const CUtensorMap& map) {
    TensorMapSlot* s = tensor_map_slot(key);
    s->key = key;
    s->map = map;
    s->used = true;
}

void rope_constants(int rope_mode, float theta, uint32_t head_dim, float* inv_freq, float* sectioned_step) {
    static thread_local float cached_theta = 0.0f, cached_step = 0.0f, step_theta = 0.0f;
    static thread_local uint32_t cached_dim = 0;
    static thread_local float table[128];
    if (rope_mode == B200KV_ROPE_NEOX_FULL) {
        const uint32_t half = head_dim / 2 > 128 ? 128 : head_dim / 2;
        if (cached_dim != head_dim || cached_theta != theta) {
            for (uint32_t i = 0; i < half; ++i)
                table[i] = std::pow(theta, -static_cast<float>(2 * i) / static_cast<float>(head_dim));
            cached_dim = head_dim;
            cached_theta = theta;
        }
        std::memcpy(inv_freq, table, half * sizeof(float));
    } else if (rope_mode == B200KV_ROPE_SECTIONED64) {
        if (step_theta != theta) {
            cached_step = std::pow(theta, -2.0f / 64.0f);
            step_theta = theta;
        }
        *sectioned_step = cached_step;
    }
}

uint32_t* current_status_word() {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return g_status_word[device].load(std::memory_order_relaxed);
}

static std::atomic<uint64_t*> g_timeline[kMaxDevices] = {};
static std::atomic<uint32_t> g_timeline_words[kMaxDevices] = {};
uint64_t* current_timeline_buffer(uint32_t ctas) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        (void)cudaGetLastError();
        return nullptr;
    }
    uint64_t* buf = g_timeline[device].load(std::memory_order_relaxed);
    return (buf != nullptr && static_cast<uint64_t>(ctas) * 8 <= g_timeline_words[device].load(std::memory_order_relaxed)) ? buf : nullptr;
}

static std::atomic<int> g_streaming_kernel{0};
int streaming_kernel_choice() { return g_streaming_kernel.load(std::memory_order_relaxed); }

cudaError_t opt_in_dynamic_smem(const void* kernel, int bytes, std::atomic<uint64_t>& done_mask) {
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return err;
    const bool tracked = device >= 0 && device < 64;
    if (tracked && (done_mask.load(std::memory_order_acquire) >> device) & 1ull) return cudaSuccess;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (err == cudaSuccess && tracked) done_mask.fetch_or(1ull << device, std::memory_order_release);
    return err;
}

void set_last_cuda_error(cudaError_t err, const char* where) {
    std::snprintf(g_last_error, sizeof g_last_error, "%s: %s (%s)", cudaGetErrorName(err),
                  cudaGetErrorString(err), where);
    (void)cudaGetLastError();  // clear the sticky-less error so later calls report their own
}

int ensure_device() {
    static thread_local int checked_device = -1;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess) {
        (void)cudaGetLastError();
        return B200KV_ERR_DEVICE;
    }
    if (device == checked_device) return B200KV_OK;
    int rc = b200kv_device_check(device);
    if (rc == B200KV_OK) checked_device = device;
    return rc;
}

int validate_view(const b200kv_view* v) {
    if (v == nullptr) return B200KV_ERR_INVALID;
    if (v->capacity == 0 || v->kv_heads == 0 || v->quant_mode > B200KV_Q8_Q8) return B200KV_ERR_INVALID;
    if (v->head_dim != 128 && v->head_dim != 256) return B200KV_ERR_UNSUPPORTED;
    if (v->qblock != 32 && v->qblock != v->head_dim) return B200KV_ERR_UNSUPPORTED;
    if (v->capacity > 0x7fffffffull) return B200KV_ERR_UNSUPPORTED;  // positions are 32-bit in the device state
    auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (is_k_q8(v->quant_mode)) {
        if (!v->key_q8 || !v->key_scales || !aligned(v->key_q8) || !aligned(v->key_scales)) return B200KV_ERR_INVALID;
    } else if (!v->key_f16 || !aligned(v->key_f16)) {
        return B200KV_ERR_INVALID;
    }
    if (is_v_q8(v->quant_mode)) {
        if (!v->value_q8 || !v->value_scales || !aligned(v->value_q8) || !aligned(v->value_scales)) return B200KV_ERR_INVALID;
    } else if (!v->value_f16 || !aligned(v->value_f16)) {
        return B200KV_ERR_INVALID;
    }
    return B200KV_OK;
}

}  // namespace b200kv

using namespace b200kv;

struct b200kv_cache {
    b200kv_view view;
    int device;
};

extern "C" {

int b200kv_version(void) { return B200KV_VERSION; }

int b200kv_set_launch_overlap(uint32_t tail_positions) {
    g_overlap_tail.store(tail_positions, std::memory_order_relaxed);
    return B200KV_OK;
}

int b200kv_set_status_word(uint32_t* device_word) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        (void)cudaGetLastError();
        return B200KV_ERR_DEVICE;
    }
    if ((reinterpret_cast<uintptr_t>(device_word) & 3u) != 0) return B200KV_ERR_INVALID;
    g_status_word[device].store(device_word, std::memory_order_relaxed);
    return B200KV_OK;
}

int b200kv_set_timeline_buffer(uint64_t* device_words, uint32_t capacity_words) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        (void)cudaGetLastError();
        return B200KV_ERR_DEVICE;
    }
    if ((reinterpret_cast<uintptr_t>(device_words) & 7u) != 0) return B200KV_ERR_INVALID;
    g_timeline[device].store(device_words, std::memory_order_relaxed);
    g_timeline_words[device].store(device_words ? capacity_words : 0, std::memory_order_relaxed);
    return B200KV_OK;
}

int b200kv_set_decode_kernel(int choice) {
    if (choice < 0 || choice > 1) return B200KV_ERR_INVALID;
    g_streaming_kernel.store(choice, std::memory_order_relaxed);
    return B200KV_OK;
}

int b200kv_workspace_reset(void* workspace, size_t workspace_bytes, void* stream) {
    if (workspace == nullptr) return B200KV_ERR_INVALID;
    int rc = ensure_device();
    if (rc != B200KV_OK) return rc;
    B200KV_CUDA_TRY(cudaMemsetAsync(workspace, 0, workspace_bytes, static_cast<cudaStream_t>(stream)));
    return B200KV_OK;
}

const char* b200kv_status_string(int status) {
    switch (status) {
        case B200KV_OK: return "ok";
        case B200KV_ERR_INVALID: return "invalid argument";
        case B200KV_ERR_UNSUPPORTED: return "unsupported shape or mode";
        case B200KV_ERR_CUDA: return "CUDA error";
        case B200KV_ERR_DEVICE: return "no sm_100 device";
        case B200KV_ERR_WORKSPACE: return "workspace too small";
        case B200KV_ERR_RANGE: return "position beyond cache capacity";
        case B200KV_ERR_FORMAT: return "bad session file";
        case B200KV_ERR_IO: return "session file I/O failed";
        case B200KV_ERR_MISMATCH: return "session does not match";
        default: return "unknown status";
    }
}

const char* b200kv_last_cuda_error(void) { return g_last_error; }

int b200kv_device_check(int device) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        (void)cudaGetLastError();
        return B200KV_ERR_DEVICE;
    }
    int major = 0, minor = 0;
    B200KV_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    B200KV_CUDA_TRY(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
    return (major == 10) ? B200KV_OK : B200KV_ERR_DEVICE;
}

static size_t side_bytes(uint64_t capacity, uint32_t kv_heads, uint32_t head_dim, uint32_t qblock, bool q8) {
    const size_t rows = static_cast<size_t>(capacity) * kv_heads;
    return q8 ? rows * (head_dim + 2u * (head_dim / qblock)) : rows * head_dim * 2u;
}

size_t b200kv_cache_bytes(uint64_t capacity, uint32_t kv_heads, uint32_t head_dim, uint32_t qblock, uint32_t quant_mode) {
    if (qblock == 0 || head_dim % qblock != 0) return 0;
    return side_bytes(capacity, kv_heads, head_dim, qblock, is_k_q8(quant_mode)) +
           side_bytes(capacity, kv_heads, head_dim, qblock, is_v_q8(quant_mode));
}

int b200kv_cache_destroy(b200kv_cache* cache) {
    if (cache == nullptr) return B200KV_OK;
    b200kv_view& v = cache->view;
    void* planes[6] = {v.key_f16, v.value_f16, v.key_q8, v.key_scales, v.value_q8, v.value_scales};
    for (void* p : planes)
        if (p != nullptr) (void)cudaFree(p);
    delete cache;
    return B200KV_OK;
}

int b200kv_cache_create(b200kv_cache** out, uint64_t capacity, uint32_t kv_heads, uint32_t head_dim,
                        uint32_t qblock, uint32_t quant_mode) {
    if (out == nullptr) return B200KV_ERR_INVALID;
    *out = nullptr;
    if (capacity == 0 || kv_heads == 0 || quant_mode > B200KV_Q8_Q8) return B200KV_ERR_INVALID;
    if (head_dim != 128 && head_dim != 256) return B200KV_ERR_UNSUPPORTED;
    if (qblock != 32 && qblock != head_dim) return B200KV_ERR_UNSUPPORTED;
    if (capacity > 0x7fffffffull) return B200KV_ERR_UNSUPPORTED;
    int rc = ensure_device();
    if (rc != B200KV_OK) return rc;
    b200kv_cache* cache = new (std::nothrow) b200kv_cache();
    if (cache == nullptr) return B200KV_ERR_INVALID;
    std::memset(&cache->view, 0, sizeof cache->view);
    (void)cudaGetDevice(&cache->device);
    b200kv_view& v = cache->view;
    v.capacity = capacity;
    v.kv_heads = kv_heads;
    v.head_dim = head_dim;
    v.qblock = qblock;
    v.quant_mode = quant_mode;
    const size_t rows = static_cast<size_t>(capacity) * kv_heads;
    const size_t q8_bytes = rows * head_dim, scale_bytes = rows * (head_dim / qblock) * 2u, f16_bytes = rows * head_dim * 2u;
    cudaError_t err = cudaSuccess;
    if (is_k_q8(quant_mode)) {
        err = cudaMalloc(reinterpret_cast<void**>(&v.key_q8), q8_bytes);
        if (err == cudaSuccess) err = cudaMalloc(&v.key_scales, scale_bytes);
    } else {
        err = cudaMalloc(&v.key_f16, f16_bytes);
    }
    if (err == cudaSuccess) {
        if (is_v_q8(quant_mode)) {
            err = cudaMalloc(reinterpret_cast<void**>(&v.value_q8), q8_bytes);
            if (err == cudaSuccess) err = cudaMalloc(&v.value_scales, scale_bytes);
        } else {
            err = cudaMalloc(&v.value_f16, f16_bytes);
        }
    }
    if (err != cudaSuccess) {
        set_last_cuda_error(err, "cudaMalloc(cache plane)");
        b200kv_cache_destroy(cache);
        return B200KV_ERR_CUDA;
    }
    rc = b200kv_cache_reset(cache, nullptr);
    if (rc == B200KV_OK) {
        cudaError_t sync = cudaStreamSynchronize(nullptr);
        if (sync != cudaSuccess) { set_last_cuda_error(sync, "cudaStreamSynchronize"); rc = B200KV_ERR_CUDA; }
    }
    if (rc != B200KV_OK) {
        b200kv_cache_destroy(cache);
        return rc;
    }
    *out = cache;
    return B200KV_OK;
}

int b200kv_cache_reset(b200kv_cache* cache, void* stream) {
    if (cache == nullptr) return B200KV_ERR_INVALID;
    const b200kv_view& v = cache->view;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t rows = static_cast<size_t>(v.capacity) * v.kv_heads;
    const size_t q8_bytes = rows * v.head_dim, scale_bytes = rows * (v.head_dim / v.qblock) * 2u, f16_bytes = rows * v.head_dim * 2u;
    if (v.key_f16) B200KV_CUDA_TRY(cudaMemsetAsync(v.key_f16, 0, f16_bytes, s));
    if (v.value_f16) B200KV_CUDA_TRY(cudaMemsetAsync(v.value_f16, 0, f16_bytes, s));
    if (v.key_q8) B200KV_CUDA_TRY(cudaMemsetAsync(v.key_q8, 0, q8_bytes, s));
    if (v.key_scales) B200KV_CUDA_TRY(cudaMemsetAsync(v.key_scales, 0, scale_bytes, s));
    if (v.value_q8) B200KV_CUDA_TRY(cudaMemsetAsync(v.value_q8, 0, q8_bytes, s));
    if (v.value_scales) B200KV_CUDA_TRY(cudaMemsetAsync(v.value_scales, 0, scale_bytes, s));
    return B200KV_OK;
}

int b200kv_cache_view(const b200kv_cache* cache, b200kv_view* out) {
    if (cache == nullptr || out == nullptr) return B200KV_ERR_INVALID;
    *out = cache->view;
    return B200KV_OK;
}

uint64_t b200kv_token_sequence_hash(const uint32_t* tokens, size_t count) {
    uint64_t hash = 0xcbf29ce484222325ull;
    for (size_t i = 0; i < count; ++i) {
        hash ^= static_cast<uint64_t>(tokens[i]);
        hash *= 0x100000001b3ull;
    }
    return hash;
}

}  // extern "C"
