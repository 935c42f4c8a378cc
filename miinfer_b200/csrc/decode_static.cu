// b200kv_decode_attn_static: decode attention for callers that may not allocate.
//
// Some hosts hand all device memory to their own pool when they start and treat any later driver
// allocation as an error (it can fail once the pool has taken everything, and it stalls the device
// while it runs); others run this library from a context where allocation calls are simply not
// permitted.  Such a caller has nowhere to get the split-K scratch that b200kv_decode_attn expects.
// This entry point brings its own: a fixed array that is part of the library image on every GPU
// that loads it.  It performs no cudaMalloc / cudaFree and calls nothing that allocates.
#include "decode_common.cuh"

#include <cmath>
#include <mutex>

namespace {

// 8 MiB per GPU, held from the moment the library is loaded until the process exits.  Enough for
// 32 query heads at head_dim 128 (6.4 MB) or 20 heads at head_dim 256 (7.9 MB), one session.
constexpr size_t kStaticScratchBytes = size_t{8} << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices] = {};   // device address of g_static_scratch, per device; null = not set up yet

// In host code `g_static_scratch` names a host-side stand-in, not device memory: handing it to a
// kernel would fault (or, where the GPU can reach host memory, quietly use the wrong bytes).  The
// real address is per device and has to be asked for with that device current.
int scratch_for_current_device(void** out) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        (void)cudaGetLastError();
        return B200KV_ERR_DEVICE;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (err != cudaSuccess || ptr == nullptr) {
            b200kv::set_last_cuda_error(err, "cudaGetSymbolAddress(g_static_scratch)");
            return B200KV_ERR_CUDA;
        }
        g_scratch_address[device] = ptr;
    }
    *out = g_scratch_address[device];
    return B200KV_OK;
}

}  // namespace

using namespace b200kv;

extern "C" {

size_t b200kv_decode_static_scratch_bytes(void) { return kStaticScratchBytes; }

int b200kv_decode_attn_static(const b200kv_view* view, const void* q, int q_dtype, const float* gate,
                              float* output, float* gated_output, uint32_t query_heads, float scale,
                              uint32_t cache_length, const b200kv_decode_state* decode_state,
                              uint32_t num_splits, void* stream) {
    int rc = validate_view(view);
    if (rc != B200KV_OK) return rc;
    if (q == nullptr || (output == nullptr && gated_output == nullptr)) return B200KV_ERR_INVALID;
    if (q_dtype != B200KV_F16 && q_dtype != B200KV_F32) return B200KV_ERR_INVALID;
    if (query_heads == 0 || query_heads % view->kv_heads != 0 || !std::isfinite(scale)) return B200KV_ERR_INVALID;
    if (query_heads / view->kv_heads > 8) return B200KV_ERR_UNSUPPORTED;
    if (decode_state == nullptr && cache_length > view->capacity) return B200KV_ERR_RANGE;
    // The shape must fit the fixed array: the same formula the caller-owned workspace is sized with.
    if (b200kv_decode_workspace_bytes(query_heads, view->head_dim, 1) > kStaticScratchBytes) return B200KV_ERR_WORKSPACE;
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    void* scratch = nullptr;
    if ((rc = scratch_for_current_device(&scratch)) != B200KV_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    // Every call shares the array and it keeps what the previous call left.  Nothing has to be cleared here: the
    // array starts out zero (static storage), every launch zeroes the tagged words it consumed, and words that a
    // launch which gave up left behind carry that launch's tag, which no later launch accepts; the plain
    // partials behind the tagged part are rewritten before they are read.

    DecodeParams p{};
    p.view = *view;
    p.decode_state = decode_state;
    p.cache_length = cache_length;
    p.sessions = 1;
    p.q = q;
    p.q_is_f16 = (q_dtype == B200KV_F16);
    p.query_heads = query_heads;
    p.scale = scale;
    const uint32_t max_length = decode_state ? static_cast<uint32_t>(view->capacity) : cache_length;
    MergeParams mp{};
    mp.query_heads = query_heads;
    mp.head_dim = view->head_dim;
    mp.gate = gate;
    mp.output = output;
    mp.gated_output = gated_output;
    return run_decode(p, *view, max_length, scratch, kStaticScratchBytes, num_splits, mp, 1, s);
}

}  // extern "C"
