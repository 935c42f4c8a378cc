// Exchange buffers for the cross-GPU step of sequence-sharded decode (b200kv_decode_attn_sharded): device memory
// that the other ranks of the node (one process per GPU) map into their address space and store into directly.
// Set-up calls, not launch calls: they allocate, and they synchronise the device.
#include "kv_common.cuh"

#include <cstring>

using namespace b200kv;

extern "C" {

int b200kv_exchange_create(size_t bytes, void** buffer, void* handle64) {
    if (buffer == nullptr || handle64 == nullptr || bytes == 0) return B200KV_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle travels as 64 opaque bytes");
    int rc = ensure_device();
    if (rc != B200KV_OK) return rc;
    void* ptr = nullptr;
    B200KV_CUDA_TRY(cudaMalloc(&ptr, bytes));
    cudaError_t err = cudaMemset(ptr, 0, bytes);   // tags start at zero
    cudaIpcMemHandle_t h;
    if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, ptr);
    if (err != cudaSuccess) {
        set_last_cuda_error(err, "b200kv_exchange_create");
        (void)cudaFree(ptr);
        return B200KV_ERR_CUDA;
    }
    std::memcpy(handle64, &h, sizeof h);
    *buffer = ptr;
    return B200KV_OK;
}

int b200kv_exchange_open(const void* handle64, void** peer_buffer) {
    if (handle64 == nullptr || peer_buffer == nullptr) return B200KV_ERR_INVALID;
    int rc = ensure_device();
    if (rc != B200KV_OK) return rc;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, sizeof h);
    void* ptr = nullptr;
    B200KV_CUDA_TRY(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    *peer_buffer = ptr;
    return B200KV_OK;
}

int b200kv_exchange_close(void* peer_buffer) {
    if (peer_buffer == nullptr) return B200KV_OK;
    B200KV_CUDA_TRY(cudaIpcCloseMemHandle(peer_buffer));
    return B200KV_OK;
}

int b200kv_exchange_destroy(void* buffer) {
    if (buffer == nullptr) return B200KV_OK;
    B200KV_CUDA_TRY(cudaFree(buffer));
    return B200KV_OK;
}

}  // extern "C"
