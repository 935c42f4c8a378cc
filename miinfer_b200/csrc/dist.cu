// Sequence-sharded decode over NCCL from a C or C++ host: the all-gather of the per-rank (m, l, acc) partials and the
// merge kernel behind three calls.  This is the collective form of the cross-GPU merge for every cache the in-kernel
// exchange (b200kv_decode_attn_sharded) does not take -- fp16 or mixed modes, head_dim 256 -- and the baseline it is
// measured against.  No counterpart in the reference (single GPU; its design notes only plan a cross-device reduction,
// docs/architecture.md:1035-1092).
//
// NCCL is not linked: the few entry points used are looked up at run time, first among the libraries the process
// has already loaded (a host that hands in its own ncclComm_t has NCCL loaded), then in libnccl.so.2.
#include "kv_common.cuh"

#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <new>

namespace {

struct UniqueId { char bytes[128]; };   // ncclUniqueId
using Comm = void*;                     // ncclComm_t
constexpr int kNcclFloat = 7;           // ncclFloat32

struct Nccl {
    int (*GetUniqueId)(UniqueId*) = nullptr;
    int (*CommInitRank)(Comm*, int, UniqueId, int) = nullptr;
    int (*CommDestroy)(Comm) = nullptr;
    int (*CommCount)(Comm, int*) = nullptr;
    int (*CommUserRank)(Comm, int*) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, Comm, cudaStream_t) = nullptr;
    bool ok = false;
};

const Nccl& nccl() {
    static Nccl api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* lib = nullptr;
        auto find = [&](const char* name) -> void* {
            void* sym = dlsym(RTLD_DEFAULT, name);
            if (sym == nullptr) {
                if (lib == nullptr) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
                if (lib != nullptr) sym = dlsym(lib, name);
            }
            return sym;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(find("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(find("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(find("ncclCommDestroy"));
        api.CommCount = reinterpret_cast<decltype(api.CommCount)>(find("ncclCommCount"));
        api.CommUserRank = reinterpret_cast<decltype(api.CommUserRank)>(find("ncclCommUserRank"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(find("ncclAllGather"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.CommCount && api.CommUserRank && api.AllGather;
    });
    return api;
}

}  // namespace

struct b200kv_dist {
    Comm comm = nullptr;
    bool owns_comm = false;
    uint32_t rank = 0, world = 1, query_heads = 0, head_dim = 0;
    float* mine = nullptr;       // [query_heads * (head_dim + 2)]: m | l | acc
    float* gathered = nullptr;   // [world][query_heads * (head_dim + 2)]
};

using namespace b200kv;

extern "C" {

int b200kv_dist_unique_id(void* id128) {
    if (id128 == nullptr) return B200KV_ERR_INVALID;
    if (!nccl().ok) return B200KV_ERR_UNSUPPORTED;
    UniqueId id;
    if (nccl().GetUniqueId(&id) != 0) return B200KV_ERR_CUDA;
    std::memcpy(id128, &id, sizeof id);
    return B200KV_OK;
}

int b200kv_dist_init(b200kv_dist** out, void* nccl_comm, const void* id128, uint32_t rank, uint32_t world, uint32_t query_heads,
                     uint32_t head_dim) {
    if (out == nullptr || query_heads == 0 || head_dim == 0 || head_dim > 1024) return B200KV_ERR_INVALID;
    if (nccl_comm == nullptr && (id128 == nullptr || world == 0 || rank >= world)) return B200KV_ERR_INVALID;
    if (!nccl().ok) return B200KV_ERR_UNSUPPORTED;
    int rc = ensure_device();
    if (rc != B200KV_OK) return rc;
    b200kv_dist* d = new (std::nothrow) b200kv_dist;
    if (d == nullptr) return B200KV_ERR_CUDA;
    if (nccl_comm != nullptr) {
        int n = 0, r = 0;
        if (nccl().CommCount(nccl_comm, &n) != 0 || nccl().CommUserRank(nccl_comm, &r) != 0 || n <= 0) { delete d; return B200KV_ERR_INVALID; }
        d->comm = nccl_comm;
        d->world = static_cast<uint32_t>(n);
        d->rank = static_cast<uint32_t>(r);
    } else {
        UniqueId id;
        std::memcpy(&id, id128, sizeof id);
        if (nccl().CommInitRank(&d->comm, static_cast<int>(world), id, static_cast<int>(rank)) != 0) { delete d; return B200KV_ERR_CUDA; }
        d->owns_comm = true;
        d->world = world;
        d->rank = rank;
    }
    d->query_heads = query_heads;
    d->head_dim = head_dim;
    const size_t part = static_cast<size_t>(query_heads) * (head_dim + 2u) * sizeof(float);
    cudaError_t err = cudaMalloc(&d->mine, part);
    if (err == cudaSuccess) err = cudaMalloc(&d->gathered, part * d->world);
    if (err == cudaSuccess) err = cudaMemset(d->mine, 0, part);
    if (err != cudaSuccess) {
        set_last_cuda_error(err, "b200kv_dist_init");
        b200kv_dist_destroy(d);
        return B200KV_ERR_CUDA;
    }
    *out = d;
    return B200KV_OK;
}

int b200kv_dist_partial(b200kv_dist* dist, float** part_m, float** part_l, float** part_acc) {
    if (dist == nullptr || part_m == nullptr || part_l == nullptr || part_acc == nullptr) return B200KV_ERR_INVALID;
    *part_m = dist->mine;
    *part_l = dist->mine + dist->query_heads;
    *part_acc = dist->mine + 2 * static_cast<size_t>(dist->query_heads);
    return B200KV_OK;
}

int b200kv_dist_merge(b200kv_dist* dist, const float* gate, float* output, float* gated_output, void* stream) {
    if (dist == nullptr || (output == nullptr && gated_output == nullptr)) return B200KV_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t count = static_cast<size_t>(dist->query_heads) * (dist->head_dim + 2u);
    if (nccl().AllGather(dist->mine, dist->gathered, count, kNcclFloat, dist->comm, s) != 0) return B200KV_ERR_CUDA;
    return b200kv_merge_partials_packed(dist->gathered, dist->world, dist->query_heads, dist->head_dim, gate, output, gated_output, stream);
}

int b200kv_dist_destroy(b200kv_dist* dist) {
    if (dist == nullptr) return B200KV_OK;
    if (dist->mine != nullptr) (void)cudaFree(dist->mine);
    if (dist->gathered != nullptr) (void)cudaFree(dist->gathered);
    if (dist->owns_comm && dist->comm != nullptr && nccl().ok) (void)nccl().CommDestroy(dist->comm);
    delete dist;
    return B200KV_OK;
}

}  // extern "C"
