// Prefix identity and the on-disk session: host code (no kernels).
//
// Replaces, for the KV part, MIInfer's PersistentSession (include/miinfer/prefill_v2/persistent_session.hpp:19-69,
// src/prefill_v2/persistent_session.cpp:27-320) and ReusableContext::check_match
// (src/prefill_v2/reusable_context.cpp:155-185).  The file starts with the reference's own packed 157-byte header
// (magic "MISS", version 20260928) followed by the prefix tokens and, per attention layer, the raw snapshot of
// AttentionLayerKvCacheStorage::download_raw.  The recurrent (GDN) section is empty: those layers are outside this
// path, so gdn_layers is 0 and a reference build, which insists on 48, rejects the file instead of misreading it.
// After the KV payload comes a 48-byte trailer with what the reference header cannot say -- kv heads, head_dim,
// scale-block width, layer count and an FNV-1a-64 checksum of the payload -- and, unlike the reference
// (persistent_session.cpp:180-189 never looks at kv_quant_mode), every one of these is validated on load.
// Files are written to "<path>.tmp" and renamed, as the reference does (:118-141).
#include "kv_common.cuh"

#include <sys/stat.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <new>
#include <stdexcept>
#include <string>
#include <string_view>
#include <vector>

namespace {

constexpr uint32_t kSessionVersion = 20260928;
constexpr uint32_t kStateLayoutVersion = 20260925;   // reusable_context.hpp:18

#pragma pack(push, 1)
struct Trailer {
    char magic[4];          // "B2KV"
    uint32_t kv_heads, head_dim, qblock, layers, quant_mode;
    uint64_t layer_bytes;   // raw snapshot bytes of one layer
    uint64_t checksum;      // FNV-1a-64 over the KV payload bytes
    uint64_t reserved;
};
#pragma pack(pop)
static_assert(sizeof(Trailer) == 48, "trailer layout");
static_assert(sizeof(b200kv_session_header) == 157, "header layout of persistent_session.hpp:19-33");

uint64_t fnv1a_bytes(const uint8_t* p, size_t n, uint64_t h = 0xcbf29ce484222325ull) {
    for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 0x100000001b3ull; }
    return h;
}

struct File {
    std::FILE* f = nullptr;
    explicit File(const char* path, const char* mode) : f(std::fopen(path, mode)) {}
    ~File() { if (f) std::fclose(f); }
    bool read(void* dst, size_t n) { return n == 0 || std::fread(dst, 1, n, f) == n; }
    bool write(const void* src, size_t n) { return n == 0 || std::fwrite(src, 1, n, f) == n; }
};

bool same_geometry(const b200kv_view* views, uint32_t layers) {
    for (uint32_t i = 1; i < layers; ++i)
        if (views[i].kv_heads != views[0].kv_heads || views[i].head_dim != views[0].head_dim || views[i].qblock != views[0].qblock ||
            views[i].quant_mode != views[0].quant_mode)
            return false;
    return true;
}

uint64_t file_size(std::FILE* f) {
    struct stat st;
    return (f != nullptr && fstat(fileno(f), &st) == 0 && st.st_size > 0) ? static_cast<uint64_t>(st.st_size) : 0;
}

// Runs an entry point's body; nothing may leave an extern "C" function as an exception.  A size taken from a damaged
// file that cannot be allocated is a format error, anything else the file system's.
template <typename F>
int guarded(F&& body) {
    try {
        return body();
    } catch (const std::bad_alloc&) {
        return B200KV_ERR_FORMAT;
    } catch (const std::length_error&) {
        return B200KV_ERR_FORMAT;
    } catch (const std::exception&) {
        return B200KV_ERR_IO;
    }
}

// Reads and checks header + tokens; leaves the file positioned at the (empty) GDN section.  Every length the header
// states is checked against the size of the file before anything is allocated from it.
int read_front(File& in, b200kv_session_header* hdr, std::vector<uint32_t>* tokens) {
    const uint64_t size = file_size(in.f);
    if (!in.read(hdr, sizeof *hdr)) return B200KV_ERR_FORMAT;
    if (std::memcmp(hdr->magic, "MISS", 4) != 0 || hdr->version != kSessionVersion) return B200KV_ERR_FORMAT;
    if (hdr->tokens_bytes != static_cast<uint64_t>(hdr->prefix_length) * sizeof(uint32_t) || hdr->prefix_length == 0) return B200KV_ERR_FORMAT;
    if (hdr->prefix_length > (1u << 28)) return B200KV_ERR_FORMAT;
    if (hdr->tokens_bytes > size || hdr->kv_bytes > size || sizeof *hdr + hdr->tokens_bytes + hdr->kv_bytes + sizeof(Trailer) != size)
        return B200KV_ERR_FORMAT;
    tokens->resize(hdr->prefix_length);
    if (!in.read(tokens->data(), hdr->tokens_bytes)) return B200KV_ERR_FORMAT;
    if (b200kv_token_sequence_hash(tokens->data(), tokens->size()) != hdr->token_hash) return B200KV_ERR_FORMAT;   // :198
    return B200KV_OK;
}

}  // namespace

extern "C" {

int b200kv_session_filename(uint64_t token_hash, uint32_t prefix_length, char* out, size_t out_bytes) {
    if (out == nullptr) return B200KV_ERR_INVALID;
    const int n = std::snprintf(out, out_bytes, "sess_%016llx_p%u.miinfer", static_cast<unsigned long long>(token_hash), prefix_length);
    return (n > 0 && static_cast<size_t>(n) < out_bytes) ? B200KV_OK : B200KV_ERR_INVALID;
}

int b200kv_prefix_match(const char* cached_model_id, const char* cached_quantization, uint32_t cached_layout_version,
                        const uint32_t* cached_tokens, uint32_t cached_length, const char* model_id, const char* quantization,
                        const uint32_t* prompt, uint32_t prompt_length) {
    if (cached_length == 0 || cached_tokens == nullptr) return B200KV_MATCH_EMPTY_CACHE;
    if (cached_layout_version != kStateLayoutVersion) return B200KV_MATCH_VERSION_MISMATCH;
    if (std::string_view(cached_model_id ? cached_model_id : "") != (model_id ? model_id : "")) return B200KV_MATCH_MODEL_MISMATCH;
    if (std::string_view(cached_quantization ? cached_quantization : "") != (quantization ? quantization : "")) return B200KV_MATCH_QUANTIZATION_MISMATCH;
    if (prompt_length < cached_length) return B200KV_MATCH_PROMPT_SHORTER;
    for (uint32_t i = 0; i < cached_length; ++i)
        if (prompt[i] != cached_tokens[i]) return B200KV_MATCH_PREFIX_MISMATCH;
    return B200KV_MATCH_EXACT;
}

int b200kv_session_write(const char* path, const char* model_id, const char* quantization, const uint32_t* tokens,
                         uint32_t prefix_length, const void* kv_payload, uint64_t layer_bytes, uint32_t layers,
                         uint32_t kv_heads, uint32_t head_dim, uint32_t qblock, uint32_t quant_mode) {
    return guarded([&]() -> int {
    if (path == nullptr || tokens == nullptr || prefix_length == 0) return B200KV_ERR_INVALID;   // the reference refuses an empty prefix (:40-42)
    if (layers != 0 && kv_payload == nullptr) return B200KV_ERR_INVALID;
    b200kv_session_header h;
    std::memset(&h, 0, sizeof h);
    std::memcpy(h.magic, "MISS", 4);
    h.version = kSessionVersion;
    std::strncpy(h.model_id, model_id ? model_id : "", sizeof h.model_id - 1);
    std::strncpy(h.quantization, quantization ? quantization : "", sizeof h.quantization - 1);
    h.prefix_length = prefix_length;
    h.token_hash = b200kv_token_sequence_hash(tokens, prefix_length);
    h.gdn_layers = 0;
    h.gdn_state_bytes = 0;
    h.gqa_layers = layers;
    h.kv_quant_mode = static_cast<uint8_t>(quant_mode);
    h.kv_bytes = layer_bytes * layers;
    h.tokens_bytes = static_cast<uint64_t>(prefix_length) * sizeof(uint32_t);
    h.created_timestamp = static_cast<uint64_t>(
        std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch()).count());
    Trailer t;
    std::memset(&t, 0, sizeof t);
    std::memcpy(t.magic, "B2KV", 4);
    t.kv_heads = kv_heads; t.head_dim = head_dim; t.qblock = qblock; t.layers = layers; t.quant_mode = quant_mode;
    t.layer_bytes = layer_bytes;
    t.checksum = fnv1a_bytes(static_cast<const uint8_t*>(kv_payload), h.kv_bytes);

    std::error_code ec;
    const std::filesystem::path final_path(path);
    if (final_path.has_parent_path()) std::filesystem::create_directories(final_path.parent_path(), ec);
    const std::string tmp = std::string(path) + ".tmp";
    {
        File out(tmp.c_str(), "wb");
        if (out.f == nullptr) return B200KV_ERR_IO;
        if (!out.write(&h, sizeof h) || !out.write(tokens, h.tokens_bytes) || !out.write(kv_payload, h.kv_bytes) || !out.write(&t, sizeof t) ||
            std::fflush(out.f) != 0) {
            std::remove(tmp.c_str());
            return B200KV_ERR_IO;
        }
    }
    std::filesystem::rename(tmp, final_path, ec);
    return ec ? B200KV_ERR_IO : B200KV_OK;
    });
}

int b200kv_session_inspect(const char* path, b200kv_session_header* header, uint32_t* tokens_out, uint32_t tokens_capacity) {
    return guarded([&]() -> int {
    if (path == nullptr || header == nullptr) return B200KV_ERR_INVALID;
    File in(path, "rb");
    if (in.f == nullptr) return B200KV_ERR_IO;
    std::vector<uint32_t> tokens;
    int rc = read_front(in, header, &tokens);
    if (rc != B200KV_OK) return rc;
    if (tokens_out != nullptr) {
        if (tokens_capacity < tokens.size()) return B200KV_ERR_INVALID;
        std::memcpy(tokens_out, tokens.data(), tokens.size() * sizeof(uint32_t));
    }
    return B200KV_OK;
    });
}

int b200kv_session_read(const char* path, const char* model_id, const char* quantization, uint32_t layers, uint32_t kv_heads,
                        uint32_t head_dim, uint32_t qblock, uint32_t quant_mode, uint32_t* tokens_out, uint32_t tokens_capacity,
                        uint32_t* prefix_length_out, void* kv_payload_out, uint64_t payload_capacity) {
    return guarded([&]() -> int {
    if (path == nullptr) return B200KV_ERR_INVALID;
    File in(path, "rb");
    if (in.f == nullptr) return B200KV_ERR_IO;
    b200kv_session_header h;
    std::vector<uint32_t> tokens;
    int rc = read_front(in, &h, &tokens);
    if (rc != B200KV_OK) return rc;
    if (std::string_view(h.model_id) != (model_id ? model_id : "") || std::string_view(h.quantization) != (quantization ? quantization : ""))
        return B200KV_ERR_MISMATCH;                                               // :186-189
    if (h.gdn_layers != 0 || h.gdn_state_bytes != 0 || h.gqa_layers != layers) return B200KV_ERR_MISMATCH;   // :190-192
    if (h.kv_quant_mode != quant_mode) return B200KV_ERR_MISMATCH;                // the check the reference leaves out
    if (h.kv_bytes > payload_capacity || (h.kv_bytes != 0 && kv_payload_out == nullptr)) return B200KV_ERR_INVALID;
    if (!in.read(kv_payload_out, h.kv_bytes)) return B200KV_ERR_FORMAT;
    Trailer t;
    if (!in.read(&t, sizeof t) || std::memcmp(t.magic, "B2KV", 4) != 0) return B200KV_ERR_FORMAT;
    if (t.kv_heads != kv_heads || t.head_dim != head_dim || t.qblock != qblock || t.layers != layers || t.quant_mode != quant_mode)
        return B200KV_ERR_MISMATCH;
    if (t.layer_bytes * layers != h.kv_bytes) return B200KV_ERR_FORMAT;
    if (t.checksum != fnv1a_bytes(static_cast<const uint8_t*>(kv_payload_out), h.kv_bytes)) return B200KV_ERR_FORMAT;
    if (tokens_out != nullptr) {
        if (tokens_capacity < tokens.size()) return B200KV_ERR_INVALID;
        std::memcpy(tokens_out, tokens.data(), tokens.size() * sizeof(uint32_t));
    }
    if (prefix_length_out != nullptr) *prefix_length_out = h.prefix_length;
    return B200KV_OK;
    });
}

int b200kv_session_find(const char* session_dir, const char* model_id, const char* quantization, const uint32_t* prompt,
                        uint32_t prompt_length, char* path_out, size_t path_bytes, uint32_t* prefix_length_out) {
    return guarded([&]() -> int {
    if (session_dir == nullptr || prompt == nullptr || path_out == nullptr) return B200KV_ERR_INVALID;
    std::error_code ec;
    if (!std::filesystem::is_directory(session_dir, ec)) return B200KV_ERR_MISMATCH;
    uint32_t best = 0;
    std::string best_path;
    std::filesystem::directory_iterator it(session_dir, ec), last;
    for (; !ec && it != last; it.increment(ec)) {
        const std::filesystem::directory_entry& entry = *it;
        if (!entry.is_regular_file(ec) || entry.path().extension() != ".miinfer") continue;
        b200kv_session_header h;
        std::vector<uint32_t> tokens;
        File in(entry.path().c_str(), "rb");
        if (in.f == nullptr || read_front(in, &h, &tokens) != B200KV_OK) continue;
        if (std::string_view(h.model_id) != (model_id ? model_id : "") || std::string_view(h.quantization) != (quantization ? quantization : "")) continue;
        if (h.prefix_length == 0 || h.prefix_length > prompt_length) continue;
        if (std::memcmp(tokens.data(), prompt, static_cast<size_t>(h.prefix_length) * sizeof(uint32_t)) != 0) continue;
        if (h.prefix_length > best) { best = h.prefix_length; best_path = entry.path().string(); }   // longest matching prefix wins (:310-313)
    }
    if (best == 0) return B200KV_ERR_MISMATCH;
    if (best_path.size() + 1 > path_bytes) return B200KV_ERR_INVALID;
    std::memcpy(path_out, best_path.c_str(), best_path.size() + 1);
    if (prefix_length_out != nullptr) *prefix_length_out = best;
    return B200KV_OK;
    });
}

int b200kv_session_save(const char* path, const char* model_id, const char* quantization, const uint32_t* tokens,
                        uint32_t prefix_length, const b200kv_view* layer_views, uint32_t layers, void* stream) {
    return guarded([&]() -> int {
    if (layer_views == nullptr || layers == 0 || prefix_length == 0) return B200KV_ERR_INVALID;
    for (uint32_t i = 0; i < layers; ++i) {
        int rc = b200kv::validate_view(&layer_views[i]);
        if (rc != B200KV_OK) return rc;
        if (prefix_length > layer_views[i].capacity) return B200KV_ERR_RANGE;
    }
    if (!same_geometry(layer_views, layers)) return B200KV_ERR_INVALID;
    const size_t layer_bytes = b200kv_snapshot_bytes(&layer_views[0], prefix_length);
    std::vector<uint8_t> payload(layer_bytes * layers);
    for (uint32_t i = 0; i < layers; ++i) {
        int rc = b200kv_snapshot_save(&layer_views[i], prefix_length, payload.data() + static_cast<size_t>(i) * layer_bytes, stream);
        if (rc != B200KV_OK) return rc;
    }
    B200KV_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));   // the reference syncs here too (:112-114)
    return b200kv_session_write(path, model_id, quantization, tokens, prefix_length, payload.data(), layer_bytes, layers,
                                layer_views[0].kv_heads, layer_views[0].head_dim, layer_views[0].qblock, layer_views[0].quant_mode);
    });
}

int b200kv_session_load(const char* path, const char* model_id, const char* quantization, const b200kv_view* layer_views,
                        uint32_t layers, uint32_t* tokens_out, uint32_t tokens_capacity, uint32_t* prefix_length_out, void* stream) {
    return guarded([&]() -> int {
    if (layer_views == nullptr || layers == 0) return B200KV_ERR_INVALID;
    for (uint32_t i = 0; i < layers; ++i) {
        int rc = b200kv::validate_view(&layer_views[i]);
        if (rc != B200KV_OK) return rc;
    }
    if (!same_geometry(layer_views, layers)) return B200KV_ERR_INVALID;
    b200kv_session_header h;
    int rc = b200kv_session_inspect(path, &h, nullptr, 0);
    if (rc != B200KV_OK) return rc;
    for (uint32_t i = 0; i < layers; ++i)
        if (h.prefix_length > layer_views[i].capacity) return B200KV_ERR_RANGE;
    // the payload must be exactly what these caches hold for that many positions: checked before it sizes a buffer
    if (h.gqa_layers != layers) return B200KV_ERR_MISMATCH;
    if (h.kv_bytes != static_cast<uint64_t>(b200kv_snapshot_bytes(&layer_views[0], h.prefix_length)) * layers)
        return h.kv_quant_mode != layer_views[0].quant_mode ? B200KV_ERR_MISMATCH : B200KV_ERR_FORMAT;
    std::vector<uint8_t> payload(h.kv_bytes);
    uint32_t prefix = 0;
    rc = b200kv_session_read(path, model_id, quantization, layers, layer_views[0].kv_heads, layer_views[0].head_dim, layer_views[0].qblock,
                             layer_views[0].quant_mode, tokens_out, tokens_capacity, &prefix, payload.data(), payload.size());
    if (rc != B200KV_OK) return rc;
    const size_t layer_bytes = b200kv_snapshot_bytes(&layer_views[0], prefix);
    if (layer_bytes * layers != payload.size()) return B200KV_ERR_FORMAT;
    for (uint32_t i = 0; i < layers; ++i) {
        rc = b200kv_snapshot_restore(&layer_views[i], prefix, payload.data() + static_cast<size_t>(i) * layer_bytes, stream);
        if (rc != B200KV_OK) return rc;
    }
    B200KV_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));   // the staging buffer dies with this call
    if (prefix_length_out != nullptr) *prefix_length_out = prefix;
    return B200KV_OK;
    });
}

}  // extern "C"
