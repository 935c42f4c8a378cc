// In-VRAM store of prefix snapshots with longest-prefix lookup, and the prefix-reuse policy of a generation request:
// host code (it allocates and frees device memory; none of it is on the per-token path).
//
// Replaces, for the KV part, the multi-snapshot machinery of MIInfer's first engine
// (tools/miinfer_cli.cpp:1043-1317: SessionCheckpoint, the compressed radix tree insert_session_prefix /
// longest_session_checkpoint, evict_oldest_session_checkpoint, the 8-entry / 3 GiB budget of :62-63, capture only at
// multiples of the 512-token prefill tile :1185) and the reuse branch of PrefillV2Model::generate
// (src/prefill_v2/model.cpp:756-767: an exact prefix strictly shorter than the prompt, the resident context first and
// the session directory second; :869-887: cache_prefix_after / cache_prefix_len, files only for prefixes of at
// least 256 tokens and only if not there yet, write errors not fatal) with the telemetry fields of GenerateStats
// (include/miinfer/prefill_v2/model.hpp:61-68).  A snapshot is kept in the compact raw layout of
// AttentionLayerKvCacheStorage::download_raw, one device allocation per entry, filled and read back with
// b200kv_snapshot_save / b200kv_snapshot_restore on device memory.
#include "kv_common.cuh"

#include <chrono>
#include <cstring>
#include <filesystem>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

// Compressed radix tree over token ids.  A node's edge holds the tokens between its parent and itself.
struct Node {
    std::vector<uint32_t> edge;
    std::unordered_map<uint32_t, std::unique_ptr<Node>> children;
    int entry = -1;   // index into the pool's entry list, or -1
};

void tree_insert(Node& root, const std::vector<uint32_t>& tokens, int entry) {
    Node* node = &root;
    size_t pos = 0;
    while (pos < tokens.size()) {
        std::unique_ptr<Node>& slot = node->children[tokens[pos]];
        if (!slot) {   // a new leaf carries the rest of the sequence
            slot = std::make_unique<Node>();
            slot->edge.assign(tokens.begin() + pos, tokens.end());
            slot->entry = entry;
            return;
        }
        Node& child = *slot;
        size_t shared = 0;
        while (shared < child.edge.size() && pos + shared < tokens.size() && child.edge[shared] == tokens[pos + shared]) ++shared;
        if (shared < child.edge.size()) {
            // the sequences part inside this edge: split it at the point of divergence
            auto upper = std::make_unique<Node>();
            upper->edge.assign(child.edge.begin(), child.edge.begin() + shared);
            std::unique_ptr<Node> lower = std::move(slot);
            lower->edge.erase(lower->edge.begin(), lower->edge.begin() + shared);
            const uint32_t key = lower->edge.front();
            upper->children.emplace(key, std::move(lower));
            slot = std::move(upper);
        }
        pos += shared;
        node = slot.get();
    }
    node->entry = entry;
}

// The entry with the longest token sequence that is a prefix of `prompt` and strictly shorter than it
// (a snapshot holds KV state, not the last position's hidden vector, so at least one token must still be run:
// src/prefill_v2/model.cpp:758-760).  `common` = tokens of the prompt the tree shares with any stored sequence.
int tree_longest(const Node& root, const uint32_t* prompt, size_t n, size_t* common) {
    const Node* node = &root;
    size_t pos = 0;
    int best = -1;
    *common = 0;
    while (pos < n) {
        const auto it = node->children.find(prompt[pos]);
        if (it == node->children.end()) break;
        const Node& child = *it->second;
        size_t shared = 0;
        while (shared < child.edge.size() && pos + shared < n && child.edge[shared] == prompt[pos + shared]) ++shared;
        if (pos + shared > *common) *common = pos + shared;
        if (shared != child.edge.size()) break;
        pos += shared;
        node = &child;
        if (node->entry >= 0 && pos < n) best = node->entry;
    }
    return best;
}

struct Entry {
    std::vector<uint32_t> tokens;
    void* payload = nullptr;       // device memory, or null for an index-only entry
    uint64_t bytes = 0;
    uint64_t last_used = 0;
    std::vector<uint64_t> layer_bytes;   // snapshot bytes per layer (offsets into the payload)
    b200kv_view geometry{};              // kv heads, head_dim, qblock, quant mode the payload was taken with
};

}  // namespace

struct b200kv_pool {
    std::mutex mutex;
    std::string model_id, quantization;
    uint32_t max_entries = 8;
    uint64_t max_bytes = 3ull << 30;
    uint32_t granularity = 512;
    std::vector<Entry> entries;
    Node root;
    uint64_t bytes = 0, clock = 0;
    b200kv_pool_counters counters{};

    void rebuild() {
        root = Node{};
        for (size_t i = 0; i < entries.size(); ++i) tree_insert(root, entries[i].tokens, static_cast<int>(i));
    }
    void drop(size_t i) {
        if (entries[i].payload != nullptr) (void)cudaFree(entries[i].payload);
        bytes -= entries[i].bytes;
        entries.erase(entries.begin() + i);
        ++counters.evictions;
    }
    void evict_oldest() {
        size_t oldest = 0;
        for (size_t i = 1; i < entries.size(); ++i)
            if (entries[i].last_used < entries[oldest].last_used) oldest = i;
        drop(oldest);
        rebuild();
    }
    int find_exact(const uint32_t* tokens, uint32_t n) const {
        for (size_t i = 0; i < entries.size(); ++i)
            if (entries[i].tokens.size() == n && std::memcmp(entries[i].tokens.data(), tokens, sizeof(uint32_t) * n) == 0) return static_cast<int>(i);
        return -1;
    }
    // Makes room for `need` bytes and registers (or refreshes) the entry of `tokens`; returns its index, or -1 when
    // the capture is skipped (granularity, or larger than the whole budget).
    int admit(const uint32_t* tokens, uint32_t n, uint64_t need, bool* fresh) {
        *fresh = false;
        if (n == 0 || (granularity > 1 && n % granularity != 0) || need > max_bytes) { ++counters.skipped; return -1; }
        const int existing = find_exact(tokens, n);
        if (existing >= 0) {
            entries[existing].last_used = ++clock;
            return existing;
        }
        while (!entries.empty() && (entries.size() >= max_entries || bytes + need > max_bytes)) evict_oldest();
        Entry e;
        e.tokens.assign(tokens, tokens + n);
        e.bytes = need;
        e.last_used = ++clock;
        entries.push_back(std::move(e));
        bytes += need;
        *fresh = true;
        rebuild();
        ++counters.captures;
        return static_cast<int>(entries.size() - 1);
    }
};

using namespace b200kv;

namespace {

int snapshot_layout(const b200kv_view* views, uint32_t layers, uint32_t tokens, std::vector<uint64_t>* per_layer, uint64_t* total) {
    *total = 0;
    per_layer->clear();
    for (uint32_t l = 0; l < layers; ++l) {
        const int rc = validate_view(&views[l]);
        if (rc != B200KV_OK) return rc;
        if (tokens > views[l].capacity) return B200KV_ERR_RANGE;
        const uint64_t b = (b200kv_snapshot_bytes(&views[l], tokens) + 255) / 256 * 256;
        per_layer->push_back(b);
        *total += b;
    }
    return B200KV_OK;
}

bool same_shape(const b200kv_view& a, const b200kv_view& b) {
    return a.kv_heads == b.kv_heads && a.head_dim == b.head_dim && a.qblock == b.qblock && a.quant_mode == b.quant_mode;
}

}  // namespace

extern "C" {

int b200kv_pool_create(b200kv_pool** out, const char* model_id, const char* quantization, uint32_t max_entries, uint64_t max_bytes,
                       uint32_t granularity) {
    if (out == nullptr) return B200KV_ERR_INVALID;
    b200kv_pool* p = new (std::nothrow) b200kv_pool;
    if (p == nullptr) return B200KV_ERR_CUDA;
    p->model_id = model_id ? model_id : "";
    p->quantization = quantization ? quantization : "";
    if (max_entries > 0) p->max_entries = max_entries;
    if (max_bytes > 0) p->max_bytes = max_bytes;
    p->granularity = granularity;
    *out = p;
    return B200KV_OK;
}

int b200kv_pool_destroy(b200kv_pool* pool) {
    if (pool == nullptr) return B200KV_OK;
    for (Entry& e : pool->entries)
        if (e.payload != nullptr) (void)cudaFree(e.payload);
    delete pool;
    return B200KV_OK;
}

int b200kv_pool_capture(b200kv_pool* pool, const uint32_t* tokens, uint32_t prefix_length, const b200kv_view* layer_views,
                        uint32_t layers, void* stream, int* captured) {
    if (captured != nullptr) *captured = 0;
    if (pool == nullptr || tokens == nullptr || layer_views == nullptr || layers == 0) return B200KV_ERR_INVALID;
    int rc = ensure_device();
    if (rc != B200KV_OK) return rc;
    std::vector<uint64_t> per_layer;
    uint64_t total = 0;
    if ((rc = snapshot_layout(layer_views, layers, prefix_length, &per_layer, &total)) != B200KV_OK) return rc;
    try {
        std::lock_guard<std::mutex> lock(pool->mutex);
        bool fresh = false;
        const int idx = pool->admit(tokens, prefix_length, total, &fresh);
        if (idx < 0) return B200KV_OK;   // skipped: not an error (the reference returns silently, tools/miinfer_cli.cpp:1185,1201)
        Entry& e = pool->entries[idx];
        if (!fresh && (e.bytes != total || e.payload == nullptr || !same_shape(e.geometry, layer_views[0]))) {
            // the same tokens captured before from caches of another shape (or as an index-only entry): start over
            pool->drop(static_cast<size_t>(idx));
            pool->rebuild();
            --pool->counters.evictions;
            const int again = pool->admit(tokens, prefix_length, total, &fresh);
            if (again < 0) return B200KV_OK;
        }
        Entry& dst = pool->entries[pool->find_exact(tokens, prefix_length)];
        if (dst.payload == nullptr) {
            const cudaError_t err = cudaMalloc(&dst.payload, total);
            if (err != cudaSuccess) {   // out of device memory: the snapshot is simply not kept (:1223-1228)
                set_last_cuda_error(err, "cudaMalloc(pool snapshot)");
                pool->drop(static_cast<size_t>(pool->find_exact(tokens, prefix_length)));
                pool->rebuild();
                --pool->counters.evictions;
                --pool->counters.captures;
                ++pool->counters.skipped;
                return B200KV_OK;
            }
        }
        dst.layer_bytes = per_layer;
        dst.geometry = layer_views[0];
        uint64_t off = 0;
        for (uint32_t l = 0; l < layers; ++l) {
            rc = b200kv_snapshot_save(&layer_views[l], prefix_length, static_cast<uint8_t*>(dst.payload) + off, stream);
            if (rc != B200KV_OK) return rc;
            off += per_layer[l];
        }
        if (captured != nullptr) *captured = 1;
    } catch (const std::exception&) {
        return B200KV_ERR_CUDA;
    }
    return B200KV_OK;
}

int b200kv_pool_capture_index_only(b200kv_pool* pool, const uint32_t* tokens, uint32_t prefix_length, uint64_t bytes, int* captured) {
    if (captured != nullptr) *captured = 0;
    if (pool == nullptr || tokens == nullptr) return B200KV_ERR_INVALID;
    try {
        std::lock_guard<std::mutex> lock(pool->mutex);
        bool fresh = false;
        const int idx = pool->admit(tokens, prefix_length, bytes, &fresh);
        if (idx >= 0 && captured != nullptr) *captured = 1;
    } catch (const std::exception&) {
        return B200KV_ERR_CUDA;
    }
    return B200KV_OK;
}

int b200kv_pool_lookup(b200kv_pool* pool, const char* model_id, const char* quantization, const uint32_t* prompt,
                       uint32_t prompt_length, uint32_t* matched_length, uint32_t* common_length) {
    if (matched_length != nullptr) *matched_length = 0;
    if (common_length != nullptr) *common_length = 0;
    if (pool == nullptr || (prompt == nullptr && prompt_length > 0)) return B200KV_ERR_INVALID;
    std::lock_guard<std::mutex> lock(pool->mutex);
    // snapshots of another model or weight quantization are not candidates (session_checkpoint_compatible, :1073-1079)
    if ((model_id != nullptr && pool->model_id != model_id) || (quantization != nullptr && pool->quantization != quantization)) {
        ++pool->counters.misses;
        return B200KV_OK;
    }
    size_t common = 0;
    const int best = tree_longest(pool->root, prompt, prompt_length, &common);
    if (common_length != nullptr) *common_length = static_cast<uint32_t>(common);
    if (best < 0) { ++pool->counters.misses; return B200KV_OK; }
    ++pool->counters.hits;
    pool->entries[best].last_used = ++pool->clock;
    if (matched_length != nullptr) *matched_length = static_cast<uint32_t>(pool->entries[best].tokens.size());
    return B200KV_OK;
}

int b200kv_pool_restore(b200kv_pool* pool, const uint32_t* prompt, uint32_t prompt_length, const b200kv_view* layer_views,
                        uint32_t layers, void* stream, uint32_t* matched_length) {
    if (matched_length != nullptr) *matched_length = 0;
    if (pool == nullptr || prompt == nullptr || layer_views == nullptr || layers == 0) return B200KV_ERR_INVALID;
    int rc = ensure_device();
    if (rc != B200KV_OK) return rc;
    std::lock_guard<std::mutex> lock(pool->mutex);
    size_t common = 0;
    const int best = tree_longest(pool->root, prompt, prompt_length, &common);
    if (best < 0 || pool->entries[best].payload == nullptr) { ++pool->counters.misses; return B200KV_OK; }
    Entry& e = pool->entries[best];
    const uint32_t n = static_cast<uint32_t>(e.tokens.size());
    if (e.layer_bytes.size() != layers) return B200KV_ERR_MISMATCH;
    for (uint32_t l = 0; l < layers; ++l) {
        if ((rc = validate_view(&layer_views[l])) != B200KV_OK) return rc;
        if (!same_shape(e.geometry, layer_views[l])) return B200KV_ERR_MISMATCH;
        if (n > layer_views[l].capacity) return B200KV_ERR_RANGE;
    }
    uint64_t off = 0;
    for (uint32_t l = 0; l < layers; ++l) {
        rc = b200kv_snapshot_restore(&layer_views[l], n, static_cast<const uint8_t*>(e.payload) + off, stream);
        if (rc != B200KV_OK) return rc;
        off += e.layer_bytes[l];
    }
    ++pool->counters.hits;
    e.last_used = ++pool->clock;
    if (matched_length != nullptr) *matched_length = n;
    return B200KV_OK;
}

int b200kv_pool_stats(b200kv_pool* pool, b200kv_pool_counters* out) {
    if (pool == nullptr || out == nullptr) return B200KV_ERR_INVALID;
    std::lock_guard<std::mutex> lock(pool->mutex);
    *out = pool->counters;
    out->entries = static_cast<uint32_t>(pool->entries.size());
    out->bytes = pool->bytes;
    return B200KV_OK;
}

// ---- the reuse policy of one generation request -------------------------------------------------------------

int b200kv_reuse_begin(const b200kv_reuse_options* options, const char* model_id, const char* quantization,
                       const char* resident_model_id, const char* resident_quantization, uint32_t resident_layout_version,
                       const uint32_t* resident_tokens, uint32_t resident_length,
                       b200kv_pool* pool, const uint32_t* prompt, uint32_t prompt_length,
                       const b200kv_view* layer_views, uint32_t layers, void* stream, b200kv_reuse_stats* stats) {
    if (options == nullptr || stats == nullptr || (prompt == nullptr && prompt_length > 0)) return B200KV_ERR_INVALID;
    std::memset(stats, 0, sizeof *stats);
    stats->suffix_tokens_dispatched = prompt_length;
    if (!options->enable_prefix_reuse) return B200KV_OK;
    const auto t0 = std::chrono::steady_clock::now();
    uint32_t prefix = 0;
    int source = B200KV_REUSE_NONE;
    // 1. the prefix already resident in the caches: exact match and strictly shorter than the prompt (model.cpp:756-767)
    if (resident_length > 0 && resident_tokens != nullptr) {
        const int match = b200kv_prefix_match(resident_model_id, resident_quantization, resident_layout_version, resident_tokens,
                                              resident_length, model_id, quantization, prompt, prompt_length);
        if (match == B200KV_MATCH_EXACT && resident_length < prompt_length) { prefix = resident_length; source = B200KV_REUSE_RESIDENT; }
    }
    // 2. the in-VRAM pool: longest stored proper prefix, cloned into the caches
    if (source == B200KV_REUSE_NONE && pool != nullptr) {
        uint32_t matched = 0;
        int rc = B200KV_OK;
        if (layers > 0 && layer_views != nullptr) {
            bool compatible;
            {
                std::lock_guard<std::mutex> lock(pool->mutex);
                compatible = (model_id == nullptr || pool->model_id == model_id) && (quantization == nullptr || pool->quantization == quantization);
            }
            if (compatible) rc = b200kv_pool_restore(pool, prompt, prompt_length, layer_views, layers, stream, &matched);
        } else {
            rc = b200kv_pool_lookup(pool, model_id, quantization, prompt, prompt_length, &matched, nullptr);
        }
        if (rc != B200KV_OK && rc != B200KV_ERR_MISMATCH) return rc;
        if (matched > 0) { prefix = matched; source = B200KV_REUSE_POOL; }
    }
    // 3. the session directory: the file with the longest matching prefix (restore_matching_session, model.cpp:769-775)
    if (source == B200KV_REUSE_NONE && options->persistent_session_dir != nullptr && options->persistent_session_dir[0] != '\0') {
        char path[4096];
        uint32_t disk_prefix = 0;
        if (b200kv_session_find(options->persistent_session_dir, model_id, quantization, prompt, prompt_length, path, sizeof path, &disk_prefix) ==
                B200KV_OK && disk_prefix > 0 && disk_prefix < prompt_length) {
            bool ok = true;
            if (layers > 0 && layer_views != nullptr) {
                uint32_t loaded = 0;
                ok = b200kv_session_load(path, model_id, quantization, layer_views, layers, nullptr, 0, &loaded, stream) == B200KV_OK &&
                     loaded == disk_prefix;
            }
            if (ok) { prefix = disk_prefix; source = B200KV_REUSE_DISK; }
        }
    }
    if (source != B200KV_REUSE_NONE) {
        if (layers > 0 && source != B200KV_REUSE_RESIDENT) (void)cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
        stats->reuse_hit = 1;
        stats->source = source;
        stats->prefix_tokens_reused = prefix;
        stats->suffix_tokens_dispatched = prompt_length - prefix;
        stats->gqa_kv_reused_tokens = prefix;
        stats->restore_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    }
    return B200KV_OK;
}

int b200kv_reuse_commit(const b200kv_reuse_options* options, const char* model_id, const char* quantization, b200kv_pool* pool,
                        const uint32_t* prompt, uint32_t prompt_length, const b200kv_view* layer_views, uint32_t layers,
                        void* stream, uint32_t* cached_length, int* wrote_file) {
    if (cached_length != nullptr) *cached_length = 0;
    if (wrote_file != nullptr) *wrote_file = 0;
    if (options == nullptr || (prompt == nullptr && prompt_length > 0)) return B200KV_ERR_INVALID;
    if (!options->cache_prefix_after || prompt_length == 0) return B200KV_OK;
    // cache_prefix_len 0 = the whole prompt, otherwise its first N tokens (model.cpp:870)
    const uint32_t save_len = options->cache_prefix_len > 0 ? (options->cache_prefix_len < prompt_length ? options->cache_prefix_len : prompt_length)
                                                             : prompt_length;
    if (cached_length != nullptr) *cached_length = save_len;   // what the caller records as its resident prefix
    if (pool != nullptr) {
        int rc;
        if (layers > 0 && layer_views != nullptr) rc = b200kv_pool_capture(pool, prompt, save_len, layer_views, layers, stream, nullptr);
        else rc = b200kv_pool_capture_index_only(pool, prompt, save_len, 0, nullptr);
        if (rc != B200KV_OK) return rc;
    }
    // a file only for prefixes of at least 256 tokens, only if it is not there yet, and a failed write is not fatal (:872-886)
    if (options->persistent_session_dir != nullptr && options->persistent_session_dir[0] != '\0' && save_len >= 256 && layers > 0 &&
        layer_views != nullptr) {
        try {
            char name[96];
            if (b200kv_session_filename(b200kv_token_sequence_hash(prompt, save_len), save_len, name, sizeof name) == B200KV_OK) {
                const std::filesystem::path path = std::filesystem::path(options->persistent_session_dir) / name;
                std::error_code ec;
                if (!std::filesystem::exists(path, ec)) {
                    const int rc = b200kv_session_save(path.string().c_str(), model_id, quantization, prompt, save_len, layer_views, layers, stream);
                    if (rc == B200KV_OK && wrote_file != nullptr) *wrote_file = 1;
                }
            }
        } catch (const std::exception&) {
            // non-fatal
        }
    }
    return B200KV_OK;
}

}  // extern "C"
