// Parameter block and split bookkeeping shared by the decode-attention kernels.
#pragma once

#include "kv_common.cuh"

#include <cuda.h>  // CUtensorMap and its enums only; the encoder is fetched at run time, libcuda is not linked

namespace b200kv {

// One session of a batched launch as it sits in the device-side view table: the
// TMA descriptors of its int8 K and V planes (tiles of 16 positions for the warp-level mma kernel, of 128 for the
// tcgen05 kernel) followed by its view.
struct alignas(128) SessionEntry {
    CUtensorMap kmap;
    CUtensorMap vmap;
    CUtensorMap kmap128;
    CUtensorMap vmap128;
    b200kv_view view;
    uint8_t pad[128 - sizeof(b200kv_view)];
};
static_assert(sizeof(SessionEntry) == 640, "table entry layout");

// Upper bound on split slots per launch: slots = sessions * splits_per_session.
constexpr uint32_t kMaxSplitsPerSession = 128;
constexpr uint32_t kSplitSlotBudget = 1024;

inline uint32_t max_splits_per_session(uint32_t sessions) {
    uint32_t s = kSplitSlotBudget / (sessions ? sessions : 1);
    if (s > kMaxSplitsPerSession) s = kMaxSplitsPerSession;
    return s ? s : 1;
}

// Cross-GPU step of a sequence-sharded launch (streaming kernel, one session).  Every rank owns an exchange
// buffer of tagged 8-byte words, [2 phases][world][query_heads][head_dim + 2], zero between launches; peers[w] is
// rank w's buffer as mapped into this process.  After merging its own splits a rank stores its partial of each
// head into slot [phase][rank] of EVERY buffer (peer stores over NVLink), then polls slot [phase][*] of its own
// buffer, merges the `world` partials and zeroes them.  Consecutive launches on one exchange alternate `phase`:
// a fast rank may already be writing the next launch's words while a slow one still reads this launch's.
// Every word carries the call's tag (phase + 1, never 0) in its upper half: words of any other call, e.g. those a
// rank stored after its peers had given up waiting for it, read as "not there yet".
constexpr int kMaxExchangeRanks = 8;
struct ExchangeParams {
    uint64_t* peers[kMaxExchangeRanks];
    uint32_t rank, world, phase, tag;
};

struct MergeParams {
    const float* part_m;   // [groups][num_parts][query_heads]
    const float* part_l;
    const float* part_acc; // [groups][num_parts][query_heads][d]
    uint32_t num_parts;
    uint32_t query_heads;
    uint32_t head_dim;
    size_t part_stride;    // floats between consecutive parts in ALL three arrays; 0 = dense (H for m/l, H*d for acc)
    const float* gate;     // [groups][query_heads][d] or null
    float* output;         // normalised, or null
    float* gated_output;   // normalised * sigmoid(gate), or null
    b200kv_q8_1_block* gated_output_q8;   // the gated output re-quantised to Q8_1 blocks of 32, or null
    float* out_m;          // when non-null: emit ONE merged partial per (group, head) instead
    float* out_l;
    float* out_acc;
    ExchangeParams xchg;   // world == 0: no cross-GPU step
};

struct DecodeParams {
    b200kv_view view;                        // single-session launch
    const SessionEntry* views;               // device table [sessions], or null
    const uint32_t* lengths;                 // device [sessions], or null
    const b200kv_decode_state* decode_state; // device, or null
    uint32_t cache_length;                   // used when neither of the above is given
    uint32_t range_begin;                    // first position scanned (sequence shard), normally 0
    // Suffix/prefill use: "session" t is query token t of ONE cache and attends
    // [0, causal_base + t + 1); prefill_state (device) overrides base and count.
    int causal;
    uint32_t causal_base;
    const b200kv_prefill_state* prefill_state;
    uint32_t sessions;
    const void* q;                           // [sessions][query_heads][d]
    int q_is_f16;
    uint32_t query_heads;
    float scale;
    uint32_t num_splits;                     // per session (batched: of the longest session)
    uint32_t split_positions;                // batched streaming launches: positions per split of a session
    float* ws_m;                             // [sessions][num_splits][query_heads]
    float* ws_l;
    float* ws_acc;                           // [sessions][num_splits][query_heads][d]
    // Fused merge (streaming kernel only): when `ws_tagged` is non-null the partials go out as tagged 8-byte words
    // ([sessions][num_splits][query_heads][head_dim + 2]) and designated CTAs combine all splits and write `fuse`'s
    // outputs; the words must be zero on entry and are zero again on exit.
    // Fused single-token append (streaming kernel, one session): the warp that owns the last tile quantises the new
    // token's K/V row of its kv head and stores it at position end-1 before it loads that tile.
    const void* new_key;                     // [kv_heads*d] of new_is_f16 ? fp16 : fp32, or null = no fused append
    const void* new_value;
    int new_is_f16;
    const float* k_norm_weight;
    int rope_mode;
    float epsilon;
    float sectioned_step;
    float inv_freq[64];                      // NeoX frequencies for d = 128
    uint32_t overlap_tail;                   // launch overlap: the last n positions of the range are read only after pdl_wait
    uint32_t head_fastest;                   // tcgen05 kernel: grid is (kv heads, splits, sessions) instead of (splits, kv heads, sessions)
    uint64_t* ws_tagged;
    uint32_t tag;                            // tag of this launch's words in ws_tagged (never 0; differs from the previous launch's)
    uint32_t* status;                        // device word that collects B200KV_STATUS_* bits of waits that ran out, or null
    uint64_t* timeline;                      // device buffer for per-CTA time stamps (tcgen05 decode kernel), or null
    MergeParams fuse;
};

// TMA descriptors are a pure function of (base address, extents, box, element type, swizzle); encoding one costs a
// driver call.  A decode loop asks for the same few dozen descriptors on every step, so each host thread keeps the last
// ones it encoded (256 entries, direct-mapped on the base address).
struct TensorMapKey {
    const void* base;
    uint64_t rows;
    uint32_t row_bytes, box_bytes, box_rows, kind;   // kind: element type and swizzle as the caller numbers them
    bool operator==(const TensorMapKey& o) const {
        return base == o.base && rows == o.rows && row_bytes == o.row_bytes && box_bytes == o.box_bytes && box_rows == o.box_rows && kind == o.kind;
    }
};
bool tensor_map_lookup(const TensorMapKey& key, CUtensorMap* out);
void tensor_map_remember(const TensorMapKey& key, const CUtensorMap& map);

// Tag for the tagged words of one launch: a process-wide counter that skips 0.
uint32_t next_launch_tag();
// The device buffer registered with b200kv_set_timeline_buffer for the current device (null if none).
uint64_t* current_timeline_buffer(uint32_t ctas);
// The device status word registered with b200kv_set_status_word for the current device (null if none).
uint32_t* current_status_word();
// Which streaming kernel serves int8 caches: 0 = the tcgen05 kernel where it applies, 1 = the warp-level mma kernel.
int streaming_kernel_choice();

// The scanned range [begin, end) of one session, resolved on the device the way
// the reference resolves its DeviceDecodeState (position + 1 entries,
// gfx906/kernels/qwen3_primitives.hip:7394-7395).
__device__ __forceinline__ void resolve_range(const DecodeParams& p, uint32_t session, const b200kv_view& view,
                                              uint32_t* begin, uint32_t* end) {
    uint32_t length = p.cache_length;
    if (p.causal) {
        uint32_t base = p.causal_base, count = p.sessions;
        if (p.prefill_state != nullptr) {
            base = p.prefill_state->base_position;
            count = p.prefill_state->token_count;
        }
        // tokens past the device-side count, or whose causal range leaves the cache, scan nothing
        length = (session < count && static_cast<uint64_t>(base) + session + 1u <= view.capacity) ? base + session + 1u : 0u;
    } else if (p.lengths != nullptr) length = p.lengths[session];
    else if (p.decode_state != nullptr) length = p.decode_state->position + 1u;
    if (length > view.capacity) length = static_cast<uint32_t>(view.capacity);
    *end = length;
    *begin = p.range_begin < length ? p.range_begin : length;
}

__device__ __forceinline__ const b200kv_view& session_view(const DecodeParams& p, uint32_t session) {
    return p.views != nullptr ? p.views[session].view : p.view;
}


int launch_merge(const MergeParams& p, uint32_t groups, cudaStream_t stream);

// Stage 1 into `workspace` (fills p.num_splits and p.ws_*).  num_splits_arg: 0 =
// choose; top bit set = use the generic kernel even where a fast one exists.
// `merge` describes where the combined result goes; *merged is set when the stage-1 kernel did the
// combine itself (then no launch_merge is needed).
int run_decode_stage1(DecodeParams& p, const b200kv_view& geometry, uint32_t max_length, void* workspace,
                      size_t workspace_bytes, uint32_t num_splits_arg, const MergeParams& merge, bool* merged,
                      cudaStream_t stream);
// Split of a caller's workspace of `bytes` bytes: tagged partials in front (two thirds), plain [m][l][acc] partials
// behind.  The split depends only on the size.
inline size_t workspace_plain_offset(size_t bytes) { return bytes / 3 * 2 / 256 * 256; }
int run_decode(DecodeParams& p, const b200kv_view& geometry, uint32_t max_length, void* workspace, size_t workspace_bytes,
               uint32_t num_splits_arg, MergeParams mp, uint32_t groups, cudaStream_t stream);

// Fast path for int8 K and V (decode_q8.cu).  Returns B200KV_ERR_UNSUPPORTED when
// the geometry has no specialised kernel, so the caller can use the generic one.
int launch_decode_q8(const DecodeParams& p, const b200kv_view& geometry, uint32_t max_length, cudaStream_t stream);
// The same launch on the tcgen05 kernel (decode_tc5.cu); B200KV_ERR_UNSUPPORTED where it does not apply.
int launch_decode_tc5(const DecodeParams& p, const b200kv_view& geometry, uint32_t max_length, cudaStream_t stream);
// head_dim 256 on tcgen05 (stage 1 only, plain partials, one session): decode_tc5_wide.cu
bool decode_tc5_wide_ok(const b200kv_view& view, uint32_t query_heads);
uint32_t pick_splits_tc5_wide(const b200kv_view& view, uint32_t max_length);
int launch_decode_tc5_wide(const DecodeParams& p, const b200kv_view& geometry, cudaStream_t stream);
uint32_t pick_splits_q8(const b200kv_view& geometry, uint32_t query_heads, uint32_t sessions, uint32_t max_length);
// TMA descriptors of a view's int8 K and V planes (rows of head_dim bytes, 128-byte swizzle).
// B200KV_ERR_UNSUPPORTED when the view cannot take the streaming kernel (then the generic kernel is used).
int encode_kv_maps(const b200kv_view& view, uint32_t tile_positions, CUtensorMap* kmap, CUtensorMap* vmap);
bool q8_fast_path_ok(const b200kv_view& view, uint32_t query_heads);

}  // namespace b200kv
