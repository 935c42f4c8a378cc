/*
 * b200kv.h -- C ABI of the B200-native quantized KV-cache path.
 *
 * This is the boundary a MIInfer maintainer binds in place of the HIP operator
 * layer for the KV path.  The reference has no FFI: its boundary is a set of
 * C++ free functions with C-compatible arguments
 * (include/miinfer/qwen3_gpu_primitives.hpp) plus one POD view struct
 * (include/miinfer/prefill_v2/kv_cache.hpp:24-46).  Every entry point below
 * names the reference interface it replaces (paths relative to the MIInfer
 * source tree).
 *
 * Conventions
 *   - Plain pointers and sizes only.  Device pointers unless stated otherwise.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *   - Every function returns a b200kv_status (0 = ok, negative = error); nothing
 *     aborts the process, reads the environment or allocates device memory in a
 *     launch call (the reference launchers abort on a bad argument,
 *     include/miinfer/hip_check.hpp:11-24, and allocate nothing).
 *   - All launches are asynchronous on `stream`; the caller owns every buffer.
 *   - There is no CPU fallback: without a usable sm_100 device every launch
 *     returns B200KV_ERR_DEVICE.
 */
#ifndef B200KV_H
#define B200KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200KV_VERSION 200 /* 0.2.0 */

#if defined(__GNUC__)
#define B200KV_API __attribute__((visibility("default")))
#else
#define B200KV_API
#endif

/* OR into `num_splits` to run the generic stage-1 kernel even where a
 * specialised one exists (testing and A/B measurement). */
#define B200KV_SPLITS_FORCE_GENERIC 0x80000000u

typedef enum b200kv_status {
    B200KV_OK = 0,
    B200KV_ERR_INVALID = -1,     /* null/mismatched argument (reference: hipErrorInvalidValue + abort) */
    B200KV_ERR_UNSUPPORTED = -2, /* shape or mode this build has no kernel for */
    B200KV_ERR_CUDA = -3,        /* a CUDA runtime call failed; see b200kv_last_cuda_error */
    B200KV_ERR_DEVICE = -4,      /* no sm_100 device */
    B200KV_ERR_WORKSPACE = -5,   /* workspace too small */
    B200KV_ERR_RANGE = -6,       /* positions beyond the cache capacity */
    B200KV_ERR_FORMAT = -7,      /* session file: bad magic/version/geometry/checksum */
    B200KV_ERR_IO = -8,          /* session file: open/read/write failed */
    B200KV_ERR_MISMATCH = -9     /* session file does not match the requested prefix */
} b200kv_status;

/* Bits a kernel ORs into the status word registered with b200kv_set_status_word when one of its bounded waits
 * runs out (the launch then ends, its outputs are NaN, and the host learns why from this word). */
#define B200KV_STATUS_COPY_TIMEOUT 1u   /* a tile copy (TMA) never completed */
#define B200KV_STATUS_SPLIT_TIMEOUT 2u  /* the in-launch merge never saw the partial of one of its splits */
#define B200KV_STATUS_PEER_TIMEOUT 4u   /* the cross-GPU merge never saw the partial of one of its peers */
#define B200KV_STATUS_PIPE_TIMEOUT 8u   /* a tensor-core pipeline stage (MMA completion) never signalled */

/* KvCacheQuantMode, include/miinfer/prefill_v2/kv_cache.hpp:16-21 (same values). */
typedef enum b200kv_quant_mode {
    B200KV_F16_F16 = 0,
    B200KV_Q8_F16 = 1, /* int8 K, fp16 V */
    B200KV_F16_Q8 = 2,
    B200KV_Q8_Q8 = 3
} b200kv_quant_mode;

typedef enum b200kv_dtype { B200KV_F16 = 0, B200KV_F32 = 1 } b200kv_dtype;

/* RoPE applied to K inside the append kernel.
 * NEOX_FULL: pairs (i, i+d/2), frequency powf(theta, -2i/d) -- qwen3_rope_kernel,
 *   gfx906/kernels/qwen3_primitives.hip:1850-1870.
 * SECTIONED64: pairs (i, i+32) on dims [0,64), angle position * s^i by successive
 *   fp32 multiplies with s = powf(theta, -2/64) -- compute_qwen35_rope_pair, .hip:622-659. */
typedef enum b200kv_rope_mode { B200KV_ROPE_NONE = 0, B200KV_ROPE_NEOX_FULL = 1, B200KV_ROPE_SECTIONED64 = 2 } b200kv_rope_mode;

/*
 * Non-owning view of one attention layer's KV cache in device memory.
 * Replaces AttentionKvCacheView (include/miinfer/prefill_v2/kv_cache.hpp:24-46):
 * same planar pointers, plus `qblock`.  Layout (head-major, as the reference):
 *   key_f16/value_f16    [kv_heads][capacity][head_dim]            fp16
 *   key_q8/value_q8      [kv_heads][capacity][head_dim]            int8
 *   key/value_scales     [kv_heads][capacity][head_dim / qblock]   fp16
 * qblock == 32 is the q8_0 format (32 int8 + one fp16 scale: 136 B per 128-wide
 * head row); qblock == head_dim is the reference's one-scale-per-row format.
 * All plane base pointers must be 16-byte aligned.
 */
typedef struct b200kv_view {
    void* key_f16;
    void* value_f16;
    int8_t* key_q8;
    void* key_scales;
    int8_t* value_q8;
    void* value_scales;
    uint64_t capacity;  /* positions per head */
    uint32_t kv_heads;
    uint32_t head_dim;  /* 128 or 256 */
    uint32_t qblock;    /* 32 or head_dim */
    uint32_t quant_mode; /* b200kv_quant_mode */
} b200kv_view;

/* Device-resident step state so a captured graph replays with new positions.
 * Same layout as DeviceDecodeState / DevicePrefillState,
 * include/miinfer/qwen3_gpu_primitives.hpp:30-45 (64-byte aligned, 64 bytes). */
typedef struct b200kv_decode_state {
    uint32_t current_token, position, generated, stop, max_generated;
    uint32_t pad_[11];
} b200kv_decode_state;
typedef struct b200kv_prefill_state {
    uint32_t base_position, token_count, total_length, kv_capacity;
    uint32_t pad_[12];
} b200kv_prefill_state;

/* One block of the Q8_1 activation format the reference's projections consume: Q8_1Block,
 * include/miinfer/q4_q8_gemv.hpp:23-27 (36 bytes: fp16 d, fp16 s = d * sum(qs), 32 int8). */
typedef struct b200kv_q8_1_block {
    uint16_t d;    /* fp16 bits */
    uint16_t s;    /* fp16 bits */
    int8_t qs[32];
} b200kv_q8_1_block;

/* ---- library / device ------------------------------------------------------ */

B200KV_API int b200kv_version(void);
B200KV_API const char* b200kv_status_string(int status);
/* Text of the last CUDA error seen by this thread's calls (empty if none). */
B200KV_API const char* b200kv_last_cuda_error(void);
/* sm_100 guard; replaces validate_device (src/device_validation.cpp:60-95), which accepts gfx906 only. */
B200KV_API int b200kv_device_check(int device);

/* Launch overlap (off by default; process-wide; no counterpart in the reference,
 * which replays a HIP graph of fully serialised kernels, src/prefill_v2/model.cpp:1136-1197).
 * With tail_positions > 0 the append, streaming decode, merge and prefill
 * kernels are launched with programmatic stream serialization: a kernel may
 * become resident, set itself up and (decode) start streaming OLD cache rows
 * while the previous kernel of the stream is still finishing -- this hides
 * launch ramp and tail between the layers of a decode step and between the
 * kernels of a prefill chunk.  The kernels order themselves: everything a preceding kernel may
 * produce -- Q, gate, the workspace, outputs, and the last `tail_positions`
 * rows of the scanned cache range -- is only touched after that kernel has
 * completed (griddepcontrol.wait).  Set tail_positions >= the number of rows
 * the preceding kernel can append (1 in a decode loop).  Device-side state
 * (decode_state, lengths) is read early, so it must not be written by a kernel
 * that itself triggers dependents early; kernels of this library never do, and
 * an ordinary kernel between two launches acts as a full barrier.  0 turns the
 * overlap off again. */
B200KV_API int b200kv_set_launch_overlap(uint32_t tail_positions);

/* Registers a 4-byte-aligned DEVICE word (on the current device; NULL = none, the default) into which every later
 * launch of this library on that device ORs a B200KV_STATUS_* bit when one of its bounded waits runs out.  The
 * reference aborts the process on any device error (include/miinfer/hip_check.hpp:11-24); here a lost copy or a
 * peer that never delivers ends the launch with NaN outputs and this word says which wait it was.  The word is
 * sticky: the caller zeroes it.  After a non-zero status the tagged words of the workspace (and, for a sharded
 * launch, of the exchange buffers of ALL ranks, behind a barrier) must be cleared before they are used again:
 * b200kv_workspace_reset, or a plain memset. */
B200KV_API int b200kv_set_status_word(uint32_t* device_word);
/* Zero-fills a decode workspace (or an exchange buffer) asynchronously on `stream`. */
B200KV_API int b200kv_workspace_reset(void* workspace, size_t workspace_bytes, void* stream);
/* Tracing (the reference times its stages with event pairs in *_profiled twins of its layer functions,
 * src/prefill_v2/attention_layer.cpp:391-549): registers a DEVICE buffer of 8-byte words on the current device (NULL =
 * off, the default) into which every CTA of session 0 of a later tcgen05 decode launch writes 8 nanosecond time
 * stamps (%globaltimer) at [(kv_head * splits + split) * 8]: CTA start, dependency wait over, set-up done, first score
 * tile seen, tile loop over, last sums folded, partial written, merge done (0 where a CTA has no such step).  Launches
 * whose grid does not fit the buffer are not traced. */
B200KV_API int b200kv_set_timeline_buffer(uint64_t* device_words, uint32_t capacity_words);
/* Which streaming kernel serves int8 caches (process-wide; for A/B measurement and tests): 0 = the tcgen05 kernels
 * where they apply (default), 1 = none of them: the warp-level mma kernel at head_dim 128, the generic kernel at
 * head_dim 256.  No counterpart in the reference. */
B200KV_API int b200kv_set_decode_kernel(int choice);

/* ---- cache storage ---------------------------------------------------------
 * Replaces class AttentionLayerKvCacheStorage (kv_cache.hpp:49-122,
 * src/prefill_v2/kv_cache.cpp:10-130): owns the 2-4 device planes of one layer. */
typedef struct b200kv_cache b200kv_cache;

/* key_bytes()+value_bytes() for a geometry, kv_cache.hpp:88-106 (scale bytes generalised to 2*head_dim/qblock per row). */
B200KV_API size_t b200kv_cache_bytes(uint64_t capacity, uint32_t kv_heads, uint32_t head_dim, uint32_t qblock, uint32_t quant_mode);
/* ctor, kv_cache.cpp:10-39: allocates on the current device and zero-fills.  capacity 0 -> B200KV_ERR_INVALID (the ctor throws). */
B200KV_API int b200kv_cache_create(b200kv_cache** out, uint64_t capacity, uint32_t kv_heads, uint32_t head_dim,
                        uint32_t qblock, uint32_t quant_mode);
/* dtor, kv_cache.cpp:41-67. */
B200KV_API int b200kv_cache_destroy(b200kv_cache* cache);
/* reset(stream), kv_cache.cpp:99-130: zero every plane, asynchronously on `stream`. */
B200KV_API int b200kv_cache_reset(b200kv_cache* cache, void* stream);
/* view(), kv_cache.hpp:68-81. */
B200KV_API int b200kv_cache_view(const b200kv_cache* cache, b200kv_view* out);

/* ---- append ----------------------------------------------------------------
 * Replaces launch_qwen35_decoupled_k_norm_rope_kv_store_batch_quant
 * (include/miinfer/qwen3_gpu_primitives.hpp:695-716; kernel
 * gfx906/kernels/qwen3_primitives.hip:7213-7326).
 * key/value: [token][kv_heads*head_dim] of `dtype`.  k_norm_weight (fp32
 * [head_dim]) may be NULL = no K RMSNorm (the reference requires it).  Token t
 * goes to position base_position + t; a non-NULL prefill_state (base_position,
 * token_count, kv_capacity>0 overrides capacity) or decode_state (position,
 * one token) is read ON THE DEVICE instead, exactly as the reference kernel does
 * (.hip:7235-7242) -- in that case `token_count` is the launch bound (rows beyond
 * the device-side count are skipped).  Quantizer: per qblock scale = amax/127
 * (1 if amax==0), inv = 1/scale, q = clamp(rint_half_even(x*inv), -128, 127),
 * scale stored as fp16 round-to-nearest (.hip:7285-7300). */
B200KV_API int b200kv_append(const b200kv_view* view, const void* key, const void* value, int dtype,
                  const float* k_norm_weight, int rope_mode, float theta, float epsilon,
                  uint32_t token_count, uint32_t base_position,
                  const b200kv_prefill_state* prefill_state, const b200kv_decode_state* decode_state,
                  void* stream);

/* ---- the query side and the step state (the operators either side of the KV path in a step) ---------------- */

/* Replaces launch_qwen35_decoupled_q_split_norm_rope_batch (include/miinfer/qwen3_gpu_primitives.hpp:869-881; kernel
 * gfx906/kernels/qwen3_primitives.hip:994-1045) and launch_qwen35_fused_q_split_norm_rope_dynamic (hpp:934-938;
 * kernel .hip:661-717).  qfull: the query projection's output [token][heads][q (head_dim) | gate (head_dim)] of
 * in_dtype.  Writes query [token][heads][head_dim] of out_dtype = RoPE(RMSNorm(q) * q_norm_weight) at position
 * base_position + token, and gate (fp32, same shape; may be NULL).  q_norm_weight may be NULL (no norm).  A
 * non-NULL prefill_state (base_position, token_count) or decode_state (position; one token) is read on the device
 * as in b200kv_append.  The norm and the RoPE are the append kernel's, bit for bit, so a query and the key
 * appended at the same position are rotated identically. */
B200KV_API int b200kv_q_split_norm_rope(const void* qfull, int in_dtype, const float* q_norm_weight, void* query, int out_dtype,
                             float* gate, uint32_t token_count, uint32_t base_position, uint32_t heads, uint32_t head_dim,
                             int rope_mode, float theta, float epsilon, const b200kv_prefill_state* prefill_state,
                             const b200kv_decode_state* decode_state, void* stream);

/* Replaces launch_qwen35_decode_state_advance (qwen3_gpu_primitives.hpp:1248-1250; kernel .hip:4417-4428): on the
 * device, record state->current_token at token_output[state->generated] (if below `capacity`), set state->stop on
 * an end-of-text token (151643, 151645) or when max_generated is reached, and advance position and generated by
 * one -- so that a captured decode graph replays at the next position without the host touching the state. */
B200KV_API int b200kv_decode_state_advance(b200kv_decode_state* state, uint32_t* token_output, uint32_t capacity, void* stream);

/* ---- decode attention ------------------------------------------------------- */

/* Workspace bytes for the split-K partials of one decode launch over
 * `sessions` sessions.  The reference keeps these in file-scope __device__
 * arrays sized for 24 heads (.hip:2104-2113); here the caller owns them.
 * The workspace must be 16-byte aligned and ZERO-FILLED ONCE before its first
 * use (cudaMemset): its first two thirds hold the tagged partials of the fused
 * merge (8-byte words {value, tag}; a zero tag means "not written yet"), which
 * every launch leaves at zero again; the last third holds plain partials.  Pass
 * the same workspace_bytes for a buffer on every call: the split between the
 * two parts is derived from it.  One workspace serves one launch at a time
 * (launches that overlap on the GPU need separate workspaces). */
B200KV_API size_t b200kv_decode_workspace_bytes(uint32_t query_heads, uint32_t head_dim, uint32_t sessions);

/* Replaces launch_qwen35_tiled_online_attention_quant_dynamic
 * (qwen3_gpu_primitives.hpp:719-739; kernels .hip:7371-7485 and 2295-2352).
 * One query token per session: q [query_heads][head_dim] of q_dtype; attends
 * positions [0, cache_length), or [0, decode_state->position + 1) read on the
 * device when decode_state != NULL (.hip:7394-7395).  output (ungated) and
 * gated_output (= output * sigmoid(gate), gate fp32 [query_heads][head_dim]) are
 * fp32 [query_heads][head_dim]; at least one must be non-NULL; gate may be NULL
 * (then gated_output == output).  num_splits 0 = choose for the device.
 * gated_output_q8 (may be NULL): the gated output re-quantised to Q8_1 blocks of 32 for the projection that
 * follows, [query_heads * head_dim / 32] blocks, as the reference's stage 2 does (.hip:2354-2383: d = amax/127,
 * q = roundf(x/d) clamped to +-127, s = d * sum(q), d and s stored as fp16).  Unlike the reference it is also
 * produced when gate is NULL (from the ungated output). */
B200KV_API int b200kv_decode_attn(const b200kv_view* view, const void* q, int q_dtype, const float* gate,
                       float* output, float* gated_output, b200kv_q8_1_block* gated_output_q8, uint32_t query_heads, float scale,
                       uint32_t cache_length, const b200kv_decode_state* decode_state,
                       void* workspace, size_t workspace_bytes, uint32_t num_splits, void* stream);

/* One decode step of a layer in ONE launch: append the new token's K/V row at `position` (or at
 * decode_state->position, read on the device) and attend positions [0, position].  Equivalent to b200kv_append
 * (one token) followed by b200kv_decode_attn(cache_length = position + 1) -- the call pair of
 * src/prefill_v2/attention_layer.cpp:599-632 -- with bit-identical cache contents; the streaming kernel does the
 * append inside the CTA that owns the last tile, which removes a launch and its latency from every layer.
 * key/value: [kv_heads*head_dim] of kv_dtype.  Caches the streaming kernel does not support fall back to the two
 * launches.  If decode_state is given the position must be below the capacity (the kernel cannot report it). */
B200KV_API int b200kv_decode_step(const b200kv_view* view, const void* key, const void* value, int kv_dtype,
                       const float* k_norm_weight, int rope_mode, float theta, float epsilon,
                       const void* q, int q_dtype, const float* gate, float* output, float* gated_output,
                       b200kv_q8_1_block* gated_output_q8, uint32_t query_heads, float scale, uint32_t position, const b200kv_decode_state* decode_state,
                       void* workspace, size_t workspace_bytes, uint32_t num_splits, void* stream);

/* Decode attention without a caller-supplied workspace and without any allocation (no counterpart in the
 * reference).  For hosts that cannot allocate device memory once they are running -- a serving process
 * that gave all device memory to its own pool at start-up and forbids driver allocations afterwards, or a
 * sandbox in which allocation calls are not allowed -- and so cannot provide the split-K scratch of
 * b200kv_decode_attn.  Same arguments and results as b200kv_decode_attn, minus the workspace pair; the scratch
 * is a fixed 8 MiB array inside the library (b200kv_decode_static_scratch_bytes), present on every GPU
 * that loads the library until the process exits.
 *   - Limit: b200kv_decode_workspace_bytes(query_heads, head_dim, 1) must not exceed that size (32 query heads
 *     at head_dim 128 and 20 at head_dim 256 fit); larger shapes return B200KV_ERR_WORKSPACE.
 *   - The first call on each device looks up the array's device address (the device must be current); make
 *     that first call before starting any stream capture.
 *   - All calls on a device share the one array: two calls whose kernels overlap on the GPU (different
 *     streams, or launch overlap between them) race on it.  Calls ordered on one stream are safe.
 *   - It calls no cudaMalloc, cudaFree or allocating library routine, and adds no work to the stream beyond
 *     the kernels b200kv_decode_attn launches (the array needs no clearing between calls: launches zero the
 *     words they consumed, and words left by a launch that gave up carry a tag no later launch accepts). */
B200KV_API size_t b200kv_decode_static_scratch_bytes(void);
B200KV_API int b200kv_decode_attn_static(const b200kv_view* view, const void* q, int q_dtype, const float* gate,
                              float* output, float* gated_output, uint32_t query_heads, float scale,
                              uint32_t cache_length, const b200kv_decode_state* decode_state,
                              uint32_t num_splits, void* stream);

/* Sequence-sharded decode attention with the cross-GPU merge inside the kernel (no counterpart in the reference,
 * which is single-GPU; the long-context workload: one 131072-token session over 1/2/4/8 GPUs).  One process per GPU; this rank attends positions
 * [range_begin, range_end) of ITS OWN cache shard, stores its per-head partial (m, l, acc) as tagged 8-byte
 * words into slot [phase][rank] of every rank's exchange buffer (plain peer stores over NVLink, no multicast),
 * polls its own buffer until the `world` partials of a head are there (bounded: a rank that never shows up turns
 * the output into NaN instead of hanging the GPU), merges them and zeroes the words again.  Every rank ends
 * with the same output.  exchange[w]: rank w's buffer as mapped into this process (exchange[rank] = its own),
 * each of b200kv_exchange_bytes() bytes.  All ranks must launch the same sequence of sharded calls.  `phase` is
 * the call's number on this exchange: any 32-bit value below 0xffffffff that all ranks agree on and that differs
 * from the previous call's by an odd amount (0, 1, 2, ... is the natural choice; a captured graph may repeat its
 * own numbers on every replay).  Its lowest bit selects one of two slots -- a fast rank may already be writing the
 * next call's words while a slow one still reads this call's -- and phase + 1 tags every word, so that words a
 * late rank stores after its peers gave up are not taken for a later call's.  If any rank's status word shows
 * B200KV_STATUS_PEER_TIMEOUT, clear the exchange buffers on all ranks behind a barrier before going on.
 * Streaming-kernel caches only (see
 * b200kv_decode_kernel_kind); others return B200KV_ERR_UNSUPPORTED and use b200kv_decode_partials + an
 * all-gather + b200kv_merge_partials_packed.  world <= 8. */
B200KV_API size_t b200kv_exchange_bytes(uint32_t query_heads, uint32_t head_dim, uint32_t world);
B200KV_API int b200kv_decode_attn_sharded(const b200kv_view* view, const void* q, int q_dtype, const float* gate,
                               float* output, float* gated_output, uint32_t query_heads, float scale,
                               uint32_t range_begin, uint32_t range_end,
                               void* const* exchange, uint32_t rank, uint32_t world, uint32_t phase,
                               void* workspace, size_t workspace_bytes, uint32_t num_splits, void* stream);

/* Set-up of the exchange buffers (these allocate and are not for the per-token path): create allocates `bytes`
 * of zeroed device memory on the current device and returns a 64-byte handle that another process on the same
 * node passes to open to map the buffer; close unmaps it, destroy frees it (after every peer has closed it). */
B200KV_API int b200kv_exchange_create(size_t bytes, void** buffer, void* handle64);
B200KV_API int b200kv_exchange_open(const void* handle64, void** peer_buffer);
B200KV_API int b200kv_exchange_close(void* peer_buffer);
B200KV_API int b200kv_exchange_destroy(void* buffer);

/* Which stage-1 kernel b200kv_decode_attn picks for this view: 1 = the streaming
 * int8 kernels (int8 K and V, head_dim 128, 1/2/4 query heads per kv head,
 * capacity a multiple of 8; merge, append and cross-GPU exchange fused in),
 * 2 = the tcgen05 stage 1 for head_dim 256 (int8 K and V, 4/6/8 query heads per
 * kv head, capacity a multiple of 8; single-session launches, the merge kernel
 * follows), 0 = the generic kernel (every other mode and shape).
 * No counterpart in the reference. */
B200KV_API int b200kv_decode_kernel_kind(const b200kv_view* view, uint32_t query_heads);

/* Batched decode over `sessions` independent caches of one geometry (no
 * counterpart in the reference, which keeps one session resident,
 * tools/miinfer_cli.cpp:5663-5676).  views: HOST array of `sessions` views
 * (same head_dim, kv_heads, qblock, quant_mode; capacities may differ);
 * lengths: DEVICE array of `sessions` uint32 cache lengths; max_length: host
 * upper bound of those lengths (sizes the launch: a session gets one split
 * per ceil(max_length / num_splits) positions, rounded up to 128, so a host
 * that knows the lengths can choose the positions per split with the pair;
 * num_splits 0 = one split per 2048 positions).  q/gate/output/gated_output:
 * [sessions][query_heads][head_dim].  view_table: DEVICE scratch of
 * b200kv_view_table_bytes(sessions) bytes, 128-byte aligned, that this call
 * fills with the views and their TMA descriptors (one blocking copy); pass
 * views == NULL to reuse the table of an earlier call with the same sessions,
 * e.g. on every decode step after the first. */
B200KV_API size_t b200kv_view_table_bytes(uint32_t sessions);
B200KV_API int b200kv_decode_attn_batched(const b200kv_view* views, void* view_table, const uint32_t* lengths,
                               uint32_t sessions, uint32_t max_length, const void* q, int q_dtype,
                               const float* gate, float* output, float* gated_output,
                               uint32_t query_heads, float scale, void* workspace, size_t workspace_bytes,
                               uint32_t num_splits, void* stream);

/* Host-side plan for b200kv_decode_attn_batched: the (num_splits, max_length) pair to pass for sessions of these
 * lengths (HOST array; zero lengths are ignored).  The pair fixes the positions per split,
 * ceil(max_length / num_splits) rounded up to 128, which the launch time depends on by up to 25 %: the plan simulates
 * how the launch's CTAs (one per split, kv head and session, dispatched in block order onto the slot that frees
 * first, each costing its tiles plus a fixed part) pack `cta_slots` slots (0 = 296: two per SM of a B200) and takes
 * the split size with the shortest makespan.  Fitted to timed launches of 10 to 80 sessions of 512 to 16384
 * positions: within 1.5 % of the best measured split size on average, 5 % at worst.  Pure host arithmetic (no
 * launch, no GPU needed), about 1 ms for 80 sessions; meant to run when the set of sessions changes, not per step.
 * No counterpart in the reference. */
B200KV_API int b200kv_plan_batched_decode(const uint32_t* lengths, uint32_t sessions, uint32_t kv_heads, uint32_t cta_slots,
                               uint32_t* num_splits, uint32_t* max_length);

/* Sequence-sharded decode, stage 1 only: online-softmax partials of this
 * shard's positions [range_begin, range_end) reduced over the local splits to
 * ONE (m, l, acc) per query head: part_m/part_l fp32 [query_heads], part_acc
 * fp32 [query_heads][head_dim] (acc unnormalised, relative to m).  The stage-1
 * arithmetic of .hip:7371-7485 restricted to a position range. */
B200KV_API int b200kv_decode_partials(const b200kv_view* view, const void* q, int q_dtype, uint32_t query_heads,
                           float scale, uint32_t range_begin, uint32_t range_end,
                           float* part_m, float* part_l, float* part_acc,
                           void* workspace, size_t workspace_bytes, uint32_t num_splits, void* stream);

/* Log-sum-exp combine of `num_parts` partials laid out [part][query_heads]
 * (m, l) and [part][query_heads][head_dim] (acc).  Replaces
 * qwen3_splitk_stage2_kernel (.hip:2295-2352); with one part per GPU it is the
 * cross-GPU merge of sequence-sharded decode.  Empty parts (l <= 0 or
 * non-finite m) are skipped as in .hip:6681,6701. */
B200KV_API int b200kv_merge_partials(const float* part_m, const float* part_l, const float* part_acc,
                          uint32_t num_parts, uint32_t query_heads, uint32_t head_dim,
                          const float* gate, float* output, float* gated_output, void* stream);

/* The same merge over PACKED partials: part r occupies query_heads*(head_dim+2) consecutive floats laid out
 * [m[query_heads] | l[query_heads] | acc[query_heads][head_dim]].  This is the buffer an all-gather of one
 * packed partial per rank produces, so sequence-sharded decode is three launches per layer:
 * b200kv_decode_partials (with part_m/part_l/part_acc pointing into the rank's packed buffer), the
 * all-gather, and this call.  No counterpart in the reference (single GPU). */
B200KV_API int b200kv_merge_partials_packed(const float* packed, uint32_t num_parts, uint32_t query_heads, uint32_t head_dim,
                                 const float* gate, float* output, float* gated_output, void* stream);

/* Sequence-sharded decode over NCCL from a C or C++ host (no counterpart in the reference): per layer, every rank
 * runs b200kv_decode_partials on its shard with the pointers b200kv_dist_partial hands out, then b200kv_dist_merge
 * all-gathers the packed partials (query_heads * (head_dim + 2) fp32 per rank) on `stream` and merges them; every
 * rank ends with the same output.  For every cache mode and shape; int8 caches at head_dim 128 have the faster
 * in-kernel exchange, b200kv_decode_attn_sharded.  init takes either an existing ncclComm_t (nccl_comm != NULL; rank
 * and world are read from it) or a 128-byte NCCL unique id created by b200kv_dist_unique_id on one rank and passed
 * to the others by the host's own means.  NCCL is looked up at run time (B200KV_ERR_UNSUPPORTED if there is none).
 * These allocate and are collective: set-up calls, not for the per-token path -- except b200kv_dist_merge.
 * b200kv_dist_destroy of a communicator created here blocks until every CUDA graph that captured a
 * b200kv_dist_merge has been destroyed (NCCL's rule): destroy those graphs first. */
typedef struct b200kv_dist b200kv_dist;
B200KV_API int b200kv_dist_unique_id(void* id128);
B200KV_API int b200kv_dist_init(b200kv_dist** out, void* nccl_comm, const void* id128, uint32_t rank, uint32_t world,
                     uint32_t query_heads, uint32_t head_dim);
B200KV_API int b200kv_dist_partial(b200kv_dist* dist, float** part_m, float** part_l, float** part_acc);
B200KV_API int b200kv_dist_merge(b200kv_dist* dist, const float* gate, float* output, float* gated_output, void* stream);
B200KV_API int b200kv_dist_destroy(b200kv_dist* dist);

/* ---- suffix / prefill attention -------------------------------------------- */

/* Minimum workspace of b200kv_prefill_attn: 0 (`workspace` may be NULL; the reference needs 32*T*heads*(2+d)
 * floats of split partials, .hip:7154-7157).  Without a workspace the mma.sync kernel runs, which keeps its
 * running state in registers. */
B200KV_API size_t b200kv_prefill_workspace_bytes(uint32_t token_count, uint32_t query_heads, uint32_t head_dim);
/* Workspace that enables the tcgen05 kernel: room for the fp16 copy of the `rows` cache positions the chunk can see
 * (rows = base_position + token_count; the whole capacity when a device-side prefill_state is used).  35.6 MB for
 * 8704 rows x 4 kv heads x d=256.  The scratch is rewritten by every call; calls that overlap on the GPU need
 * separate workspaces.  Cache rows below `rows` must hold finite values (freshly created caches are zero). */
B200KV_API size_t b200kv_prefill_scratch_bytes(uint64_t rows, uint32_t kv_heads, uint32_t head_dim);
/* Optional extra room behind that scratch (workspace_bytes >= scratch + this): when a chunk has too few query rows
 * to give every SM a row tile (512 tokens x 6 heads per kv head = 96 tiles on 148 SMs), the tcgen05 kernel then also
 * splits the KV range of each tile over up to 8 CTAs, which leave unnormalised partials here for a merge kernel.
 * 50 MB for 512 tokens x 24 heads x d=256.  Without it the launch runs unsplit. */
B200KV_API size_t b200kv_prefill_split_bytes(uint32_t token_count, uint32_t query_heads, uint32_t kv_heads, uint32_t head_dim);

/* Replaces launch_qwen35_splitk_suffix_attention_quant
 * (qwen3_gpu_primitives.hpp:670-692; kernels .hip:6788-7119 and 6637-6725).
 * q, gate, gated_output: [token][query_heads][head_dim] (q of q_dtype, the
 * others fp32; gate may be NULL).  Query token t attends cache positions
 * [0, base_position + t + 1): the chunk must already have been appended.  A
 * non-NULL prefill_state overrides base_position/token_count on the device
 * (.hip:6810-6814).  Tokens whose causal length exceeds the capacity get a
 * zero row (the reference leaves them unwritten, .hip:6830). */
B200KV_API int b200kv_prefill_attn(const b200kv_view* view, const void* q, int q_dtype, const float* gate,
                        float* gated_output, uint32_t token_count, uint32_t base_position,
                        uint32_t query_heads, float scale, const b200kv_prefill_state* prefill_state,
                        void* workspace, size_t workspace_bytes, void* stream);

/* The tcgen05 kernel's pre-pass ahead of time: converts cache positions [0, prepared_rows) to fp16 into `workspace`,
 * laid out for a chunk that sees `rows` positions (rows = base_position + token_count of the attention call that
 * follows; the capacity when that call uses a device-side prefill_state).  b200kv_prefill_attn_prepared is
 * b200kv_prefill_attn for a workspace that holds those rows already: its own pre-pass then converts only
 * [prepared_rows, rows) -- normally the chunk just appended.  The prefix of a layer does not depend on the chunk, so
 * a host can run the prepare call of layer l + 1 on a second stream beside the attention of layer l (two workspaces in
 * turn; order the calls with events: the prepare call after the attention that last used its workspace, the attention
 * after its prepare call).  Positions below prepared_rows must not change between the two calls.  No counterpart in the
 * reference.  B200KV_ERR_WORKSPACE when the workspace is too small for `rows`. */
B200KV_API int b200kv_prefill_prepare(const b200kv_view* view, uint32_t prepared_rows, uint64_t rows, void* workspace,
                           size_t workspace_bytes, void* stream);
B200KV_API int b200kv_prefill_attn_prepared(const b200kv_view* view, const void* q, int q_dtype, const float* gate,
                                 float* gated_output, uint32_t token_count, uint32_t base_position,
                                 uint32_t query_heads, float scale, const b200kv_prefill_state* prefill_state,
                                 void* workspace, size_t workspace_bytes, uint32_t prepared_rows, void* stream);

/* ---- prefix snapshot / restore ---------------------------------------------
 * Raw compact layout of AttentionLayerKvCacheStorage::download_raw/upload_raw
 * (src/prefill_v2/kv_cache.cpp:214-369): K first -- per kv head the int8 slice
 * of `tokens` rows followed by its scale slice (or the fp16 slice) -- then V the
 * same way; capacity-strided rows are compacted to `tokens`. */
B200KV_API size_t b200kv_snapshot_bytes(const b200kv_view* view, uint64_t tokens);
/* dst/src may be device memory or (pinned or pageable) host memory; the copies
 * are issued on `stream` and, like the reference with a non-null stream
 * (src/prefill_v2/persistent_session.cpp:112-114), NOT synchronised. */
B200KV_API int b200kv_snapshot_save(const b200kv_view* view, uint64_t tokens, void* dst, void* stream);
B200KV_API int b200kv_snapshot_restore(const b200kv_view* view, uint64_t tokens, const void* src, void* stream);
/* Device-to-device copy of the first `tokens` positions of src into dst (both
 * caches of one geometry; capacities may differ): one kernel launch.  The
 * in-VRAM counterpart of copy_session_checkpoint/restore_session_checkpoint,
 * tools/miinfer_cli.cpp:1248-1317. */
B200KV_API int b200kv_snapshot_clone(const b200kv_view* dst, const b200kv_view* src, uint64_t tokens, void* stream);

/* download_key / download_value, src/prefill_v2/kv_cache.cpp:132-212: the first `tokens` positions of one side as
 * fp32 [kv_head][tokens][head_dim] in HOST memory, dequantised (int8 value x the fp16 scale of its block; fp16 values
 * widened).  Blocking; for inspection and tests, not the per-token path.  tokens > capacity -> B200KV_ERR_RANGE
 * (the reference throws). */
B200KV_API int b200kv_download_key(const b200kv_view* view, uint64_t tokens, float* host_dst, void* stream);
B200KV_API int b200kv_download_value(const b200kv_view* view, uint64_t tokens, float* host_dst, void* stream);

/* ---- prefix identity and the on-disk session (host side) -------------------- */

/* 64-bit FNV-1a-style hash, one xor+multiply round per token id (not per byte):
 * compute_token_sequence_hash, include/miinfer/prefill_v2/reusable_context.hpp:38-45. */
B200KV_API uint64_t b200kv_token_sequence_hash(const uint32_t* tokens, size_t count);

/* ReusableContext::MatchResult, include/miinfer/prefill_v2/reusable_context.hpp:97-105 (same seven outcomes, same order). */
typedef enum b200kv_match {
    B200KV_MATCH_EXACT = 0,
    B200KV_MATCH_PREFIX_MISMATCH = 1,
    B200KV_MATCH_MODEL_MISMATCH = 2,
    B200KV_MATCH_QUANTIZATION_MISMATCH = 3,
    B200KV_MATCH_EMPTY_CACHE = 4,
    B200KV_MATCH_PROMPT_SHORTER = 5,
    B200KV_MATCH_VERSION_MISMATCH = 6
} b200kv_match;

/* ReusableContext::check_match, src/prefill_v2/reusable_context.cpp:155-185: can the cached prefix (its model id,
 * quantization id, state layout version -- 20260925 is the current one -- and tokens) be reused for `prompt`?
 * Returns a b200kv_match.  Host only. */
B200KV_API int b200kv_prefix_match(const char* cached_model_id, const char* cached_quantization, uint32_t cached_layout_version,
                        const uint32_t* cached_tokens, uint32_t cached_length, const char* model_id, const char* quantization,
                        const uint32_t* prompt, uint32_t prompt_length);

/* PersistentSessionHeader, include/miinfer/prefill_v2/persistent_session.hpp:19-33: same packed 157 bytes. */
#pragma pack(push, 1)
typedef struct b200kv_session_header {
    char magic[4];              /* "MISS" */
    uint32_t version;           /* 20260928 */
    char model_id[64];
    char quantization[32];
    uint32_t prefix_length;
    uint64_t token_hash;
    uint32_t gdn_layers;        /* 0 here: recurrent layers are outside this path */
    uint64_t gdn_state_bytes;   /* 0 */
    uint32_t gqa_layers;
    uint8_t kv_quant_mode;
    uint64_t kv_bytes;
    uint64_t tokens_bytes;
    uint64_t created_timestamp;
} b200kv_session_header;
#pragma pack(pop)

/* PersistentSession::format_session_filename, persistent_session.cpp:27-32: "sess_<hash:016x>_p<length>.miinfer". */
B200KV_API int b200kv_session_filename(uint64_t token_hash, uint32_t prefix_length, char* out, size_t out_bytes);
/* save_to_file, persistent_session.cpp:34-142: snapshot the first `prefix_length` positions of every layer and write
 * header | tokens | KV | trailer atomically (tmp file + rename).  Synchronises `stream`. */
B200KV_API int b200kv_session_save(const char* path, const char* model_id, const char* quantization, const uint32_t* tokens,
                        uint32_t prefix_length, const b200kv_view* layer_views, uint32_t layers, void* stream);
/* inspect_file, persistent_session.cpp:144-166: header (and tokens, if tokens_out != NULL) without touching a GPU. */
B200KV_API int b200kv_session_inspect(const char* path, b200kv_session_header* header, uint32_t* tokens_out, uint32_t tokens_capacity);
/* load_from_file, persistent_session.cpp:168-267: validates magic, version, model, quantization, layer count, token
 * hash -- and, beyond the reference, the KV quant mode, geometry and a payload checksum -- then restores every layer.
 * B200KV_ERR_FORMAT = damaged file, B200KV_ERR_MISMATCH = a valid file for something else. */
B200KV_API int b200kv_session_load(const char* path, const char* model_id, const char* quantization, const b200kv_view* layer_views,
                        uint32_t layers, uint32_t* tokens_out, uint32_t tokens_capacity, uint32_t* prefix_length_out, void* stream);
/* find_matching_session, persistent_session.cpp:269-320: the file in `session_dir` with the longest prefix of `prompt`. */
B200KV_API int b200kv_session_find(const char* session_dir, const char* model_id, const char* quantization, const uint32_t* prompt,
                        uint32_t prompt_length, char* path_out, size_t path_bytes, uint32_t* prefix_length_out);
/* The file format without a GPU: write/read with the KV payload in host memory (what save/load do around the
 * device copies).  layer_bytes = b200kv_snapshot_bytes of one layer. */
B200KV_API int b200kv_session_write(const char* path, const char* model_id, const char* quantization, const uint32_t* tokens,
                         uint32_t prefix_length, const void* kv_payload, uint64_t layer_bytes, uint32_t layers,
                         uint32_t kv_heads, uint32_t head_dim, uint32_t qblock, uint32_t quant_mode);
B200KV_API int b200kv_session_read(const char* path, const char* model_id, const char* quantization, uint32_t layers, uint32_t kv_heads,
                        uint32_t head_dim, uint32_t qblock, uint32_t quant_mode, uint32_t* tokens_out, uint32_t tokens_capacity,
                        uint32_t* prefix_length_out, void* kv_payload_out, uint64_t payload_capacity);

/* ---- in-VRAM snapshot pool and the prefix-reuse policy (host side; these allocate: not for the per-token path) ---- */

/* A store of prefix snapshots in device memory with longest-prefix lookup: the multi-snapshot machinery of the
 * reference's first engine, tools/miinfer_cli.cpp:1043-1317 (SessionCheckpoint, a compressed radix tree over the
 * token ids, least-recently-used eviction) for the KV part.  max_entries 0 = 8 and max_bytes 0 = 3 GiB, the
 * reference's budget (tools/miinfer_cli.cpp:62-63); granularity = only prefixes whose length is a multiple of it
 * are captured (the reference: 512, the prefill tile, :1185; 0 or 1 = any length).  model_id / quantization
 * identify what the snapshots belong to: lookups for another identity find nothing (:1073-1079). */
typedef struct b200kv_pool b200kv_pool;
typedef struct b200kv_pool_counters {
    uint32_t entries;
    uint64_t bytes;
    uint64_t hits, misses, captures, evictions, skipped;
} b200kv_pool_counters;
B200KV_API int b200kv_pool_create(b200kv_pool** out, const char* model_id, const char* quantization, uint32_t max_entries,
                       uint64_t max_bytes, uint32_t granularity);
B200KV_API int b200kv_pool_destroy(b200kv_pool* pool);
/* capture_session_checkpoint (:1184-1228): keep the first prefix_length positions of every layer under `tokens`
 * (device-to-device, on `stream`); an entry with the same tokens is refreshed; the oldest entries are evicted to stay
 * within the budget.  *captured (may be NULL) = 0 when the capture was skipped (granularity, larger than the whole
 * budget, or no device memory left), which is not an error. */
B200KV_API int b200kv_pool_capture(b200kv_pool* pool, const uint32_t* tokens, uint32_t prefix_length, const b200kv_view* layer_views,
                        uint32_t layers, void* stream, int* captured);
/* The same bookkeeping without a payload, for a host that keeps the snapshot bytes elsewhere: `bytes` is what the
 * entry counts against the budget. */
B200KV_API int b200kv_pool_capture_index_only(b200kv_pool* pool, const uint32_t* tokens, uint32_t prefix_length, uint64_t bytes, int* captured);
/* longest_session_checkpoint (:1126-1148): length of the longest stored sequence that is a prefix of `prompt` and
 * strictly shorter than it (0 = none); *common_length (may be NULL) = how many leading prompt tokens the index shares
 * with any stored sequence.  A hit marks the entry as used. */
B200KV_API int b200kv_pool_lookup(b200kv_pool* pool, const char* model_id, const char* quantization, const uint32_t* prompt,
                       uint32_t prompt_length, uint32_t* matched_length, uint32_t* common_length);
/* restore_session_checkpoint (:1290-1317): look up as above and copy the entry's positions into the caches. */
B200KV_API int b200kv_pool_restore(b200kv_pool* pool, const uint32_t* prompt, uint32_t prompt_length, const b200kv_view* layer_views,
                        uint32_t layers, void* stream, uint32_t* matched_length);
B200KV_API int b200kv_pool_stats(b200kv_pool* pool, b200kv_pool_counters* out);

/* The prefix-reuse fields of GenerateOptions and the reuse telemetry of GenerateStats,
 * include/miinfer/prefill_v2/model.hpp:27-68. */
typedef struct b200kv_reuse_options {
    int enable_prefix_reuse;
    int cache_prefix_after;
    uint32_t cache_prefix_len;           /* 0 = the whole prompt */
    const char* persistent_session_dir;  /* NULL or "" = no files */
} b200kv_reuse_options;
typedef enum b200kv_reuse_source { B200KV_REUSE_NONE = 0, B200KV_REUSE_RESIDENT = 1, B200KV_REUSE_POOL = 2, B200KV_REUSE_DISK = 3 } b200kv_reuse_source;
typedef struct b200kv_reuse_stats {
    int reuse_hit;
    int source;                          /* b200kv_reuse_source */
    uint32_t prefix_tokens_reused;
    uint32_t suffix_tokens_dispatched;
    uint32_t gqa_kv_reused_tokens;
    double restore_ms;
} b200kv_reuse_stats;
/* The reuse branch at the start of PrefillV2Model::generate (src/prefill_v2/model.cpp:751-775): decide how much of
 * `prompt` need not be prefilled and bring that prefix into the caches.  Tried in this order: the prefix already
 * resident in the caches (resident_* describe it; an exact match strictly shorter than the prompt; nothing is
 * copied), the pool (may be NULL; no counterpart in that function), the session directory.  With layers == 0 only the
 * decision is taken (no device work).  The caller prefills prompt[stats->prefix_tokens_reused:]. */
B200KV_API int b200kv_reuse_begin(const b200kv_reuse_options* options, const char* model_id, const char* quantization,
                       const char* resident_model_id, const char* resident_quantization, uint32_t resident_layout_version,
                       const uint32_t* resident_tokens, uint32_t resident_length, b200kv_pool* pool, const uint32_t* prompt,
                       uint32_t prompt_length, const b200kv_view* layer_views, uint32_t layers, void* stream, b200kv_reuse_stats* stats);
/* The step after prefill (model.cpp:868-887): with cache_prefix_after, *cached_length = the prefix the caller now
 * treats as resident (cache_prefix_len, or the whole prompt); it is captured into the pool (if any) and, when a
 * session directory is set and the prefix has at least 256 tokens and no file yet, saved there (a failed write is
 * not an error; *wrote_file says whether one was written). */
B200KV_API int b200kv_reuse_commit(const b200kv_reuse_options* options, const char* model_id, const char* quantization, b200kv_pool* pool,
                        const uint32_t* prompt, uint32_t prompt_length, const b200kv_view* layer_views, uint32_t layers, void* stream,
                        uint32_t* cached_length, int* wrote_file);

#ifdef __cplusplus
}
#endif
#endif /* B200KV_H */
