// Split-K GQA decode attention: entry points, the log-sum-exp merge kernel and
// the generic stage-1 kernel that covers every cache mode (fp16 or int8 K/V,
// block or row scales).  The specialised int8 streaming kernel lives in
// decode_q8.cu and is preferred whenever it supports the geometry.
//
// Stage-1 arithmetic follows MIInfer's decode kernel
// (gfx906/kernels/qwen3_primitives.hip:7371-7485) with the per-row scale
// generalised to per-block scales; the merge follows its stage 2
// (.hip:2295-2352).  Unlike the reference the partials live in a caller-owned
// workspace, not in file-scope device arrays (.hip:2111-2113), so launches on
// different streams do not interfere.
#include "decode_common.cuh"

#include <cmath>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace b200kv {

// ---------------------------------------------------------------------------
// Generic stage 1: one warp per (query head, split, session); lane L owns the
// D/32 consecutive dims starting at L*D/32.
// ---------------------------------------------------------------------------
template <int D, bool K_Q8, bool V_Q8>
__global__ void __launch_bounds__(32) decode_generic_kernel(const __grid_constant__ DecodeParams p) {
    constexpr int E = D / 32;
    const uint32_t head = blockIdx.x, split = blockIdx.y, session = blockIdx.z;
    const int lane = threadIdx.x;
    const b200kv_view& view = session_view(p, session);
    uint32_t begin, end;
    resolve_range(p, session, view, &begin, &end);
    const uint32_t per = (end - begin + p.num_splits - 1) / p.num_splits;
    const uint32_t pos0 = begin + split * per;
    const uint32_t pos1 = min(pos0 + per, end);
    const uint32_t kv_head = head / (p.query_heads / view.kv_heads);
    const uint32_t nblk = D / view.qblock;
    const uint32_t blk = (nblk == 1) ? 0u : static_cast<uint32_t>(lane * E) / 32u;

    float q[E];
    const size_t q_base = (static_cast<size_t>(session) * p.query_heads + head) * D + lane * E;
#pragma unroll
    for (int i = 0; i < E; ++i)
        q[i] = p.q_is_f16 ? __half2float(static_cast<const __half*>(p.q)[q_base + i])
                          : static_cast<const float*>(p.q)[q_base + i];

    float acc[E];
#pragma unroll
    for (int i = 0; i < E; ++i) acc[i] = 0.0f;
    float m = -INFINITY, l = 0.0f;

    const size_t head_row0 = static_cast<size_t>(kv_head) * view.capacity;
    for (uint32_t pos = pos0; pos < pos1; ++pos) {
        const size_t row = head_row0 + pos;
        float kf[E], vf[E];
        float ks = 1.0f, vs = 1.0f;
        if (K_Q8) {
            const int8_t* src = view.key_q8 + row * D + lane * E;
#pragma unroll
            for (int w = 0; w < E / 4; ++w) {
                const uint32_t raw = reinterpret_cast<const uint32_t*>(src)[w];
#pragma unroll
                for (int b = 0; b < 4; ++b) kf[w * 4 + b] = static_cast<float>(static_cast<int8_t>(raw >> (8 * b)));
            }
            ks = __half2float(static_cast<const __half*>(view.key_scales)[row * nblk + blk]);
        } else {
            const __half* src = static_cast<const __half*>(view.key_f16) + row * D + lane * E;
#pragma unroll
            for (int i = 0; i < E; ++i) kf[i] = __half2float(src[i]);
        }
        float prod = 0.0f;
#pragma unroll
        for (int i = 0; i < E; ++i) prod = fmaf(q[i], kf[i], prod);
        const float dot = warp_sum(prod * ks) * p.scale;

        const float m_new = fmaxf(m, dot);
        const float alpha = __expf(m - m_new);  // m == -inf on the first position: exp(-inf) = 0
        const float weight = __expf(dot - m_new);
        l = l * alpha + weight;
        m = m_new;

        if (V_Q8) {
            const int8_t* src = view.value_q8 + row * D + lane * E;
#pragma unroll
            for (int w = 0; w < E / 4; ++w) {
                const uint32_t raw = reinterpret_cast<const uint32_t*>(src)[w];
#pragma unroll
                for (int b = 0; b < 4; ++b) vf[w * 4 + b] = static_cast<float>(static_cast<int8_t>(raw >> (8 * b)));
            }
            vs = __half2float(static_cast<const __half*>(view.value_scales)[row * nblk + blk]);
        } else {
            const __half* src = static_cast<const __half*>(view.value_f16) + row * D + lane * E;
#pragma unroll
            for (int i = 0; i < E; ++i) vf[i] = __half2float(src[i]);
        }
        const float ew = weight * vs;
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] = fmaf(acc[i], alpha, ew * vf[i]);
    }

    const size_t slot = (static_cast<size_t>(session) * p.num_splits + split) * p.query_heads + head;
#pragma unroll
    for (int i = 0; i < E; ++i) p.ws_acc[slot * D + lane * E + i] = acc[i];
    if (lane == 0) {
        p.ws_m[slot] = m;
        p.ws_l[slot] = l;
    }
}

// ---------------------------------------------------------------------------
// Merge (stage 2): one block per (head, group), one thread per dim.  The (m, l)
// of all parts are staged in shared memory first so the accumulation is a run
// of independent loads.  A part with l <= 0 or m == -inf is empty and skipped
// (gfx906/kernels/qwen3_primitives.hip:6681,6701); a NaN part propagates.
// ---------------------------------------------------------------------------
__global__ void merge_kernel(const __grid_constant__ MergeParams p) {
    extern __shared__ float sh[];   // a[num_parts], then gmax, gsum
    // the next kernel of the stream (the next layer's stage 1) may become resident; this one waits for its partials
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t head = blockIdx.x, group = blockIdx.y, dim = threadIdx.x;
    const uint32_t H = p.query_heads, D = p.head_dim, S = p.num_parts;
    const size_t base = static_cast<size_t>(group) * S * H + head;
    const size_t ml_stride = p.part_stride ? p.part_stride : H;   // packed parts (one buffer per rank) or dense arrays
    float* sa = sh;
    float* sl = sh + S;
    for (uint32_t s = dim; s < S; s += blockDim.x) {
        sa[s] = p.part_m[base + static_cast<size_t>(s) * ml_stride];
        sl[s] = p.part_l[base + static_cast<size_t>(s) * ml_stride];
    }
    __syncthreads();
    if (dim < 32) {
        float gmax = -INFINITY;
        for (uint32_t s = dim; s < S; s += 32)
            if (!(sl[s] <= 0.0f) && sa[s] != -INFINITY) gmax = fmaxf(gmax, sa[s]);
        gmax = warp_max(gmax);
        float gsum = 0.0f;
        for (uint32_t s = dim; s < S; s += 32) {
            const float a = (!(sl[s] <= 0.0f) && sa[s] != -INFINITY) ? __expf(sa[s] - gmax) : 0.0f;
            gsum = fmaf(sl[s], a, gsum);
            sa[s] = a;
        }
        gsum = warp_sum(gsum);
        if (dim == 0) { sh[2 * S] = gmax; sh[2 * S + 1] = gsum; }
    }
    __syncthreads();
    const float gmax = sh[2 * S], gsum = sh[2 * S + 1];
    const float* accp = p.part_acc + base * D + dim;
    const size_t stride = p.part_stride ? p.part_stride : static_cast<size_t>(H) * D;
    // four running sums (part s goes to sum s % 4, a tail of S % 4 parts to sum 0); the loads are issued sixteen at a time so
    // that a launch with a few dozen parts needs two or three trips to L2, not one per four parts
    float t[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const uint32_t S4 = S & ~3u;
    for (uint32_t s0 = 0; s0 < S; s0 += 16) {
        float a[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) a[i] = (s0 + i < S) ? accp[(s0 + i) * stride] : 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t s = s0 + i;
            if (s < S4) t[i & 3] = fmaf(a[i], sa[s], t[i & 3]);
            else if (s < S) t[0] = fmaf(a[i], sa[s], t[0]);
        }
    }
    const float total = (t[0] + t[1]) + (t[2] + t[3]);
    const size_t out_idx = (static_cast<size_t>(group) * H + head) * D + dim;
    if (p.out_m != nullptr) {
        p.out_acc[out_idx] = total;
        if (dim == 0) {
            p.out_m[static_cast<size_t>(group) * H + head] = gmax;
            p.out_l[static_cast<size_t>(group) * H + head] = gsum;
        }
        return;
    }
    const float o = gsum > 0.0f ? total / gsum : (gsum == gsum ? 0.0f : gsum);
    if (p.output != nullptr) p.output[out_idx] = o;
    if (p.gated_output != nullptr || p.gated_output_q8 != nullptr) {
        float g = o;
        if (p.gate != nullptr) g = o * (1.0f / (1.0f + __expf(-p.gate[out_idx])));
        if (p.gated_output != nullptr) p.gated_output[out_idx] = g;
        if (p.gated_output_q8 != nullptr) {
            // Q8_1 block of 32 consecutive dims = one warp (gfx906/kernels/qwen3_primitives.hip:2354-2383);
            // IEEE operations so that a host restatement reproduces the bits
            const float amax = warp_max(fabsf(g));
            const float dq = __fdiv_rn(amax, 127.0f);
            const float id = dq != 0.0f ? __fdiv_rn(1.0f, dq) : 0.0f;
            const int q = max(-127, min(127, static_cast<int>(roundf(__fmul_rn(g, id)))));
            int qs = q;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) qs += __shfl_xor_sync(0xffffffffu, qs, off);
            b200kv_q8_1_block* dst = p.gated_output_q8 + out_idx / 32;
            dst->qs[dim & 31] = static_cast<int8_t>(q);
            if ((dim & 31) == 0) {
                const __half dh = __float2half_rn(dq), sh = __float2half_rn(__fmul_rn(static_cast<float>(qs), dq));
                dst->d = *reinterpret_cast<const uint16_t*>(&dh);
                dst->s = *reinterpret_cast<const uint16_t*>(&sh);
            }
        }
    }
}

int launch_merge(const MergeParams& p, uint32_t groups, cudaStream_t stream) {
    if (p.num_parts > 4096) return B200KV_ERR_UNSUPPORTED;
    B200KV_CUDA_TRY(launch_kernel(merge_kernel, dim3(p.query_heads, groups), dim3(p.head_dim), (2 * p.num_parts + 2) * sizeof(float), stream, true, p));
    return B200KV_OK;
}

static uint32_t pick_splits_generic(uint32_t query_heads, uint32_t sessions, uint32_t max_length) {
    // one warp per (head, split, session): aim at ~16 warps per SM on 148 SMs
    uint32_t want = (148u * 16u + query_heads * sessions - 1) / (query_heads * sessions);
    uint32_t by_length = (max_length + 63) / 64;  // at least 64 positions per split
    uint32_t s = want < by_length ? want : by_length;
    const uint32_t cap = max_splits_per_session(sessions);
    if (s > cap) s = cap;
    return s ? s : 1;
}

template <int D>
static void launch_generic(const DecodeParams& p, uint32_t mode, dim3 grid, cudaStream_t s) {
    switch (mode) {
        case B200KV_F16_F16: decode_generic_kernel<D, false, false><<<grid, 32, 0, s>>>(p); break;
        case B200KV_Q8_F16: decode_generic_kernel<D, true, false><<<grid, 32, 0, s>>>(p); break;
        case B200KV_F16_Q8: decode_generic_kernel<D, false, true><<<grid, 32, 0, s>>>(p); break;
        default: decode_generic_kernel<D, true, true><<<grid, 32, 0, s>>>(p); break;
    }
}

// Runs stage 1 (streaming kernel if available, else generic) into the workspace.
// Workspace layout: [tagged partials of the streaming kernel (zero between launches)] [m] [l] [acc].
int run_decode_stage1(DecodeParams& p, const b200kv_view& geometry, uint32_t max_length, void* workspace,
                      size_t workspace_bytes, uint32_t num_splits_arg, const MergeParams& merge, bool* merged,
                      cudaStream_t stream) {
    *merged = false;
    const bool force_generic = (num_splits_arg & B200KV_SPLITS_FORCE_GENERIC) != 0;
    uint32_t num_splits = num_splits_arg & ~B200KV_SPLITS_FORCE_GENERIC;
    const uint32_t cap = max_splits_per_session(p.sessions);
    bool use_fast = !force_generic && q8_fast_path_ok(geometry, p.query_heads);
    // head_dim 256: a tcgen05 stage 1 for single-session launches (it leaves plain partials, like the generic kernel)
    const bool use_wide = !force_generic && !use_fast && p.views == nullptr && p.lengths == nullptr && !p.causal && p.sessions == 1 &&
                          p.new_key == nullptr && streaming_kernel_choice() != 1 && decode_tc5_wide_ok(geometry, p.query_heads);
    if (num_splits == 0) {
        uint32_t fast = use_fast ? pick_splits_q8(geometry, p.query_heads, p.sessions, max_length) : 0;
        if (fast == 0) use_fast = false;
        num_splits = use_fast ? fast : (use_wide ? pick_splits_tc5_wide(geometry, max_length) : pick_splits_generic(p.query_heads, p.sessions, max_length));
    }
    if (num_splits > cap) num_splits = cap;
    const size_t slots = static_cast<size_t>(p.sessions) * num_splits * p.query_heads;
    const size_t plain_bytes = slots * (geometry.head_dim + 2u) * sizeof(float);
    if (workspace == nullptr) return B200KV_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return B200KV_ERR_INVALID;
    const size_t plain_offset = workspace_plain_offset(workspace_bytes);
    if (workspace_bytes - plain_offset < plain_bytes) return B200KV_ERR_WORKSPACE;
    p.num_splits = num_splits;
    p.ws_m = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + plain_offset);
    p.ws_l = p.ws_m + slots;
    p.ws_acc = p.ws_l + slots;
    p.status = current_status_word();
    p.timeline = current_timeline_buffer(num_splits * geometry.kv_heads);
    if (use_fast) {
        if (plain_offset < 2 * plain_bytes) return B200KV_ERR_WORKSPACE;
        // The in-launch merge; a lone split that has to produce Q8_1 blocks goes through the merge kernel instead
        // (a block of 32 outputs is quantised by 16 cooperating threads, which the single-split shortcut has not).
        const bool fuse_merge = !(num_splits == 1 && merge.gated_output_q8 != nullptr && merge.xchg.world <= 1);
        p.ws_tagged = fuse_merge ? static_cast<uint64_t*>(workspace) : nullptr;
        p.tag = next_launch_tag();
        p.fuse = merge;
        int rc = B200KV_ERR_UNSUPPORTED;
        if (streaming_kernel_choice() != 1) rc = launch_decode_tc5(p, geometry, max_length, stream);
        if (rc == B200KV_ERR_UNSUPPORTED) rc = launch_decode_q8(p, geometry, max_length, stream);
        if (rc == B200KV_OK) *merged = fuse_merge;
        if (rc != B200KV_ERR_UNSUPPORTED) return rc;
        p.ws_tagged = nullptr;
    }
    if (use_wide) {
        const int rc = launch_decode_tc5_wide(p, geometry, stream);
        if (rc != B200KV_ERR_UNSUPPORTED) return rc;
    }
    dim3 grid(p.query_heads, num_splits, p.sessions);
    if (geometry.head_dim == 128) launch_generic<128>(p, geometry.quant_mode, grid, stream);
    else launch_generic<256>(p, geometry.quant_mode, grid, stream);
    B200KV_CUDA_TRY(cudaGetLastError());
    return B200KV_OK;
}

// Stage 1 followed (unless the kernel merged by itself) by the merge kernel.
int run_decode(DecodeParams& p, const b200kv_view& geometry, uint32_t max_length, void* workspace, size_t workspace_bytes,
               uint32_t num_splits_arg, MergeParams mp, uint32_t groups, cudaStream_t stream) {
    bool merged = false;
    int rc = run_decode_stage1(p, geometry, max_length, workspace, workspace_bytes, num_splits_arg, mp, &merged, stream);
    if (rc != B200KV_OK || merged) return rc;
    mp.part_m = p.ws_m;
    mp.part_l = p.ws_l;
    mp.part_acc = p.ws_acc;
    mp.num_parts = p.num_splits;
    return launch_merge(mp, groups, stream);
}

// What b200kv_decode_attn_batched staged into a device view table, kept on the host so that later calls with
// views == NULL need no device-to-host copy (which would stall the stream once per layer and step).
struct TableRecord { b200kv_view geometry; bool fast; uint32_t sessions; };
static std::mutex g_tables_mutex;
static std::unordered_map<uint64_t, TableRecord> g_tables;   // keyed by (device, address): addresses repeat across devices

static uint64_t table_key(const void* table) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) (void)cudaGetLastError();
    // device pointers use at most 57 bits; the ordinal goes on top
    return (static_cast<uint64_t>(device & 0x7f) << 57) ^ static_cast<uint64_t>(reinterpret_cast<uintptr_t>(table));
}

static void remember_table(const void* table, const b200kv_view& geometry, bool fast, uint32_t sessions) {
    std::lock_guard<std::mutex> lock(g_tables_mutex);
    if (g_tables.size() > 4096) g_tables.clear();   // tables come and go with their sessions; forgetting only costs a fetch
    g_tables[table_key(table)] = TableRecord{geometry, fast, sessions};
}

static bool recall_table(const void* table, uint32_t sessions, b200kv_view* geometry, bool* fast) {
    std::lock_guard<std::mutex> lock(g_tables_mutex);
    const auto it = g_tables.find(table_key(table));
    if (it == g_tables.end() || it->second.sessions != sessions) return false;
    *geometry = it->second.geometry;
    *fast = it->second.fast;
    return true;
}

static int check_heads(const b200kv_view* view, uint32_t query_heads, float scale) {
    if (query_heads == 0 || query_heads % view->kv_heads != 0 || !std::isfinite(scale)) return B200KV_ERR_INVALID;
    if (query_heads / view->kv_heads > 8) return B200KV_ERR_UNSUPPORTED;
    return B200KV_OK;
}

}  // namespace b200kv

using namespace b200kv;

extern "C" {

int b200kv_decode_kernel_kind(const b200kv_view* view, uint32_t query_heads) {
    if (validate_view(view) != B200KV_OK) return 0;
    if (q8_fast_path_ok(*view, query_heads)) return 1;
    return decode_tc5_wide_ok(*view, query_heads) ? 2 : 0;
}

size_t b200kv_view_table_bytes(uint32_t sessions) { return sizeof(SessionEntry) * static_cast<size_t>(sessions ? sessions : 1); }

size_t b200kv_decode_workspace_bytes(uint32_t query_heads, uint32_t head_dim, uint32_t sessions) {
    if (sessions == 0) sessions = 1;
    const size_t slots = static_cast<size_t>(sessions) * max_splits_per_session(sessions) * query_heads;
    // plain partials behind, twice that for the tagged partials of the streaming kernels in front
    return (slots * (head_dim + 2u) * sizeof(float) + 255) / 256 * 256 * 3;
}

int b200kv_decode_attn(const b200kv_view* view, const void* q, int q_dtype, const float* gate,
                       float* output, float* gated_output, b200kv_q8_1_block* gated_output_q8, uint32_t query_heads, float scale,
                       uint32_t cache_length, const b200kv_decode_state* decode_state,
                       void* workspace, size_t workspace_bytes, uint32_t num_splits, void* stream) {
    int rc = validate_view(view);
    if (rc != B200KV_OK) return rc;
    // at least one output, as the reference launcher demands (gfx906/kernels/qwen3_primitives.hip:7509-7512)
    if (q == nullptr || (output == nullptr && gated_output == nullptr && gated_output_q8 == nullptr)) return B200KV_ERR_INVALID;
    if (q_dtype != B200KV_F16 && q_dtype != B200KV_F32) return B200KV_ERR_INVALID;
    if ((rc = check_heads(view, query_heads, scale)) != B200KV_OK) return rc;
    if (decode_state == nullptr && cache_length > view->capacity) return B200KV_ERR_RANGE;
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    DecodeParams p{};
    p.view = *view;
    p.decode_state = decode_state;
    p.cache_length = cache_length;
    p.sessions = 1;
    p.q = q;
    p.q_is_f16 = (q_dtype == B200KV_F16);
    p.query_heads = query_heads;
    p.scale = scale;
    // with a device-side length the launch is sized for the whole cache
    const uint32_t max_length = decode_state ? static_cast<uint32_t>(view->capacity) : cache_length;
    MergeParams mp{};
    mp.query_heads = query_heads;
    mp.head_dim = view->head_dim;
    mp.gate = gate;
    mp.output = output;
    mp.gated_output = gated_output;
    mp.gated_output_q8 = gated_output_q8;
    return run_decode(p, *view, max_length, workspace, workspace_bytes, num_splits, mp, 1, s);
}

int b200kv_decode_step(const b200kv_view* view, const void* key, const void* value, int kv_dtype,
                       const float* k_norm_weight, int rope_mode, float theta, float epsilon,
                       const void* q, int q_dtype, const float* gate, float* output, float* gated_output,
                       b200kv_q8_1_block* gated_output_q8, uint32_t query_heads, float scale, uint32_t position,
                       const b200kv_decode_state* decode_state, void* workspace, size_t workspace_bytes, uint32_t num_splits, void* stream) {
    int rc = validate_view(view);
    if (rc != B200KV_OK) return rc;
    if (key == nullptr || value == nullptr || q == nullptr || (output == nullptr && gated_output == nullptr && gated_output_q8 == nullptr))
        return B200KV_ERR_INVALID;
    if ((kv_dtype != B200KV_F16 && kv_dtype != B200KV_F32) || (q_dtype != B200KV_F16 && q_dtype != B200KV_F32)) return B200KV_ERR_INVALID;
    if (rope_mode < B200KV_ROPE_NONE || rope_mode > B200KV_ROPE_SECTIONED64) return B200KV_ERR_INVALID;
    if (!std::isfinite(theta) || !std::isfinite(epsilon) || (rope_mode != B200KV_ROPE_NONE && !(theta > 0.0f))) return B200KV_ERR_INVALID;
    if ((rc = check_heads(view, query_heads, scale)) != B200KV_OK) return rc;
    if (decode_state == nullptr && position >= view->capacity) return B200KV_ERR_RANGE;
    const bool force_generic = (num_splits & B200KV_SPLITS_FORCE_GENERIC) != 0;
    if (force_generic || !q8_fast_path_ok(*view, query_heads)) {
        // no fused kernel for this cache: the two launches the fused one stands for
        rc = b200kv_append(view, key, value, kv_dtype, k_norm_weight, rope_mode, theta, epsilon, 1, position, nullptr, decode_state, stream);
        if (rc != B200KV_OK) return rc;
        return b200kv_decode_attn(view, q, q_dtype, gate, output, gated_output, gated_output_q8, query_heads, scale, position + 1,
                                  decode_state, workspace, workspace_bytes, num_splits, stream);
    }
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DecodeParams p{};
    p.view = *view;
    p.decode_state = decode_state;
    p.cache_length = position + 1;
    p.sessions = 1;
    p.q = q;
    p.q_is_f16 = (q_dtype == B200KV_F16);
    p.query_heads = query_heads;
    p.scale = scale;
    p.new_key = key;
    p.new_value = value;
    p.new_is_f16 = (kv_dtype == B200KV_F16);
    p.k_norm_weight = k_norm_weight;
    p.rope_mode = rope_mode;
    p.epsilon = epsilon;
    rope_constants(rope_mode, theta, view->head_dim, p.inv_freq, &p.sectioned_step);
    const uint32_t max_length = decode_state ? static_cast<uint32_t>(view->capacity) : position + 1;
    MergeParams mp{};
    mp.query_heads = query_heads;
    mp.head_dim = view->head_dim;
    mp.gate = gate;
    mp.output = output;
    mp.gated_output = gated_output;
    mp.gated_output_q8 = gated_output_q8;
    return run_decode(p, *view, max_length, workspace, workspace_bytes, num_splits, mp, 1, s);
}

int b200kv_decode_attn_batched(const b200kv_view* views, void* view_table, const uint32_t* lengths,
                               uint32_t sessions, uint32_t max_length, const void* q, int q_dtype,
                               const float* gate, float* output, float* gated_output,
                               uint32_t query_heads, float scale, void* workspace, size_t workspace_bytes,
                               uint32_t num_splits, void* stream) {
    if (sessions == 0) return B200KV_OK;
    if (view_table == nullptr || lengths == nullptr || q == nullptr || (output == nullptr && gated_output == nullptr))
        return B200KV_ERR_INVALID;
    if (q_dtype != B200KV_F16 && q_dtype != B200KV_F32) return B200KV_ERR_INVALID;
    if (sessions > 65535) return B200KV_ERR_UNSUPPORTED;
    int rc;
    bool geometry_fast = false;
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    b200kv_view geometry;
    if (views != nullptr) {
        for (uint32_t i = 0; i < sessions; ++i) {
            if ((rc = validate_view(&views[i])) != B200KV_OK) return rc;
            if (views[i].head_dim != views[0].head_dim || views[i].kv_heads != views[0].kv_heads ||
                views[i].qblock != views[0].qblock || views[i].quant_mode != views[0].quant_mode)
                return B200KV_ERR_INVALID;
        }
        geometry = views[0];
        // Entries are staged in host memory and copied once; the copy from pageable memory completes
        // (as far as the host buffer is concerned) before cudaMemcpyAsync returns.
        std::vector<SessionEntry> staged(sessions);
        bool fast_ok = true;
        for (uint32_t i = 0; i < sessions; ++i) {
            std::memset(&staged[i], 0, sizeof(SessionEntry));
            staged[i].view = views[i];
            if (!q8_fast_path_ok(views[i], query_heads) || encode_kv_maps(views[i], 16, &staged[i].kmap, &staged[i].vmap) != B200KV_OK ||
                encode_kv_maps(views[i], 128, &staged[i].kmap128, &staged[i].vmap128) != B200KV_OK)
                fast_ok = false;
        }
        if (!fast_ok)
            for (uint32_t i = 0; i < sessions; ++i) std::memset(&staged[i].kmap, 0, 4 * sizeof(CUtensorMap));
        geometry_fast = fast_ok;
        B200KV_CUDA_TRY(cudaMemcpyAsync(view_table, staged.data(), sizeof(SessionEntry) * sessions, cudaMemcpyHostToDevice, s));
        B200KV_CUDA_TRY(cudaStreamSynchronize(s));
        remember_table(view_table, geometry, geometry_fast, sessions);
    } else if (recall_table(view_table, sessions, &geometry, &geometry_fast)) {
        // the table was filled by an earlier call of this process: nothing to fetch, the launch stays asynchronous
    } else {
        // a table this process has no record of: fetch the geometry of entry 0 (synchronises the stream)
        SessionEntry first;
        B200KV_CUDA_TRY(cudaMemcpyAsync(&first, view_table, sizeof first, cudaMemcpyDeviceToHost, s));
        B200KV_CUDA_TRY(cudaStreamSynchronize(s));
        geometry = first.view;
        if ((rc = validate_view(&geometry)) != B200KV_OK) return rc;
        // an all-zero descriptor marks a table whose sessions cannot take the streaming kernel
        const uint64_t* words = reinterpret_cast<const uint64_t*>(&first.kmap);
        geometry_fast = false;
        for (int w = 0; w < 16; ++w) geometry_fast = geometry_fast || words[w] != 0;
    }
    if ((rc = check_heads(&geometry, query_heads, scale)) != B200KV_OK) return rc;

    DecodeParams p{};
    p.view = geometry;
    p.views = static_cast<const SessionEntry*>(view_table);
    p.lengths = lengths;
    p.sessions = sessions;
    p.q = q;
    p.q_is_f16 = (q_dtype == B200KV_F16);
    p.query_heads = query_heads;
    p.scale = scale;
    if (!geometry_fast) num_splits |= B200KV_SPLITS_FORCE_GENERIC;
    MergeParams mp{};
    mp.query_heads = query_heads;
    mp.head_dim = geometry.head_dim;
    mp.gate = gate;
    mp.output = output;
    mp.gated_output = gated_output;
    return run_decode(p, geometry, max_length, workspace, workspace_bytes, num_splits, mp, sessions, s);
}

int b200kv_decode_partials(const b200kv_view* view, const void* q, int q_dtype, uint32_t query_heads,
                           float scale, uint32_t range_begin, uint32_t range_end,
                           float* part_m, float* part_l, float* part_acc,
                           void* workspace, size_t workspace_bytes, uint32_t num_splits, void* stream) {
    int rc = validate_view(view);
    if (rc != B200KV_OK) return rc;
    if (q == nullptr || part_m == nullptr || part_l == nullptr || part_acc == nullptr) return B200KV_ERR_INVALID;
    if (q_dtype != B200KV_F16 && q_dtype != B200KV_F32) return B200KV_ERR_INVALID;
    if ((rc = check_heads(view, query_heads, scale)) != B200KV_OK) return rc;
    if (range_end > view->capacity || range_begin > range_end) return B200KV_ERR_RANGE;
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    DecodeParams p{};
    p.view = *view;
    p.cache_length = range_end;
    p.range_begin = range_begin;
    p.sessions = 1;
    p.q = q;
    p.q_is_f16 = (q_dtype == B200KV_F16);
    p.query_heads = query_heads;
    p.scale = scale;
    MergeParams mp{};
    mp.query_heads = query_heads;
    mp.head_dim = view->head_dim;
    mp.out_m = part_m;
    mp.out_l = part_l;
    mp.out_acc = part_acc;
    return run_decode(p, *view, range_end - range_begin, workspace, workspace_bytes, num_splits, mp, 1, s);
}

size_t b200kv_exchange_bytes(uint32_t query_heads, uint32_t head_dim, uint32_t world) {
    // [2 slots][world][query_heads][head_dim + 2] tagged 8-byte words
    return static_cast<size_t>(2) * (world ? world : 1) * query_heads * (head_dim + 2u) * sizeof(uint64_t);
}

int b200kv_decode_attn_sharded(const b200kv_view* view, const void* q, int q_dtype, const float* gate,
                               float* output, float* gated_output, uint32_t query_heads, float scale,
                               uint32_t range_begin, uint32_t range_end,
                               void* const* exchange, uint32_t rank, uint32_t world, uint32_t phase,
                               void* workspace, size_t workspace_bytes, uint32_t num_splits, void* stream) {
    int rc = validate_view(view);
    if (rc != B200KV_OK) return rc;
    if (q == nullptr || (output == nullptr && gated_output == nullptr) || exchange == nullptr) return B200KV_ERR_INVALID;
    if (q_dtype != B200KV_F16 && q_dtype != B200KV_F32) return B200KV_ERR_INVALID;
    if ((rc = check_heads(view, query_heads, scale)) != B200KV_OK) return rc;
    if (range_end > view->capacity || range_begin > range_end) return B200KV_ERR_RANGE;
    if (world == 0 || world > static_cast<uint32_t>(kMaxExchangeRanks) || rank >= world || phase == 0xffffffffu) return B200KV_ERR_INVALID;
    for (uint32_t w = 0; w < world; ++w)
        if (exchange[w] == nullptr || (reinterpret_cast<uintptr_t>(exchange[w]) & 15u) != 0) return B200KV_ERR_INVALID;
    // the exchange lives inside the streaming kernel; other cache modes use b200kv_decode_partials + a collective
    if (!q8_fast_path_ok(*view, query_heads) || (num_splits & B200KV_SPLITS_FORCE_GENERIC)) return B200KV_ERR_UNSUPPORTED;
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    DecodeParams p{};
    p.view = *view;
    p.cache_length = range_end;
    p.range_begin = range_begin;
    p.sessions = 1;
    p.q = q;
    p.q_is_f16 = (q_dtype == B200KV_F16);
    p.query_heads = query_heads;
    p.scale = scale;
    MergeParams mp{};
    mp.query_heads = query_heads;
    mp.head_dim = view->head_dim;
    mp.gate = gate;
    mp.output = output;
    mp.gated_output = gated_output;
    for (uint32_t w = 0; w < world; ++w) mp.xchg.peers[w] = static_cast<uint64_t*>(exchange[w]);
    mp.xchg.rank = rank;
    mp.xchg.world = world;
    mp.xchg.phase = phase;
    mp.xchg.tag = phase + 1u;   // never 0
    // a shard may be empty (range_begin == range_end): the kernel still runs, contributes l = 0 and takes part in the exchange
    const uint32_t span = range_end - range_begin;
    return run_decode(p, *view, span ? span : 1, workspace, workspace_bytes, num_splits, mp, 1, s);
}

int b200kv_merge_partials(const float* part_m, const float* part_l, const float* part_acc,
                          uint32_t num_parts, uint32_t query_heads, uint32_t head_dim,
                          const float* gate, float* output, float* gated_output, void* stream) {
    if (part_m == nullptr || part_l == nullptr || part_acc == nullptr || num_parts == 0 || query_heads == 0)
        return B200KV_ERR_INVALID;
    if (output == nullptr && gated_output == nullptr) return B200KV_ERR_INVALID;
    if (head_dim == 0 || head_dim > 1024) return B200KV_ERR_UNSUPPORTED;
    int rc;
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    MergeParams mp{};
    mp.part_m = part_m;
    mp.part_l = part_l;
    mp.part_acc = part_acc;
    mp.num_parts = num_parts;
    mp.query_heads = query_heads;
    mp.head_dim = head_dim;
    mp.gate = gate;
    mp.output = output;
    mp.gated_output = gated_output;
    return launch_merge(mp, 1, static_cast<cudaStream_t>(stream));
}

int b200kv_merge_partials_packed(const float* packed, uint32_t num_parts, uint32_t query_heads, uint32_t head_dim,
                                 const float* gate, float* output, float* gated_output, void* stream) {
    if (packed == nullptr || num_parts == 0 || query_heads == 0) return B200KV_ERR_INVALID;
    if (output == nullptr && gated_output == nullptr) return B200KV_ERR_INVALID;
    if (head_dim == 0 || head_dim > 1024) return B200KV_ERR_UNSUPPORTED;
    int rc;
    if ((rc = ensure_device()) != B200KV_OK) return rc;
    MergeParams mp{};
    mp.part_m = packed;
    mp.part_l = packed + query_heads;
    mp.part_acc = packed + 2 * static_cast<size_t>(query_heads);
    mp.part_stride = static_cast<size_t>(query_heads) * (head_dim + 2u);
    mp.num_parts = num_parts;
    mp.query_heads = query_heads;
    mp.head_dim = head_dim;
    mp.gate = gate;
    mp.output = output;
    mp.gated_output = gated_output;
    return launch_merge(mp, 1, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
