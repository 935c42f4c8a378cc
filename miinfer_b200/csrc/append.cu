// Fused KV append: (optional K RMSNorm) -> RoPE on K -> int8 quantization with
// fp16 block scales (or fp16 passthrough) -> cache write, for K and V of every
// (token, kv_head) row in one launch.
//
// Behaviour follows MIInfer's store kernel
// (gfx906/kernels/qwen3_primitives.hip:7213-7326): same operation order, same
// quantizer, positions optionally read from device-resident state.  The mapping
// is new: the unit of work is one PASS of one token -- 16 K blocks and 16 V blocks of 32 dims, i.e. four kv heads
// at head_dim 128, two at 256 -- and every warp of a grid sized to the device takes one contiguous run of units.
//   - K rows: lane L holds elements L, L+32, L+64, ... so a q8_0 block is one register index across the warp (its
//     maximum is one `redux.sync` on the bits of |x|), both RoPE pairings (i, i+d/2) and (i, i+32) pair two
//     registers of the SAME lane, and the reference's shared-memory binary tree for the sum of squares (stride
//     d/2 .. 1) becomes register adds followed by a shuffle-down tree that adds exactly the same pairs in the same
//     order (bit-identical sum).  Elements are read and written one by one: every access of the warp is one
//     contiguous run of 32 elements, so nothing is staged.
//   - V rows, which are only quantised: lane L holds the 4 (8) consecutive elements 4L .. (8L ..), one vector load and
//     one vector store per row; a block is 8 (4) neighbouring lanes and its maximum takes 3 (2) shuffles.
//   - the sines and cosines depend on the token only and are computed when a warp's run reaches a new token;
//   - the warp-uniform IEEE divisions are spread over the lanes: lane h takes head h's 1/rms, lanes 0-15 the K
//     blocks' amax/127 and reciprocal, lanes 16-31 the V blocks'; the results come back by shuffle.
// (Earlier layouts -- a warp per row pair with every division repeated by all lanes; all rows lane-strided through
// shared-memory staging rows -- ran at 0.11 and 0.33 of the HBM rate on 8192-token chunks; this one at 0.37.  Fetching a
// unit's rows one unit ahead of the arithmetic measured slower: 34 us against 21.5.)
// The row arithmetic is the same, operation for operation, as append_row.cuh's (used by the decode kernel's fused
// single-token append and the query-side kernel): all three write identical bits.
#include "append_row.cuh"

#include <algorithm>
#include <cmath>
#include <type_traits>

namespace b200kv {

struct AppendParams {
    b200kv_view view;
    const void* key;
    const void* value;
    const float* k_norm_weight;
    const b200kv_prefill_state* prefill_state;
    const b200kv_decode_state* decode_state;
    uint32_t token_count;
    uint32_t base_position;
    int rope_mode;
    float epsilon;
    float sectioned_step;    // powf(theta, -2/64)
    float inv_freq[128];     // NeoX: powf(theta, -2i/d), i < d/2
};

constexpr int kAppendWarps = 2;
constexpr int kAppendCtasPerSm = 8;    // 128 registers per thread: a pass keeps 32 row values per lane (10, 12 and 16 CTAs spill and measured slower)

__device__ __forceinline__ int quantize_s8(float v) {
    // round to nearest even and saturate to [-128, 127] (NaN -> 0): __float2int_rn followed by the clamp, in one step
    int q;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(v));
    return q;
}
// max over the warp of non-negative floats (NaN counts as 0, as with fmaxf): one redux on the bit patterns
__device__ __forceinline__ float warp_amax(float a) {
    return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fmaxf(a, 0.0f))));
}

template <int D, bool IN_F16>
__global__ void __launch_bounds__(kAppendWarps * 32, kAppendCtasPerSm)
append_kernel(const __grid_constant__ AppendParams p, const bool vec) {
    constexpr int NJ = D / 32;                  // q8_0 blocks per row = K registers per lane
    constexpr int HB = 16 / NJ;                 // kv heads per pass: 16 K blocks + 16 V blocks, one scale per lane
    constexpr int GS = 32 / NJ;                 // lanes that share one V block (each holds NJ consecutive elements of it)
    __shared__ float freq_s[D / 2];
    __shared__ float kmax_s[kAppendWarps][16];
    // Let the next kernel of the stream become resident now (it orders itself against this one), then wait
    // for everything before us: K/V inputs and the device-side position come from preceding kernels.
    pdl_launch_dependents();
    pdl_wait();

    uint32_t base_position = p.base_position;
    uint32_t token_count = p.token_count;
    uint64_t capacity = p.view.capacity;
    if (p.prefill_state != nullptr) {
        base_position = p.prefill_state->base_position;
        token_count = min(token_count, p.prefill_state->token_count);
        if (p.prefill_state->kv_capacity > 0) capacity = p.prefill_state->kv_capacity;
    } else if (p.decode_state != nullptr) {
        base_position = p.decode_state->position;
        token_count = min(token_count, 1u);
    }
    if (p.rope_mode == B200KV_ROPE_NEOX_FULL)
        for (int i = threadIdx.x; i < D / 2; i += kAppendWarps * 32) freq_s[i] = p.inv_freq[i];
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t H = p.view.kv_heads;
    const uint32_t mode = p.view.quant_mode;
    const bool k_q8 = (mode == B200KV_Q8_F16 || mode == B200KV_Q8_Q8);
    const bool v_q8 = (mode == B200KV_F16_Q8 || mode == B200KV_Q8_Q8);
    const bool row_scale = p.view.qblock == D;
    const bool have_norm = p.k_norm_weight != nullptr;
    const int rope_mode = p.rope_mode;

    float w[NJ];
    if (have_norm) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) w[j] = p.k_norm_weight[lane + 32 * j];
    }
    float sn[NJ / 2], cs[NJ / 2];   // what depends on the token alone: the rotation of every pair this lane holds

    // One pass: K and V of kv heads g0 .. g0 + hn - 1 of one token.
    //   K rows: lane L holds elements L, L+32, ... (a block = one register index across the warp), fetched and stored
    //           element by element -- every access of the warp is one contiguous run of 32 elements;
    //   V rows: lane L holds the NJ consecutive elements NJ*L ..  (a block = GS neighbouring lanes), one vector load and
    //           one vector store per row.
    // FAST: a full pass (hn == HB) of an int8/int8 cache with q8_0 blocks -- every check below is decided at compile time.
    auto pass = [&](auto fast_c, uint32_t token, uint32_t g0, uint64_t position, int hn) {
        constexpr bool FAST = decltype(fast_c)::value;
        if constexpr (FAST) hn = HB;
        const bool kq = FAST || k_q8, vq = FAST || v_q8, rows = !FAST && row_scale;
        const uint64_t row0 = g0 * capacity + position;   // cache row of the pass's first head; the next head is `capacity` rows on
        const size_t in0 = (static_cast<size_t>(token) * H + g0) * D;
        float kx[HB][NJ], vx[HB][NJ];
#pragma unroll
        for (int h = 0; h < HB; ++h) {
            if (!FAST && h >= hn) break;
            const size_t in_h = in0 + static_cast<size_t>(h) * D;
            if (IN_F16) {
                const __half* ksrc = static_cast<const __half*>(p.key) + in_h;
                const __half* vsrc = static_cast<const __half*>(p.value) + in_h + NJ * lane;
#pragma unroll
                for (int j = 0; j < NJ; ++j) kx[h][j] = __half2float(ksrc[lane + 32 * j]);
                if (vec) {
                    if constexpr (NJ == 4) {
                        const uint2 raw = *reinterpret_cast<const uint2*>(vsrc);
                        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                        vx[h][0] = a.x; vx[h][1] = a.y; vx[h][2] = b.x; vx[h][3] = b.y;
                    } else {
                        const uint4 raw = *reinterpret_cast<const uint4*>(vsrc);
                        const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
                            vx[h][2 * i] = a.x; vx[h][2 * i + 1] = a.y;
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < NJ; ++j) vx[h][j] = __half2float(vsrc[j]);
                }
            } else {
                const float* ksrc = static_cast<const float*>(p.key) + in_h;
                const float* vsrc = static_cast<const float*>(p.value) + in_h + NJ * lane;
#pragma unroll
                for (int j = 0; j < NJ; ++j) kx[h][j] = ksrc[lane + 32 * j];
                if (vec) {
#pragma unroll
                    for (int i = 0; i < NJ / 4; ++i) {
                        const float4 a = *reinterpret_cast<const float4*>(vsrc + 4 * i);
                        vx[h][4 * i] = a.x; vx[h][4 * i + 1] = a.y; vx[h][4 * i + 2] = a.z; vx[h][4 * i + 3] = a.w;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < NJ; ++j) vx[h][j] = vsrc[j];
                }
            }
        }

        // ---- K: RMSNorm * weight.  The reference's shared-memory tree (stride D/2 .. 1): register adds, then a shuffle-down
        //      tree over the same pairs; lane h then takes head h's IEEE division and square root ----
        if (have_norm) {
            float ss_mine = 0.0f;
#pragma unroll
            for (int h = 0; h < HB; ++h) {
                if (!FAST && h >= hn) break;
                float sq[NJ];
#pragma unroll
                for (int j = 0; j < NJ; ++j) sq[j] = __fmul_rn(kx[h][j], kx[h][j]);
#pragma unroll
                for (int half = NJ / 2; half >= 1; half >>= 1)
#pragma unroll
                    for (int j = 0; j < half; ++j) sq[j] = __fadd_rn(sq[j], sq[j + half]);
                float ss = sq[0];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, o));
                ss = __shfl_sync(0xffffffffu, ss, 0);
                if (lane == h) ss_mine = ss;
            }
            const float r_mine = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss_mine, static_cast<float>(D)), p.epsilon)));
#pragma unroll
            for (int h = 0; h < HB; ++h) {
                if (!FAST && h >= hn) break;
                const float r = __shfl_sync(0xffffffffu, r_mine, h);
#pragma unroll
                for (int j = 0; j < NJ; ++j) kx[h][j] = __fmul_rn(__fmul_rn(kx[h][j], r), w[j]);
            }
        }
        // ---- K: RoPE
        if (rope_mode == B200KV_ROPE_NEOX_FULL) {
#pragma unroll
            for (int h = 0; h < HB; ++h) {
                if (!FAST && h >= hn) break;
#pragma unroll
                for (int j = 0; j < NJ / 2; ++j) {
                    const float x0 = kx[h][j], x1 = kx[h][j + NJ / 2];
                    kx[h][j] = __fsub_rn(__fmul_rn(x0, cs[j]), __fmul_rn(x1, sn[j]));
                    kx[h][j + NJ / 2] = __fadd_rn(__fmul_rn(x0, sn[j]), __fmul_rn(x1, cs[j]));
                }
            }
        } else if (rope_mode == B200KV_ROPE_SECTIONED64) {
#pragma unroll
            for (int h = 0; h < HB; ++h) {
                if (!FAST && h >= hn) break;
                const float x0 = kx[h][0], x1 = kx[h][1];
                kx[h][0] = __fsub_rn(__fmul_rn(x0, cs[0]), __fmul_rn(x1, sn[0]));
                kx[h][1] = __fadd_rn(__fmul_rn(x0, sn[0]), __fmul_rn(x1, cs[0]));
            }
        }

        // ---- block maxima.  K: one redux per block, the 16 results through shared memory to lanes 0-15 (lane = HB... NJ*h + j).
        //      V: a block's GS lanes reduce among themselves; lane 16 + NJ*h + j fetches the result from the block's first lane.
        //      With one scale per row (rows): lanes h and 16 + h. ----
        float amax_mine = 0.0f;
#pragma unroll
        for (int h = 0; h < HB; ++h) {
            if (!FAST && h >= hn) break;
            if (rows) {
                float a = 0.0f, b = 0.0f;
#pragma unroll
                for (int j = 0; j < NJ; ++j) { a = fmaxf(a, fabsf(kx[h][j])); b = fmaxf(b, fabsf(vx[h][j])); }
                a = warp_amax(a); b = warp_amax(b);
                if (lane == h) amax_mine = a;
                if (lane == 16 + h) amax_mine = b;
            } else {
#pragma unroll
                for (int j = 0; j < NJ; ++j) kmax_s[warp][NJ * h + j] = warp_amax(fabsf(kx[h][j]));   // every lane holds the value: no predicate
                float b = 0.0f;
#pragma unroll
                for (int j = 0; j < NJ; ++j) b = fmaxf(b, fabsf(vx[h][j]));
#pragma unroll
                for (int o = GS / 2; o > 0; o >>= 1) b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, o));
                const float got = __shfl_sync(0xffffffffu, b, (lane & (NJ - 1)) * GS);   // block j = lane % NJ of head h
                if ((lane >> 4) == 1 && ((lane & 15) / NJ) == h) amax_mine = got;
            }
        }
        if (!rows) {
            __syncwarp();
            if (lane < 16) amax_mine = kmax_s[warp][lane];
            __syncwarp();   // the next pass overwrites the words
        }
        // ---- scales: amax / 127, its reciprocal, the fp16 scale to the cache -- one block per lane
        const float scale_mine = (amax_mine > 0.0f) ? __fdiv_rn(amax_mine, 127.0f) : 1.0f;
        const float inv_mine = (scale_mine > 0.0f) ? __fdiv_rn(1.0f, scale_mine) : 1.0f;
        {
            const int side = lane >> 4, idx = lane & 15;
            const int h = rows ? idx : idx / NJ, j = rows ? 0 : idx % NJ;
            const bool mine = rows ? idx < hn : h < hn;
            if (mine && (side == 0 ? kq : vq)) {
                __half* plane = static_cast<__half*>(side == 0 ? p.view.key_scales : p.view.value_scales);
                const uint64_t r = row0 + static_cast<uint64_t>(h) * capacity;
                plane[rows ? r : r * NJ + j] = __float2half_rn(scale_mine);
            }
        }
        // ---- quantise and store
#pragma unroll
        for (int h = 0; h < HB; ++h) {
            if (!FAST && h >= hn) break;
            const uint64_t r = row0 + static_cast<uint64_t>(h) * capacity;
            if (kq) {
                int8_t* dst = p.view.key_q8 + r * D + lane;
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const float inv = __shfl_sync(0xffffffffu, inv_mine, rows ? h : NJ * h + j);
                    dst[32 * j] = static_cast<int8_t>(quantize_s8(__fmul_rn(kx[h][j], inv)));
                }
            } else {
                __half* dst = static_cast<__half*>(p.view.key_f16) + r * D + lane;
#pragma unroll
                for (int j = 0; j < NJ; ++j) dst[32 * j] = __float2half_rn(kx[h][j]);
            }
            if (vq) {
                const float inv = __shfl_sync(0xffffffffu, inv_mine, 16 + (rows ? h : NJ * h + lane / GS));
                uint32_t packed[NJ / 4];
#pragma unroll
                for (int i = 0; i < NJ / 4; ++i) {
                    const uint32_t b0 = quantize_s8(__fmul_rn(vx[h][4 * i], inv)) & 0xff, b1 = quantize_s8(__fmul_rn(vx[h][4 * i + 1], inv)) & 0xff;
                    const uint32_t b2 = quantize_s8(__fmul_rn(vx[h][4 * i + 2], inv)) & 0xff, b3 = quantize_s8(__fmul_rn(vx[h][4 * i + 3], inv)) & 0xff;
                    packed[i] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
                }
                int8_t* dst = p.view.value_q8 + r * D + NJ * lane;
                if constexpr (NJ == 4) *reinterpret_cast<uint32_t*>(dst) = packed[0];
                else *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[1]);
            } else {
                __half* dst = static_cast<__half*>(p.view.value_f16) + r * D + NJ * lane;
#pragma unroll
                for (int j = 0; j < NJ; j += 2) *reinterpret_cast<__half2*>(dst + j) = __floats2half2_rn(vx[h][j], vx[h][j + 1]);
            }
        }
    };

    // The unit of work is one pass of one token; every warp of the grid takes one contiguous run of units, so a
    // large launch spreads evenly over the resident warps (and a warp meets few tokens), while a small one
    // spreads the passes of a token over several warps.  (32-bit arithmetic: the host keeps units below 2^32.)
    const uint32_t passes = (H + HB - 1) / HB;
    const uint32_t total_units = token_count * passes;
    const uint32_t warps = gridDim.x * kAppendWarps;
    const uint32_t per_warp = (total_units + warps - 1) / warps;
    const uint32_t unit0 = min(total_units, (blockIdx.x * kAppendWarps + warp) * per_warp);
    const uint32_t unit1 = min(total_units, unit0 + per_warp);
    uint32_t token = unit0 / passes;
    uint32_t pass_index = unit0 - token * passes;
    bool fresh = true;   // the rotation has to be computed for `token`
    const bool fast_cache = k_q8 && v_q8 && !row_scale;
    for (uint32_t unit = unit0; unit < unit1; ++unit) {
        const uint64_t position = static_cast<uint64_t>(base_position) + token;
        if (position < capacity) {   // never write outside the cache
            if (fresh) {
                fresh = false;
                if (rope_mode == B200KV_ROPE_NEOX_FULL) {
#pragma unroll
                    for (int j = 0; j < NJ / 2; ++j)
                        sincos_pinned(__fmul_rn(static_cast<float>(static_cast<uint32_t>(position)), freq_s[lane + 32 * j]), &sn[j], &cs[j]);
                } else if (rope_mode == B200KV_ROPE_SECTIONED64) {
                    float angle = static_cast<float>(static_cast<uint32_t>(position));
                    for (int i = 0; i < lane; ++i) angle = __fmul_rn(angle, p.sectioned_step);
                    sincos_pinned(angle, &sn[0], &cs[0]);
                }
            }
            const uint32_t g0 = pass_index * HB;
            const int hn = static_cast<int>(min(static_cast<uint32_t>(HB), H - g0));
            if (fast_cache && hn == HB) pass(std::true_type{}, token, g0, position, hn);
            else pass(std::false_type{}, token, g0, position, hn);
        }
        if (++pass_index == passes) {
            pass_index = 0;
            ++token;
            fresh = true;
        }
    }
}

}  // namespace b200kv

using namespace b200kv;

extern "C" int b200kv_append(const b200kv_view* view, const void* key, const void* value, int dtype,
                             const float* k_norm_weight, int rope_mode, float theta, float epsilon,
                             uint32_t token_count, uint32_t base_position,
                             const b200kv_prefill_state* prefill_state, const b200kv_decode_state* decode_state,
                             void* stream) {
    int rc = validate_view(view);
    if (rc != B200KV_OK) return rc;
    if (key == nullptr || value == nullptr || (dtype != B200KV_F16 && dtype != B200KV_F32)) return B200KV_ERR_INVALID;
    if (rope_mode < B200KV_ROPE_NONE || rope_mode > B200KV_ROPE_SECTIONED64) return B200KV_ERR_INVALID;
    if (!std::isfinite(theta) || !std::isfinite(epsilon)) return B200KV_ERR_INVALID;
    if (rope_mode != B200KV_ROPE_NONE && !(theta > 0.0f)) return B200KV_ERR_INVALID;
    if (token_count == 0) return B200KV_OK;
    if (prefill_state == nullptr && decode_state == nullptr &&
        static_cast<uint64_t>(base_position) + token_count > view->capacity)
        return B200KV_ERR_RANGE;
    rc = ensure_device();
    if (rc != B200KV_OK) return rc;

    AppendParams p{};
    p.view = *view;
    p.key = key;
    p.value = value;
    p.k_norm_weight = k_norm_weight;
    p.prefill_state = prefill_state;
    p.decode_state = decode_state;
    p.token_count = token_count;
    p.base_position = base_position;
    p.rope_mode = rope_mode;
    p.epsilon = epsilon;
    rope_constants(rope_mode, theta, view->head_dim, p.inv_freq, &p.sectioned_step);

    const uint32_t d = view->head_dim;
    const uint32_t heads_per_pass = 512 / d;   // 16 K blocks and 16 V blocks of 32 dims per pass
    const uint64_t units = static_cast<uint64_t>(token_count) * ((view->kv_heads + heads_per_pass - 1) / heads_per_pass);
    if (units >= (1ull << 32)) return B200KV_ERR_RANGE;
    int device = 0, sms = 0;
    B200KV_CUDA_TRY(cudaGetDevice(&device));
    B200KV_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const uint64_t resident = static_cast<uint64_t>(sms) * kAppendCtasPerSm;
    const unsigned grid = static_cast<unsigned>(std::min<uint64_t>((units + kAppendWarps - 1) / kAppendWarps, resident));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool f16 = (dtype == B200KV_F16);
    const bool vec = (reinterpret_cast<uintptr_t>(value) & 15u) == 0;   // vector loads of the V rows need an aligned input
    const dim3 block(kAppendWarps * 32);
    cudaError_t err;
    auto launch = [&](auto kernel) { return launch_kernel(kernel, grid, block, 0, s, true, p, vec); };
    if (d == 128) err = f16 ? launch(append_kernel<128, true>) : launch(append_kernel<128, false>);
    else err = f16 ? launch(append_kernel<256, true>) : launch(append_kernel<256, false>);
    B200KV_CUDA_TRY(err);
    return B200KV_OK;
}
