// Fused KV append: (optional K RMSNorm) -> RoPE on K -> int8 quantization with
// fp16 block scales (or fp16 passthrough) -> cache write, for K and V of every
// (token, kv_head) row in one launch.
//
// Behaviour follows MIInfer's store kernel
// (gfx906/kernels/qwen3_primitives.hip:7213-7326): same operation order, same
// quantizer, positions optionally read from device-resident state.  The mapping
// is new: the unit of work is one PASS of one token -- 16 q8_0 blocks, K and V of two kv
// heads at head_dim 128 or of one at 256 -- and every warp of a grid sized to the device
// takes one contiguous run of units.  Within a row lane L holds elements L, L+32, L+64, ... so
//   - a q8_0 block (32 consecutive dims) is one register index across the warp
//     and its amax is one `redux.sync` on the bits of |x|;
//   - both RoPE pairings (i, i+d/2) and (i, i+32) pair two registers of the SAME
//     lane, so the rotation needs no exchange; the sines and cosines depend on the
//     token only and are computed when a warp's run reaches a new token, not per head;
//   - the reference's shared-memory binary tree for the sum of squares (stride
//     d/2 .. 1) becomes register adds followed by a shuffle-down tree that adds
//     exactly the same pairs in the same order (bit-identical sum);
//   - the warp-uniform IEEE divisions (1/rms per head, amax/127 and its reciprocal
//     per block) are spread over the lanes -- lane i does head i, then block i --
//     and handed back through shared memory instead of being repeated by all 32 lanes.
// Input rows are fetched with 16-byte loads, all of a pass in flight at once, and re-read
// from a per-warp staging area in the lane-strided order; output rows are staged through
// shared memory and written with 16-byte stores (whole 128/256-byte cache rows).
// The row arithmetic is the same, operation for operation, as append_row.cuh's (used by the
// decode kernel's fused single-token append and the query-side kernel): all three write
// identical bits.
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

__device__ __forceinline__ int quantize_s8(float v) {
    // round to nearest even and saturate to [-128, 127] (NaN -> 0): __float2int_rn followed by the clamp, in one step
    int q;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(v));
    return q;
}

template <int ITEMS> struct AppendTuning;
template <> struct AppendTuning<16> { static constexpr int kCtasPerSm = 16; };
template <> struct AppendTuning<32> { static constexpr int kCtasPerSm = 12; };   // measured: equal on 8192-token chunks, slower on 512
template <> struct AppendTuning<64> { static constexpr int kCtasPerSm = 8; };    // measured: 17 % slower on 8192-token chunks

template <int D, bool IN_F16, int ITEMS>
__global__ void __launch_bounds__(kAppendWarps * 32, AppendTuning<ITEMS>::kCtasPerSm)
append_kernel(const __grid_constant__ AppendParams p, const bool vec) {
    constexpr int NJ = D / 32;
    constexpr int GH = ITEMS / (2 * NJ);        // kv heads per pass: K and V of GH heads make ITEMS q8_0 blocks
    constexpr int kEsize = IN_F16 ? 2 : 4;
    constexpr int kRowBytes = D * kEsize;
    __shared__ __align__(16) uint8_t in_stage[kAppendWarps][2][GH * kRowBytes];   // [warp][K | V][head][D]
    __shared__ __align__(16) int8_t out_stage[kAppendWarps][2][GH * D];
    __shared__ __align__(16) float amax_s[kAppendWarps][ITEMS];
    __shared__ __align__(16) float inv_s[kAppendWarps][ITEMS];
    __shared__ float norm_s[kAppendWarps][GH];
    __shared__ float freq_s[D / 2];
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

    // One pass: K and V of kv heads g0 .. g0 + hn - 1 of one token.  FAST: a full pass (hn == GH) of an int8/int8
    // cache with q8_0 blocks -- every check below is decided at compile time.
    auto pass = [&](auto fast_c, uint32_t token, uint32_t g0, uint64_t position, int hn) {
        constexpr bool FAST = decltype(fast_c)::value;
        if constexpr (FAST) hn = GH;
        const bool kq = FAST || k_q8, vq = FAST || v_q8, rows = !FAST && row_scale;
        const uint64_t row0 = g0 * capacity + position;   // cache row of the pass's first head; the next head is `capacity` rows on
        // ---- the pass's K and V rows (contiguous in the [token][kv_heads * D] inputs) into the staging area
        {
            const size_t in_off = (static_cast<size_t>(token) * H + g0) * kRowBytes;
            const uint8_t* ksrc = static_cast<const uint8_t*>(p.key) + in_off;
            const uint8_t* vsrc = static_cast<const uint8_t*>(p.value) + in_off;
            const int bytes = hn * kRowBytes;
            if (vec) {
                constexpr int kIters = (GH * kRowBytes + 511) / 512;
                constexpr bool kExact = kIters * 512 == GH * kRowBytes;
#pragma unroll
                for (int side = 0; side < 2; ++side) {
                    const uint8_t* src = side == 0 ? ksrc : vsrc;
                    uint4 reg[kIters];
#pragma unroll
                    for (int it = 0; it < kIters; ++it) {
                        const int off = it * 512 + lane * 16;
                        if ((FAST && kExact) || off < bytes) reg[it] = *reinterpret_cast<const uint4*>(src + off);
                    }
#pragma unroll
                    for (int it = 0; it < kIters; ++it) {
                        const int off = it * 512 + lane * 16;
                        if ((FAST && kExact) || off < bytes) *reinterpret_cast<uint4*>(&in_stage[warp][side][off]) = reg[it];
                    }
                }
            } else {   // inputs that are not 16-byte aligned: element by element
                using elem_t = typename std::conditional<IN_F16, uint16_t, uint32_t>::type;
                for (int i = lane; i < hn * D; i += 32) {
                    reinterpret_cast<elem_t*>(in_stage[warp][0])[i] = reinterpret_cast<const elem_t*>(ksrc)[i];
                    reinterpret_cast<elem_t*>(in_stage[warp][1])[i] = reinterpret_cast<const elem_t*>(vsrc)[i];
                }
            }
            __syncwarp();
        }
        float x[GH][2][NJ];
#pragma unroll
        for (int h = 0; h < GH; ++h) {
            if (!FAST && h >= hn) break;
#pragma unroll
            for (int s = 0; s < 2; ++s)
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    if (IN_F16) x[h][s][j] = __half2float(reinterpret_cast<const __half*>(in_stage[warp][s])[h * D + lane + 32 * j]);
                    else x[h][s][j] = reinterpret_cast<const float*>(in_stage[warp][s])[h * D + lane + 32 * j];
                }
        }

        // ---- K: RMSNorm * weight
        if (have_norm) {
#pragma unroll
            for (int h = 0; h < GH; ++h) {
                if (!FAST && h >= hn) break;
                float sq[NJ];
#pragma unroll
                for (int j = 0; j < NJ; ++j) sq[j] = __fmul_rn(x[h][0][j], x[h][0][j]);
#pragma unroll
                for (int half = NJ / 2; half >= 1; half >>= 1)
#pragma unroll
                    for (int j = 0; j < half; ++j) sq[j] = __fadd_rn(sq[j], sq[j + half]);
                float ss = sq[0];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, o));
                if (lane == 0) norm_s[warp][h] = ss;
            }
            __syncwarp();
            if (lane < hn)
                norm_s[warp][lane] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(norm_s[warp][lane], static_cast<float>(D)), p.epsilon)));
            __syncwarp();
#pragma unroll
            for (int h = 0; h < GH; ++h) {
                if (!FAST && h >= hn) break;
                const float r = norm_s[warp][h];
#pragma unroll
                for (int j = 0; j < NJ; ++j) x[h][0][j] = __fmul_rn(__fmul_rn(x[h][0][j], r), w[j]);
            }
        }
        // ---- K: RoPE
        if (rope_mode == B200KV_ROPE_NEOX_FULL) {
#pragma unroll
            for (int h = 0; h < GH; ++h) {
                if (!FAST && h >= hn) break;
#pragma unroll
                for (int j = 0; j < NJ / 2; ++j) {
                    const float x0 = x[h][0][j], x1 = x[h][0][j + NJ / 2];
                    x[h][0][j] = __fsub_rn(__fmul_rn(x0, cs[j]), __fmul_rn(x1, sn[j]));
                    x[h][0][j + NJ / 2] = __fadd_rn(__fmul_rn(x0, sn[j]), __fmul_rn(x1, cs[j]));
                }
            }
        } else if (rope_mode == B200KV_ROPE_SECTIONED64) {
#pragma unroll
            for (int h = 0; h < GH; ++h) {
                if (!FAST && h >= hn) break;
                const float x0 = x[h][0][0], x1 = x[h][0][1];
                x[h][0][0] = __fsub_rn(__fmul_rn(x0, cs[0]), __fmul_rn(x1, sn[0]));
                x[h][0][1] = __fadd_rn(__fmul_rn(x0, sn[0]), __fmul_rn(x1, cs[0]));
            }
        }

        // ---- block maxima (NaN counts as 0, as with fmaxf), one shared-memory word per block; every lane holds
        //      the reduced value, so the store needs no predicate
#pragma unroll
        for (int h = 0; h < GH; ++h) {
            if (!FAST && h >= hn) break;
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                if (rows) {
                    float a = 0.0f;
#pragma unroll
                    for (int j = 0; j < NJ; ++j) a = fmaxf(a, fabsf(x[h][s][j]));
                    amax_s[warp][h * 2 + s] = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(a)));
                } else {
#pragma unroll
                    for (int j = 0; j < NJ; ++j)
                        amax_s[warp][(h * 2 + s) * NJ + j] =
                            __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fmaxf(fabsf(x[h][s][j]), 0.0f))));
                }
            }
        }
        __syncwarp();
        // ---- scales: lane i takes block i (and i + 32): amax / 127, its reciprocal, the fp16 scale to the cache
        {
            const int shift = rows ? 0 : (NJ == 4 ? 2 : 3);   // log2(blocks per row)
            const int items = (hn * 2) << shift;
#pragma unroll
            for (int it = 0; it < (ITEMS + 31) / 32; ++it) {
                const int item = lane + 32 * it;
                if (item < items) {
                    const float amax = amax_s[warp][item];
                    const float scale = (amax > 0.0f) ? __fdiv_rn(amax, 127.0f) : 1.0f;
                    inv_s[warp][item] = (scale > 0.0f) ? __fdiv_rn(1.0f, scale) : 1.0f;
                    const int hs = item >> shift, j = item - (hs << shift);
                    const int h = hs >> 1, s = hs & 1;
                    if (s == 0 ? kq : vq) {
                        __half* plane = static_cast<__half*>(s == 0 ? p.view.key_scales : p.view.value_scales);
                        plane[((row0 + h * capacity) << shift) + j] = __float2half_rn(scale);
                    }
                }
            }
        }
        __syncwarp();
        // ---- quantise into the output staging rows
#pragma unroll
        for (int h = 0; h < GH; ++h) {
            if (!FAST && h >= hn) break;
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                if (!(s == 0 ? kq : vq)) continue;
                float inv[NJ];
                if (rows) {
                    const float one = inv_s[warp][h * 2 + s];
#pragma unroll
                    for (int j = 0; j < NJ; ++j) inv[j] = one;
                } else {
#pragma unroll
                    for (int j4 = 0; j4 < NJ / 4; ++j4) {
                        const float4 f = *reinterpret_cast<const float4*>(&inv_s[warp][(h * 2 + s) * NJ + 4 * j4]);
                        inv[4 * j4] = f.x; inv[4 * j4 + 1] = f.y; inv[4 * j4 + 2] = f.z; inv[4 * j4 + 3] = f.w;
                    }
                }
#pragma unroll
                for (int j = 0; j < NJ; ++j)
                    out_stage[warp][s][h * D + lane + 32 * j] = static_cast<int8_t>(quantize_s8(__fmul_rn(x[h][s][j], inv[j])));
            }
        }
        __syncwarp();
        // ---- cache rows out: 16 bytes per lane, 32 / (D/16) rows per store instruction
        {
            constexpr int kLanesPerRow = D / 16;
            constexpr int kRowsPerStore = 32 / kLanesPerRow;
            const int sub = lane / kLanesPerRow, chunk = lane % kLanesPerRow;
#pragma unroll
            for (int r0 = 0; r0 < 2 * GH; r0 += kRowsPerStore) {
                const int rr = r0 + sub, s = rr / GH, h = rr % GH;
                if ((FAST || h < hn) && (s == 0 ? kq : vq)) {
                    int8_t* plane = s == 0 ? p.view.key_q8 : p.view.value_q8;
                    *reinterpret_cast<uint4*>(plane + (row0 + h * capacity) * D + chunk * 16) =
                        *reinterpret_cast<const uint4*>(&out_stage[warp][s][h * D + chunk * 16]);
                }
            }
        }
        // ---- sides kept in fp16: straight from the registers
        if (!FAST && (!k_q8 || !v_q8)) {
#pragma unroll
            for (int h = 0; h < GH; ++h) {
                if (h >= hn) break;
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    if (s == 0 ? k_q8 : v_q8) continue;
                    __half* dst = static_cast<__half*>(s == 0 ? p.view.key_f16 : p.view.value_f16) + (row0 + h * capacity) * D;
#pragma unroll
                    for (int j = 0; j < NJ; ++j) dst[lane + 32 * j] = __float2half_rn(x[h][s][j]);
                }
            }
        }
        __syncwarp();   // the staging areas are reused by the next pass
    };

    // The unit of work is one pass of one token; every warp of the grid takes one contiguous run of units, so a
    // large launch spreads evenly over the resident warps (and a warp meets few tokens), while a small one
    // spreads the passes of a token over several warps.  (32-bit arithmetic: the host keeps units below 2^32.)
    const uint32_t passes = (H + GH - 1) / GH;
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
            const uint32_t g0 = pass_index * GH;
            const int hn = static_cast<int>(min(static_cast<uint32_t>(GH), H - g0));
            if (fast_cache && hn == GH) pass(std::true_type{}, token, g0, position, hn);
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
    if (rope_mode == B200KV_ROPE_NEOX_FULL) {
        const uint32_t d = view->head_dim;
        for (uint32_t i = 0; i < d / 2; ++i)
            p.inv_freq[i] = std::pow(theta, -static_cast<float>(2 * i) / static_cast<float>(d));
    } else if (rope_mode == B200KV_ROPE_SECTIONED64) {
        p.sectioned_step = std::pow(theta, -2.0f / 64.0f);
    }

    constexpr int kItems = 16;   // q8_0 blocks per pass: K and V of 2 kv heads at head_dim 128, of 1 at 256 (32 and 64 measured slower)
    const uint32_t d = view->head_dim;
    const uint32_t heads_per_pass = kItems * 16 / d;
    const uint64_t units = static_cast<uint64_t>(token_count) * ((view->kv_heads + heads_per_pass - 1) / heads_per_pass);
    if (units >= (1ull << 32)) return B200KV_ERR_RANGE;
    int device = 0, sms = 0;
    B200KV_CUDA_TRY(cudaGetDevice(&device));
    B200KV_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const uint64_t resident = static_cast<uint64_t>(sms) * AppendTuning<kItems>::kCtasPerSm;
    const unsigned grid = static_cast<unsigned>(std::min<uint64_t>((units + kAppendWarps - 1) / kAppendWarps, resident));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool f16 = (dtype == B200KV_F16);
    const bool vec = ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value)) & 15u) == 0;   // 16-byte loads need aligned inputs
    const dim3 block(kAppendWarps * 32);
    cudaError_t err;
    auto launch = [&](auto kernel) { return launch_kernel(kernel, grid, block, 0, s, true, p, vec); };
    if (d == 128) err = f16 ? launch(append_kernel<128, true, kItems>) : launch(append_kernel<128, false, kItems>);
    else err = f16 ? launch(append_kernel<256, true, kItems>) : launch(append_kernel<256, false, kItems>);
    B200KV_CUDA_TRY(err);
    return B200KV_OK;
}
