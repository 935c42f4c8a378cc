// Streaming split-K GQA decode attention over an int8 (q8_0 or row-scaled) KV
// cache, head_dim 128 -- the kernel the decode benchmark runs.
//
// What it computes is MIInfer's decode stage 1
// (gfx906/kernels/qwen3_primitives.hip:7371-7485) with block scales; how it is
// laid out is specific to B200:
//
//  * One CTA = 4 warps = one (kv head, split).  ALL query heads of the kv-head
//    group share every K/V byte the CTA loads (the reference re-reads the cache
//    once per query head).
//  * Each warp owns a private 3-stage ring of 32-position tiles in shared
//    memory, filled by TMA: the K tile through a tensor map with the 128-byte
//    swizzle (rows of 128 int8), V and both scale tiles with plain bulk copies.
//    One lane issues the copies; completion is an mbarrier per stage.  Warps
//    never synchronise with each other in the main loop.
//  * Q.K runs on the integer dot-product pipe: Q is quantised once per launch to
//    int16 with a per-head scale (15 bits + sign: finer than the fp16 inputs'
//    11-bit mantissa for the elements that matter), and dp2a multiplies packed
//    int16 pairs by K's int8 bytes directly -- no int8->float conversion at all
//    on the K side.  The exact int32 block sums are scaled by the fp16 block
//    scales in fp32.  Lane layout: 8 positions x 4 heads per round; the swizzle
//    makes the 8 rows' 16-byte chunks hit distinct banks while every lane keeps
//    its head's Q in registers with static indices.
//  * P.V stays in fp32: lane = (position mod 4, 16-dim chunk), 4 heads x 16
//    dims of accumulators per lane; int8->fp32 by byte-permute into the mantissa
//    of 2^23 and one subtract (the conversion pipe is 8x slower than that), the
//    multiply-adds as packed f32x2.  Accumulators are rescaled only on tiles
//    where a head's running max moved.
//  * Softmax is the online form in base 2; each warp keeps (m, l, acc) for the
//    whole launch, the CTA merges its 4 warps in shared memory and writes one
//    partial per (split, query head) for the log-sum-exp merge kernel.
#include "decode_common.cuh"

#include <cstring>
#include <mutex>

namespace b200kv {

namespace {

constexpr int kWarps = 4;
constexpr int kTile = 32;    // positions per warp tile
constexpr int kStages = 3;
constexpr int kD = 128;
constexpr uint32_t kSpinLimit = 1u << 24;

template <int NBLK>
struct Smem {
    static constexpr int kKTile = kTile * kD;              // 4096
    static constexpr int kSTile = kTile * NBLK * 2;        // 256 (q8_0) or 64 (row scale)
    static constexpr int kKBytes = kWarps * kStages * kKTile;
    static constexpr int kOffV = kKBytes;
    static constexpr int kOffKS = kOffV + kKBytes;
    static constexpr int kOffVS = kOffKS + kWarps * kStages * kSTile;
    static constexpr int kOffW = kOffVS + kWarps * kStages * kSTile;     // [warp][kTile][4] float weights
    static constexpr int kOffAlpha = kOffW + kWarps * kTile * 4 * 4;     // [warp][4] float
    static constexpr int kOffQ = kOffAlpha + kWarps * 4 * 4;             // [4][kD] int16
    static constexpr int kOffQmul = kOffQ + 4 * kD * 2;                  // [4] float
    static constexpr int kOffBar = kOffQmul + 16;                        // [warp][stage] mbarrier
    static constexpr int kTotal = kOffBar + kWarps * kStages * 8;
    static constexpr int kAlloc = kTotal + 1024;                         // slack to align the base to 1024
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: returns false if the phase did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t ok;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

__device__ __forceinline__ float2 cvt2(uint32_t x, uint32_t sel_lo, uint32_t sel_hi) {
    // bytes of x are int8+128; placed in the mantissa of 2^23 they read 8388608 + u
    float2 f;
    f.x = __uint_as_float(__byte_perm(x, 0x4B000000u, sel_lo));
    f.y = __uint_as_float(__byte_perm(x, 0x4B000000u, sel_hi));
    return __fadd2_rn(f, make_float2(-8388736.0f, -8388736.0f));
}

// G query heads per kv head (1, 2 or 4); NBLK scales per row (4 = q8_0 blocks of 32, 1 = one per row).
template <int G, int NBLK, bool Q_F16>
__global__ void __launch_bounds__(kWarps * 32, 2)
decode_q8_kernel(const __grid_constant__ DecodeParams p, const __grid_constant__ CUtensorMap kmap_single) {
    using L = Smem<NBLK>;
    constexpr int PPR = 32 / G;       // positions per Q.K round
    constexpr int ROUNDS = kTile / PPR;  // == G
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t split = blockIdx.x, kv_head = blockIdx.y, session = blockIdx.z;
    const b200kv_view& view = session_view(p, session);
    const CUtensorMap* kmap = p.views != nullptr ? &p.views[session].kmap : &kmap_single;
    uint32_t begin, end;
    resolve_range(p, session, view, &begin, &end);

    // ---- this warp's tiles ---------------------------------------------------------
    const uint32_t tile_begin = begin / kTile, tile_end = (end + kTile - 1) / kTile;
    const uint64_t total_tiles = end > begin ? tile_end - tile_begin : 0;
    const uint32_t nwarps = p.num_splits * kWarps, gw = split * kWarps + warp;
    const uint32_t t0 = tile_begin + static_cast<uint32_t>(total_tiles * gw / nwarps);
    const uint32_t t1 = tile_begin + static_cast<uint32_t>(total_tiles * (gw + 1) / nwarps);
    const int ntiles = static_cast<int>(t1 - t0);

    uint8_t* k_stage = smem + warp * kStages * L::kKTile;
    uint8_t* v_stage = smem + L::kOffV + warp * kStages * L::kKTile;
    uint8_t* ks_stage = smem + L::kOffKS + warp * kStages * L::kSTile;
    uint8_t* vs_stage = smem + L::kOffVS + warp * kStages * L::kSTile;
    float* w_tile = reinterpret_cast<float*>(smem + L::kOffW) + warp * kTile * 4;
    float* alpha_s = reinterpret_cast<float*>(smem + L::kOffAlpha) + warp * 4;
    int16_t* q16 = reinterpret_cast<int16_t*>(smem + L::kOffQ);
    float* qmul_s = reinterpret_cast<float*>(smem + L::kOffQmul);
    const uint32_t bar0 = smem_u32(smem + L::kOffBar) + warp * kStages * 8;

    const uint64_t head_row0 = static_cast<uint64_t>(kv_head) * view.capacity;
    const int8_t* v_plane = view.value_q8 + head_row0 * kD;
    const uint8_t* ks_plane = static_cast<const uint8_t*>(view.key_scales) + head_row0 * NBLK * 2;
    const uint8_t* vs_plane = static_cast<const uint8_t*>(view.value_scales) + head_row0 * NBLK * 2;

    auto issue = [&](int i) {
        const int stage = i % kStages;
        const uint32_t pos0 = (t0 + i) * kTile;
        const uint32_t rows = min(static_cast<uint32_t>(kTile), static_cast<uint32_t>(view.capacity) - pos0);
        const uint32_t bar = bar0 + stage * 8;
        mbar_expect_tx(bar, L::kKTile + rows * kD + 2 * rows * NBLK * 2);
        tma_load_2d(smem_u32(k_stage + stage * L::kKTile), kmap, 0, static_cast<int>(head_row0 + pos0), bar);
        bulk_load(smem_u32(v_stage + stage * L::kKTile), v_plane + static_cast<size_t>(pos0) * kD, rows * kD, bar);
        bulk_load(smem_u32(ks_stage + stage * L::kSTile), ks_plane + static_cast<size_t>(pos0) * NBLK * 2, rows * NBLK * 2, bar);
        bulk_load(smem_u32(vs_stage + stage * L::kSTile), vs_plane + static_cast<size_t>(pos0) * NBLK * 2, rows * NBLK * 2, bar);
    };

    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(bar0 + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int i = 0; i < kStages && i < ntiles; ++i) issue(i);   // the cache does not depend on Q: start streaming first
    }

    // ---- quantise Q to int16, one warp per head ---------------------------------------
    if (warp < G) {
        const uint32_t head = kv_head * G + warp;
        const size_t qb = (static_cast<size_t>(session) * p.query_heads + head) * kD + lane * 4;
        float q[4];
        if (Q_F16) {
            const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __half*>(p.q) + qb);
            const __half2 a = *reinterpret_cast<const __half2*>(&raw.x), b = *reinterpret_cast<const __half2*>(&raw.y);
            q[0] = __low2float(a); q[1] = __high2float(a); q[2] = __low2float(b); q[3] = __high2float(b);
        } else {
            const float4 raw = *reinterpret_cast<const float4*>(static_cast<const float*>(p.q) + qb);
            q[0] = raw.x; q[1] = raw.y; q[2] = raw.z; q[3] = raw.w;
        }
        const float amax = warp_max(fmaxf(fmaxf(fabsf(q[0]), fabsf(q[1])), fmaxf(fabsf(q[2]), fabsf(q[3]))));
        const float inv = amax > 0.0f ? 32767.0f / amax : 0.0f;
        short4 packed;
        packed.x = static_cast<short>(__float2int_rn(q[0] * inv));
        packed.y = static_cast<short>(__float2int_rn(q[1] * inv));
        packed.z = static_cast<short>(__float2int_rn(q[2] * inv));
        packed.w = static_cast<short>(__float2int_rn(q[3] * inv));
        *reinterpret_cast<short4*>(q16 + warp * kD + lane * 4) = packed;
        // scores are kept in base-2 units: dot * (amax/32767) * softmax_scale * log2(e)
        if (lane == 0) qmul_s[warp] = (amax / 32767.0f) * p.scale * 1.4426950408889634f;
    }
    __syncthreads();

    const int g = lane % G, pl = lane / G;       // Q.K role: head g of position pl (+ PPR * round)
    const int r4 = lane >> 3, c = lane & 7;      // P.V role: positions r4 + 4j, dims [16c, 16c+16)
    int qreg[kD / 2];
#pragma unroll
    for (int i = 0; i < kD / 8; ++i) {
        const uint4 t = reinterpret_cast<const uint4*>(q16 + g * kD)[i];
        qreg[4 * i] = static_cast<int>(t.x); qreg[4 * i + 1] = static_cast<int>(t.y);
        qreg[4 * i + 2] = static_cast<int>(t.z); qreg[4 * i + 3] = static_cast<int>(t.w);
    }
    const float qmul = qmul_s[g];

    float2 acc[G][8];
#pragma unroll
    for (int h = 0; h < G; ++h)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[h][k] = make_float2(0.0f, 0.0f);
    float m_run = -INFINITY, l_run = 0.0f;
    bool failed = false;

    for (int i = 0; i < ntiles; ++i) {
        const int stage = i % kStages;
        if (!mbar_wait(bar0 + stage * 8, (i / kStages) & 1)) { failed = true; break; }
        const uint32_t pos0 = (t0 + i) * kTile;
        const int lo = begin > pos0 ? static_cast<int>(begin - pos0) : 0;
        const int hi = end - pos0 < static_cast<uint32_t>(kTile) ? static_cast<int>(end - pos0) : kTile;
        const uint8_t* kt = k_stage + stage * L::kKTile;
        const uint8_t* vt = v_stage + stage * L::kKTile;
        const uint8_t* kst = ks_stage + stage * L::kSTile;
        const uint8_t* vst = vs_stage + stage * L::kSTile;

        // ---- Q.K: ROUNDS rounds of PPR positions x G heads -----------------------------
        float s[ROUNDS];
#pragma unroll
        for (int r = 0; r < ROUNDS; ++r) {
            const int pos = r * PPR + pl;
            const uint4* krow = reinterpret_cast<const uint4*>(kt + pos * kD);
            const int swz = pos & 7;
            float ksf[NBLK];
            if constexpr (NBLK == 4) {
                const uint2 raw = *reinterpret_cast<const uint2*>(kst + pos * 8);
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                ksf[0] = a.x; ksf[1] = a.y; ksf[2] = b.x; ksf[3] = b.y;
            } else {
                ksf[0] = __half2float(*reinterpret_cast<const __half*>(kst + pos * 2));
            }
            float total = 0.0f;
            int isum = 0;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
                const uint4 kw = krow[ch ^ swz];
                isum = __dp2a_lo(qreg[8 * ch + 0], static_cast<int>(kw.x), isum);
                isum = __dp2a_hi(qreg[8 * ch + 1], static_cast<int>(kw.x), isum);
                isum = __dp2a_lo(qreg[8 * ch + 2], static_cast<int>(kw.y), isum);
                isum = __dp2a_hi(qreg[8 * ch + 3], static_cast<int>(kw.y), isum);
                isum = __dp2a_lo(qreg[8 * ch + 4], static_cast<int>(kw.z), isum);
                isum = __dp2a_hi(qreg[8 * ch + 5], static_cast<int>(kw.z), isum);
                isum = __dp2a_lo(qreg[8 * ch + 6], static_cast<int>(kw.w), isum);
                isum = __dp2a_hi(qreg[8 * ch + 7], static_cast<int>(kw.w), isum);
                if constexpr (NBLK == 4) {
                    if (ch & 1) {   // a 32-dim block ends every second chunk
                        total = fmaf(static_cast<float>(isum), ksf[ch >> 1], total);
                        isum = 0;
                    }
                }
            }
            if constexpr (NBLK == 1) total = static_cast<float>(isum) * ksf[0];
            s[r] = (pos >= lo && pos < hi) ? total * qmul : -INFINITY;
        }

        // ---- online softmax (base 2) ------------------------------------------------------
        float mt = s[0];
#pragma unroll
        for (int r = 1; r < ROUNDS; ++r) mt = fmaxf(mt, s[r]);
#pragma unroll
        for (int o = G; o < 32; o <<= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
        const float m_new = fmaxf(m_run, mt);              // finite: every tile holds a valid position
        const float alpha = exp2f(m_run - m_new);
        float lsum = 0.0f;
#pragma unroll
        for (int r = 0; r < ROUNDS; ++r) {
            const float w = exp2f(s[r] - m_new);
            lsum += w;
            w_tile[(r * PPR + pl) * 4 + g] = w;
        }
        l_run = fmaf(l_run, alpha, lsum);
        m_run = m_new;
        if (pl == 0) alpha_s[g] = alpha;
        __syncwarp();

        // ---- P.V -----------------------------------------------------------------------------
        {
            float al[G];
            bool moved = false;
#pragma unroll
            for (int h = 0; h < G; ++h) { al[h] = alpha_s[h]; moved = moved || (al[h] != 1.0f); }
            if (moved) {
#pragma unroll
                for (int h = 0; h < G; ++h)
#pragma unroll
                    for (int k = 0; k < 8; ++k) { acc[h][k].x *= al[h]; acc[h][k].y *= al[h]; }
            }
        }
#pragma unroll 2
        for (int j = 0; j < kTile / 4; ++j) {
            const int pos = r4 + 4 * j;
            const uint4 vw = *reinterpret_cast<const uint4*>(vt + pos * kD + c * 16);
            const float vsf = __half2float(*reinterpret_cast<const __half*>(vst + (NBLK == 4 ? pos * 8 + (c >> 1) * 2 : pos * 2)));
            const bool valid = pos >= lo && pos < hi;
            float2 ew[G];
#pragma unroll
            for (int h = 0; h < G; ++h) {
                const float e = valid ? w_tile[pos * 4 + h] * vsf : 0.0f;   // select, not multiply: stale scales may be inf/nan
                ew[h] = make_float2(e, e);
            }
            const uint32_t words[4] = {vw.x ^ 0x80808080u, vw.y ^ 0x80808080u, vw.z ^ 0x80808080u, vw.w ^ 0x80808080u};
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const float2 f01 = cvt2(words[wi], 0x7440u, 0x7441u);
                const float2 f23 = cvt2(words[wi], 0x7442u, 0x7443u);
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    acc[h][2 * wi] = __ffma2_rn(ew[h], f01, acc[h][2 * wi]);
                    acc[h][2 * wi + 1] = __ffma2_rn(ew[h], f23, acc[h][2 * wi + 1]);
                }
            }
        }
        __syncwarp();   // every lane is done with this stage and with w_tile
        if (lane == 0 && i + kStages < ntiles) issue(i + kStages);
    }

    // ---- reduce inside the warp: acc over the 4 position groups, l over the PPR position lanes -----------
#pragma unroll
    for (int h = 0; h < G; ++h)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            acc[h][k].x += __shfl_xor_sync(0xffffffffu, acc[h][k].x, 8);
            acc[h][k].y += __shfl_xor_sync(0xffffffffu, acc[h][k].y, 8);
            acc[h][k].x += __shfl_xor_sync(0xffffffffu, acc[h][k].x, 16);
            acc[h][k].y += __shfl_xor_sync(0xffffffffu, acc[h][k].y, 16);
        }
#pragma unroll
    for (int o = G; o < 32; o <<= 1) l_run += __shfl_xor_sync(0xffffffffu, l_run, o);
    if (failed) { m_run = __int_as_float(0x7fc00000); l_run = m_run; }   // a copy never arrived: poison the partial

    // ---- merge the CTA's warps through shared memory (each warp reuses its own K ring) ---------------------
    // layout per warp: m[4], l[4], acc[G][128]
    float* mine = reinterpret_cast<float*>(k_stage);
    if (pl == 0) { mine[g] = m_run; mine[4 + g] = l_run; }
    if (r4 == 0) {
#pragma unroll
        for (int h = 0; h < G; ++h)
#pragma unroll
            for (int k = 0; k < 8; ++k)
                *reinterpret_cast<float2*>(mine + 8 + h * kD + c * 16 + 2 * k) = acc[h][k];
    }
    __syncthreads();
    {
        const int dim = threadIdx.x;   // 128 threads == 128 dims
#pragma unroll
        for (int h = 0; h < G; ++h) {
            float mw[kWarps], M = -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float* src = reinterpret_cast<const float*>(smem + w * kStages * L::kKTile);
                mw[w] = src[h];
                M = fmaxf(M, mw[w]);   // NaN-poisoned partials propagate through l below
            }
            float lt = 0.0f, at = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float* src = reinterpret_cast<const float*>(smem + w * kStages * L::kKTile);
                const float a = (mw[w] == -INFINITY) ? 0.0f : exp2f(mw[w] - M);
                lt = fmaf(src[4 + h], a, lt);
                at = fmaf(src[8 + h * kD + dim], a, at);
            }
            const uint32_t head = kv_head * G + h;
            const size_t slot = (static_cast<size_t>(session) * p.num_splits + split) * p.query_heads + head;
            p.ws_acc[slot * kD + dim] = at;
            if (dim == 0) {
                p.ws_m[slot] = M * 0.6931471805599453f;   // back to natural-log units for the merge
                p.ws_l[slot] = lt;
            }
        }
    }
}

// ---- host side -----------------------------------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encoder() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(sym);
        else
            (void)cudaGetLastError();
    });
    return fn;
}

template <int G, int NBLK, bool Q_F16>
int launch_one(const DecodeParams& p, const CUtensorMap& kmap, dim3 grid, cudaStream_t stream) {
    using L = Smem<NBLK>;
    static std::once_flag once;   // one per kernel instantiation
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(decode_q8_kernel<G, NBLK, Q_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc);
    });
    if (attr_err != cudaSuccess) { set_last_cuda_error(attr_err, "cudaFuncSetAttribute(decode_q8)"); return B200KV_ERR_CUDA; }
    decode_q8_kernel<G, NBLK, Q_F16><<<grid, kWarps * 32, L::kAlloc, stream>>>(p, kmap);
    B200KV_CUDA_TRY(cudaGetLastError());
    return B200KV_OK;
}

template <int G, int NBLK>
int launch_variant(const DecodeParams& p, const CUtensorMap& kmap, dim3 grid, cudaStream_t stream) {
    return p.q_is_f16 ? launch_one<G, NBLK, true>(p, kmap, grid, stream) : launch_one<G, NBLK, false>(p, kmap, grid, stream);
}

}  // namespace

bool q8_fast_path_ok(const b200kv_view& view, uint32_t query_heads) {
    if (view.quant_mode != B200KV_Q8_Q8 || view.head_dim != kD) return false;
    if (view.qblock != 32 && view.qblock != kD) return false;
    if (view.capacity % 8 != 0) return false;   // bulk copies of the scale planes need 16-byte aligned tile starts
    if (view.kv_heads == 0 || query_heads % view.kv_heads != 0) return false;
    const uint32_t g = query_heads / view.kv_heads;
    if (g != 1 && g != 2 && g != 4) return false;
    if (static_cast<uint64_t>(view.kv_heads) * view.capacity > 0x7fffffffull) return false;  // TMA row coordinate is int32
    return encoder() != nullptr;
}

int encode_k_map(const b200kv_view& view, CUtensorMap* out) {
    EncodeFn fn = encoder();
    if (fn == nullptr) return B200KV_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {kD, static_cast<cuuint64_t>(view.kv_heads) * view.capacity};
    const cuuint64_t strides[1] = {kD};
    const cuuint32_t box[2] = {kD, kTile};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, view.key_q8, dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? B200KV_OK : B200KV_ERR_UNSUPPORTED;
}

uint32_t pick_splits_q8(const b200kv_view& geometry, uint32_t query_heads, uint32_t sessions, uint32_t max_length) {
    if (!q8_fast_path_ok(geometry, query_heads)) return 0;
    // two CTAs of 4 warps per SM; every warp should see at least two tiles
    const uint32_t ctas = 148u * 2u;
    const uint32_t units = geometry.kv_heads * sessions;
    uint32_t s = (ctas + units / 2) / units;   // nearest to one full wave
    if (s == 0) s = 1;
    const uint32_t tiles = (max_length + kTile - 1) / kTile;
    uint32_t by_tiles = tiles / (2 * kWarps);
    if (by_tiles == 0) by_tiles = 1;
    if (s > by_tiles) s = by_tiles;
    const uint32_t cap = max_splits_per_session(sessions);
    if (s > cap) s = cap;
    return s ? s : 1;
}

int launch_decode_q8(const DecodeParams& p, const b200kv_view& geometry, uint32_t /*max_length*/, cudaStream_t stream) {
    if (!q8_fast_path_ok(geometry, p.query_heads)) return B200KV_ERR_UNSUPPORTED;
    CUtensorMap kmap;
    if (p.views == nullptr) {
        int rc = encode_k_map(geometry, &kmap);
        if (rc != B200KV_OK) return rc;
    } else {
        std::memset(&kmap, 0, sizeof kmap);   // per-session descriptors come from the device table
    }
    const uint32_t g = p.query_heads / geometry.kv_heads;
    const bool blocks = geometry.qblock == 32;
    dim3 grid(p.num_splits, geometry.kv_heads, p.sessions);
    switch (g) {
        case 1: return blocks ? launch_variant<1, 4>(p, kmap, grid, stream) : launch_variant<1, 1>(p, kmap, grid, stream);
        case 2: return blocks ? launch_variant<2, 4>(p, kmap, grid, stream) : launch_variant<2, 1>(p, kmap, grid, stream);
        default: return blocks ? launch_variant<4, 4>(p, kmap, grid, stream) : launch_variant<4, 1>(p, kmap, grid, stream);
    }
}

}  // namespace b200kv
