// Streaming split-K GQA decode attention over an int8 (q8_0 or row-scaled) KV
// cache, head_dim 128 -- the kernel the decode benchmark runs.
//
// What it computes is MIInfer's decode stage 1
// (gfx906/kernels/qwen3_primitives.hip:7371-7485) with block scales; how it is
// laid out is specific to B200:
//
//  * One CTA = one (kv head, split) = 4 warp PAIRS.  ALL query heads of the
//    kv-head group share every K/V byte the CTA loads (the reference re-reads
//    the cache once per query head).
//  * A pair is a K-warp and a V-warp working on the same sequence of
//    32-position tiles.  The K-warp streams K tiles and block scales, computes
//    the scores and the online softmax and hands (weights, rescale factors) to
//    its V-warp through a 4-slot ring in shared memory; the V-warp streams V
//    tiles and accumulates P.V.  Splitting the roles halves the registers each
//    warp needs (Q lives only in K-warps, the output accumulators only in
//    V-warps), so 16 warps are resident per SM instead of 8, and the integer
//    (Q.K) and floating-point (P.V) instruction streams of different warps
//    interleave on each scheduler.
//  * Every warp owns a private 3-stage ring of tiles filled by TMA: the K tile
//    through a tensor map with the 128-byte swizzle (rows of 128 int8), V and
//    both scale tiles with plain bulk copies.  One lane issues the copies;
//    completion is an mbarrier per stage.  Pairs never synchronise with each
//    other in the main loop; the hand-off inside a pair is two mbarriers per slot.
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
//    of 2^23 and one packed multiply-add that removes the offset (the conversion
//    pipe is 8x slower than that), the multiply-adds as packed f32x2.  Folding
//    the offset into a per-block bias that is subtracted once per launch was
//    measured: 2% faster, 10x less accurate (1.5e-4), so it is not used.
//    Accumulators are rescaled only on tiles where a head's running max moved.
//  * Softmax is the online form in base 2; each pair keeps (m, l, acc) for the
//    whole launch, the CTA merges its 4 pairs in shared memory and writes one
//    partial per (split, query head) for the log-sum-exp merge kernel.
//  * Every wait is bounded: a copy or hand-off that never arrives poisons the
//    partial with NaN instead of hanging the GPU.
#include "append_row.cuh"
#include "decode_common.cuh"

#include <cstring>
#include <mutex>

namespace b200kv {

namespace {

constexpr int kPairs = 4;     // warp pairs per CTA: warps 0..3 are K-warps, 4..7 their V-warps
constexpr int kTile = 32;     // positions per tile
constexpr int kKStages = 3;   // TMA ring depth of a K-warp (K tile + both scale tiles)
constexpr int kVStages = 2;   // TMA ring depth of a V-warp (V tile)
constexpr int kSlots = 2;     // weight hand-off ring depth per pair
constexpr int kD = 128;
constexpr uint32_t kSpinLimit = 1u << 20;   // bounded waits: a lost copy or hand-off ends the kernel with a poisoned partial
constexpr uint32_t kPositionsPerSplit = 2048;   // batched launches: one split per this many positions of a session
#ifndef B200KV_PV_UNROLL
#define B200KV_PV_UNROLL 2
#endif
constexpr int kPvUnroll = B200KV_PV_UNROLL;   // positions of the P.V loop in flight per lane

template <int NBLK>
struct Smem {
    static constexpr int kKTile = kTile * kD;                    // 4096
    static constexpr int kSTile = kTile * NBLK * 2;              // 256 (q8_0) or 64 (row scale)
    static constexpr int kBlkStride = kTile * 4 * 4 + 64;          // ew[pos][head] fp32 of one block, padded against bank conflicts
    static constexpr int kSlotBytes = NBLK * kBlkStride + 16;      // ew[blk][pos][head] + alpha[4]
    static constexpr int kOffV = kPairs * kKStages * kKTile;
    static constexpr int kOffS = kOffV + kPairs * kVStages * kKTile;     // [pair][stage][ks | vs]
    static constexpr int kOffW = kOffS + kPairs * kKStages * 2 * kSTile;
    static constexpr int kOffQ = kOffW + kPairs * kSlots * kSlotBytes;   // [4][kD] int16
    static constexpr int kOffQmul = kOffQ + 4 * kD * 2;                  // [4] float
    static constexpr int kOffMisc = kOffQmul + 16;                       // merge scratch: m/l/a [4][128] floats x3
    static constexpr int kOffBar = kOffMisc + 3 * 4 * 128 * 4;
    static constexpr int kBarsPerPair = kKStages + kVStages + 2 * kSlots;  // kfull, vfull, wfull, wempty
    static constexpr int kTotal = kOffBar + kPairs * kBarsPerPair * 8;
    static constexpr int kAlloc = kTotal + 1024;                         // slack to align the base to 1024
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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

// Two int8 bytes of x (already offset by +128) to fp32: placed in the mantissa of
// 2^23 they read 8388608 + u; one packed multiply-add removes the offset.
__device__ __forceinline__ float2 cvt2(uint32_t x, uint32_t sel_lo, uint32_t sel_hi) {
    float2 f;
    f.x = __uint_as_float(__byte_perm(x, 0x4B000000u, sel_lo));
    f.y = __uint_as_float(__byte_perm(x, 0x4B000000u, sel_hi));
    return __ffma2_rn(f, make_float2(1.0f, 1.0f), make_float2(-8388736.0f, -8388736.0f));
}

// ---- fused single-token append -----------------------------------------------------------------------------
// Kept out of line so the rarely-taken path does not widen the register allocation of the streaming loops.
// Loads the new row of `kv_head` (lane L: elements L, L+32, L+64, L+96).
__device__ __noinline__ void load_new_row(const void* src, int is_f16, uint32_t kv_head, int lane, float (&x)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const size_t i = static_cast<size_t>(kv_head) * kD + lane + 32 * j;
        x[j] = is_f16 ? __half2float(static_cast<const __half*>(src)[i]) : static_cast<const float*>(src)[i];
    }
}

// Quantises the new K and V rows of `kv_head` and stores them (int8 + fp16 block scales) at cache row `row_index`.
template <int NBLK>
__device__ __noinline__ void fused_append_row(const DecodeParams& p, const b200kv_view& view, uint32_t kv_head, uint32_t position,
                                              uint64_t row_index, int lane) {
    float k[4], v[4];
    load_new_row(p.new_key, p.new_is_f16, kv_head, lane, k);
    load_new_row(p.new_value, p.new_is_f16, kv_head, lane, v);
    transform_k_row<kD>(k, lane, position, p.k_norm_weight, p.epsilon, p.rope_mode, p.inv_freq, p.sectioned_step);
    int8_t kq[4], vq[4];
    float ksc[4], vsc[4];
    quantize_row<4>(k, NBLK == 1, kq, ksc);
    quantize_row<4>(v, NBLK == 1, vq, vsc);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        view.key_q8[row_index * kD + lane + 32 * j] = kq[j];
        view.value_q8[row_index * kD + lane + 32 * j] = vq[j];
    }
    if (lane < NBLK) {
        static_cast<__half*>(view.key_scales)[row_index * NBLK + lane] = __float2half_rn(ksc[NBLK == 1 ? 0 : lane]);
        static_cast<__half*>(view.value_scales)[row_index * NBLK + lane] = __float2half_rn(vsc[NBLK == 1 ? 0 : lane]);
    }
}

// G query heads per kv head (1, 2 or 4); NBLK scales per row (4 = q8_0 blocks of 32, 1 = one per row).
template <int G, int NBLK, bool Q_F16>
__global__ void __launch_bounds__(kPairs * 64, 2)
decode_q8_kernel(const __grid_constant__ DecodeParams p, const __grid_constant__ CUtensorMap kmap_single) {
    using L = Smem<NBLK>;
    constexpr int PPR = 32 / G;          // positions per Q.K round
    constexpr int ROUNDS = kTile / PPR;  // == G
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    __shared__ int s_last;

    pdl_launch_dependents();   // the next kernel of the stream may become resident as SMs free up; it orders itself

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pair = warp & (kPairs - 1);
    const bool is_k_warp = warp < kPairs;
    const uint32_t split = blockIdx.x, kv_head = blockIdx.y, session = blockIdx.z;
    const b200kv_view& view = session_view(p, session);
    uint32_t begin, end;
    resolve_range(p, session, view, &begin, &end);

    // Batched launches size the grid for the longest session; a shorter session uses only as many splits as its
    // own length warrants (every CTA of the session derives the same number) and the surplus CTAs leave at once.
    uint32_t num_splits = p.num_splits;
    if (p.lengths != nullptr) {
        const uint32_t want = (end - begin + kPositionsPerSplit - 1) / kPositionsPerSplit;
        num_splits = min(num_splits, max(want, 1u));
        if (split >= num_splits) return;
    }

    // ---- this pair's tiles -----------------------------------------------------------
    const uint32_t tile_begin = begin / kTile, tile_end = (end + kTile - 1) / kTile;
    const uint64_t total_tiles = end > begin ? tile_end - tile_begin : 0;
    const uint32_t npairs = num_splits * kPairs, gp = split * kPairs + pair;
    // A fused append costs its pair about one tile's time: it is counted as one extra unit at the end of the range,
    // so the pair that does it is handed one tile less.
    const bool fuse = p.new_key != nullptr;
    const uint64_t units = total_tiles + (fuse ? 1 : 0);
    const uint64_t u0 = units * gp / npairs, u1 = units * (gp + 1) / npairs;
    const uint32_t t0 = tile_begin + static_cast<uint32_t>(u0 < total_tiles ? u0 : total_tiles);
    const uint32_t t1 = tile_begin + static_cast<uint32_t>(u1 < total_tiles ? u1 : total_tiles);
    const int ntiles = static_cast<int>(t1 - t0);
    const bool owner = fuse && ntiles > 0 && t1 == tile_end;   // this pair holds the tile of the appended token
    // With launch overlap the previous kernel may still be appending: rows at or above early_end wait for it.  The
    // row a fused append writes is never loaded early either.
    uint32_t early_end = end > p.overlap_tail ? end - p.overlap_tail : 0;
    if (fuse && early_end >= end) early_end = end - 1;

    uint8_t* k_ring = smem + pair * kKStages * L::kKTile;
    uint8_t* v_ring = smem + L::kOffV + pair * kVStages * L::kKTile;
    uint8_t* s_ring = smem + L::kOffS + pair * kKStages * 2 * L::kSTile;
    uint8_t* w_ring = smem + L::kOffW + pair * kSlots * L::kSlotBytes;
    int16_t* q16 = reinterpret_cast<int16_t*>(smem + L::kOffQ);
    float* qmul_s = reinterpret_cast<float*>(smem + L::kOffQmul);
    const uint32_t bars = smem_u32(smem + L::kOffBar) + pair * L::kBarsPerPair * 8;
    const uint32_t bar_kfull = bars, bar_vfull = bars + kKStages * 8;
    const uint32_t bar_wfull = bar_vfull + kVStages * 8, bar_wempty = bar_wfull + kSlots * 8;

    const uint64_t head_row0 = static_cast<uint64_t>(kv_head) * view.capacity;

    // barriers of a pair are initialised by its K-warp before either warp uses them
    if (is_k_warp && lane == 0) {
        for (int s = 0; s < L::kBarsPerPair; ++s) mbar_init(bars + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    bool failed = false;
    // merge area of the pair (reuses its K ring once the main loop is over): m[4], l[4], pad[24], acc[G][128]
    float* mine = reinterpret_cast<float*>(k_ring);

    if (is_k_warp) {
        // =========================== K-warp: scores, softmax, weights ===========================
        const CUtensorMap* kmap = p.views != nullptr ? &p.views[session].kmap : &kmap_single;
        const uint8_t* ks_plane = static_cast<const uint8_t*>(view.key_scales) + head_row0 * NBLK * 2;
        const uint8_t* vs_plane = static_cast<const uint8_t*>(view.value_scales) + head_row0 * NBLK * 2;
        auto issue = [&](int i) {
            const int stage = i % kKStages;
            const uint32_t pos0 = (t0 + i) * kTile;
            const uint32_t rows = min(static_cast<uint32_t>(kTile), static_cast<uint32_t>(view.capacity) - pos0);
            const uint32_t bar = bar_kfull + stage * 8;
            mbar_expect_tx(bar, L::kKTile + 2 * rows * NBLK * 2);
            tma_load_2d(smem_u32(k_ring + stage * L::kKTile), kmap, 0, static_cast<int>(head_row0 + pos0), bar);
            uint8_t* sdst = s_ring + stage * 2 * L::kSTile;
            bulk_load(smem_u32(sdst), ks_plane + static_cast<size_t>(pos0) * NBLK * 2, rows * NBLK * 2, bar);
            bulk_load(smem_u32(sdst + L::kSTile), vs_plane + static_cast<size_t>(pos0) * NBLK * 2, rows * NBLK * 2, bar);
        };
        // old cache rows do not depend on the preceding kernels: start streaming them before waiting for those
        int issued = 0;
        if (lane == 0)
            while (issued < kKStages && issued < ntiles && (t0 + issued + 1) * kTile <= early_end) issue(issued++);
        pdl_wait();
        if (owner) {
            // the new row goes to the cache first; its tile is loaded (by TMA, an asynchronous-proxy read) only afterwards
            fused_append_row<NBLK>(p, view, kv_head, end - 1, head_row0 + end - 1, lane);
            __threadfence();
            asm volatile("fence.proxy.async;" ::: "memory");
            // arrive without waiting: the V-warp joins this barrier only before its LAST tile, long after it has
            // consumed weights this warp still has to produce
            asm volatile("bar.arrive %0, 64;" ::"r"(2 + pair) : "memory");
        }
        if (lane == 0)
            while (issued < kKStages && issued < ntiles) issue(issued++);

        // quantise Q to int16, one K-warp per head
        if (pair < G) {
            const uint32_t head = kv_head * G + pair;
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
            *reinterpret_cast<short4*>(q16 + pair * kD + lane * 4) = packed;
            // scores are kept in base-2 units: dot * (amax/32767) * softmax_scale * log2(e)
            if (lane == 0) qmul_s[pair] = (amax / 32767.0f) * p.scale * 1.4426950408889634f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kPairs * 32) : "memory");   // K-warps only

        const int g = lane % G, pl = lane / G;   // head g of position pl (+ PPR * round)
        int qreg[kD / 2];
#pragma unroll
        for (int i = 0; i < kD / 8; ++i) {
            const uint4 t = reinterpret_cast<const uint4*>(q16 + g * kD)[i];
            qreg[4 * i] = static_cast<int>(t.x); qreg[4 * i + 1] = static_cast<int>(t.y);
            qreg[4 * i + 2] = static_cast<int>(t.z); qreg[4 * i + 3] = static_cast<int>(t.w);
        }
        const float qmul = qmul_s[g];
        float m_run = -INFINITY, l_run = 0.0f;
        // per-lane byte offsets that do not change from tile to tile
        // byte offset of logical 16-byte chunk ch of this lane's row in round 0; the 128-byte swizzle stores it
        // at chunk (ch ^ (row & 7)), and row & 7 == pl & 7 in every round (PPR is a multiple of 8, or pl < 8)
        uint32_t koff[8];
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) koff[ch] = static_cast<uint32_t>(pl) * kD + (static_cast<uint32_t>(ch ^ (pl & 7)) << 4);
        const uint32_t s_lane = static_cast<uint32_t>(pl) * NBLK * 2;
        const uint32_t w_lane = static_cast<uint32_t>(pl * 4 + g) * 4;

        for (int i = 0; i < ntiles; ++i) {
            const int stage = i % kKStages, slot = i % kSlots;
            if (!mbar_wait(bar_kfull + stage * 8, (i / kKStages) & 1)) { failed = true; break; }
            const uint32_t pos0 = (t0 + i) * kTile;
            const int lo = begin > pos0 ? static_cast<int>(begin - pos0) : 0;
            const int hi = end - pos0 < static_cast<uint32_t>(kTile) ? static_cast<int>(end - pos0) : kTile;
            const uint8_t* kt = k_ring + stage * L::kKTile;
            const uint8_t* kst = s_ring + stage * 2 * L::kSTile + s_lane;

            float s[ROUNDS];
#ifdef B200KV_SKIP_QK
#pragma unroll
            for (int r = 0; r < ROUNDS; ++r) s[r] = static_cast<float>(kt[r * 16] + qreg[r]) * qmul;
#else
#pragma unroll
            for (int r = 0; r < ROUNDS; ++r) {
                const uint8_t* krow = kt + r * PPR * kD;
                float ksf[NBLK];
                if constexpr (NBLK == 4) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(kst + r * PPR * 8);
                    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    ksf[0] = a.x; ksf[1] = a.y; ksf[2] = b.x; ksf[3] = b.y;
                } else {
                    ksf[0] = __half2float(*reinterpret_cast<const __half*>(kst + r * PPR * 2));
                }
                float total = 0.0f;
                int isum0 = 0, isum1 = 0;
#pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    const uint4 kw = *reinterpret_cast<const uint4*>(krow + koff[ch]);
                    isum0 = __dp2a_lo(qreg[8 * ch + 0], static_cast<int>(kw.x), isum0);
                    isum1 = __dp2a_hi(qreg[8 * ch + 1], static_cast<int>(kw.x), isum1);
                    isum0 = __dp2a_lo(qreg[8 * ch + 2], static_cast<int>(kw.y), isum0);
                    isum1 = __dp2a_hi(qreg[8 * ch + 3], static_cast<int>(kw.y), isum1);
                    isum0 = __dp2a_lo(qreg[8 * ch + 4], static_cast<int>(kw.z), isum0);
                    isum1 = __dp2a_hi(qreg[8 * ch + 5], static_cast<int>(kw.z), isum1);
                    isum0 = __dp2a_lo(qreg[8 * ch + 6], static_cast<int>(kw.w), isum0);
                    isum1 = __dp2a_hi(qreg[8 * ch + 7], static_cast<int>(kw.w), isum1);
                    if constexpr (NBLK == 4) {
                        if (ch & 1) {   // a 32-dim block ends every second chunk
                            total = fmaf(static_cast<float>(isum0 + isum1), ksf[ch >> 1], total);
                            isum0 = 0; isum1 = 0;
                        }
                    }
                }
                if constexpr (NBLK == 1) total = static_cast<float>(isum0 + isum1) * ksf[0];
                const int pos = r * PPR + pl;
                s[r] = (pos >= lo && pos < hi) ? total * qmul : -INFINITY;
            }
#endif

            // online softmax, base 2
            float mt = s[0];
#pragma unroll
            for (int r = 1; r < ROUNDS; ++r) mt = fmaxf(mt, s[r]);
#pragma unroll
            for (int o = G; o < 32; o <<= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
            const float m_new = fmaxf(m_run, mt);              // finite: every tile holds a valid position
            const float alpha = exp2f(m_run - m_new);
            float w[ROUNDS], lsum = 0.0f;
#pragma unroll
            for (int r = 0; r < ROUNDS; ++r) { w[r] = exp2f(s[r] - m_new); lsum += w[r]; }
            l_run = fmaf(l_run, alpha, lsum);
            m_run = m_new;

            // effective weights w * value_scale[block] for the V-warp: ew[blk][pos][head]
            if (!mbar_wait(bar_wempty + slot * 8, ((i / kSlots) & 1) ^ 1)) { failed = true; break; }
            uint8_t* wt = w_ring + slot * L::kSlotBytes;
            const uint8_t* vst = kst + L::kSTile;
#pragma unroll
            for (int r = 0; r < ROUNDS; ++r) {
                const bool valid = w[r] > 0.0f;   // masked positions have weight exactly 0; their scales may be stale inf/nan
                if constexpr (NBLK == 4) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(vst + r * PPR * 8);
                    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    float* dst = reinterpret_cast<float*>(wt + w_lane + r * PPR * 16);
                    const float e0 = valid ? w[r] * a.x : 0.0f, e1 = valid ? w[r] * a.y : 0.0f;
                    const float e2 = valid ? w[r] * b.x : 0.0f, e3 = valid ? w[r] * b.y : 0.0f;
                    dst[0 * L::kBlkStride / 4] = e0; dst[1 * L::kBlkStride / 4] = e1;
                    dst[2 * L::kBlkStride / 4] = e2; dst[3 * L::kBlkStride / 4] = e3;

                } else {
                    const float v = __half2float(*reinterpret_cast<const __half*>(vst + r * PPR * 2));
                    const float e0 = valid ? w[r] * v : 0.0f;
                    *reinterpret_cast<float*>(wt + w_lane + r * PPR * 16) = e0;
                }
            }
            if (pl == 0) reinterpret_cast<float*>(wt + NBLK * L::kBlkStride)[g] = alpha;
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_wfull + slot * 8);
                if (i + kKStages < ntiles) issue(i + kKStages);
            }
        }
#pragma unroll
        for (int o = G; o < 32; o <<= 1) l_run += __shfl_xor_sync(0xffffffffu, l_run, o);
        if (failed) { m_run = __int_as_float(0x7fc00000); l_run = m_run; }   // poison the partial
        if (pl == 0) { mine[g] = m_run; mine[4 + g] = l_run; }
    } else {
        // =========================== V-warp: P.V accumulation ============================
        const int8_t* v_plane = view.value_q8 + head_row0 * kD;
        auto issue = [&](int i) {
            const int stage = i % kVStages;
            const uint32_t pos0 = (t0 + i) * kTile;
            const uint32_t rows = min(static_cast<uint32_t>(kTile), static_cast<uint32_t>(view.capacity) - pos0);
            const uint32_t bar = bar_vfull + stage * 8;
            mbar_expect_tx(bar, rows * kD);
            bulk_load(smem_u32(v_ring + stage * L::kKTile), v_plane + static_cast<size_t>(pos0) * kD, rows * kD, bar);
        };
        int issued = 0;   // kept identical in all lanes: the hand-shake below is warp-wide
        while (issued < kVStages && issued < ntiles && (t0 + issued + 1) * kTile <= early_end) {
            if (lane == 0) issue(issued);
            ++issued;
        }
        pdl_wait();
        while (issued < kVStages && issued < ntiles) {
            // the tile of a fused append is loaded only after the K-warp has stored the new row
            if (owner && issued == ntiles - 1) asm volatile("bar.sync %0, 64;" ::"r"(2 + pair) : "memory");
            if (lane == 0) issue(issued);
            ++issued;
        }

        const int r4 = lane >> 3, c = lane & 7;   // positions r4 + 4j, dims [16c, 16c+16)
        const uint32_t v_lane = static_cast<uint32_t>(r4) * kD + c * 16;
        const uint32_t w_lane = static_cast<uint32_t>(NBLK == 4 ? (c >> 1) : 0) * L::kBlkStride + r4 * 16;
        float2 acc[G][8];
#pragma unroll
        for (int h = 0; h < G; ++h)
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[h][k] = make_float2(0.0f, 0.0f);

        for (int i = 0; i < ntiles; ++i) {
            const int stage = i % kVStages, slot = i % kSlots;
            if (!mbar_wait(bar_vfull + stage * 8, (i / kVStages) & 1)) { failed = true; break; }
            if (!mbar_wait(bar_wfull + slot * 8, (i / kSlots) & 1)) { failed = true; break; }
            const uint8_t* vt = v_ring + stage * L::kKTile + v_lane;
            const uint8_t* wt = w_ring + slot * L::kSlotBytes;
            {
                float al[4];
                *reinterpret_cast<float4*>(al) = *reinterpret_cast<const float4*>(wt + NBLK * L::kBlkStride);
                bool moved = false;
#pragma unroll
                for (int h = 0; h < G; ++h) moved = moved || (al[h] != 1.0f);
                if (moved) {
#pragma unroll
                    for (int h = 0; h < G; ++h) {
                        const float2 a2 = make_float2(al[h], al[h]);
#pragma unroll
                        for (int k = 0; k < 8; ++k) acc[h][k] = __fmul2_rn(acc[h][k], a2);
                    }
                }
            }
            const uint8_t* wl = wt + w_lane;
#ifdef B200KV_SKIP_PV
            acc[0][0].x += static_cast<float>(vt[0]) * wl[0];
#else
#pragma unroll kPvUnroll
            for (int j = 0; j < kTile / 4; ++j) {
                const uint4 vw = *reinterpret_cast<const uint4*>(vt + j * 4 * kD);
                float wv[4];
                *reinterpret_cast<float4*>(wv) = *reinterpret_cast<const float4*>(wl + j * 64);
                float2 ew[G];
#pragma unroll
                for (int h = 0; h < G; ++h) ew[h] = make_float2(wv[h], wv[h]);
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
#endif
            __syncwarp();   // every lane is done with this stage and this weight slot
            if (owner && i + kVStages == ntiles - 1) asm volatile("bar.sync %0, 64;" ::"r"(2 + pair) : "memory");
            if (lane == 0) {
                mbar_arrive(bar_wempty + slot * 8);
                if (i + kVStages < ntiles) issue(i + kVStages);
            }
        }
        // sum the 4 position groups
#pragma unroll
        for (int h = 0; h < G; ++h)
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                acc[h][k].x += __shfl_xor_sync(0xffffffffu, acc[h][k].x, 8);
                acc[h][k].y += __shfl_xor_sync(0xffffffffu, acc[h][k].y, 8);
                acc[h][k].x += __shfl_xor_sync(0xffffffffu, acc[h][k].x, 16);
                acc[h][k].y += __shfl_xor_sync(0xffffffffu, acc[h][k].y, 16);
            }
        if (failed) acc[0][0].x = __int_as_float(0x7fc00000);
        // the K-warp of this pair is past its last K tile once the last weights have arrived
        if (r4 == 0) {
#pragma unroll
            for (int h = 0; h < G; ++h)
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    *reinterpret_cast<float2*>(mine + 32 + h * kD + c * 16 + 2 * k) = acc[h][k];
        }
    }
    __syncthreads();

    // ---- merge the CTA's pairs: 256 threads = 2 head slots x 128 dims ---------------------------------------
    const int dim = threadIdx.x & (kD - 1);
    for (int h = threadIdx.x >> 7; h < G; h += 2) {
        float mw[kPairs], M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kPairs; ++w) {
            const float* src = reinterpret_cast<const float*>(smem + w * kKStages * L::kKTile);
            mw[w] = src[h];
            M = fmaxf(M, mw[w]);
        }
        float lt = 0.0f, at = 0.0f;
#pragma unroll
        for (int w = 0; w < kPairs; ++w) {
            const float* src = reinterpret_cast<const float*>(smem + w * kKStages * L::kKTile);
            const float a = (mw[w] == -INFINITY) ? 0.0f : exp2f(mw[w] - M);   // NaN (poison) propagates
            lt = fmaf(src[4 + h], a, lt);
            at = fmaf(src[32 + h * kD + dim], a, at);
        }
        const uint32_t head = kv_head * G + h;
        const size_t slot_idx = (static_cast<size_t>(session) * p.num_splits + split) * p.query_heads + head;
        p.ws_acc[slot_idx * kD + dim] = at;
        if (dim == 0) {
            p.ws_m[slot_idx] = M * 0.6931471805599453f;   // natural-log units, as the merge kernel expects
            p.ws_l[slot_idx] = lt;
        }
    }
    if (p.counters == nullptr) return;   // a separate merge kernel follows

    // ---- the last CTA of this (session, kv head) to finish merges all splits -------------------------------------
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t prev = atomicAdd(p.counters + session * gridDim.y + kv_head, 1u);
        s_last = (prev + 1 == num_splits);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const uint32_t S = num_splits;     // <= kMaxSplitsPerSession == 128; the partial arrays keep the launch-wide stride
    float* sm = reinterpret_cast<float*>(smem + L::kOffMisc);   // [4][128] m -> a
    float* sl = sm + 4 * 128;                                   // [4][128] l
    float* sg = sl + 4 * 128;                                   // [4] merged max, [4] merged sum
    for (uint32_t idx = threadIdx.x; idx < G * S; idx += blockDim.x) {
        const uint32_t h = idx / S, sp = idx % S;
        const size_t slot_idx = (static_cast<size_t>(session) * p.num_splits + sp) * p.query_heads + kv_head * G + h;
        sm[h * 128 + sp] = __ldcg(p.ws_m + slot_idx);
        sl[h * 128 + sp] = __ldcg(p.ws_l + slot_idx);
    }
    __syncthreads();
    if (warp < G) {   // one warp per head: global max, rescale factors, merged sum
        const int h = warp;
        float M = -INFINITY;
        for (uint32_t sp = lane; sp < S; sp += 32) {
            const float m = sm[h * 128 + sp], l = sl[h * 128 + sp];
            if (!(l <= 0.0f) && m != -INFINITY) M = fmaxf(M, m);   // keeps NaN partials in play
        }
        M = warp_max(M);
        float lsum = 0.0f;
        for (uint32_t sp = lane; sp < S; sp += 32) {
            const float m = sm[h * 128 + sp], l = sl[h * 128 + sp];
            const float a = (!(l <= 0.0f) && m != -INFINITY) ? __expf(m - M) : 0.0f;
            sm[h * 128 + sp] = a;
            lsum = fmaf(l, a, lsum);
        }
        lsum = warp_sum(lsum);
        if (lane == 0) { sg[h] = M; sg[4 + h] = lsum; }
    }
    __syncthreads();
    // 256 threads = 4 heads x 2 halves of the splits x 32 float4 columns: each thread issues its loads
    // in batches of 10 -- warps issue in order, so a loop of dependent load/use pairs would pay the L2 latency per step
    {
        const int col = threadIdx.x & 31, part = (threadIdx.x >> 5) & 1, h = threadIdx.x >> 6;
        float4 tot = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (h < G) {
            const uint32_t head = kv_head * G + h;
            const size_t stride = static_cast<size_t>(p.query_heads) * kD;
            const float* accp = p.ws_acc + ((static_cast<size_t>(session) * p.num_splits) * p.query_heads + head) * kD + col * 4;
            for (uint32_t sp0 = part; sp0 < S; sp0 += 20) {
                float4 v[10];
#pragma unroll
                for (int u = 0; u < 10; ++u) {
                    const uint32_t sp = sp0 + 2 * u;
                    v[u] = sp < S ? __ldcg(reinterpret_cast<const float4*>(accp + sp * stride)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
#pragma unroll
                for (int u = 0; u < 10; ++u) {
                    const uint32_t sp = sp0 + 2 * u;
                    const float a = sp < S ? sm[h * 128 + sp] : 0.0f;
                    tot.x = fmaf(v[u].x, a, tot.x); tot.y = fmaf(v[u].y, a, tot.y);
                    tot.z = fmaf(v[u].z, a, tot.z); tot.w = fmaf(v[u].w, a, tot.w);
                }
            }
        }
        // fold the two halves through shared memory (the pairs' merge areas are free by now)
        float4* fold = reinterpret_cast<float4*>(smem);
        if (part == 1) fold[h * 32 + col] = tot;
        __syncthreads();
        if (part == 0 && h < G) {
            const float4 o2 = fold[h * 32 + col];
            tot.x += o2.x; tot.y += o2.y; tot.z += o2.z; tot.w += o2.w;
            const uint32_t head = kv_head * G + h;
            const float gsum = sg[4 + h];
            const size_t out_idx = (static_cast<size_t>(session) * p.query_heads + head) * kD + col * 4;
            if (p.fuse.out_m != nullptr) {   // sequence shard: one merged, unnormalised partial
                *reinterpret_cast<float4*>(p.fuse.out_acc + out_idx) = tot;
                if (col == 0) {
                    p.fuse.out_m[static_cast<size_t>(session) * p.query_heads + head] = sg[h];
                    p.fuse.out_l[static_cast<size_t>(session) * p.query_heads + head] = gsum;
                }
            } else {
                const float inv = gsum > 0.0f ? 1.0f / gsum : (gsum == gsum ? 0.0f : gsum);
                float4 o = make_float4(tot.x * inv, tot.y * inv, tot.z * inv, tot.w * inv);
                if (p.fuse.output != nullptr) *reinterpret_cast<float4*>(p.fuse.output + out_idx) = o;
                if (p.fuse.gated_output != nullptr) {
                    if (p.fuse.gate != nullptr) {
                        const float4 gt = *reinterpret_cast<const float4*>(p.fuse.gate + out_idx);
                        o.x *= 1.0f / (1.0f + __expf(-gt.x)); o.y *= 1.0f / (1.0f + __expf(-gt.y));
                        o.z *= 1.0f / (1.0f + __expf(-gt.z)); o.w *= 1.0f / (1.0f + __expf(-gt.w));
                    }
                    *reinterpret_cast<float4*>(p.fuse.gated_output + out_idx) = o;
                }
            }
        }
    }
    if (threadIdx.x == 0) p.counters[session * gridDim.y + kv_head] = 0;   // leave the workspace ready for the next launch
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
    B200KV_CUDA_TRY(launch_kernel(decode_q8_kernel<G, NBLK, Q_F16>, grid, dim3(kPairs * 64), L::kAlloc, stream, true, p, kmap));
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
    // two CTAs of 4 warp pairs per SM; every pair should see at least two tiles
    const uint32_t ctas = 148u * 2u;
    const uint32_t units = geometry.kv_heads * sessions;
    uint32_t s = (ctas + units / 2) / units;   // nearest to one full wave
    if (s == 0) s = 1;
    if (sessions > 1) {   // mixed lengths: enough splits that the longest session is cut into kPositionsPerSplit pieces
        const uint32_t by_length = (max_length + kPositionsPerSplit - 1) / kPositionsPerSplit;
        if (by_length > s) s = by_length;
    }
    const uint32_t tiles = (max_length + kTile - 1) / kTile;
    uint32_t by_tiles = tiles / (2 * kPairs);
    if (by_tiles == 0) by_tiles = 1;
    if (s > by_tiles) s = by_tiles;
    const uint32_t cap = max_splits_per_session(sessions);
    if (s > cap) s = cap;
    return s ? s : 1;
}

int launch_decode_q8(const DecodeParams& p_in, const b200kv_view& geometry, uint32_t /*max_length*/, cudaStream_t stream) {
    if (!q8_fast_path_ok(geometry, p_in.query_heads)) return B200KV_ERR_UNSUPPORTED;
    DecodeParams p = p_in;
    p.overlap_tail = launch_overlap_tail();
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
