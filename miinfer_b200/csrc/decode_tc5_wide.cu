// Streaming split-K GQA decode attention for head_dim 256 (MIInfer's own geometry: 24 query heads over 4 kv heads,
// gfx906/kernels/qwen3_primitives.hip:7371-7485) on the 5th-generation tensor cores: the design of decode_tc5.cu --
// tcgen05.mma kind::i8 straight from the TMA-filled tiles, accumulators in TMEM, the cache bytes never in a register --
// widened to 8 blocks of 32 dims and up to 8 query heads per kv head.  Differences from the 128-dim kernel:
//
//  * a tile of 128 positions is two 128-byte-wide halves of every row (two tensor copies per operand, 64 KB per
//    tile for K and V together); K tiles go through a ring of 2 stages that are free again as soon as their score MMAs
//    have run, V tiles (with both scale tiles) through a ring of 3 that are held until the tile's P.V has run, each ring
//    with its own producer thread; one CTA (all 512 TMEM columns) lives on an SM;
//  * S^T = K . Q^T: 8 MMAs of N = 16 per tile (one per q8_0 block; Q's two int8 planes of up to 8 heads fill all 16
//    rows of the operand), 128 TMEM columns per S buffer;
//  * O^T += V^T . P per half of the dims (M = 128 each): P[position] holds, for each of the half's 4 blocks, 16 bytes
//    (hi bytes of heads 0-7, lo bytes of heads 0-7) = two 32-byte swizzle spans = 64 B-operand columns; the thread of a
//    dim keeps its own block's 16 columns of each half;
//  * with one CTA on an SM nothing else hides a tile's chain S MMA -> softmax -> P -> P.V MMA -> fold, so two groups of 128
//    softmax threads take the even and the odd tiles (S, P and O are double-buffered: a buffer per group), each with its own
//    running maxima, sums and accumulators, which are merged once at the end;
//  * it is stage 1 only: the partials leave as plain (m, l, acc) and the merge kernel follows, and it neither appends
//    nor exchanges (those stay with the 128-dim kernels); a launch that asks for them is declined.
//  * Every wait is bounded, as there.
#include "decode_common.cuh"

#include <climits>
#include <cstring>
#include <mutex>

namespace b200kv {

namespace {

constexpr int kD = 256;
constexpr int kTileM = 128;            // positions per tile = rows of the S MMA = TMEM lanes
constexpr int kKStages = 2;            // K tiles: a stage is free again as soon as its score MMAs have run
constexpr int kVStages = 3;            // V tiles (and both scale tiles): held until the tile's P.V has run
constexpr int kThreads = 384;
constexpr int kConsumers = 128;        // softmax threads per group; warps 0-3 take the even tiles, warps 4-7 the odd ones
constexpr int kProducerWarp = 8, kMmaWarp = 9, kPvWarp = 10, kVProducerWarp = 11;
constexpr uint32_t kSpin = 1u << 20;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0;          // two S buffers of 8 blocks x 16 columns
constexpr uint32_t kColO = 256;        // two O buffers of 2 halves x 64 columns: (block of the half, plane, head)
constexpr float kPMax = 65535.0f;
constexpr int kHalfTile = kTileM * 128;   // one 128-byte-wide half of a K or V tile

template <int NBLK>
struct Smem {
    static constexpr int kKTile = 2 * kHalfTile;                       // 32768
    static constexpr int kSTile = kTileM * NBLK * 2;                   // 2048 (q8_0) or 256 (row scale)
    static constexpr int kOffK = 0;
    static constexpr int kOffV = kKStages * kKTile;
    static constexpr int kOffP = (kKStages + kVStages) * kKTile;       // 2 x [half][span][128 positions][32 B]
    static constexpr int kPBuf = 2 * 2 * kTileM * 32;                  // 16384
    static constexpr int kOffQ = kOffP + 2 * kPBuf;                    // [half][16 rows][128 B]
    static constexpr int kOffS = kOffQ + 2 * 16 * 128;                 // [V stage][ks | vs]
    static constexpr int kOffXch = kOffS + kVStages * 2 * kSTile;      // [2 groups][2 parities][4 warps][16] words: tile maxima
    static constexpr int kOffL = kOffXch + 2 * 2 * 4 * 16 * 4;         // [2 groups][4 warps][8] row sums
    static constexpr int kOffQmul = kOffL + 2 * 4 * 8 * 4;             // [8]
    static constexpr int kOffBar = kOffQmul + 32;
    static constexpr int kNumBars = 2 * kKStages + 2 * kVStages + 8;   // k_full k_empty v_full v_empty s_full[2] s_empty[2] p_full[2] p_empty[2]
    static constexpr int kOffMisc = kOffBar + kNumBars * 8;            // tmem slot, fail flag
    static constexpr int kTotal = kOffMisc + 16;
    static constexpr int kAlloc = kTotal + 1024;                       // slack to align the base to 1024
};
static_assert(Smem<8>::kAlloc <= 232448, "one CTA per SM");

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false if the phase did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpin; ++spin)
        if (mbar_try(bar, parity)) return true;
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
// Shared-memory matrix descriptor (sm_100 format).  K-major operands: rows of 128 bytes, 8-row groups `sbo` apart.
// MN-major operands: one swizzle span (128 or 32 bytes) contiguous along M/N, consecutive k one span apart, groups of
// 8 k `sbo` apart, further spans along M/N `lbo` apart.  `layout`: 2 = 128-byte swizzle, 6 = 32-byte swizzle.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(layout) << 61;
    return d;
}
__host__ __device__ constexpr uint32_t umma_idesc_i8(uint32_t m, uint32_t n, uint32_t a_signed, uint32_t b_signed, uint32_t a_mn_major,
                                                     uint32_t b_mn_major = 0) {
    return (2u << 4) | (a_signed << 7) | (b_signed << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p; }"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 16 consecutive 32-bit columns of this thread's TMEM lane (issue only; pair with tmem_ld_wait)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Order-preserving map of fp32 to int32 (for redux.sync.max) and back.
__device__ __forceinline__ int ordered(float f) { const int i = __float_as_int(f); return i ^ ((i >> 31) & 0x7fffffff); }
__device__ __forceinline__ float unordered(int i) { return __int_as_float(i ^ ((i >> 31) & 0x7fffffff)); }

// NBLK scales per row (8 = q8_0 blocks of 32, 1 = one per row); G query heads per kv head (at most 8).
template <int NBLK, int G, bool Q_F16>
__global__ void __launch_bounds__(kThreads, 1)
decode_tc5_wide_kernel(const __grid_constant__ DecodeParams p, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
    using L = Smem<NBLK>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 1024-aligned, still a shared-space pointer
    const uint32_t sbase = smem_u32(smem);

    pdl_launch_dependents();   // the next kernel of the stream may become resident as SMs free up; it orders itself

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t split = blockIdx.x, kv_head = blockIdx.y, session = blockIdx.z;
    const b200kv_view& view = p.view;
    uint32_t begin, end;
    resolve_range(p, session, view, &begin, &end);
    const uint32_t num_splits = p.num_splits;

    // ---- this CTA's tiles (tiles are aligned to multiples of 128 positions of the cache) --------------------
    const uint32_t tile_begin = begin / kTileM, tile_end = (end + kTileM - 1) / kTileM;
    const uint64_t total_tiles = end > begin ? tile_end - tile_begin : 0;
    const uint32_t t0 = tile_begin + static_cast<uint32_t>(total_tiles * split / num_splits);
    const uint32_t t1 = tile_begin + static_cast<uint32_t>(total_tiles * (split + 1) / num_splits);
    const int ntiles = static_cast<int>(t1 - t0);
    // With launch overlap the previous kernel may still be appending: rows at or above early_end wait for it.
    const uint32_t early_end = end > p.overlap_tail ? end - p.overlap_tail : 0;

    const uint32_t bar0 = sbase + L::kOffBar;
    auto bar_k_full = [&](int s) { return bar0 + s * 8; };
    auto bar_k_empty = [&](int s) { return bar0 + (kKStages + s) * 8; };
    auto bar_v_full = [&](int s) { return bar0 + (2 * kKStages + s) * 8; };
    auto bar_v_empty = [&](int s) { return bar0 + (2 * kKStages + kVStages + s) * 8; };
    constexpr int kB0 = 2 * kKStages + 2 * kVStages;
    auto bar_s_full = [&](int b) { return bar0 + (kB0 + b) * 8; };
    auto bar_s_empty = [&](int b) { return bar0 + (kB0 + 2 + b) * 8; };
    auto bar_p_full = [&](int b) { return bar0 + (kB0 + 4 + b) * 8; };
    auto bar_p_empty = [&](int b) { return bar0 + (kB0 + 6 + b) * 8; };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
    uint32_t* fail_flag = tmem_slot + 1;

    const uint64_t head_row0 = static_cast<uint64_t>(kv_head) * view.capacity;
    const uint8_t* ks_plane = static_cast<const uint8_t*>(view.key_scales) + head_row0 * NBLK * 2;
    const uint8_t* vs_plane = static_cast<const uint8_t*>(view.value_scales) + head_row0 * NBLK * 2;
    const uint32_t capacity = static_cast<uint32_t>(view.capacity);
    const int row_base = static_cast<int>(head_row0);

    // Tile i of this CTA: its K halves into K stage i % kKStages, its V halves and both scale tiles into V stage i % kVStages.
    auto issue_k = [&](int i) {
        const int stage = i % kKStages;
        const uint32_t pos0 = (t0 + i) * kTileM;
        const uint32_t bar = bar_k_full(stage);
        mbar_expect_tx(bar, L::kKTile);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
            tma_load_2d(sbase + L::kOffK + stage * L::kKTile + hf * kHalfTile, &kmap, hf * 128, row_base + static_cast<int>(pos0), bar);
    };
    auto issue_v = [&](int i) {
        const int stage = i % kVStages;
        const uint32_t pos0 = (t0 + i) * kTileM;
        const uint32_t sbytes = min(static_cast<uint32_t>(kTileM), capacity - pos0) * (NBLK * 2);
        const uint32_t bar = bar_v_full(stage);
        mbar_expect_tx(bar, L::kKTile + 2 * sbytes);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
            tma_load_2d(sbase + L::kOffV + stage * L::kKTile + hf * kHalfTile, &vmap, hf * 128, row_base + static_cast<int>(pos0), bar);
        const uint32_t sdst = sbase + L::kOffS + stage * 2 * L::kSTile;
        bulk_load(sdst, ks_plane + static_cast<size_t>(pos0) * (NBLK * 2), sbytes, bar);
        bulk_load(sdst + L::kSTile, vs_plane + static_cast<size_t>(pos0) * (NBLK * 2), sbytes, bar);
    };

    // ---- set-up ---------------------------------------------------------------------------------------------
    // tiles whose rows are old enough to be fetched before the dependency wait
    int early = 0;
    while (early < ntiles && early < kVStages && (t0 + early + 1) * kTileM <= early_end) ++early;
    const int k_early = min(early, kKStages), v_early = early;
    if (warp == kProducerWarp) {
        if (lane == 0) {
            for (int s = 0; s < kKStages; ++s) { mbar_init(bar_k_full(s), 1); mbar_init(bar_k_empty(s), 1); }
            for (int s = 0; s < kVStages; ++s) { mbar_init(bar_v_full(s), 1); mbar_init(bar_v_empty(s), 1); }
            for (int b = 0; b < 2; ++b) {
                mbar_init(bar_s_full(b), 1); mbar_init(bar_s_empty(b), kConsumers);
                mbar_init(bar_p_full(b), kConsumers); mbar_init(bar_p_empty(b), 1);
            }
            *fail_flag = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            // old cache rows do not depend on the preceding kernels: start streaming them before waiting for those
            for (int i = 0; i < v_early; ++i) { if (i < k_early) issue_k(i); issue_v(i); }
        }
    } else if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_wait();
    // the rest of the first ring fill, by the thread that set the barriers up
    if (warp == kProducerWarp && lane == 0)
        for (int i = 0; i < min(kVStages, ntiles); ++i) {
            if (i >= k_early && i < kKStages) issue_k(i);
            if (i >= v_early) issue_v(i);
        }

    // ---- Q: 15 bits per head as two int8 planes (q = 128 hi + lo).  Rows of the B operand of S^T = K . Q^T: hi planes of
    //      heads 0-7 in rows 0-7, lo planes in rows 8-15 (rows of heads past G are zero); one 16 x 128-byte tile per half
    //      of the dims.  Warp w quantises head w; lane L holds dims 8L .. 8L+7. ----
    {
        uint2 hi8 = make_uint2(0, 0), lo8 = make_uint2(0, 0);
        float qm = 0.0f;
        if (warp < G) {
            const uint32_t head = kv_head * G + warp;
            const size_t qb = (static_cast<size_t>(session) * p.query_heads + head) * kD + lane * 8;
            float q[8];
            if (Q_F16) {
                const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const __half*>(p.q) + qb);
                const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) { q[2 * i] = __low2float(h2[i]); q[2 * i + 1] = __high2float(h2[i]); }
            } else {
                const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(p.q) + qb);
                const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(p.q) + qb + 4);
                q[0] = a.x; q[1] = a.y; q[2] = a.z; q[3] = a.w; q[4] = b.x; q[5] = b.y; q[6] = b.z; q[7] = b.w;
            }
            float am = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(q[i]));
            const float amax = warp_max(am);
            // q = 128*hi + lo with hi in [-127, 127] and lo in [-64, 63]: |q| <= 16319
            const float inv = amax > 0.0f ? 16319.0f / amax : 0.0f;
            uint32_t hw[2] = {0, 0}, lw[2] = {0, 0};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int qi = __float2int_rn(q[i] * inv);
                const int hi = (qi + 64) >> 7, lo = qi - (hi << 7);
                hw[i >> 2] |= static_cast<uint32_t>(hi & 0xff) << (8 * (i & 3));
                lw[i >> 2] |= static_cast<uint32_t>(lo & 0xff) << (8 * (i & 3));
            }
            hi8 = make_uint2(hw[0], hw[1]);
            lo8 = make_uint2(lw[0], lw[1]);
            // scores are kept in base-2 units: dot * (amax/16319) * softmax_scale * log2(e)
            qm = (amax / 16319.0f) * p.scale * 1.4426950408889634f;
        }
        if (warp < 8) {
        if (lane == 0) reinterpret_cast<float*>(smem + L::kOffQmul)[warp] = qm;
        // dims 8*lane .. 8*lane+7 of row n: half lane >> 4, 16-byte chunk ((lane & 15) >> 1) ^ (n & 7), bytes (lane & 1) * 8
        const int n_hi = warp, n_lo = 8 + warp;
        uint8_t* qt = smem + L::kOffQ + (lane >> 4) * (16 * 128);
        *reinterpret_cast<uint2*>(qt + n_hi * 128 + (((((lane & 15) >> 1) ^ (n_hi & 7))) << 4) + (lane & 1) * 8) = hi8;
        *reinterpret_cast<uint2*>(qt + n_lo * 128 + (((((lane & 15) >> 1) ^ (n_lo & 7))) << 4) + (lane & 1) * 8) = lo8;
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // Q was written by ordinary stores, the MMA reads it through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    bool failed = false;

    if (warp == kProducerWarp) {
        // =============================== TMA producer, K tiles ===============================
        if (lane == 0) {
            for (int i = min(kKStages, ntiles); i < ntiles; ++i) {
                // K stage i % kKStages is free once the score MMAs of tile i - kKStages have completed
                if (!mbar_wait(bar_k_empty(i % kKStages), static_cast<uint32_t>((i / kKStages - 1) & 1))) { failed = true; break; }
                issue_k(i);
            }
        }
    } else if (warp == kVProducerWarp) {
        // =============================== TMA producer, V and scale tiles ===============================
        if (lane == 0) {
            for (int i = min(kVStages, ntiles); i < ntiles; ++i) {
                // V stage i % kVStages is free once the P.V of tile i - kVStages has completed
                if (!mbar_wait(bar_v_empty(i % kVStages), static_cast<uint32_t>((i / kVStages - 1) & 1))) { failed = true; break; }
                issue_v(i);
            }
        }
    } else if (warp == kMmaWarp) {
        // =============================== issuer of S^T = K . Q^T ===============================
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_i8(kTileM, 16, 1, 1, 0);   // K (signed) x Q planes (signed), both K-major
            for (int i = 0; i < ntiles; ++i) {
                const int stage = i % kKStages, buf = i & 1;
                if (!mbar_wait(bar_s_empty(buf), static_cast<uint32_t>(((i >> 1) & 1) ^ 1))) { failed = true; break; }   // S buffer read out (tile i - 2)
                if (!mbar_wait(bar_k_full(stage), static_cast<uint32_t>((i / kKStages) & 1))) { failed = true; break; }  // K tile landed
                tc_fence_after();
                const uint32_t kt = sbase + L::kOffK + stage * L::kKTile;
#pragma unroll
                for (int b = 0; b < 8; ++b)   // one q8_0 block of 32 dims per MMA, each into its own 16 columns
                    umma_i8(tmem_base + kColS + buf * 128 + b * 16, umma_desc(kt + (b >> 2) * kHalfTile + 32 * (b & 3), 16, 1024, 2),
                            umma_desc(sbase + L::kOffQ + (b >> 2) * (16 * 128) + 32 * (b & 3), 16, 1024, 2), idesc_s, 0);
                umma_commit(bar_s_full(buf));
                umma_commit(bar_k_empty(stage));    // K stage may be refilled
            }
        }
    } else if (warp == kPvWarp) {
        // =============================== issuer of O^T = V^T . P ===============================
        if (lane == 0) {
            constexpr uint32_t idesc_o = umma_idesc_i8(128, 64, 1, 0, 1, 1);    // V^T (signed, MN-major) x P planes (unsigned, MN-major)
            for (int i = 0; i < ntiles; ++i) {
                const int stage = i % kVStages, buf = i & 1;
                if (!mbar_wait(bar_p_full(buf), static_cast<uint32_t>((i >> 1) & 1))) { failed = true; break; }
                if (!mbar_wait(bar_v_full(stage), static_cast<uint32_t>((i / kVStages) & 1))) { failed = true; break; }   // long complete: the V tile's landing, observed by this thread
                tc_fence_after();
                const uint32_t vt = sbase + L::kOffV + stage * L::kKTile;
                const uint32_t pt = sbase + L::kOffP + buf * L::kPBuf;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                    for (int j = 0; j < 4; ++j)   // 32 positions per MMA
                        umma_i8(tmem_base + kColO + buf * 128 + hf * 64, umma_desc(vt + hf * kHalfTile + j * (32 * 128), kHalfTile, 1024, 2),
                                umma_desc(pt + hf * (2 * kTileM * 32) + j * (32 * 32), kTileM * 32, 256, 6), idesc_o, j > 0);
                umma_commit(bar_p_empty(buf));      // P buffer free, the tile's sums complete
                umma_commit(bar_v_empty(stage));    // V stage (and its scale tiles) may be refilled
            }
        }
    }

    if (warp < 8) {
        // =============================== softmax threads: one per position of a tile, two groups ===============================
        // Group g (warps 4g .. 4g+3) takes the tiles i with i % 2 == g and with them S, P and O buffer g.
        const int grp = warp >> 2, wq = warp & 3, ltid = tid & 127;   // wq: the warp's quarter of the TMEM lanes; ltid: position in the tile / dim in a half
        // what a group hands to the epilogue: this thread's dims (ltid and 128 + ltid), heads 0..G-1, relative to m_run
        float acc[2][G];
        float m_run[G], l_run[G];          // l_run: sums over this thread's positions only
        float pend[2][G];                  // per half: fixed-point scale of the sums in flight in this group's O buffer (own block)
#pragma unroll
        for (int h = 0; h < G; ++h) {
            acc[0][h] = acc[1][h] = 0.0f; m_run[h] = -INFINITY; l_run[h] = 0.0f;
            pend[0][h] = pend[1][h] = 0.0f;
        }
        const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;
        float qmul[G];
#pragma unroll
        for (int h = 0; h < G; ++h) qmul[h] = reinterpret_cast<const float*>(smem + L::kOffQmul)[h];
        // P is the MN-major B operand: per half of the dims and per 32-byte span (two blocks), this position's row of 32
        // bytes, 32-byte swizzle: 16-byte chunk c of row r sits at 32 r + ((c ^ ((r >> 2) & 1)) << 4)
        const uint32_t p_row = static_cast<uint32_t>(ltid) * 32u;
        const uint32_t p_flip = static_cast<uint32_t>((ltid >> 2) & 1) << 4;
        int* xch = reinterpret_cast<int*>(smem + L::kOffXch);
        const int buf = grp;
        auto wait = [&](uint32_t bar, uint32_t parity) { if (!failed && !mbar_wait(bar, parity)) failed = true; };
        auto group_sync = [&]() {
            if (grp == 0) asm volatile("bar.sync 3, 128;" ::: "memory");
            else asm volatile("bar.sync 4, 128;" ::: "memory");
        };
        auto fold_o = [&]() {   // the completed sums of a tile: own block's 16 columns of each half -> fp32 accumulators
            tc_fence_after();
            int o0[16], o1[16];
            tmem_ld16(tmem_base + lane_addr + kColO + buf * 128 + wq * 16, o0);
            tmem_ld16(tmem_base + lane_addr + kColO + buf * 128 + 64 + wq * 16, o1);
            tmem_ld_wait();
            tc_fence_before();
#pragma unroll
            for (int h = 0; h < G; ++h) {
                acc[0][h] = fmaf(static_cast<float>(o0[h] * 256 + o0[8 + h]), pend[0][h], acc[0][h]);
                acc[1][h] = fmaf(static_cast<float>(o1[h] * 256 + o1[8 + h]), pend[1][h], acc[1][h]);
            }
        };

        int last_i = -1;
        for (int i = grp; i < ntiles; i += 2) {
            last_i = i;
            const int stage = i % kVStages;
            // A parity wait tells "this phase is over" only to a waiter that has seen the phase before it.  A group takes every
            // other tile, the ring has three stages, so a group would skip phases of a stage; it therefore also waits for the
            // tile in between (the other group's), which has normally landed long before.
            if (i > 0) wait(bar_v_full((i - 1) % kVStages), static_cast<uint32_t>(((i - 1) / kVStages) & 1));
            wait(bar_v_full(stage), static_cast<uint32_t>((i / kVStages) & 1));   // the scale tiles of this stage (async-proxy writes)
            wait(bar_s_full(buf), static_cast<uint32_t>((i >> 1) & 1));
            tc_fence_after();

            const uint32_t pos = (t0 + i) * kTileM + ltid;
            const bool valid = pos >= begin && pos < end;
            const uint8_t* kst = smem + L::kOffS + stage * 2 * L::kSTile;
            const uint8_t* vst = kst + L::kSTile;
            float ks[8], vs[8];
            uint32_t vs_bits[8];
            if constexpr (NBLK == 8) {
                const uint4 kr = *reinterpret_cast<const uint4*>(kst + ltid * 16), vr = *reinterpret_cast<const uint4*>(vst + ltid * 16);
                const uint32_t kw[4] = {kr.x, kr.y, kr.z, kr.w}, vw[4] = {vr.x, vr.y, vr.z, vr.w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float2 kf = __half22float2(*reinterpret_cast<const __half2*>(&kw[w])), vf = __half22float2(*reinterpret_cast<const __half2*>(&vw[w]));
                    ks[2 * w] = kf.x; ks[2 * w + 1] = kf.y; vs[2 * w] = vf.x; vs[2 * w + 1] = vf.y;
                    vs_bits[2 * w] = vw[w] & 0xffffu; vs_bits[2 * w + 1] = vw[w] >> 16;
                }
            } else {
                const uint16_t kr = *reinterpret_cast<const uint16_t*>(kst + ltid * 2), vr = *reinterpret_cast<const uint16_t*>(vst + ltid * 2);
#pragma unroll
                for (int b = 0; b < 8; ++b) { ks[b] = __half2float(__ushort_as_half(kr)); vs[b] = __half2float(__ushort_as_half(vr)); vs_bits[b] = vr; }
            }
            // scores of this position, base-2 units: per block 16 sums (hi planes of heads 0-7, lo planes of heads 0-7)
            float a[G];
#pragma unroll
            for (int h = 0; h < G; ++h) a[h] = 0.0f;
#pragma unroll
            for (int b0 = 0; b0 < 8; b0 += 4) {
                int sv[4][16];
#pragma unroll
                for (int b = 0; b < 4; ++b) tmem_ld16(tmem_base + lane_addr + kColS + buf * 128 + (b0 + b) * 16, sv[b]);
                tmem_ld_wait();
#pragma unroll
                for (int b = 0; b < 4; ++b)
#pragma unroll
                    for (int h = 0; h < G; ++h) a[h] = fmaf(static_cast<float>(sv[b][h] * 128 + sv[b][8 + h]), ks[b0 + b], a[h]);
            }
            tc_fence_before();
            mbar_arrive(bar_s_empty(buf));   // this thread's part of S is in registers
            float s[G];
#pragma unroll
            for (int h = 0; h < G; ++h) s[h] = valid ? a[h] * qmul[h] : -INFINITY;   // positions outside the range (or rows never written) are masked
            // ---- tile maxima (scores per head, value scales per block): redux inside the warp, one exchange across the group's four ----
            const int par = (i >> 1) & 1;   // the exchange area is double-buffered by the parity of the group's tile count
            {
                int* dst = xch + ((grp * 2 + par) * 4 + wq) * 16;
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    const int mx = __reduce_max_sync(0xffffffffu, ordered(s[h]));
                    if (lane == 0) dst[h] = mx;
                }
#pragma unroll
                for (int b = 0; b < (NBLK == 8 ? 8 : 1); ++b) {
                    const uint32_t vmx = __reduce_max_sync(0xffffffffu, valid ? vs_bits[b] : 0u);   // positive fp16 order like integers
                    if (lane == 0) dst[8 + b] = static_cast<int>(vmx);
                }
            }
            group_sync();
            float m_tile[G], vs_max[8];
            {
                int mx[G];
                uint32_t vmx[8];
#pragma unroll
                for (int h = 0; h < G; ++h) mx[h] = INT_MIN;
#pragma unroll
                for (int b = 0; b < 8; ++b) vmx[b] = 0;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int* src = xch + ((grp * 2 + par) * 4 + w) * 16;
#pragma unroll
                    for (int h = 0; h < G; ++h) mx[h] = max(mx[h], src[h]);
#pragma unroll
                    for (int b = 0; b < (NBLK == 8 ? 8 : 1); ++b) vmx[b] = max(vmx[b], static_cast<uint32_t>(src[8 + b]));
                }
#pragma unroll
                for (int h = 0; h < G; ++h) m_tile[h] = unordered(mx[h]);
#pragma unroll
                for (int b = 0; b < 8; ++b) vs_max[b] = __half2float(__ushort_as_half(static_cast<uint16_t>(vmx[NBLK == 8 ? b : 0])));
            }
            // ---- online softmax: new running maximum, weights, and the tile's fixed-point scales ----
            float wn[G], nscale[2][G];   // weights normalised to the tile maximum (<= 1); fixed-point scale of this tile (own block of each half)
            float vs_own[2];
#pragma unroll
            for (int hf = 0; hf < 2; ++hf)
                vs_own[hf] = wq == 0 ? vs_max[4 * hf] : wq == 1 ? vs_max[4 * hf + 1] : wq == 2 ? vs_max[4 * hf + 2] : vs_max[4 * hf + 3];
#pragma unroll
            for (int h = 0; h < G; ++h) {
                const float m_new = fmaxf(m_run[h], m_tile[h]);
                const float alpha = (m_run[h] == -INFINITY) ? 0.0f : exp2f(m_run[h] - m_new);
                acc[0][h] *= alpha; acc[1][h] *= alpha; l_run[h] *= alpha;
                pend[0][h] *= alpha; pend[1][h] *= alpha;
                m_run[h] = m_new;
                const float w = (s[h] == -INFINITY) ? 0.0f : exp2f(s[h] - m_new);
                l_run[h] += w;
                const float wmax = (m_tile[h] == -INFINITY) ? 0.0f : exp2f(m_tile[h] - m_new);
                wn[h] = wmax > 0.0f ? __fdividef(w, wmax) : 0.0f;
                nscale[0][h] = wmax * vs_own[0] * (1.0f / kPMax);
                nscale[1][h] = wmax * vs_own[1] * (1.0f / kPMax);
            }
            // ---- this group's P and O buffer were last used by tile i - 2: its P.V has completed; fold its sums first ----
            if (i >= 2) {
                wait(bar_p_empty(buf), static_cast<uint32_t>(((i >> 1) - 1) & 1));
                fold_o();
            }
#pragma unroll
            for (int h = 0; h < G; ++h) { pend[0][h] = nscale[0][h]; pend[1][h] = nscale[1][h]; }
            // [block]: w * value_scale as 16-bit fixed point, 16 bytes per block: hi bytes of heads 0-7, lo bytes of heads 0-7
            const uint32_t pt = sbase + L::kOffP + buf * L::kPBuf + p_row;
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                const float wv = (valid && vs_max[b] > 0.0f) ? vs[b] * __fdividef(kPMax, vs_max[b]) : 0.0f;
                uint32_t pq[8];
#pragma unroll
                for (int h = 0; h < 8; ++h) pq[h] = h < G ? min(__float2uint_rn(wn[h < G ? h : 0] * wv), 65535u) : 0u;
                const uint32_t p01 = pq[0] | (pq[1] << 16), p23 = pq[2] | (pq[3] << 16), p45 = pq[4] | (pq[5] << 16), p67 = pq[6] | (pq[7] << 16);
                const uint32_t hi_a = __byte_perm(p01, p23, 0x7531), hi_b = __byte_perm(p45, p67, 0x7531);
                const uint32_t lo_a = __byte_perm(p01, p23, 0x6420), lo_b = __byte_perm(p45, p67, 0x6420);
                // half b >> 2, span (b >> 1) & 1, chunk b & 1
                const uint32_t dst = pt + static_cast<uint32_t>(b >> 2) * (2 * kTileM * 32) + static_cast<uint32_t>((b >> 1) & 1) * (kTileM * 32) +
                                     ((static_cast<uint32_t>(b & 1) << 4) ^ p_flip);
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(hi_a), "r"(hi_b), "r"(lo_a), "r"(lo_b) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(bar_p_full(buf));
        }
        // the group's last tile's sums
        if (last_i >= 0) {
            wait(bar_p_empty(buf), static_cast<uint32_t>((last_i >> 1) & 1));
            fold_o();
        }
        // ---- row sums over the group ----
#pragma unroll
        for (int h = 0; h < G; ++h) l_run[h] = warp_sum(l_run[h]);
        float* lsm = reinterpret_cast<float*>(smem + L::kOffL);   // [2 groups][4 warps][8]
        if (lane == 0) {
#pragma unroll
            for (int h = 0; h < G; ++h) lsm[(grp * 4 + wq) * 8 + h] = l_run[h];
            if (failed) atomicOr(fail_flag, 1u);
        }
        // ---- the odd tiles' group hands its state to the even tiles' group through its own P buffer (the P.V MMAs that read it
        //      have completed; the other buffer may still be feeding the even group's last P.V) ----
        float* hand = reinterpret_cast<float*>(smem + L::kOffP + L::kPBuf);   // [3 * G][128]: acc of half 0, acc of half 1, maxima
        if (grp == 1) {
#pragma unroll
            for (int h = 0; h < G; ++h) {
                hand[(0 * G + h) * 128 + ltid] = acc[0][h];
                hand[(1 * G + h) * 128 + ltid] = acc[1][h];
                hand[(2 * G + h) * 128 + ltid] = m_run[h];
            }
        }
        asm volatile("bar.sync 5, 256;" ::: "memory");
        if (grp == 0) {
            // a wait that ran out anywhere in the pipeline ends in a wait of these threads running out
            const bool poisoned = *reinterpret_cast<volatile uint32_t*>(fail_flag) != 0;
            if (poisoned && tid == 0 && p.status != nullptr) atomicOr(p.status, B200KV_STATUS_PIPE_TIMEOUT);
#pragma unroll
            for (int h = 0; h < G; ++h) {
                float l0 = 0.0f, l1 = 0.0f;
#pragma unroll
                for (int w = 0; w < 4; ++w) { l0 += lsm[w * 8 + h]; l1 += lsm[(4 + w) * 8 + h]; }
                const float m1 = hand[(2 * G + h) * 128 + ltid];   // uniform over the group's threads
                const float M = fmaxf(m_run[h], m1);
                const float s0 = (m_run[h] == -INFINITY) ? 0.0f : exp2f(m_run[h] - M), s1 = (m1 == -INFINITY) ? 0.0f : exp2f(m1 - M);
                float a0 = fmaf(acc[0][h], s0, hand[(0 * G + h) * 128 + ltid] * s1);
                float a1 = fmaf(acc[1][h], s0, hand[(1 * G + h) * 128 + ltid] * s1);
                float lt = fmaf(l0, s0, l1 * s1);
                float mh = M * 0.6931471805599453f;   // natural-log units, as the merge expects
                if (poisoned) { a0 = a1 = mh = lt = __int_as_float(0x7fc00000); }
                const size_t slot = (static_cast<size_t>(session) * p.num_splits + split) * p.query_heads + kv_head * G + h;
                p.ws_acc[slot * kD + ltid] = a0;
                p.ws_acc[slot * kD + 128 + ltid] = a1;
                if (ltid == 0) { p.ws_m[slot] = mh; p.ws_l[slot] = lt; }
            }
        }
    }

    // ---- teardown: every role arrives here, with or without a timeout; TMEM is always released ----
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn wide_encoder() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(sym);
        else
            (void)cudaGetLastError();
    });
    return fn;
}

// int8 plane [kv_heads * capacity][256]: boxes of 128 bytes x 128 rows, 128-byte swizzle
bool encode_wide_plane(CUtensorMap* map, int8_t* plane, const b200kv_view& view) {
    EncodeFn fn = wide_encoder();
    if (fn == nullptr) return false;
    const TensorMapKey key{plane, static_cast<uint64_t>(view.kv_heads) * view.capacity, static_cast<uint32_t>(kD), 128u,
                           static_cast<uint32_t>(kTileM), 1u};   // kind 1: bytes, 128-byte swizzle
    if (tensor_map_lookup(key, map)) return true;
    const cuuint64_t dims[2] = {kD, static_cast<cuuint64_t>(view.kv_heads) * view.capacity};
    const cuuint64_t strides[1] = {kD};
    const cuuint32_t box[2] = {128, kTileM};
    const cuuint32_t elem[2] = {1, 1};
    if (fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, plane, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    tensor_map_remember(key, *map);
    return true;
}

template <int NBLK, int G, bool Q_F16>
int launch_one(const DecodeParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap, dim3 grid, cudaStream_t stream) {
    using L = Smem<NBLK>;
    static std::atomic<uint64_t> done{0};   // one per kernel instantiation: devices that have opted in
    const cudaError_t attr_err = opt_in_dynamic_smem(reinterpret_cast<const void*>(decode_tc5_wide_kernel<NBLK, G, Q_F16>), L::kAlloc, done);
    if (attr_err != cudaSuccess) { set_last_cuda_error(attr_err, "cudaFuncSetAttribute(decode_tc5_wide)"); return B200KV_ERR_CUDA; }
    B200KV_CUDA_TRY(launch_kernel(decode_tc5_wide_kernel<NBLK, G, Q_F16>, grid, dim3(kThreads), L::kAlloc, stream, true, p, kmap, vmap));
    return B200KV_OK;
}

template <int NBLK, int G>
int launch_q(const DecodeParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap, dim3 grid, cudaStream_t stream) {
    return p.q_is_f16 ? launch_one<NBLK, G, true>(p, kmap, vmap, grid, stream) : launch_one<NBLK, G, false>(p, kmap, vmap, grid, stream);
}

}  // namespace

bool decode_tc5_wide_ok(const b200kv_view& view, uint32_t query_heads) {
    if (view.quant_mode != B200KV_Q8_Q8 || view.head_dim != kD) return false;
    if (view.qblock != 32 && view.qblock != kD) return false;
    if (view.capacity % 8 != 0) return false;   // bulk copies of the scale planes need 16-byte aligned tile starts
    if (view.kv_heads == 0 || query_heads % view.kv_heads != 0) return false;
    const uint32_t g = query_heads / view.kv_heads;
    if (g != 4 && g != 6 && g != 8) return false;
    if (static_cast<uint64_t>(view.kv_heads) * view.capacity > 0x7fffffffull) return false;  // TMA row coordinate is int32
    return wide_encoder() != nullptr;
}

// One CTA per SM; every CTA should see at least two tiles.
uint32_t pick_splits_tc5_wide(const b200kv_view& view, uint32_t max_length) {
    uint32_t s = (148u + view.kv_heads / 2) / view.kv_heads;
    const uint32_t tiles = (max_length + kTileM - 1) / kTileM;
    if (s > tiles / 2) s = tiles / 2;
    const uint32_t cap = max_splits_per_session(1);
    if (s > cap) s = cap;
    return s ? s : 1;
}

// Stage 1 of a single-session launch into the plain partial arrays (p.ws_m / ws_l / ws_acc, p.num_splits set by the
// caller); B200KV_ERR_UNSUPPORTED when the launch is not one this kernel takes.
int launch_decode_tc5_wide(const DecodeParams& p_in, const b200kv_view& geometry, cudaStream_t stream) {
    if (!decode_tc5_wide_ok(geometry, p_in.query_heads)) return B200KV_ERR_UNSUPPORTED;
    if (p_in.views != nullptr || p_in.lengths != nullptr || p_in.causal || p_in.sessions != 1 || p_in.new_key != nullptr)
        return B200KV_ERR_UNSUPPORTED;
    DecodeParams p = p_in;
    p.overlap_tail = launch_overlap_tail();
    p.ws_tagged = nullptr;
    CUtensorMap kmap, vmap;
    if (!encode_wide_plane(&kmap, geometry.key_q8, geometry) || !encode_wide_plane(&vmap, geometry.value_q8, geometry)) return B200KV_ERR_UNSUPPORTED;
    const bool blocks = geometry.qblock == 32;
    const uint32_t g = p.query_heads / geometry.kv_heads;
    dim3 grid(p.num_splits, geometry.kv_heads, 1);
    if (blocks) {
        if (g == 4) return launch_q<8, 4>(p, kmap, vmap, grid, stream);
        if (g == 6) return launch_q<8, 6>(p, kmap, vmap, grid, stream);
        return launch_q<8, 8>(p, kmap, vmap, grid, stream);
    }
    if (g == 4) return launch_q<1, 4>(p, kmap, vmap, grid, stream);
    if (g == 6) return launch_q<1, 6>(p, kmap, vmap, grid, stream);
    return launch_q<1, 8>(p, kmap, vmap, grid, stream);
}

}  // namespace b200kv
