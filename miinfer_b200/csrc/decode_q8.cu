// Streaming split-K GQA decode attention over an int8 (q8_0 or row-scaled) KV
// cache, head_dim 128 -- the kernel the decode benchmark runs.
//
// What it computes is MIInfer's decode stage 1
// (gfx906/kernels/qwen3_primitives.hip:7371-7485) with block scales; how it is
// laid out is specific to B200:
//
//  * One CTA = one (kv head, split) = 8 independent warps.  ALL query heads of
//    the kv-head group share every K/V byte the CTA loads (the reference
//    re-reads the cache once per query head).
//  * Every warp owns a private 3-stage ring of 16-position tiles filled by TMA:
//    K and V tiles through tensor maps with the 128-byte swizzle (rows of 128
//    int8), both scale tiles with plain bulk copies; one mbarrier per stage.
//    One lane issues the copies.  Warps never synchronise with each other in
//    the main loop.
//  * Both contractions run on the tensor cores through warp-level mma, which is
//    what lets 16 warps per SM keep up with HBM: with scalar integer dot
//    products and packed fp32 multiply-adds the same loop was bound by the FMA
//    pipe at about half of the memory rate.  The arithmetic is arranged so that
//    nothing is lost against that scalar version:
//      - Q.K^T is m16n8k32 int8 x int8 -> int32 (exact).  Q is quantised once
//        per launch to 15 bits per head (q = 128*hi + lo, two int8 planes); the
//        hi plane sits in rows 0-7 of the A operand and the lo plane in rows
//        8-15, so one instruction yields both partial sums, recombined exactly
//        in int32.  K is the B operand straight from the swizzled tile
//        (ldmatrix), no conversion.  One k-step of 32 is one q8_0 block; its
//        int32 sum is scaled by the fp16 block scale in fp32.
//      - P.V is m16n8k16 fp16 x fp16 -> fp32 with V^T as the A operand (16 dims
//        x 16 positions) and the weights as B (16 positions x 8 columns).  V's
//        int8 bytes become EXACT fp16 integers (byte-permute two positions'
//        bytes into one word, one logic op to form 0x64xx, one packed subtract).
//        The weight w * value_scale is split into an fp16 high part and an fp16
//        remainder; the high parts of the 4 heads use columns 0-3 and the
//        remainders columns 4-7, so the split costs no extra instructions and
//        keeps 22 bits of each weight.  The two column groups are added once,
//        when the warp stores its result.
//      - The score fragment (rows = heads, columns = positions) is already the
//        layout the weight operand needs (rows = positions, columns = heads):
//        rows 4-7 of the Q operand repeat rows 0-3, so lanes 16-31 hold the
//        same scores as lanes 0-15 and produce the remainder columns without
//        any exchange.  Weights never leave registers.
//  * Softmax is the online form in base 2 with a lazily updated reference
//    maximum (accumulators are rescaled only when a head's maximum has grown by
//    more than 2^6); each warp keeps (m, l, acc) for the whole launch, the CTA
//    merges its 8 warps in shared memory and writes one partial per (split,
//    query head); the last CTA of a kv head to finish merges all splits.
//  * Every wait is bounded: a copy that never arrives poisons the partial with
//    NaN instead of hanging the GPU.
#include "decode_tail.cuh"

#include <cstring>
#include <mutex>

namespace b200kv {

namespace {

constexpr int kWarps = 8;     // warps per CTA, each with its own tile ring
constexpr int kTile = 16;     // positions per tile: one P.V k-step, two Q.K n-tiles
constexpr int kStages = 3;    // TMA ring depth per warp
constexpr int kD = 128;
constexpr uint32_t kSpinLimit = 1u << 20;   // bounded waits: a lost copy ends the kernel with a poisoned partial
constexpr uint32_t kPositionsPerSplit = 2048;   // batched launches, split count left to the library: one split per this many positions
constexpr int kAppendUnits = 4;    // a fused append is balanced as this many tiles of work
constexpr float kRescaleSlack = 6.0f;   // log2 units a head's maximum may exceed the reference before a rescale

template <int NBLK>
struct Smem {
    static constexpr int kKTile = kTile * kD;                    // 2048
    static constexpr int kSTile = kTile * NBLK * 2;              // 128 (q8_0) or 32 (row scale)
    static constexpr int kOffV = kWarps * kStages * kKTile;
    static constexpr int kOffS = 2 * kOffV;                              // [warp][stage][ks | vs]
    static constexpr int kOffQ = kOffS + kWarps * kStages * 2 * kSTile;  // int8 hi[4][kD], lo[4][kD]
    static constexpr int kOffQmul = kOffQ + 2 * 4 * kD;                  // [4] float
    static constexpr int kOffMisc = kOffQmul + 16;                       // merger scratch: fold area of the split groups
    static constexpr int kOffBar = kOffMisc + (8 + 3 * 64 * 2) * 4;
    static constexpr int kTotal = kOffBar + kWarps * kStages * 8;
    static constexpr int kAlloc = kTotal + 1024;                         // slack to align the base to 1024
    static constexpr int kWarpArea = kStages * kKTile;                   // a warp's K ring doubles as its merge area
};
static_assert(Smem<4>::kWarpArea >= (8 * kD + 8) * 4, "merge area of a warp: 8 columns x 128 dims + m[4] + l[4]");

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
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// c (+)= A(16x32 int8, row) * B(32x8 int8, col), int32 accumulators
__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// c = A * B with a zero accumulator input (no registers to clear)
__device__ __forceinline__ void mma_s8_zero(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    const int z = 0;
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(z));
}
// c += A(16x16 fp16, row) * B(16x8 fp16, col), fp32 accumulators
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// A transposed 8x8 load of 16-bit elements hands each lane the word [p0.d0, p0.d1, p1.d0, p1.d1]: two
// consecutive positions p0, p1 of two consecutive dims d0, d1.  These return the two positions of d0 (bytes 0, 2)
// and of d1 (bytes 1, 3) as exact half2 integers: each byte lands in the mantissa of 0x64xx (= 1024 + u) with its
// sign bit flipped (u = x + 128), and 1152 is subtracted.
__device__ __forceinline__ uint32_t s8_even_bytes_to_half2(uint32_t w) {
    const uint32_t r = (w & 0x00FF00FFu) ^ 0x64806480u;
    const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&r), __half2half2(__ushort_as_half(0x6480)));   // 0x6480 = 1152
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t s8_odd_bytes_to_half2(uint32_t w) {
    const uint32_t r = __byte_perm(w, 0x64646464u, 0x4341) ^ 0x00800080u;
    const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&r), __half2half2(__ushort_as_half(0x6480)));
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// G query heads per kv head (1, 2 or 4); NBLK scales per row (4 = q8_0 blocks of 32, 1 = one per row).
template <int G, int NBLK, bool Q_F16>
__global__ void __launch_bounds__(kWarps * 32, 2)
decode_q8_kernel(const __grid_constant__ DecodeParams p, const __grid_constant__ CUtensorMap kmap_single,
                 const __grid_constant__ CUtensorMap vmap_single) {
    using L = Smem<NBLK>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 1024-aligned, still a shared-space pointer

    pdl_launch_dependents();   // the next kernel of the stream may become resident as SMs free up; it orders itself

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;   // mma fragment coordinates
    const uint32_t split = blockIdx.x, kv_head = blockIdx.y, session = blockIdx.z;
    const b200kv_view& view = session_view(p, session);
    uint32_t begin, end;
    resolve_range(p, session, view, &begin, &end);

    // Batched launches size the grid for the longest session; a shorter session uses only as many splits as its
    // own length warrants (every CTA of the session derives the same number) and the surplus CTAs leave at once.
    uint32_t num_splits = p.num_splits;
    if (p.lengths != nullptr) {
        const uint32_t want = (end - begin + p.split_positions - 1) / p.split_positions;
        num_splits = min(num_splits, max(want, 1u));
        if (split >= num_splits) return;
    }

    // ---- this warp's tiles -----------------------------------------------------------
    const uint32_t tile_begin = begin / kTile, tile_end = (end + kTile - 1) / kTile;
    const uint64_t total_tiles = end > begin ? tile_end - tile_begin : 0;
    const uint32_t nworkers = num_splits * kWarps, gw = split * kWarps + warp;
    // A fused append is counted as extra units at the end of the range, so the warp that does it is handed fewer tiles.
    const bool fuse = p.new_key != nullptr;
    const uint64_t units = total_tiles + (fuse ? kAppendUnits : 0);
    const uint64_t u0 = units * gw / nworkers, u1 = units * (gw + 1) / nworkers;
    const uint32_t t0 = tile_begin + static_cast<uint32_t>(u0 < total_tiles ? u0 : total_tiles);
    const uint32_t t1 = tile_begin + static_cast<uint32_t>(u1 < total_tiles ? u1 : total_tiles);
    const int ntiles = static_cast<int>(t1 - t0);
    const bool owner = fuse && ntiles > 0 && t1 == tile_end;   // this warp holds the tile of the appended token
    // With launch overlap the previous kernel may still be appending: rows at or above early_end wait for it.  The
    // row a fused append writes is never loaded early either.
    uint32_t early_end = end > p.overlap_tail ? end - p.overlap_tail : 0;
    if (fuse && early_end >= end) early_end = end - 1;

    uint8_t* k_ring = smem + warp * kStages * L::kKTile;
    uint8_t* v_ring = smem + L::kOffV + warp * kStages * L::kKTile;
    uint8_t* s_ring = smem + L::kOffS + warp * kStages * 2 * L::kSTile;
    int8_t* q_hi = reinterpret_cast<int8_t*>(smem + L::kOffQ);
    int8_t* q_lo = q_hi + 4 * kD;
    float* qmul_s = reinterpret_cast<float*>(smem + L::kOffQmul);
    const uint32_t bars = smem_u32(smem + L::kOffBar) + warp * kStages * 8;
    const uint64_t head_row0 = static_cast<uint64_t>(kv_head) * view.capacity;

    // the barriers of a warp are its own
    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(bars + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    const CUtensorMap* kmap = p.views != nullptr ? &p.views[session].kmap : &kmap_single;
    const CUtensorMap* vmap = p.views != nullptr ? &p.views[session].vmap : &vmap_single;
    const uint8_t* ks_plane = static_cast<const uint8_t*>(view.key_scales) + head_row0 * NBLK * 2;
    const uint8_t* vs_plane = static_cast<const uint8_t*>(view.value_scales) + head_row0 * NBLK * 2;
    const uint32_t k_ring_u = smem_u32(k_ring), v_ring_u = smem_u32(v_ring), s_ring_u = smem_u32(s_ring);
    const uint32_t capacity = static_cast<uint32_t>(view.capacity);
    const int row_base = static_cast<int>(head_row0);
    auto issue = [&](int i, int stage) {
        const uint32_t pos0 = (t0 + i) * kTile;
        const uint32_t sbytes = min(static_cast<uint32_t>(kTile), capacity - pos0) * (NBLK * 2);
        const uint32_t bar = bars + stage * 8;
        mbar_expect_tx(bar, 2 * L::kKTile + 2 * sbytes);
        tma_load_2d(k_ring_u + stage * L::kKTile, kmap, 0, row_base + static_cast<int>(pos0), bar);
        tma_load_2d(v_ring_u + stage * L::kKTile, vmap, 0, row_base + static_cast<int>(pos0), bar);
        const uint32_t sdst = s_ring_u + stage * 2 * L::kSTile;
        bulk_load(sdst, ks_plane + pos0 * (NBLK * 2), sbytes, bar);
        bulk_load(sdst + L::kSTile, vs_plane + pos0 * (NBLK * 2), sbytes, bar);
    };
    // old cache rows do not depend on the preceding kernels: start streaming them before waiting for those
    int issued = 0;
    if (lane == 0)
        while (issued < kStages && issued < ntiles && (t0 + issued + 1) * kTile <= early_end) { issue(issued, issued); ++issued; }
    pdl_wait();
    // The new row of a fused append is fetched now, while the memory system is still quiet: once every warp's ring
    // is streaming, a dependent load waits behind tens of megabytes of queued tile traffic (microseconds).
    float new_k[4], new_v[4];
    if (owner) {
        tail::load_new_row(p.new_key, p.new_is_f16, kv_head, lane, new_k);
        tail::load_new_row(p.new_value, p.new_is_f16, kv_head, lane, new_v);
    }
    {
        // the tile that holds the row of a fused append is loaded only after that row has been stored (below)
        const int limit = owner ? ntiles - 1 : ntiles;
        if (lane == 0)
            while (issued < kStages && issued < limit) { issue(issued, issued); ++issued; }
    }

    // ---- quantise Q to 15 bits (two int8 planes), one warp per head; heads the group does not have are zero ----
    if (warp < 4) {
        uint32_t hi4 = 0, lo4 = 0;
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
            // q = 128*hi + lo with hi in [-127, 127] and lo in [-64, 63]: |q| <= 16319
            const float inv = amax > 0.0f ? 16319.0f / amax : 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int qi = __float2int_rn(q[i] * inv);
                const int hi = (qi + 64) >> 7, lo = qi - (hi << 7);
                hi4 |= static_cast<uint32_t>(hi & 0xff) << (8 * i);
                lo4 |= static_cast<uint32_t>(lo & 0xff) << (8 * i);
            }
            // scores are kept in base-2 units: dot * (amax/16319) * softmax_scale * log2(e)
            if (lane == 0) qmul_s[warp] = (amax / 16319.0f) * p.scale * 1.4426950408889634f;
        } else if (lane == 0) {
            qmul_s[warp] = 0.0f;
        }
        reinterpret_cast<uint32_t*>(q_hi + warp * kD)[lane] = hi4;
        reinterpret_cast<uint32_t*>(q_lo + warp * kD)[lane] = lo4;
    }
    __syncthreads();

    if (owner) {
        // After the barrier, so that only this warp (which was handed fewer tiles) pays for the append.  The new row
        // goes to the cache first; its tile is loaded (by TMA, an asynchronous-proxy read) only afterwards.
        tail::fused_append_row<NBLK>(p, view, new_k, new_v, end - 1, head_row0 + end - 1, lane);
        __threadfence();
        asm volatile("fence.proxy.async;" ::: "memory");
        __syncwarp();
        if (lane == 0)
            while (issued < kStages && issued < ntiles) { issue(issued, issued); ++issued; }
    }

    // A operand of Q.K^T, per k-step (= one 32-dim block): rows g and g+8 are the hi and lo planes of head g & 3
    uint32_t qa[4][4];
    {
        const int h = g & 3;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            qa[ks][0] = *reinterpret_cast<const uint32_t*>(q_hi + h * kD + 32 * ks + 4 * t);
            qa[ks][1] = *reinterpret_cast<const uint32_t*>(q_lo + h * kD + 32 * ks + 4 * t);
            qa[ks][2] = *reinterpret_cast<const uint32_t*>(q_hi + h * kD + 32 * ks + 16 + 4 * t);
            qa[ks][3] = *reinterpret_cast<const uint32_t*>(q_lo + h * kD + 32 * ks + 16 + 4 * t);
        }
    }
    const float qmul = qmul_s[g & 3];
    const bool remainder_lane = g >= 4;   // this lane feeds a remainder column of the weight operand

    // P.V accumulators: M-tile mt holds dims 16*mt + 2*row {+0: rows 0-7, +1: rows 8-15}, all in block mt >> 1;
    // columns 2t, 2t+1 of this lane: high parts of heads 0..3 (t < 2) or remainders (t >= 2)
    float acc[8][4];
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;
    float m_ref = -INFINITY, l_run = 0.0f;
    bool failed = false;

    // per-lane shared-memory offsets that do not change from tile to tile
    // ldmatrix: lane supplies the row address of matrix (lane>>3) = 16-byte chunk 4h + (lane>>3) of row (lane&7) [+8 for n-tile 1]
    const uint32_t ldm_row = static_cast<uint32_t>(lane & 7) * kD;
    const uint32_t ldm_c0 = static_cast<uint32_t>(((lane >> 3)) ^ (lane & 7)) << 4;         // chunks 0..3
    const uint32_t ldm_c1 = static_cast<uint32_t>((4 + (lane >> 3)) ^ (lane & 7)) << 4;     // chunks 4..7
    // V: transposed ldmatrix x4 number c (c = 0..3) fetches the 8x16-byte matrices (rows 0-7, chunk 2c), (rows 8-15,
    // chunk 2c), (rows 0-7, chunk 2c+1), (rows 8-15, chunk 2c+1); this lane supplies row (lane&7) of matrix (lane>>3)
    uint32_t v_off[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t mi = lane >> 3, r = lane & 7;
        v_off[c] = (8 * (mi & 1) + r) * kD + ((static_cast<uint32_t>(2 * c + (mi >> 1)) ^ r) << 4);
    }

    int stage = 0;
    uint32_t phase = 0;
    for (int i = 0; i < ntiles; ++i) {
        if (!mbar_wait(bars + stage * 8, phase)) { failed = true; break; }
        const uint32_t pos0 = (t0 + i) * kTile;
        const int lo = begin > pos0 ? static_cast<int>(begin - pos0) : 0;
        const int hi = end - pos0 < static_cast<uint32_t>(kTile) ? static_cast<int>(end - pos0) : kTile;
        const uint32_t kt = smem_u32(k_ring + stage * L::kKTile);
        const uint32_t vt = v_ring_u + stage * L::kKTile;
        const uint8_t* kst = s_ring + stage * 2 * L::kSTile;
        const uint8_t* vst = kst + L::kSTile;

        // ---- scores of this lane: head g & 3, positions 8j + 2t + {0, 1} -------------------------
        float s[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            uint32_t kb[8];
            {
                uint32_t r[4];
                ldmatrix_x4(kt + j * 8 * kD + ldm_row + ldm_c0, r);
                kb[0] = r[0]; kb[1] = r[1]; kb[2] = r[2]; kb[3] = r[3];
                ldmatrix_x4(kt + j * 8 * kD + ldm_row + ldm_c1, r);
                kb[4] = r[0]; kb[5] = r[1]; kb[6] = r[2]; kb[7] = r[3];
            }
            if constexpr (NBLK == 4) {
                // scales of positions 8j+2t and 8j+2t+1: 2 x 4 halves, contiguous
                const uint4 raw = *reinterpret_cast<const uint4*>(kst + (8 * j + 2 * t) * 8);
                const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                const float2 a1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                const float2 b0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.z));
                const float2 b1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.w));
                const float ksa[4] = {a0.x, a0.y, a1.x, a1.y}, ksb[4] = {b0.x, b0.y, b1.x, b1.y};
                float sa = 0.0f, sb = 0.0f;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    int c[4];
                    mma_s8_zero(c, qa[ks], kb[2 * ks], kb[2 * ks + 1]);
                    sa = fmaf(static_cast<float>((c[0] << 7) + c[2]), ksa[ks], sa);
                    sb = fmaf(static_cast<float>((c[1] << 7) + c[3]), ksb[ks], sb);
                }
                s[j][0] = sa; s[j][1] = sb;
            } else {
                const __half2 raw = *reinterpret_cast<const __half2*>(kst + (8 * j + 2 * t) * 2);
                const float2 sc = __half22float2(raw);
                int c[4];
                mma_s8_zero(c, qa[0], kb[0], kb[1]);
#pragma unroll
                for (int ks = 1; ks < 4; ++ks) mma_s8(c, qa[ks], kb[2 * ks], kb[2 * ks + 1]);
                s[j][0] = static_cast<float>((c[0] << 7) + c[2]) * sc.x;
                s[j][1] = static_cast<float>((c[1] << 7) + c[3]) * sc.y;
            }
            s[j][0] *= qmul;
            s[j][1] *= qmul;
        }
        const bool partial = lo > 0 || hi < kTile;   // only the first and the last tile of a range
        if (partial) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int pos = 8 * j + 2 * t + e;
                    if (pos < lo || pos >= hi) s[j][e] = -INFINITY;
                }
        }

        // ---- online softmax, base 2, lazily updated reference maximum ----------------------------
        float mt_ = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 1));
        mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 2));
        const bool grow = mt_ > m_ref + kRescaleSlack;   // also true for the first tile (m_ref = -inf); NaN scores never grow
        if (__any_sync(0xffffffffu, grow)) {
            const float m_new = grow ? mt_ : m_ref;
            const float alpha = (m_ref == -INFINITY) ? 0.0f : exp2f(m_ref - m_new);   // 1 for heads that did not move
            l_run *= alpha;
            m_ref = m_new;
            // columns 2t, 2t+1 belong to heads (2t)&3, (2t+1)&3, whose factors sit in lanes 4*head
            const float a0 = __shfl_sync(0xffffffffu, alpha, ((2 * t) & 3) * 4);
            const float a1 = __shfl_sync(0xffffffffu, alpha, ((2 * t + 1) & 3) * 4);
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) { acc[mt][0] *= a0; acc[mt][1] *= a1; acc[mt][2] *= a0; acc[mt][3] *= a1; }
        }
        float w[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                w[j][e] = exp2f(s[j][e] - m_ref);   // masked positions: exp2(-inf) = 0 (m_ref is finite once a tile was seen)
                l_run += w[j][e];
            }

        // ---- weight operand: w * value_scale per block, high part or remainder depending on the lane ----
        uint32_t wb[NBLK][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float vs[2][NBLK];
            if constexpr (NBLK == 4) {
                const uint4 raw = *reinterpret_cast<const uint4*>(vst + (8 * j + 2 * t) * 8);
                const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                const float2 a1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                const float2 b0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.z));
                const float2 b1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.w));
                vs[0][0] = a0.x; vs[0][1] = a0.y; vs[0][2] = a1.x; vs[0][3] = a1.y;
                vs[1][0] = b0.x; vs[1][1] = b0.y; vs[1][2] = b1.x; vs[1][3] = b1.y;
            } else {
                const float2 sc = __half22float2(*reinterpret_cast<const __half2*>(vst + (8 * j + 2 * t) * 2));
                vs[0][0] = sc.x; vs[1][0] = sc.y;
            }
            if (partial) {   // masked positions have weight exactly 0, but their scales may be stale inf/nan
#pragma unroll
                for (int blk = 0; blk < NBLK; ++blk) {
                    if (!(w[j][0] > 0.0f)) vs[0][blk] = 0.0f;
                    if (!(w[j][1] > 0.0f)) vs[1][blk] = 0.0f;
                }
            }
#pragma unroll
            for (int blk = 0; blk < NBLK; ++blk) {
                const float e0 = w[j][0] * vs[0][blk];
                const float e1 = w[j][1] * vs[1][blk];
                const __half2 h2 = __floats2half2_rn(e0, e1);
                const float2 back = __half22float2(h2);
                const uint32_t rem = pack_half2(e0 - back.x, e1 - back.y);
                wb[blk][j] = remainder_lane ? rem : *reinterpret_cast<const uint32_t*>(&h2);
            }
        }

        // ---- P.V: A = V^T of this tile, exact fp16 integers --------------------------------------
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t vw[4];
            ldmatrix_x4_trans(vt + v_off[c], vw);
            const uint32_t b0 = wb[NBLK == 4 ? c : 0][0], b1 = wb[NBLK == 4 ? c : 0][1];
            mma_f16(acc[2 * c], s8_even_bytes_to_half2(vw[0]), s8_odd_bytes_to_half2(vw[0]),
                    s8_even_bytes_to_half2(vw[1]), s8_odd_bytes_to_half2(vw[1]), b0, b1);
            mma_f16(acc[2 * c + 1], s8_even_bytes_to_half2(vw[2]), s8_odd_bytes_to_half2(vw[2]),
                    s8_even_bytes_to_half2(vw[3]), s8_odd_bytes_to_half2(vw[3]), b0, b1);
        }

        __syncwarp();   // every lane is done with this stage
        if (lane == 0 && i + kStages < ntiles) issue(i + kStages, stage);
        if (++stage == kStages) { stage = 0; phase ^= 1; }
    }

    // ---- the warp's result into its merge area: acc[8 columns][128 dims], m[4], l[4] ----------------------
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (failed) { m_ref = __int_as_float(0x7fc00000); l_run = m_ref; }   // poison the partial
    float* mine = reinterpret_cast<float*>(k_ring);
    __syncwarp();
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
        const int dim = 16 * mt + 2 * g;
        *reinterpret_cast<float2*>(mine + (2 * t) * kD + dim) = make_float2(acc[mt][0], acc[mt][2]);
        *reinterpret_cast<float2*>(mine + (2 * t + 1) * kD + dim) = make_float2(acc[mt][1], acc[mt][3]);
    }
    if (t == 0 && g < 4) { mine[8 * kD + g] = m_ref; mine[8 * kD + 4 + g] = l_run; }
    __syncthreads();

    // ---- merge the CTA's warps: 256 threads = 2 head slots x 128 dims ---------------------------------------
    const int dim = threadIdx.x & (kD - 1);
    for (int h = threadIdx.x >> 7; h < G; h += 2) {
        float mw[kWarps], M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float* src = reinterpret_cast<const float*>(smem + w * L::kWarpArea);
            mw[w] = src[8 * kD + h];
            M = fmaxf(M, mw[w]);
        }
        float lt = 0.0f, at = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float* src = reinterpret_cast<const float*>(smem + w * L::kWarpArea);
            const float a = (mw[w] == -INFINITY) ? 0.0f : exp2f(mw[w] - M);   // NaN (poison) propagates
            lt = fmaf(src[8 * kD + 4 + h], a, lt);
            at = fmaf(src[h * kD + dim] + src[(4 + h) * kD + dim], a, at);
        }
        const uint32_t head = kv_head * G + h;
        const float m_nat = M * 0.6931471805599453f;   // natural-log units, as the merge expects
        tail::emit_partial(p, session, split, num_splits, head, dim, at, m_nat, lt);
    }
    if (failed) tail::report(p, B200KV_STATUS_COPY_TIMEOUT);
    if (p.ws_tagged == nullptr) return;   // a separate merge kernel follows
    // the CTA of split h merges query head h of this kv head once all splits' tagged partials have landed
    tail::fused_merge(p, session, kv_head, split, num_splits, G, reinterpret_cast<float*>(smem + L::kOffMisc));
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
int launch_one(const DecodeParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap, dim3 grid, cudaStream_t stream) {
    using L = Smem<NBLK>;
    static std::atomic<uint64_t> done{0};   // one per kernel instantiation: devices that have opted in
    const cudaError_t attr_err = opt_in_dynamic_smem(reinterpret_cast<const void*>(decode_q8_kernel<G, NBLK, Q_F16>), L::kAlloc, done);
    if (attr_err != cudaSuccess) { set_last_cuda_error(attr_err, "cudaFuncSetAttribute(decode_q8)"); return B200KV_ERR_CUDA; }
    B200KV_CUDA_TRY(launch_kernel(decode_q8_kernel<G, NBLK, Q_F16>, grid, dim3(kWarps * 32), L::kAlloc, stream, true, p, kmap, vmap));
    return B200KV_OK;
}

template <int G, int NBLK>
int launch_variant(const DecodeParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap, dim3 grid, cudaStream_t stream) {
    return p.q_is_f16 ? launch_one<G, NBLK, true>(p, kmap, vmap, grid, stream) : launch_one<G, NBLK, false>(p, kmap, vmap, grid, stream);
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

namespace {
int encode_plane_map(int8_t* plane, const b200kv_view& view, uint32_t tile_positions, CUtensorMap* out) {
    EncodeFn fn = encoder();
    if (fn == nullptr) return B200KV_ERR_UNSUPPORTED;
    const TensorMapKey key{plane, static_cast<uint64_t>(view.kv_heads) * view.capacity, static_cast<uint32_t>(kD), static_cast<uint32_t>(kD),
                           tile_positions, 1u};   // kind 1: bytes, 128-byte swizzle
    if (tensor_map_lookup(key, out)) return B200KV_OK;
    const cuuint64_t dims[2] = {kD, static_cast<cuuint64_t>(view.kv_heads) * view.capacity};
    const cuuint64_t strides[1] = {kD};
    const cuuint32_t box[2] = {kD, tile_positions};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, plane, dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return B200KV_ERR_UNSUPPORTED;
    tensor_map_remember(key, *out);
    return B200KV_OK;
}
}  // namespace

int encode_kv_maps(const b200kv_view& view, uint32_t tile_positions, CUtensorMap* kmap, CUtensorMap* vmap) {
    int rc = encode_plane_map(view.key_q8, view, tile_positions, kmap);
    if (rc == B200KV_OK) rc = encode_plane_map(view.value_q8, view, tile_positions, vmap);
    return rc;
}

uint32_t pick_splits_q8(const b200kv_view& geometry, uint32_t query_heads, uint32_t sessions, uint32_t max_length) {
    if (!q8_fast_path_ok(geometry, query_heads)) return 0;
    // two CTAs of 8 warps per SM; every warp should see at least two tiles
    const uint32_t ctas = 148u * 2u;
    const uint32_t units = geometry.kv_heads * sessions;
    uint32_t s = (ctas + units / 2) / units;   // nearest to one full wave
    if (s == 0) s = 1;
    if (sessions > 1) {   // mixed lengths: enough splits that the longest session is cut into kPositionsPerSplit pieces
        const uint32_t by_length = (max_length + kPositionsPerSplit - 1) / kPositionsPerSplit;
        if (by_length > s) s = by_length;
    }
    const uint32_t tiles = (max_length + kTile - 1) / kTile;
    uint32_t by_tiles = tiles / (2 * kWarps);
    if (by_tiles == 0) by_tiles = 1;
    if (s > by_tiles) s = by_tiles;
    const uint32_t cap = max_splits_per_session(sessions);
    if (s > cap) s = cap;
    return s ? s : 1;
}

int launch_decode_q8(const DecodeParams& p_in, const b200kv_view& geometry, uint32_t max_length, cudaStream_t stream) {
    if (!q8_fast_path_ok(geometry, p_in.query_heads)) return B200KV_ERR_UNSUPPORTED;
    DecodeParams p = p_in;
    p.overlap_tail = launch_overlap_tail();
    // Batched launches: the split count is that of the longest session; a session gets one split per
    // `split_positions` of its own length (a multiple of the 128 positions one round of the 8 warps covers).
    const uint32_t per_split = (max_length + p.num_splits - 1) / (p.num_splits ? p.num_splits : 1);
    p.split_positions = (per_split + 127u) / 128u * 128u;
    if (p.split_positions < 256u) p.split_positions = 256u;
    CUtensorMap kmap, vmap;
    if (p.views == nullptr) {
        int rc = encode_kv_maps(geometry, kTile, &kmap, &vmap);
        if (rc != B200KV_OK) return rc;
    } else {
        std::memset(&kmap, 0, sizeof kmap);   // per-session descriptors come from the device table
        std::memset(&vmap, 0, sizeof vmap);
    }
    const uint32_t g = p.query_heads / geometry.kv_heads;
    const bool blocks = geometry.qblock == 32;
    dim3 grid(p.num_splits, geometry.kv_heads, p.sessions);
    switch (g) {
        case 1: return blocks ? launch_variant<1, 4>(p, kmap, vmap, grid, stream) : launch_variant<1, 1>(p, kmap, vmap, grid, stream);
        case 2: return blocks ? launch_variant<2, 4>(p, kmap, vmap, grid, stream) : launch_variant<2, 1>(p, kmap, vmap, grid, stream);
        default: return blocks ? launch_variant<4, 4>(p, kmap, vmap, grid, stream) : launch_variant<4, 1>(p, kmap, vmap, grid, stream);
    }
}

}  // namespace b200kv
