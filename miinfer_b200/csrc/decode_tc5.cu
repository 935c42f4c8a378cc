// Streaming split-K GQA decode attention over an int8 (q8_0 or row-scaled) KV cache on the 5th-generation tensor
// cores: tcgen05.mma kind::i8 with accumulators in TMEM, operands straight from the TMA-filled shared-memory tiles.
//
// What it computes is MIInfer's decode stage 1 (gfx906/kernels/qwen3_primitives.hip:7371-7485) with block scales,
// followed in the same launch by its stage 2 (decode_tail.cuh).  Why it exists next to decode_q8.cu: with warp-level
// mma every K and V byte still travels through registers (ldmatrix, int8 -> fp16 conversion of V, fragment
// shuffling), about 560 warp instructions per 16 positions, and instruction issue, not HBM, bounds that kernel.
// Here the cache bytes never enter a register:
//
//  * One CTA = one (kv head, split).  A producer thread streams tiles of 128 positions -- K and V through tensor
//    maps with the 128-byte swizzle (rows of 128 int8 = one swizzle row), the two fp16 scale tiles with bulk
//    copies -- into a 3-stage ring; one mbarrier per stage.
//  * S^T = K . Q^T: the K tile as it lies is the A operand (M = 128 positions, K-major), Q is quantised once per
//    launch to 15 bits per head (q = 128 hi + lo, two int8 planes = 8 of the 16 rows of the B operand).  One MMA
//    per q8_0 block of 32 dims (kind::i8 has K = 32), each into its own 16 TMEM columns, so the per-block key
//    scales can be applied to exact int32 sums: 128 threads (one per position = TMEM lane) read their 32 sums with
//    tcgen05.ld and finish the scores in fp32.
//  * Online softmax in base 2: the tile maximum per head is found with redux.sync inside each warp and one exchange
//    through shared memory between the four warps; the running maximum is uniform across the CTA.
//  * O^T += V^T . P: the V tile as it lies is the A operand again, this time MN-major (M = 128 dims, K = positions),
//    and P is written by the 128 threads as unsigned 16-bit fixed point in two uint8 planes, pre-multiplied by the
//    value scale of each block: P[position][(block, plane, head)] = 32 B-operand columns, MN-major too (rows of 32
//    bytes, 32-byte swizzle), so that a thread stores its position's 32 bytes with two 16-byte stores and one MMA
//    chain yields, for every dim, the sums of all four blocks' weightings, of which the thread of that dim keeps its
//    own block's (the other three quarters are the price of per-block value scales: tensor throughput is not what
//    bounds this kernel).  The fixed-point scale is per tile, head and block (tile maximum of the weights x tile
//    maximum of the value scales / 65535), so the int32 sums are exact and every tile is folded into fp32 accumulators
//    in registers (4 per thread) once its MMA chain has completed; rescaling at a new maximum costs a dozen multiplies.
//    P and the sums are double-buffered, so the softmax threads never wait for the chain of the tile they have just
//    handed over.
//  * The CTA's partial leaves as tagged words and the CTA of split h merges head h (decode_tail.cuh), as in decode_q8.cu.
//  * Every wait is bounded.  A wait that runs out sets a status bit, poisons the partial with NaN and lets the CTA
//    finish in the normal way (all later waits are skipped, barriers are still attended, TMEM is freed).
#include "decode_tail.cuh"

#include <climits>
#include <cstring>

namespace b200kv {

namespace {

constexpr int kD = 128;
constexpr int kTileM = 128;            // positions per tile = rows of the S MMA = TMEM lanes
constexpr int kStages = 3;
// Warps 0-3: softmax threads, one per position of a tile (TMEM lane = position = tid).  Warp 4: TMA producer.  Warp 5:
// issuer of the S = K.Q^T MMAs and TMEM owner.  Warp 6: issuer of the P.V MMAs.  Warp 7: the fused single-token
// append.  Two issuers, so that each sleeps on its own barriers instead of one thread polling both (a polling warp
// takes issue slots from the softmax warps).  (Two softmax threads per position, each with two of the four heads,
// measured no faster: in steady state the loop runs at the memory system's pace either way.)
constexpr int kThreads = 256;
constexpr int kConsumers = 128;
constexpr int kProducerWarp = 4, kMmaWarp = 5, kPvWarp = 6, kAppendWarp = 7;
constexpr uint32_t kSpin = 1u << 20;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0;          // two S buffers of 4 blocks x 16 columns
constexpr uint32_t kColO = 128;        // two O buffers of 32 columns: (block, plane, head)
constexpr float kPMax = 65535.0f;
constexpr int kEarlyTiles = 2;         // ring stages filled before the launch is released (3 measured no better: the early
                                       // copies of a launch compete with the merge of the one before it; pulling later
                                       // tiles -- its own, or through a hint the next launch's -- towards L2 measured slower)

template <int NBLK>
struct Smem {
    static constexpr int kKTile = kTileM * kD;                        // 16384
    static constexpr int kSTile = kTileM * NBLK * 2;                  // 1024 (q8_0) or 256 (row scale)
    static constexpr int kOffK = 0;
    static constexpr int kOffV = kStages * kKTile;
    static constexpr int kOffP = 2 * kStages * kKTile;                // 2 x [128 positions][32 B], MN-major, 32-byte swizzle
    static constexpr int kOffQ = kOffP + 2 * kTileM * 32;             // [8 rows][128 B]: the Q planes (rows 8-15 of the 16-row operand: see below)
    static constexpr int kOffS = kOffQ + 8 * 128;                     // [stage][ks | vs]
    static constexpr int kOffXch = kOffS + kStages * 2 * kSTile;      // [2 parities][4 warps][8] words: tile maxima
    static constexpr int kOffL = kOffXch + 2 * 4 * 8 * 4;             // [4 warps][4] row sums
    static constexpr int kOffQmul = kOffL + 64;                       // [4]
    static constexpr int kOffBar = kOffQmul + 16;
    static constexpr int kNumBars = 2 * kStages + 9;                  // full[3] empty[3] s_full[2] s_empty[2] p_full[2] p_empty[2] row
    static constexpr int kOffMisc = kOffBar + kNumBars * 8;           // tmem slot, fail flag
    static constexpr int kTotal = kOffMisc + 16;
    static constexpr int kAlloc = kTotal + 1024;                      // slack to align the base to 1024
};
static_assert(Smem<4>::kAlloc <= 115712, "two CTAs per SM");
static_assert(2 * kTileM * 32 >= (8 + 3 * 64 * 2) * 4, "the merger's scratch fits where P was");

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

// Shared-memory matrix descriptor (sm_100 format): start address, leading/stride byte offsets (all >> 4),
// descriptor version 1, swizzle mode.  K-major operands: rows of 128 bytes, 8-row groups `sbo` apart.
// MN-major operands: one swizzle span (128 or 32 bytes) contiguous along M/N, consecutive k one span apart, groups of
// 8 k `sbo` apart, further spans along M/N `lbo` apart.
// `layout`: 2 = 128-byte swizzle, 6 = 32-byte swizzle.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(layout) << 61;
    return d;
}
// Instruction descriptor for kind::i8: int32 accumulate; operand formats (1 = signed, 0 = unsigned) and majors
// (0 = K-major, 1 = MN-major).
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
// 8 consecutive 32-bit columns of this thread's TMEM lane (issue only; pair with tmem_ld_wait)
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Order-preserving map of fp32 to int32 (for redux.sync.max) and back.
__device__ __forceinline__ int ordered(float f) { const int i = __float_as_int(f); return i ^ ((i >> 31) & 0x7fffffff); }
__device__ __forceinline__ float unordered(int i) { return __int_as_float(i ^ ((i >> 31) & 0x7fffffff)); }

// NBLK scales per row (4 = q8_0 blocks of 32, 1 = one per row); up to 4 query heads per kv head.
template <int NBLK, bool Q_F16>
__global__ void __launch_bounds__(kThreads, 2)
decode_tc5_kernel(const __grid_constant__ DecodeParams p, const __grid_constant__ CUtensorMap kmap_single,
                  const __grid_constant__ CUtensorMap vmap_single) {
    using L = Smem<NBLK>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 1024-aligned, still a shared-space pointer
    const uint32_t sbase = smem_u32(smem);

    pdl_launch_dependents();   // the next kernel of the stream may become resident as SMs free up; it orders itself

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // single-session launches put the kv head fastest (measured 0.4 us per launch better than split fastest at 32K: the CTAs that are dispatched last, into
    // the slots the previous launch's mergers hold longest, are then spread over all kv heads instead of being two heads'
    // worth; giving those last splits fewer tiles on top of that measured no better); batched launches keep the splits
    // fastest, which measured 2 % better there
    const uint32_t kv_head = p.head_fastest ? blockIdx.x : blockIdx.y, split = p.head_fastest ? blockIdx.y : blockIdx.x, session = blockIdx.z;
    // optional per-CTA time stamps (b200kv_set_timeline_buffer): 8 words per CTA -- start, dependency wait over, set-up
    // barrier passed, first S tile seen, loop end, last sums folded, partial emitted, merge done
    const bool TL = p.timeline != nullptr && session == 0;
    uint64_t* tl = TL ? p.timeline + (static_cast<size_t>(kv_head) * (p.head_fastest ? gridDim.y : gridDim.x) + split) * 8 : nullptr;
    if (TL && tid == 0) tl[0] = global_ns();
    const b200kv_view& view = session_view(p, session);
    uint32_t begin, end;
    resolve_range(p, session, view, &begin, &end);
    const int G = static_cast<int>(p.query_heads / view.kv_heads);

    // Batched launches size the grid for the longest session; a shorter session uses only as many splits as its
    // own length warrants (every CTA of the session derives the same number) and the surplus CTAs leave at once.
    uint32_t num_splits = p.num_splits;
    if (p.lengths != nullptr) {
        const uint32_t want = (end - begin + p.split_positions - 1) / p.split_positions;
        num_splits = min(num_splits, max(want, 1u));
        if (split >= num_splits) return;
    }

    // ---- this CTA's tiles (tiles are aligned to multiples of 128 positions of the cache) --------------------
    const uint32_t tile_begin = begin / kTileM, tile_end = (end + kTileM - 1) / kTileM;
    const uint64_t total_tiles = end > begin ? tile_end - tile_begin : 0;
    const uint32_t t0 = tile_begin + static_cast<uint32_t>(total_tiles * split / num_splits);
    const uint32_t t1 = tile_begin + static_cast<uint32_t>(total_tiles * (split + 1) / num_splits);
    const int ntiles = static_cast<int>(t1 - t0);
    const bool fuse = p.new_key != nullptr;
    const bool owner = fuse && ntiles > 0 && t1 == tile_end;   // this CTA holds the tile of the appended token
    // With launch overlap the previous kernel may still be appending: rows at or above early_end wait for it.  The
    // row a fused append writes is never loaded early either.
    uint32_t early_end = end > p.overlap_tail ? end - p.overlap_tail : 0;
    if (fuse && early_end >= end) early_end = end - 1;

    const uint32_t bar0 = sbase + L::kOffBar;
    auto bar_full = [&](int s) { return bar0 + s * 8; };
    auto bar_empty = [&](int s) { return bar0 + (kStages + s) * 8; };
    auto bar_s_full = [&](int b) { return bar0 + (2 * kStages + b) * 8; };
    auto bar_s_empty = [&](int b) { return bar0 + (2 * kStages + 2 + b) * 8; };
    auto bar_p_full = [&](int b) { return bar0 + (2 * kStages + 4 + b) * 8; };
    auto bar_p_empty = [&](int b) { return bar0 + (2 * kStages + 6 + b) * 8; };
    const uint32_t bar_row = bar0 + (2 * kStages + 8) * 8;   // the appended row is in the cache
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
    uint32_t* fail_flag = tmem_slot + 1;

    const uint64_t head_row0 = static_cast<uint64_t>(kv_head) * view.capacity;
    const CUtensorMap* kmap = p.views != nullptr ? &p.views[session].kmap128 : &kmap_single;
    const CUtensorMap* vmap = p.views != nullptr ? &p.views[session].vmap128 : &vmap_single;
    const uint8_t* ks_plane = static_cast<const uint8_t*>(view.key_scales) + head_row0 * NBLK * 2;
    const uint8_t* vs_plane = static_cast<const uint8_t*>(view.value_scales) + head_row0 * NBLK * 2;
    const uint32_t capacity = static_cast<uint32_t>(view.capacity);
    const int row_base = static_cast<int>(head_row0);

    // Tile i of this CTA into ring stage i % kStages (producer thread only).
    auto issue = [&](int i) {
        const int stage = i % kStages;
        const uint32_t pos0 = (t0 + i) * kTileM;
        const uint32_t sbytes = min(static_cast<uint32_t>(kTileM), capacity - pos0) * (NBLK * 2);
        const uint32_t bar = bar_full(stage);
        mbar_expect_tx(bar, 2 * L::kKTile + 2 * sbytes);
        tma_load_2d(sbase + L::kOffK + stage * L::kKTile, kmap, 0, row_base + static_cast<int>(pos0), bar);
        tma_load_2d(sbase + L::kOffV + stage * L::kKTile, vmap, 0, row_base + static_cast<int>(pos0), bar);
        const uint32_t sdst = sbase + L::kOffS + stage * 2 * L::kSTile;
        bulk_load(sdst, ks_plane + static_cast<size_t>(pos0) * (NBLK * 2), sbytes, bar);
        bulk_load(sdst + L::kSTile, vs_plane + static_cast<size_t>(pos0) * (NBLK * 2), sbytes, bar);
    };

    // ---- set-up ---------------------------------------------------------------------------------------------
    int issued = 0;
    if (warp == kProducerWarp) {
        if (lane == 0) {
            for (int s = 0; s < kStages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
            for (int b = 0; b < 2; ++b) {
                mbar_init(bar_s_full(b), 1); mbar_init(bar_s_empty(b), kConsumers);
                mbar_init(bar_p_full(b), kConsumers); mbar_init(bar_p_empty(b), 1);
            }
            mbar_init(bar_row, 1);
            *fail_flag = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            // old cache rows do not depend on the preceding kernels: start streaming them before waiting for those
            while (issued < kEarlyTiles && issued < ntiles && (t0 + issued + 1) * kTileM <= early_end) { issue(issued); ++issued; }
        }
    } else if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_wait();
    if (TL && tid == 0) tl[1] = global_ns();
    // The new row of a fused append is fetched now, while the memory system is still quiet (once the rings stream, a
    // dependent load waits behind megabytes of queued tile traffic); its own warp transforms and stores it after the
    // set-up barrier, while the other warps are already at work on the tiles before it.
    float new_k[4], new_v[4];
    const bool appends = warp == kAppendWarp && owner;
    if (appends) {
        tail::load_new_row(p.new_key, p.new_is_f16, kv_head, lane, new_k);
        tail::load_new_row(p.new_value, p.new_is_f16, kv_head, lane, new_v);
    }
    if (warp == kProducerWarp && lane == 0) {
        const int limit = owner ? ntiles - 1 : ntiles;   // the tile that holds the appended row is loaded only after the row is stored
        while (issued < kStages && issued < limit) { issue(issued); ++issued; }
    }

    // ---- Q: 15 bits per head as two int8 planes.  Rows of the B operand of S^T = K . Q^T:
    //      [hi h0 .. hi h3, lo h0 .. lo h3].  The operand has 16 rows (the smallest N next to
    //      M = 128 that every kind::i8 shape table lists); rows 8-15 are whatever follows in shared memory (the scale
    //      tiles): they only produce columns 8-15 of S, which nobody reads, and integer sums of arbitrary bytes are harmless ----
    if (warp < 4) {
        uint32_t hi4 = 0, lo4 = 0;
        float qm = 0.0f;
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
            qm = (amax / 16319.0f) * p.scale * 1.4426950408889634f;
        }
        if (lane == 0) reinterpret_cast<float*>(smem + L::kOffQmul)[warp] = qm;
        // dims 4*lane .. 4*lane+3 of row n: 16-byte chunk (lane >> 2) ^ (n & 7), bytes (lane & 3) * 4
        const int n_hi = warp, n_lo = 4 + warp;
        *reinterpret_cast<uint32_t*>(smem + L::kOffQ + n_hi * 128 + ((((lane >> 2) ^ (n_hi & 7))) << 4) + (lane & 3) * 4) = hi4;
        *reinterpret_cast<uint32_t*>(smem + L::kOffQ + n_lo * 128 + ((((lane >> 2) ^ (n_lo & 7))) << 4) + (lane & 3) * 4) = lo4;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // Q was written by ordinary stores, the MMA reads it through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (TL && tid == 0) tl[2] = global_ns();

    bool failed = false;

    if (warp == kProducerWarp) {
        // =============================== TMA producer ===============================
        if (lane == 0) {
            for (int i = issued; i < ntiles; ++i) {
                // stage i % kStages is free once the P.V of tile i - kStages has completed
                if (i >= kStages && !mbar_wait(bar_empty(i % kStages), static_cast<uint32_t>((i / kStages - 1) & 1))) { failed = true; break; }
                if (owner && i == ntiles - 1 && !mbar_wait(bar_row, 0)) { failed = true; break; }
                issue(i);
            }
        }
    } else if (warp == kAppendWarp) {
        // =============================== fused append of the new token's row ===============================
        if (appends) {
            tail::fused_append_row<NBLK>(p, view, new_k, new_v, end - 1, head_row0 + end - 1, lane);
            __threadfence();
            asm volatile("fence.proxy.async;" ::: "memory");   // the row goes to the cache first; its tile is read by TMA (async proxy) afterwards
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_row);
        }
    } else if (warp == kMmaWarp) {
        // =============================== issuer of S^T = K . Q^T ===============================
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_i8(kTileM, 16, 1, 1, 0);   // K (signed) x Q planes (signed), both K-major
            for (int i = 0; i < ntiles; ++i) {
                const int stage = i % kStages, buf = i & 1;
                if (!mbar_wait(bar_s_empty(buf), static_cast<uint32_t>(((i >> 1) & 1) ^ 1))) { failed = true; break; }   // S buffer read out (tile i - 2)
                if (!mbar_wait(bar_full(stage), static_cast<uint32_t>((i / kStages) & 1))) { failed = true; break; }     // tile landed
                tc_fence_after();
                const uint32_t kt = sbase + L::kOffK + stage * L::kKTile;
#pragma unroll
                for (int b = 0; b < 4; ++b)   // one q8_0 block of 32 dims per MMA, each into its own 16 columns
                    umma_i8(tmem_base + kColS + buf * 64 + b * 16, umma_desc(kt + 32 * b, 16, 1024, 2),
                            umma_desc(sbase + L::kOffQ + 32 * b, 16, 1024, 2), idesc_s, 0);
                umma_commit(bar_s_full(buf));
            }
        }
    } else if (warp == kPvWarp) {
        // =============================== issuer of O^T = V^T . P ===============================
        if (lane == 0) {
            constexpr uint32_t idesc_o = umma_idesc_i8(kD, 32, 1, 0, 1, 1);    // V^T (signed, MN-major) x P planes (unsigned, MN-major)
            for (int i = 0; i < ntiles; ++i) {
                const int stage = i % kStages, buf = i & 1;
                if (!mbar_wait(bar_p_full(buf), static_cast<uint32_t>((i >> 1) & 1))) { failed = true; break; }
                if (!mbar_wait(bar_full(stage), static_cast<uint32_t>((i / kStages) & 1))) { failed = true; break; }   // long complete: the V tile's landing, observed by this thread
                tc_fence_after();
                const uint32_t vt = sbase + L::kOffV + stage * L::kKTile;
                const uint32_t pt = sbase + L::kOffP + buf * (kTileM * 32);
#pragma unroll
                for (int j = 0; j < 4; ++j)   // 32 positions per MMA
                    umma_i8(tmem_base + kColO + buf * 32, umma_desc(vt + j * (32 * kD), kTileM * kD, 1024, 2),
                            umma_desc(pt + j * (32 * 32), 32, 256, 6), idesc_o, j > 0);
                umma_commit(bar_p_empty(buf));      // P buffer free, the tile's sums complete
                umma_commit(bar_empty(stage));      // ring stage may be refilled
            }
        }
    }

    // what the softmax threads hand to the epilogue: this thread's dim (= tid), heads 0..3, relative to m_run
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float m_run[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};

    if (warp < 4) {
        // =============================== softmax threads: one per position of a tile ===============================
        const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
        float qmul[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) qmul[h] = reinterpret_cast<const float*>(smem + L::kOffQmul)[h];
        // P is the MN-major B operand: this position's 32 bytes (column n = 8*block + 4*plane + head) form one row of
        // 32 bytes, 32-byte swizzle: 16-byte chunk c of row r sits at 32 r + ((c ^ ((r >> 2) & 1)) << 4)
        const uint32_t p_row = static_cast<uint32_t>(tid) * 32u;
        const uint32_t p_flip = static_cast<uint32_t>((tid >> 2) & 1) << 4;
        int* xch = reinterpret_cast<int*>(smem + L::kOffXch);
        float l_run[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // sums over this thread's positions only
        // per O buffer: fixed-point scale of the sums in flight (own block), relative to m_run
        float pend_a[4] = {0.0f, 0.0f, 0.0f, 0.0f}, pend_b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        auto wait = [&](uint32_t bar, uint32_t parity) { if (!failed && !mbar_wait(bar, parity)) failed = true; };
        auto fold_o = [&](int buf) {   // the completed sums of a tile: own block's 8 columns -> fp32 accumulators
            int o[8];
            tc_fence_after();
            tmem_ld8(tmem_base + lane_addr + kColO + buf * 32 + warp * 8, o);
            tmem_ld_wait();
            tc_fence_before();
#pragma unroll
            for (int h = 0; h < 4; ++h) acc[h] = fmaf(static_cast<float>(o[h] * 256 + o[4 + h]), buf ? pend_b[h] : pend_a[h], acc[h]);
        };

        for (int i = 0; i < ntiles; ++i) {
            const int stage = i % kStages, buf = i & 1;
            wait(bar_full(stage), static_cast<uint32_t>((i / kStages) & 1));      // the scale tiles of this stage (async-proxy writes)
            wait(bar_s_full(buf), static_cast<uint32_t>((i >> 1) & 1));
            if (TL && i == 0 && tid == 0) tl[3] = global_ns();
            tc_fence_after();
            int sv[4][8];   // per block: hi sums of heads 0-3, lo sums of heads 0-3
#pragma unroll
            for (int b = 0; b < 4; ++b) tmem_ld8(tmem_base + lane_addr + kColS + buf * 64 + b * 16, sv[b]);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(bar_s_empty(buf));   // this thread's part of S is in registers

            const uint32_t pos = (t0 + i) * kTileM + tid;
            const bool valid = pos >= begin && pos < end;
            const uint8_t* kst = smem + L::kOffS + stage * 2 * L::kSTile;
            const uint8_t* vst = kst + L::kSTile;
            float ks[4], vs[4];
            uint32_t vs_bits[NBLK];
            if constexpr (NBLK == 4) {
                const uint2 kr = *reinterpret_cast<const uint2*>(kst + tid * 8), vr = *reinterpret_cast<const uint2*>(vst + tid * 8);
                const float2 k01 = __half22float2(*reinterpret_cast<const __half2*>(&kr.x)), k23 = __half22float2(*reinterpret_cast<const __half2*>(&kr.y));
                const float2 v01 = __half22float2(*reinterpret_cast<const __half2*>(&vr.x)), v23 = __half22float2(*reinterpret_cast<const __half2*>(&vr.y));
                ks[0] = k01.x; ks[1] = k01.y; ks[2] = k23.x; ks[3] = k23.y;
                vs[0] = v01.x; vs[1] = v01.y; vs[2] = v23.x; vs[3] = v23.y;
                vs_bits[0] = vr.x & 0xffffu; vs_bits[1] = vr.x >> 16; vs_bits[2] = vr.y & 0xffffu; vs_bits[3] = vr.y >> 16;
            } else {
                const uint16_t kr = *reinterpret_cast<const uint16_t*>(kst + tid * 2), vr = *reinterpret_cast<const uint16_t*>(vst + tid * 2);
                ks[0] = ks[1] = ks[2] = ks[3] = __half2float(__ushort_as_half(kr));
                vs[0] = vs[1] = vs[2] = vs[3] = __half2float(__ushort_as_half(vr));
                vs_bits[0] = vr;
            }
            // scores of this position, base-2 units; positions outside the range (or rows never written) are masked
            float s[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                float a = 0.0f;
                if constexpr (NBLK == 4) {
#pragma unroll
                    for (int b = 0; b < 4; ++b) a = fmaf(static_cast<float>(sv[b][h] * 128 + sv[b][4 + h]), ks[b], a);
                } else {
                    a = static_cast<float>((sv[0][h] + sv[1][h] + sv[2][h] + sv[3][h]) * 128 + (sv[0][4 + h] + sv[1][4 + h] + sv[2][4 + h] + sv[3][4 + h])) * ks[0];
                }
                s[h] = valid ? a * qmul[h] : -INFINITY;
            }
            // ---- tile maxima (scores per head, value scales per block): redux inside the warp, one exchange across the four ----
            {
                int mx[4];
                uint32_t vmx[NBLK];
#pragma unroll
                for (int h = 0; h < 4; ++h) mx[h] = __reduce_max_sync(0xffffffffu, ordered(s[h]));
#pragma unroll
                for (int b = 0; b < NBLK; ++b) vmx[b] = __reduce_max_sync(0xffffffffu, valid ? vs_bits[b] : 0u);   // positive fp16 order like integers
                if (lane == 0) {
                    int* dst = xch + (buf * 4 + warp) * 8;
                    *reinterpret_cast<int4*>(dst) = make_int4(mx[0], mx[1], mx[2], mx[3]);
                    if constexpr (NBLK == 4) *reinterpret_cast<uint4*>(dst + 4) = make_uint4(vmx[0], vmx[1], vmx[2], vmx[3]);
                    else dst[4] = static_cast<int>(vmx[0]);
                }
            }
            asm volatile("bar.sync 3, 128;" ::: "memory");
            float m_tile[4], vs_max[4];
            {
                int mx[4] = {INT_MIN, INT_MIN, INT_MIN, INT_MIN};
                uint32_t vmx[4] = {0, 0, 0, 0};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int* src = xch + (buf * 4 + w) * 8;
                    const int4 a = *reinterpret_cast<const int4*>(src);
                    mx[0] = max(mx[0], a.x); mx[1] = max(mx[1], a.y); mx[2] = max(mx[2], a.z); mx[3] = max(mx[3], a.w);
                    if constexpr (NBLK == 4) {
                        const uint4 b = *reinterpret_cast<const uint4*>(src + 4);
                        vmx[0] = max(vmx[0], b.x); vmx[1] = max(vmx[1], b.y); vmx[2] = max(vmx[2], b.z); vmx[3] = max(vmx[3], b.w);
                    } else {
                        vmx[0] = max(vmx[0], static_cast<uint32_t>(src[4]));
                    }
                }
#pragma unroll
                for (int h = 0; h < 4; ++h) m_tile[h] = unordered(mx[h]);
#pragma unroll
                for (int b = 0; b < 4; ++b) vs_max[b] = __half2float(__ushort_as_half(static_cast<uint16_t>(vmx[NBLK == 4 ? b : 0])));
            }
            // ---- online softmax: new running maximum, weights, and the tile's fixed-point scales ----
            float wn[4], nscale[4];   // weights normalised to the tile maximum (<= 1); fixed-point scale of this tile (own block)
            const float vs_own = warp == 0 ? vs_max[0] : warp == 1 ? vs_max[1] : warp == 2 ? vs_max[2] : vs_max[3];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const float m_new = fmaxf(m_run[h], m_tile[h]);
                const float alpha = (m_run[h] == -INFINITY) ? 0.0f : exp2f(m_run[h] - m_new);
                acc[h] *= alpha; l_run[h] *= alpha; pend_a[h] *= alpha; pend_b[h] *= alpha;
                m_run[h] = m_new;
                const float w = (s[h] == -INFINITY) ? 0.0f : exp2f(s[h] - m_new);
                l_run[h] += w;
                const float wmax = (m_tile[h] == -INFINITY) ? 0.0f : exp2f(m_tile[h] - m_new);
                wn[h] = wmax > 0.0f ? __fdividef(w, wmax) : 0.0f;
                nscale[h] = wmax * vs_own * (1.0f / kPMax);
            }
            // [block]: w * value_scale as 16-bit fixed point, then the planes: hi bytes of heads 0-3, lo bytes of heads 0-3
            uint32_t p_hi[4], p_lo[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float wv = (valid && vs_max[b] > 0.0f) ? vs[b] * __fdividef(kPMax, vs_max[b]) : 0.0f;
                uint32_t pq[4];
#pragma unroll
                for (int h = 0; h < 4; ++h) pq[h] = min(__float2uint_rn(wn[h] * wv), 65535u);
                const uint32_t p01 = pq[0] | (pq[1] << 16), p23 = pq[2] | (pq[3] << 16);
                p_hi[b] = __byte_perm(p01, p23, 0x7531);
                p_lo[b] = __byte_perm(p01, p23, 0x6420);
            }
            // ---- P and O buffer `buf` were last used by tile i - 2: its P.V has completed; fold its sums first ----
            if (i >= 2) {
                wait(bar_p_empty(buf), static_cast<uint32_t>(((i >> 1) - 1) & 1));
                fold_o(buf);
            }
#pragma unroll
            for (int h = 0; h < 4; ++h) { if (buf) pend_b[h] = nscale[h]; else pend_a[h] = nscale[h]; }
            const uint32_t pt = sbase + L::kOffP + buf * (kTileM * 32) + p_row;
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(pt + p_flip), "r"(p_hi[0]), "r"(p_lo[0]), "r"(p_hi[1]), "r"(p_lo[1]) : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(pt + (p_flip ^ 16u)), "r"(p_hi[2]), "r"(p_lo[2]), "r"(p_hi[3]), "r"(p_lo[3]) : "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(bar_p_full(buf));
        }
        if (TL && tid == 0) tl[4] = global_ns();
        // the last two tiles' sums
        if (ntiles >= 2) {
            const int buf = (ntiles - 2) & 1;
            wait(bar_p_empty(buf), static_cast<uint32_t>(((ntiles - 2) >> 1) & 1));
            fold_o(buf);
        }
        if (ntiles >= 1) {
            const int buf = (ntiles - 1) & 1;
            wait(bar_p_empty(buf), static_cast<uint32_t>(((ntiles - 1) >> 1) & 1));
            fold_o(buf);
        }
        if (TL && tid == 0) tl[5] = global_ns();
        // ---- row sums over the CTA, then the CTA's partial leaves at once: thread = dim holds all four heads ----
#pragma unroll
        for (int h = 0; h < 4; ++h) l_run[h] = warp_sum(l_run[h]);
        if (lane == 0) {
            *reinterpret_cast<float4*>(smem + L::kOffL + warp * 16) = make_float4(l_run[0], l_run[1], l_run[2], l_run[3]);
            if (failed) atomicOr(fail_flag, 1u);
        }
        asm volatile("bar.sync 3, 128;" ::: "memory");
        float lt[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float4 a = *reinterpret_cast<const float4*>(smem + L::kOffL + w * 16);
            lt[0] += a.x; lt[1] += a.y; lt[2] += a.z; lt[3] += a.w;
        }
        // a wait that ran out anywhere in the pipeline ends in a wait of these threads running out
        const bool poisoned = *reinterpret_cast<volatile uint32_t*>(fail_flag) != 0;
        if (poisoned && tid == 0) tail::report(p, B200KV_STATUS_PIPE_TIMEOUT);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            if (h >= G) break;
            float at = acc[h], mh = m_run[h] * 0.6931471805599453f, lh = lt[h];   // natural-log units, as the merge expects
            if (poisoned) { at = __int_as_float(0x7fc00000); mh = at; lh = at; }
            tail::emit_partial(p, session, split, num_splits, kv_head * G + h, tid, at, mh, lh);
        }
        if (TL && tid == 0) tl[6] = global_ns();
    }

    // ---- teardown: every role arrives here, with or without a timeout; TMEM is always released ----
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (p.ws_tagged == nullptr) return;   // a separate merge kernel follows
    // the CTA of split h merges query head h of this kv head once all splits' tagged partials have landed (256 threads;
    // the merger's scratch takes the place of the P buffers, which every MMA has long consumed)
    tail::fused_merge(p, session, kv_head, split, num_splits, G, reinterpret_cast<float*>(smem + L::kOffP));
    if (TL && tid == 0) tl[7] = global_ns();
}

// ---- host side -----------------------------------------------------------------------------------------

template <int NBLK, bool Q_F16>
int launch_one(const DecodeParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap, dim3 grid, cudaStream_t stream) {
    using L = Smem<NBLK>;
    static std::atomic<uint64_t> done{0};   // one per kernel instantiation: devices that have opted in
    const cudaError_t attr_err = opt_in_dynamic_smem(reinterpret_cast<const void*>(decode_tc5_kernel<NBLK, Q_F16>), L::kAlloc, done);
    if (attr_err != cudaSuccess) { set_last_cuda_error(attr_err, "cudaFuncSetAttribute(decode_tc5)"); return B200KV_ERR_CUDA; }
    B200KV_CUDA_TRY(launch_kernel(decode_tc5_kernel<NBLK, Q_F16>, grid, dim3(kThreads), L::kAlloc, stream, true, p, kmap, vmap));
    return B200KV_OK;
}

}  // namespace

int launch_decode_tc5(const DecodeParams& p_in, const b200kv_view& geometry, uint32_t max_length, cudaStream_t stream) {
    if (!q8_fast_path_ok(geometry, p_in.query_heads)) return B200KV_ERR_UNSUPPORTED;
    DecodeParams p = p_in;
    p.overlap_tail = launch_overlap_tail();
    // Batched launches: the split count is that of the longest session; a session gets one split per
    // `split_positions` of its own length (a multiple of the tile).
    const uint32_t per_split = (max_length + p.num_splits - 1) / (p.num_splits ? p.num_splits : 1);
    p.split_positions = (per_split + 127u) / 128u * 128u;
    if (p.split_positions < 256u) p.split_positions = 256u;
    CUtensorMap kmap, vmap;
    if (p.views == nullptr) {
        int rc = encode_kv_maps(geometry, kTileM, &kmap, &vmap);
        if (rc != B200KV_OK) return rc;
    } else {
        std::memset(&kmap, 0, sizeof kmap);   // per-session descriptors come from the device table
        std::memset(&vmap, 0, sizeof vmap);
    }
    const bool blocks = geometry.qblock == 32;
    p.head_fastest = p.lengths == nullptr ? 1u : 0u;
    const dim3 grid = p.head_fastest ? dim3(geometry.kv_heads, p.num_splits, p.sessions) : dim3(p.num_splits, geometry.kv_heads, p.sessions);
    if (blocks) return p.q_is_f16 ? launch_one<4, true>(p, kmap, vmap, grid, stream) : launch_one<4, false>(p, kmap, vmap, grid, stream);
    return p.q_is_f16 ? launch_one<1, true>(p, kmap, vmap, grid, stream) : launch_one<1, false>(p, kmap, vmap, grid, stream);
}

}  // namespace b200kv
