// Suffix / prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Same function as prefill_mma.cu (MIInfer's suffix kernels,
// gfx906/kernels/qwen3_primitives.hip:6788-7119 and 6637-6725), built for sm_100a:
//
//  1. A streaming pre-pass dequantises the positions the chunk can see, [0, kv_end), once per launch into an
//     fp16 scratch in the caller's workspace (K and V planes, [kv_head][row][d]); with int8 -> fp16 exact up to
//     the one rounding of q * scale.  The scratch (35.6 MB at 8704 x 4 x 256) stays in the 126 MB L2.
//  2. The attention kernel gives each CTA 128 query ROWS of one kv head (a row is a (token, head-of-group)
//     pair, so the G heads of a group share every K/V tile) and walks the causal range in tiles of 64 positions,
//     two tiles at a time:
//       - two threads feed the K ring (two stages of a PAIR of tiles each) and the V ring (two tiles) with TMA
//         tensor copies (64x64 boxes, 128-byte swizzle: exactly the canonical shared-memory layout of the MMA
//         operands; the two tiles of a pair lie in rows 0-63 and 64-127 of every slab, one B operand);
//       - one thread issues S = Q.K^T for a pair of tiles at once (tcgen05.mma M128 x N128, K = d, Q read from
//         TMEM: an MMA of this shape costs about the same at N = 64 and N = 128, so pairs halve the time the score
//         MMAs hold the tensor pipe), another O += P.V per tile (M128 x N = d, K = 64; V consumed MN-major, as
//         stored) into the O accumulator in TMEM; completion is tracked by tcgen05.commit on mbarriers;
//       - two groups of 128 softmax threads, one thread per row in each, take the first and the second tile of
//         every pair: tcgen05.ld the S row, scale/mask (causal length per row, .hip:6829), online softmax in base
//         2 with LAZY rescaling (O and the running sums are only rescaled when a row's maximum grows by more
//         than 2^8; P <= 256 fits fp16; the row's reference maximum is handed from tile to tile through shared
//         memory), write P as fp16 into one of two swizzled A-operand tiles, and at the end scale O by 1/sum,
//         apply the sigmoid gate (.hip:6714-6723) and store.
//     TMEM: S (pair) | Q | O = 128 + d/2 + d columns.  Shared memory: 2 x 2 K tiles + 2 V tiles + 2 P tiles.
// Every mbarrier wait is bounded; a wait that runs out poisons the output rows with NaN, and the CTA still frees
// its TMEM and exits.
#include "decode_common.cuh"
#include "dequant.cuh"

#include <cstring>
#include <mutex>

namespace b200kv {

namespace {

constexpr int kBM = 128;          // query rows per CTA
constexpr int kBN = 64;           // positions per KV tile
constexpr int kSoftmaxThreads = 256;              // two groups of one thread per query row: even tiles, odd tiles
constexpr int kTmaWarp = kSoftmaxThreads / 32;     // TMA producer of the K tiles
constexpr int kSWarp = kTmaWarp + 1;               // S = Q.K^T issuer / TMEM owner
constexpr int kPvWarp = kTmaWarp + 2;              // O += P.V issuer
constexpr int kTmaVWarp = kTmaWarp + 3;            // TMA producer of the V tiles (a K load never waits for a V stage)
constexpr int kThreads = kSoftmaxThreads + 128;
constexpr int kKPairs = 2;                         // K ring: stages of two tiles each (one S MMA covers a pair)
constexpr uint32_t kSpin = 1u << 20;
constexpr float kRescaleThreshold = 8.0f;        // log2 units

struct Tc5Params {
    CUtensorMap kmap, vmap;      // fp16 [kv_heads * rows][d], box 64 x 64, 128-byte swizzle
    const void* q;               // [token][query_heads][D]
    int q_is_f16;
    const float* gate;
    float* out;
    uint32_t token_count, base_position;
    const b200kv_prefill_state* prefill_state;
    uint32_t query_heads, kv_heads;
    uint64_t capacity;           // cache capacity (causal ranges past it give zero rows)
    uint32_t scratch_rows;       // rows per kv head in the fp16 scratch
    float scale_log2;
    // KV split: blockIdx.z walks tiles [ntiles*z/S, ntiles*(z+1)/S) of its rows and leaves an unnormalised partial
    // (O, reference maximum, sum) for prefill_merge_kernel.  kv_splits == 1: the kernel writes the output itself.
    uint32_t kv_splits;
    uint32_t rows_padded;        // query rows per kv head, rounded up to the row tile
    float* part_o;               // [split][kv_head][rows_padded][D]
    float2* part_ml;             // [split][kv_head][rows_padded] {maximum in log2 units, sum}
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpin; ++spin) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading/stride byte offsets (all >> 4),
// descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// Instruction descriptor for kind::f16: fp32 accumulate, fp16 A and B, M x N, operand majors (0 = K-major, 1 = MN-major).
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t m, uint32_t n, uint32_t a_mn_major, uint32_t b_mn_major) {
    return (1u << 4) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
        "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,"
        "%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
        "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32_bits(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,"
        "%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
          "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]),
          "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
          "r"(v[30]), "r"(v[31])
        : "memory");
}
// P.V with the A operand (P, fp16, K-major: one query row per TMEM lane, two elements per 32-bit column) read from TMEM
__device__ __forceinline__ void umma_f16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D>
struct Layout {
    static constexpr int kSlabs = D / 64;                  // 128-byte (64 x fp16) slabs along d
    static constexpr int kTileBytes = kSlabs * kBN * 128;  // one K or V tile: [slab][row][128 B]
    static constexpr int kPairBytes = 2 * kTileBytes;      // two K tiles as one B operand: [slab][128 rows][128 B]
    static constexpr int kOffK = 0;
    static constexpr int kOffV = kOffK + kKPairs * kPairBytes;
    static constexpr int kOffP = kOffV + 2 * kTileBytes;   // 2 x [row][128 B] fp16 P tiles
    static constexpr int kPBytes = kBM * 128;
    static constexpr int kOffBar = kOffP + 2 * kPBytes;
    static constexpr int kNumBars = 20;   // 16 used
    static constexpr int kOffRef = kOffBar + kNumBars * 8 + 16;   // [128 rows] {reference maximum, sequence}: handed from tile to tile
    static constexpr int kOffSum = kOffK;                         // [2 groups][128 rows] partial row sums: the K ring is idle in the epilogue
    static constexpr int kTotal = kOffRef + kBM * 8;
    static constexpr int kAlloc = kTotal;   // the dynamic shared memory is declared 1024-byte aligned; the kernel checks it
    static constexpr uint32_t kTmemCols = 512;
    static constexpr uint32_t kColS = 0, kColQ = 128, kColO = 256;   // S: 2 x 64, Q: D/2 (fp16 pairs), O: D
};

template <int D>
__global__ void __launch_bounds__(kThreads, 1) prefill_tc5_kernel(const __grid_constant__ Tc5Params p) {
    using L = Layout<D>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + L::kOffBar;
    auto bar = [&](int i) { return bar0 + i * 8; };
    enum { K_FULL = 0, K_EMPTY = 2, V_FULL = 4, V_EMPTY = 6, S_FULL = 8, S_EMPTY = 9, P_FULL = 11, P_EMPTY = 13, O_DONE = 15 };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kOffBar + L::kNumBars * 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t kv_head = blockIdx.y;
    const uint32_t G = p.query_heads / p.kv_heads;
    uint32_t base = p.base_position, count = p.token_count;
    if (p.prefill_state != nullptr) {
        pdl_wait();   // the state may be the preceding kernel's output
        base = p.prefill_state->base_position;
        count = min(count, p.prefill_state->token_count);
    }
    const uint32_t total_rows = p.token_count * G;
    const uint32_t row0 = blockIdx.x * kBM;
    // The next kernel of the stream (the merge of the KV splits) may become resident once every CTA has got here; it
    // orders itself against this one.  This kernel's own dependency wait comes after its set-up.
    pdl_launch_dependents();
    if (row0 >= total_rows) return;

    // longest causal range among this CTA's rows (rows are token-major; see prefill_mma.cu)
    uint32_t kv_end = 0;
    if (count > 0 && p.capacity > base) {
        const uint32_t t_first = row0 / G, t_last = (min(row0 + kBM, total_rows) - 1) / G;
        const uint64_t t_cap = p.capacity - base - 1;
        uint64_t t_max = t_last;
        if (t_max > count - 1) t_max = count - 1;
        if (t_max > t_cap) t_max = t_cap;
        if (t_max >= t_first) kv_end = base + static_cast<uint32_t>(t_max) + 1u;
    }
    if (kv_end > p.scratch_rows) kv_end = p.scratch_rows;   // never read past what the pre-pass wrote
    const int ntiles_all = static_cast<int>((kv_end + kBN - 1) / kBN);
    const int split = static_cast<int>(blockIdx.z), nsplit = static_cast<int>(p.kv_splits);
    const int tile0 = static_cast<int>(static_cast<long long>(ntiles_all) * split / nsplit);
    const int ntiles = static_cast<int>(static_cast<long long>(ntiles_all) * (split + 1) / nsplit) - tile0;   // tiles of this CTA

    // The layout (swizzled TMA tiles, MMA descriptors) needs the 1024-byte alignment the declaration above asks for; the
    // allocation has no slack for rounding up, so that a CTA of the neighbouring kernels fits beside this one on an SM.
    // Should a driver ever hand out another base, nothing of the layout is touched: the CTA's rows come out as NaN.
    if ((sbase & 1023u) != 0) {
        pdl_wait();
        const float nan = __int_as_float(0x7fc00000);
        for (uint32_t r = tid; r < static_cast<uint32_t>(kBM); r += kThreads)
            if (nsplit > 1 && row0 + r < total_rows)
                p.part_ml[(static_cast<size_t>(split) * p.kv_heads + kv_head) * p.rows_padded + row0 + r] = make_float2(0.0f, nan);
        if (nsplit == 1)
            for (uint32_t i = tid; i < static_cast<uint32_t>(kBM) * (D / 4); i += kThreads) {
                const uint32_t gr = row0 + i / (D / 4);
                if (gr >= total_rows) continue;
                const size_t off = (static_cast<size_t>(gr / G) * p.query_heads + kv_head * G + gr % G) * D + (i % (D / 4)) * 4;
                *reinterpret_cast<float4*>(p.out + off) = make_float4(nan, nan, nan, nan);
            }
        return;
    }

    // ---- set-up: barriers, TMEM, Q tile -----------------------------------------------------------------
    if (tid == 0) {
        for (int i = 0; i < L::kNumBars; ++i)
            mbar_init(bar(i), (i == S_EMPTY || i == S_EMPTY + 1 || i == P_FULL || i == P_FULL + 1) ? kBM : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < kBM * 2; i += kThreads) reinterpret_cast<uint32_t*>(smem + L::kOffRef)[i] = 0;
    if (warp == kSWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(L::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();   // Q, the fp16 scratch and the device-side state come from preceding kernels
    // Q: the CTA's rows as fp16 pairs in TMEM (row = lane, dims 2c and 2c+1 in column c), the A operand of every S MMA:
    // read from there it costs no shared-memory bandwidth, which at N = 64 would bound the MMA.  Each of a row's two
    // softmax threads stores half of the row.
    if (warp < kSoftmaxThreads / 32) {
        const int r = tid & (kBM - 1), half = tid >> 7;
        const uint32_t gr = row0 + r;
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const bool live = gr < total_rows;
        const uint32_t token = live ? gr / G : 0, head = kv_head * G + (live ? gr % G : 0);
        const size_t off = (static_cast<size_t>(token) * p.query_heads + head) * D + half * (D / 2);
#pragma unroll 1
        for (int c0 = 0; c0 < D / 4; c0 += 32) {   // 32 columns = 64 dims per store
            uint32_t w[32];
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (live) {
                    const size_t e = off + (c0 + i) * 2;
                    if (p.q_is_f16) {
                        v = *reinterpret_cast<const uint4*>(static_cast<const __half*>(p.q) + e);
                    } else {
                        const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(p.q) + e);
                        const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(p.q) + e + 4);
                        v = make_uint4(pack_half2(a.x, a.y), pack_half2(a.z, a.w), pack_half2(b.x, b.y), pack_half2(b.z, b.w));
                    }
                }
                w[i] = v.x; w[i + 1] = v.y; w[i + 2] = v.z; w[i + 3] = v.w;
            }
            tmem_st32_bits(tmem_base + lane_addr + L::kColQ + half * (D / 4) + c0, w);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    bool failed = false;

    if (warp == kTmaWarp) {
        // =============================== TMA producer, K tiles ===============================
        // A ring stage holds a PAIR of tiles, tile 2i in rows 0-63 and tile 2i+1 in rows 64-127 of every slab, so that
        // one MMA instruction (N = 128) covers both.
        if (lane == 0) {
            const int row_base = static_cast<int>(kv_head * p.scratch_rows);
            for (int i = 0; 2 * i < ntiles; ++i) {
                const int ps = i % kKPairs, n = min(2, ntiles - 2 * i);
                if (!mbar_wait(bar(K_EMPTY + ps), static_cast<uint32_t>((i / kKPairs) & 1) ^ 1)) break;
                mbar_expect_tx(bar(K_FULL + ps), n * L::kTileBytes);
                for (int t = 0; t < n; ++t)
                    for (int s = 0; s < L::kSlabs; ++s)
                        tma_load_2d(sbase + L::kOffK + ps * L::kPairBytes + s * (2 * kBN * 128) + t * (kBN * 128), &p.kmap, s * 64,
                                    row_base + (tile0 + 2 * i + t) * kBN, bar(K_FULL + ps));
            }
        }
    } else if (warp == kTmaVWarp) {
        // =============================== TMA producer, V tiles ===============================
        if (lane == 0) {
            const int row_base = static_cast<int>(kv_head * p.scratch_rows);
            for (int j = 0; j < ntiles; ++j) {
                const int st = j & 1;
                const uint32_t ph = static_cast<uint32_t>((j >> 1) & 1);
                if (!mbar_wait(bar(V_EMPTY + st), ph ^ 1)) break;
                mbar_expect_tx(bar(V_FULL + st), L::kTileBytes);
                for (int s = 0; s < L::kSlabs; ++s)
                    tma_load_2d(sbase + L::kOffV + st * L::kTileBytes + s * (kBN * 128), &p.vmap, s * 64, row_base + (tile0 + j) * kBN, bar(V_FULL + st));
            }
        }
    } else if (warp == kSWarp) {
        // =============================== S = Q.K^T issuer ===============================
        // One chain of D/16 MMAs per PAIR of tiles (N = 128: the first tile's scores land in S columns 0-63, the second
        // one's in 64-127).  An MMA instruction of this shape costs about 90 clocks whatever its N up to 128, so a
        // pair costs what a single tile would.
        if (lane == 0) {
            constexpr uint32_t idesc_pair = umma_idesc(kBM, 2 * kBN, 0, 0), idesc_one = umma_idesc(kBM, kBN, 0, 0);
            for (int i = 0; 2 * i < ntiles; ++i) {
                const int ps = i % kKPairs, n = min(2, ntiles - 2 * i);
                if (!mbar_wait(bar(K_FULL + ps), static_cast<uint32_t>((i / kKPairs) & 1))) break;
                // both groups have read the previous pair's scores (only the last pair can be a single tile)
                if (!mbar_wait(bar(S_EMPTY), static_cast<uint32_t>(i & 1) ^ 1) || !mbar_wait(bar(S_EMPTY + 1), static_cast<uint32_t>(i & 1) ^ 1)) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t b = sbase + L::kOffK + ps * L::kPairBytes + (kk >> 2) * (2 * kBN * 128) + (kk & 3) * 32;
                    umma_f16_a_tmem(tmem_base + L::kColS, tmem_base + L::kColQ + kk * 8, umma_desc(b, 16, 1024), n == 2 ? idesc_pair : idesc_one, kk > 0);
                }
                umma_commit(bar(S_FULL));         // scores ready for both softmax groups
                umma_commit(bar(K_EMPTY + ps));   // K stage may be refilled
            }
        }
    } else if (warp == kPvWarp) {
        // =============================== O += P.V issuer ===============================
        if (lane == 0) {
            constexpr uint32_t idesc_o = umma_idesc(kBM, D, 0, 1);
            for (int j = 0; j < ntiles; ++j) {
                const int st = j & 1;
                const uint32_t ph = static_cast<uint32_t>((j >> 1) & 1);
                if (!mbar_wait(bar(V_FULL + st), ph)) break;
                if (!mbar_wait(bar(P_FULL + st), ph)) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < kBN / 16; ++kk) {
                    const uint32_t b = sbase + L::kOffV + st * L::kTileBytes + kk * (16 * 128);      // V: MN-major, 16 positions per step
                    const uint32_t a = sbase + L::kOffP + st * L::kPBytes + kk * 32;               // P: K-major, one 128-byte slab
                    umma_f16(tmem_base + L::kColO, umma_desc(a, 16, 1024), umma_desc(b, kBN * 128, 1024), idesc_o, (j > 0 || kk > 0));
                }
                umma_commit(bar(P_EMPTY + st));   // P buffer free, O holds tiles 0..j
                umma_commit(bar(V_EMPTY + st));
                if (j == ntiles - 1) umma_commit(bar(O_DONE));   // O complete: the epilogue's signal for both groups
            }
        }
    } else {
        // =============================== softmax rows ===============================
        // Two groups of 128 threads, one thread per query row in each: warps 0-3 take the even tiles, warps 4-7 the odd
        // ones (a warp reaches the 32 TMEM lanes of its number modulo 4), so two tiles are in flight: while one group
        // works through its exponentials the other one's S arrives and its P.V runs.  A row's reference maximum is handed
        // from tile to tile through an 8-byte {value, sequence} word in shared memory; each thread keeps the partial row
        // sum of its own tiles, relative to the reference it last saw.
        const int r = tid & (kBM - 1), grp = tid >> 7;       // row of this thread == its TMEM lane; tile parity
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t gr = row0 + r;
        uint32_t len = 0;
        if (gr < total_rows) {
            const uint32_t token = gr / G;
            const uint64_t l64 = static_cast<uint64_t>(base) + token + 1u;
            len = (token < count && l64 <= p.capacity) ? static_cast<uint32_t>(l64) : 0u;
        }
        volatile unsigned long long* ref = reinterpret_cast<volatile unsigned long long*>(smem + L::kOffRef) + r;
        auto ref_after = [&](uint32_t seq, float* value) -> bool {   // the reference as tile seq-1 left it
            for (uint32_t spin = 0; spin < kSpin; ++spin) {
                const unsigned long long w = *ref;
                if (static_cast<uint32_t>(w >> 32) == seq) { *value = __uint_as_float(static_cast<uint32_t>(w)); return true; }
            }
            return false;
        };
        float m_known = -INFINITY, l_sum = 0.0f;   // l_sum is relative to m_known
        auto rebase = [&](float m_new) {
            if (m_new != m_known) {
                l_sum *= (m_known == -INFINITY) ? 0.0f : ex2_approx(m_known - m_new);
                m_known = m_new;
            }
        };
        const int st = grp;
        for (int j = grp; j < ntiles; j += 2) {
            const uint32_t ph = static_cast<uint32_t>((j >> 1) & 1);   // parity of the tile's pair
            if (!mbar_wait(bar(S_FULL), ph)) { failed = true; break; }
            tc_fence_after();
            float s[kBN];
            {
                uint32_t lo[32], hi[32];
                tmem_ld32_nowait(tmem_base + lane_addr + L::kColS + st * kBN, lo);
                tmem_ld32_nowait(tmem_base + lane_addr + L::kColS + st * kBN + 32, hi);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) { s[i] = __uint_as_float(lo[i]); s[32 + i] = __uint_as_float(hi[i]); }
            }
            tc_fence_before();
            mbar_arrive(bar(S_EMPTY + st));   // this row of S is in registers
            const uint32_t pos0 = static_cast<uint32_t>(tile0 + j) * kBN;
            // Raw scores stay unscaled; the softmax scale is folded into the exponent: p = 2^(s*c - m*c).
            // Only the tiles that straddle this row's causal length need the mask.
            if (pos0 + kBN > len) {
#pragma unroll
                for (int i = 0; i < kBN; ++i) s[i] = (pos0 + i < len) ? s[i] : -INFINITY;
            }
            float mt = -INFINITY;
#pragma unroll
            for (int i = 0; i < kBN; ++i) mt = fmaxf(mt, s[i]);
            mt *= p.scale_log2;   // scale > 0: the maximum commutes with it
            // the reference as the previous tile (the other group's) left it; lazy rescale: keep it unless this tile's
            // maximum outgrew it by more than the threshold
            float m_prev = -INFINITY;
            if (j > 0 && !ref_after(static_cast<uint32_t>(j), &m_prev)) { failed = true; break; }
            float alpha = 1.0f, m_new = m_prev;
            if (mt > m_prev + kRescaleThreshold || (m_prev == -INFINITY && mt > -INFINITY)) {
                alpha = (m_prev == -INFINITY) ? 0.0f : ex2_approx(m_prev - mt);
                m_new = mt;
            }
            // published at once (the other group's thread of this row waits for it): no later work may be scheduled before it
            asm volatile("st.volatile.shared.u64 [%0], %1;" ::"r"(smem_u32(const_cast<unsigned long long*>(ref))),
                         "l"((static_cast<unsigned long long>(static_cast<uint32_t>(j) + 1u) << 32) | __float_as_uint(m_new)) : "memory");
            rebase(m_new);
            const float neg_ref = (m_new == -INFINITY) ? 0.0f : -m_new;
            float sum = 0.0f;
            uint32_t pk[kBN / 2];
#pragma unroll
            for (int i = 0; i < kBN; i += 2) {
                const float p0 = ex2_approx(fmaf(s[i], p.scale_log2, neg_ref)), p1 = ex2_approx(fmaf(s[i + 1], p.scale_log2, neg_ref));
                const __half2 h = __floats2half2_rn(p0, p1);
                // the sum uses the rounded values the MMA will multiply, so numerator and denominator stay consistent
                const float2 hf = __half22float2(h);
                sum += hf.x + hf.y;
                pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
            }
            l_sum += sum;
            // this group's P buffer is free once the P.V of its previous tile has completed
            if (!mbar_wait(bar(P_EMPTY + st), ph ^ 1)) { failed = true; break; }
            tc_fence_after();
            if (__any_sync(0xffffffffu, alpha != 1.0f) && j > 0) {
                // rare: the reference moved.  O holds tiles 0..j-1 once the previous tile's P.V (the other group's) has
                // completed; then this warp rescales its 32 rows of O in TMEM before its own P is released.
                if (!mbar_wait(bar(P_EMPTY + (st ^ 1)), static_cast<uint32_t>(((j - 1) >> 1) & 1))) { failed = true; break; }
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    float o[32];
                    tmem_ld32(tmem_base + lane_addr + L::kColO + c0, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= alpha;
                    tmem_st32(tmem_base + lane_addr + L::kColO + c0, o);
                }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");   // the rescale's stores, if any
            uint8_t* prow = smem + L::kOffP + st * L::kPBytes + r * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            mbar_arrive(bar(P_FULL + st));
        }
        // ---- epilogue: O / sum, gate, store; each thread of a row's pair half of the columns ----
        if (!failed && ntiles > 0 && !mbar_wait(bar(O_DONE), 0)) failed = true;
        tc_fence_after();
        {
            float m_final = -INFINITY;
            if (!failed && ntiles > 0 && !ref_after(static_cast<uint32_t>(ntiles), &m_final)) failed = true;
            rebase(m_final);
            float* sums = reinterpret_cast<float*>(smem + L::kOffSum);
            sums[grp * kBM + r] = failed ? __int_as_float(0x7fc00000) : l_sum;
            asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
            l_sum = sums[r] + sums[kBM + r];
            if (l_sum != l_sum) failed = true;   // either thread of the row gave up
            const float m_ref = m_final;
            const int hsel = grp;
            // tcgen05.ld is warp-collective: every lane takes part, rows past the launch only skip the store
            const bool live = gr < total_rows;
            const uint32_t token = live ? gr / G : 0, head = kv_head * G + (live ? gr % G : 0);
            const size_t off = (static_cast<size_t>(token) * p.query_heads + head) * D;
            const float inv = l_sum > 0.0f ? 1.0f / l_sum : 0.0f;
            const bool have_o = ntiles > 0 && !__any_sync(0xffffffffu, failed);
            const bool partial = nsplit > 1;
            const size_t prow_idx = (static_cast<size_t>(split) * p.kv_heads + kv_head) * p.rows_padded + row0 + r;
            if (partial && live && hsel == 0)   // a poisoned or empty partial is recognised by its sum
                p.part_ml[prow_idx] = make_float2(m_ref, failed ? __int_as_float(0x7fc00000) : (len == 0 ? 0.0f : l_sum));
#pragma unroll 1
            for (int c0 = hsel * (D / 2); c0 < (hsel + 1) * (D / 2); c0 += 32) {
                float o[32];
                if (have_o) {
                    tmem_ld32(tmem_base + lane_addr + L::kColO + c0, o);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = failed ? __int_as_float(0x7fc00000) : 0.0f;
                }
                if (!live) continue;
                if (partial) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(p.part_o + prow_idx * D + c0 + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
                    continue;
                }
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float4 v = make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
                    if (failed) v = make_float4(o[i], o[i], o[i], o[i]);
                    else if (len == 0) v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (p.gate != nullptr) {
                        const float4 g = *reinterpret_cast<const float4*>(p.gate + off + c0 + i);
                        v.x *= 1.0f / (1.0f + __expf(-g.x)); v.y *= 1.0f / (1.0f + __expf(-g.y));
                        v.z *= 1.0f / (1.0f + __expf(-g.z)); v.w *= 1.0f / (1.0f + __expf(-g.w));
                    }
                    *reinterpret_cast<float4*>(p.out + off + c0 + i) = v;
                }
            }
        }
    }

    // ---- teardown: every role arrives here, with or without a timeout; TMEM is always released ----
    tc_fence_before();
    __syncthreads();
    if (warp == kSWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::kTmemCols) : "memory");
    }
}

// ---- merge of the KV splits: out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), gate -------------------------------
struct PrefillMergeParams {
    const float* part_o;
    const float2* part_ml;
    const float* gate;
    float* out;
    uint32_t kv_splits, kv_heads, query_heads, rows_padded, total_rows;   // total_rows = token_count * G per kv head
};

template <int D>
__global__ void __launch_bounds__(256) prefill_merge_kernel(const __grid_constant__ PrefillMergeParams p) {
    constexpr int VPR = D / 4;   // float4 per row
    pdl_launch_dependents();
    pdl_wait();   // the partials are the attention kernel's output
    const uint32_t kv_head = blockIdx.y, G = p.query_heads / p.kv_heads;
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<size_t>(p.total_rows) * VPR) return;
    const uint32_t gr = static_cast<uint32_t>(idx / VPR), c = static_cast<uint32_t>(idx % VPR) * 4;
    float m[8], l[8], M = -INFINITY;   // kv_splits <= 8
    for (uint32_t s = 0; s < p.kv_splits; ++s) {
        const float2 ml = p.part_ml[(static_cast<size_t>(s) * p.kv_heads + kv_head) * p.rows_padded + gr];
        m[s] = ml.x; l[s] = ml.y;
        if (!(ml.y <= 0.0f) && ml.x != -INFINITY) M = fmaxf(M, ml.x);   // keeps NaN partials in play
    }
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float lsum = 0.0f;
    for (uint32_t s = 0; s < p.kv_splits; ++s) {
        if (l[s] <= 0.0f || m[s] == -INFINITY) continue;   // empty split: its O was never written
        const float w = exp2f(m[s] - M);
        const float4 o = *reinterpret_cast<const float4*>(p.part_o + ((static_cast<size_t>(s) * p.kv_heads + kv_head) * p.rows_padded + gr) * D + c);
        acc.x = fmaf(o.x, w, acc.x); acc.y = fmaf(o.y, w, acc.y); acc.z = fmaf(o.z, w, acc.z); acc.w = fmaf(o.w, w, acc.w);
        lsum = fmaf(l[s], w, lsum);
    }
    const float inv = lsum > 0.0f ? 1.0f / lsum : (lsum == lsum ? 0.0f : lsum);
    float4 v = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
    const uint32_t token = gr / G, head = kv_head * G + gr % G;
    const size_t off = (static_cast<size_t>(token) * p.query_heads + head) * D + c;
    if (p.gate != nullptr) {
        const float4 g = *reinterpret_cast<const float4*>(p.gate + off);
        v.x *= 1.0f / (1.0f + __expf(-g.x)); v.y *= 1.0f / (1.0f + __expf(-g.y));
        v.z *= 1.0f / (1.0f + __expf(-g.z)); v.w *= 1.0f / (1.0f + __expf(-g.w));
    }
    *reinterpret_cast<float4*>(p.out + off) = v;
}

// ---- pre-pass: dequantise [0, rows) of every kv head to fp16 ---------------------------------------------------------
struct DequantParams {
    b200kv_view view;
    __half* k_out;       // [kv_heads][scratch_rows][D]
    __half* v_out;
    uint32_t rows;       // positions that hold data; rows from here up to row_end are zero-filled
    uint32_t scratch_rows;
    uint32_t row_begin;  // this launch converts positions [row_begin, row_end): the rows below were converted ahead of
    uint32_t row_end;    // the chunk (b200kv_prefill_prepare), possibly beside the previous layer's attention
};

template <int D>
__global__ void __launch_bounds__(256) dequant_prefix_kernel(const __grid_constant__ DequantParams p) {
    constexpr int CPR = D / 16;
    pdl_launch_dependents();
    pdl_wait();   // the cache rows of this chunk come from the append kernel just before
    const uint32_t head = blockIdx.y, side = blockIdx.z;   // side 0 = K, 1 = V
    const uint32_t mode = p.view.quant_mode;
    const bool q8 = side == 0 ? (mode == B200KV_Q8_F16 || mode == B200KV_Q8_Q8) : (mode == B200KV_F16_Q8 || mode == B200KV_Q8_Q8);
    const int8_t* q = side == 0 ? p.view.key_q8 : p.view.value_q8;
    const __half* sc = static_cast<const __half*>(side == 0 ? p.view.key_scales : p.view.value_scales);
    const __half* f16 = static_cast<const __half*>(side == 0 ? p.view.key_f16 : p.view.value_f16);
    __half* out = (side == 0 ? p.k_out : p.v_out) + static_cast<size_t>(head) * p.scratch_rows * D;
    const uint32_t nblk = D / p.view.qblock;
    const uint64_t head_row0 = static_cast<uint64_t>(head) * p.view.capacity;
    const size_t total = static_cast<size_t>(p.row_end) * CPR;   // rows past `rows` are zero-filled: the last tile reads them
    for (size_t idx = static_cast<size_t>(p.row_begin) * CPR + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t pos = static_cast<uint32_t>(idx / CPR), c16 = static_cast<uint32_t>(idx % CPR);
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
        if (pos >= p.rows) {
            // padding row of the last tile: P is 0 there, but 0 * (stale NaN) would still poison O
        } else if (q8) {
            const uint64_t grow = head_row0 + pos;
            const uint4 raw = *reinterpret_cast<const uint4*>(q + grow * D + c16 * 16);
            dequant16(raw, sc[grow * nblk + (nblk == 1 ? 0 : c16 / 2)], &lo, &hi);
        } else {
            const uint4* src = reinterpret_cast<const uint4*>(f16 + (head_row0 + pos) * D + c16 * 16);
            lo = src[0]; hi = src[1];
        }
        uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(pos) * D + c16 * 16);
        dst[0] = lo; dst[1] = hi;
    }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn tc5_encoder() {
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

bool encode_f16_plane(CUtensorMap* map, void* base, uint32_t d, uint64_t rows) {
    EncodeFn fn = tc5_encoder();
    if (fn == nullptr) return false;
    const TensorMapKey key{base, rows, d * 2u, 128u, static_cast<uint32_t>(kBN), 2u};   // kind 2: fp16, 128-byte swizzle
    if (tensor_map_lookup(key, map)) return true;
    const cuuint64_t dims[2] = {d, rows};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(d) * 2};
    const cuuint32_t box[2] = {64, kBN};
    const cuuint32_t elem[2] = {1, 1};
    if (fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    tensor_map_remember(key, *map);
    return true;
}

// The pre-pass over positions [row_begin, row_end) of every kv head, K and V.
template <int D>
int launch_dequant(const b200kv_view& view, __half* k_scratch, __half* v_scratch, uint32_t rows, uint32_t scratch_rows,
                   uint32_t row_begin, uint32_t row_end, cudaStream_t stream) {
    if (row_begin >= row_end) return B200KV_OK;
    DequantParams dp{};
    dp.view = view;
    dp.k_out = k_scratch;
    dp.v_out = v_scratch;
    dp.rows = rows;
    dp.scratch_rows = scratch_rows;
    dp.row_begin = row_begin;
    dp.row_end = row_end;
    const size_t units = static_cast<size_t>(row_end - row_begin) * (D / 16);
    unsigned blocks = static_cast<unsigned>((units + 255) / 256);
    if (blocks > 148u * 4u) blocks = 148u * 4u;
    B200KV_CUDA_TRY(launch_kernel(dequant_prefix_kernel<D>, dim3(blocks, view.kv_heads, 2), dim3(256), 0, stream, true, dp));
    return B200KV_OK;
}

template <int D>
int launch_tc5(const b200kv_view& view, Tc5Params& p, __half* k_scratch, __half* v_scratch, uint32_t rows, uint32_t prepared_rows,
               cudaStream_t stream) {
    using L = Layout<D>;
    static std::atomic<uint64_t> done{0};   // one per kernel instantiation: devices that have opted in
    const cudaError_t attr_err = opt_in_dynamic_smem(reinterpret_cast<const void*>(prefill_tc5_kernel<D>), L::kAlloc, done);
    if (attr_err != cudaSuccess) { set_last_cuda_error(attr_err, "cudaFuncSetAttribute(prefill_tc5)"); return B200KV_ERR_CUDA; }
    if (rows > 0) {
        const int rc = launch_dequant<D>(view, k_scratch, v_scratch, rows, p.scratch_rows, prepared_rows < rows ? prepared_rows : rows,
                                         p.scratch_rows, stream);
        if (rc != B200KV_OK) return rc;
    }
    const uint32_t G = p.query_heads / p.kv_heads;
    const uint32_t row_tiles = (p.token_count * G + kBM - 1) / kBM;
    B200KV_CUDA_TRY(launch_kernel(prefill_tc5_kernel<D>, dim3(row_tiles, p.kv_heads, p.kv_splits), dim3(kThreads), L::kAlloc, stream, true, p));
    if (p.kv_splits > 1) {
        PrefillMergeParams mp{};
        mp.part_o = p.part_o;
        mp.part_ml = p.part_ml;
        mp.gate = p.gate;
        mp.out = p.out;
        mp.kv_splits = p.kv_splits;
        mp.kv_heads = p.kv_heads;
        mp.query_heads = p.query_heads;
        mp.rows_padded = p.rows_padded;
        mp.total_rows = p.token_count * G;
        const size_t work = static_cast<size_t>(mp.total_rows) * (D / 4);
        B200KV_CUDA_TRY(launch_kernel(prefill_merge_kernel<D>, dim3(static_cast<unsigned>((work + 255) / 256), p.kv_heads), dim3(256), 0, stream, true, mp));
    }
    return B200KV_OK;
}

}  // namespace

size_t prefill_tc5_workspace_bytes(uint32_t rows, uint32_t kv_heads, uint32_t head_dim) {
    const size_t r = (static_cast<size_t>(rows) + kBN - 1) / kBN * kBN;
    return 2 * r * kv_heads * head_dim * sizeof(__half) + 1024;   // K and V planes, 1 KB to align the base
}

constexpr uint32_t kMaxKvSplits = 8;

// Extra workspace that lets a launch split the KV range of every row tile over several CTAs (partials of `splits` splits).
size_t prefill_tc5_split_bytes(uint32_t token_count, uint32_t query_heads, uint32_t kv_heads, uint32_t head_dim, uint32_t splits) {
    if (kv_heads == 0 || query_heads % kv_heads != 0) return 0;
    const size_t rows_padded = (static_cast<size_t>(token_count) * (query_heads / kv_heads) + kBM - 1) / kBM * kBM;
    return static_cast<size_t>(splits) * kv_heads * rows_padded * (head_dim + 2) * sizeof(float);
}

// How many KV splits fill the SMs best: one CTA per SM, `units` row-tile CTAs per split.
static uint32_t pick_kv_splits(uint32_t units, uint32_t min_tiles) {
    const uint32_t sms = 148;
    uint32_t best = 1;
    double best_eff = static_cast<double>(units) / ((units + sms - 1) / sms * sms);
    for (uint32_t s = 2; s <= kMaxKvSplits; ++s) {
        if (min_tiles < 8 * s) break;   // every split should still walk a few tiles
        const double eff = static_cast<double>(units) * s / ((units * s + sms - 1) / sms * sms);
        if (eff > best_eff * 1.15) { best = s; best_eff = eff; }   // a split costs a partial round trip: only for a clear gain
    }
    return best;
}

// Returns B200KV_ERR_UNSUPPORTED when this path cannot run (no workspace, no TMA encoder); the caller then uses the
// register-resident mma.sync kernel.
int launch_prefill_tc5(const b200kv_view& view, const void* q, int q_is_f16, const float* gate, float* out,
                       uint32_t token_count, uint32_t base_position, const b200kv_prefill_state* prefill_state,
                       uint32_t query_heads, float scale, void* workspace, size_t workspace_bytes, uint32_t prepared_rows,
                       cudaStream_t stream) {
    // rows the chunk can see: known on the host unless a device-side state overrides it (then: the whole cache)
    uint64_t rows = prefill_state ? view.capacity : static_cast<uint64_t>(base_position) + token_count;
    if (rows > view.capacity) rows = view.capacity;
    const uint32_t scratch_rows = static_cast<uint32_t>((rows + kBN - 1) / kBN * kBN);
    if (workspace == nullptr || workspace_bytes < prefill_tc5_workspace_bytes(static_cast<uint32_t>(rows), view.kv_heads, view.head_dim))
        return B200KV_ERR_UNSUPPORTED;
    if (static_cast<uint64_t>(view.kv_heads) * scratch_rows > 0x7fffffffull) return B200KV_ERR_UNSUPPORTED;
    uint8_t* ws = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(workspace) + 1023) & ~static_cast<uintptr_t>(1023));
    __half* k_scratch = reinterpret_cast<__half*>(ws);
    __half* v_scratch = k_scratch + static_cast<size_t>(view.kv_heads) * scratch_rows * view.head_dim;
    Tc5Params p{};
    if (!encode_f16_plane(&p.kmap, k_scratch, view.head_dim, static_cast<uint64_t>(view.kv_heads) * scratch_rows) ||
        !encode_f16_plane(&p.vmap, v_scratch, view.head_dim, static_cast<uint64_t>(view.kv_heads) * scratch_rows))
        return B200KV_ERR_UNSUPPORTED;
    p.q = q;
    p.q_is_f16 = q_is_f16;
    p.gate = gate;
    p.out = out;
    p.token_count = token_count;
    p.base_position = base_position;
    p.prefill_state = prefill_state;
    p.query_heads = query_heads;
    p.kv_heads = view.kv_heads;
    p.capacity = view.capacity;
    p.scratch_rows = scratch_rows;
    p.scale_log2 = scale * 1.4426950408889634f;
    // KV split when the row tiles alone leave SMs idle and the caller's workspace has room for the partials
    p.kv_splits = 1;
    {
        const uint32_t G = query_heads / view.kv_heads;
        const uint32_t row_tiles = (token_count * G + kBM - 1) / kBM;
        const uint32_t min_tiles = static_cast<uint32_t>((static_cast<uint64_t>(prefill_state ? 0 : base_position) + kBN - 1) / kBN);
        uint32_t want = pick_kv_splits(row_tiles * view.kv_heads, min_tiles);
        const size_t scratch = prefill_tc5_workspace_bytes(static_cast<uint32_t>(rows), view.kv_heads, view.head_dim);
        while (want > 1 && workspace_bytes < scratch + 1024 + prefill_tc5_split_bytes(token_count, query_heads, view.kv_heads, view.head_dim, want)) --want;
        if (want > 1) {
            p.kv_splits = want;
            p.rows_padded = row_tiles * kBM;
            uint8_t* part = reinterpret_cast<uint8_t*>(v_scratch + static_cast<size_t>(view.kv_heads) * scratch_rows * view.head_dim);
            part = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(part) + 1023) & ~static_cast<uintptr_t>(1023));
            p.part_o = reinterpret_cast<float*>(part);
            p.part_ml = reinterpret_cast<float2*>(p.part_o + static_cast<size_t>(want) * view.kv_heads * p.rows_padded * view.head_dim);
        }
    }
    return view.head_dim == 128 ? launch_tc5<128>(view, p, k_scratch, v_scratch, static_cast<uint32_t>(rows), prepared_rows, stream)
                                : launch_tc5<256>(view, p, k_scratch, v_scratch, static_cast<uint32_t>(rows), prepared_rows, stream);
}

// The pre-pass alone, for positions [0, prepared_rows), into the scratch laid out for a chunk that sees `rows` positions
// (the same `rows` the attention call derives: base_position + token_count, or the capacity with a device-side state).
int launch_prefill_tc5_prepare(const b200kv_view& view, uint32_t prepared_rows, uint64_t rows, void* workspace, size_t workspace_bytes,
                               cudaStream_t stream) {
    if (rows > view.capacity) rows = view.capacity;
    if (prepared_rows > rows) return B200KV_ERR_RANGE;
    const uint32_t scratch_rows = static_cast<uint32_t>((rows + kBN - 1) / kBN * kBN);
    if (workspace == nullptr || workspace_bytes < prefill_tc5_workspace_bytes(static_cast<uint32_t>(rows), view.kv_heads, view.head_dim))
        return B200KV_ERR_WORKSPACE;
    if (static_cast<uint64_t>(view.kv_heads) * scratch_rows > 0x7fffffffull) return B200KV_ERR_UNSUPPORTED;
    uint8_t* ws = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(workspace) + 1023) & ~static_cast<uintptr_t>(1023));
    __half* k_scratch = reinterpret_cast<__half*>(ws);
    __half* v_scratch = k_scratch + static_cast<size_t>(view.kv_heads) * scratch_rows * view.head_dim;
    return view.head_dim == 128 ? launch_dequant<128>(view, k_scratch, v_scratch, prepared_rows, scratch_rows, 0, prepared_rows, stream)
                                : launch_dequant<256>(view, k_scratch, v_scratch, prepared_rows, scratch_rows, 0, prepared_rows, stream);
}

}  // namespace b200kv
