// What the two streaming decode kernels (decode_q8.cu: warp-level mma; decode_tc5.cu: tcgen05) share after
// their tile loops: the tagged-word partials, the merge of a kv head's splits inside the launch, the cross-GPU
// exchange of a sequence shard, and the single-token append a decode step fuses in.
//
// The merge is MIInfer's decode stage 2 (gfx906/kernels/qwen3_primitives.hip:2295-2352) with the empty-split rule
// of its suffix twin (.hip:6681,6701); the optional Q8_1 re-quantisation of the output follows .hip:2354-2383.
#pragma once

#include "append_row.cuh"
#include "decode_common.cuh"

namespace b200kv {
namespace tail {

constexpr uint32_t kPollLimit = 1u << 17;   // polls of a merger (each a trip to L2 or to a peer) before it gives up

// Tagged partials: every float of a split's partial travels as one 8-byte word {value, tag}.  An 8-byte store is
// indivisible, so a reader that sees the tag also sees the value: no fence and no counter stand between the CTA that
// produced a partial and the CTA that merges it.  The tag is the launch's own (never 0): a word left behind by an
// earlier launch that gave up waiting carries another tag and reads as "not there yet".  The merger zeroes what it
// consumed.
__device__ __forceinline__ uint64_t tagged_word(float v, uint32_t tag) { return (static_cast<uint64_t>(tag) << 32) | __float_as_uint(v); }
__device__ __forceinline__ void st_tagged(uint64_t* dst, float v, uint32_t tag) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(dst), "l"(tagged_word(v, tag)) : "memory");
}
__device__ __forceinline__ void ld_tagged2(const uint64_t* src, uint64_t& a, uint64_t& b) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(src) : "memory");
}
__device__ __forceinline__ bool tagged_ready(uint64_t a, uint64_t b, uint32_t tag) {
    return static_cast<uint32_t>(a >> 32) == tag && static_cast<uint32_t>(b >> 32) == tag;
}
// the same words across GPUs: stores into a peer's memory, loads of words a peer stored into ours
__device__ __forceinline__ void st_tagged_sys(uint64_t* dst, float v, uint32_t tag) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(tagged_word(v, tag)) : "memory");
}
__device__ __forceinline__ void ld_tagged2_sys(const uint64_t* src, uint64_t& a, uint64_t& b) {
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(src) : "memory");
}
__device__ __forceinline__ void zero2(uint64_t* dst) {
    asm volatile("st.global.v2.u64 [%0], {%1,%1};" ::"l"(dst), "l"(0ull) : "memory");
}

// A bounded wait ran out: leave a sticky bit in the caller's status word (if one was registered).
__device__ __forceinline__ void report(const DecodeParams& p, uint32_t bit) {
    if (p.status != nullptr) atomicOr(p.status, bit);
}

// ---- fused single-token append -----------------------------------------------------------------------------
// Kept out of line so the rarely-taken path does not widen the register allocation of the streaming loops.
// Loads the new row of `kv_head` (lane L: elements L, L+32, L+64, L+96); head_dim 128.
static __device__ __noinline__ void load_new_row(const void* src, int is_f16, uint32_t kv_head, int lane, float (&x)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const size_t i = static_cast<size_t>(kv_head) * 128 + lane + 32 * j;
        x[j] = is_f16 ? __half2float(static_cast<const __half*>(src)[i]) : static_cast<const float*>(src)[i];
    }
}

// Quantises the new K and V rows of a kv head (already in registers) and stores them (int8 + fp16 block scales) at
// cache row `row_index`.  One warp; head_dim 128.
template <int NBLK>
static __device__ __noinline__ void fused_append_row(const DecodeParams& p, const b200kv_view& view, float (&k)[4], float (&v)[4],
                                              uint32_t position, uint64_t row_index, int lane) {
    constexpr int kD = 128;
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

// ---- where a CTA's partial of one (query head, dim) goes -----------------------------------------------------
// kD = 128.  `at` is the unnormalised accumulator relative to the maximum m_nat (natural-log units), `lt` the sum.
__device__ __forceinline__ void emit_partial(const DecodeParams& p, uint32_t session, uint32_t split, uint32_t num_splits,
                                             uint32_t head, int dim, float at, float m_nat, float lt) {
    constexpr int kD = 128;
    constexpr int kPartialWords = kD + 2;
    const size_t slot_idx = (static_cast<size_t>(session) * p.num_splits + split) * p.query_heads + head;
    if (p.ws_tagged != nullptr && num_splits == 1 && p.fuse.xchg.world <= 1) {
        // a single split has nothing to merge with: the result leaves from here (short contexts)
        const size_t out_idx = (static_cast<size_t>(session) * p.query_heads + head) * kD + dim;
        if (p.fuse.out_m != nullptr) {
            p.fuse.out_acc[out_idx] = at;
            if (dim == 0) {
                p.fuse.out_m[static_cast<size_t>(session) * p.query_heads + head] = m_nat;
                p.fuse.out_l[static_cast<size_t>(session) * p.query_heads + head] = lt;
            }
        } else {
            const float inv = lt > 0.0f ? 1.0f / lt : (lt == lt ? 0.0f : lt);
            float o = at * inv;
            if (p.fuse.output != nullptr) p.fuse.output[out_idx] = o;
            if (p.fuse.gated_output != nullptr) {
                if (p.fuse.gate != nullptr) o *= 1.0f / (1.0f + __expf(-p.fuse.gate[out_idx]));
                p.fuse.gated_output[out_idx] = o;
            }
        }
    } else if (p.ws_tagged != nullptr) {
        uint64_t* dst = p.ws_tagged + slot_idx * kPartialWords;
        st_tagged(dst + dim, at, p.tag);
        if (dim == 0) { st_tagged(dst + kD, m_nat, p.tag); st_tagged(dst + kD + 1, lt, p.tag); }
    } else {
        p.ws_acc[slot_idx * kD + dim] = at;
        if (dim == 0) { p.ws_m[slot_idx] = m_nat; p.ws_l[slot_idx] = lt; }
    }
}
// True when emit_partial wrote final results or plain partials, i.e. no in-launch merge follows for this CTA's work.
__device__ __forceinline__ bool merge_not_needed(const DecodeParams& p, uint32_t num_splits) {
    return p.ws_tagged == nullptr || (num_splits == 1 && p.fuse.xchg.world <= 1);
}

// Cross-GPU step of a sequence-sharded launch, run by the 64 threads (pair of dims `pr`) that hold the merged
// partial of `head`: store it into every rank's exchange buffer, wait (bounded) for the partials of all ranks in
// our own buffer, merge them into (tot, gsum) and zero the words again.  Uses named barrier 1 (64 threads).
__device__ __forceinline__ void exchange_partials(const DecodeParams& p, uint32_t head, int pr, float m_local, float2& tot,
                                                  float& gsum, bool lost) {
    constexpr int kD = 128;
    constexpr int kPartialWords = kD + 2;
    const ExchangeParams& x = p.fuse.xchg;
    const uint32_t tag = x.tag, slot = x.phase & 1u;
    const size_t words_per_rank = static_cast<size_t>(p.query_heads) * kPartialWords;
    const size_t mine_off = (static_cast<size_t>(slot) * x.world + x.rank) * words_per_rank + static_cast<size_t>(head) * kPartialWords;
    for (uint32_t w = 0; w < x.world; ++w) {
        uint64_t* dst = x.peers[w] + mine_off;
        st_tagged_sys(dst + 2 * pr, tot.x, tag);
        st_tagged_sys(dst + 2 * pr + 1, tot.y, tag);
        if (pr == 0) { st_tagged_sys(dst + kD, m_local, tag); st_tagged_sys(dst + kD + 1, gsum, tag); }
    }
    uint64_t* in = x.peers[x.rank] + static_cast<size_t>(slot) * x.world * words_per_rank + static_cast<size_t>(head) * kPartialWords;
    float fa[kMaxExchangeRanks], fb[kMaxExchangeRanks], fm[kMaxExchangeRanks], fl[kMaxExchangeRanks];
#pragma unroll
    for (int w = 0; w < kMaxExchangeRanks; ++w) { fa[w] = fb[w] = 0.0f; fm[w] = -INFINITY; fl[w] = 0.0f; }
    uint32_t pending = (1u << x.world) - 1u, ml_pending = pending;
    bool gave_up = false;
    for (uint32_t polls = 0; (pending | ml_pending) != 0 && !lost; ++polls) {
        if (polls >= kPollLimit) { lost = true; gave_up = true; break; }
        // all loads first, all checks afterwards: a check between two loads would serialise their trips
        uint64_t wa[kMaxExchangeRanks], wb[kMaxExchangeRanks], wm[kMaxExchangeRanks], wl[kMaxExchangeRanks];
#pragma unroll
        for (int w = 0; w < kMaxExchangeRanks; ++w) {
            wa[w] = wb[w] = wm[w] = wl[w] = 0;
            if (pending & (1u << w)) ld_tagged2_sys(in + w * words_per_rank + 2 * pr, wa[w], wb[w]);
            if (ml_pending & (1u << w)) ld_tagged2_sys(in + w * words_per_rank + kD, wm[w], wl[w]);
        }
#pragma unroll
        for (int w = 0; w < kMaxExchangeRanks; ++w) {
            if ((pending & (1u << w)) && tagged_ready(wa[w], wb[w], tag)) {
                fa[w] = __uint_as_float(static_cast<uint32_t>(wa[w]));
                fb[w] = __uint_as_float(static_cast<uint32_t>(wb[w]));
                pending &= ~(1u << w);
            }
            if ((ml_pending & (1u << w)) && tagged_ready(wm[w], wl[w], tag)) {
                fm[w] = __uint_as_float(static_cast<uint32_t>(wm[w]));
                fl[w] = __uint_as_float(static_cast<uint32_t>(wl[w]));
                ml_pending &= ~(1u << w);
            }
        }
    }
    if (gave_up) report(p, B200KV_STATUS_PEER_TIMEOUT);
    float M2 = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMaxExchangeRanks; ++w)
        if (!(fl[w] <= 0.0f) && fm[w] != -INFINITY) M2 = fmaxf(M2, fm[w]);   // ranks beyond `world` keep l = 0
    float2 t2 = make_float2(0.0f, 0.0f);
    float l2 = 0.0f;
#pragma unroll
    for (int w = 0; w < kMaxExchangeRanks; ++w) {
        const float a = (!(fl[w] <= 0.0f) && fm[w] != -INFINITY) ? __expf(fm[w] - M2) : 0.0f;
        l2 = fmaf(fl[w], a, l2);
        t2.x = fmaf(fa[w], a, t2.x);
        t2.y = fmaf(fb[w], a, t2.y);
    }
    if (lost) { t2.x = t2.y = l2 = __int_as_float(0x7fc00000); }
    tot = t2;
    gsum = l2;
    // consumed: every thread zeroes its accumulator words; (m, l) only after all 64 threads have read them
    for (uint32_t w = 0; w < x.world; ++w) zero2(in + w * words_per_rank + 2 * pr);
    asm volatile("bar.sync 1, 64;" ::: "memory");
    if (pr == 0)
        for (uint32_t w = 0; w < x.world; ++w) zero2(in + w * words_per_rank + kD);
}

// Normalise, gate and store the merged result of one head (64 threads, two dims each), with the optional Q8_1
// re-quantisation of the gated output the reference's stage 2 offers for the projection that follows
// (.hip:2354-2383: blocks of 32, d = amax/127, q = roundf(x/d) clamped to +-127, s = d * sum(q), both fp16).
// Uses named barrier 1 (64 threads) only when the Q8_1 output is requested.
__device__ __forceinline__ void write_merged(const MergeParams& f, uint32_t session, uint32_t head, int pr, float2 tot, float gsum,
                                             float m_merged) {
    constexpr int kD = 128;
    const size_t out_idx = (static_cast<size_t>(session) * f.query_heads + head) * kD + 2 * pr;
    if (f.out_m != nullptr) {   // sequence shard: one merged, unnormalised partial
        *reinterpret_cast<float2*>(f.out_acc + out_idx) = tot;
        if (pr == 0) {
            f.out_m[static_cast<size_t>(session) * f.query_heads + head] = m_merged;
            f.out_l[static_cast<size_t>(session) * f.query_heads + head] = gsum;
        }
        return;
    }
    const float inv = gsum > 0.0f ? 1.0f / gsum : (gsum == gsum ? 0.0f : gsum);
    float2 o = make_float2(tot.x * inv, tot.y * inv);
    if (f.output != nullptr) *reinterpret_cast<float2*>(f.output + out_idx) = o;
    if (f.gated_output != nullptr || f.gated_output_q8 != nullptr) {
        if (f.gate != nullptr) {
            const float2 gt = *reinterpret_cast<const float2*>(f.gate + out_idx);
            o.x *= 1.0f / (1.0f + __expf(-gt.x)); o.y *= 1.0f / (1.0f + __expf(-gt.y));
        }
        if (f.gated_output != nullptr) *reinterpret_cast<float2*>(f.gated_output + out_idx) = o;
        if (f.gated_output_q8 != nullptr) {
            // a block of 32 values = 16 consecutive threads of a warp
            float amax = fmaxf(fabsf(o.x), fabsf(o.y));
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            const float dq = __fdiv_rn(amax, 127.0f);                       // IEEE operations: a host restatement reproduces the bits
            const float id = dq != 0.0f ? __fdiv_rn(1.0f, dq) : 0.0f;
            const int q0 = max(-127, min(127, static_cast<int>(roundf(__fmul_rn(o.x, id)))));
            const int q1 = max(-127, min(127, static_cast<int>(roundf(__fmul_rn(o.y, id)))));
            int qs = q0 + q1;
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) qs += __shfl_xor_sync(0xffffffffu, qs, off);
            const size_t block = ((static_cast<size_t>(session) * f.query_heads + head) * kD) / 32 + (pr >> 4);
            b200kv_q8_1_block* dst = f.gated_output_q8 + block;
            reinterpret_cast<char2*>(dst->qs)[pr & 15] = make_char2(static_cast<signed char>(q0), static_cast<signed char>(q1));
            if ((pr & 15) == 0) {
                const __half dh = __float2half_rn(dq), sh = __float2half_rn(__fmul_rn(static_cast<float>(qs), dq));
                dst->d = *reinterpret_cast<const uint16_t*>(&dh);
                dst->s = *reinterpret_cast<const uint16_t*>(&sh);
            }
        }
    }
}

// ---- fused merge: the CTA of split h merges query head h of its kv head (h, h + splits, ... if there are fewer
// splits than heads).  It polls the tagged partials of all splits -- normally they are all there by the time it
// has finished its own share -- and every other CTA simply leaves.  (Electing instead the CTAs that arrive last, with
// an atomic counter behind the partial stores, measured slower: the atomic's round trip and the merger reading its
// own partial back through L2 cost more than the polls they save.)  Called by ALL 256 threads of the CTA after they
// have issued their emit_partial stores (the CTAs that have nothing to merge return at once); uses named barriers
// 1 (64 threads) and 2 (256 threads).  fold_area: (8 + 3 * 64 * 2) floats of shared memory nothing else uses any more.
__device__ __forceinline__ void fused_merge(const DecodeParams& p, uint32_t session, uint32_t kv_head, uint32_t split,
                                            uint32_t num_splits, int G, float* fold_area) {
    constexpr int kD = 128;
    constexpr int kPartialWords = kD + 2;
    if (merge_not_needed(p, num_splits)) return;
    const uint32_t S = num_splits;     // <= kMaxSplitsPerSession == 128; the partial arrays keep the launch-wide stride
    const uint32_t rank = split;
    if (rank >= static_cast<uint32_t>(G)) return;
    const uint32_t tag = p.tag;
    float* fold_ml = fold_area;                                   // [3] x {max, sum} of split groups 1..3
    float2* fold = reinterpret_cast<float2*>(fold_ml + 8);        // [3][64] partial sums of split groups 1..3
    constexpr int kBatch = 10;   // splits per thread and round: 4 groups x 10 = 40 splits in one trip to L2
    // 256 threads = 4 split groups (sp % 4) x 64 pairs of dims.  A group merges its own splits on line (every thread
    // of a group also reads the group's (m, l) words itself: no staging, no barrier), then the 4 groups are folded.
    const int grp = threadIdx.x >> 6, pr = threadIdx.x & 63;
    for (uint32_t h = rank; h < static_cast<uint32_t>(G); h += S) {
        const uint32_t head = kv_head * G + h;
        const size_t stride = static_cast<size_t>(p.query_heads) * kPartialWords;   // words between consecutive splits
        uint64_t* base = p.ws_tagged + ((static_cast<size_t>(session) * p.num_splits) * p.query_heads + head) * kPartialWords;
        bool lost = false;
        float2 tot = make_float2(0.0f, 0.0f);
        float Mg = -INFINITY, lg = 0.0f;
        for (uint32_t sp0 = 0; sp0 < S; sp0 += 4 * kBatch) {
            // Poll in rounds: every round re-issues, back to back, the loads of all words of this thread that have
            // not shown their tag yet, so that once the last partial has landed one trip to L2 completes the set.
            float fa[kBatch], fb[kBatch], fm[kBatch], fl[kBatch];
            uint32_t pending = 0;
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                fa[u] = fb[u] = fl[u] = 0.0f;
                fm[u] = -INFINITY;
                if (sp0 + grp + 4 * u < S) pending |= 1u << u;
            }
            uint32_t ml_pending = pending;
            for (uint32_t polls = 0; (pending | ml_pending) != 0 && !lost; ++polls) {
                if (polls >= kPollLimit) { lost = true; report(p, B200KV_STATUS_SPLIT_TIMEOUT); break; }
                // all loads first, all checks afterwards: a check between two loads would serialise their trips
                uint64_t wa[kBatch], wb[kBatch], wm[kBatch], wl[kBatch];
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    uint64_t* src = base + (sp0 + grp + 4 * u) * stride;
                    wa[u] = wb[u] = wm[u] = wl[u] = 0;
                    if (pending & (1u << u)) ld_tagged2(src + 2 * pr, wa[u], wb[u]);
                    if (ml_pending & (1u << u)) ld_tagged2(src + kD, wm[u], wl[u]);
                }
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    if ((pending & (1u << u)) && tagged_ready(wa[u], wb[u], tag)) {
                        fa[u] = __uint_as_float(static_cast<uint32_t>(wa[u]));
                        fb[u] = __uint_as_float(static_cast<uint32_t>(wb[u]));
                        pending &= ~(1u << u);
                    }
                    if ((ml_pending & (1u << u)) && tagged_ready(wm[u], wl[u], tag)) {
                        fm[u] = __uint_as_float(static_cast<uint32_t>(wm[u]));
                        fl[u] = __uint_as_float(static_cast<uint32_t>(wl[u]));
                        ml_pending &= ~(1u << u);
                    }
                }
            }
            float Mr = Mg;
#pragma unroll
            for (int u = 0; u < kBatch; ++u)
                if (!(fl[u] <= 0.0f) && fm[u] != -INFINITY) Mr = fmaxf(Mr, fm[u]);   // keeps NaN partials in play
            const float keep = (Mg == -INFINITY) ? 0.0f : __expf(Mg - Mr);
            tot.x *= keep; tot.y *= keep; lg *= keep;
            Mg = Mr;
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const float a = (!(fl[u] <= 0.0f) && fm[u] != -INFINITY) ? __expf(fm[u] - Mg) : 0.0f;
                lg = fmaf(fl[u], a, lg);
                tot.x = fmaf(fa[u], a, tot.x);
                tot.y = fmaf(fb[u], a, tot.y);
            }
            // consumed: accumulator words by the thread that read them; (m, l) words are read by all 64 threads of
            // the group, so they are zeroed after the fold barrier below
#pragma unroll
            for (int u = 0; u < kBatch; ++u)
                if (sp0 + grp + 4 * u < S) zero2(base + (sp0 + grp + 4 * u) * stride + 2 * pr);
        }
        if (lost) tot.x = tot.y = lg = __int_as_float(0x7fc00000);
        // fold the 4 split groups through shared memory
        if (grp > 0) {
            fold[(grp - 1) * 64 + pr] = tot;
            if (pr == 0) { fold_ml[2 * (grp - 1)] = Mg; fold_ml[2 * (grp - 1) + 1] = lg; }
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");
        for (uint32_t sp = threadIdx.x; sp < S; sp += 256)   // every thread of every group is past its polls
            zero2(base + sp * stride + kD);
        if (grp == 0) {
            float M = Mg;
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float mk = fold_ml[2 * k], lk = fold_ml[2 * k + 1];
                if (!(lk <= 0.0f) && mk != -INFINITY) M = fmaxf(M, mk);
            }
            {
                const float a0 = (!(lg <= 0.0f) && Mg != -INFINITY) ? __expf(Mg - M) : 0.0f;
                tot.x *= a0; tot.y *= a0; lg *= a0;
            }
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float mk = fold_ml[2 * k], lk = fold_ml[2 * k + 1];
                const float a = (!(lk <= 0.0f) && mk != -INFINITY) ? __expf(mk - M) : 0.0f;
                const float2 o2 = fold[k * 64 + pr];
                tot.x = fmaf(o2.x, a, tot.x); tot.y = fmaf(o2.y, a, tot.y);
                lg = fmaf(lk, a, lg);
            }
            float gsum = lg;
            const float m_merged = M;
            if (p.fuse.xchg.world > 1) exchange_partials(p, head, pr, m_merged, tot, gsum, lost);
            write_merged(p.fuse, session, head, pr, tot, gsum, m_merged);
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");   // the fold area is reused by the next head of this CTA
    }
}

}  // namespace tail
}  // namespace b200kv
