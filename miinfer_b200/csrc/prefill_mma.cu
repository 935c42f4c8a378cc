// Suffix / prefill cross-query attention over a quantized prefix on tensor cores.
//
// Replaces MIInfer's suffix kernels (gfx906/kernels/qwen3_primitives.hip:6788-7119
// stage 1, 6637-6725 stage 2).  The reference launches one wave per (query token,
// head pair, split): every wave re-streams its whole causal KV range and the
// partials of 32 splits go through a 400 MB workspace.  Here one CTA owns 64
// query ROWS of one kv head -- a row is a (token, head-of-the-group) pair, so all
// G query heads of the group share each dequantised K/V tile -- walks the causal
// range once in tiles of 64 positions, and keeps the running (max, sum, output)
// in registers: no workspace, no second kernel, KV read once per 64 rows.
//
// Per tile: int8 K/V rows are loaded with 16-byte loads, dequantised to fp16
// (byte-permute into the mantissa of 1024.0h, an exact subtract of the offset and
// one multiply by the block scale per pair: a single rounding per value) into XOR-swizzled
// shared memory; S = Q.K^T and O += P.V run as m16n8k16 tensor-core MMAs with
// fp32 accumulation (ldmatrix operands; P goes from the S accumulators straight
// into A fragments); softmax is the online form in base 2; causality is the
// per-row length base_position + token + 1 (.hip:6829); the sigmoid gate is
// applied with the final 1/sum (.hip:6714-6723).
#include "decode_common.cuh"
#include "dequant.cuh"

#include <mutex>

namespace b200kv {

namespace {

constexpr int kBM = 64;       // query rows per CTA (4 warps x 16)
constexpr int kBN = 64;       // positions per KV tile
constexpr int kThreads = 128;

struct PrefillParams {
    b200kv_view view;
    const void* q;           // [token][query_heads][D]
    int q_is_f16;
    const float* gate;       // [token][query_heads][D] or null
    float* out;              // [token][query_heads][D]
    uint32_t token_count;
    uint32_t base_position;
    const b200kv_prefill_state* prefill_state;
    uint32_t query_heads;
    float scale_log2;        // softmax scale * log2(e)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a [rows][D] fp16 tile: chunks are XORed with the row's
// low bits so that the 8 rows an ldmatrix phase touches land in distinct banks.
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return static_cast<uint32_t>(row) * (D * 2) + (static_cast<uint32_t>(chunk ^ (row & 7)) << 4);
}

// Loads positions [pos0, pos0 + kBN) of one kv head into a swizzled fp16 tile; rows at or beyond `limit` are zero.
template <int D>
__device__ __forceinline__ void load_tile(uint8_t* tile, bool is_q8, const int8_t* q8, const __half* scales, const __half* f16,
                                          uint32_t nblk, uint64_t head_row0, uint32_t pos0, uint32_t limit, int tid) {
    if (is_q8) {
        constexpr int CPR = D / 16;   // 16-byte int8 chunks per row
#pragma unroll 4
        for (int idx = tid; idx < kBN * CPR; idx += kThreads) {
            const int row = idx / CPR, c16 = idx % CPR;
            const uint32_t pos = pos0 + row;
            uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
            if (pos < limit) {
                const uint64_t grow = head_row0 + pos;
                const uint4 raw = *reinterpret_cast<const uint4*>(q8 + grow * D + c16 * 16);
                const __half sc = scales[grow * nblk + (nblk == 1 ? 0 : c16 / 2)];
                dequant16(raw, sc, &lo, &hi);
            }
            *reinterpret_cast<uint4*>(tile + tile_off<D>(row, 2 * c16)) = lo;
            *reinterpret_cast<uint4*>(tile + tile_off<D>(row, 2 * c16 + 1)) = hi;
        }
    } else {
        constexpr int CPR = D / 8;    // 16-byte fp16 chunks per row
#pragma unroll 4
        for (int idx = tid; idx < kBN * CPR; idx += kThreads) {
            const int row = idx / CPR, c = idx % CPR;
            const uint32_t pos = pos0 + row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (pos < limit) v = *reinterpret_cast<const uint4*>(f16 + (head_row0 + pos) * D + c * 8);
            *reinterpret_cast<uint4*>(tile + tile_off<D>(row, c)) = v;
        }
    }
}

template <int D>
__global__ void __launch_bounds__(kThreads, (D == 256 ? 2 : 3))
prefill_mma_kernel(const __grid_constant__ PrefillParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* q_tile = smem;
    uint8_t* k_tile = smem + kBM * D * 2;
    uint8_t* v_tile = k_tile + kBN * D * 2;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t kv_head = blockIdx.y;
    const uint32_t G = p.query_heads / p.view.kv_heads;
    uint32_t base = p.base_position, count = p.token_count;
    if (p.prefill_state != nullptr) {
        base = p.prefill_state->base_position;
        count = min(count, p.prefill_state->token_count);
    }
    const uint32_t total_rows = p.token_count * G;       // rows this launch owns (written even if past `count`: zeros)
    const uint32_t row0 = blockIdx.x * kBM;
    if (row0 >= total_rows) return;
    const uint64_t capacity = p.view.capacity;
    const uint32_t mode = p.view.quant_mode;
    const bool k_q8 = (mode == B200KV_Q8_F16 || mode == B200KV_Q8_Q8), v_q8 = (mode == B200KV_F16_Q8 || mode == B200KV_Q8_Q8);
    const uint32_t nblk = D / p.view.qblock;
    const uint64_t head_row0 = static_cast<uint64_t>(kv_head) * capacity;

    // causal length of a row: base + token + 1, or 0 when the token is past the device-side count or the cache
    auto row_length = [&](uint32_t r) -> uint32_t {
        if (r >= total_rows) return 0u;
        const uint32_t token = r / G;
        const uint64_t len = static_cast<uint64_t>(base) + token + 1u;
        return (token < count && len <= capacity) ? static_cast<uint32_t>(len) : 0u;
    };

    // ---- stage Q (fp16, swizzled) ---------------------------------------------------------
    {
        constexpr int CPR = D / 8;
        for (int idx = tid; idx < kBM * CPR; idx += kThreads) {
            const int r = idx / CPR, c = idx % CPR;
            const uint32_t gr = row0 + r;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (gr < total_rows) {
                const uint32_t token = gr / G, head = kv_head * G + gr % G;
                const size_t off = (static_cast<size_t>(token) * p.query_heads + head) * D + c * 8;
                if (p.q_is_f16) {
                    v = *reinterpret_cast<const uint4*>(static_cast<const __half*>(p.q) + off);
                } else {
                    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(p.q) + off);
                    const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(p.q) + off + 4);
                    v = make_uint4(pack_half2(a.x, a.y), pack_half2(a.z, a.w), pack_half2(b.x, b.y), pack_half2(b.z, b.w));
                }
            }
            *reinterpret_cast<uint4*>(q_tile + tile_off<D>(r, c)) = v;
        }
    }

    // this thread's two rows: lane/4 and lane/4 + 8 of the warp's 16
    const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
    const uint32_t len_lo = row_length(row0 + r_lo), len_hi = row_length(row0 + r_hi);
    // the CTA scans up to its longest row: lengths grow with the token index until they drop to 0 (token past the
    // device-side count, or causal range past the cache), so the longest row belongs to the last token still valid
    uint32_t kv_end = 0;
    if (count > 0 && capacity > base) {
        const uint32_t t_first = row0 / G, t_last = (min(row0 + kBM, total_rows) - 1) / G;
        const uint64_t t_cap = capacity - base - 1;   // largest token whose range fits the cache
        uint64_t t_max = t_last;
        if (t_max > count - 1) t_max = count - 1;
        if (t_max > t_cap) t_max = t_cap;
        if (t_max >= t_first) kv_end = base + static_cast<uint32_t>(t_max) + 1u;
    }

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = 0.0f; o[i][1] = 0.0f; o[i][2] = 0.0f; o[i][3] = 0.0f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;

    const uint32_t q_base = smem_u32(q_tile), k_base = smem_u32(k_tile), v_base = smem_u32(v_tile);

    for (uint32_t pos0 = 0; pos0 < kv_end; pos0 += kBN) {
        __syncthreads();   // everyone is done with the previous tile (and Q is staged on the first pass)
        load_tile<D>(k_tile, k_q8, p.view.key_q8, static_cast<const __half*>(p.view.key_scales),
                     static_cast<const __half*>(p.view.key_f16), nblk, head_row0, pos0, kv_end, tid);
        load_tile<D>(v_tile, v_q8, p.view.value_q8, static_cast<const __half*>(p.view.value_scales),
                     static_cast<const __half*>(p.view.value_f16), nblk, head_row0, pos0, kv_end, tid);
        __syncthreads();

        // ---- S = Q . K^T (16 rows x 64 positions per warp) -----------------------------------
        float s[kBN / 8][4];
#pragma unroll
        for (int j = 0; j < kBN / 8; ++j) { s[j][0] = 0.0f; s[j][1] = 0.0f; s[j][2] = 0.0f; s[j][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t a0, a1, a2, a3;
            ldsm_x4(q_base + tile_off<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)), a0, a1, a2, a3);
#pragma unroll
            for (int nb = 0; nb < kBN / 16; ++nb) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(k_base + tile_off<D>(nb * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
                mma_16816(s[2 * nb], a0, a1, a2, a3, b0, b1);
                mma_16816(s[2 * nb + 1], a0, a1, a2, a3, b2, b3);
            }
        }

        // ---- causal mask, online softmax (base 2) ----------------------------------------------
        float mt_lo = -INFINITY, mt_hi = -INFINITY;
#pragma unroll
        for (int j = 0; j < kBN / 8; ++j) {
            const uint32_t col = pos0 + j * 8 + (lane & 3) * 2;
            s[j][0] = (col < len_lo) ? s[j][0] * p.scale_log2 : -INFINITY;
            s[j][1] = (col + 1 < len_lo) ? s[j][1] * p.scale_log2 : -INFINITY;
            s[j][2] = (col < len_hi) ? s[j][2] * p.scale_log2 : -INFINITY;
            s[j][3] = (col + 1 < len_hi) ? s[j][3] * p.scale_log2 : -INFINITY;
            mt_lo = fmaxf(mt_lo, fmaxf(s[j][0], s[j][1]));
            mt_hi = fmaxf(mt_hi, fmaxf(s[j][2], s[j][3]));
        }
        mt_lo = fmaxf(mt_lo, __shfl_xor_sync(0xffffffffu, mt_lo, 1));
        mt_lo = fmaxf(mt_lo, __shfl_xor_sync(0xffffffffu, mt_lo, 2));
        mt_hi = fmaxf(mt_hi, __shfl_xor_sync(0xffffffffu, mt_hi, 1));
        mt_hi = fmaxf(mt_hi, __shfl_xor_sync(0xffffffffu, mt_hi, 2));
        const float mn_lo = fmaxf(m_lo, mt_lo), mn_hi = fmaxf(m_hi, mt_hi);
        const float ms_lo = (mn_lo == -INFINITY) ? 0.0f : mn_lo, ms_hi = (mn_hi == -INFINITY) ? 0.0f : mn_hi;   // fully masked so far
        const float al_lo = exp2f(m_lo - ms_lo), al_hi = exp2f(m_hi - ms_hi);
        m_lo = mn_lo; m_hi = mn_hi;
        float sum_lo = 0.0f, sum_hi = 0.0f;
        uint32_t pa[kBN / 16][4];
#pragma unroll
        for (int j = 0; j < kBN / 8; ++j) {
            const float p0 = exp2f(s[j][0] - ms_lo), p1 = exp2f(s[j][1] - ms_lo);
            const float p2 = exp2f(s[j][2] - ms_hi), p3 = exp2f(s[j][3] - ms_hi);
            sum_lo += p0 + p1; sum_hi += p2 + p3;
            // accumulators of position tiles 2kk, 2kk+1 are exactly the A fragment of k-step kk
            pa[j >> 1][(j & 1) * 2] = pack_half2(p0, p1);
            pa[j >> 1][(j & 1) * 2 + 1] = pack_half2(p2, p3);
        }
        l_lo = fmaf(l_lo, al_lo, sum_lo);
        l_hi = fmaf(l_hi, al_hi, sum_hi);
        if (al_lo != 1.0f || al_hi != 1.0f) {
#pragma unroll
            for (int i = 0; i < D / 8; ++i) { o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi; }
        }

        // ---- O += P . V ------------------------------------------------------------------------
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
#pragma unroll
            for (int nd = 0; nd < D / 16; ++nd) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(v_base + tile_off<D>(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), nd * 2 + (lane >> 4)), b0, b1, b2, b3);
                mma_16816(o[2 * nd], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                mma_16816(o[2 * nd + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
            }
        }
    }

    // ---- finish: row sums across the quad, 1/sum, gate, store ----------------------------------
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = l_lo > 0.0f ? 1.0f / l_lo : 0.0f, inv_hi = l_hi > 0.0f ? 1.0f / l_hi : 0.0f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const uint32_t gr = row0 + (half ? r_hi : r_lo);
        if (gr >= total_rows) continue;
        const uint32_t token = gr / G, head = kv_head * G + gr % G;
        const size_t off = (static_cast<size_t>(token) * p.query_heads + head) * D + (lane & 3) * 2;
        const float inv = half ? inv_hi : inv_lo;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            float2 v = make_float2(o[i][half * 2] * inv, o[i][half * 2 + 1] * inv);
            if (p.gate != nullptr) {
                const float2 g = *reinterpret_cast<const float2*>(p.gate + off + i * 8);
                v.x *= 1.0f / (1.0f + __expf(-g.x));
                v.y *= 1.0f / (1.0f + __expf(-g.y));
            }
            *reinterpret_cast<float2*>(p.out + off + i * 8) = v;
        }
    }
}

template <int D>
int launch_prefill(const PrefillParams& p, cudaStream_t stream) {
    constexpr int kSmem = (kBM + 2 * kBN) * D * 2;
    static std::atomic<uint64_t> done{0};   // one per kernel instantiation: devices that have opted in
    const cudaError_t attr_err = opt_in_dynamic_smem(reinterpret_cast<const void*>(prefill_mma_kernel<D>), kSmem, done);
    if (attr_err != cudaSuccess) { set_last_cuda_error(attr_err, "cudaFuncSetAttribute(prefill_mma)"); return B200KV_ERR_CUDA; }
    const uint32_t G = p.query_heads / p.view.kv_heads;
    const uint32_t row_tiles = (p.token_count * G + kBM - 1) / kBM;
    prefill_mma_kernel<D><<<dim3(row_tiles, p.view.kv_heads), kThreads, kSmem, stream>>>(p);
    B200KV_CUDA_TRY(cudaGetLastError());
    return B200KV_OK;
}

}  // namespace

int launch_prefill_mma(const b200kv_view& view, const void* q, int q_is_f16, const float* gate, float* out,
                       uint32_t token_count, uint32_t base_position, const b200kv_prefill_state* prefill_state,
                       uint32_t query_heads, float scale, cudaStream_t stream) {
    PrefillParams p{};
    p.view = view;
    p.q = q;
    p.q_is_f16 = q_is_f16;
    p.gate = gate;
    p.out = out;
    p.token_count = token_count;
    p.base_position = base_position;
    p.prefill_state = prefill_state;
    p.query_heads = query_heads;
    p.scale_log2 = scale * 1.4426950408889634f;
    return view.head_dim == 128 ? launch_prefill<128>(p, stream) : launch_prefill<256>(p, stream);
}

}  // namespace b200kv
