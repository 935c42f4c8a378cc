/*
 * kv_oracle.c -- CPU restatement of MIInfer's quantized KV-cache hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * with and the timed CPU baseline; nothing in the shipped library links, loads
 * or calls it.  Plain C (gcc, -O2 -ffp-contract=off -pthread).  Every function
 * names the reference file:line whose arithmetic it follows (paths are relative
 * to the MIInfer source tree).
 *
 * Parity pin: the fp16 conversions, NeoX RoPE, softmax and the fp32 attention
 * loop are checked against (a) the reference's own host primitives compiled in
 * place (oracle/_ref, built by oracle/Makefile) and (b) the reference's stored
 * layer-0 traces (tests/golden/m4a4_four_position.npz).  The int8 store and the
 * quantized attention kernels have NO stored vectors and NO CPU implementation
 * in the reference (its tests only compare two GPU kernels with each other), so
 * for those two this file is a restatement of the HIP kernels' arithmetic and
 * their bit-level parity is "unpinned" by reference data.  What the reference
 * does publish for them is pinned: on the inputs of its quantized-attention
 * test (tests/qwen3_quant_kv_attention_test.cpp:79-154, drawn here from the same
 * std::mt19937(42) stream) the suffix split-K restatement with the test's host
 * quantiser gives the errors its experiment record quotes -- max-abs 0.001263,
 * MAE 0.000011, cosine 0.999973 (experiments/EXP-V2-0024-quantized-prefix-kv.md:
 * 122-126) -- to every printed digit (tests/test_statistical_pin.py).
 *
 * Deliberate, documented deviations from the HIP kernels (both sides of the
 * parity tests -- this file and the CUDA kernels -- use the same definition):
 *   - rsqrtf(x) (approximate on a GPU) is defined as 1.0f / sqrtf(x);
 *   - cosf/sinf differ by ulps between math libraries, so RoPE trig is a pinned
 *     routine built from IEEE double fma only (kvo_sincos_pinned); the libm
 *     variant is kept (trig_mode 0) for checks against reference traces;
 *   - a*b-c*d style expressions are evaluated without fused contraction.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>

#define KVO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* A small pthread parallel-for (the reference's host loop is single-threaded; */
/* the thread count is only raised for the "all host cores" baseline figure)   */
/* ------------------------------------------------------------------------- */

static int kvo_threads = 1;
KVO_API int kvo_num_threads(void) { return kvo_threads; }
KVO_API void kvo_set_num_threads(int n) { kvo_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }

typedef void (*kvo_body_fn)(size_t index, void* ctx);
typedef struct { kvo_body_fn fn; void* ctx; size_t count; size_t next; pthread_mutex_t lock; } kvo_job;

static void* kvo_worker(void* arg) {
    kvo_job* job = (kvo_job*)arg;
    for (;;) {
        pthread_mutex_lock(&job->lock);
        size_t i = job->next++;
        pthread_mutex_unlock(&job->lock);
        if (i >= job->count) return NULL;
        job->fn(i, job->ctx);
    }
}

static void kvo_parallel_for(size_t count, kvo_body_fn fn, void* ctx) {
    int nt = kvo_threads;
    if ((size_t)nt > count) nt = (int)count;
    if (nt <= 1) { for (size_t i = 0; i < count; ++i) fn(i, ctx); return; }
    kvo_job job = { fn, ctx, count, 0, PTHREAD_MUTEX_INITIALIZER };
    pthread_t tid[256];
    for (int t = 1; t < nt; ++t) pthread_create(&tid[t], NULL, kvo_worker, &job);
    kvo_worker(&job);
    for (int t = 1; t < nt; ++t) pthread_join(tid[t], NULL);
}

/* ------------------------------------------------------------------------- */
/* fp16 <-> fp32, bit exact                                                   */
/* ------------------------------------------------------------------------- */

/* Follows fp16_bits_to_float, src/qwen3_primitives.cpp:67-91. */
KVO_API float kvo_half_to_float(uint16_t bits) {
    uint32_t sign = ((uint32_t)(bits & 0x8000u)) << 16;
    uint32_t exponent = (bits >> 10) & 0x1fu;
    uint32_t fraction = bits & 0x03ffu;
    uint32_t value = sign;
    if (exponent == 0) {
        if (fraction != 0) {
            uint32_t shift = 0;
            while ((fraction & 0x0400u) == 0) { fraction <<= 1; ++shift; }
            fraction &= 0x03ffu;
            value |= (127u - 15u - shift + 1u) << 23;
            value |= fraction << 13;
        }
    } else if (exponent == 0x1fu) {
        value |= 0x7f800000u | (fraction << 13);
    } else {
        value |= (exponent + (127u - 15u)) << 23;
        value |= fraction << 13;
    }
    float out;
    memcpy(&out, &value, sizeof out);
    return out;
}

/* Round-to-nearest-even fp32 -> fp16; follows float_to_half_bits_rn,
 * src/qwen3_layer.cpp:27-61 (same results as __float2half_rn on the device). */
KVO_API uint16_t kvo_float_to_half_rn(float value) {
    uint32_t bits;
    memcpy(&bits, &value, sizeof bits);
    uint32_t sign = (bits >> 16) & 0x8000u;
    uint32_t exponent = (bits >> 23) & 0xffu;
    uint32_t mantissa = bits & 0x7fffffu;
    if (exponent == 0xffu) return (uint16_t)(sign | 0x7c00u | (mantissa ? 0x0200u : 0u));
    int he = (int)exponent - 127 + 15;
    if (he <= 0) {
        if (he < -10) return (uint16_t)sign;
        uint32_t significand = mantissa | 0x00800000u;
        int shift = 14 - he;
        uint32_t rounded = significand >> shift;
        uint32_t remainder = significand & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (remainder > halfway || (remainder == halfway && (rounded & 1u))) ++rounded;
        return (uint16_t)(sign | rounded);
    }
    if (he >= 31) return (uint16_t)(sign | 0x7c00u);
    uint32_t rm = mantissa >> 13;
    uint32_t remainder = mantissa & 0x1fffu;
    if (remainder > 0x1000u || (remainder == 0x1000u && (rm & 1u))) {
        ++rm;
        if (rm == 0x400u) {
            if (he + 1 >= 31) return (uint16_t)(sign | 0x7c00u);
            return (uint16_t)(sign | ((uint32_t)(he + 1) << 10));
        }
    }
    return (uint16_t)(sign | ((uint32_t)he << 10) | rm);
}

KVO_API void kvo_half_to_float_array(const uint16_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = kvo_half_to_float(in[i]);
}
KVO_API void kvo_float_to_half_array(const float* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = kvo_float_to_half_rn(in[i]);
}

/* ------------------------------------------------------------------------- */
/* RoPE                                                                       */
/* ------------------------------------------------------------------------- */

/* Pinned sin/cos of an fp32 angle.  Not in the reference: it replaces
 * cosf/sinf (gfx906/kernels/qwen3_primitives.hip:655-656, 1862-1863) whose bits
 * are library-specific.  IEEE double fma/mul/rint only, so a GPU evaluating the
 * same sequence returns the same floats.  Cody-Waite reduction by pi/2 with a
 * two-term constant, Taylor polynomials to x^17 / x^16 on |r| <= pi/4. */
KVO_API void kvo_sincos_pinned(float angle, float* s_out, float* c_out) {
    const double two_over_pi = 0x1.45f306dc9c883p-1;
    const double pio2_hi = 0x1.921fb54442d18p+0;
    const double pio2_lo = 0x1.1a62633145c07p-54;
    double x = (double)angle;
    double kd = rint(x * two_over_pi);
    double r = fma(-kd, pio2_hi, x);
    r = fma(-kd, pio2_lo, r);
    double z = r * r;
    double ps = 0x1.952c77030ad4ap-49;
    ps = fma(ps, z, -0x1.ae7f3e733b81fp-41);
    ps = fma(ps, z, 0x1.6124613a86d09p-33);
    ps = fma(ps, z, -0x1.ae64567f544e4p-26);
    ps = fma(ps, z, 0x1.71de3a556c734p-19);
    ps = fma(ps, z, -0x1.a01a01a01a01ap-13);
    ps = fma(ps, z, 0x1.1111111111111p-7);
    ps = fma(ps, z, -0x1.5555555555555p-3);
    double sr = fma(ps * z, r, r);
    double pc = 0x1.ae7f3e733b81fp-45;
    pc = fma(pc, z, -0x1.93974a8c07c9dp-37);
    pc = fma(pc, z, 0x1.1eed8eff8d898p-29);
    pc = fma(pc, z, -0x1.27e4fb7789f5cp-22);
    pc = fma(pc, z, 0x1.a01a01a01a01ap-16);
    pc = fma(pc, z, -0x1.6c16c16c16c17p-10);
    pc = fma(pc, z, 0x1.5555555555555p-5);
    pc = fma(pc, z, -0.5);
    double cr = fma(pc, z, 1.0);
    int q = (int)((long long)kd & 3LL);
    double sv = (q & 1) ? cr : sr;
    double cv = (q & 1) ? sr : cr;
    if (q == 2 || q == 3) sv = -sv;
    if (q == 1 || q == 2) cv = -cv;
    *s_out = (float)sv;
    *c_out = (float)cv;
}

static void kvo_sincos(float angle, int trig_mode, float* s, float* c) {
    if (trig_mode == 0) { *s = sinf(angle); *c = cosf(angle); }
    else kvo_sincos_pinned(angle, s, c);
}

/* NeoX frequency for pair i: powf(theta, -2i/d); follows rope_qwen3_reference,
 * src/qwen3_primitives.cpp:122-124 and qwen3_rope_kernel, .hip:1859. */
KVO_API float kvo_neox_inv_freq(float theta, uint32_t pair, uint32_t head_dim) {
    return powf(theta, -(float)(2 * pair) / (float)head_dim);
}

/* Angle of the sectioned Qwen3.5 RoPE for pair `local` (<32): position scaled by
 * powf(theta, -2/64) `local` times with successive fp32 multiplies; every
 * section resolves to the text position.  Follows compute_qwen35_rope_pair,
 * gfx906/kernels/qwen3_primitives.hip:622-659. */
KVO_API float kvo_sectioned64_angle(float theta, uint32_t local, uint32_t position) {
    float a = (float)position;
    const float step = powf(theta, -2.0f / 64.0f);
    for (uint32_t i = 0; i < local; ++i) a *= step;
    return a;
}

/* rope_mode: 0 none, 1 NeoX over the full head (pairs i, i+d/2), 2 sectioned on
 * dims [0,64) (pairs i, i+32).  trig_mode: 0 libm, 1 pinned.  In place on one
 * head row.  NeoX follows src/qwen3_primitives.cpp:109-135; sectioned follows
 * .hip:7270-7279. */
KVO_API void kvo_rope_row(float* row, uint32_t head_dim, uint32_t position, float theta,
                          int rope_mode, int trig_mode) {
    if (rope_mode == 1) {
        uint32_t half = head_dim / 2;
        for (uint32_t i = 0; i < half; ++i) {
            float angle = (float)position * kvo_neox_inv_freq(theta, i, head_dim);
            float s, c;
            kvo_sincos(angle, trig_mode, &s, &c);
            float x0 = row[i], x1 = row[i + half];
            row[i] = x0 * c - x1 * s;
            row[i + half] = x0 * s + x1 * c;
        }
    } else if (rope_mode == 2) {
        for (uint32_t i = 0; i < 32 && i + 32 < head_dim; ++i) {
            float angle = kvo_sectioned64_angle(theta, i, position);
            float s, c;
            kvo_sincos(angle, trig_mode, &s, &c);
            float x0 = row[i], x1 = row[i + 32];
            row[i] = x0 * c - x1 * s;
            row[i + 32] = x0 * s + x1 * c;
        }
    }
}

KVO_API void kvo_rope_heads(const float* in, float* out, uint32_t heads, uint32_t head_dim,
                            uint32_t position, float theta, int rope_mode, int trig_mode) {
    memcpy(out, in, (size_t)heads * head_dim * sizeof(float));
    for (uint32_t h = 0; h < heads; ++h)
        kvo_rope_row(out + (size_t)h * head_dim, head_dim, position, theta, rope_mode, trig_mode);
}

/* ------------------------------------------------------------------------- */
/* Cache view (host memory), same fields as the device view                   */
/* ------------------------------------------------------------------------- */

typedef struct kvo_view {
    uint16_t* key_f16;     /* [kv_heads][capacity][head_dim] or NULL            */
    uint16_t* value_f16;
    int8_t* key_q8;        /* [kv_heads][capacity][head_dim] or NULL            */
    uint16_t* key_scales;  /* [kv_heads][capacity][head_dim/qblock] fp16 bits   */
    int8_t* value_q8;
    uint16_t* value_scales;
    uint64_t capacity;
    uint32_t kv_heads;
    uint32_t head_dim;
    uint32_t qblock;       /* 32 (q8_0) or head_dim (the reference's row scale) */
    uint32_t quant_mode;   /* 0 f16/f16, 1 q8/f16, 2 f16/q8, 3 q8/q8; include/miinfer/prefill_v2/kv_cache.hpp:16-21 */
} kvo_view;

static int kvo_k_q8(const kvo_view* v) { return v->quant_mode == 1 || v->quant_mode == 3; }
static int kvo_v_q8(const kvo_view* v) { return v->quant_mode == 2 || v->quant_mode == 3; }

/* ------------------------------------------------------------------------- */
/* Append (store kernel)                                                      */
/* ------------------------------------------------------------------------- */

/* One quantization block.  quant_style 0 = the store kernel
 * (.hip:7285-7300): scale = amax>0 ? amax/127 : 1, inv = 1/scale, q =
 * round-half-even(x*inv) clamped to [-128,127], fp16 scale by RN.
 * quant_style 1 = the host quantizers (src/qwen3_layer.cpp:99-126,
 * tests/qwen3_quant_kv_attention_test.cpp:131-136): half-away rounding, clamp
 * [-127,127], inverse 0 for an all-zero block (stored scale 0). */
KVO_API void kvo_quantize_block(const float* x, uint32_t n, int quant_style, int8_t* q, uint16_t* scale_bits) {
    float amax = 0.0f;
    for (uint32_t i = 0; i < n; ++i) amax = fmaxf(amax, fabsf(x[i]));
    if (quant_style == 0) {
        float scale = (amax > 0.0f) ? (amax / 127.0f) : 1.0f;
        float inv = (scale > 0.0f) ? (1.0f / scale) : 1.0f;
        for (uint32_t i = 0; i < n; ++i) {
            float scaled = x[i] * inv;
            int v = (int)rintf(scaled); /* default rounding mode: nearest-even == __float2int_rn */
            if (v < -128) v = -128;
            if (v > 127) v = 127;
            q[i] = (int8_t)v;
        }
        *scale_bits = kvo_float_to_half_rn(scale);
    } else {
        float scale = amax / 127.0f;
        float inv = (scale > 0.0f) ? (1.0f / scale) : 0.0f;
        for (uint32_t i = 0; i < n; ++i) {
            float r = roundf(x[i] * inv);
            if (r < -127.0f) r = -127.0f;
            if (r > 127.0f) r = 127.0f;
            q[i] = (int8_t)r;
        }
        *scale_bits = kvo_float_to_half_rn(scale);
    }
}

/* Sum of squares by the store kernel's shared-memory binary tree: stride d/2
 * down to 1, element t += element t+stride (.hip:7257-7264). */
static float kvo_tree_sum_squares(const float* x, uint32_t d, float* scratch) {
    for (uint32_t i = 0; i < d; ++i) scratch[i] = x[i] * x[i];
    for (uint32_t stride = d / 2; stride > 0; stride /= 2)
        for (uint32_t t = 0; t < stride; ++t) scratch[t] += scratch[t + stride];
    return scratch[0];
}

/* Append `token_count` tokens at positions base_position + t.
 * key/value: fp32 [token][kv_heads*head_dim] (fp16 inputs are upcast exactly by
 * the caller).  k_norm_weight may be NULL (no K RMSNorm).  Follows
 * qwen35_decoupled_k_norm_rope_kv_store_batch_quant_kernel, .hip:7213-7326:
 * K: RMSNorm*w -> RoPE -> quantize/store; V: quantize/store.  Returns 0, or -1
 * if a position would fall outside the cache (the kernel's launcher contract). */
KVO_API int kvo_append(const kvo_view* view, const float* key, const float* value,
                       const float* k_norm_weight, uint32_t token_count, uint32_t base_position,
                       int rope_mode, float theta, float epsilon, int trig_mode, int quant_style) {
    const uint32_t d = view->head_dim, H = view->kv_heads, qb = view->qblock;
    if ((uint64_t)base_position + token_count > view->capacity) return -1;
    float* row = (float*)malloc(sizeof(float) * d * 2);
    float* scratch = row + d;
    const uint32_t nblk = d / qb;
    for (uint32_t t = 0; t < token_count; ++t) {
        for (uint32_t h = 0; h < H; ++h) {
            const float* k = key + ((size_t)t * H + h) * d;
            const float* v = value + ((size_t)t * H + h) * d;
            const uint32_t pos = base_position + t;
            if (k_norm_weight) {
                float ss = kvo_tree_sum_squares(k, d, scratch);
                float r = 1.0f / sqrtf(ss / (float)d + epsilon);
                for (uint32_t i = 0; i < d; ++i) row[i] = k[i] * r * k_norm_weight[i];
            } else {
                memcpy(row, k, sizeof(float) * d);
            }
            kvo_rope_row(row, d, pos, theta, rope_mode, trig_mode);
            size_t base = ((size_t)h * view->capacity + pos) * d;
            size_t sbase = ((size_t)h * view->capacity + pos) * nblk;
            if (kvo_k_q8(view)) {
                for (uint32_t b = 0; b < nblk; ++b)
                    kvo_quantize_block(row + b * qb, qb, quant_style, view->key_q8 + base + b * qb,
                                       view->key_scales + sbase + b);
            } else {
                for (uint32_t i = 0; i < d; ++i) view->key_f16[base + i] = kvo_float_to_half_rn(row[i]);
            }
            if (kvo_v_q8(view)) {
                for (uint32_t b = 0; b < nblk; ++b)
                    kvo_quantize_block(v + b * qb, qb, quant_style, view->value_q8 + base + b * qb,
                                       view->value_scales + sbase + b);
            } else {
                for (uint32_t i = 0; i < d; ++i) view->value_f16[base + i] = kvo_float_to_half_rn(v[i]);
            }
        }
    }
    free(row);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* Attention                                                                  */
/* ------------------------------------------------------------------------- */

/* q . k_row in fp32: per block (sum of q_i * (float)k8_i) * fp16 scale, blocks
 * added in order; for an fp16 cache the plain fp32 dot.  The per-position
 * arithmetic of .hip:7425-7440 with the per-row scale generalised to blocks. */
static float kvo_qk(const kvo_view* v, const float* q, uint32_t kv_head, uint64_t pos) {
    const uint32_t d = v->head_dim;
    size_t base = ((size_t)kv_head * v->capacity + pos) * d;
    if (kvo_k_q8(v)) {
        const uint32_t qb = v->qblock, nblk = d / qb;
        const int8_t* k8 = v->key_q8 + base;
        const uint16_t* ks = v->key_scales + ((size_t)kv_head * v->capacity + pos) * nblk;
        float total = 0.0f;
        for (uint32_t b = 0; b < nblk; ++b) {
            float prod = 0.0f;
            for (uint32_t i = 0; i < qb; ++i) prod += q[b * qb + i] * (float)k8[b * qb + i];
            total += prod * kvo_half_to_float(ks[b]);
        }
        return total;
    }
    const uint16_t* kh = v->key_f16 + base;
    float prod = 0.0f;
    for (uint32_t i = 0; i < d; ++i) prod += q[i] * kvo_half_to_float(kh[i]);
    return prod;
}

/* acc[i] = acc[i]*alpha + weight * value_row[i] in fp32 (.hip:7457-7476). */
static void kvo_pv(const kvo_view* v, float* acc, float alpha, float weight, uint32_t kv_head, uint64_t pos) {
    const uint32_t d = v->head_dim;
    size_t base = ((size_t)kv_head * v->capacity + pos) * d;
    if (kvo_v_q8(v)) {
        const uint32_t qb = v->qblock, nblk = d / qb;
        const int8_t* v8 = v->value_q8 + base;
        const uint16_t* vs = v->value_scales + ((size_t)kv_head * v->capacity + pos) * nblk;
        for (uint32_t b = 0; b < nblk; ++b) {
            float ew = weight * kvo_half_to_float(vs[b]);
            for (uint32_t i = 0; i < qb; ++i) acc[b * qb + i] = acc[b * qb + i] * alpha + ew * (float)v8[b * qb + i];
        }
    } else {
        const uint16_t* vh = v->value_f16 + base;
        for (uint32_t i = 0; i < d; ++i) acc[i] = acc[i] * alpha + weight * kvo_half_to_float(vh[i]);
    }
}

static float kvo_sigmoid(float g) { return 1.0f / (1.0f + expf(-g)); }

/* The tolerance target ("fp32-accumulated reference"): for each query head a
 * full two-pass softmax over dequantised values -- fp32 dot, scores * scale,
 * max-subtracted exp with a double denominator (softmax_reference,
 * src/qwen3_primitives.cpp:137-146), fp32 P.V in position order
 * (src/qwen3_layer.cpp:355-384).  q: fp32 [query_heads][d].  out (ungated) and
 * gated_out (out * sigmoid(gate)) may each be NULL. */
typedef struct {
    const kvo_view* view; const float* q; const float* gate; float* out; float* gated_out;
    uint32_t query_heads; float scale; uint64_t length;
} kvo_decode_ref_ctx;

static void kvo_decode_ref_head(size_t h, void* p) {
    const kvo_decode_ref_ctx* c = (const kvo_decode_ref_ctx*)p;
    const kvo_view* view = c->view;
    const uint32_t d = view->head_dim;
    const uint32_t kvh = (uint32_t)h / (c->query_heads / view->kv_heads);
    const uint64_t length = c->length;
    float* scores = (float*)malloc(sizeof(float) * (length ? length : 1));
    float* acc = (float*)calloc(d, sizeof(float));
    float maximum = -INFINITY;
    for (uint64_t pos = 0; pos < length; ++pos) {
        scores[pos] = kvo_qk(view, c->q + h * d, kvh, pos) * c->scale;
        if (scores[pos] > maximum) maximum = scores[pos];
    }
    double denominator = 0.0;
    for (uint64_t pos = 0; pos < length; ++pos) denominator += exp((double)(scores[pos] - maximum));
    for (uint64_t pos = 0; pos < length; ++pos) {
        float prob = (float)(exp((double)(scores[pos] - maximum)) / denominator);
        kvo_pv(view, acc, 1.0f, prob, kvh, pos);
    }
    for (uint32_t i = 0; i < d; ++i) {
        float o = length ? acc[i] : 0.0f;
        if (c->out) c->out[h * d + i] = o;
        if (c->gated_out) c->gated_out[h * d + i] = c->gate ? o * kvo_sigmoid(c->gate[h * d + i]) : o;
    }
    free(scores);
    free(acc);
}

KVO_API void kvo_decode_attn_ref(const kvo_view* view, const float* q, const float* gate, float* out,
                                 float* gated_out, uint32_t query_heads, float scale, uint64_t length) {
    kvo_decode_ref_ctx ctx = { view, q, gate, out, gated_out, query_heads, scale, length };
    kvo_parallel_for(query_heads, kvo_decode_ref_head, &ctx);
}

/* Split heuristic of the decode launcher: <=512 -> 4, <=2048 -> 8, <=8192 -> 16,
 * <=16384 -> 32, else 64 (attention_splits_for_length, .hip:2106-2109). */
KVO_API uint32_t kvo_attention_splits_for_length(uint64_t length) {
    return length <= 512 ? 4 : length <= 2048 ? 8 : length <= 8192 ? 16 : length <= 16384 ? 32 : 64;
}

/* Stage 1 of split-K decode in the kernel's own order: split s covers
 * [s*ceil(L/S), min((s+1)*ceil(L/S), L)); online softmax with the
 * "score > m" branch structure of .hip:7444-7452; an empty split leaves
 * (m, l, acc) = (-inf, 0, 0).  Partials: m,l [S][query_heads]; acc
 * [S][query_heads][d].  range_begin/range_end restrict the scan to a shard of
 * positions (sequence-sharded decode): the splits then divide that range. */
typedef struct {
    const kvo_view* view; const float* q; uint32_t query_heads; float scale;
    uint64_t range_begin, range_end; uint32_t num_splits; float* part_m; float* part_l; float* part_acc;
} kvo_partials_ctx;

static void kvo_partials_unit(size_t unit, void* p) {
    const kvo_partials_ctx* c = (const kvo_partials_ctx*)p;
    const kvo_view* view = c->view;
    const uint32_t d = view->head_dim, query_heads = c->query_heads;
    const uint32_t s = (uint32_t)(unit / query_heads), h = (uint32_t)(unit % query_heads);
    const uint32_t kvh = h / (query_heads / view->kv_heads);
    const uint64_t length = c->range_end > c->range_begin ? c->range_end - c->range_begin : 0;
    const uint64_t per = (length + c->num_splits - 1) / c->num_splits;
    uint64_t p0 = c->range_begin + (uint64_t)s * per;
    uint64_t p1 = p0 + per < c->range_end ? p0 + per : c->range_end;
    float m = -INFINITY, l = 0.0f;
    float* acc = c->part_acc + ((size_t)s * query_heads + h) * d;
    for (uint32_t i = 0; i < d; ++i) acc[i] = 0.0f;
    for (uint64_t pos = p0; pos < p1; ++pos) {
        float dot = kvo_qk(view, c->q + (size_t)h * d, kvh, pos) * c->scale;
        float alpha = 1.0f, weight;
        if (dot > m) {
            alpha = expf(m - dot);
            l = l * alpha + 1.0f;
            m = dot;
            weight = 1.0f;
        } else {
            weight = expf(dot - m);
            l += weight;
        }
        kvo_pv(view, acc, alpha, weight, kvh, pos);
    }
    c->part_m[(size_t)s * query_heads + h] = m;
    c->part_l[(size_t)s * query_heads + h] = l;
}

KVO_API void kvo_decode_partials(const kvo_view* view, const float* q, uint32_t query_heads, float scale,
                                 uint64_t range_begin, uint64_t range_end, uint32_t num_splits,
                                 float* part_m, float* part_l, float* part_acc) {
    kvo_partials_ctx ctx = { view, q, query_heads, scale, range_begin, range_end, num_splits, part_m, part_l, part_acc };
    kvo_parallel_for((size_t)num_splits * query_heads, kvo_partials_unit, &ctx);
}

/* Stage 2 / log-sum-exp combine over `num_parts` partials laid out
 * [part][query_heads]([d]).  M = max m; alpha = expf(m - M) (0 for an empty
 * part); out = (sum acc*alpha) / (sum l*alpha), 0 if the sum is not positive;
 * gate applied as out * sigmoid(g).  Follows qwen3_splitk_stage2_kernel,
 * .hip:2295-2352, with the empty-part skip of the suffix combine
 * (.hip:6681,6701).  This is also the cross-GPU merge. */
KVO_API void kvo_merge_partials(const float* part_m, const float* part_l, const float* part_acc,
                                uint32_t num_parts, uint32_t query_heads, uint32_t head_dim,
                                const float* gate, float* out, float* gated_out) {
    for (uint32_t h = 0; h < query_heads; ++h) {
        float gmax = -INFINITY;
        for (uint32_t s = 0; s < num_parts; ++s) gmax = fmaxf(gmax, part_m[(size_t)s * query_heads + h]);
        float gsum = 0.0f;
        for (uint32_t s = 0; s < num_parts; ++s) {
            float m = part_m[(size_t)s * query_heads + h], l = part_l[(size_t)s * query_heads + h];
            if (l > 0.0f && isfinite(m)) gsum += l * expf(m - gmax);
        }
        for (uint32_t i = 0; i < head_dim; ++i) {
            float total = 0.0f;
            for (uint32_t s = 0; s < num_parts; ++s) {
                float m = part_m[(size_t)s * query_heads + h], l = part_l[(size_t)s * query_heads + h];
                if (l > 0.0f && isfinite(m))
                    total += part_acc[((size_t)s * query_heads + h) * head_dim + i] * expf(m - gmax);
            }
            float o = gsum > 0.0f ? total / gsum : 0.0f;
            if (out) out[(size_t)h * head_dim + i] = o;
            if (gated_out) gated_out[(size_t)h * head_dim + i] = gate ? o * kvo_sigmoid(gate[(size_t)h * head_dim + i]) : o;
        }
    }
}

/* Re-quantisation of a decode output row to Q8_1 blocks of 32 for the projection that follows, as the
 * reference's stage 2 does it (qwen3_splitk_stage2_kernel, .hip:2354-2383): scale = amax / 127,
 * q = roundf(x * (1 / scale)) clamped to [-127, 127] (half away from zero, unlike the cache quantizer),
 * d = fp16(scale), s = fp16((float)sum(q) * scale).  Block layout: Q8_1Block,
 * include/miinfer/q4_q8_gemv.hpp:23-27 (fp16 d, fp16 s, 32 int8 = 36 bytes).  x: fp32 [count], count % 32 == 0. */
KVO_API void kvo_quantize_q8_1(const float* x, size_t count, uint8_t* blocks) {
    for (size_t b = 0; b < count / 32; ++b) {
        const float* v = x + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
        const float scale = amax / 127.0f;
        const float inv = scale != 0.0f ? 1.0f / scale : 0.0f;
        int sum = 0;
        int8_t* qs = (int8_t*)(blocks + b * 36 + 4);
        for (int i = 0; i < 32; ++i) {
            int q = (int)roundf(v[i] * inv);
            q = q < -127 ? -127 : (q > 127 ? 127 : q);
            qs[i] = (int8_t)q;
            sum += q;
        }
        const uint16_t d = kvo_float_to_half_rn(scale), sh = kvo_float_to_half_rn((float)sum * scale);
        memcpy(blocks + b * 36, &d, 2);
        memcpy(blocks + b * 36 + 2, &sh, 2);
    }
}

/* Query side of an attention layer: de-interleave the projection output [token][heads][q (d) | gate (d)],
 * RMSNorm * weight on q (same binary-tree sum of squares as the store kernel), RoPE at base_position + token,
 * write q and gate as [token][heads][d].  Follows qwen35_decoupled_q_split_norm_rope_batch_kernel
 * (.hip:994-1045) and its single-token twin qwen35_fused_q_split_norm_rope_kernel (.hip:661-717); the norm, the
 * RoPE and the deviations (1/sqrtf, pinned trig) are exactly those of kvo_append, so Q and K are rotated by
 * identical bits.  q_norm_weight may be NULL (no norm), rope_mode as kvo_append. */
KVO_API void kvo_q_split_norm_rope(const float* qfull, const float* q_norm_weight, float* query_rope, float* gate,
                                   uint32_t token_count, uint32_t base_position, uint32_t heads, uint32_t head_dim,
                                   int rope_mode, float theta, float epsilon, int trig_mode) {
    const uint32_t d = head_dim;
    float* scratch = (float*)malloc(sizeof(float) * d);
    for (uint32_t t = 0; t < token_count; ++t)
        for (uint32_t h = 0; h < heads; ++h) {
            const float* src = qfull + ((size_t)t * heads + h) * 2 * d;
            float* row = query_rope + ((size_t)t * heads + h) * d;
            if (gate) memcpy(gate + ((size_t)t * heads + h) * d, src + d, sizeof(float) * d);
            if (q_norm_weight) {
                float ss = kvo_tree_sum_squares(src, d, scratch);
                float r = 1.0f / sqrtf(ss / (float)d + epsilon);
                for (uint32_t i = 0; i < d; ++i) row[i] = src[i] * r * q_norm_weight[i];
            } else {
                memcpy(row, src, sizeof(float) * d);
            }
            kvo_rope_row(row, d, base_position + t, theta, rope_mode, trig_mode);
        }
    free(scratch);
}

/* Device-side step bookkeeping of a replayed decode graph: qwen35_decode_state_advance_kernel, .hip:4417-4428.
 * state: the 16 words of a DeviceDecodeState {current_token, position, generated, stop, max_generated, ...}. */
KVO_API void kvo_decode_state_advance(uint32_t* state, uint32_t* token_output, uint32_t capacity) {
    const uint32_t generated = state[2];
    if (generated < capacity) token_output[generated] = state[0];
    state[3] = (state[3] || state[0] == 151643u || state[0] == 151645u || generated + 1 >= state[4]) ? 1u : 0u;
    state[1] += 1;
    state[2] = generated + 1;
}

/* Split-K decode end to end in kernel order (stage 1 + stage 2). */
KVO_API void kvo_decode_attn_splitk(const kvo_view* view, const float* q, const float* gate, float* out,
                                    float* gated_out, uint32_t query_heads, float scale, uint64_t length,
                                    uint32_t num_splits) {
    if (num_splits == 0) num_splits = kvo_attention_splits_for_length(length);
    const uint32_t d = view->head_dim;
    float* m = (float*)malloc(sizeof(float) * num_splits * query_heads * (2 + (size_t)d));
    float* l = m + (size_t)num_splits * query_heads;
    float* acc = l + (size_t)num_splits * query_heads;
    kvo_decode_partials(view, q, query_heads, scale, 0, length, num_splits, m, l, acc);
    kvo_merge_partials(m, l, acc, num_splits, query_heads, d, gate, out, gated_out);
    free(m);
}

/* Suffix / prefill cross-query attention, tolerance-target flavour: query token
 * t attends cache positions [0, base_position + t + 1) (the chunk has already
 * been appended; causal inside the chunk, full over the prefix), two-pass
 * softmax as kvo_decode_attn_ref.  q, gate, out: fp32 [token][query_heads][d].
 * Causal length follows .hip:6829; gating follows .hip:6714-6723. */
typedef struct {
    const kvo_view* view; const float* q; const float* gate; float* gated_out;
    uint32_t token_count, base_position, query_heads; float scale; uint32_t num_splits;
} kvo_suffix_ctx;

static void kvo_suffix_ref_unit(size_t unit, void* p) {
    const kvo_suffix_ctx* c = (const kvo_suffix_ctx*)p;
    const kvo_view* view = c->view;
    const uint32_t d = view->head_dim, query_heads = c->query_heads;
    const uint32_t t = (uint32_t)(unit / query_heads), h = (uint32_t)(unit % query_heads);
    const uint64_t length = (uint64_t)c->base_position + t + 1;
    float* dst = c->gated_out + ((size_t)t * query_heads + h) * d;
    if (length > view->capacity) { for (uint32_t i = 0; i < d; ++i) dst[i] = 0.0f; return; }
    const uint32_t kvh = h / (query_heads / view->kv_heads);
    const float* qrow = c->q + ((size_t)t * query_heads + h) * d;
    float* scores = (float*)malloc(sizeof(float) * length);
    float* acc = (float*)calloc(d, sizeof(float));
    float maximum = -INFINITY;
    for (uint64_t pos = 0; pos < length; ++pos) {
        scores[pos] = kvo_qk(view, qrow, kvh, pos) * c->scale;
        if (scores[pos] > maximum) maximum = scores[pos];
    }
    double denominator = 0.0;
    for (uint64_t pos = 0; pos < length; ++pos) denominator += exp((double)(scores[pos] - maximum));
    for (uint64_t pos = 0; pos < length; ++pos)
        kvo_pv(view, acc, 1.0f, (float)(exp((double)(scores[pos] - maximum)) / denominator), kvh, pos);
    for (uint32_t i = 0; i < d; ++i) {
        float o = acc[i];
        if (c->gate) o *= kvo_sigmoid(c->gate[((size_t)t * query_heads + h) * d + i]);
        dst[i] = o;
    }
    free(scores);
    free(acc);
}

KVO_API void kvo_suffix_attn_ref(const kvo_view* view, const float* q, const float* gate, float* gated_out,
                                 uint32_t token_count, uint32_t base_position, uint32_t query_heads, float scale) {
    kvo_suffix_ctx ctx = { view, q, gate, gated_out, token_count, base_position, query_heads, scale, 0 };
    kvo_parallel_for((size_t)token_count * query_heads, kvo_suffix_ref_unit, &ctx);
}

/* Suffix attention in kernel order: per (token, head) `num_splits` splits of
 * the causal range, online softmax per split, stage-2 combine that skips empty
 * splits and multiplies by sigmoid(gate) before 1/sum (.hip:6819-6848,
 * 6637-6725). */
static void kvo_suffix_splitk_unit(size_t unit, void* p) {
    const kvo_suffix_ctx* c = (const kvo_suffix_ctx*)p;
    const kvo_view* view = c->view;
    const uint32_t d = view->head_dim, query_heads = c->query_heads, num_splits = c->num_splits;
    const uint32_t t = (uint32_t)(unit / query_heads), h = (uint32_t)(unit % query_heads);
    const uint64_t length = (uint64_t)c->base_position + t + 1;
    float* dst = c->gated_out + ((size_t)t * query_heads + h) * d;
    if (length > view->capacity) return;
    const uint32_t kvh = h / (query_heads / view->kv_heads);
    const float* qrow = c->q + ((size_t)t * query_heads + h) * d;
    const uint64_t chunk = (length + num_splits - 1) / num_splits;
    float pm[64], pl[64];
    float* pacc = (float*)calloc((size_t)num_splits * d, sizeof(float));
    for (uint32_t s = 0; s < num_splits; ++s) {
        uint64_t p0 = (uint64_t)s * chunk, p1 = p0 + chunk < length ? p0 + chunk : length;
        float m = -INFINITY, l = 0.0f;
        for (uint64_t pos = p0; pos < p1; ++pos) {
            float dot = kvo_qk(view, qrow, kvh, pos) * c->scale;
            float alpha = 1.0f, weight;
            if (dot > m) { alpha = expf(m - dot); l = l * alpha + 1.0f; m = dot; weight = 1.0f; }
            else { weight = expf(dot - m); l += weight; }
            kvo_pv(view, pacc + (size_t)s * d, alpha, weight, kvh, pos);
        }
        pm[s] = m; pl[s] = l;
    }
    float gmax = -INFINITY, gsum = 0.0f;
    for (uint32_t s = 0; s < num_splits; ++s) if (pm[s] > gmax) gmax = pm[s];
    for (uint32_t s = 0; s < num_splits; ++s)
        if (pl[s] > 0.0f && isfinite(pm[s])) gsum += pl[s] * expf(pm[s] - gmax);
    float inv = gsum > 0.0f ? 1.0f / gsum : 0.0f;
    for (uint32_t i = 0; i < d; ++i) {
        float total = 0.0f;
        for (uint32_t s = 0; s < num_splits; ++s)
            if (pl[s] > 0.0f && isfinite(pm[s])) total += pacc[(size_t)s * d + i] * expf(pm[s] - gmax);
        if (c->gate) total *= kvo_sigmoid(c->gate[((size_t)t * query_heads + h) * d + i]);
        dst[i] = total * inv;
    }
    free(pacc);
}

KVO_API void kvo_suffix_attn_splitk(const kvo_view* view, const float* q, const float* gate, float* gated_out,
                                    uint32_t token_count, uint32_t base_position, uint32_t query_heads,
                                    float scale, uint32_t num_splits) {
    if (num_splits == 0 || num_splits > 64) num_splits = 64;
    kvo_suffix_ctx ctx = { view, q, gate, gated_out, token_count, base_position, query_heads, scale, num_splits };
    kvo_parallel_for((size_t)token_count * query_heads, kvo_suffix_splitk_unit, &ctx);
}

/* ------------------------------------------------------------------------- */
/* Snapshot raw layout                                                        */
/* ------------------------------------------------------------------------- */

static size_t kvo_side_bytes(const kvo_view* v, int q8, uint64_t tokens) {
    const size_t d = v->head_dim, nblk = d / v->qblock;
    return q8 ? (size_t)tokens * v->kv_heads * (d + 2 * nblk) : (size_t)tokens * v->kv_heads * d * 2;
}

/* raw_tokens_bytes, src/prefill_v2/kv_cache.cpp:214-225 (scale bytes per row
 * generalised from 2 to 2*d/qblock). */
KVO_API size_t kvo_raw_tokens_bytes(const kvo_view* v, uint64_t tokens) {
    return kvo_side_bytes(v, kvo_k_q8(v), tokens) + kvo_side_bytes(v, kvo_v_q8(v), tokens);
}

static size_t kvo_copy_side(const kvo_view* v, int q8, uint16_t* f16, int8_t* q, uint16_t* sc, uint64_t tokens,
                            uint8_t* blob, int to_blob) {
    const size_t d = v->head_dim, nblk = d / v->qblock;
    size_t off = 0;
    for (uint32_t h = 0; h < v->kv_heads; ++h) {
        if (q8) {
            int8_t* qp = q + (size_t)h * v->capacity * d;
            uint16_t* sp = sc + (size_t)h * v->capacity * nblk;
            if (to_blob) memcpy(blob + off, qp, tokens * d); else memcpy(qp, blob + off, tokens * d);
            off += tokens * d;
            if (to_blob) memcpy(blob + off, sp, tokens * nblk * 2); else memcpy(sp, blob + off, tokens * nblk * 2);
            off += tokens * nblk * 2;
        } else {
            uint16_t* fp = f16 + (size_t)h * v->capacity * d;
            if (to_blob) memcpy(blob + off, fp, tokens * d * 2); else memcpy(fp, blob + off, tokens * d * 2);
            off += tokens * d * 2;
        }
    }
    return off;
}

/* download_raw / upload_raw, src/prefill_v2/kv_cache.cpp:227-369: K first (per
 * head: int8 slice of `tokens` rows, then its scale slice; or the fp16 slice),
 * then V the same way; capacity-strided rows compacted to `tokens`. */
KVO_API int kvo_download_raw(const kvo_view* v, uint64_t tokens, uint8_t* blob) {
    if (tokens > v->capacity) return -1;
    size_t off = kvo_copy_side(v, kvo_k_q8(v), v->key_f16, v->key_q8, v->key_scales, tokens, blob, 1);
    kvo_copy_side(v, kvo_v_q8(v), v->value_f16, v->value_q8, v->value_scales, tokens, blob + off, 1);
    return 0;
}
KVO_API int kvo_upload_raw(const kvo_view* v, uint64_t tokens, const uint8_t* blob) {
    if (tokens > v->capacity) return -1;
    size_t off = kvo_copy_side(v, kvo_k_q8(v), v->key_f16, v->key_q8, v->key_scales, tokens, (uint8_t*)blob, 0);
    kvo_copy_side(v, kvo_v_q8(v), v->value_f16, v->value_q8, v->value_scales, tokens, (uint8_t*)blob + off, 0);
    return 0;
}

/* FNV-1a-style 64-bit hash with one round per TOKEN (the whole u32 is xored in,
 * then one multiply by the FNV prime) -- compute_token_sequence_hash,
 * include/miinfer/prefill_v2/reusable_context.hpp:38-45. */
KVO_API uint64_t kvo_token_sequence_hash(const uint32_t* tokens, size_t count) {
    uint64_t hash = 0xcbf29ce484222325ull;
    for (size_t i = 0; i < count; ++i) {
        hash ^= (uint64_t)tokens[i];
        hash *= 0x100000001b3ull;
    }
    return hash;
}
