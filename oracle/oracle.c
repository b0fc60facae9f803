/*
 * CPU oracle for the paged-KV full-attention path (TEST INFRASTRUCTURE, not product code).
 *
 * A plain-C restatement of what the reference engine computes on this path, used only as the checker by the
 * tests, by the smoke check and by the benchmark's CPU-baseline leg.  The shipped library never links, loads or
 * calls anything in this file.
 *
 * Every function names the reference source it follows (paths relative to the reference project root).
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (no fast-math: the quantisers must round exactly like
 * the reference's fp32 code).
 *
 * What is bit-exact here and what is not:
 *   - f16 conversion, q8_0 and q4_0 quantisers, row sizes, paged addressing, kv_append: bit-exact restatements.
 *   - attention: evaluated in fp64 (the reference's independent test kernel does the same sum in fp32); it is the
 *     accuracy yardstick, compared with a tolerance.
 *   - rmsnorm / RoPE / sigmoid use the host libm (rsqrt, powf, cosf, sinf, expf differ from the device libm in
 *     the last ulp), so attn_prep outputs are compared with a tolerance here; byte equality of attn_prep is
 *     checked on the GPU against the reference's own kernels.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_KV_F16 1u  /* src/fast/attn.cuh:14 */
#define ORC_KV_Q4_0 2u /* src/fast/attn.cuh:15 */
#define ORC_KV_Q8_0 8u /* src/fast/attn.cuh:16 */

/* Field-for-field the reference's cache view, src/fast/attn.cuh:18-32. */
typedef struct {
    uint32_t type;
    int32_t n_ctx, Hkv, D;
    void *k, *v;
    const int32_t *pt;   /* page table(s); NULL = contiguous */
    const int32_t *rtab; /* per-row offsets into pt; NULL = 0 */
    int32_t psh;
    size_t pstride;
} orc_kv;

/* ---- IEEE binary16 <-> binary32, round to nearest even (what __float2half / __half2float do,
 *      used at src/fast/attn.cu:252-253 and src/fast/kv_q8.cuh:25,48) ---- */
uint16_t orc_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) return (uint16_t) (sign | (ax > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (ax >= 0x477ff000u) return (uint16_t) (sign | 0x7c00u); /* rounds to >= 65520 -> inf */
    if (ax < 0x33000001u) return (uint16_t) sign;               /* <= 2^-25 -> 0 (tie to even) */
    int e = (int) (ax >> 23) - 127;
    uint32_t m = (ax & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { /* subnormal half */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t) (e + 15) << 10;
        m &= 0x7fffffu;
    }
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q; /* may carry into the exponent: still correct */
    return (uint16_t) (sign | (base + q));
}

float orc_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t) (h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 31u, m = h & 0x3ffu, x;
    if (e == 31u) x = sign | 0x7f800000u | (m << 13);
    else if (e) x = sign | ((e + 112u) << 23) | (m << 13);
    else if (!m) x = sign;
    else {
        int k = 0;
        while (!(m & 0x400u)) { m <<= 1; ++k; }
        x = sign | ((uint32_t) (113 - k) << 23) | ((m & 0x3ffu) << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* bytes of one position (all kv heads) of K or V: src/fast/attn.cu:501-503 */
size_t orc_kv_row_bytes(uint32_t type, int Hkv, int D) {
    return type == ORC_KV_F16 ? (size_t) Hkv * D * 2 : type == ORC_KV_Q8_0 ? (size_t) Hkv * (D / 32) * 34 : (size_t) Hkv * (D / 32) * 18;
}
static size_t head_bytes(uint32_t type, int D) { return orc_kv_row_bytes(type, 1, D); }

/* byte offset of position p of query row t: src/fast/kv_page.cuh:20-31 */
size_t orc_kv_off(const orc_kv *c, int t, int p) {
    const size_t rowb = orc_kv_row_bytes(c->type, c->Hkv, c->D);
    if (!c->pt) return (size_t) p * rowb;
    const int32_t *tab = c->rtab ? c->pt + c->rtab[t] : c->pt;
    return (size_t) tab[p >> c->psh] * c->pstride + (size_t) (p & ((1 << c->psh) - 1)) * rowb;
}

/* q8_0 head row: the D/32 f16 scales first, then the D int8 quants (src/fast/kv_q8.cuh:1-5,20-26);
 * arithmetic of ggml's quantize_row_q8_0_ref (third_party/llama.cpp-fork/ggml/src/ggml-quants.c:276-299). */
void orc_quant_q8_0_head(const float *x, uint8_t *head, int D) {
    const int nb = D / 32;
    for (int b = 0; b < nb; ++b) {
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[b * 32 + i]));
        const float d = amax / 127.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        for (int i = 0; i < 32; ++i) ((int8_t *) (head + nb * 2))[b * 32 + i] = (int8_t) (int) roundf(x[b * 32 + i] * id);
        const uint16_t hd = orc_f32_to_f16(d);
        memcpy(head + 2 * b, &hd, 2);
    }
}

/* q4_0 head row = D/32 ggml block_q4_0 (src/fast/kv_q8.cuh:28-49; ggml-quants.c:113-148): the element of largest
 * magnitude, first one on ties, sets d = max / -8; q = min(15, (int)(x*id + 8.5f)), product rounded before the add. */
void orc_quant_q4_0_head(const float *x, uint8_t *head, int D) {
    const int nb = D / 32;
    for (int b = 0; b < nb; ++b) {
        const float *xb = x + b * 32;
        uint8_t *blk = head + b * 18;
        float amax = 0.0f, mx = 0.0f;
        for (int i = 0; i < 32; ++i)
            if (amax < fabsf(xb[i])) { amax = fabsf(xb[i]); mx = xb[i]; }
        const float d = mx / -8.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        const uint16_t hd = orc_f32_to_f16(d);
        memcpy(blk, &hd, 2);
        for (int i = 0; i < 16; ++i) {
            volatile float p0 = xb[i] * id, p1 = xb[i + 16] * id; /* volatile: the product is rounded on its own */
            int q0 = (int) (p0 + 8.5f), q1 = (int) (p1 + 8.5f);
            if (q0 > 15) q0 = 15;
            if (q1 > 15) q1 = 15;
            blk[2 + i] = (uint8_t) ((q0 & 0xff) | (q1 << 4));
        }
    }
}

void orc_f16_head(const float *x, uint8_t *head, int D) {
    for (int i = 0; i < D; ++i) {
        const uint16_t h = orc_f32_to_f16(x[i]);
        memcpy(head + 2 * i, &h, 2);
    }
}

static void quant_head(uint32_t type, const float *x, uint8_t *head, int D) {
    if (type == ORC_KV_F16) orc_f16_head(x, head, D);
    else if (type == ORC_KV_Q8_0) orc_quant_q8_0_head(x, head, D);
    else orc_quant_q4_0_head(x, head, D);
}

/* one cache element as float: tests/fast_attn_test.cu:34-46 */
float orc_kv_read(const uint8_t *head, uint32_t type, int D, int d) {
    uint16_t h;
    if (type == ORC_KV_F16) {
        memcpy(&h, head + 2 * d, 2);
        return orc_f16_to_f32(h);
    }
    if (type == ORC_KV_Q8_0) {
        memcpy(&h, head + 2 * (d >> 5), 2);
        return orc_f16_to_f32(h) * (float) ((const int8_t *) (head + (D / 32) * 2))[d];
    }
    const uint8_t *b = head + (d >> 5) * 18;
    memcpy(&h, b, 2);
    const int i = d & 31;
    const uint8_t by = b[2 + (i & 15)];
    return (float) ((int) (i < 16 ? (by & 15) : (by >> 4)) - 8) * orc_f16_to_f32(h);
}

/* dequantise one head row to D floats */
void orc_dequant_head(const uint8_t *head, uint32_t type, int D, float *out) {
    for (int d = 0; d < D; ++d) out[d] = orc_kv_read(head, type, D, d);
}

/* k, v [T][Hkv][D] f32 -> cache rows.  pos == NULL: row t goes to position p0 + t (kv_append, src/fast/attn.cu:583);
 * pos != NULL: to pos[t] (the device-position form used by attn_prep, src/fast/fused.cu:512).  ldk / ldv: row
 * strides in floats. */
void orc_kv_append(const orc_kv *c, const float *k, const float *v, int p0, const int32_t *pos, int T, int ldk, int ldv) {
    const size_t hb = head_bytes(c->type, c->D);
    if (ldk <= 0) ldk = c->Hkv * c->D;
    if (ldv <= 0) ldv = c->Hkv * c->D;
    for (int t = 0; t < T; ++t) {
        const size_t o = orc_kv_off(c, t, pos ? pos[t] : p0 + t);
        for (int h = 0; h < c->Hkv; ++h) {
            quant_head(c->type, k + (size_t) t * ldk + (size_t) h * c->D, (uint8_t *) c->k + o + h * hb, c->D);
            quant_head(c->type, v + (size_t) t * ldv + (size_t) h * c->D, (uint8_t *) c->v + o + h * hb, c->D);
        }
    }
}

/* RMSNorm of one head followed by NEOX partial RoPE, in place on x[D].
 * Norm: src/fast/fused.cu:531-546 (64 threads, one float4 each, xor-butterfly then cross-warp sum).
 * RoPE: src/kernels.cu:108-119 == src/fast/fused.cu:548-558. */
static void norm_rope_head(float *x, const float *w, int D, int pos, int n_rot, float freq_base, float eps) {
    /* sum of squares in the reference's order: per float4 a.x*a.x + a.y*a.y + a.z*a.z + a.w*a.w (contracted into a
     * multiply and three fused multiply-adds), lanes combined by an xor butterfly inside each warp of 32, then the
     * warp sums combined the same way */
    const int D4 = D / 4;
    int nthr = (D4 + 31) & ~31;
    float part[1024 / 4];
    for (int i = 0; i < nthr; ++i) {
        float s = 0.0f;
        if (i < D4) {
            const float *a = x + 4 * i;
            float t = a[0] * a[0];
            t = fmaf(a[1], a[1], t);
            t = fmaf(a[2], a[2], t);
            t = fmaf(a[3], a[3], t);
            s += t;
        }
        part[i] = s;
    }
    const int nw = nthr / 32;
    float wsum[32];
    for (int w = 0; w < 32; ++w) wsum[w] = 0.0f;
    for (int w = 0; w < nw; ++w) {
        float v[32];
        for (int l = 0; l < 32; ++l) v[l] = part[w * 32 + l];
        for (int o = 16; o > 0; o >>= 1) {
            float n[32];
            for (int l = 0; l < 32; ++l) n[l] = v[l] + v[l ^ o];
            memcpy(v, n, sizeof v);
        }
        wsum[w] = v[0];
    }
    float ss;
    if (nw == 1) ss = wsum[0];
    else {
        float v[32];
        for (int l = 0; l < 32; ++l) v[l] = l < nw ? wsum[l] : 0.0f;
        for (int o = 16; o > 0; o >>= 1) {
            float n[32];
            for (int l = 0; l < 32; ++l) n[l] = v[l] + v[l ^ o];
            memcpy(v, n, sizeof v);
        }
        ss = v[0];
    }
    const float sc = 1.0f / sqrtf(ss / (float) D + eps);
    for (int i = 0; i < D; ++i) {
        float o = x[i] * sc;
        if (w) o *= w[i];
        x[i] = o;
    }
    const int half = n_rot / 2;
    for (int j = 0; j < half; ++j) {
        const float theta = (float) pos * powf(freq_base, -2.0f * j / n_rot);
        const float c = cosf(theta), sn = sinf(theta);
        const float x0 = x[j], x1 = x[j + half];
        x[j] = x0 * c - x1 * sn;
        x[j + half] = x0 * sn + x1 * c;
    }
}

/* Attention-layer input prep, src/fast/fused.cu:502-573,677-721 (== k::split_q_gate + rmsnorm + k::rope_neox +
 * kv_append, src/model.cu:186-196): qg [T][Hq][2D] -> q [T][Hq][D], gate [T][Hq*D]; k -> norm+rope -> K cache row;
 * v -> V cache row.  p0 < 0: the cache row of token t is pos[t]; the rotary angle always uses pos[t].
 * kpre (optional, [T][Hkv][D]): the K values right before quantisation, for tolerance checks. */
void orc_attn_prep(const float *qg, const float *k, const float *v, const float *q_norm, const float *k_norm,
                   const int32_t *pos, float *q, float *gate, const orc_kv *c, int p0, int T, int Hq, int Hkv, int D,
                   int n_rot, float freq_base, float eps, int ldq, int ldk, int ldv, float *kpre) {
    if (ldq <= 0) ldq = Hq * 2 * D;
    if (ldk <= 0) ldk = Hkv * D;
    if (ldv <= 0) ldv = Hkv * D;
    const size_t hb = head_bytes(c->type, D);
    float *tmp = (float *) malloc(sizeof(float) * (size_t) D);
    for (int t = 0; t < T; ++t) {
        const int row = p0 < 0 ? pos[t] : p0 + t;
        const size_t o = orc_kv_off(c, t, row);
        for (int h = 0; h < Hq; ++h) {
            const float *src = qg + (size_t) t * ldq + (size_t) h * 2 * D;
            memcpy(gate + ((size_t) t * Hq + h) * D, src + D, sizeof(float) * (size_t) D);
            memcpy(tmp, src, sizeof(float) * (size_t) D);
            norm_rope_head(tmp, q_norm, D, pos[t], n_rot, freq_base, eps);
            memcpy(q + ((size_t) t * Hq + h) * D, tmp, sizeof(float) * (size_t) D);
        }
        for (int h = 0; h < Hkv; ++h) {
            memcpy(tmp, k + (size_t) t * ldk + (size_t) h * D, sizeof(float) * (size_t) D);
            norm_rope_head(tmp, k_norm, D, pos[t], n_rot, freq_base, eps);
            if (kpre) memcpy(kpre + ((size_t) t * Hkv + h) * D, tmp, sizeof(float) * (size_t) D);
            quant_head(c->type, tmp, (uint8_t *) c->k + o + h * hb, D);
            quant_head(c->type, v + (size_t) t * ldv + (size_t) h * D, (uint8_t *) c->v + o + h * hb, D);
        }
    }
    free(tmp);
}

/* NEOX partial RoPE alone on x [T][H][D] (src/kernels.cu:108-123), for the prefill per-op path. */
void orc_rope_neox(float *x, const int32_t *pos, int T, int H, int D, int n_rot, float freq_base) {
    const int half = n_rot / 2;
    for (int t = 0; t < T; ++t)
        for (int h = 0; h < H; ++h) {
            float *xr = x + ((size_t) t * H + h) * D;
            for (int j = 0; j < half; ++j) {
                const float theta = (float) pos[t] * powf(freq_base, -2.0f * j / n_rot);
                const float c = cosf(theta), sn = sinf(theta);
                const float a = xr[j], b = xr[j + half];
                xr[j] = a * c - b * sn;
                xr[j + half] = a * sn + b * c;
            }
        }
}

/* Causal GQA attention of T query rows over the (paged, quantised) cache, evaluated in fp64.
 * Semantics: src/fast/attn.cuh:37-39,61-66 and tests/fast_attn_test.cu:51-67 — row t sits at position
 * P_t = pos ? pos[t] : p0 + t of its own sequence (page table pt + rtab[t]) and sees keys [0, P_t]; q is multiplied
 * by scale (fp32) before the dot product; q head h reads kv head h / (Hq / Hkv).
 * Key window [k_lo, k_hi): only keys in the window are used (k_hi <= 0 means no upper limit) — the unit of a
 * sequence-sharded partial.  Outputs (any may be NULL):
 *   out  [T][Hq][D]  normalised result acc / l (rows with no visible key in the window: zeros)
 *   oacc [T][Hq][D]  unnormalised sum of exp(s - m) * v,  om / ol [T][Hq]  its max m (-inf if empty) and sum l
 * gate [T][Hq*D] != NULL: out is multiplied by the sigmoid of the gate logits (src/kernels.cu:85-88). */
void orc_attention(const float *q, const orc_kv *c, float *out, int T, int p0, const int32_t *pos, int Hq, float scale,
                   const float *gate, int k_lo, int k_hi, float *oacc, float *om, float *ol) {
    const int D = c->D, G = Hq / c->Hkv;
    const size_t hb = head_bytes(c->type, D);
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int t = 0; t < T; ++t)
        for (int h = 0; h < Hq; ++h) {
            const int hk = h / G;
            const int n = (pos ? pos[t] : p0 + t) + 1;
            const int hi = (k_hi > 0 && k_hi < n) ? k_hi : n;
            double *acc = (double *) calloc((size_t) D, sizeof(double));
            float *qs = (float *) malloc(sizeof(float) * (size_t) D);
            float *row = (float *) malloc(sizeof(float) * (size_t) D);
            for (int d = 0; d < D; ++d) qs[d] = q[((size_t) t * Hq + h) * D + d] * scale;
            double m = -INFINITY, l = 0.0;
            for (int j = k_lo; j < hi; ++j) {
                const size_t o = orc_kv_off(c, t, j) + hk * hb;
                orc_dequant_head((const uint8_t *) c->k + o, c->type, D, row);
                double s = 0.0;
                for (int d = 0; d < D; ++d) s += (double) qs[d] * (double) row[d];
                const double nm = s > m ? s : m;
                const double f = exp(m - nm), p = exp(s - nm);
                orc_dequant_head((const uint8_t *) c->v + o, c->type, D, row);
                l = l * f + p;
                for (int d = 0; d < D; ++d) acc[d] = acc[d] * f + p * (double) row[d];
                m = nm;
            }
            const size_t ro = ((size_t) t * Hq + h) * D;
            if (oacc) for (int d = 0; d < D; ++d) oacc[ro + d] = (float) acc[d];
            if (om) om[(size_t) t * Hq + h] = (float) m;
            if (ol) ol[(size_t) t * Hq + h] = (float) l;
            if (out) for (int d = 0; d < D; ++d) {
                float y = l > 0.0 ? (float) (acc[d] / l) : 0.0f;
                if (gate) y = y * (1.0f / (1.0f + expf(-gate[ro + d])));
                out[ro + d] = y;
            }
            free(acc);
            free(qs);
            free(row);
        }
}

/* Merge of nparts partial results in part order, the reference's split combine (src/fast/attn_dec2.cu:430-450):
 * M = max_s m_s; out = sum_s e^{m_s - M} A_s / sum_s e^{m_s - M} l_s, parts with m_s = -inf skipped.
 * oacc [nparts][R][D], om / ol [nparts][R], out [R][D]; optional sigmoid gate [R][D]. */
void orc_merge(const float *oacc, const float *om, const float *ol, int nparts, int R, int D, const float *gate, float *out) {
    for (int r = 0; r < R; ++r) {
        double M = -INFINITY;
        for (int s = 0; s < nparts; ++s) if ((double) om[(size_t) s * R + r] > M) M = om[(size_t) s * R + r];
        double den = 0.0;
        for (int s = 0; s < nparts; ++s) {
            const float ms = om[(size_t) s * R + r];
            if (ms == -INFINITY) continue;
            den += exp((double) ms - M) * (double) ol[(size_t) s * R + r];
        }
        for (int d = 0; d < D; ++d) {
            double num = 0.0;
            for (int s = 0; s < nparts; ++s) {
                const float ms = om[(size_t) s * R + r];
                if (ms == -INFINITY) continue;
                num += exp((double) ms - M) * (double) oacc[((size_t) s * R + r) * D + d];
            }
            float y = den > 0.0 ? (float) (num / den) : 0.0f;
            if (gate) y = y * (1.0f / (1.0f + expf(-gate[(size_t) r * D + d])));
            out[(size_t) r * D + d] = y;
        }
    }
}

/* x *= sigmoid(g): src/kernels.cu:85-88, src/fast/fused.cu:248,262-273 */
void orc_sigmoid_mul(float *x, const float *g, int64_t n) {
    for (int64_t i = 0; i < n; ++i) x[i] = x[i] * (1.0f / (1.0f + expf(-g[i])));
}

/* Re-pack one q8_0 head row (scales first, then quants) into ggml's interleaved block_q8_0 x D/32
 * ({f16 d; int8 qs[32]}, ggml-common.h) and back: same values, different byte order (src/fast/kv_q8.cuh:1-5). */
void orc_q8_head_to_ggml(const uint8_t *head, uint8_t *blocks, int D) {
    const int nb = D / 32;
    for (int b = 0; b < nb; ++b) {
        memcpy(blocks + b * 34, head + 2 * b, 2);
        memcpy(blocks + b * 34 + 2, head + nb * 2 + b * 32, 32);
    }
}
void orc_q8_ggml_to_head(const uint8_t *blocks, uint8_t *head, int D) {
    const int nb = D / 32;
    for (int b = 0; b < nb; ++b) {
        memcpy(head + 2 * b, blocks + b * 34, 2);
        memcpy(head + nb * 2 + b * 32, blocks + b * 34 + 2, 32);
    }
}
