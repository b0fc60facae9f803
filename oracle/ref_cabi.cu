// extern "C" doorway to the REFERENCE engine's own attention kernels (TEST INFRASTRUCTURE, not product code).
//
// Compiled together with the reference's unmodified sources (src/fast/{attn,attn_dec2,attn_fold,fused}.cu and
// src/kernels.cu, taken where they lie in the reference checkout) into oracle/_ref/libp100e_ref.so by oracle/Makefile.
// Only the tests load it, to compare this repository's kernels with the reference's on identical inputs.
#include "fast/attn.cuh"
#include "fast/attn_dec2.cuh"
#include "fast/attn_fold.cuh"
#include "fast/fused.cuh"
#include "kernels.cuh"

namespace F = p100e::fast;
namespace K = p100e::k;

extern "C" {

struct ref_kv {   // same fields as p100e::fast::kv_cache (src/fast/attn.cuh:18-32)
    uint32_t type;
    int32_t n_ctx, Hkv, D;
    void * k;
    void * v;
    const int32_t * pt;
    const int32_t * rtab;
    int32_t psh;
    size_t pstride;
};

static F::kv_cache conv(const ref_kv * r) {
    F::kv_cache c;
    c.type = r->type; c.n_ctx = r->n_ctx; c.Hkv = r->Hkv; c.D = r->D; c.k = r->k; c.v = r->v;
    c.pt = r->pt; c.rtab = r->rtab; c.psh = r->psh; c.pstride = r->pstride;
    return c;
}
#define VIS __attribute__((visibility("default")))

VIS size_t ref_kv_row_bytes(uint32_t type, int Hkv, int D) { return F::kv_row_bytes(type, Hkv, D); }
VIS void ref_kv_append(const ref_kv * r, const float * k, const float * v, int p0, int T, void * s) {
    F::kv_cache c = conv(r);
    F::kv_append(c, k, v, p0, T, (cudaStream_t) s);
}
VIS void ref_kv_append_dev(const ref_kv * r, const float * k, const float * v, const int32_t * p0_dev, int T, void * s) {
    F::kv_cache c = conv(r);
    F::kv_append_dev(c, k, v, p0_dev, T, (cudaStream_t) s);
}
VIS int ref_attn_decode(const float * q, const ref_kv * r, float * out, int T, int p0, int Hq, float scale, void * s) {
    return F::attn_decode(q, conv(r), out, T, p0, Hq, scale, (cudaStream_t) s) ? 0 : 1;
}
VIS int ref_attn_decode_dev(const float * q, const ref_kv * r, float * out, int T, const int32_t * p0_dev, int max_n, int Hq,
                            float scale, void * s) {
    return F::attn_decode_dev(q, conv(r), out, T, p0_dev, max_n, Hq, scale, (cudaStream_t) s) ? 0 : 1;
}
VIS int ref_attn_decode_rows(const float * q, const ref_kv * r, float * out, int T, const int32_t * pos, int Hq, float scale,
                             void * s) {
    return F::attn_decode_rows(q, conv(r), out, T, pos, Hq, scale, (cudaStream_t) s) ? 0 : 1;
}
VIS int ref_attn_prefill(const float * q, const ref_kv * r, float * out, int T, int p0, int Hq, float scale, void * s) {
    return F::attn_prefill(q, conv(r), out, T, p0, Hq, scale, (cudaStream_t) s) ? 0 : 1;
}
VIS size_t ref_attn_fold_scratch_bytes(int T, int Hkv, int chunk, int nsplit) {
    return F::attn_fold_scratch_bytes(T, Hkv, chunk, nsplit);
}
VIS int ref_attn_fold(const float * q, const ref_kv * r, float * out, int T, int p0, int Hq, float scale, void * scratch,
                      size_t scratch_bytes, void * s) {
    return F::attn_fold(q, conv(r), out, T, p0, Hq, scale, scratch, scratch_bytes, (cudaStream_t) s) ? 0 : 1;
}
VIS int ref_attn_prep(const float * qg, const float * k, const float * v, const float * qn, const float * kn,
                      const int32_t * pos, float * q, float * gate, const ref_kv * r, int p0, int T, int Hq, int Hkv, int D,
                      int n_rot, float freq_base, float eps, void * s) {
    F::kv_cache c = conv(r);
    return F::attn_prep(qg, k, v, qn, kn, pos, q, gate, c, p0, T, Hq, Hkv, D, n_rot, freq_base, eps, (cudaStream_t) s) ? 0 : 1;
}
VIS int ref_attn_prep_mrope(const float * qg, const float * k, const float * v, const float * qn, const float * kn,
                            const int32_t * pos, float * q, float * gate, const ref_kv * r, int p0, int T, int Hq, int Hkv, int D,
                            int n_rot, float freq_base, float eps, void * s, const int32_t * mp, int stride, int s0, int s1, int s2,
                            int sect) {
    F::kv_cache c = conv(r);
    F::mrope_pos mr;
    mr.p = mp; mr.stride = stride; mr.s0 = s0; mr.s1 = s1; mr.s2 = s2; mr.sect = sect;
    return F::attn_prep(qg, k, v, qn, kn, pos, q, gate, c, p0, T, Hq, Hkv, D, n_rot, freq_base, eps, (cudaStream_t) s, 0, 0, 0, mr) ? 0 : 1;
}
VIS void ref_sigmoid_mul(float * x, const float * g, int64_t n, void * s) { F::sigmoid_mul(x, g, n, (cudaStream_t) s); }
VIS void ref_k_sigmoid_mul(float * x, const float * g, int64_t n, void * s) { K::sigmoid_mul(x, g, n, (cudaStream_t) s); }
VIS int ref_ew_quant(int op, const float * a, const float * b, float * y, void * qbuf, int T, int n, void * s) {
    return F::ew_quant((F::ew_op) op, a, b, y, qbuf, T, n, (cudaStream_t) s) ? 0 : 1;
}
VIS void ref_k_rope_neox(float * x, const int32_t * pos, int T, int H, int D, int n_rot, float freq_base, void * s) {
    K::rope_neox(x, pos, T, H, D, n_rot, freq_base, (cudaStream_t) s);
}
VIS void ref_k_attention(const float * q, const float * kc, const float * vc, float * out, int T, int p0, int Hq, int Hkv, int D,
                         float scale, void * s) {
    K::attention(q, kc, vc, out, T, p0, Hq, Hkv, D, scale, (cudaStream_t) s);
}
VIS int ref_attn_dec2_nsplit(int Hkv) { return F::attn_dec2_nsplit(Hkv); }

}  // extern "C"
