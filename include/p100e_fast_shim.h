// Header-only C++ shim: re-creates the reference's `namespace p100e::fast` attention interface (src/fast/attn.cuh,
// attn_dec2.cuh, attn_fold.cuh, fused.cuh, mrope.cuh in the reference project) on top of the C ABI of libb200attn.so, so
// that callers written against the reference (tp_model.cu:1384-1397,1728-1749,2905-2920; tp_mtp.cu) compile unchanged:
// same names, same argument lists and defaults, bool results (true = kernels enqueued, false = nothing launched).
// Include this instead of "fast/attn.cuh" / "fast/attn_dec2.cuh" / "fast/attn_fold.cuh" / the attention part of
// "fast/fused.cuh" and link libb200attn.so.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

#include "b200attn.h"

namespace p100e::fast {

constexpr uint32_t KV_F16 = B200_KV_F16;    // src/fast/attn.cuh:14
constexpr uint32_t KV_Q4_0 = B200_KV_Q4_0;  // :15
constexpr uint32_t KV_Q8_0 = B200_KV_Q8_0;  // :16
constexpr int ATTN_MAX_ROWS = B200_ATTN_MAX_ROWS;   // :66

struct kv_cache {   // src/fast/attn.cuh:18-32, same fields and defaults
    uint32_t type = KV_F16;
    int n_ctx = 0, Hkv = 0, D = 0;
    void * k = nullptr;
    void * v = nullptr;
    const int32_t * pt = nullptr;
    const int32_t * rtab = nullptr;
    int psh = 0;
    size_t pstride = 0;
};
static_assert(sizeof(kv_cache) == sizeof(b200_kv_cache), "kv_cache must match b200_kv_cache field for field");

struct mrope_pos {   // src/fast/mrope.cuh:16-21
    const int32_t * p = nullptr;
    int stride = 0;
    int s0 = 0, s1 = 0, s2 = 0;
    int sect = 0;
};
enum ew_op : int { EW_SILU_MUL = 0, EW_SIGMOID_MUL = 1 };   // src/fast/fused.cuh:93

namespace detail {
inline const b200_kv_cache * c(const kv_cache & x) { return reinterpret_cast<const b200_kv_cache *>(&x); }
}

inline size_t kv_row_bytes(uint32_t type, int Hkv, int D) { return b200_kv_row_bytes(type, Hkv, D); }
inline kv_cache kv_alloc(uint32_t type, int n_ctx, int Hkv, int D) {
    kv_cache out;
    b200_kv_cache tmp;
    b200_kv_alloc(&tmp, type, n_ctx, Hkv, D);   // k == nullptr on failure, as the reference
    out.type = tmp.type; out.n_ctx = tmp.n_ctx; out.Hkv = tmp.Hkv; out.D = tmp.D; out.k = tmp.k; out.v = tmp.v;
    return out;
}
inline void kv_free(kv_cache & x) { b200_kv_free(reinterpret_cast<b200_kv_cache *>(&x)); }
inline void kv_append(kv_cache & x, const float * k, const float * v, int p0, int T, cudaStream_t s) {
    b200_kv_append(detail::c(x), k, v, p0, T, s);
}
inline void kv_append_dev(kv_cache & x, const float * k, const float * v, const int32_t * p0_dev, int T, cudaStream_t s) {
    b200_kv_append_dev(detail::c(x), k, v, p0_dev, T, s);
}
inline bool attn_decode(const float * q, const kv_cache & x, float * out, int T, int p0, int Hq, float scale, cudaStream_t s) {
    return b200_attn_decode(q, detail::c(x), out, T, p0, Hq, scale, s) == B200_OK;
}
inline bool attn_decode_dev(const float * q, const kv_cache & x, float * out, int T, const int32_t * p0_dev, int max_n, int Hq,
                            float scale, cudaStream_t s) {
    return b200_attn_decode_dev(q, detail::c(x), out, T, p0_dev, max_n, Hq, scale, s) == B200_OK;
}
inline bool attn_decode_rows(const float * q, const kv_cache & x, float * out, int T, const int32_t * pos, int Hq, float scale,
                             cudaStream_t s) {
    return b200_attn_decode_rows(q, detail::c(x), out, T, pos, Hq, scale, s) == B200_OK;
}
inline bool attn_decode2(const float * q, const kv_cache & x, float * out, int T, int p0, const int32_t * p0_dev, int Hq,
                         float scale, cudaStream_t s, const int32_t * pos_rows = nullptr) {
    return b200_attn_decode2(q, detail::c(x), out, T, p0, p0_dev, Hq, scale, s, pos_rows) == B200_OK;
}
inline int attn_dec2_nsplit(int Hkv) { return b200_attn_dec2_nsplit(Hkv); }
inline void attn_dec2_set_nsplit(int n) { b200_attn_dec2_set_nsplit(n); }
inline bool attn_dec2_reload_env() { return b200_attn_dec2_reload_env() != 0; }
inline bool attn_prefill(const float * q, const kv_cache & x, float * out, int T, int p0, int Hq, float scale, cudaStream_t s) {
    return b200_attn_prefill(q, detail::c(x), out, T, p0, Hq, scale, s) == B200_OK;
}
inline bool attn_prefill_variant(const float * q, const kv_cache & x, float * out, int T, int p0, int Hq, float scale,
                                 cudaStream_t s, int variant) {
    return b200_attn_prefill_variant(q, detail::c(x), out, T, p0, Hq, scale, s, variant) == B200_OK;
}
inline size_t attn_fold_scratch_bytes(int T, int Hkv, int chunk, int nsplit) {
    return b200_attn_fold_scratch_bytes(T, Hkv, chunk, nsplit);
}
inline bool attn_fold(const float * q, const kv_cache & x, float * out, int T, int p0, int Hq, float scale, void * scratch,
                      size_t scratch_bytes, cudaStream_t s, int chunk = 0, int nsplit = 0) {
    return b200_attn_fold(q, detail::c(x), out, T, p0, Hq, scale, scratch, scratch_bytes, s, chunk, nsplit) == B200_OK;
}
inline void kv_fill_random(kv_cache & x, int p0, int p1, uint32_t seed, cudaStream_t s) {
    b200_kv_fill_random(detail::c(x), p0, p1, seed, s);
}
inline bool attn_prep(const float * qg, const float * k, const float * v, const float * q_norm, const float * k_norm,
                      const int32_t * pos, float * q, float * gate, kv_cache & x, int p0, int T, int Hq, int Hkv, int D,
                      int n_rot, float freq_base, float eps, cudaStream_t s, int ldq = 0, int ldk = 0, int ldv = 0,
                      const mrope_pos & mr = mrope_pos{}) {
    b200_mrope_pos m{mr.p, mr.stride, mr.s0, mr.s1, mr.s2, mr.sect};
    return b200_attn_prep(qg, k, v, q_norm, k_norm, pos, q, gate, detail::c(x), p0, T, Hq, Hkv, D, n_rot, freq_base, eps, s, ldq,
                          ldk, ldv, mr.p ? &m : nullptr) == B200_OK;
}
inline bool ew_quant(ew_op op, const float * a, const float * b, float * y, void * qbuf, int T, int n, cudaStream_t s,
                     int lda = 0, int ldb = 0) {
    return b200_ew_quant((int) op, a, b, y, qbuf, T, n, s, lda, ldb) == B200_OK;
}
inline void sigmoid_mul(float * x, const float * g, int64_t n, cudaStream_t s) { b200_sigmoid_mul(x, g, n, s); }

}  // namespace p100e::fast
