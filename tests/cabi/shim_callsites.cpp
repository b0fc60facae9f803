// Compile-only check of include/p100e_fast_shim.h: the call forms the reference engine uses for this path
// (src/tp_model.cu:1384-1397 fused decode layer, :1705-1749 per-op layer and KV-only catch-up, :2899-2920 prefill,
// tests/attn_dec_bench.cu split sweep) written against namespace p100e::fast must compile unchanged.
// Built with `g++ -fsyntax-only` by tests/test_abi.py; never linked or run.
#include <algorithm>
#include <cmath>
#include <stdexcept>

#include "p100e_fast_shim.h"

namespace fast = p100e::fast;

struct rank_state {
    float * a, * b, * c, * d, * e, * g, * w_scratch;
    void * aq;
    int32_t * pos;
    cudaStream_t s;
};

void fused_layer(rank_state & S, fast::kv_cache kv, const float * q, const float * kk, const float * v, const float * q_norm,
                 const float * k_norm, int nseq, int T, int Hl, int HKVl, int HD_, int NROT_, float rope_base_, float eps_, int n_ctx_,
                 const fast::mrope_pos & mr) {
    if (!fast::attn_prep(q, kk, v, q_norm, k_norm, S.pos, S.c, S.d, kv, -1, T, Hl, HKVl, HD_, NROT_, rope_base_, eps_, S.s, 0, 0, 0, mr))
        throw std::runtime_error("fast::attn_prep: unsupported shape");
    if (nseq == 1) {
        if (!fast::attn_decode_dev(S.c, kv, S.b, T, S.pos, n_ctx_, Hl, 1.0f / sqrtf((float) HD_), S.s))
            throw std::runtime_error("fast::attn_decode_dev: no kernel ran");
    } else if (!fast::attn_decode_rows(S.c, kv, S.b, T, S.pos, Hl, 1.0f / sqrtf((float) HD_), S.s))
        throw std::runtime_error("fast::attn_decode_rows: unsupported shape");
    if (!fast::ew_quant(fast::EW_SIGMOID_MUL, S.b, S.d, S.b, S.aq, T, Hl * HD_, S.s)) fast::sigmoid_mul(S.b, S.d, (int64_t) T * Hl * HD_, S.s);
}

void per_op_layer(rank_state & S, fast::kv_cache kv, int p0, int T, int Hl, int HD_, bool kv_only) {
    if (kv_only) { fast::kv_append(kv, S.e, S.g, p0, T, S.s); return; }
    fast::kv_append(kv, S.e, S.g, p0, T, S.s);
    if (!(T > 4 && T <= fast::ATTN_MAX_ROWS && fast::attn_decode2(S.c, kv, S.b, T, p0, nullptr, Hl, 1.0f / sqrtf((float) HD_), S.s)))
        for (int t0 = 0; t0 < T; t0 += 4) {
            const int nt = std::min(4, T - t0);
            if (!fast::attn_decode(S.c + (size_t) t0 * Hl * HD_, kv, S.b + (size_t) t0 * Hl * HD_, nt, p0 + t0, Hl, 1.0f / sqrtf((float) HD_), S.s))
                throw std::runtime_error("fast::attn_decode: no kernel ran");
        }
    fast::sigmoid_mul(S.b, S.d, (int64_t) T * Hl * HD_, S.s);
}

void forward_prefill(rank_state & S, fast::kv_cache kv, int n_past, int T, int Hl, int HD_, size_t scratch_elems_, bool use_fold, bool env_attn) {
    fast::kv_append(kv, S.e, S.g, n_past, T, S.s);
    const float scale = 1.0f / sqrtf((float) HD_);
    const bool folded = use_fold && fast::attn_fold(S.c, kv, S.b, T, n_past, Hl, scale, S.w_scratch, scratch_elems_ * 4, S.s);
    if (!folded && !(env_attn && fast::attn_prefill(S.c, kv, S.b, T, n_past, Hl, scale, S.s)) &&
        !(T > 4 && T <= fast::ATTN_MAX_ROWS && fast::attn_decode2(S.c, kv, S.b, T, n_past, nullptr, Hl, scale, S.s)))
        throw std::runtime_error("no kernel ran");
    (void) fast::attn_fold_scratch_bytes(T, kv.Hkv, 0, 0);
    (void) fast::attn_prefill_variant(S.c, kv, S.b, T, n_past, Hl, scale, S.s, 2);
}

void bench_and_setup(fast::kv_cache & kv, cudaStream_t s) {
    fast::kv_fill_random(kv, 0, kv.n_ctx, 1234u, s);
    (void) fast::attn_dec2_nsplit(kv.Hkv);
    fast::attn_dec2_set_nsplit(16);
    (void) fast::attn_dec2_reload_env();
    fast::kv_cache c2 = fast::kv_alloc(fast::KV_Q8_0, 1024, 4, 256);
    (void) fast::kv_row_bytes(fast::KV_Q4_0, 4, 256);
    const int32_t * p0_dev = nullptr;
    fast::kv_append_dev(c2, nullptr, nullptr, p0_dev, 1, s);
    fast::kv_free(c2);
}
