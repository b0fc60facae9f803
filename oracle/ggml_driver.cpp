// extern "C" doorway to the reference's CPU attention path: the vendored ggml CPU backend's flash_attn_ext
// (third_party/llama.cpp-fork/ggml/src/ggml-cpu/ops.cpp:8614-8850 in the reference project) and its reference
// quantisers (ggml-quants.c:113-148,276-299).  TEST / BENCHMARK-BASELINE INFRASTRUCTURE, not product code.
// Compiled with the vendored ggml sources, taken where they lie, into oracle/_ref/libggml_ref.so by oracle/Makefile.
#include <cstdint>
#include <cstring>
#include <cstdlib>
#include <cmath>
#include <vector>

#include "ggml.h"
#include "ggml-cpu.h"

extern "C" {
// from ggml-quants.h (C linkage)
void quantize_row_q4_0_ref(const float * x, void * y, int64_t k);
void quantize_row_q8_0_ref(const float * x, void * y, int64_t k);

#define VIS __attribute__((visibility("default")))

// k values -> k/32 ggml blocks (q8_0: 34 B {f16 d, int8[32]}; q4_0: 18 B {f16 d, 16 nibble bytes})
VIS void ggml_ref_quantize_q8_0(const float * x, void * y, int64_t k) { quantize_row_q8_0_ref(x, y, k); }
VIS void ggml_ref_quantize_q4_0(const float * x, void * y, int64_t k) { quantize_row_q4_0_ref(x, y, k); }
VIS uint16_t ggml_ref_fp32_to_fp16(float f) { return ggml_fp32_to_fp16(f); }
VIS float ggml_ref_fp16_to_fp32(uint16_t h) { return ggml_fp16_to_fp32(h); }

// One slot of decode / verify attention through ggml_flash_attn_ext on n_threads CPU threads.
//   q    [q_len][Hq][D] f32
//   k, v [n_kv][Hkv] head rows as ggml blocks of `type` (1 = f16, 2 = q4_0, 8 = q8_0), i.e. ggml tensors
//        [D, n_kv, Hkv] with nb1 = Hkv * head_bytes, nb2 = head_bytes
//   row j of the slot sits at position n_kv - q_len + j (causal among the q_len rows): f16 mask [n_kv_pad, q_len_pad]
//   out  [q_len][Hq][D] f32
// reps > 1 repeats the graph compute (timing).  Returns 0 on success.
VIS int ggml_ref_flash_attn(const float * q, const void * k, const void * v, int type, int n_kv, int q_len, int Hq, int Hkv,
                            int D, float scale, int n_threads, int reps, float * out) {
    const ggml_type kt = (ggml_type) type;
    const size_t hb = ggml_row_size(kt, D);
    const int n_kv_pad = (n_kv + 255) / 256 * 256, q_pad = (q_len + 63) / 64 * 64;
    const size_t ctx_bytes = (size_t) q_len * Hq * D * 4 * 3 + (size_t) n_kv_pad * q_pad * 2 + ((size_t) 64 << 20) +
                             (size_t) n_threads * (D * 16 + 1024);
    ggml_init_params ip = {ctx_bytes, nullptr, false};
    ggml_context * ctx = ggml_init(ip);
    if (!ctx) return 1;
    ggml_tensor * tq = ggml_new_tensor_3d(ctx, GGML_TYPE_F32, D, q_len, Hq);
    // q comes as [q_len][Hq][D]; ggml wants [D, q_len, Hq] contiguous
    for (int j = 0; j < q_len; ++j)
        for (int h = 0; h < Hq; ++h)
            memcpy((char *) tq->data + ((size_t) h * q_len + j) * D * 4, q + ((size_t) j * Hq + h) * D, (size_t) D * 4);
    // K, V as views over the caller's memory (no copy): header tensors without data, then point them
    ggml_tensor * tk = ggml_new_tensor_3d(ctx, kt, D, 1, 1);
    ggml_tensor * tv = ggml_new_tensor_3d(ctx, kt, D, 1, 1);
    for (ggml_tensor * t : {tk, tv}) {
        t->ne[1] = n_kv; t->ne[2] = Hkv;
        t->nb[1] = hb * Hkv; t->nb[2] = hb; t->nb[3] = hb * Hkv * n_kv;
    }
    tk->data = const_cast<void *>(k);
    tv->data = const_cast<void *>(v);
    ggml_tensor * mask = ggml_new_tensor_2d(ctx, GGML_TYPE_F16, n_kv_pad, q_pad);
    {
        const ggml_fp16_t z = ggml_fp32_to_fp16(0.0f), ninf = ggml_fp32_to_fp16(-INFINITY);
        ggml_fp16_t * m = (ggml_fp16_t *) mask->data;
        for (int j = 0; j < q_pad; ++j)
            for (int i = 0; i < n_kv_pad; ++i)
                m[(size_t) j * n_kv_pad + i] = (j < q_len && i <= n_kv - q_len + j) ? z : ninf;
    }
    ggml_tensor * o = ggml_flash_attn_ext(ctx, tq, tk, tv, mask, scale, 0.0f, 0.0f);   // [D, Hq, q_len]
    ggml_cgraph * gf = ggml_new_graph(ctx);
    ggml_build_forward_expand(gf, o);
    for (int r = 0; r < (reps > 0 ? reps : 1); ++r)
        if (ggml_graph_compute_with_ctx(ctx, gf, n_threads) != GGML_STATUS_SUCCESS) { ggml_free(ctx); return 2; }
    memcpy(out, o->data, (size_t) q_len * Hq * D * 4);
    ggml_free(ctx);
    return 0;
}
}
