// Prefill attention entry points (tensor-core kernel under construction in this file).
#include "common.cuh"
using namespace b200;
extern "C" {
int b200_attn_prefill(const float *, const b200_kv_cache *, float *, int, int, int, float, void *) { B200_REFUSE(B200_ERR_SHAPE, "attn_prefill: not built"); }
int b200_attn_prefill_variant(const float *, const b200_kv_cache *, float *, int, int, int, float, void *, int) { B200_REFUSE(B200_ERR_SHAPE, "attn_prefill: not built"); }
size_t b200_attn_fold_scratch_bytes(int, int, int, int) { return 0; }
int b200_attn_fold(const float *, const b200_kv_cache *, float *, int, int, int, float, void *, size_t, void *, int, int) { B200_REFUSE(B200_ERR_SHAPE, "attn_fold: not built"); }
int b200_attn_prefill_gated(const float *, const b200_kv_cache *, float *, const float *, int, int, int, float, void *, size_t, void *) { B200_REFUSE(B200_ERR_SHAPE, "attn_prefill: not built"); }
}
