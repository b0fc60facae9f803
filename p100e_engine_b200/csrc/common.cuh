// Shared device/host helpers of the B200 paged-KV attention library: cache addressing, block quantisers,
// small PTX wrappers (mbarrier, bulk async copy, warp MMA) and the device status word.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#include "../../include/b200attn.h"

namespace b200 {

constexpr int DH = 256;   // head dim of the attention kernels
constexpr int GQA = 6;    // query heads per kv head
constexpr int NBLK = DH / 32;

#define B200_NEG_INF __int_as_float(0xff800000)

// ---- status word -----------------------------------------------------------------------------------------------
// One word per device in global memory; kernels OR a code into it instead of trapping. Codes:
enum : unsigned {
    ST_WAIT_TIMEOUT = 1u,   // an mbarrier wait ran out of its time limit
    ST_BAD_PAGE = 2u,       // a page-table entry was negative
    ST_BAD_ALIGN = 4u,      // an address that must be 16-byte aligned was not
    ST_BAD_POS = 8u         // a row position lay beyond the caller's max_n (or beyond n_ctx of a contiguous cache): the keys
                            // past the limit were left out instead of being read
};
unsigned * device_status_word();          // device pointer for the current device (allocated on first use), or nullptr
void count_launch(int n = 1);
// bf16 token rows -> K rotated and K, V quantised into cache rows p0 + t; q (optional) rotated into fp32 q_out; cs_out
// (optional) receives each token's cos / sin table [T][n_rot]; rope0 >= 0: the angles come from positions rope0 + t instead
// of p0 + t; k == v == nullptr: only q is rotated (defined in kv_append.cu)
int rope_append_launch(const uint16_t * q, const uint16_t * k, const uint16_t * v, float * q_out, float * cs_out,
                       const b200_kv_cache * c, int p0, int T, int Hq, int Hkv, int D, int n_rot, float freq_base, cudaStream_t s,
                       const char * who, int rope0 = -1);

// ---- row sizes (reference: kv_row_bytes, src/fast/attn.cu:501-503) ---------------------------------------------
__host__ __device__ constexpr int head_bytes(uint32_t type, int D = DH) {
    return type == B200_KV_F16 ? D * 2 : type == B200_KV_Q8_0 ? (D / 32) * 34 : (D / 32) * 18;
}

// ---- paged addressing (reference: kv_pg / kv_off, src/fast/kv_page.cuh:11-31) ----------------------------------
struct kv_view {
    char * k;
    char * v;
    const int32_t * pt;
    const int32_t * rtab;
    int psh;
    int Hkv;
    unsigned long long pstride;
    unsigned long long rowb;
};

inline kv_view view_of(const b200_kv_cache & c) {
    kv_view g;
    g.k = (char *) c.k; g.v = (char *) c.v; g.pt = c.pt; g.rtab = c.rtab; g.psh = c.psh; g.Hkv = c.Hkv;
    g.pstride = c.pstride;
    g.rowb = (unsigned long long) c.Hkv * head_bytes(c.type, c.D);
    return g;
}

// page table of query row t (nullptr when contiguous)
__device__ __forceinline__ const int32_t * kv_tab(const kv_view & g, int t) {
    return g.pt ? (g.rtab ? g.pt + g.rtab[t] : g.pt) : nullptr;
}
// byte offset of position p, 64-bit throughout
__device__ __forceinline__ unsigned long long kv_off_tab(const kv_view & g, const int32_t * tab, int p) {
    if (!tab) return (unsigned long long) p * g.rowb;
    return (unsigned long long) tab[p >> g.psh] * g.pstride + (unsigned long long) (p & ((1 << g.psh) - 1)) * g.rowb;
}

// ---- block quantisers ------------------------------------------------------------------------------------------
// q8_0 (reference: q8_quant_block_warp, src/fast/kv_q8.cuh:20-26 == ggml quantize_row_q8_0_ref): d = amax / 127,
// id = d ? 1 / d : 0, q = (int8) roundf(x * id).  amax is an exact maximum, so any reduction order gives the same d.
__device__ __forceinline__ float q8_scale(float amax, float & id) {
    const float d = amax / 127.0f;
    id = d != 0.0f ? 1.0f / d : 0.0f;
    return d;
}
__device__ __forceinline__ int q8_quant(float x, float id) { return (int) roundf(x * id); }

// q4_0 (reference: q4_quant_block_warp, src/fast/kv_q8.cuh:32-49 == ggml quantize_row_q4_0_ref): the element of
// largest magnitude, lowest index on ties, gives d = max / -8; q = min(15, (int)(x * id + 8.5f)) with the product
// rounded before the add.  (a, idx) pairs are totally ordered, so any reduction order finds the same element.
__device__ __forceinline__ void q4_argmax_merge(float & a, int & idx, float oa, int oi) {
    if (oa > a || (oa == a && oi < idx)) { a = oa; idx = oi; }
}
__device__ __forceinline__ int q4_quant(float x, float id) {
    return min(15, (int) __fadd_rn(__fmul_rn(x, id), 8.5f));
}

// ---- partial NEOX rotation -------------------------------------------------------------------------------------
// One rotary pair.  Written with explicit roundings (one product rounded, the other fused into the add) so that every
// kernel of the library produces the same bits whatever the surrounding code looks like; the choice of the fused product is
// the one nvcc makes for the reference's x0*c - x1*s / x0*s + x1*c (src/fast/fused.cu:552-557; checked bytewise against
// the reference kernels).
__device__ __forceinline__ void rot_pair(float x0, float x1, float c, float sn, float & y0, float & y1) {
    y0 = __fmaf_rn(x0, c, -__fmul_rn(x1, sn));
    y1 = __fmaf_rn(x1, c, __fmul_rn(x0, sn));
}

// ---- PTX helpers -----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t * bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t * bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t * bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: gives up after ~2 s, records ST_WAIT_TIMEOUT and returns false (the caller carries on with whatever
// is in shared memory; the host sees the status word and discards the result).
__device__ __forceinline__ bool mbar_wait(uint64_t * bar, uint32_t parity, unsigned * status) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    for (int i = 0; i < (1 << 26); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255) == 255 && globaltimer_ns() - t0 > 2000000000ull) break;
    }
    if (status) atomicOr(status, ST_WAIT_TIMEOUT);
    return false;
}
// 1-D bulk async copy global -> shared (TMA unit), completion counted in bytes on an mbarrier.
// dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void * dst, const void * src, uint32_t bytes, uint64_t * bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// D (fp32, 16x8) += A (f16, 16x16, row) * B (f16, 16x8, col)
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// same, with the accumulator starting from c (kept in its own registers)
__device__ __forceinline__ void mma16816_from(float (&d)[4], const float4 c, const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c.x), "f"(c.y), "f"(c.z), "f"(c.w));
}

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// ---- a16 activation format -------------------------------------------------------------------------------------
// The format the engine's next projection reads (reference: src/fast/a16q.cuh:4-10, a16_quant8 :21-45, consumed by
// matvec_prequantized, src/tp_model.cu:1394-1398): per 32 consecutive values one scale pair (amax, sum of value / amax) as
// half2 and the 32 scaled values as 16 half2 in a fixed slot order; for T rows of n values, the scaled values of all groups
// come first ([T * n/32][16] half2), the scale pairs after them ([T * n/32] half2).
// This helper serves epilogues whose result sits in registers as one float4 per lane: eight neighbouring lanes (l = lane & 7)
// hold one group, lane l its values 4l..4l+3; all eight call together from a fully active warp.  The bytes are fixed by
// the format: the maximum is exact in any order, the scaling is one rounded multiply by the IEEE reciprocal, and the sum
// runs 0 + y0 + y1 + y2 + y3 inside a lane and then over lane distances 4, 2, 1.
__device__ __forceinline__ void a16_store_lanes8(const float4 x, __half2 * __restrict__ qbuf, size_t group, size_t n_groups,
                                                 bool live) {
    const int l = threadIdx.x & 7;
    float amax = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    if (!(amax < 65520.0f)) amax = 65504.0f;                       // keeps the stored scale a finite half
    const float inv = amax > 0.0f ? __frcp_rn(amax) : 0.0f;
    const float y0 = __fmul_rn(x.x, inv), y1 = __fmul_rn(x.y, inv), y2 = __fmul_rn(x.z, inv), y3 = __fmul_rn(x.w, inv);
    float sum = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(0.0f, y0), y1), y2), y3);
    sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, 4));
    sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, 2));
    sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, 1));
    if (!live) return;
    __half2 * q = qbuf + group * 16;
    // lanes l and l + 4 interleave: slots 4k .. 4k+3 = (lane k: y0,y2) (lane k+4: y0,y2) (lane k: y1,y3) (lane k+4: y1,y3)
    const int slot = 4 * (l & 3) + (l >> 2);
    q[slot] = __floats2half2_rn(y0, y2);
    q[slot + 2] = __floats2half2_rn(y1, y3);
    if (l == 0) qbuf[n_groups * 16 + group] = __floats2half2_rn(amax, sum);
}

inline bool aligned16(const void * p) { return ((uintptr_t) p & 15) == 0; }

#define B200_REFUSE(code, ...) do { fprintf(stderr, "b200attn: " __VA_ARGS__); fprintf(stderr, "\n"); return (code); } while (0)

// after a launch: B200_OK, or B200_ERR_CUDA with the runtime's message
inline int launch_status(const char * what) {
    const cudaError_t e = cudaPeekAtLastError();
    if (e == cudaSuccess) return B200_OK;
    fprintf(stderr, "b200attn: %s: %s\n", what, cudaGetErrorString(e));
    return B200_ERR_CUDA;
}

}  // namespace b200
