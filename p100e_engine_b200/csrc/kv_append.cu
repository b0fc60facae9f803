// KV append, attention input prep (norm + partial RoPE + quantise + append), cache helpers and the sigmoid gate.
//
// Cache bytes are produced by the same fp32 recipes as the reference quantisers (src/fast/kv_q8.cuh:20-49,
// src/fast/attn.cu:245-283 in the reference project), so every position written here is byte-identical to what the
// reference writes for the same inputs, paged or contiguous.
#include "common.cuh"

#include <cuda_bf16.h>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <vector>

namespace b200 {

// ---------------------------------------------------------------------------------------------- library state ----
static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((uint64_t) n, std::memory_order_relaxed); }

static unsigned * g_status[64];
unsigned * device_status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    unsigned *& p = g_status[dev & 63];
    if (!p) {
        if (cudaMalloc(&p, 256) != cudaSuccess) { cudaGetLastError(); p = nullptr; return nullptr; }
        cudaMemset(p, 0, 256);
    }
    return p;
}

namespace {

// ------------------------------------------------------------------------------------------------ quantisers ----
// One full warp converts 32 consecutive values (lane = value index) of block b of a head row and stores them.
template <uint32_t KT>
__device__ __forceinline__ void store_block_warp(float x, int lane, char * head, int b, int nb) {
    if constexpr (KT == B200_KV_F16) {
        reinterpret_cast<__half *>(head)[b * 32 + lane] = __float2half(x);
    } else if constexpr (KT == B200_KV_Q8_0) {
        float amax = fabsf(x);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        float id;
        const float d = q8_scale(amax, id);
        reinterpret_cast<int8_t *>(head + nb * 2)[b * 32 + lane] = (int8_t) q8_quant(x, id);
        if (lane == 0) reinterpret_cast<__half *>(head)[b] = __float2half(d);
    } else {
        float a = fabsf(x);
        int idx = lane;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float oa = __shfl_xor_sync(0xffffffffu, a, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            q4_argmax_merge(a, idx, oa, oi);
        }
        const float xm = __shfl_sync(0xffffffffu, x, idx);
        const float mx = a > 0.0f ? xm : 0.0f;
        const float d = mx / -8.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        const int q = q4_quant(x, id);
        const int qhi = __shfl_down_sync(0xffffffffu, q, 16);
        char * blk = head + b * 18;
        if (lane < 16) blk[2 + lane] = (char) (q | (qhi << 4));
        if (lane == 0) *reinterpret_cast<__half *>(blk) = __float2half(d);
    }
}

// k, v [T][Hkv][D] f32 -> cache rows; one warp per 32-value block of K and of V.
// grid (ceil(Hkv*D/32 / 8), T), 256 threads.
template <uint32_t KT>
__global__ void __launch_bounds__(256) append_k(const float * __restrict__ k, const float * __restrict__ v, kv_view g,
                                                int p0, const int32_t * __restrict__ p0p, int D, unsigned * status) {
    if (p0p) p0 = *p0p;
    const int t = blockIdx.y;
    const int nb = D / 32, nblk = g.Hkv * nb;
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= nblk) return;
    const int lane = threadIdx.x & 31, h = i / nb, b = i - h * nb;
    const int32_t * tab = kv_tab(g, t);
    if (tab && tab[(p0 + t) >> g.psh] < 0) { if (lane == 0) atomicOr(status, ST_BAD_PAGE); return; }
    const unsigned long long o = kv_off_tab(g, tab, p0 + t) + (unsigned long long) h * head_bytes(KT, D);
    const size_t src = (size_t) t * g.Hkv * D + (size_t) i * 32 + lane;
    store_block_warp<KT>(k[src], lane, g.k + o, b, nb);
    store_block_warp<KT>(v[src], lane, g.v + o, b, nb);
}

// ------------------------------------------------------------------------------------------- attention prep ----
// NEOX rotation of one pair.  Written with explicit roundings (one product rounded, the other fused into the add) so that
// every kernel of this file produces the same bits whatever the surrounding code looks like; the choice of the fused product
// is the one nvcc makes for the reference's x0*c - x1*s / x0*s + x1*c (checked bytewise against the reference kernels).
__device__ __forceinline__ void rot_pair(float x0, float x1, float c, float sn, float & y0, float & y1) {
    y0 = __fmaf_rn(x0, c, -__fmul_rn(x1, sn));
    y1 = __fmaf_rn(x1, c, __fmul_rn(x0, sn));
}

__device__ __forceinline__ float butterfly_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// position of rotary pair j of row t under interleaved M-RoPE (semantics of src/fast/mrope.cuh:23-31)
__device__ __forceinline__ int mrope_position(const b200_mrope_pos & m, int t, int j) {
    const int sector = j % m.sect;
    int s;
    if (sector % 3 == 1 && sector < 3 * m.s1) s = 1;
    else if (sector % 3 == 2 && sector < 3 * m.s2) s = 2;
    else if (sector % 3 == 0 && sector < 3 * m.s0) s = 0;
    else return 0;
    return m.p[s * m.stride + t];
}

template <typename TIN> __device__ __forceinline__ float ld_f32(const TIN * p, size_t i);
template <> __device__ __forceinline__ float ld_f32<float>(const float * p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16 * p, size_t i) { return __bfloat162float(p[i]); }

// One block per (item b, token t): items 0..Hq-1 = q heads, Hq..Hq+Hkv-1 = k heads, then the v heads.
// blockDim = D/4 rounded up to a warp multiple; thread i owns values 4i..4i+3 for the norm.
//   NORM  : RMSNorm with weights qn / kn before the rotation (the decode path, reference attn_prep_k fused.cu:502-573)
//   !NORM : rotation only (the prefill path: k::rope_neox + kv_append, reference src/tp_model.cu:2899-2908)
//   SPLITQ: q rows are [q | gate] pairs of 2*D values (gate copied out)
// The sum of squares keeps the reference's order: per thread a.x*a.x + a.y*a.y + a.z*a.z + a.w*a.w, xor butterfly inside
// each warp, warp sums combined by a second butterfly (block_sum, fused.cu:56-67); the rotation is written with the
// reference's expressions so that the compiler contracts them the same way.
template <uint32_t KT, typename TIN, bool NORM, bool SPLITQ, bool MR>
__global__ void prep_k(const TIN * __restrict__ qg, const TIN * __restrict__ k, const TIN * __restrict__ v,
                       const float * __restrict__ qn, const float * __restrict__ kn, const int32_t * __restrict__ pos,
                       float * __restrict__ q, float * __restrict__ gate, kv_view g, int p0, int Hq, int Hkv, int D,
                       int n_rot, float freq_base, float eps, int ldq, int ldk, int ldv, b200_mrope_pos mr,
                       const int32_t * __restrict__ crow, unsigned * status) {
    extern __shared__ float smr[];   // D floats: the head after norm, rotated in place
    __shared__ float wsum[32];
    const int t = blockIdx.y, b = blockIdx.x, i = threadIdx.x, D4 = D >> 2;
    const int lane = i & 31, wid = i >> 5, nw = blockDim.x >> 5, nb = D / 32;
    const bool isq = b < Hq;
    if (isq && !qg) return;
    const int ppos = pos ? pos[t] : p0 + t;         // rotary position
    const int row = crow ? crow[t] : p0 < 0 ? ppos : p0 + t;   // cache position (crow: explicit, < 0 = not stored here)
    unsigned long long roff = 0;
    if (!isq) {
        if (row < 0) return;
        const int32_t * tab = kv_tab(g, t);
        if (tab && tab[row >> g.psh] < 0) { if (i == 0) atomicOr(status, ST_BAD_PAGE); return; }
        roff = kv_off_tab(g, tab, row);
    }
    if (b >= Hq + Hkv) {   // v head: no norm, no rotation
        const int h = b - Hq - Hkv;
        const TIN * src = v + (size_t) t * ldv + (size_t) h * D;
        char * head = g.v + roff + (unsigned long long) h * head_bytes(KT, D);
        for (int bb = wid; bb < nb; bb += nw) store_block_warp<KT>(ld_f32(src, (size_t) bb * 32 + lane), lane, head, bb, nb);
        return;
    }
    const int h = isq ? b : b - Hq;
    const TIN * src = isq ? qg + (size_t) t * ldq + (size_t) h * (SPLITQ ? 2 : 1) * D : k + (size_t) t * ldk + (size_t) h * D;
    float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (i < D4) {
        a = make_float4(ld_f32(src, 4 * i), ld_f32(src, 4 * i + 1), ld_f32(src, 4 * i + 2), ld_f32(src, 4 * i + 3));
        if (isq && SPLITQ) {
            float4 gv = make_float4(ld_f32(src, D + 4 * i), ld_f32(src, D + 4 * i + 1), ld_f32(src, D + 4 * i + 2),
                                    ld_f32(src, D + 4 * i + 3));
            reinterpret_cast<float4 *>(gate + ((size_t) t * Hq + h) * D)[i] = gv;
        }
    }
    if constexpr (NORM) {
        const float * w = isq ? qn : kn;
        float ss = 0.0f;
        if (i < D4) ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        ss = butterfly_sum(ss);
        if (nw > 1) {
            __syncthreads();
            if (lane == 0) wsum[wid] = ss;
            __syncthreads();
            ss = lane < nw ? wsum[lane] : 0.0f;
            ss = butterfly_sum(ss);
        }
        const float sc = rsqrtf(ss / D + eps);
        if (i < D4) {
            float4 o = a;
            o.x *= sc; o.y *= sc; o.z *= sc; o.w *= sc;
            if (w) { const float4 ww = reinterpret_cast<const float4 *>(w)[i]; o.x *= ww.x; o.y *= ww.y; o.z *= ww.z; o.w *= ww.w; }
            reinterpret_cast<float4 *>(smr)[i] = o;
        }
    } else {
        if (i < D4) reinterpret_cast<float4 *>(smr)[i] = a;
    }
    __syncthreads();
    const int half = n_rot / 2;
    for (int j = i; j < half; j += blockDim.x) {
        float theta;
        if constexpr (MR) theta = (float) mrope_position(mr, t, j) * powf(freq_base, -2.0f * j / n_rot);
        else theta = (float) ppos * powf(freq_base, -2.0f * j / n_rot);
        const float c = cosf(theta), sn = sinf(theta);
        rot_pair(smr[j], smr[j + half], c, sn, smr[j], smr[j + half]);
    }
    __syncthreads();
    if (isq) {
        float4 * dst = reinterpret_cast<float4 *>(q + ((size_t) t * Hq + h) * D);
        for (int e = i; e < D4; e += blockDim.x) dst[e] = reinterpret_cast<const float4 *>(smr)[e];
    } else {
        char * head = g.k + roff + (unsigned long long) h * head_bytes(KT, D);
        for (int bb = wid; bb < nb; bb += nw) store_block_warp<KT>(smr[bb * 32 + lane], lane, head, bb, nb);
    }
}

// The prefill path over whole token rows (bf16 in, no norm): one block of ROPE_THR threads per token.  cos / sin of a rotary
// pair depend on the token and the pair only, so they are computed once per token instead of once per head (same
// expressions, same values); q rows move as 16-byte loads / 32-byte stores; the K heads are rotated in shared memory and
// every warp then quantises 32-value blocks of K and V.  Needs n_rot % 16 == 0 and 16-byte aligned rows.
__device__ __forceinline__ void bf16x8_to_f32(const uint4 u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { f[2 * e] = __uint_as_float(w[e] << 16); f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u); }
}
#ifndef ROPE_THR
#define ROPE_THR 128
#endif
template <uint32_t KT>
__global__ void __launch_bounds__(ROPE_THR) rope_rows_k(const __nv_bfloat16 * __restrict__ qg, const __nv_bfloat16 * __restrict__ k,
                                                   const __nv_bfloat16 * __restrict__ v, float * __restrict__ q, kv_view g, int p0,
                                                   int Hq, int Hkv, int D, int n_rot, float freq_base, unsigned * status) {
    extern __shared__ float smr[];   // cos[half] | sin[half] | K heads [Hkv][D]
    const int t = blockIdx.x, i = threadIdx.x, half = n_rot / 2, lane = i & 31, wid = i >> 5, nb = D / 32;
    float * cs = smr, * kb = smr + n_rot;
    const int ppos = p0 + t;
    for (int j = i; j < half; j += ROPE_THR) {
        const float theta = (float) ppos * powf(freq_base, -2.0f * j / n_rot);
        cs[j] = cosf(theta);
        cs[half + j] = sinf(theta);
    }
    for (int e = i; e < Hkv * D / 8; e += ROPE_THR) {
        float f[8];
        bf16x8_to_f32(__ldg(reinterpret_cast<const uint4 *>(k + (size_t) t * Hkv * D) + e), f);
        reinterpret_cast<float4 *>(kb)[2 * e] = make_float4(f[0], f[1], f[2], f[3]);
        reinterpret_cast<float4 *>(kb)[2 * e + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
    // the dims past n_rot of every q head are converted and copied first: they need no cos / sin, so this traffic (most of the
    // row) runs while the first warp is still busy with the trigonometry
    const int PI = half / 8, CI = (D - n_rot) / 8;   // per head: items of 8 rotary pairs, items of 8 plain values
    if (qg) {
        for (int it = i; it < Hq * CI; it += ROPE_THR) {
            const int h = it / CI, d0 = n_rot + (it - h * CI) * 8;
            float a[8];
            bf16x8_to_f32(__ldg(reinterpret_cast<const uint4 *>(qg + ((size_t) t * Hq + h) * D + d0)), a);
            float * dst = q + ((size_t) t * Hq + h) * D + d0;
            reinterpret_cast<float4 *>(dst)[0] = make_float4(a[0], a[1], a[2], a[3]);
            reinterpret_cast<float4 *>(dst)[1] = make_float4(a[4], a[5], a[6], a[7]);
        }
    }
    __syncthreads();
    if (qg) {
        for (int it = i; it < Hq * PI; it += ROPE_THR) {
            const int h = it / PI, d0 = (it - h * PI) * 8;
            const __nv_bfloat16 * src = qg + ((size_t) t * Hq + h) * D;
            float * dst = q + ((size_t) t * Hq + h) * D;
            float a[8], b[8], y0[8], y1[8];
            bf16x8_to_f32(__ldg(reinterpret_cast<const uint4 *>(src + d0)), a);
            bf16x8_to_f32(__ldg(reinterpret_cast<const uint4 *>(src + d0 + half)), b);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float c = cs[d0 + e], sn = cs[half + d0 + e];
                rot_pair(a[e], b[e], c, sn, y0[e], y1[e]);
            }
            reinterpret_cast<float4 *>(dst + d0)[0] = make_float4(y0[0], y0[1], y0[2], y0[3]);
            reinterpret_cast<float4 *>(dst + d0)[1] = make_float4(y0[4], y0[5], y0[6], y0[7]);
            reinterpret_cast<float4 *>(dst + d0 + half)[0] = make_float4(y1[0], y1[1], y1[2], y1[3]);
            reinterpret_cast<float4 *>(dst + d0 + half)[1] = make_float4(y1[4], y1[5], y1[6], y1[7]);
        }
    }
    for (int e = i; e < Hkv * half; e += ROPE_THR) {
        const int h = e / half, j = e - h * half;
        const float c = cs[j], sn = cs[half + j];
        rot_pair(kb[h * D + j], kb[h * D + j + half], c, sn, kb[h * D + j], kb[h * D + j + half]);
    }
    __syncthreads();
    const int row = p0 + t;
    const int32_t * tab = kv_tab(g, t);
    if (tab && tab[row >> g.psh] < 0) { if (i == 0) atomicOr(status, ST_BAD_PAGE); return; }
    const unsigned long long roff = kv_off_tab(g, tab, row);
    for (int bb = wid; bb < Hkv * nb; bb += ROPE_THR / 32) {
        const int h = bb / nb, b = bb - h * nb;
        const unsigned long long ho = roff + (unsigned long long) h * head_bytes(KT, D);
        store_block_warp<KT>(kb[bb * 32 + lane], lane, g.k + ho, b, nb);
        store_block_warp<KT>(__bfloat162float(v[(size_t) t * Hkv * D + bb * 32 + lane]), lane, g.v + ho, b, nb);
    }
}

// --------------------------------------------------------------------------------------------------- filler ----
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}
// one thread per 16-bit word of the rows p0..p1-1 (all kv heads), K and V
__global__ void fill_random_k(kv_view g, uint32_t type, int D, int p0, int p1, uint32_t seed) {
    const int hw = head_bytes(type, D) / 2, roww = hw * g.Hkv;
    const size_t n = (size_t) (p1 - p0) * roww;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t) gridDim.x * blockDim.x) {
        const int p = p0 + (int) (i / roww), w = (int) (i % roww), wh = w % hw;
        const uint32_t h = mix32((uint32_t) (p * 2654435761u) ^ mix32((uint32_t) w + seed));
        uint16_t a, b;
        if (type == B200_KV_F16) {
            a = __half_as_ushort(__float2half((float) (h & 0xffff) / 32768.0f - 1.0f));
            b = __half_as_ushort(__float2half((float) (h >> 16) / 32768.0f - 1.0f));
        } else if ((type == B200_KV_Q8_0 && wh < D / 32) || (type == B200_KV_Q4_0 && wh % 9 == 0)) {
            a = b = __half_as_ushort(__float2half(type == B200_KV_Q8_0 ? 1.0f / 127.0f : 0.125f));
        } else {
            a = (uint16_t) h; b = (uint16_t) (h >> 16);
        }
        const unsigned long long o = kv_off_tab(g, kv_tab(g, 0), p) + (unsigned long long) w * 2;
        *reinterpret_cast<uint16_t *>(g.k + o) = a;
        *reinterpret_cast<uint16_t *>(g.v + o) = b;
    }
}

// ----------------------------------------------------------------------------------------------------- gate ----
__device__ __forceinline__ float sigm(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float silu(float v) { return v / (1.0f + expf(-v)); }

__global__ void sigmoid_mul_k(float * __restrict__ x, const float * __restrict__ gt, int64_t n) {
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x)
        x[i] *= sigm(gt[i]);
}

// y = op(a, b) over [T][n] with one float4 per thread; qbuf != nullptr also emits the a16 activation layout consumed by
// the next projection (reference: a16_quant8, src/fast/a16q.cuh:21-45): per 32 values amax (clamped to the largest
// finite half), the values divided by amax as 16 half2 in a fixed slot order, and (amax, sum) as a half2.
template <int OP>
__global__ void ew_k(const float * __restrict__ a, const float * __restrict__ b, float * __restrict__ y, __half2 * qbuf,
                     int n, int lda, int ldb) {
    const int n4 = n >> 2, t = blockIdx.y, T = gridDim.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const bool act = i < n4;
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (act) {
        const float4 av = reinterpret_cast<const float4 *>(a + (int64_t) t * lda)[i];
        const float4 bv = reinterpret_cast<const float4 *>(b + (int64_t) t * ldb)[i];
        if (OP == 0) { v[0] = silu(av.x) * bv.x; v[1] = silu(av.y) * bv.y; v[2] = silu(av.z) * bv.z; v[3] = silu(av.w) * bv.w; }
        else { v[0] = av.x * sigm(bv.x); v[1] = av.y * sigm(bv.y); v[2] = av.z * sigm(bv.z); v[3] = av.w * sigm(bv.w); }
        reinterpret_cast<float4 *>(y + (int64_t) t * n)[i] = make_float4(v[0], v[1], v[2], v[3]);
    }
    if (!qbuf) return;
    // 8 consecutive lanes own one 32-value group
    const int l = threadIdx.x & 7, ng = n >> 5, grp = i >> 3;
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int s = 4; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s, 8));
    amax = amax < 65520.0f ? amax : 65504.0f;
    const float id = amax > 0.0f ? 1.0f / amax : 0.0f;
    float sum = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e) { v[e] = __fmul_rn(v[e], id); sum = __fadd_rn(sum, v[e]); }
#pragma unroll
    for (int s = 4; s > 0; s >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, s, 8));
    if (!act) return;
    __half2 * qs = qbuf + ((size_t) t * ng + grp) * 16;
    __half2 * ads = qbuf + (size_t) T * ng * 16 + (size_t) t * ng + grp;
    if (l == 0) *ads = __halves2half2(__float2half(amax), __float2half(sum));
    const int off = l >= 4 ? 1 : 0, kk = l - 4 * off;
    qs[4 * kk + 0 + off] = __halves2half2(__float2half(v[0]), __float2half(v[2]));
    qs[4 * kk + 2 + off] = __halves2half2(__float2half(v[1]), __float2half(v[3]));
}

bool type_ok(uint32_t t) { return t == B200_KV_F16 || t == B200_KV_Q8_0 || t == B200_KV_Q4_0; }

int append_impl(const b200_kv_cache * c, const float * k, const float * v, int p0, const int32_t * p0p, int T, cudaStream_t s) {
    if (!c || !c->k || !c->v || !k || !v) B200_REFUSE(B200_ERR_SHAPE, "kv_append: null cache or input");
    if (!type_ok(c->type) || c->D <= 0 || c->D % 32 || c->Hkv <= 0) B200_REFUSE(B200_ERR_SHAPE, "kv_append: unsupported type %u / D %d / Hkv %d", c->type, c->D, c->Hkv);
    if (T <= 0) return B200_OK;
    if (!p0p && !c->pt && (p0 < 0 || p0 + T > c->n_ctx)) B200_REFUSE(B200_ERR_SHAPE, "kv_append: rows %d..%d outside n_ctx %d", p0, p0 + T - 1, c->n_ctx);
    unsigned * st = device_status_word();
    if (!st) return B200_ERR_CUDA;
    const kv_view g = view_of(*c);
    const int nblk = c->Hkv * c->D / 32;
    const dim3 grid((nblk + 7) / 8, T);
    if (c->type == B200_KV_F16) append_k<B200_KV_F16><<<grid, 256, 0, s>>>(k, v, g, p0, p0p, c->D, st);
    else if (c->type == B200_KV_Q8_0) append_k<B200_KV_Q8_0><<<grid, 256, 0, s>>>(k, v, g, p0, p0p, c->D, st);
    else append_k<B200_KV_Q4_0><<<grid, 256, 0, s>>>(k, v, g, p0, p0p, c->D, st);
    count_launch();
    return launch_status("kv_append");
}

template <typename TIN, bool NORM, bool SPLITQ>
int prep_launch(const TIN * qg, const TIN * k, const TIN * v, const float * qn, const float * kn, const int32_t * pos,
                float * q, float * gate, const b200_kv_cache * c, int p0, int T, int Hq, int Hkv, int D, int n_rot,
                float freq_base, float eps, cudaStream_t s, int ldq, int ldk, int ldv, const b200_mrope_pos * mr,
                const int32_t * crow = nullptr) {
    unsigned * st = device_status_word();
    if (!st) return B200_ERR_CUDA;
    const kv_view g = view_of(*c);
    const int thr = ((D / 4) + 31) & ~31;
    const dim3 grid(Hq + 2 * Hkv, T);
    const size_t smem = (size_t) D * sizeof(float);
    b200_mrope_pos m{};
    const bool use_mr = mr && mr->p;
    if (use_mr) m = *mr;
#define PREP(KT_) do { if (use_mr) prep_k<KT_, TIN, NORM, SPLITQ, true><<<grid, thr, smem, s>>>(qg, k, v, qn, kn, pos, q, gate, g, p0, Hq, Hkv, D, n_rot, freq_base, eps, ldq, ldk, ldv, m, crow, st); \
                      else prep_k<KT_, TIN, NORM, SPLITQ, false><<<grid, thr, smem, s>>>(qg, k, v, qn, kn, pos, q, gate, g, p0, Hq, Hkv, D, n_rot, freq_base, eps, ldq, ldk, ldv, m, crow, st); } while (0)
    if (c->type == B200_KV_F16) PREP(B200_KV_F16);
    else if (c->type == B200_KV_Q8_0) PREP(B200_KV_Q8_0);
    else PREP(B200_KV_Q4_0);
#undef PREP
    count_launch();
    return launch_status("attn_prep");
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_kv_row_bytes(uint32_t type, int Hkv, int D) { return (size_t) Hkv * head_bytes(type, D); }

int b200_kv_alloc(b200_kv_cache * out, uint32_t type, int n_ctx, int Hkv, int D) {
    if (!out) return B200_ERR_SHAPE;
    memset(out, 0, sizeof *out);
    out->type = type; out->n_ctx = n_ctx; out->Hkv = Hkv; out->D = D;
    if (!type_ok(type) || (type != B200_KV_F16 && D % 32) || n_ctx <= 0 || Hkv <= 0 || D <= 0) B200_REFUSE(B200_ERR_SHAPE, "kv_alloc: unsupported type %u / shape", type);
    const size_t bytes = b200_kv_row_bytes(type, Hkv, D) * (size_t) n_ctx;
    if (cudaMalloc(&out->k, bytes) != cudaSuccess || cudaMalloc(&out->v, bytes) != cudaSuccess) {
        cudaGetLastError();
        b200_kv_free(out);
        B200_REFUSE(B200_ERR_ALLOC, "kv_alloc: %zu bytes x 2 could not be allocated", bytes);
    }
    return B200_OK;
}

void b200_kv_free(b200_kv_cache * c) {
    if (!c) return;
    if (c->k) cudaFree(c->k);
    if (c->v) cudaFree(c->v);
    c->k = c->v = nullptr;
}

int b200_kv_fill_random(const b200_kv_cache * c, int p0, int p1, uint32_t seed, void * stream) {
    if (!c || !c->k || !c->v || !type_ok(c->type) || c->D % 32) B200_REFUSE(B200_ERR_SHAPE, "kv_fill_random: unsupported cache");
    if (p1 <= p0) return B200_OK;
    fill_random_k<<<1184, 256, 0, (cudaStream_t) stream>>>(view_of(*c), c->type, c->D, p0, p1, seed);
    count_launch();
    return launch_status("kv_fill_random");
}

int b200_kv_append(const b200_kv_cache * c, const float * k, const float * v, int p0, int T, void * stream) {
    return append_impl(c, k, v, p0, nullptr, T, (cudaStream_t) stream);
}
int b200_kv_append_dev(const b200_kv_cache * c, const float * k, const float * v, const int32_t * p0_dev, int T, void * stream) {
    if (!p0_dev) B200_REFUSE(B200_ERR_SHAPE, "kv_append_dev: p0_dev is null");
    return append_impl(c, k, v, 0, p0_dev, T, (cudaStream_t) stream);
}

int b200_attn_prep(const float * qg, const float * k, const float * v, const float * q_norm, const float * k_norm,
                   const int32_t * pos, float * q, float * gate, const b200_kv_cache * c, int p0, int T, int Hq, int Hkv,
                   int D, int n_rot, float freq_base, float eps, void * stream, int ldq, int ldk, int ldv,
                   const b200_mrope_pos * mr) {
    if (T <= 0) return B200_OK;
    if (ldq <= 0) ldq = Hq * 2 * D;
    if (ldk <= 0) ldk = Hkv * D;
    if (ldv <= 0) ldv = Hkv * D;
    if (!c || !qg || !k || !v || !pos || !q || !gate) B200_REFUSE(B200_ERR_SHAPE, "attn_prep: null argument");
    if (ldq < Hq * 2 * D || ldk < Hkv * D || ldv < Hkv * D || ldq % 4 || ldk % 4) B200_REFUSE(B200_ERR_SHAPE, "attn_prep: bad row strides");
    if (!type_ok(c->type) || !c->k || c->D != D || c->Hkv != Hkv || D % 128 || D > 1024 || n_rot > D || n_rot % 2 ||
        !aligned16(qg) || !aligned16(k) || !aligned16(q) || !aligned16(gate) || (q_norm && !aligned16(q_norm)) ||
        (k_norm && !aligned16(k_norm)) || (p0 >= 0 && !c->pt && p0 + T > c->n_ctx))
        B200_REFUSE(B200_ERR_SHAPE, "attn_prep: unsupported shape / cache / alignment (D=%d Hkv=%d n_rot=%d)", D, Hkv, n_rot);
    if (mr && mr->p && mr->sect <= 0) B200_REFUSE(B200_ERR_SHAPE, "attn_prep: M-RoPE sections sum to 0");
    return prep_launch<float, true, true>(qg, k, v, q_norm, k_norm, pos, q, gate, c, p0, T, Hq, Hkv, D, n_rot, freq_base,
                                          eps, (cudaStream_t) stream, ldq, ldk, ldv, mr);
}

int b200_attn_prep_rows(const float * qg, const float * k, const float * v, const float * q_norm, const float * k_norm,
                        const int32_t * rope_pos, const int32_t * cache_row, float * q, float * gate, const b200_kv_cache * c,
                        int T, int Hq, int Hkv, int D, int n_rot, float freq_base, float eps, void * stream) {
    if (T <= 0) return B200_OK;
    if (!c || !qg || !k || !v || !rope_pos || !cache_row || !q || !gate) B200_REFUSE(B200_ERR_SHAPE, "attn_prep_rows: null argument");
    if (!type_ok(c->type) || !c->k || c->D != D || c->Hkv != Hkv || D % 128 || D > 1024 || n_rot > D || n_rot % 2 ||
        !aligned16(qg) || !aligned16(k) || !aligned16(q) || !aligned16(gate) || (q_norm && !aligned16(q_norm)) ||
        (k_norm && !aligned16(k_norm)))
        B200_REFUSE(B200_ERR_SHAPE, "attn_prep_rows: unsupported shape / cache / alignment (D=%d Hkv=%d n_rot=%d)", D, Hkv, n_rot);
    return prep_launch<float, true, true>(qg, k, v, q_norm, k_norm, rope_pos, q, gate, c, -1, T, Hq, Hkv, D, n_rot, freq_base,
                                          eps, (cudaStream_t) stream, Hq * 2 * D, Hkv * D, Hkv * D, nullptr, cache_row);
}

int b200_rope_append_bf16(const uint16_t * q, const uint16_t * k, const uint16_t * v, float * q_out,
                          const b200_kv_cache * c, int p0, int T, int Hq, int Hkv, int D, int n_rot, float freq_base,
                          void * stream) {
    if (T <= 0) return B200_OK;
    if (!c || !k || !v || (q && !q_out)) B200_REFUSE(B200_ERR_SHAPE, "rope_append_bf16: null argument");
    if (!type_ok(c->type) || !c->k || c->D != D || c->Hkv != Hkv || D % 128 || D > 1024 || n_rot > D || n_rot % 2 || p0 < 0 ||
        (!c->pt && p0 + T > c->n_ctx) || (q_out && !aligned16(q_out)))
        B200_REFUSE(B200_ERR_SHAPE, "rope_append_bf16: unsupported shape / cache (D=%d Hkv=%d n_rot=%d p0=%d)", D, Hkv, n_rot, p0);
    const size_t smem = ((size_t) n_rot + (size_t) Hkv * D) * sizeof(float);
    if (n_rot % 16 == 0 && smem <= 48 * 1024 && aligned16(q) && aligned16(k) && aligned16(v)) {   // whole-row kernel
        unsigned * st = device_status_word();
        if (!st) return B200_ERR_CUDA;
        const kv_view g = view_of(*c);
        const __nv_bfloat16 * qb = (const __nv_bfloat16 *) q, * kb = (const __nv_bfloat16 *) k, * vb = (const __nv_bfloat16 *) v;
        cudaStream_t s = (cudaStream_t) stream;
        if (c->type == B200_KV_F16) rope_rows_k<B200_KV_F16><<<T, ROPE_THR, smem, s>>>(qb, kb, vb, q_out, g, p0, Hq, Hkv, D, n_rot, freq_base, st);
        else if (c->type == B200_KV_Q8_0) rope_rows_k<B200_KV_Q8_0><<<T, ROPE_THR, smem, s>>>(qb, kb, vb, q_out, g, p0, Hq, Hkv, D, n_rot, freq_base, st);
        else rope_rows_k<B200_KV_Q4_0><<<T, ROPE_THR, smem, s>>>(qb, kb, vb, q_out, g, p0, Hq, Hkv, D, n_rot, freq_base, st);
        count_launch();
        return launch_status("rope_append_bf16");
    }
    return prep_launch<__nv_bfloat16, false, false>((const __nv_bfloat16 *) q, (const __nv_bfloat16 *) k, (const __nv_bfloat16 *) v,
                                                    nullptr, nullptr, nullptr, q_out, nullptr, c, p0, T, Hq, Hkv, D, n_rot,
                                                    freq_base, 0.0f, (cudaStream_t) stream, Hq * D, Hkv * D, Hkv * D, nullptr);
}

int b200_sigmoid_mul(float * x, const float * g, int64_t n, void * stream) {
    if (n <= 0) return B200_OK;
    if (!x || !g) B200_REFUSE(B200_ERR_SHAPE, "sigmoid_mul: null argument");
    const int64_t blocks = (n + 255) / 256;
    sigmoid_mul_k<<<(unsigned) (blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, (cudaStream_t) stream>>>(x, g, n);
    count_launch();
    return launch_status("sigmoid_mul");
}

int b200_ew_quant(int op, const float * a, const float * b, float * y, void * qbuf, int T, int n, void * stream, int lda, int ldb) {
    if (T <= 0 || n <= 0) return B200_OK;
    if (lda <= 0) lda = n;
    if (ldb <= 0) ldb = n;
    if ((op != 0 && op != 1) || n % 32 || !a || !b || !y || !aligned16(a) || !aligned16(b) || !aligned16(y) || lda < n || ldb < n ||
        lda % 4 || ldb % 4 || (T > 1 && y == a && lda != n))
        B200_REFUSE(B200_ERR_SHAPE, "ew_quant: unsupported op / shape / alignment");
    const int thr = 128;
    const dim3 grid((unsigned) ((n / 4 + thr - 1) / thr), (unsigned) T);
    if (op == 0) ew_k<0><<<grid, thr, 0, (cudaStream_t) stream>>>(a, b, y, (__half2 *) qbuf, n, lda, ldb);
    else ew_k<1><<<grid, thr, 0, (cudaStream_t) stream>>>(a, b, y, (__half2 *) qbuf, n, lda, ldb);
    count_launch();
    return launch_status("ew_quant");
}

int b200_last_device_status(void * stream) {
    unsigned * st = device_status_word();
    if (!st) return -1;
    unsigned h = 0;
    if (cudaStreamSynchronize((cudaStream_t) stream) != cudaSuccess) return -1;
    if (cudaMemcpy(&h, st, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (h) cudaMemset(st, 0, 4);
    return (int) h;
}

uint64_t b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
const char * b200_version(void) { return "b200attn 0.1 (sm_100a)"; }

}  // extern "C"
