// KV append, attention input prep (norm + partial RoPE + quantise + append), cache fillers and the sigmoid gate.
//
// Cache bytes are fixed by the reference's formats and fp32 recipes (src/fast/kv_q8.cuh:20-49, src/fast/attn.cu:245-283 in
// the reference project): every position written here is byte-identical to what the reference writes for the same inputs,
// paged or contiguous.  The kernels are organised per token, not per head: one CTA takes a whole token row, computes the
// token's cos / sin once, and its warps walk the row's heads (query heads with their gate halves, K heads, V heads), each
// head staying inside one warp from the load to the cache bytes, so nothing but the cos / sin table crosses a block barrier.
#include "common.cuh"

#include <cuda_bf16.h>
#include <algorithm>
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
// One full warp turns 32 consecutive values (lane = value index) of block b of a head row into cache bytes.
// The block statistics come from the warp-wide integer reductions of the hardware (one instruction each): |x| of finite
// floats orders like its bit pattern, so the q8_0 maximum is a redux.max of the bits, and the q4_0 pick (largest
// magnitude, lowest index on ties) is that maximum followed by a redux.min over the lanes that hold it.
template <uint32_t KT>
__device__ __forceinline__ void block_to_cache(float x, int lane, char * head, int b, int nb) {
    if constexpr (KT == B200_KV_F16) {
        reinterpret_cast<__half *>(head)[b * 32 + lane] = __float2half(x);
    } else {
        const unsigned mag = __float_as_uint(fabsf(x));
        const unsigned top = __reduce_max_sync(0xffffffffu, mag);
        if constexpr (KT == B200_KV_Q8_0) {
            float id;
            const float d = q8_scale(__uint_as_float(top), id);
            reinterpret_cast<int8_t *>(head + nb * 2)[b * 32 + lane] = (int8_t) q8_quant(x, id);
            if (lane == 0) reinterpret_cast<__half *>(head)[b] = __float2half(d);
        } else {
            const unsigned who = __reduce_min_sync(0xffffffffu, mag == top ? (unsigned) lane : 32u);
            const float pick = __shfl_sync(0xffffffffu, x, (int) (who & 31u));
            const float mx = top ? pick : 0.0f;   // the signed value of the pick (0 for an all-zero block)
            const float d = mx / -8.0f;
            const float id = d != 0.0f ? 1.0f / d : 0.0f;
            const unsigned q = (unsigned) q4_quant(x, id);
            // byte i = value i | value i+16 << 4; neighbouring bytes leave as one 16-bit store (the block's bytes start at +2)
            const unsigned byte = q | (__shfl_down_sync(0xffffffffu, q, 16) << 4);
            const unsigned pair = byte | (__shfl_down_sync(0xffffffffu, byte, 1) << 8);
            char * blk = head + b * 18;
            if (lane < 16 && !(lane & 1)) *reinterpret_cast<uint16_t *>(blk + 2 + lane) = (uint16_t) pair;
            if (lane == 0) *reinterpret_cast<__half *>(blk) = __float2half(d);
        }
    }
}

__device__ __forceinline__ float lanes_sum(float v) {   // xor butterfly, distances 16 .. 1: the order the cache bytes were defined with
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// rotary position of pair j of row t when the positions come as three interleaved streams (t, h, w); semantics of the
// reference's mrope_pick (src/fast/mrope.cuh:23-31): section = j mod sect picks stream section mod 3 while that stream still
// has sections left (section < 3 * count), else position 0
__device__ __forceinline__ int mrope_position(const b200_mrope_pos & m, int t, int j) {
    const int section = j % m.sect, stream = section % 3;
    const int count = stream == 0 ? m.s0 : stream == 1 ? m.s1 : m.s2;
    return section < 3 * count ? m.p[stream * m.stride + t] : 0;
}

// ------------------------------------------------------------------------------------------- per-token kernel ----
struct tok_args {
    const float * qg; const float * k; const float * v;     // activations (qg: per head D query values then D gate logits)
    const float * qn; const float * kn;                     // RMSNorm weights
    const int32_t * pos;                                    // rotary positions (device) or nullptr for p0 + t
    const int32_t * crow;                                   // explicit cache rows (< 0: not stored here) or nullptr
    const int32_t * p0p;                                    // device first position (append_dev) or nullptr
    float * q; float * gate;
    kv_view g;
    int p0, Hq, Hkv, D, n_rot;
    float freq_base, eps;
    int ldq, ldk, ldv;
    b200_mrope_pos mr;
    unsigned * status;
};
constexpr int TOK_WARPS = 8;
constexpr int MAXF4 = 8;   // float4 per lane of one head: D <= 1024

// PREP: attention input prep of the decode path (reference semantics: attn_prep_k, src/fast/fused.cu:502-573): per q head
// the gate half is copied out and q = rope(rmsnorm(q) * q_norm); per K head the same norm and rotation, then the cache bytes;
// V heads go to the cache as they are.  !PREP: plain append of k, v rows (reference: kv_append, src/fast/attn.cu:245-283).
// One CTA per token, one head per warp at a time.  The sum of squares keeps the defining order: per group of four values
// x0*x0 + x1*x1 + x2*x2 + x3*x3, a 32-lane butterfly over every 32 consecutive groups, then the butterfly of those results.
template <uint32_t KT, bool PREP, bool MR>
__global__ void __launch_bounds__(TOK_WARPS * 32) token_k(const tok_args a) {
    extern __shared__ float sm[];   // cos[half] | sin[half] | TOK_WARPS staged heads of D floats
    const int t = blockIdx.x, lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int D = a.D, nb = D / 32, nf = D / 128, half = a.n_rot / 2;
    float * cs = sm, * st = sm + a.n_rot + w * D;
    int row;
    if constexpr (PREP) {
        const int ppos = a.pos ? a.pos[t] : a.p0 + t;
        row = a.crow ? a.crow[t] : a.p0 < 0 ? ppos : a.p0 + t;
        for (int j = threadIdx.x; j < half; j += TOK_WARPS * 32) {
            float theta;
            if constexpr (MR) theta = (float) mrope_position(a.mr, t, j) * powf(a.freq_base, -2.0f * j / a.n_rot);
            else theta = (float) ppos * powf(a.freq_base, -2.0f * j / a.n_rot);
            cs[j] = cosf(theta);
            cs[half + j] = sinf(theta);
        }
        __syncthreads();
    } else {
        row = (a.p0p ? *a.p0p : a.p0) + t;
    }
    unsigned long long roff = 0;
    bool stored = row >= 0;
    if (stored) {
        const int32_t * tab = kv_tab(a.g, t);
        if (tab && tab[row >> a.g.psh] < 0) { if (threadIdx.x == 0) atomicOr(a.status, ST_BAD_PAGE); stored = false; }
        else roff = kv_off_tab(a.g, tab, row);
    }
    const int n_q = PREP && a.qg ? a.Hq : 0;
    for (int it = w; it < n_q + 2 * a.Hkv; it += TOK_WARPS) {
        const bool is_q = it < n_q, is_v = it >= n_q + a.Hkv;
        const int h = is_q ? it : is_v ? it - n_q - a.Hkv : it - n_q;
        if (!is_q && !stored) continue;
        char * head = (is_v ? a.g.v : a.g.k) + roff + (unsigned long long) h * head_bytes(KT, D);
        if (is_v || !PREP) {   // no norm, no rotation: 32 values per step straight from the activations
            const float * src = is_v ? a.v + (size_t) t * a.ldv + (size_t) h * D : a.k + (size_t) t * a.ldk + (size_t) h * D;
            float x[MAXF4 * 4];
#pragma unroll
            for (int b = 0; b < MAXF4 * 4; ++b) if (b < nb) x[b] = src[b * 32 + lane];
#pragma unroll
            for (int b = 0; b < MAXF4 * 4; ++b) if (b < nb) block_to_cache<KT>(x[b], lane, head, b, nb);
            continue;
        }
        if constexpr (PREP) {
            const float4 * src = reinterpret_cast<const float4 *>(is_q ? a.qg + (size_t) t * a.ldq + (size_t) h * 2 * D
                                                                       : a.k + (size_t) t * a.ldk + (size_t) h * D);
            float4 x[MAXF4];
#pragma unroll
            for (int j = 0; j < MAXF4; ++j) if (j < nf) x[j] = src[lane + 32 * j];
            if (is_q) {   // the gate half of the head moves on unchanged
                float4 * gd = reinterpret_cast<float4 *>(a.gate + ((size_t) t * a.Hq + h) * D);
#pragma unroll
                for (int j = 0; j < MAXF4; ++j) if (j < nf) gd[lane + 32 * j] = src[D / 4 + lane + 32 * j];
            }
            float part[MAXF4];
#pragma unroll
            for (int j = 0; j < MAXF4; ++j) {
                float ss = 0.0f;
                if (j < nf) ss += x[j].x * x[j].x + x[j].y * x[j].y + x[j].z * x[j].z + x[j].w * x[j].w;
                part[j] = lanes_sum(ss);
            }
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) {   // the butterfly of the per-32-group results (absent groups count as 0)
                float nx[MAXF4];
#pragma unroll
                for (int j = 0; j < MAXF4; ++j) nx[j] = part[j] + part[j ^ o];
#pragma unroll
                for (int j = 0; j < MAXF4; ++j) part[j] = nx[j];
            }
            const float sc = rsqrtf(part[0] / D + a.eps);
            const float4 * wt = reinterpret_cast<const float4 *>(is_q ? a.qn : a.kn);
#pragma unroll
            for (int j = 0; j < MAXF4; ++j)
                if (j < nf) {
                    float4 o = x[j];
                    o.x *= sc; o.y *= sc; o.z *= sc; o.w *= sc;
                    if (wt) { const float4 ww = wt[lane + 32 * j]; o.x *= ww.x; o.y *= ww.y; o.z *= ww.z; o.w *= ww.w; }
                    reinterpret_cast<float4 *>(st)[lane + 32 * j] = o;
                }
            __syncwarp();
            for (int j = lane; j < half; j += 32) rot_pair(st[j], st[j + half], cs[j], cs[half + j], st[j], st[j + half]);
            __syncwarp();
            if (is_q) {
                float4 * dst = reinterpret_cast<float4 *>(a.q + ((size_t) t * a.Hq + h) * D);
#pragma unroll
                for (int j = 0; j < MAXF4; ++j) if (j < nf) dst[lane + 32 * j] = reinterpret_cast<const float4 *>(st)[lane + 32 * j];
            } else {
                for (int b = 0; b < nb; ++b) block_to_cache<KT>(st[b * 32 + lane], lane, head, b, nb);
            }
            __syncwarp();   // the staged head is reused by this warp's next item
        }
    }
}

// The prefill path over whole token rows (bf16 in, no norm): one block of ROPE_THR threads per token.  cos / sin of a rotary
// pair depend on the token and the pair only, so they are computed once per token instead of once per head (same
// expressions, same values); q rows move as 16-byte loads / 32-byte stores; the K heads are rotated in shared memory and
// every warp then quantises 32-value blocks of K and V.  Needs n_rot % 16 == 0; rows that are not 16-byte aligned are
// read element by element.
// cs_out != nullptr: the token's table (cos[half] | sin[half]) is also written to cs_out[t * n_rot ..] for the attention
// kernel that rotates the bf16 query rows itself.
__device__ __forceinline__ void bf16x8_to_f32(const uint4 u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { f[2 * e] = __uint_as_float(w[e] << 16); f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u); }
}
// eight consecutive bf16 values: one 16-byte load when the rows are 16-byte aligned, element loads otherwise (same values)
__device__ __forceinline__ void ld_bf16x8(const __nv_bfloat16 * p, bool vec, float (&f)[8]) {
    if (vec) { bf16x8_to_f32(__ldg(reinterpret_cast<const uint4 *>(p)), f); return; }
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = __bfloat162float(p[e]);
}
#ifndef ROPE_THR
#define ROPE_THR 128
#endif
template <uint32_t KT>
__global__ void __launch_bounds__(ROPE_THR) rope_rows_k(const __nv_bfloat16 * __restrict__ qg, const __nv_bfloat16 * __restrict__ k,
                                                   const __nv_bfloat16 * __restrict__ v, float * __restrict__ q, float * __restrict__ cs_out,
                                                   kv_view g, int p0, int rope0, int Hq, int Hkv, int D, int n_rot, float freq_base,
                                                   int vec, unsigned * status) {
    extern __shared__ float smr[];   // cos[half] | sin[half] | K heads [Hkv][D]
    const int t = blockIdx.x, i = threadIdx.x, half = n_rot / 2, lane = i & 31, wid = i >> 5, nb = D / 32;
    float * cs = smr, * kb = smr + n_rot;
    const int ppos = rope0 + t;   // the angle's position; the cache row is p0 + t (they differ on a sequence shard)
    for (int j = i; j < half; j += ROPE_THR) {
        const float theta = (float) ppos * powf(freq_base, -2.0f * j / n_rot);
        const float c = cosf(theta), sn = sinf(theta);
        cs[j] = c;
        cs[half + j] = sn;
        if (cs_out) { cs_out[(size_t) t * n_rot + j] = c; cs_out[(size_t) t * n_rot + half + j] = sn; }
    }
    for (int e = i; k && e < Hkv * D / 8; e += ROPE_THR) {
        float f[8];
        ld_bf16x8(k + (size_t) t * Hkv * D + (size_t) e * 8, vec, f);
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
            ld_bf16x8(qg + ((size_t) t * Hq + h) * D + d0, vec, a);
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
            ld_bf16x8(src + d0, vec, a);
            ld_bf16x8(src + d0 + half, vec, b);
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
    if (!k) return;   // q only
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
        block_to_cache<KT>(kb[bb * 32 + lane], lane, g.k + ho, b, nb);
        block_to_cache<KT>(__bfloat162float(v[(size_t) t * Hkv * D + bb * 32 + lane]), lane, g.v + ho, b, nb);
    }
}

// -------------------------------------------------------------------------------------------------- fillers ----
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}
// the K and V 16-bit words number wh of a head row, from one hash: finite values, scales 1/127 (q8_0) or 1/8 (q4_0)
__device__ __forceinline__ void filler_words(uint32_t type, int D, int wh, uint32_t h, uint16_t & a, uint16_t & b) {
    if (type == B200_KV_F16) {
        a = __half_as_ushort(__float2half((float) (h & 0xffff) / 32768.0f - 1.0f));
        b = __half_as_ushort(__float2half((float) (h >> 16) / 32768.0f - 1.0f));
    } else if ((type == B200_KV_Q8_0 && wh < D / 32) || (type == B200_KV_Q4_0 && wh % 9 == 0)) {
        a = b = __half_as_ushort(__float2half(type == B200_KV_Q8_0 ? 1.0f / 127.0f : 0.125f));
    } else {
        a = (uint16_t) h; b = (uint16_t) (h >> 16);
    }
}
// one thread per 16-bit word of the rows p0..p1-1 (all kv heads), K and V (reference: kv_fill_random, src/fast/attn.cu:559-581)
__global__ void fill_random_k(kv_view g, uint32_t type, int D, int p0, int p1, uint32_t seed) {
    const int hw = head_bytes(type, D) / 2, roww = hw * g.Hkv;
    const size_t n = (size_t) (p1 - p0) * roww;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t) gridDim.x * blockDim.x) {
        const int p = p0 + (int) (i / roww), w = (int) (i % roww), wh = w % hw;
        const uint32_t h = mix32((uint32_t) (p * 2654435761u) ^ mix32((uint32_t) w + seed));
        uint16_t a, b;
        filler_words(type, D, wh, h, a, b);
        const unsigned long long o = kv_off_tab(g, kv_tab(g, 0), p) + (unsigned long long) w * 2;
        *reinterpret_cast<uint16_t *>(g.k + o) = a;
        *reinterpret_cast<uint16_t *>(g.v + o) = b;
    }
}
// Fill the sequences of a paged pool so that the contents depend on (seed, slot, global position, global kv head) only,
// not on where the rows live: two differently sharded pools (kv heads split over ranks, pages of a sequence dealt
// round-robin over n_seq sequence shards) hold the same values for the same (slot, position, head).  Slot s owns
// len[s] local positions through the table row pt + s * table_stride; local position lp = (page lpg, offset o) is global
// position ((lpg * n_seq + seq_rank) << psh) + o.  grid (x, slot).
__global__ void fill_slots_k(kv_view g, uint32_t type, int D, const int32_t * __restrict__ len, int table_stride, uint32_t seed,
                             int head0, int n_seq, int seq_rank) {
    const int s = blockIdx.y, hw = head_bytes(type, D) / 2, roww = hw * g.Hkv;
    const int32_t * tab = g.pt + (size_t) s * table_stride;
    const size_t n = (size_t) len[s] * roww;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t) gridDim.x * blockDim.x) {
        const int lp = (int) (i / roww), w = (int) (i % roww), hd = w / hw, wh = w - hd * hw;
        const int gp = (((lp >> g.psh) * n_seq + seq_rank) << g.psh) + (lp & ((1 << g.psh) - 1));
        const uint32_t h = mix32((uint32_t) gp * 2654435761u ^ mix32((uint32_t) ((head0 + hd) * hw + wh) + seed) ^
                                 mix32((uint32_t) s * 0x9e3779b9u + 0x85ebca6bu));
        uint16_t a, b;
        filler_words(type, D, wh, h, a, b);
        const unsigned long long o = kv_off_tab(g, tab, lp) + (unsigned long long) w * 2;
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

// y = op(a, b) over [T][n]; qbuf != nullptr also writes the a16 copy (see a16_store_lanes8).  Warps walk the (row, 128-value
// segment) items of the whole problem with a grid stride, one float4 per lane, so any T x n fills the machine the same way.
template <int OP>
__global__ void __launch_bounds__(256) ew_k(const float * __restrict__ a, const float * __restrict__ b, float * __restrict__ y,
                                            __half2 * __restrict__ qbuf, int T, int n, int lda, int ldb) {
    const int n4 = n >> 2, segs = (n4 + 31) >> 5, lane = threadIdx.x & 31;
    const long long items = (long long) T * segs, stride = (long long) gridDim.x * (blockDim.x >> 5);
    for (long long it = (long long) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); it < items; it += stride) {
        const int t = (int) (it / segs), i = (int) (it - (long long) t * segs) * 32 + lane;
        const bool live = i < n4;
        float4 r = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (live) {
            const float4 av = reinterpret_cast<const float4 *>(a + (int64_t) t * lda)[i];
            const float4 bv = reinterpret_cast<const float4 *>(b + (int64_t) t * ldb)[i];
            if (OP == 0) r = make_float4(silu(av.x) * bv.x, silu(av.y) * bv.y, silu(av.z) * bv.z, silu(av.w) * bv.w);
            else r = make_float4(av.x * sigm(bv.x), av.y * sigm(bv.y), av.z * sigm(bv.z), av.w * sigm(bv.w));
            reinterpret_cast<float4 *>(y + (int64_t) t * n)[i] = r;
        }
        if (qbuf) a16_store_lanes8(r, qbuf, (size_t) t * (n >> 5) + (i >> 3), (size_t) T * (n >> 5), live);
    }
}

bool type_ok(uint32_t t) { return t == B200_KV_F16 || t == B200_KV_Q8_0 || t == B200_KV_Q4_0; }

template <bool PREP>
int token_launch(const tok_args & a, uint32_t type, int T, bool mrope, cudaStream_t s, const char * who) {
    const size_t smem = ((size_t) a.n_rot + (size_t) TOK_WARPS * a.D) * sizeof(float);
#define TOKEN(KT_) do { if (PREP && mrope) token_k<KT_, PREP, PREP><<<T, TOK_WARPS * 32, smem, s>>>(a); \
                        else token_k<KT_, PREP, false><<<T, TOK_WARPS * 32, smem, s>>>(a); } while (0)
    if (type == B200_KV_F16) TOKEN(B200_KV_F16);
    else if (type == B200_KV_Q8_0) TOKEN(B200_KV_Q8_0);
    else TOKEN(B200_KV_Q4_0);
#undef TOKEN
    count_launch();
    return launch_status(who);
}

int append_impl(const b200_kv_cache * c, const float * k, const float * v, int p0, const int32_t * p0p, int T, cudaStream_t s) {
    if (!c || !c->k || !c->v || !k || !v) B200_REFUSE(B200_ERR_SHAPE, "kv_append: null cache or input");
    if (!type_ok(c->type) || c->D <= 0 || c->D % 32 || c->D > 1024 || c->Hkv <= 0) B200_REFUSE(B200_ERR_SHAPE, "kv_append: unsupported type %u / D %d / Hkv %d", c->type, c->D, c->Hkv);
    if (T <= 0) return B200_OK;
    if (!p0p && !c->pt && (p0 < 0 || p0 + T > c->n_ctx)) B200_REFUSE(B200_ERR_SHAPE, "kv_append: rows %d..%d outside n_ctx %d", p0, p0 + T - 1, c->n_ctx);
    tok_args a{};
    a.k = k; a.v = v; a.p0p = p0p; a.p0 = p0; a.g = view_of(*c);
    a.Hq = 0; a.Hkv = c->Hkv; a.D = c->D; a.n_rot = 0; a.ldk = a.ldv = c->Hkv * c->D;
    a.status = device_status_word();
    if (!a.status) return B200_ERR_CUDA;
    return token_launch<false>(a, c->type, T, false, s, "kv_append");
}

int prep_impl(const float * qg, const float * k, const float * v, const float * qn, const float * kn, const int32_t * pos,
              const int32_t * crow, float * q, float * gate, const b200_kv_cache * c, int p0, int T, int Hq, int Hkv, int D, int n_rot,
              float freq_base, float eps, cudaStream_t s, int ldq, int ldk, int ldv, const b200_mrope_pos * mr, const char * who) {
    tok_args a{};
    a.qg = qg; a.k = k; a.v = v; a.qn = qn; a.kn = kn; a.pos = pos; a.crow = crow; a.q = q; a.gate = gate;
    a.g = view_of(*c);
    a.p0 = p0; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.n_rot = n_rot; a.freq_base = freq_base; a.eps = eps;
    a.ldq = ldq; a.ldk = ldk; a.ldv = ldv;
    const bool mrope = mr && mr->p;
    if (mrope) a.mr = *mr;
    a.status = device_status_word();
    if (!a.status) return B200_ERR_CUDA;
    return token_launch<true>(a, c->type, T, mrope, s, who);
}

}  // namespace

// bf16 rows -> K rotated, K and V quantised into rows p0 + t; q (optional) rotated to fp32 q_out; cs_out (optional) receives
// the tokens' cos / sin table.  Shared by b200_rope_append_bf16 and the bf16 prefill entry point.
int rope_append_launch(const uint16_t * q, const uint16_t * k, const uint16_t * v, float * q_out, float * cs_out, const b200_kv_cache * c,
                       int p0, int T, int Hq, int Hkv, int D, int n_rot, float freq_base, cudaStream_t s, const char * who, int rope0) {
    if (T <= 0) return B200_OK;
    if (rope0 < 0) rope0 = p0;
    if (!c || (!k != !v) || (!k && !q) || (q && !q_out)) B200_REFUSE(B200_ERR_SHAPE, "%s: null argument", who);
    if (!type_ok(c->type) || !c->k || c->D != D || c->Hkv != Hkv || D % 128 || D > 1024 || n_rot > D || n_rot % 16 || p0 < 0 ||
        (!c->pt && p0 + T > c->n_ctx) || (q_out && !aligned16(q_out)))
        B200_REFUSE(B200_ERR_SHAPE, "%s: unsupported shape / cache / alignment (D=%d Hkv=%d n_rot=%d p0=%d; n_rot must be a multiple of 16)", who, D, Hkv, n_rot, p0);
    const int vec = aligned16(q) && aligned16(k) && aligned16(v) ? 1 : 0;
    const size_t smem = ((size_t) n_rot + (size_t) Hkv * D) * sizeof(float);
    if (smem > 48 * 1024) B200_REFUSE(B200_ERR_SHAPE, "%s: Hkv * D too large for one token block", who);
    unsigned * st = device_status_word();
    if (!st) return B200_ERR_CUDA;
    const kv_view g = view_of(*c);
    const __nv_bfloat16 * qb = (const __nv_bfloat16 *) q, * kb = (const __nv_bfloat16 *) k, * vb = (const __nv_bfloat16 *) v;
    if (c->type == B200_KV_F16) rope_rows_k<B200_KV_F16><<<T, ROPE_THR, smem, s>>>(qb, kb, vb, q_out, cs_out, g, p0, rope0, Hq, Hkv, D, n_rot, freq_base, vec, st);
    else if (c->type == B200_KV_Q8_0) rope_rows_k<B200_KV_Q8_0><<<T, ROPE_THR, smem, s>>>(qb, kb, vb, q_out, cs_out, g, p0, rope0, Hq, Hkv, D, n_rot, freq_base, vec, st);
    else rope_rows_k<B200_KV_Q4_0><<<T, ROPE_THR, smem, s>>>(qb, kb, vb, q_out, cs_out, g, p0, rope0, Hq, Hkv, D, n_rot, freq_base, vec, st);
    count_launch();
    return launch_status(who);
}

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

int b200_kv_fill_slots(const b200_kv_cache * c, int n_slots, const int32_t * len, int table_stride, uint32_t seed, int head0, int n_seq,
                       int seq_rank, void * stream) {
    if (!c || !c->k || !c->v || !c->pt || !len || !type_ok(c->type) || c->D % 32 || n_slots < 1 || n_slots > 65535 || table_stride < 1 ||
        n_seq < 1 || seq_rank < 0 || seq_rank >= n_seq || head0 < 0)
        B200_REFUSE(B200_ERR_SHAPE, "kv_fill_slots: unsupported cache / arguments (a paged cache is required)");
    fill_slots_k<<<dim3(64, (unsigned) n_slots), 256, 0, (cudaStream_t) stream>>>(view_of(*c), c->type, c->D, len, table_stride, seed, head0,
                                                                                  n_seq, seq_rank);
    count_launch();
    return launch_status("kv_fill_slots");
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
    if (!c || !k || !v || !pos || (qg && (!q || !gate))) B200_REFUSE(B200_ERR_SHAPE, "attn_prep: null argument");
    if (ldq < Hq * 2 * D || ldk < Hkv * D || ldv < Hkv * D || ldq % 4 || ldk % 4) B200_REFUSE(B200_ERR_SHAPE, "attn_prep: bad row strides");
    if (!type_ok(c->type) || !c->k || c->D != D || c->Hkv != Hkv || D % 128 || D > 1024 || n_rot > D || n_rot % 2 ||
        !aligned16(qg) || !aligned16(k) || !aligned16(q) || !aligned16(gate) || (q_norm && !aligned16(q_norm)) ||
        (k_norm && !aligned16(k_norm)) || (p0 >= 0 && !c->pt && p0 + T > c->n_ctx))
        B200_REFUSE(B200_ERR_SHAPE, "attn_prep: unsupported shape / cache / alignment (D=%d Hkv=%d n_rot=%d)", D, Hkv, n_rot);
    if (mr && mr->p && mr->sect <= 0) B200_REFUSE(B200_ERR_SHAPE, "attn_prep: M-RoPE sections sum to 0");
    return prep_impl(qg, k, v, q_norm, k_norm, pos, nullptr, q, gate, c, p0, T, Hq, Hkv, D, n_rot, freq_base, eps, (cudaStream_t) stream,
                     ldq, ldk, ldv, mr, "attn_prep");
}

int b200_attn_prep_rows(const float * qg, const float * k, const float * v, const float * q_norm, const float * k_norm,
                        const int32_t * rope_pos, const int32_t * cache_row, float * q, float * gate, const b200_kv_cache * c,
                        int T, int Hq, int Hkv, int D, int n_rot, float freq_base, float eps, void * stream) {
    if (T <= 0) return B200_OK;
    if (!c || !k || !v || !rope_pos || !cache_row || (qg && (!q || !gate))) B200_REFUSE(B200_ERR_SHAPE, "attn_prep_rows: null argument");
    if (!type_ok(c->type) || !c->k || c->D != D || c->Hkv != Hkv || D % 128 || D > 1024 || n_rot > D || n_rot % 2 ||
        !aligned16(qg) || !aligned16(k) || !aligned16(q) || !aligned16(gate) || (q_norm && !aligned16(q_norm)) ||
        (k_norm && !aligned16(k_norm)))
        B200_REFUSE(B200_ERR_SHAPE, "attn_prep_rows: unsupported shape / cache / alignment (D=%d Hkv=%d n_rot=%d)", D, Hkv, n_rot);
    return prep_impl(qg, k, v, q_norm, k_norm, rope_pos, cache_row, q, gate, c, -1, T, Hq, Hkv, D, n_rot, freq_base, eps,
                     (cudaStream_t) stream, Hq * 2 * D, Hkv * D, Hkv * D, nullptr, "attn_prep_rows");
}

int b200_rope_append_bf16(const uint16_t * q, const uint16_t * k, const uint16_t * v, float * q_out,
                          const b200_kv_cache * c, int p0, int T, int Hq, int Hkv, int D, int n_rot, float freq_base,
                          void * stream) {
    return rope_append_launch(q, k, v, q_out, nullptr, c, p0, T, Hq, Hkv, D, n_rot, freq_base, (cudaStream_t) stream, "rope_append_bf16", -1);
}
int b200_rope_append_bf16_at(const uint16_t * q, const uint16_t * k, const uint16_t * v, float * q_out, const b200_kv_cache * c, int row0,
                             int rope0, int T, int Hq, int Hkv, int D, int n_rot, float freq_base, void * stream) {
    if (rope0 < 0) B200_REFUSE(B200_ERR_SHAPE, "rope_append_bf16_at: negative rotary position");
    return rope_append_launch(q, k, v, q_out, nullptr, c, row0, T, Hq, Hkv, D, n_rot, freq_base, (cudaStream_t) stream, "rope_append_bf16_at", rope0);
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
    const long long items = (long long) T * ((n / 4 + 31) / 32);
    const unsigned blocks = (unsigned) std::min<long long>((items + 7) / 8, 148 * 8);
    if (op == 0) ew_k<0><<<blocks, 256, 0, (cudaStream_t) stream>>>(a, b, y, (__half2 *) qbuf, T, n, lda, ldb);
    else ew_k<1><<<blocks, 256, 0, (cudaStream_t) stream>>>(a, b, y, (__half2 *) qbuf, T, n, lda, ldb);
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
const char * b200_version(void) { return "b200attn 0.2 (sm_100a)"; }

}  // extern "C"
