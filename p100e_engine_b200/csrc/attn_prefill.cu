// Chunked causal prefill attention over the paged f16 / q8_0 / q4_0 cache on the sm_100a tensor cores (tcgen05 + TMEM).
//
// Two kernels per call:
//   kv_tiles_k   dequantises the visible keys once into f16 "tile images" in scratch: per (kv head, 64-key tile) a
//                32 KB K image and a 32 KB V image laid out exactly as the tensor core reads them from shared memory
//                (un-swizzled canonical layout, see umma.cuh; 8-key groups 4 KB apart, so two images side by side form
//                one 128-key operand), so the main kernel fetches a tile with one bulk copy.
//   prefill_k    one CTA per (128 query rows of one kv head): rows n = 6 t + hh (token t, head hh of the GQA group) on
//                the MMA M axis, keys in steps of 128 (a pair of images).  Per step: S = Q K^T as 16 MMAs m128n128k16
//                (Q from tensor memory, fp32 S in tensor memory), online softmax in base 2 with two threads per row
//                (64 keys each, no shuffles), P to shared memory as f16, O += P V as 8 MMAs m128n256k16 accumulated in
//                tensor memory.  Warp roles: 8 softmax warps, 1 bulk-copy producer warp, 1 MMA-issue warp.  The MMA
//                queue alternates Q K^T of step J+1 and P V of step J, so the tensor pipe has work while the softmax
//                of a step runs; S is single-buffered (the next Q K^T starts when the softmax threads hold S in
//                registers), P is double-buffered.  The running output is rescaled only when a row's maximum grows by
//                more than 2^8 (P stays below 256 in f16).  Epilogue: O / l, optional sigmoid gate.
// f16 operands (int8 * f16 scale is not representable in bf16's 8 significand bits), fp32 accumulation.
// Long contexts run as several passes over consecutive key ranges (as many keys as the scratch holds tile images for):
// a row tile whose keys continue in a later pass leaves its unnormalised O in the output buffer and (max, sum) beside it,
// and the next pass loads them back into tensor memory; the pass that holds a row tile's last key writes the result.
// Q may come as bf16 rows straight from the projection: the partial rotation is then applied while the rows are converted
// for tensor memory (cos / sin per token from a table the append kernel wrote), so no fp32 copy of Q goes through HBM.
//
// Reference counterparts: attn_fold (src/fast/attn_fold.cu:562-649: per chunk dequantise to f16 in scratch, HFMA2 tile
// GEMMs on CUDA cores), attn_prefill (src/fast/attn.cu:457-499, fp32 CUDA cores).
#include "umma.cuh"

#include <cuda_bf16.h>

#include <algorithm>
#include <atomic>
#include <mutex>

namespace b200 {
namespace {

constexpr int BM = 128;                 // query rows per CTA
constexpr int BN = 64;                  // keys per tile image
constexpr int BP = 2 * BN;              // keys per step: S tile = 128 rows x 128 keys
constexpr int IMG = BN * DH * 2;        // bytes of one tile image (32 KB)
constexpr int P_BYTES = BM * BP * 2;    // 32 KB
constexpr int Q_BYTES = BM * DH * 2;    // 64 KB
constexpr int EPI_BYTES = 8 * 32 * 33 * 4;   // per softmax warp a 32 x 33 float tile for the row-wise epilogue
constexpr int NSOFT = 256;              // softmax threads: two per query row (key halves of a tile, dim halves of the output)
constexpr int NTHR_PF = NSOFT + 64;     // 8 softmax warps + producer + MMA issuer
constexpr int W_PROD = NSOFT / 32, W_MMA = W_PROD + 1;
constexpr float LOG2E_PF = 1.4426950408889634f;
constexpr float RESCALE_GAP = 8.0f;     // rescale O when a row maximum grows by more than this (log2 units)

constexpr int NSTG = 3;                         // V ring depth (64-key images)
constexpr int SM_K = 0;                         // one pair of K images (the epilogue tiles reuse it)
constexpr int SM_EPI = SM_K;
constexpr int SM_V = SM_K + 2 * IMG;            // NSTG images
constexpr int SM_P = SM_V + NSTG * IMG;         // 2 buffers
constexpr int SM_XCH = SM_P + 2 * P_BYTES;      // [2][128] floats exchanged between the two threads of a row
constexpr int SM_BAR = SM_XCH + 1024;           // mbarriers + tmem base
constexpr int SM_TOTAL = SM_BAR + 256;
static_assert(SM_TOTAL <= 227 * 1024 && EPI_BYTES <= 2 * IMG, "prefill_k shared memory");

// ---- pre-pass: cache rows -> f16 tile images -------------------------------------------------------------------
// grid (n_tiles, Hkv), 256 threads; thread = (key, 8-dim chunk).  Image byte of (key, dim) = (key/8)*4096 + (dim/8)*128 +
// (key%8)*16 + (dim%8)*2 for K (K-major B operand) and for V (MN-major B operand) alike.  Keys >= n_keys are zero.
template <uint32_t KT>
__global__ void __launch_bounds__(256) kv_tiles_k(kv_view g, int kb, int n_keys, unsigned char * __restrict__ tiles, int n_tiles,
                                                  unsigned * status) {
    const int tile = blockIdx.x, hk = blockIdx.y;   // tile j of the pass holds keys kb + 64 j ..; keys >= n_keys are zero
    unsigned char * kimg = tiles + ((size_t) hk * n_tiles + tile) * (2 * IMG);
    unsigned char * vimg = kimg + IMG;
    const int32_t * tab = kv_tab(g, 0);
    for (int i = threadIdx.x; i < BN * 32; i += 256) {
        const int key = i & (BN - 1), dc = i >> 6;
        const int kk = kb + tile * BN + key;
        uint4 ko = make_uint4(0, 0, 0, 0), vo = ko;
        if (kk < n_keys) {
            bool ok = true;
            if (tab && tab[kk >> g.psh] < 0) { atomicOr(status, ST_BAD_PAGE); ok = false; }
            if (ok) {
                const unsigned long long off = kv_off_tab(g, tab, kk) + (unsigned long long) hk * head_bytes(KT);
                const unsigned char * kr = (const unsigned char *) g.k + off, * vr = (const unsigned char *) g.v + off;
                if constexpr (KT == B200_KV_F16) {
                    ko = *reinterpret_cast<const uint4 *>(kr + dc * 16);
                    vo = *reinterpret_cast<const uint4 *>(vr + dc * 16);
                } else {
                    float kf[8], vf[8];
                    if constexpr (KT == B200_KV_Q8_0) {
                        const float dk = __half2float(reinterpret_cast<const __half *>(kr)[dc >> 2]);
                        const float dv = __half2float(reinterpret_cast<const __half *>(vr)[dc >> 2]);
                        const uint2 qk = *reinterpret_cast<const uint2 *>(kr + 16 + dc * 8);
                        const uint2 qv = *reinterpret_cast<const uint2 *>(vr + 16 + dc * 8);
                        const int8_t * a = reinterpret_cast<const int8_t *>(&qk), * b = reinterpret_cast<const int8_t *>(&qv);
#pragma unroll
                        for (int e = 0; e < 8; ++e) { kf[e] = dk * (float) a[e]; vf[e] = dv * (float) b[e]; }
                    } else {
                        const int blk = dc >> 2, sub = dc & 3;   // dims 8 sub .. 8 sub + 7 of the block: bytes (8 sub) % 16 .., nibble sub / 2
                        const unsigned char * kb = kr + blk * 18, * vb = vr + blk * 18;
                        const float dk = __half2float(*reinterpret_cast<const __half *>(kb));
                        const float dv = __half2float(*reinterpret_cast<const __half *>(vb));
                        const int sh = (sub >> 1) * 4, b0 = 2 + (sub & 1) * 8;
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            kf[e] = dk * (float) ((int) ((kb[b0 + e] >> sh) & 15) - 8);
                            vf[e] = dv * (float) ((int) ((vb[b0 + e] >> sh) & 15) - 8);
                        }
                    }
                    ko = make_uint4(pack_h2(kf[0], kf[1]), pack_h2(kf[2], kf[3]), pack_h2(kf[4], kf[5]), pack_h2(kf[6], kf[7]));
                    vo = make_uint4(pack_h2(vf[0], vf[1]), pack_h2(vf[2], vf[3]), pack_h2(vf[4], vf[5]), pack_h2(vf[6], vf[7]));
                }
            }
        }
        *reinterpret_cast<uint4 *>(kimg + (key >> 3) * 4096 + dc * 128 + (key & 7) * 16) = ko;
        *reinterpret_cast<uint4 *>(vimg + (key >> 3) * 4096 + dc * 128 + (key & 7) * 16) = vo;
    }
}

struct pf_args {
    const float * q;              // [T][Hq][256] f32, already rotated, or nullptr
    const __nv_bfloat16 * qb;     // [T][Hq][256] bf16, not yet rotated (used when q is null); needs cs
    const float * cs;             // [T][64]: cos of the 32 rotary pairs, then sin (written by the append kernel)
    const float * gate;           // [T][Hq*256] f32 or nullptr
    const __nv_bfloat16 * gate_b; // the gate as bf16 (used when gate is null) or nullptr
    float * out;                  // [T][Hq][256] f32: the result; between passes the running unnormalised O
    __nv_bfloat16 * out_b;        // the result as bf16 (optional; out is then only the carry buffer)
    float * ml;                   // [T*Hq][2] running (maximum in log2 units, sum) between passes
    float * pm, * pl;             // partial form: [T*Hq] maximum (natural-log units) and sum; out keeps the unnormalised O
    __half2 * qbuf;               // a16 copy of the result (optional)
    const int32_t * lim;          // per token: last visible key (device), or nullptr for p0 + t
    const unsigned char * tiles;
    int n_tiles;                  // tile images per head in scratch
    int kb, ke;                   // keys of this pass: kb (a multiple of 128) .. ke - 1
    int T, p0, Hq, Hkv;
    float qscale;                 // softmax scale * log2(e)
    unsigned * status;
};

// 1 / (1 + 2^(-g log2 e)) with the hardware exponential and reciprocal (relative error ~1e-7 against expf and an IEEE divide)
__device__ __forceinline__ float fast_sigmoid(float g) { return __fdividef(1.0f, 1.0f + ex2f(-g * LOG2E_PF)); }

__device__ __forceinline__ void mbar_arrive(uint64_t * bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void bf16x8_widen(const uint4 u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { f[2 * e] = __uint_as_float(w[e] << 16); f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u); }
}

__global__ void __launch_bounds__(NTHR_PF, 1) prefill_k(const pf_args a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t * bars = reinterpret_cast<uint64_t *>(smem + SM_BAR);
    uint64_t * k_full = bars, * k_free = bars + 1, * s_full = bars + 2, * s_free = bars + 3, * v_full = bars + 4, * v_free = bars + 8,
             * p_full = bars + 12, * pv_done = bars + 14, * o_done = bars + 16, * q_ready = bars + 17;
    uint32_t * tbase_p = reinterpret_cast<uint32_t *>(bars + 18);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int mtile = (int) gridDim.x - 1 - (int) blockIdx.x;   // heaviest (latest rows) first
    const int hk = blockIdx.y;
    const int R = a.T * GQA;                                    // rows of this kv head
    const int n0 = mtile * BM;
    const int t_last = min(n0 + BM - 1, R - 1) / GQA;           // last token of the tile
    const int n_keys_vis = (a.lim ? a.lim[t_last] : a.p0 + t_last) + 1;   // keys any row of the tile can see (limits do not decrease with t)
    // This pass covers keys kb .. ke-1.  A tile whose keys ended in an earlier pass has been written already; a tile
    // whose keys go on past ke leaves its running state behind for the next pass.
    if (n_keys_vis <= a.kb && a.kb > 0) return;
    const bool carry_in = a.kb > 0;
    const bool carry_out = n_keys_vis > a.ke;
    const int n_keys_pass = max(0, min(n_keys_vis, a.ke) - a.kb);
    const int ntiles = (n_keys_pass + BN - 1) / BN;             // 64-key images of this pass
    const int nsteps = (ntiles + 1) / 2;                        // 128-key steps; the last one may hold a single image

    if (tid == 0) {
        mbar_init(k_full, 1); mbar_init(k_free, 1); mbar_init(s_full, 1); mbar_init(s_free, NSOFT);
        for (int b = 0; b < NSTG; ++b) { mbar_init(&v_full[b], 1); mbar_init(&v_free[b], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&p_full[b], NSOFT); mbar_init(&pv_done[b], 1); }
        mbar_init(o_done, 1);
        mbar_init(q_ready, 1);
        mbar_fence_init();
    }
    if (warp == 0) umma::tmem_alloc(tbase_p, 512);
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tb = *tbase_p;
    const uint32_t t_S = tb, t_O = tb + BP, t_Q = tb + BP + DH;   // S at columns 0..127, O at 128..383, Q (f16 pairs) at 384..511

    // row bookkeeping of the softmax threads, shared by the prologue, the loop and the epilogue: a warp owns the 32 rows of its
    // tensor-memory lanes; for row-wise global accesses 8 lanes cover 128 bytes of one row, a warp instruction touches 4 rows
    const uint32_t lane_off = (uint32_t) ((warp & 3) * 32) << 16;
    const int sub = lane >> 3, col = 4 * (lane & 7);
    float m_ref = B200_NEG_INF, l = 0.0f;

    if (warp < W_PROD) {
        // Q rows -> f16, scaled by softmax scale * log2(e), into tensor memory as the A operand of Q K^T: lane = row,
        // column c holds dims 2c, 2c+1.  The two threads of a row take 128 dims each, 64 dims per slab.
        const int r = tid & (BM - 1), hf = tid >> 7, n = n0 + r;
        const int t = n / GQA, hh = n - t * GQA;
        const size_t rowidx = (size_t) t * a.Hq + hk * GQA + hh;
        const float sc = a.qscale;
        if (a.q) {
            const float4 * src = n < R ? reinterpret_cast<const float4 *>(a.q + rowidx * DH) : nullptr;
#pragma unroll 1
            for (int d0 = hf * (DH / 2); d0 < (hf + 1) * (DH / 2); d0 += 64) {
                float4 x[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) x[u] = src ? __ldg(src + d0 / 4 + u) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                uint32_t w[32];
#pragma unroll
                for (int u = 0; u < 16; ++u) { w[2 * u] = pack_h2(x[u].x * sc, x[u].y * sc); w[2 * u + 1] = pack_h2(x[u].z * sc, x[u].w * sc); }
                umma::tmem_st32(t_Q + lane_off + d0 / 2, w);
            }
        } else {
            // bf16 rows as the projection wrote them: widen, rotate the 32 pairs (j, j + 32) of the first 64 dims with the
            // token's cos / sin (same expressions and roundings as the append kernel), scale, round to f16
            const uint4 * src = n < R ? reinterpret_cast<const uint4 *>(a.qb + rowidx * DH) : nullptr;
#pragma unroll 1
            for (int d0 = hf * (DH / 2); d0 < (hf + 1) * (DH / 2); d0 += 64) {
                float f[64];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    float e8[8];
                    bf16x8_widen(src ? __ldg(src + d0 / 8 + u) : make_uint4(0, 0, 0, 0), e8);
#pragma unroll
                    for (int e = 0; e < 8; ++e) f[8 * u + e] = e8[e];
                }
                if (d0 == 0 && src) {
                    const float4 * cs4 = reinterpret_cast<const float4 *>(a.cs + (size_t) t * 64);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const float4 c4 = __ldg(cs4 + u), s4 = __ldg(cs4 + 8 + u);
                        const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) rot_pair(f[4 * u + e], f[32 + 4 * u + e], cc[e], ss[e], f[4 * u + e], f[32 + 4 * u + e]);
                    }
                }
                uint32_t w[32];
#pragma unroll
                for (int u = 0; u < 32; ++u) w[u] = pack_h2(f[2 * u] * sc, f[2 * u + 1] * sc);
                umma::tmem_st32(t_Q + lane_off + d0 / 2, w);
            }
        }
        if (carry_in) {
            // the running O of the earlier passes goes back into tensor memory (read row-wise, handed over through a
            // per-warp tile in the P buffers, which nothing uses before the barrier below), with the row's maximum and sum
            float * tile = reinterpret_cast<float *>(smem + SM_P) + warp * (32 * 33);
            const int c_lo = hf * (DH / 2), c_hi = c_lo + DH / 2;
#pragma unroll 1
            for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
#pragma unroll
                for (int q8 = 0; q8 < 8; ++q8) {
                    const int rl = 4 * q8 + sub, nr = n0 + (warp & 3) * 32 + rl;
                    const int tr = nr / GQA, hr = nr - tr * GQA;
                    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (nr < R) v = *reinterpret_cast<const float4 *>(a.out + ((size_t) tr * a.Hq + hk * GQA + hr) * DH + c0 + col);
                    tile[rl * 33 + col] = v.x; tile[rl * 33 + col + 1] = v.y; tile[rl * 33 + col + 2] = v.z; tile[rl * 33 + col + 3] = v.w;
                }
                __syncwarp();
                uint32_t o[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(tile[lane * 33 + c]);
                umma::tmem_st32(t_O + lane_off + c0, o);
                __syncwarp();
            }
            if (n < R) {
                m_ref = a.ml[rowidx * 2];
                l = hf == 0 ? a.ml[rowidx * 2 + 1] : 0.0f;
            }
        }
        umma::tmem_st_wait();
        umma::fence_before_sync();
        asm volatile("bar.sync 1, %0;" ::"n"(NSOFT) : "memory");   // the softmax warps: every Q (and O) row is in place
        if (tid == 0) mbar_arrive(q_ready);
    }
    const bool any_gate = a.gate || a.gate_b;
    if (warp >= W_PROD && any_gate && !carry_out && (lane & 15) != 0) {
        // idle lanes of the producer and MMA warps pull this CTA's gate rows (contiguous per token: 6 heads) into L2
        const int t_first = n0 / GQA;
        const int esz = a.gate ? 4 : 2;
        const char * g0 = a.gate ? reinterpret_cast<const char *>(a.gate + ((size_t) t_first * a.Hq + hk * GQA) * DH)
                                 : reinterpret_cast<const char *>(a.gate_b + ((size_t) t_first * a.Hq + hk * GQA) * DH);
        const int idx = (warp - W_PROD) * 30 + lane - 1 - (lane > 16);
        for (int t = t_first; t <= t_last; ++t)
            for (int ln = idx; ln < GQA * DH * esz / 128; ln += 60)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(g0 + (size_t) (t - t_first) * a.Hq * DH * esz + ln * 128));
    }
    if (warp == W_PROD) {
        // ---------------- producer: K in pairs of images (lane 0), V image by image through a ring (lane 16) ----------------
        const unsigned char * src = a.tiles + (size_t) hk * a.n_tiles * (2 * IMG);
        if (lane == 0) {
            for (int J = 0; J < nsteps; ++J) {
                if (J >= 1) mbar_wait(k_free, (uint32_t) ((J - 1) & 1), a.status);   // Q K^T of step J-1 has read the pair
                const int n_img = min(2, ntiles - 2 * J);
                mbar_expect_tx(k_full, (uint32_t) n_img * IMG);
                for (int h = 0; h < n_img; ++h)
                    bulk_g2s(smem + SM_K + h * IMG, src + (size_t) (2 * J + h) * (2 * IMG), IMG, k_full);
            }
        } else if (lane == 16) {
            for (int j = 0; j < ntiles; ++j) {
                const int s = j % NSTG;
                if (j >= NSTG) mbar_wait(&v_free[s], (uint32_t) ((j / NSTG - 1) & 1), a.status);   // P V of image j-NSTG has read the slot
                mbar_expect_tx(&v_full[s], IMG);
                bulk_g2s(smem + SM_V + s * IMG, src + (size_t) j * (2 * IMG) + IMG, IMG, &v_full[s]);
            }
        }
    } else if (warp == W_MMA) {
        // ---------------- MMA issuer: Q K^T of step J+1 is queued before P V of step J ----------------
        if (lane == 0) {
            constexpr uint32_t id_qk = umma::idesc_f16(BM, BP, false, false);   // S[128 x 128] = Q (tensor memory) * K^T (K-major)
            constexpr uint32_t id_pv = umma::idesc_f16(BM, DH, false, true);    // O[128 x 256] += P (K-major) * V (MN-major)
            const uint32_t k_s = smem_u32(smem + SM_K);
            auto issue_qk = [&](int J) {
                mbar_wait(k_full, (uint32_t) (J & 1), a.status);
                if (J >= 1) mbar_wait(s_free, (uint32_t) ((J - 1) & 1), a.status);   // the softmax threads hold S of step J-1 in registers
                umma::fence_after_sync();
                // K pair: K-major, 8-key groups 4096 apart (SBO), 8-dim chunks 128 apart (LBO); 16 dims = 256 bytes per k-step.
                // A step with a single image multiplies whatever the second half of the buffer holds: those keys lie past
                // every row of the tile and are masked.
#pragma unroll 4
                for (int ks = 0; ks < DH / 16; ++ks)
                    umma::mma_ts(t_S, t_Q + ks * 8, umma::smem_desc(k_s + ks * 256, 128, 4096), id_qk, ks > 0);
                umma::commit(s_full);
                umma::commit(k_free);
            };
            auto issue_pv = [&](int J) {
                const int b = J & 1;
                mbar_wait(&p_full[b], (uint32_t) ((J >> 1) & 1), a.status);
                const uint32_t p_s = smem_u32(smem + SM_P + b * P_BYTES);
                const int n_img = min(2, ntiles - 2 * J);
                for (int h = 0; h < n_img; ++h) {
                    const int j = 2 * J + h, st = j % NSTG;
                    mbar_wait(&v_full[st], (uint32_t) ((j / NSTG) & 1), a.status);
                    umma::fence_after_sync();
                    const uint32_t v_s = smem_u32(smem + SM_V + st * IMG);
#pragma unroll
                    for (int ks = 0; ks < BN / 16; ++ks)   // P: K-major, 8-key chunks 2048 apart; V: MN-major, 8-key groups 4096 apart (LBO),
                                                           // 8-dim chunks 128 apart (SBO)
                        umma::mma_ss(t_O, umma::smem_desc(p_s + (h * 4 + ks) * 2 * 2048, 2048, 128),
                                     umma::smem_desc(v_s + ks * 2 * 4096, 4096, 128), id_pv, (carry_in || j > 0 || ks > 0) ? 1u : 0u);
                    umma::commit(&v_free[st]);
                }
                umma::commit(&pv_done[b]);
            };
            mbar_wait(q_ready, 0, a.status);
            umma::fence_after_sync();
            if (nsteps > 0) issue_qk(0);
            for (int J = 0; J < nsteps; ++J) {
                if (J + 1 < nsteps) issue_qk(J + 1);
                issue_pv(J);
            }
            umma::commit(o_done);
        }
    } else {
        // ---------------- softmax: two threads per row ----------------
        // Thread (row r, half hf) owns keys 64 hf .. 64 hf + 63 of every step and, in the epilogue, output dims 128 hf ..
        // The two warps that share 32 rows (warps w and w + 4, the same tensor-memory lanes) meet once per step at a
        // 64-thread barrier that ORs their "a maximum grew" votes; both keep the same reference maximum in registers.
        const int r = tid & (BM - 1), hf = tid >> 7, n = n0 + r;
        const int t_row = n / GQA;
        const int pos = n < R ? (a.lim ? a.lim[t_row] : a.p0 + t_row) : -1;
        const int pair_bar = 2 + (warp & 3);
        float * xch = reinterpret_cast<float *>(smem + SM_XCH);
        for (int J = 0; J < nsteps; ++J) {
            mbar_wait(s_full, (uint32_t) (J & 1), a.status);
            umma::fence_after_sync();
            uint32_t sr[2][32];
            umma::tmem_ld32(t_S + lane_off + 64 * hf, sr[0]);
            umma::tmem_ld32(t_S + lane_off + 64 * hf + 32, sr[1]);
            umma::tmem_ld_wait();
            umma::fence_before_sync();
            mbar_arrive(s_free);   // S is in registers: the next Q K^T may overwrite it
            const int k0 = a.kb + J * BP + 64 * hf;
            const bool diag = k0 + 63 > pos;   // some key of this half is masked for this row
            if (__any_sync(0xffffffffu, diag)) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (k0 + 32 * h + c > pos) sr[h][c] = __float_as_uint(B200_NEG_INF);
            }
            float mx4[4] = {B200_NEG_INF, B200_NEG_INF, B200_NEG_INF, B200_NEG_INF};   // four chains: the maximum is latency-bound
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int c = 0; c < 32; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[h][c]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // lazy rescale: only when some row of the warp pair outgrew its reference maximum
            const int grow_here = mx > m_ref + RESCALE_GAP || (m_ref == B200_NEG_INF && mx != B200_NEG_INF);
            int grow_any;
            asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.s32 q, %1, 0;\n\tbarrier.red.or.pred p, %2, 64, q;\n\tselp.s32 %0, 1, 0, p;\n\t}"
                         : "=r"(grow_any) : "r"(grow_here), "r"(pair_bar) : "memory");
            if (grow_any) {
                xch[hf * BM + r] = mx;
                asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
                const float mxr = fmaxf(xch[r], xch[BM + r]);
                asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");   // both have read before the next use of xch
                float f = 1.0f;
                if (mxr > m_ref + RESCALE_GAP || (m_ref == B200_NEG_INF && mxr != B200_NEG_INF)) {
                    f = m_ref == B200_NEG_INF ? 0.0f : ex2f(m_ref - mxr);
                    m_ref = mxr;
                    l *= f;
                }
                if (J > 0 || carry_in) {
                    if (J > 0) mbar_wait(&pv_done[(J - 1) & 1], (uint32_t) (((J - 1) >> 1) & 1), a.status);   // P V of step J-1 has landed in O
                    umma::fence_after_sync();
#pragma unroll 1
                    for (int c0 = hf * (DH / 2); c0 < (hf + 1) * (DH / 2); c0 += 32) {
                        uint32_t o[32];
                        umma::tmem_ld32(t_O + lane_off + c0, o);
                        umma::tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
                        umma::tmem_st32(t_O + lane_off + c0, o);
                    }
                    umma::tmem_st_wait();
                    umma::fence_before_sync();
                }
            }
            const float mref_safe = m_ref == B200_NEG_INF ? 0.0f : m_ref;
            if (J >= 2) mbar_wait(&pv_done[J & 1], (uint32_t) (((J >> 1) - 1) & 1), a.status);   // P buffer no longer read
            // K-major P image of the step: key chunk kc (8 keys) at kc * 2048, row at 16 bytes; this thread's chunks are 8 hf ..
            unsigned char * prow = smem + SM_P + (J & 1) * P_BYTES + (8 * hf) * 2048 + r * 16;
            float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int c8 = 0; c8 < 4; ++c8) {
                    uint32_t w4[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        // ex2(-inf) = 0: masked keys need no special case (mref_safe is finite)
                        const float p0 = ex2f(__uint_as_float(sr[h][c8 * 8 + 2 * e]) - mref_safe);
                        const float p1 = ex2f(__uint_as_float(sr[h][c8 * 8 + 2 * e + 1]) - mref_safe);
                        l4[e] += p0 + p1;
                        w4[e] = pack_h2(p0, p1);
                    }
                    *reinterpret_cast<uint4 *>(prow + (4 * h + c8) * 2048) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            umma::fence_async_smem();
            umma::fence_before_sync();
            mbar_arrive(&p_full[J & 1]);
        }
        // ---------------- epilogue ----------------
        // final:   O / l, gate, store (f32 and / or bf16, a16 copy);  carry_out: unnormalised O, (maximum, sum) for the next pass;
        // partial: unnormalised O with the maximum in natural-log units and the sum, for a merge across sequence shards
        xch[hf * BM + r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        l = xch[r] + xch[BM + r];
        mbar_wait(o_done, 0, a.status);
        umma::fence_after_sync();
        const bool raw = carry_out || a.pm;   // O leaves unnormalised
        const bool have_o = nsteps > 0 || carry_in;   // a tile that has seen no key at all (a sequence shard) holds nothing in O
        const float inv = raw ? 1.0f : (l > 0.0f ? 1.0f / l : 0.0f);
        if (n < R && hf == 0) {
            const size_t rowidx = (size_t) t_row * a.Hq + hk * GQA + (n - t_row * GQA);
            if (carry_out) { a.ml[rowidx * 2] = m_ref; a.ml[rowidx * 2 + 1] = l; }
            else if (a.pm) { a.pm[rowidx] = m_ref * 0.6931471805599453f; a.pl[rowidx] = l; }
        }
        // A 32-column slab of O goes through a private shared-memory tile so that global accesses run along rows.
        float * tile = reinterpret_cast<float *>(smem + SM_EPI) + warp * (32 * 33);
        const int c_lo = hf * (DH / 2), c_hi = c_lo + DH / 2;
        size_t orow[8];
        bool live[8];
#pragma unroll
        for (int q8 = 0; q8 < 8; ++q8) {
            const int nr = n0 + (warp & 3) * 32 + 4 * q8 + sub;
            const int tr = nr / GQA, hr = nr - tr * GQA;
            live[q8] = nr < R;
            orow[q8] = ((size_t) tr * a.Hq + hk * GQA + hr) * DH + col;
        }
        const bool gated = any_gate && !raw;
        auto gate_at = [&](size_t o) {
            if (a.gate) return __ldg(reinterpret_cast<const float4 *>(a.gate + o));
            const uint2 u = __ldg(reinterpret_cast<const uint2 *>(a.gate_b + o));
            return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                               __uint_as_float(u.y & 0xffff0000u));
        };
        float4 gn[8];   // gate values of the next slab, requested one slab ahead
#pragma unroll
        for (int q8 = 0; q8 < 8; ++q8) gn[q8] = (gated && live[q8]) ? gate_at(orow[q8] + c_lo) : make_float4(0.f, 0.f, 0.f, 0.f);
        const size_t n_groups = (size_t) a.T * a.Hq * (DH / 32);
#pragma unroll 1
        for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
            float4 gv[8];
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) {
                gv[q8] = gn[q8];
                if (gated && live[q8] && c0 + 32 < c_hi) gn[q8] = gate_at(orow[q8] + c0 + 32);
            }
            uint32_t o[32];
            if (have_o) {
                umma::tmem_ld32(t_O + lane_off + c0, o);
                umma::tmem_ld_wait();
            } else {
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = 0u;
            }
#pragma unroll
            for (int c = 0; c < 32; ++c) tile[lane * 33 + c] = __uint_as_float(o[c]) * inv;
            __syncwarp();
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) {
                const int rl = 4 * q8 + sub;
                float4 y = make_float4(tile[rl * 33 + col], tile[rl * 33 + col + 1], tile[rl * 33 + col + 2], tile[rl * 33 + col + 3]);
                if (gated) {
                    y.x *= fast_sigmoid(gv[q8].x); y.y *= fast_sigmoid(gv[q8].y);
                    y.z *= fast_sigmoid(gv[q8].z); y.w *= fast_sigmoid(gv[q8].w);
                }
                if (live[q8]) {
                    if (raw || !a.out_b) *reinterpret_cast<float4 *>(a.out + orow[q8] + c0) = y;
                    if (!raw && a.out_b) {
                        const __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
                        *reinterpret_cast<uint2 *>(a.out_b + orow[q8] + c0) =
                            make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
                    }
                }
                // the a16 copy for the projection that follows: the eight lanes of a row segment hold one 32-value group
                if (a.qbuf && !raw) a16_store_lanes8(y, a.qbuf, (orow[q8] + c0) / 32, n_groups, live[q8]);
            }
            __syncwarp();
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tb, 512);
}

// ------------------------------------------------------------------------------------------------ host side ----
constexpr size_t TILE_BYTES_PER_KEY = 2 * IMG / BN;   // K and V images: 1 KiB per key and kv head
constexpr int DEFAULT_PASS_KEYS = 8192;               // keys per pass that attn_fold_scratch_bytes(T, Hkv, 0, 0) provides for
constexpr size_t OWN_SCRATCH_TILE_CAP = (size_t) 256 << 20;   // library scratch holds tile images for at most this many bytes per pass

size_t align256(size_t v) { return (v + 255) & ~(size_t) 255; }
size_t ml_bytes(int T, int Hkv) { return align256((size_t) T * Hkv * GQA * 2 * sizeof(float)); }
size_t tile_bytes(int keys, int Hkv) { return (size_t) ((keys + BP - 1) / BP * BP) * Hkv * TILE_BYTES_PER_KEY; }

// Library scratch of the prefill entry points that take none from the caller: one buffer per (device, stream), sized on
// first use for the call at hand (tile images capped at OWN_SCRATCH_TILE_CAP per pass; longer contexts take more passes).
// A later call that needs more gets a new buffer half as large again at least; the old one stays allocated until the
// process exits, so nothing is freed under work in flight and no stream is synchronised.
struct own_scratch { int dev = -1; cudaStream_t s = nullptr; void * p = nullptr; size_t cap = 0; };
own_scratch g_own[64];
int g_nown = 0;
std::mutex g_pf_mu;

void * own_scratch_for(size_t bytes, cudaStream_t s, size_t * cap_out) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(g_pf_mu);
    own_scratch * e = nullptr;
    for (int i = 0; i < g_nown; ++i) if (g_own[i].dev == dev && g_own[i].s == s) e = &g_own[i];
    if (!e) {
        if (g_nown == 64) return nullptr;
        e = &g_own[g_nown++];
        e->dev = dev; e->s = s;
    }
    if (bytes > e->cap) {
        const size_t want = std::max(bytes, e->cap + e->cap / 2);
        void * p = nullptr;
        if (cudaMalloc(&p, want) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        e->p = p;
        e->cap = want;
    }
    *cap_out = e->cap;
    return e->p;
}

struct pf_io {
    const float * q; const __nv_bfloat16 * qb; const float * cs;
    const float * gate; const __nv_bfloat16 * gate_b;
    float * out; __nv_bfloat16 * out_b; float * pm, * pl; void * qbuf;
    const int32_t * lim;
};

// n_keys: keys the last row sees (p0 + T, or the host's bound on lim[T-1] + 1).  scratch == nullptr: library scratch.
int prefill_run(const pf_io & io, const b200_kv_cache * c, int T, int p0, int n_keys, int Hq, float scale, void * scratch,
                size_t scratch_bytes, cudaStream_t s, const char * who) {
    if (!c || (!io.q && !io.qb) || (!io.out && !io.out_b) || !c->k || !c->v) B200_REFUSE(B200_ERR_SHAPE, "%s: null argument", who);
    if (c->D != DH || Hq != GQA * c->Hkv || c->Hkv <= 0 || T < 1 || p0 < 0 || n_keys < 0)
        B200_REFUSE(B200_ERR_SHAPE, "%s: unsupported shape (D=%d Hq=%d Hkv=%d T=%d p0=%d)", who, c->D, Hq, c->Hkv, T, p0);
    if (c->type != B200_KV_F16 && c->type != B200_KV_Q8_0 && c->type != B200_KV_Q4_0) B200_REFUSE(B200_ERR_SHAPE, "%s: unsupported cache type %u", who, c->type);
    if (!aligned16(c->k) || !aligned16(c->v) || (io.q && !aligned16(io.q)) || (io.qb && !aligned16(io.qb)) || (io.out && !aligned16(io.out)) ||
        (io.out_b && !aligned16(io.out_b)) || (io.gate && !aligned16(io.gate)) || (io.gate_b && !aligned16(io.gate_b)) ||
        (c->pt && c->pstride % 16) || (io.qbuf && ((uintptr_t) io.qbuf & 3)))
        B200_REFUSE(B200_ERR_SHAPE, "%s: cache base, page stride, q, out and gate must be 16-byte aligned", who);
    if (!c->pt && n_keys > c->n_ctx) B200_REFUSE(B200_ERR_SHAPE, "%s: keys 0..%d outside n_ctx %d", who, n_keys - 1, c->n_ctx);
    if (io.pm && (!io.pl || !io.out)) B200_REFUSE(B200_ERR_SHAPE, "%s: the partial form needs part_o, part_m and part_l", who);
    // scratch: [running (max, sum) per row][running O when the result leaves as bf16 only][tile images of one pass]
    const size_t fixed = ml_bytes(T, c->Hkv);
    const size_t carry = io.out ? 0 : align256((size_t) T * Hq * DH * sizeof(float));
    const size_t per_step = (size_t) BP * c->Hkv * TILE_BYTES_PER_KEY;
    const size_t full = tile_bytes(std::max(n_keys, 1), c->Hkv);
    if (!scratch) {
        const size_t want = fixed + carry + std::min(full, std::max(OWN_SCRATCH_TILE_CAP / per_step, (size_t) 1) * per_step) + 256;
        scratch = own_scratch_for(want, s, &scratch_bytes);
        if (!scratch) B200_REFUSE(B200_ERR_ALLOC, "%s: %zu bytes of scratch could not be allocated", who, want);
    } else if ((uintptr_t) scratch & 255) {
        B200_REFUSE(B200_ERR_SCRATCH, "%s: scratch must be 256-byte aligned", who);
    }
    // one pass if the tile images of every visible key fit (no running O is needed then), else as many keys per pass as fit
    size_t steps_fit = scratch_bytes > fixed ? (scratch_bytes - fixed) / per_step : 0;
    bool multi = steps_fit * per_step < full;
    if (multi) steps_fit = scratch_bytes > fixed + carry ? (scratch_bytes - fixed - carry) / per_step : 0;
    if (steps_fit < 1)
        B200_REFUSE(B200_ERR_SCRATCH, "%s: scratch too small (%zu bytes given; %zu needed for one 128-key step, %zu for a single pass over %d keys)",
                    who, scratch_bytes, fixed + carry + per_step, fixed + full, n_keys);
    const long long keys_per_pass = (long long) std::min<size_t>(steps_fit, (size_t) 1 << 22) * BP;
    unsigned * st = device_status_word();
    if (!st) return B200_ERR_CUDA;
    static std::atomic<bool> attr_done[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(prefill_k, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL) != cudaSuccess)
            return launch_status("attn_prefill (shared memory attribute)");
        attr_done[dev & 63].store(true, std::memory_order_release);
    }
    unsigned char * base = (unsigned char *) scratch;
    pf_args a;
    a.q = io.q; a.qb = io.q ? nullptr : io.qb; a.cs = io.cs;
    a.gate = io.gate; a.gate_b = io.gate ? nullptr : io.gate_b;
    a.ml = reinterpret_cast<float *>(base);
    a.out = io.out ? io.out : multi ? reinterpret_cast<float *>(base + fixed) : nullptr;
    a.out_b = io.out_b; a.pm = io.pm; a.pl = io.pl; a.qbuf = (__half2 *) io.qbuf; a.lim = io.lim;
    unsigned char * tiles = base + fixed + (multi ? carry : 0);
    a.tiles = tiles;
    a.T = T; a.p0 = p0; a.Hq = Hq; a.Hkv = c->Hkv; a.qscale = scale * LOG2E_PF; a.status = st;
    const kv_view g = view_of(*c);
    const int n_mtiles = (T * GQA + BM - 1) / BM;
    int launches = 0;
    long long kb = 0;
    do {   // at least one pass, also when no key is visible (a sequence shard that owns nothing yet): it writes the empty result
        const long long ke = std::min<long long>(kb + keys_per_pass, std::max(n_keys, 1));
        const int n_tiles = (int) ((ke - kb + BN - 1) / BN);
        const dim3 tg(n_tiles, c->Hkv);
        if (c->type == B200_KV_F16) kv_tiles_k<B200_KV_F16><<<tg, 256, 0, s>>>(g, (int) kb, n_keys, tiles, n_tiles, st);
        else if (c->type == B200_KV_Q8_0) kv_tiles_k<B200_KV_Q8_0><<<tg, 256, 0, s>>>(g, (int) kb, n_keys, tiles, n_tiles, st);
        else kv_tiles_k<B200_KV_Q4_0><<<tg, 256, 0, s>>>(g, (int) kb, n_keys, tiles, n_tiles, st);
        a.n_tiles = n_tiles; a.kb = (int) kb; a.ke = (int) ke;
        prefill_k<<<dim3(n_mtiles, c->Hkv), NTHR_PF, SM_TOTAL, s>>>(a);
        launches += 2;
        kb = ke;
    } while (kb < n_keys);
    count_launch(launches);
    return launch_status(who);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_attn_prefill(const float * q, const b200_kv_cache * c, float * out, int T, int p0, int Hq, float scale, void * stream) {
    const pf_io io = {q, nullptr, nullptr, nullptr, nullptr, out, nullptr, nullptr, nullptr, nullptr, nullptr};
    return prefill_run(io, c, T, p0, p0 + T, Hq, scale, nullptr, 0, (cudaStream_t) stream, "attn_prefill");
}
int b200_attn_prefill_variant(const float * q, const b200_kv_cache * c, float * out, int T, int p0, int Hq, float scale, void * stream,
                              int variant) {
    (void) variant;   // the reference's variants are bitwise-equal schedules of one fp32 algorithm; there is one kernel here
    return b200_attn_prefill(q, c, out, T, p0, Hq, scale, stream);
}
// Scratch for passes of `chunk` keys (chunk <= 0: DEFAULT_PASS_KEYS); any amount from one 128-key step upwards works, a
// context that does not fit takes more passes.  nsplit has no meaning here.
size_t b200_attn_fold_scratch_bytes(int T, int Hkv, int chunk, int nsplit) {
    (void) nsplit;
    if (T < 1 || Hkv < 1) return 0;
    return ml_bytes(T, Hkv) + tile_bytes(chunk > 0 ? chunk : DEFAULT_PASS_KEYS, Hkv);
}
int b200_attn_fold(const float * q, const b200_kv_cache * c, float * out, int T, int p0, int Hq, float scale, void * scratch,
                   size_t scratch_bytes, void * stream, int chunk, int nsplit) {
    (void) nsplit;
    if (!scratch) B200_REFUSE(B200_ERR_SCRATCH, "attn_fold: scratch is null");
    if (chunk > 0 && c && c->Hkv > 0 && T > 0)   // the caller's chunk caps the keys per pass (it may be smaller than the scratch allows)
        scratch_bytes = std::min(scratch_bytes, ml_bytes(T, c->Hkv) + tile_bytes(chunk, c->Hkv));
    const pf_io io = {q, nullptr, nullptr, nullptr, nullptr, out, nullptr, nullptr, nullptr, nullptr, nullptr};
    return prefill_run(io, c, T, p0, p0 + T, Hq, scale, scratch, scratch_bytes, (cudaStream_t) stream, "attn_fold");
}
int b200_attn_prefill_gated(const float * q, const b200_kv_cache * c, float * out, const float * gate, int T, int p0, int Hq,
                            float scale, void * scratch, size_t scratch_bytes, void * stream) {
    const pf_io io = {q, nullptr, nullptr, gate, nullptr, out, nullptr, nullptr, nullptr, nullptr, nullptr};
    return prefill_run(io, c, T, p0, p0 + T, Hq, scale, scratch, scratch_bytes, (cudaStream_t) stream, "attn_prefill_gated");
}
int b200_attn_prefill_gated_a16(const float * q, const b200_kv_cache * c, float * out, const float * gate, void * qbuf, int T, int p0,
                                int Hq, float scale, void * scratch, size_t scratch_bytes, void * stream) {
    if (!qbuf || !out) B200_REFUSE(B200_ERR_SHAPE, "attn_prefill_gated_a16: out / qbuf is null");
    const pf_io io = {q, nullptr, nullptr, gate, nullptr, out, nullptr, nullptr, nullptr, qbuf, nullptr};
    return prefill_run(io, c, T, p0, p0 + T, Hq, scale, scratch, scratch_bytes, (cudaStream_t) stream, "attn_prefill_gated_a16");
}
int b200_attn_prefill_partial(const float * q, const b200_kv_cache * c, float * part_o, float * part_m, float * part_l,
                              const int32_t * last_key, int max_keys, int T, int Hq, float scale, void * scratch, size_t scratch_bytes,
                              void * stream) {
    if (!last_key || !part_o || !part_m || !part_l) B200_REFUSE(B200_ERR_SHAPE, "attn_prefill_partial: null argument");
    const pf_io io = {q, nullptr, nullptr, nullptr, nullptr, part_o, nullptr, part_m, part_l, nullptr, last_key};
    return prefill_run(io, c, T, 0, max_keys, Hq, scale, scratch, scratch_bytes, (cudaStream_t) stream, "attn_prefill_partial");
}

size_t b200_attn_prefill_bf16_scratch_bytes(int T, int Hkv, int pass_keys, int out_is_bf16) {
    if (T < 1 || Hkv < 1) return 0;
    const size_t carry = out_is_bf16 ? align256((size_t) T * Hkv * GQA * DH * sizeof(float)) : 0;
    return align256((size_t) T * 64 * sizeof(float)) + ml_bytes(T, Hkv) + carry + tile_bytes(pass_keys > 0 ? pass_keys : DEFAULT_PASS_KEYS, Hkv);
}
int b200_attn_prefill_bf16(const uint16_t * q, const uint16_t * k, const uint16_t * v, const float * gate_f32,
                           const uint16_t * gate_bf16, float * out_f32, uint16_t * out_bf16, void * qbuf, const b200_kv_cache * c,
                           int p0, int T, int Hq, int n_rot, float freq_base, float scale, void * scratch, size_t scratch_bytes,
                           void * stream) {
    const char * who = "attn_prefill_bf16";
    if (!q || !k || !v || !c || !scratch) B200_REFUSE(B200_ERR_SHAPE, "%s: null argument (scratch is required)", who);
    if (n_rot != 64 || c->D != DH || T < 1) B200_REFUSE(B200_ERR_SHAPE, "%s: needs D = 256 and n_rot = 64 (got D=%d n_rot=%d)", who, c->D, n_rot);
    if (((uintptr_t) scratch & 255)) B200_REFUSE(B200_ERR_SCRATCH, "%s: scratch must be 256-byte aligned", who);
    const size_t cs_bytes = align256((size_t) T * 64 * sizeof(float));
    if (scratch_bytes <= cs_bytes) B200_REFUSE(B200_ERR_SCRATCH, "%s: scratch too small", who);
    float * cs = reinterpret_cast<float *>(scratch);
    // K: rotation + quantise + append, V: quantise + append; the tokens' cos / sin go to the table the attention kernel reads
    const int rc = rope_append_launch(nullptr, k, v, nullptr, cs, c, p0, T, Hq, c->Hkv, DH, n_rot, freq_base, (cudaStream_t) stream, who);
    if (rc != B200_OK) return rc;
    const pf_io io = {nullptr, (const __nv_bfloat16 *) q, cs, gate_f32, (const __nv_bfloat16 *) gate_bf16, out_f32,
                      (__nv_bfloat16 *) out_bf16, nullptr, nullptr, qbuf, nullptr};
    return prefill_run(io, c, T, p0, p0 + T, Hq, scale, (unsigned char *) scratch + cs_bytes, scratch_bytes - cs_bytes,
                       (cudaStream_t) stream, who);
}

}  // extern "C"
