// Chunked causal prefill attention over the paged f16 / q8_0 / q4_0 cache on the sm_100a tensor cores (tcgen05 + TMEM).
//
// Two kernels per call:
//   kv_tiles_k   dequantises the visible keys once into f16 "tile images" in scratch: per (kv head, 64-key tile) a
//                32 KB K image and a 32 KB V image laid out exactly as the tensor core reads them from shared memory
//                (un-swizzled canonical layout, see umma.cuh), so the main kernel fetches a tile with one bulk copy.
//   prefill_k    one CTA per (128 query rows of one kv head): rows n = 6 t + hh (token t, head hh of the GQA group) on
//                the MMA M axis.  Per 64-key tile: S = Q K^T (tcgen05.mma, fp32 in tensor memory), online softmax in
//                base 2 with one thread per row (no shuffles), P written as f16 over the S columns it came from (P V
//                takes its A operand from tensor memory), O += P V accumulated in tensor memory.  Warp roles: 4 softmax
//                warps, 1 bulk-copy producer warp, 1 MMA-issue warp; S of tile j+1 is computed (second S buffer in tensor
//                memory) while the softmax of tile j runs.  The running output is rescaled only when a row's maximum
//                grows by more than 2^8 (P stays below 256 in f16).  Epilogue: O / l, optional sigmoid gate.
// f16 operands (int8 * f16 scale is not representable in bf16's 8 significand bits), fp32 accumulation.
//
// Reference counterparts: attn_fold (src/fast/attn_fold.cu:562-649: per chunk dequantise to f16 in scratch, HFMA2 tile
// GEMMs on CUDA cores), attn_prefill (src/fast/attn.cu:457-499, fp32 CUDA cores).
#include "umma.cuh"

#include <algorithm>
#include <mutex>

namespace b200 {
namespace {

constexpr int BM = 128;                 // query rows per CTA
constexpr int BN = 64;                  // keys per tile
constexpr int IMG = BN * DH * 2;        // bytes of one tile image (32 KB)
constexpr int Q_BYTES = BM * DH * 2;    // 64 KB
constexpr int EPI_BYTES = 4 * 32 * 33 * 4;   // per softmax warp a 32 x 33 float tile for the row-wise epilogue
constexpr int NTHR_PF = 192;            // 4 softmax warps + producer + MMA issuer
constexpr float LOG2E_PF = 1.4426950408889634f;
constexpr float RESCALE_GAP = 8.0f;     // rescale O when a row maximum grows by more than this (log2 units)

constexpr int NSTG = 3;                 // K and V ring depth (Q lives in tensor memory, not in shared memory)
constexpr int SM_K = 0;                         // NSTG stages
constexpr int SM_V = SM_K + NSTG * IMG;         // NSTG stages
constexpr int SM_EPI = SM_V + NSTG * IMG;       // epilogue tiles
constexpr int SM_BAR = SM_EPI + EPI_BYTES;      // mbarriers + tmem base
constexpr int SM_TOTAL = SM_BAR + 256;

// ---- pre-pass: cache rows -> f16 tile images -------------------------------------------------------------------
// grid (n_tiles, Hkv), 256 threads; thread = (key, 8-dim chunk).  Image byte of (key, dim) = (dim/8)*1024 + key*16 +
// (dim%8)*2 for K (K-major B operand) and for V (MN-major B operand) alike.  Keys >= n_keys are zero.
template <uint32_t KT>
__global__ void __launch_bounds__(256) kv_tiles_k(kv_view g, int n_keys, unsigned char * __restrict__ tiles, int n_tiles,
                                                  unsigned * status) {
    const int tile = blockIdx.x, hk = blockIdx.y;
    unsigned char * kimg = tiles + ((size_t) hk * n_tiles + tile) * (2 * IMG);
    unsigned char * vimg = kimg + IMG;
    const int32_t * tab = kv_tab(g, 0);
    for (int i = threadIdx.x; i < BN * 32; i += 256) {
        const int key = i & (BN - 1), dc = i >> 6;
        const int kk = tile * BN + key;
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
        *reinterpret_cast<uint4 *>(kimg + dc * 1024 + key * 16) = ko;
        *reinterpret_cast<uint4 *>(vimg + dc * 1024 + key * 16) = vo;
    }
}

struct pf_args {
    const float * q;          // [T][Hq][256]
    const float * gate;       // [T][Hq*256] or nullptr
    float * out;              // [T][Hq][256]
    const unsigned char * tiles;
    int n_tiles;              // tiles per head in scratch
    int T, p0, Hq, Hkv;
    float qscale;             // softmax scale * log2(e)
    unsigned * status;
};

// 1 / (1 + 2^(-g log2 e)) with the hardware exponential and reciprocal (relative error ~1e-7 against expf and an IEEE divide)
__device__ __forceinline__ float fast_sigmoid(float g) { return __fdividef(1.0f, 1.0f + ex2f(-g * LOG2E_PF)); }

__device__ __forceinline__ void mbar_arrive(uint64_t * bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(NTHR_PF, 1) prefill_k(const pf_args a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t * bars = reinterpret_cast<uint64_t *>(smem + SM_BAR);
    uint64_t * k_full = bars, * k_free = bars + 4, * v_full = bars + 8, * v_free = bars + 12, * s_full = bars + 16,
             * p_full = bars + 20, * pv_done = bars + 22, * o_done = bars + 24, * q_ready = bars + 25;
    uint32_t * tbase_p = reinterpret_cast<uint32_t *>(bars + 26);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int mtile = (int) gridDim.x - 1 - (int) blockIdx.x;   // heaviest (latest rows) first
    const int hk = blockIdx.y;
    const int R = a.T * GQA;                                    // rows of this kv head
    const int n0 = mtile * BM;
    const int t_last = min(n0 + BM - 1, R - 1) / GQA;           // last token of the tile
    const int n_keys_vis = a.p0 + t_last + 1;                   // keys any row of the tile can see
    const int ntiles = (n_keys_vis + BN - 1) / BN;

    if (tid == 0) {
        for (int b = 0; b < NSTG; ++b) {
            mbar_init(&k_full[b], 1); mbar_init(&k_free[b], 1);
            mbar_init(&v_full[b], 1); mbar_init(&v_free[b], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&s_full[b], 1);
            mbar_init(&p_full[b], 128); mbar_init(&pv_done[b], 1);
        }
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
    const uint32_t t_S = tb, t_O = tb + 2 * BN, t_Q = tb + 2 * BN + DH;   // S x2 at columns 0 / 64, O at 128..383, Q (f16 pairs) at 384..511

    if (warp < 4) {
        // Q rows -> f16, scaled by softmax scale * log2(e), into tensor memory as the A operand of Q K^T: thread = row =
        // lane, column c holds dims 2c, 2c+1.  64 dims per slab: 16 loads in flight per thread.
        const int n = n0 + tid;
        const uint32_t lane_off = (uint32_t) (warp * 32) << 16;
        const float4 * src = nullptr;
        if (n < R) {
            const int t = n / GQA, hh = n - t * GQA;
            src = reinterpret_cast<const float4 *>(a.q + ((size_t) t * a.Hq + hk * GQA + hh) * DH);
        }
#pragma unroll 1
        for (int d0 = 0; d0 < DH; d0 += 64) {
            float4 x[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) x[u] = src ? __ldg(src + d0 / 4 + u) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            uint32_t w[32];
            const float sc = a.qscale;
#pragma unroll
            for (int u = 0; u < 16; ++u) { w[2 * u] = pack_h2(x[u].x * sc, x[u].y * sc); w[2 * u + 1] = pack_h2(x[u].z * sc, x[u].w * sc); }
            umma::tmem_st32(t_Q + lane_off + d0 / 2, w);
        }
        umma::tmem_st_wait();
        umma::fence_before_sync();
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the four softmax warps: every Q row is in place
        if (tid == 0) mbar_arrive(q_ready);
    }
    if (warp >= 4 && a.gate && (lane & 15) != 0) {
        // idle lanes of the producer and MMA warps pull this CTA's gate rows (contiguous per token: 6 heads x 1 KB) into L2
        const int t_first = n0 / GQA;
        const char * g0 = reinterpret_cast<const char *>(a.gate + ((size_t) t_first * a.Hq + hk * GQA) * DH);
        const int idx = (warp - 4) * 30 + lane - 1 - (lane > 16);
        for (int t = t_first; t <= t_last; ++t)
            for (int ln = idx; ln < GQA * DH * 4 / 128; ln += 60)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(g0 + (size_t) (t - t_first) * a.Hq * DH * 4 + ln * 128));
    }
    if (warp == 4) {
        // ---------------- producer: one bulk copy per image; K (lane 0) and V (lane 16) rings run independently ----------------
        const unsigned char * src = a.tiles + (size_t) hk * a.n_tiles * (2 * IMG);
        if (lane == 0) {
            for (int j = 0; j < ntiles; ++j) {
                const int s = j % NSTG;
                if (j >= NSTG) mbar_wait(&k_free[s], (uint32_t) ((j / NSTG - 1) & 1), a.status);   // Q K^T of tile j-NSTG has read the stage
                mbar_expect_tx(&k_full[s], IMG);
                bulk_g2s(smem + SM_K + s * IMG, src + (size_t) j * (2 * IMG), IMG, &k_full[s]);
            }
        } else if (lane == 16) {
            for (int j = 0; j < ntiles; ++j) {
                const int s = j % NSTG;
                if (j >= NSTG) mbar_wait(&v_free[s], (uint32_t) ((j / NSTG - 1) & 1), a.status);   // P V of tile j-NSTG has read the stage
                mbar_expect_tx(&v_full[s], IMG);
                bulk_g2s(smem + SM_V + s * IMG, src + (size_t) j * (2 * IMG) + IMG, IMG, &v_full[s]);
            }
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer: Q K^T of tile j+1 is queued before P V of tile j ----------------
        if (lane == 0) {
            constexpr uint32_t id_qk = umma::idesc_f16(BM, BN, false, false);   // S[128 x 64] = Q (K-major) * K^T (K-major)
            constexpr uint32_t id_pv = umma::idesc_f16(BM, DH, false, true);    // O[128 x 256] += P (K-major) * V (MN-major)
            auto issue_qk = [&](int j) {
                const int b = j & 1, st = j % NSTG;
                mbar_wait(&k_full[st], (uint32_t) ((j / NSTG) & 1), a.status);
                // S buffer b still holds P of tile j-2 until P V of that tile has read it: that MMA was issued before this
                // one by this thread, and the tensor pipe runs in issue order, so no barrier is needed
                umma::fence_after_sync();
                const uint32_t k_s = smem_u32(smem + SM_K + st * IMG);
#pragma unroll 4
                for (int ks = 0; ks < DH / 16; ++ks)
                    umma::mma_ts(t_S + b * BN, t_Q + ks * 8, umma::smem_desc(k_s + ks * 2 * 1024, 1024, 128), id_qk, ks > 0);   // Q from tensor memory
                umma::commit(&s_full[b]);
                umma::commit(&k_free[st]);
            };
            mbar_wait(q_ready, 0, a.status);
            umma::fence_after_sync();
            issue_qk(0);
            for (int j = 0; j < ntiles; ++j) {
                if (j + 1 < ntiles) issue_qk(j + 1);
                const int b = j & 1, st = j % NSTG;
                mbar_wait(&v_full[st], (uint32_t) ((j / NSTG) & 1), a.status);
                mbar_wait(&p_full[b], (uint32_t) ((j >> 1) & 1), a.status);
                umma::fence_after_sync();
                const uint32_t v_s = smem_u32(smem + SM_V + st * IMG);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks)   // P from tensor memory (the first 32 columns of S buffer b: 16 keys = 8 columns
                                                       // per step); V image: MN-major, key groups of 8 contiguous (LBO 128), dim groups 1024 apart
                    umma::mma_ts(t_O, t_S + b * BN + ks * 8, umma::smem_desc(v_s + ks * 2 * 128, 128, 1024),
                                 id_pv, (j > 0 || ks > 0) ? 1u : 0u);
                umma::commit(&v_free[st]);
                umma::commit(&pv_done[b]);
            }
            umma::commit(o_done);
        }
    } else {
        // ---------------- softmax: thread = row ----------------
        const int r = tid, n = n0 + r;
        const int t_row = n / GQA;
        const int pos = n < R ? a.p0 + t_row : -1;
        const uint32_t lane_off = (uint32_t) (warp * 32) << 16;
        float m_ref = B200_NEG_INF, l = 0.0f;
        for (int j = 0; j < ntiles; ++j) {
            mbar_wait(&s_full[j & 1], (uint32_t) ((j >> 1) & 1), a.status);
            umma::fence_after_sync();
            uint32_t sr[2][32];
            umma::tmem_ld32(t_S + (j & 1) * BN + lane_off, sr[0]);
            umma::tmem_ld32(t_S + (j & 1) * BN + lane_off + 32, sr[1]);
            umma::tmem_ld_wait();
            const int k0 = j * BN;
            const bool diag = k0 + BN - 1 > pos;   // some key of the tile is masked for this row
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
            // lazy rescale: only when some row of the warp outgrew its reference maximum
            const bool grow = mx > m_ref + RESCALE_GAP || (m_ref == B200_NEG_INF && mx != B200_NEG_INF);
            if (__any_sync(0xffffffffu, grow)) {
                float f = 1.0f;
                if (grow) {
                    f = m_ref == B200_NEG_INF ? 0.0f : ex2f(m_ref - mx);
                    m_ref = mx;
                    l *= f;
                }
                if (j > 0) {
                    mbar_wait(&pv_done[(j - 1) & 1], (uint32_t) (((j - 1) >> 1) & 1), a.status);   // P V of tile j-1 has landed in O
                    umma::fence_after_sync();
#pragma unroll 1
                    for (int c0 = 0; c0 < DH; c0 += 32) {
                        uint32_t o[32];
                        umma::tmem_ld32(t_O + lane_off + c0, o);
                        umma::tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
                        umma::tmem_st32(t_O + lane_off + c0, o);
                    }
                    umma::tmem_st_wait();
                }
            }
            const float mref_safe = m_ref == B200_NEG_INF ? 0.0f : m_ref;
            // P (f16) overwrites the first 32 columns of this S buffer: column c of the row's lane = keys 2c, 2c+1, the A
            // operand layout of P V.  S is in registers by now, and the next Q K^T into this buffer is queued behind P V.
            uint32_t pw[32];
            float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int c2 = 0; c2 < 16; ++c2) {
                    // ex2(-inf) = 0: masked keys need no special case (mref_safe is finite)
                    const float p0 = ex2f(__uint_as_float(sr[h][2 * c2]) - mref_safe);
                    const float p1 = ex2f(__uint_as_float(sr[h][2 * c2 + 1]) - mref_safe);
                    l4[c2 & 3] += p0 + p1;
                    pw[16 * h + c2] = pack_h2(p0, p1);
                }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            umma::tmem_st32(t_S + (j & 1) * BN + lane_off, pw);
            umma::tmem_st_wait();
            umma::fence_before_sync();
            mbar_arrive(&p_full[j & 1]);
        }
        // ---------------- epilogue: O / l, gate, store ----------------
        mbar_wait(o_done, 0, a.status);
        umma::fence_after_sync();
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        // Each warp owns the 32 rows of its tensor-memory lanes.  A 32-column slab of O goes through a private
        // shared-memory tile so that global accesses run along rows: 8 lanes cover the 128
        // bytes of one row, a warp instruction touches 4 rows.
        float * tile = reinterpret_cast<float *>(smem + SM_EPI) + warp * (32 * 33);
        const int sub = lane >> 3, col = 4 * (lane & 7);
        size_t orow[8];
        bool live[8];
#pragma unroll
        for (int q8 = 0; q8 < 8; ++q8) {
            const int nr = n0 + warp * 32 + 4 * q8 + sub;
            const int tr = nr / GQA, hr = nr - tr * GQA;
            live[q8] = nr < R;
            orow[q8] = ((size_t) tr * a.Hq + hk * GQA + hr) * DH + col;
        }
        float4 gn[8];   // gate values of the next slab, requested one slab ahead
#pragma unroll
        for (int q8 = 0; q8 < 8; ++q8)
            gn[q8] = (a.gate && live[q8]) ? __ldg(reinterpret_cast<const float4 *>(a.gate + orow[q8])) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int c0 = 0; c0 < DH; c0 += 32) {
            float4 gv[8];
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) {
                gv[q8] = gn[q8];
                if (a.gate && live[q8] && c0 + 32 < DH) gn[q8] = __ldg(reinterpret_cast<const float4 *>(a.gate + orow[q8] + c0 + 32));
            }
            uint32_t o[32];
            umma::tmem_ld32(t_O + lane_off + c0, o);
            umma::tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) tile[lane * 33 + c] = __uint_as_float(o[c]) * inv;
            __syncwarp();
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) {
                const int rl = 4 * q8 + sub;
                if (live[q8]) {
                    float4 y = make_float4(tile[rl * 33 + col], tile[rl * 33 + col + 1], tile[rl * 33 + col + 2], tile[rl * 33 + col + 3]);
                    if (a.gate) {
                        y.x *= fast_sigmoid(gv[q8].x); y.y *= fast_sigmoid(gv[q8].y);
                        y.z *= fast_sigmoid(gv[q8].z); y.w *= fast_sigmoid(gv[q8].w);
                    }
                    *reinterpret_cast<float4 *>(a.out + orow[q8] + c0) = y;
                }
            }
            __syncwarp();
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tb, 512);
}

// ------------------------------------------------------------------------------------------------ host side ----
size_t scratch_need(int n_keys, int Hkv) {
    const size_t n_tiles = (size_t) (n_keys + BN - 1) / BN;
    return n_tiles * Hkv * (2 * IMG) + 256;
}

struct own_scratch { int dev = -1; void * p = nullptr; size_t cap = 0; };
own_scratch g_own[16];
std::mutex g_pf_mu;

void * own_scratch_for(size_t bytes, cudaStream_t s) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(g_pf_mu);
    own_scratch & e = g_own[dev & 15];
    if (bytes > e.cap) {
        if (e.p) { cudaStreamSynchronize(s); cudaFree(e.p); e.p = nullptr; e.cap = 0; }
        if (cudaMalloc(&e.p, bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        e.cap = bytes;
    }
    return e.p;
}

int prefill_impl(const float * q, const b200_kv_cache * c, float * out, const float * gate, int T, int p0, int Hq, float scale,
                 void * scratch, size_t scratch_bytes, cudaStream_t s, const char * who) {
    if (!c || !q || !out || !c->k || !c->v) B200_REFUSE(B200_ERR_SHAPE, "%s: null argument", who);
    if (c->D != DH || Hq != GQA * c->Hkv || c->Hkv <= 0 || T < 1 || p0 < 0)
        B200_REFUSE(B200_ERR_SHAPE, "%s: unsupported shape (D=%d Hq=%d Hkv=%d T=%d p0=%d)", who, c->D, Hq, c->Hkv, T, p0);
    if (c->type != B200_KV_F16 && c->type != B200_KV_Q8_0 && c->type != B200_KV_Q4_0) B200_REFUSE(B200_ERR_SHAPE, "%s: unsupported cache type %u", who, c->type);
    if (!aligned16(c->k) || !aligned16(c->v) || !aligned16(q) || !aligned16(out) || (gate && !aligned16(gate)) || (c->pt && c->pstride % 16))
        B200_REFUSE(B200_ERR_SHAPE, "%s: cache base, page stride, q, out and gate must be 16-byte aligned", who);
    if (!c->pt && p0 + T > c->n_ctx) B200_REFUSE(B200_ERR_SHAPE, "%s: rows %d..%d outside n_ctx %d", who, p0, p0 + T - 1, c->n_ctx);
    const int n_keys = p0 + T;
    const size_t need = scratch_need(n_keys, c->Hkv);
    if (!scratch) {
        scratch = own_scratch_for(need, s);
        if (!scratch) B200_REFUSE(B200_ERR_ALLOC, "%s: %zu bytes of scratch could not be allocated", who, need);
    } else if (scratch_bytes < need || ((uintptr_t) scratch & 255)) {
        B200_REFUSE(B200_ERR_SCRATCH, "%s: scratch too small or not 256-byte aligned (%zu bytes given, %zu needed for %d keys)", who,
                    scratch_bytes, need, n_keys);
    }
    unsigned * st = device_status_word();
    if (!st) return B200_ERR_CUDA;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63]) {
        if (cudaFuncSetAttribute(prefill_k, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL) != cudaSuccess)
            return launch_status("attn_prefill (shared memory attribute)");
        attr_done[dev & 63] = true;
    }
    const int n_tiles = (n_keys + BN - 1) / BN;
    const kv_view g = view_of(*c);
    const dim3 tg(n_tiles, c->Hkv);
    if (c->type == B200_KV_F16) kv_tiles_k<B200_KV_F16><<<tg, 256, 0, s>>>(g, n_keys, (unsigned char *) scratch, n_tiles, st);
    else if (c->type == B200_KV_Q8_0) kv_tiles_k<B200_KV_Q8_0><<<tg, 256, 0, s>>>(g, n_keys, (unsigned char *) scratch, n_tiles, st);
    else kv_tiles_k<B200_KV_Q4_0><<<tg, 256, 0, s>>>(g, n_keys, (unsigned char *) scratch, n_tiles, st);
    pf_args a;
    a.q = q; a.gate = gate; a.out = out; a.tiles = (const unsigned char *) scratch; a.n_tiles = n_tiles;
    a.T = T; a.p0 = p0; a.Hq = Hq; a.Hkv = c->Hkv; a.qscale = scale * LOG2E_PF; a.status = st;
    const int n_mtiles = (T * GQA + BM - 1) / BM;
    prefill_k<<<dim3(n_mtiles, c->Hkv), NTHR_PF, SM_TOTAL, s>>>(a);
    count_launch(2);
    return launch_status(who);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_attn_prefill(const float * q, const b200_kv_cache * c, float * out, int T, int p0, int Hq, float scale, void * stream) {
    return prefill_impl(q, c, out, nullptr, T, p0, Hq, scale, nullptr, 0, (cudaStream_t) stream, "attn_prefill");
}
int b200_attn_prefill_variant(const float * q, const b200_kv_cache * c, float * out, int T, int p0, int Hq, float scale, void * stream,
                              int variant) {
    (void) variant;   // the reference's variants are bitwise-equal schedules of one fp32 algorithm; there is one kernel here
    return prefill_impl(q, c, out, nullptr, T, p0, Hq, scale, nullptr, 0, (cudaStream_t) stream, "attn_prefill");
}
// scratch for a call whose visible context (p0 + T) is at most `chunk` keys; chunk <= 0: T keys (p0 = 0). nsplit unused.
size_t b200_attn_fold_scratch_bytes(int T, int Hkv, int chunk, int nsplit) {
    (void) nsplit;
    return scratch_need(chunk > 0 ? chunk : T, Hkv);
}
int b200_attn_fold(const float * q, const b200_kv_cache * c, float * out, int T, int p0, int Hq, float scale, void * scratch,
                   size_t scratch_bytes, void * stream, int chunk, int nsplit) {
    (void) chunk; (void) nsplit;
    if (!scratch) B200_REFUSE(B200_ERR_SCRATCH, "attn_fold: scratch is null");
    return prefill_impl(q, c, out, nullptr, T, p0, Hq, scale, scratch, scratch_bytes, (cudaStream_t) stream, "attn_fold");
}
int b200_attn_prefill_gated(const float * q, const b200_kv_cache * c, float * out, const float * gate, int T, int p0, int Hq,
                            float scale, void * scratch, size_t scratch_bytes, void * stream) {
    return prefill_impl(q, c, out, gate, T, p0, Hq, scale, scratch, scratch_bytes, (cudaStream_t) stream, "attn_prefill_gated");
}

}  // extern "C"
