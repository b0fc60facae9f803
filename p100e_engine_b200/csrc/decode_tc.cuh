// Batched decode / verify on the 5th-generation tensor cores (tcgen05), for quantised caches and the even split of a
// batch over the SMs.  Included by attn_decode.cu inside its namespace (dec_args, traits, the tensor maps and the split
// plan are defined there).
//
// One CTA per SM walks its run of keys in tiles of 128.  Per tile and kv head:
//   K rows (TMA -> staging) --16 worker warps: int8 / nibble -> f16 * block scale--> tensor memory, lane = key
//   S^T[128 keys x rows]  = K (A operand in tensor memory) * Q^T (B operand, K-major image in shared memory)
//   V rows (TMA -> staging) --workers--> f16 image [key][dim] in shared memory
//   workers: S^T -> mask -> P = 2^(S - reference maximum + 8) as f16 -> P image [row][key] in shared memory
//   O[rows x 256] += P (A operand, shared memory) * V (B operand, MN-major image)
// The MMAs and the TMA copies are issued by one thread of a 17th warp; the workers meet it through mbarriers only, and each
// other once per tile (the vote on "some score outgrew its reference maximum").  Against the mma.sync kernel this takes
// the multiply-adds, the fragment shuffling and the per-tile accumulator traffic out of the instruction stream: what the
// CUDA cores still do is the widening of 2 x 128 x 256 cache values per tile and 128 x rows exponentials.
//
// Every wait is bounded (mbar_wait gives up after two seconds and records ST_WAIT_TIMEOUT).

constexpr int UT = 128;                       // keys per tile
constexpr int TC_WORKERS = 512, TC_THR = TC_WORKERS + 32;
constexpr int TC_NBUF = 3;                    // staging ring: K(i), V(i), K(i+1), V(i+1), .. walk three buffers
constexpr int TC_HDR = 2048;                  // barriers, reference maxima, exchange arrays, page entries
constexpr int TC_PGS = 256;                   // page-table entries of a run kept in shared memory
constexpr int TC_VF = UT * DH * 2;            // f16 image of a tile's V rows
constexpr int TC_QI = 32 * 32 * 16;           // f16 image of up to 32 query rows
constexpr int TC_PLBO = 528;                  // bytes between the 8-key chunks of the P image (512 + 16: stores of a warp spread over the banks)
constexpr int TC_PI = 10240;                  // P image: 16 chunks, read as 128 rows (rows >= 32 alias the following chunks)

template <uint32_t KT> constexpr size_t tc_smem_bytes() { return TC_HDR + (size_t) TC_NBUF * UT * traits<KT>::HB + TC_VF + TC_QI + TC_PI; }

__device__ __forceinline__ void tc_arrive(uint64_t * bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_bar_workers() { asm volatile("bar.sync 1, %0;" ::"n"(TC_WORKERS) : "memory"); }
__device__ __forceinline__ int tc_vote_workers(int v) {
    int r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.s32 q, %1, 0;\n\tbarrier.red.or.pred p, 1, %2, q;\n\tselp.s32 %0, 1, 0, p;\n\t}"
                 : "=r"(r) : "r"(v), "n"(TC_WORKERS) : "memory");
    return r;
}

// One 32-value block of a cache row -> 16 registers of f16 pairs (register m = dims 2m, 2m+1 of the block), each value the
// rounded product of the stored integer and the block's f16 scale.
template <uint32_t KT>
__device__ __forceinline__ void tc_block(const unsigned char * row, int blk, uint32_t (&r)[16]) {
    if constexpr (KT == B200_KV_Q8_0) {
        const uint4 a = *reinterpret_cast<const uint4 *>(row + 16 + 32 * blk), b = *reinterpret_cast<const uint4 *>(row + 32 + 32 * blk);
        const uint32_t sc = *reinterpret_cast<const uint16_t *>(row + 2 * blk);
        const uint32_t d2 = sc | (sc << 16);
        const uint32_t wv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t x = wv[j] ^ 0x80808080u;
            r[2 * j] = hmul2_u32(cvt_i8x2<0>(x), d2);
            r[2 * j + 1] = hmul2_u32(cvt_i8x2<1>(x), d2);
        }
    } else {
        // block at byte 18 blk: f16 scale, then 16 bytes (byte j = dim j | dim j + 16 << 4); 4-byte aligned for even blk
        uint32_t q[4], sc;
        if ((blk & 1) == 0) {
            const uint32_t * p = reinterpret_cast<const uint32_t *>(row + 18 * blk);
            const uint32_t w0 = p[0], w1 = p[1], w2 = p[2], w3 = p[3], w4 = p[4];
            sc = w0 & 0xffffu;
            q[0] = __funnelshift_r(w0, w1, 16); q[1] = __funnelshift_r(w1, w2, 16);
            q[2] = __funnelshift_r(w2, w3, 16); q[3] = __funnelshift_r(w3, w4, 16);
        } else {
            const uint32_t * p = reinterpret_cast<const uint32_t *>(row + 18 * blk - 2);
            sc = p[0] >> 16;
            q[0] = p[1]; q[1] = p[2]; q[2] = p[3]; q[3] = p[4];
        }
        const uint32_t d2 = sc | (sc << 16);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lo = q[j] & 0x0f0f0f0fu, hi = (q[j] >> 4) & 0x0f0f0f0fu;
            r[2 * j] = hmul2_u32(cvt_n4x2<0>(lo), d2);
            r[2 * j + 1] = hmul2_u32(cvt_n4x2<1>(lo), d2);
            r[8 + 2 * j] = hmul2_u32(cvt_n4x2<0>(hi), d2);
            r[8 + 2 * j + 1] = hmul2_u32(cvt_n4x2<1>(hi), d2);
        }
    }
}

// NC = score columns (16 for up to two verify rows, 32 for up to four): column 8 j + h = verify row j, head h of the group
// (h < 6); columns with h = 6, 7 are padding (zero query rows).
template <uint32_t KT, int NC>
__global__ void __launch_bounds__(TC_THR, 1)
decode_tc_k(const dec_args a, const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV) {
    extern __shared__ __align__(1024) unsigned char smem[];
    constexpr int HB = traits<KT>::HB, BUF = UT * HB;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const bool worker = w < TC_WORKERS / 32;
    const int lq = w & 3, gq = (w >> 2) & 3;     // worker warp: tensor-memory lane quarter, column / block group
    const int hk = (int) (blockIdx.x % (unsigned) a.g.Hkv), ui = (int) (blockIdx.x / (unsigned) a.g.Hkv);
    if (ui >= *a.n_cta) return;
    const int s0 = a.cta_seg[ui], s1 = a.cta_seg[ui + 1];
    if (s0 >= s1) return;

    uint64_t * full = reinterpret_cast<uint64_t *>(smem);                       // [TC_NBUF] staging buffer filled
    uint64_t * s_full = full + 4, * pv_done = full + 5, * kconv = full + 6, * p_ready = full + 7;
    uint32_t * tbase_p = reinterpret_cast<uint32_t *>(smem + 64);
    float * mref = reinterpret_cast<float *>(smem + 128);                        // [32] reference maximum per column (log2 units)
    float * fsc = reinterpret_cast<float *>(smem + 256);                         // [32] rescale factor of the last move
    float * wx = reinterpret_cast<float *>(smem + 384);                          // [4][32] per lane quarter: maxima / sums
    int * pgs = reinterpret_cast<int *>(smem + 1024);                            // [TC_PGS]
    unsigned char * stg = smem + TC_HDR, * VF = stg + TC_NBUF * BUF, * QI = VF + TC_VF, * PI = QI + TC_QI;

    if (tid == 0) {
        for (int b = 0; b < TC_NBUF; ++b) mbar_init(&full[b], 1);
        mbar_init(s_full, 1); mbar_init(pv_done, 1);
        mbar_init(kconv, TC_WORKERS / 32); mbar_init(p_ready, TC_WORKERS / 32);
        mbar_fence_init();
    }
    if (w == TC_WORKERS / 32) umma::tmem_alloc(tbase_p, 512);
    for (int i = tid; i < TC_PI / 16; i += TC_THR) reinterpret_cast<uint4 *>(PI)[i] = make_uint4(0, 0, 0, 0);   // padding rows stay zero
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tb = *tbase_p;
    const uint32_t tA = tb, tS = tb + 128, tO = tb + 256;   // K as f16 pairs (128 columns), S^T (NC), O (256)
    const uint32_t lane_off = (uint32_t) (32 * lq) << 16;
    const int R = a.q_len * GQA;

    int g = 0;   // tiles this CTA has walked: parities of the per-tile barriers; 2 g = staging items before the run
    for (int sg = s0; sg < s1; ++sg) {
        const int4 seg = a.segs[sg];
        const int slot = seg.x, k_lo = seg.y;
        const size_t unit = (size_t) sg * a.g.Hkv + hk;
        int n_slot = 0;
        for (int j = 0; j < a.q_len; ++j) n_slot = max(n_slot, row_pos(a, slot, j) + 1);
        {
            const int lim = key_limit(a);
            if (n_slot > lim) { if (tid == 0) atomicOr(a.status, ST_BAD_POS); n_slot = lim; }
        }
        const int k_hi = min(seg.z, n_slot);
        const int nt = k_hi > k_lo ? (k_hi - k_lo + UT - 1) / UT : 0;
        if (nt == 0) continue;
        const int32_t * tab = a.g.pt ? a.g.pt + (a.g.rtab ? a.g.rtab[slot * a.q_len] : 0) : nullptr;
        const int pg0 = tab ? k_lo >> a.g.psh : 0;

        if (worker) {
            if (tab) {
                const int npg = min(TC_PGS, ((k_hi - 1) >> a.g.psh) - pg0 + 1);
                for (int j = tid; j < npg; j += TC_WORKERS) pgs[j] = tab[pg0 + j];
            }
            // Q rows -> f16, scaled, as the K-major B operand: byte(n, d) = (n / 8) * 128 + (d / 8) * (NC * 16) + (n % 8) * 16 + (d % 8) * 2
            for (int i = tid; i < NC * 32; i += TC_WORKERS) {
                const int n = i & (NC - 1), kc = i / NC, grp = n >> 3, hh = n & 7;
                uint4 pk = make_uint4(0, 0, 0, 0);
                if (hh < GQA && grp < a.q_len) {
                    const float4 * src = reinterpret_cast<const float4 *>(a.q + ((size_t) (slot * a.q_len + grp) * a.Hq + hk * GQA + hh) * DH + kc * 8);
                    const float4 v0 = src[0], v1 = src[1];
                    pk = make_uint4(pack_h2(v0.x * a.qscale, v0.y * a.qscale), pack_h2(v0.z * a.qscale, v0.w * a.qscale),
                                    pack_h2(v1.x * a.qscale, v1.y * a.qscale), pack_h2(v1.z * a.qscale, v1.w * a.qscale));
                }
                *reinterpret_cast<uint4 *>(QI + grp * 128 + kc * (NC * 16) + hh * 16) = pk;
            }
            if (tid < 32) mref[tid] = B200_NEG_INF;
            umma::fence_async_smem();
        }
        __syncthreads();

        if (!worker) {
            // ---------------- issuer: TMA copies and MMAs ----------------
            if (lane == 0) {
                auto issue = [&](int q) {   // item q of the run: K rows of tile q / 2 (q even) or its V rows (q odd)
                    if (q >= 2 * nt) return;
                    const int p_t = k_lo + (q >> 1) * UT;
                    const int buf = (2 * g + q) % TC_NBUF;
                    unsigned char * dst = stg + (size_t) buf * BUF;
                    const CUtensorMap * map = (q & 1) ? &mapV : &mapK;
                    const int nbox = p_t + TILE < k_hi ? 2 : 1;   // 64-position boxes that hold keys of the run
                    mbar_expect_tx(&full[buf], (uint32_t) nbox * TILE * HB);
                    for (int h = 0; h < nbox; ++h) {
                        const int p = p_t + h * TILE;
                        int y = p, z = 0;
                        if (tab) {
                            const int idx = (p >> a.g.psh) - pg0;
                            z = idx < TC_PGS ? pgs[idx] : tab[p >> a.g.psh];
                            y = p & ((1 << a.g.psh) - 1);
                            if (z < 0) { atomicOr(a.status, ST_BAD_PAGE); z = 0; }
                        }
                        tma_box3(dst + h * TILE * HB, map, hk * (HB / 2), y, z, &full[buf]);
                    }
                };
                issue(0); issue(1); issue(2);
                constexpr uint32_t id_qk = umma::idesc_f16(UT, NC, false, false);   // S^T[128 x NC] = K (tensor memory) * Q^T (K-major)
                constexpr uint32_t id_pv = umma::idesc_f16(UT, DH, false, true);    // O[128 x 256] += P (K-major) * V (MN-major)
                const uint32_t q_s = smem_u32(QI), p_s = smem_u32(PI), v_s = smem_u32(VF);
                for (int i = 0; i < nt; ++i) {
                    const uint32_t par = (uint32_t) ((g + i) & 1);
                    mbar_wait(kconv, par, a.status);       // every worker warp has written its part of K and is done with the K staging
                    umma::fence_after_sync();
#pragma unroll
                    for (int ks = 0; ks < DH / 16; ++ks)
                        umma::mma_ts(tS, tA + ks * 8, umma::smem_desc(q_s + ks * 2 * (NC * 16), NC * 16, 128), id_qk, ks > 0);
                    umma::commit(s_full);
                    issue(2 * i + 3);
                    mbar_wait(p_ready, par, a.status);     // P and the V image are in place, the V staging is free
                    umma::fence_after_sync();
#pragma unroll
                    for (int ks = 0; ks < UT / 16; ++ks)
                        umma::mma_ss(tO, umma::smem_desc(p_s + ks * 2 * TC_PLBO, TC_PLBO, 128), umma::smem_desc(v_s + ks * 2 * 4096, 4096, 128),
                                     id_pv, (i > 0 || ks > 0) ? 1u : 0u);
                    umma::commit(pv_done);
                    issue(2 * i + 4);
                }
            }
            __syncwarp();
        } else {
            // ---------------- workers ----------------
            const bool act = gq < a.q_len && gq < NC / 8;           // this warp's columns 8 gq .. 8 gq + 5 hold verify row gq
            const int pos_g = act ? row_pos(a, slot, gq) : -1;
            float l_acc[GQA];
#pragma unroll
            for (int e = 0; e < GQA; ++e) l_acc[e] = 0.0f;
            for (int i = 0; i < nt; ++i) {
                const int gi = g + i, p_t = k_lo + i * UT;
                // ---- K rows -> tensor memory (lane = key; this warp: blocks 2 gq, 2 gq + 1 of keys 32 lq ..)
                {
                    const int qi = 2 * gi, buf = qi % TC_NBUF;
                    mbar_wait(&full[buf], (uint32_t) ((qi / TC_NBUF) & 1), a.status);
                    const unsigned char * row = stg + (size_t) buf * BUF + (32 * lq + lane) * HB;
#pragma unroll
                    for (int bb = 0; bb < 2; ++bb) {
                        uint32_t r[16];
                        tc_block<KT>(row, 2 * gq + bb, r);
                        umma::tmem_st16(tA + lane_off + (2 * gq + bb) * 16, r);
                    }
                    umma::tmem_st_wait();
                    umma::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) tc_arrive(kconv);
                }
                // ---- V rows -> f16 image, MN-major: byte(key, d) = (d / 8) * 128 + (key / 8) * 4096 + (key % 8) * 16 + (d % 8) * 2
                {
                    const int qi = 2 * gi + 1, buf = qi % TC_NBUF;
                    mbar_wait(&full[buf], (uint32_t) ((qi / TC_NBUF) & 1), a.status);
                    if (gi > 0) mbar_wait(pv_done, (uint32_t) ((gi - 1) & 1), a.status);   // the previous P V has read the image and P
                    const int key = tid & (UT - 1), kb = tid >> 7;
                    const unsigned char * row = stg + (size_t) buf * BUF + key * HB;
                    const bool valid = p_t + key < k_hi;   // rows past the run's last key may hold anything: they enter as zeros
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int blk = kb + 4 * u;
                        uint32_t r[16];
                        if (valid) tc_block<KT>(row, blk, r);
                        else {
#pragma unroll
                            for (int c = 0; c < 16; ++c) r[c] = 0u;
                        }
                        unsigned char * dst = VF + (4 * blk) * 128 + (key >> 3) * 4096 + (key & 7) * 16;
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            *reinterpret_cast<uint4 *>(dst + c * 128) = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
                    }
                }
                // ---- scores of this thread's key for the six heads of verify row gq
                mbar_wait(s_full, (uint32_t) (gi & 1), a.status);
                umma::fence_after_sync();
                float s[GQA];
                int grow = 0;
                if (act) {
                    uint32_t sr[8];
                    umma::tmem_ld8(tS + lane_off + 8 * gq, sr);
                    umma::tmem_ld_wait();
                    const int key_abs = p_t + 32 * lq + lane;
                    const bool masked = key_abs > pos_g || key_abs >= k_hi;
#pragma unroll
                    for (int e = 0; e < GQA; ++e) {
                        s[e] = masked ? B200_NEG_INF : __uint_as_float(sr[e]);
                        grow |= s[e] > mref[8 * gq + e] + REF_GAP;
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < GQA; ++e) s[e] = B200_NEG_INF;
                }
                // A column's reference maximum trails its true maximum by at most REF_GAP; it moves (and O, l are rescaled)
                // only when some key of the tile outgrows it, which the workers find out with one vote per tile.
                if (tc_vote_workers(grow)) {
                    if (act) {
#pragma unroll
                        for (int e = 0; e < GQA; ++e) {
                            float mx = s[e];
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                            if (lane == 0) wx[lq * 32 + 8 * gq + e] = mx;
                        }
                    }
                    tc_bar_workers();
                    if (tid < 32) {
                        float f = 1.0f;
                        if ((tid >> 3) < a.q_len && (tid & 7) < GQA) {
                            const float mx = fmaxf(fmaxf(wx[tid], wx[32 + tid]), fmaxf(wx[64 + tid], wx[96 + tid]));
                            const float m_old = mref[tid];
                            if (mx > m_old + REF_GAP) { f = ex2f(m_old - mx); mref[tid] = mx; }   // 2^(-inf) = 0 on the first move
                        }
                        fsc[tid] = f;
                    }
                    tc_bar_workers();
                    if (act) {
#pragma unroll
                        for (int e = 0; e < GQA; ++e) l_acc[e] *= fsc[8 * gq + e];
                    }
                    if (lq == 0 && i > 0) {   // O rows live in lanes 0..31: the four warps of lane quarter 0 take 64 columns each
                        const float f = fsc[lane];
                        if (__any_sync(0xffffffffu, f != 1.0f)) {
#pragma unroll 1
                            for (int h = 0; h < 2; ++h) {
                                uint32_t o[32];
                                umma::tmem_ld32(tO + 64 * gq + 32 * h, o);
                                umma::tmem_ld_wait();
#pragma unroll
                                for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
                                umma::tmem_st32(tO + 64 * gq + 32 * h, o);
                            }
                            umma::tmem_st_wait();
                        }
                    }
                }
                // ---- P = 2^(S - reference + 8) as f16 into the K-major A image: byte(row, key) = (row / 8) * 128 + (key / 8) * TC_PLBO + (row % 8) * 16 + (key % 8) * 2
                if (act) {
                    const int kk = 32 * lq + lane;
                    unsigned char * pd = PI + gq * 128 + (kk >> 3) * TC_PLBO + (kk & 7) * 2;
#pragma unroll
                    for (int e = 0; e < GQA; ++e) {
                        const float m = mref[8 * gq + e];
                        const __half p = __float2half_rn(ex2f(s[e] - (m == B200_NEG_INF ? 0.0f : m) + PSHIFT));
                        l_acc[e] += __half2float(p);
                        *reinterpret_cast<__half *>(pd + e * 16) = p;
                    }
                }
                umma::fence_async_smem();
                umma::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc_arrive(p_ready);
            }
            // ---------------- the run's partial (O, reference maximum, sum) ----------------
            mbar_wait(pv_done, (uint32_t) ((g + nt - 1) & 1), a.status);
            umma::fence_after_sync();
            if (act) {
#pragma unroll
                for (int e = 0; e < GQA; ++e) {
                    float v = l_acc[e];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (lane == 0) wx[lq * 32 + 8 * gq + e] = v;
                }
            }
            tc_bar_workers();
            if (tid < 32 && (tid >> 3) < a.q_len && (tid & 7) < GQA) {
                const int r = (tid >> 3) * GQA + (tid & 7);
                a.pm[unit * R + r] = mref[tid];
                a.pl[unit * R + r] = (wx[tid] + wx[32 + tid]) + (wx[64 + tid] + wx[96 + tid]);
            }
            if (lq == 0) {
                const bool live = (lane >> 3) < a.q_len && (lane & 7) < GQA;
                const int r = (lane >> 3) * GQA + (lane & 7);
#pragma unroll 1
                for (int h = 0; h < 2; ++h) {
                    uint32_t o[32];
                    umma::tmem_ld32(tO + 64 * gq + 32 * h, o);
                    umma::tmem_ld_wait();
                    if (live) {
                        float4 * dst = reinterpret_cast<float4 *>(a.po + (unit * R + r) * DH + 64 * gq + 32 * h);
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            dst[c] = make_float4(__uint_as_float(o[4 * c]), __uint_as_float(o[4 * c + 1]), __uint_as_float(o[4 * c + 2]),
                                                 __uint_as_float(o[4 * c + 3]));
                    }
                }
            }
            umma::fence_before_sync();
        }
        g += nt;
        __syncthreads();   // the run's shared memory and tensor memory are no longer read
    }
    if (w == TC_WORKERS / 32) {
        umma::fence_after_sync();
        umma::tmem_dealloc(tb, 512);
    }
}
