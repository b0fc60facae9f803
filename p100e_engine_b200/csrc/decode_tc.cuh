// Batched verify (two to four rows per slot) on the 5th-generation tensor cores (tcgen05), for q8_0 caches and the even
// split of a batch over the SMs.  Included by attn_decode.cu inside its namespace (dec_args, traits, the tensor maps and the split
// plan are defined there).
//
// One CTA per SM walks its run of keys in tiles of 128.  Per tile and kv head:
//   K rows (TMA -> staging) --16 worker warps: int8 -> f16 * block scale--> tensor memory, lane = key
//   S^T[128 keys x rows]   = K (A operand in tensor memory) * Q^T (B operand, K-major image in shared memory)
//   V rows (TMA -> staging) --workers--> f16 image [key][dim] in shared memory
//   workers: S^T -> mask -> P = 2^(S - reference maximum + 8) as f16 -> P image [row][key] in shared memory
//   O^T[256 dims x rows]  += V^T (A operand, the MN-major image, two halves of 128 dims) * P^T (B operand, K-major image)
// Two more warps issue: warp 16 the MMAs, warp 17 the TMA copies (a TMA instruction can hold its thread while the copy
// unit's queue is full, which must not delay an MMA).  Both walk their loops with all 32 lanes and let one elected lane
// issue, so that tensor-memory addresses and descriptors are warp-uniform values: the MMA and TMA instructions take their
// operands from uniform registers, and an issuer that ran as a single diverged lane spent most of a tile moving operands.
// The workers meet the issuers through mbarriers only, and each other once per tile (the vote on "some score outgrew its
// reference maximum").  K and S^T are double-buffered in tensor memory: in iteration i the workers widen the K rows of
// tile i + 1, start the load of tile i's scores from tensor memory, write tile i's V image, then publish K(i + 1) (its
// tensor-memory stores have landed by then) and turn to the scores: the Q K^T of a tile has a whole conversion phase to
// finish, and neither tensor-memory latency is waited for.  Barriers that a waiter could fall two phases behind on exist
// once per buffer (parity alone cannot tell phase n from phase n + 2).
//
// Against the mma.sync kernel this takes the multiply-adds, the fragment shuffling and the per-tile accumulator traffic out
// of the instruction stream: what the CUDA cores still do is the widening of 2 x 128 x 256 cache values per tile (seven
// instructions per four values) and 128 x rows exponentials.
//
// Every wait is bounded (mbar_wait gives up after two seconds and records ST_WAIT_TIMEOUT).

constexpr int UT = 128;                       // keys per tile
constexpr int TC_WORKERS = 512, TC_THR = TC_WORKERS + 64;   // 16 worker warps, the MMA warp, the TMA warp
constexpr int TC_NBUF = 4;                    // staging ring, in the order the workers consume: K0, K1, V0, K2, V1, ..
constexpr int TC_HDR = 2048;                  // barriers, reference maxima, exchange arrays, page entries
constexpr int TC_PGS = 224;                   // page-table entries of a run kept in shared memory
constexpr int TC_VF = UT * DH * 2;            // f16 image of a tile's V rows
constexpr int TC_QI = 32 * 32 * 16;           // f16 image of up to 32 query rows
constexpr int TC_PLBO = 528;                  // bytes between the 8-key chunks of the P image (512 + 16: stores of a warp spread over the banks)
constexpr int TC_PI = 8704;                   // P image: 16 chunks of up to 32 rows

constexpr int TC_HB = head_bytes(B200_KV_Q8_0);   // the kernel serves q8_0 rows: 8 f16 block scales, then 256 int8
constexpr size_t tc_smem_bytes() { return TC_HDR + (size_t) TC_NBUF * UT * TC_HB + TC_VF + TC_QI + TC_PI; }

__device__ __forceinline__ void tc_arrive(uint64_t * bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// A wait that records which one gave up (bits 8.. of the status word, beside ST_WAIT_TIMEOUT).  The first probe is inline
// (the hardware suspends the thread inside it for a while); only a probe that fails enters the timed loop, out of line.
__device__ __noinline__ void tc_wait_slow(uint64_t * bar, uint32_t parity, unsigned * status, int site) {
    if (!mbar_wait(bar, parity, status)) atomicOr(status, 0x100u << site);
}
__device__ __forceinline__ void tc_wait(uint64_t * bar, uint32_t parity, unsigned * status, int site) {
    if (!mbar_try_wait(bar, parity)) tc_wait_slow(bar, parity, status, site);
}
__device__ __forceinline__ void tc_bar_workers() { asm volatile("bar.sync 1, %0;" ::"n"(TC_WORKERS) : "memory"); }
__device__ __forceinline__ int tc_vote_workers(int v) {
    int r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.s32 q, %1, 0;\n\tbarrier.red.or.pred p, 1, %2, q;\n\tselp.s32 %0, 1, 0, p;\n\t}"
                 : "=r"(r) : "r"(v), "n"(TC_WORKERS) : "memory");
    return r;
}

// One 32-value block of a q8_0 row -> 16 registers of f16 pairs (register m = dims 2m, 2m+1 of the block), each value the
// rounded product of the stored integer and the block's f16 scale, given as the pair d2.  d2 = 0 gives zeros whatever the
// bytes are: the integer part is finite for every bit pattern.
__device__ __forceinline__ void tc_block(const unsigned char * row, int blk, uint32_t d2, uint32_t (&r)[16]) {
    const uint4 a = *reinterpret_cast<const uint4 *>(row + 16 + 32 * blk), b = *reinterpret_cast<const uint4 *>(row + 32 + 32 * blk);
    const uint32_t wv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t x = wv[j] ^ 0x80808080u;
        r[2 * j] = hmul2_u32(cvt_i8x2<0>(x), d2);
        r[2 * j + 1] = hmul2_u32(cvt_i8x2<1>(x), d2);
    }
}

// NC = score columns (16 for up to two verify rows, 32 for up to four): column 8 j + h = verify row j, head h of the group
// (h < 6); columns with h = 6, 7 are padding (zero query rows).
template <int NC>
__global__ void __launch_bounds__(TC_THR, 1)
decode_tc_k(const dec_args a, const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV) {
    extern __shared__ __align__(1024) unsigned char smem[];
    constexpr int HB = TC_HB, BUF = UT * HB;
    const int tid = threadIdx.x, lane = tid & 31;
    const int w = __shfl_sync(0xffffffffu, tid >> 5, 0);   // the warp index as a warp-uniform value
    const bool worker = w < TC_WORKERS / 32;
    const int lq = w & 3, gq = (w >> 2) & 3;     // worker warp: tensor-memory lane quarter, column / block group
    const int hk = (int) (blockIdx.x % (unsigned) a.g.Hkv), ui = (int) (blockIdx.x / (unsigned) a.g.Hkv);
    if (ui >= *a.n_cta) return;
    const int s0 = a.cta_seg[ui], s1 = a.cta_seg[ui + 1];
    if (s0 >= s1) return;

    uint64_t * full = reinterpret_cast<uint64_t *>(smem);                       // [TC_NBUF] staging buffer filled
    uint64_t * s_full = full + 4;                                                // [2] Q K^T of a tile has landed in S^T buffer b
    uint64_t * kconv = full + 6;                                                 // [2] K of a tile is in tensor-memory buffer b (per buffer: the
                                                                                 // workers run up to a tile ahead of the issuer)
    uint64_t * p_ready = full + 8;                                               // [2] P and the V image of a tile are written
    uint64_t * pv_done = full + 10;
    uint32_t * tbase_p = reinterpret_cast<uint32_t *>(smem + 120);
    float * mref = reinterpret_cast<float *>(smem + 128);                        // [32] reference maximum per column (log2 units)
    float * fsc = reinterpret_cast<float *>(smem + 256);                         // [32] rescale factor of the last move
    float * wx = reinterpret_cast<float *>(smem + 384);                          // [4][32] per lane quarter: maxima / sums
    float2 * mm = reinterpret_cast<float2 *>(smem + 896);                        // [32] (reference + REF_GAP, finite reference - PSHIFT)
    int * pgs = reinterpret_cast<int *>(smem + 1152);                            // [TC_PGS]
    unsigned char * stg = smem + TC_HDR, * VF = stg + TC_NBUF * BUF, * QI = VF + TC_VF, * PI = QI + TC_QI;

    if (tid == 0) {
        for (int b = 0; b < TC_NBUF; ++b) mbar_init(&full[b], 1);
        mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1); mbar_init(pv_done, 1);
        mbar_init(&kconv[0], TC_WORKERS / 32); mbar_init(&kconv[1], TC_WORKERS / 32);
        mbar_init(&p_ready[0], TC_WORKERS / 32); mbar_init(&p_ready[1], TC_WORKERS / 32);
        mbar_fence_init();
    }
    if (w == TC_WORKERS / 32) umma::tmem_alloc(tbase_p, 512);
    for (int i = tid; i < TC_PI / 16; i += TC_THR) reinterpret_cast<uint4 *>(PI)[i] = make_uint4(0, 0, 0, 0);   // padding rows stay zero
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tb = *tbase_p;
    // tensor memory: K as f16 pairs (2 x 128 columns), S^T (2 x 32), O^T (two halves of 128 dims, NC columns each)
    const uint32_t tA = tb, tS = tb + 256, tO = tb + 320;
    const uint32_t lane_off = (uint32_t) (32 * lq) << 16;
    const int R = a.q_len * GQA;
    // the O^T columns this worker warp rescales and writes out: half hO of the dims, columns 16 cO .. 16 cO + 15
    const int hO = gq & 1, cO = gq >> 1;
    const bool o_warp = 16 * cO < NC;

    int g = 0;   // tiles this CTA has walked (parities of the per-tile barriers); 2 g = staging items before the run
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
        const int ib = 2 * g;
        // Staging item q of the run, in the order the workers consume them (K0, K1, V0, K2, V1, .., K(nt-1), V(nt-2), V(nt-1)):
        // one or two 64-position boxes (boxes past the run's end hold no key) into ring buffer (2 g + q) mod 4.  Called by the
        // whole TMA warp with warp-uniform arguments; the elected lane issues.  staged: page entries come from shared memory.
        auto issue_item = [&](int q, bool lead, bool staged) {
            const bool is_v = q == 2 * nt - 1 || (q > 0 && (q & 1) == 0);
            const int tile = q == 0 ? 0 : q == 2 * nt - 1 ? nt - 1 : is_v ? (q - 2) >> 1 : (q + 1) >> 1;
            const int p_t = k_lo + tile * UT;
            const CUtensorMap * map = is_v ? &mapV : &mapK;
            const int nbox = p_t + TILE < k_hi ? 2 : 1;
            const int buf = (ib + q) & (TC_NBUF - 1);
            unsigned char * dst = stg + (size_t) buf * BUF;
            if (lead) mbar_expect_tx(&full[buf], (uint32_t) nbox * TILE * HB);
            for (int h = 0; h < nbox; ++h) {
                const int p = p_t + h * TILE;
                int y = p, z = 0;
                if (tab) {
                    const int idx = (p >> a.g.psh) - pg0;
                    z = staged && idx < TC_PGS ? pgs[idx] : tab[p >> a.g.psh];
                    y = p & ((1 << a.g.psh) - 1);
                    if (z < 0) { if (lead) atomicOr(a.status, ST_BAD_PAGE); z = 0; }
                }
                if (lead) tma_box3(dst + h * TILE * HB, map, hk * (HB / 2), y, z, &full[buf]);
            }
        };
        // The ring is empty at the start of a run (the previous run's end barrier): its first items go out now, before the
        // workers stage the page entries and the query rows, so that the copies fly during that prologue.
        if (w == TC_WORKERS / 32 + 1) {
            const bool lead = umma::elect_one();
            for (int q = 0; q < TC_NBUF && q < 2 * nt; ++q) issue_item(q, lead, false);
        }
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
            if (tid < 32) { mref[tid] = B200_NEG_INF; mm[tid] = make_float2(B200_NEG_INF, -PSHIFT); }
            umma::fence_async_smem();
        }
        __syncthreads();

        if (!worker) {
            // ---------------- two issuer warps: MMAs (warp 16) and TMA copies (warp 17) ----------------
            // All 32 lanes walk the loops and wait, so that counters, addresses and descriptors are warp-uniform values
            // (the MMA and TMA instructions take their operands from uniform registers); one elected lane issues.  The
            // copies have a warp of their own because a TMA instruction can hold its thread for as long as the copy
            // unit's queue is full, which must not delay the next MMA.
            const bool lead = umma::elect_one();
            const int nt_u = __shfl_sync(0xffffffffu, nt, 0), g_u = __shfl_sync(0xffffffffu, g, 0);
            if (w == TC_WORKERS / 32) {
                const uint32_t tb_u = __shfl_sync(0xffffffffu, tb, 0);
                const uint32_t tA_u = tb_u, tS_u = tb_u + 256, tO_u = tb_u + 320;
                constexpr uint32_t id_qk = umma::idesc_f16(UT, NC, false, false);   // S^T[128 x NC] = K (tensor memory) * Q^T (K-major)
                constexpr uint32_t id_pv = umma::idesc_f16(UT, NC, true, false);    // O^T[128 x NC] += V^T (MN-major) * P^T (K-major)
                const uint32_t q_s = smem_u32(QI), p_s = smem_u32(PI), v_s = smem_u32(VF);
                auto qk = [&](int j) {   // tile j: waits for its K in tensor memory, queues Q K^T
                    const int G = g_u + j, b = G & 1;
                    tc_wait(&kconv[b], (uint32_t) ((G >> 1) & 1), a.status, 0);
                    umma::fence_after_sync();
                    if (lead) {
#pragma unroll
                        for (int ks = 0; ks < DH / 16; ++ks)
                            umma::mma_ts(tS_u + 32 * b, tA_u + 128 * b + ks * 8, umma::smem_desc(q_s + ks * 2 * (NC * 16), NC * 16, 128), id_qk, ks > 0);
                        umma::commit(&s_full[b]);
                    }
                };
                qk(0);
                for (int i = 0; i < nt_u; ++i) {
                    if (i + 1 < nt_u) qk(i + 1);
                    const int G = g_u + i;
                    tc_wait(&p_ready[G & 1], (uint32_t) ((G >> 1) & 1), a.status, 1);     // P and the V image are in place
                    umma::fence_after_sync();
                    if (lead) {
#pragma unroll
                        for (int ks = 0; ks < UT / 16; ++ks)
#pragma unroll
                            for (int h = 0; h < 2; ++h)   // V image: 8-key groups 4096 apart (LBO), 8-dim groups 128 apart (SBO); P: 8-key chunks TC_PLBO apart
                                umma::mma_ss(tO_u + h * NC, umma::smem_desc(v_s + ks * 2 * 4096 + h * 2048, 4096, 128),
                                             umma::smem_desc(p_s + ks * 2 * TC_PLBO, TC_PLBO, 128), id_pv, (i > 0 || ks > 0) ? 1u : 0u);
                        umma::commit(pv_done);
                    }
                }
            } else {
                for (int q = TC_NBUF; q < 2 * nt_u; ++q) {   // the first TC_NBUF items went out before the prologue
                    // its buffer held item q - 4: the K rows of a tile are free once every worker has widened them, the V
                    // rows once every worker has written its part of the image
                    const int pq = q - TC_NBUF;
                    const bool was_v = pq > 0 && (pq & 1) == 0;
                    const int G = g_u + (pq == 0 ? 0 : was_v ? (pq - 2) >> 1 : (pq + 1) >> 1);
                    tc_wait(was_v ? &p_ready[G & 1] : &kconv[G & 1], (uint32_t) ((G >> 1) & 1), a.status, 7);
                    issue_item(q, lead, true);
                }
            }
            __syncwarp();
        } else {
            // ---------------- workers ----------------
            const bool act = gq < a.q_len && gq < NC / 8;           // this warp's columns 8 gq .. 8 gq + 5 hold verify row gq
            const int pos_g = act ? row_pos(a, slot, gq) : -1;
            const int kk = 32 * lq + lane;                          // this thread's key of the tile in the K and score phases
            const int vkey = tid & (UT - 1), vb = tid >> 7;         // and its key / first block in the V phase
            const unsigned char * const krow0 = stg + kk * HB, * const vrow0 = stg + vkey * HB;
            unsigned char * const vdst = VF + vb * 512 + (vkey >> 3) * 4096 + (vkey & 7) * 16;
            unsigned char * const pdst = PI + gq * 128 + (kk >> 3) * TC_PLBO + (kk & 7) * 2;
            const float4 * mm4 = reinterpret_cast<const float4 *>(mm) + 4 * gq;
            float l_acc[GQA];
#pragma unroll
            for (int e = 0; e < GQA; ++e) l_acc[e] = 0.0f;
            int cons = ib;   // staging items are consumed in ring order: K0, K1, V0, K2, V1, ..

            // K rows of a tile -> tensor-memory buffer tb_k (lane = key; this warp: blocks 2 gq, 2 gq + 1 of keys 32 lq ..).
            // The stores are left in flight: k_publish waits for them and tells the issuers.
            auto k_store = [&](int G) {
                const int buf = cons & (TC_NBUF - 1);
                tc_wait(&full[buf], (uint32_t) ((cons >> 2) & 1), a.status, 2);
                ++cons;
                const unsigned char * row = krow0 + buf * BUF;
                const uint32_t sc2 = *reinterpret_cast<const uint32_t *>(row + 4 * gq);   // the two blocks' scales
#pragma unroll
                for (int bb = 0; bb < 2; ++bb) {
                    uint32_t r[16];
                    tc_block(row, 2 * gq + bb, __byte_perm(sc2, sc2, bb ? 0x3232 : 0x1010), r);
                    umma::tmem_st16(tA + 128 * (G & 1) + lane_off + (2 * gq + bb) * 16, r);
                }
            };
            auto k_publish = [&](int G) {
                umma::tmem_st_wait();
                umma::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc_arrive(&kconv[G & 1]);
            };

            k_store(g);
            k_publish(g);
            for (int i = 0; i < nt; ++i) {
                const int G = g + i, p_t = k_lo + i * UT;
                if (i + 1 < nt) k_store(G + 1);
                // ---- this tile's scores: the load from tensor memory flies during the V phase
                tc_wait(&s_full[G & 1], (uint32_t) ((G >> 1) & 1), a.status, 5);
                umma::fence_after_sync();
                uint32_t sr[8];
                if (act) umma::tmem_ld8(tS + 32 * (G & 1) + lane_off + 8 * gq, sr);
                // ---- V rows -> f16 image, MN-major: byte(key, d) = (d / 8) * 128 + (key / 8) * 4096 + (key % 8) * 16 + (d % 8) * 2
                {
                    const int buf = cons & (TC_NBUF - 1);
                    tc_wait(&full[buf], (uint32_t) ((cons >> 2) & 1), a.status, 3);
                    if (G > 0) tc_wait(pv_done, (uint32_t) ((G - 1) & 1), a.status, 4);   // the previous P V has read the image and P
                    ++cons;
                    const unsigned char * row = vrow0 + buf * BUF;
                    const bool valid = p_t + vkey < k_hi;   // rows past the run's last key may hold anything: they enter as zeros
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        uint32_t r[16];
                        const uint32_t sc = valid ? *reinterpret_cast<const uint16_t *>(row + 2 * (vb + 4 * u)) : 0u;
                        tc_block(row, vb + 4 * u, __byte_perm(sc, sc, 0x1010), r);
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            *reinterpret_cast<uint4 *>(vdst + u * 2048 + c * 128) = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
                    }
                }
                if (i + 1 < nt) k_publish(G + 1);
                // ---- scores of this thread's key for the six heads of verify row gq
                float s[GQA], ofs[GQA];
                int grow = 0;
                if (act) {
                    umma::tmem_ld_wait();
                    const float4 m0 = mm4[0], m1 = mm4[1], m2 = mm4[2];
                    const float gap[GQA] = {m0.x, m0.z, m1.x, m1.z, m2.x, m2.z};
                    ofs[0] = m0.y; ofs[1] = m0.w; ofs[2] = m1.y; ofs[3] = m1.w; ofs[4] = m2.y; ofs[5] = m2.w;
#pragma unroll
                    for (int e = 0; e < GQA; ++e) s[e] = __uint_as_float(sr[e]);
                    if (p_t + UT - 1 > pos_g || p_t + UT > k_hi) {   // only tiles that reach past the row's last key or the run's end
                        const int key_abs = p_t + kk;
                        if (key_abs > pos_g || key_abs >= k_hi) {
#pragma unroll
                            for (int e = 0; e < GQA; ++e) s[e] = B200_NEG_INF;
                        }
                    }
#pragma unroll
                    for (int e = 0; e < GQA; ++e) grow |= s[e] > gap[e];
                } else {
#pragma unroll
                    for (int e = 0; e < GQA; ++e) { s[e] = B200_NEG_INF; ofs[e] = 0.0f; }
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
                            if (mx > m_old + REF_GAP) {   // mx is finite here
                                f = ex2f(m_old - mx);     // 2^(-inf) = 0 on the first move
                                mref[tid] = mx;
                                mm[tid] = make_float2(mx + REF_GAP, mx - PSHIFT);
                            }
                        }
                        fsc[tid] = f;
                    }
                    tc_bar_workers();
                    if (act) {
                        const float4 m0 = mm4[0], m1 = mm4[1], m2 = mm4[2];
                        ofs[0] = m0.y; ofs[1] = m0.w; ofs[2] = m1.y; ofs[3] = m1.w; ofs[4] = m2.y; ofs[5] = m2.w;
#pragma unroll
                        for (int e = 0; e < GQA; ++e) l_acc[e] *= fsc[8 * gq + e];
                    }
                    if (i > 0 && o_warp) {   // O^T: lane = dim, column = row; this warp's 16 columns of its half
                        const float4 * f4 = reinterpret_cast<const float4 *>(fsc) + 4 * cO;
                        const float4 fa = f4[0], fb = f4[1], fc = f4[2], fd = f4[3];
                        const float f[16] = {fa.x, fa.y, fa.z, fa.w, fb.x, fb.y, fb.z, fb.w, fc.x, fc.y, fc.z, fc.w, fd.x, fd.y, fd.z, fd.w};
                        bool any = false;
#pragma unroll
                        for (int c = 0; c < 16; ++c) any = any || f[c] != 1.0f;
                        if (any) {
                            uint32_t o[16];
                            umma::tmem_ld16(tO + lane_off + hO * NC + 16 * cO, o);
                            umma::tmem_ld_wait();
#pragma unroll
                            for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f[c]);
                            umma::tmem_st16(tO + lane_off + hO * NC + 16 * cO, o);
                            umma::tmem_st_wait();
                        }
                    }
                }
                // ---- P = 2^(S - reference + 8) as f16 into the K-major image: byte(row, key) = (row / 8) * 128 + (key / 8) * TC_PLBO + (row % 8) * 16 + (key % 8) * 2
                if (act) {
#pragma unroll
                    for (int e = 0; e < GQA; ++e) {
                        const float p = ex2f(s[e] - ofs[e]);
                        l_acc[e] += p;
                        *reinterpret_cast<__half *>(pdst + e * 16) = __float2half_rn(p);
                    }
                }
                umma::fence_async_smem();
                umma::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc_arrive(&p_ready[G & 1]);
            }
            // ---------------- the run's partial (O, reference maximum, sum) ----------------
            tc_wait(pv_done, (uint32_t) ((g + nt - 1) & 1), a.status, 6);
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
            if (o_warp) {
                uint32_t o[16];
                umma::tmem_ld16(tO + lane_off + hO * NC + 16 * cO, o);
                umma::tmem_ld_wait();
                float * dst = a.po + unit * R * DH + 128 * hO + kk;
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const int col = 16 * cO + c, jg = col >> 3, hh = col & 7;
                    if (jg < a.q_len && hh < GQA) dst[(size_t) (jg * GQA + hh) * DH] = __uint_as_float(o[c]);
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
