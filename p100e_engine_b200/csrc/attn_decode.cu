// Split-KV decode / MTP-verify attention over the paged f16 / q8_0 / q4_0 cache, sm_100a.
//
// Work unit = (slot, kv head, key chunk): one CTA of 4 warps walks its chunk in 64-key tiles; four CTAs per SM for three row
// tiles (q_len 3..4), five for two, six for one (q_len 1), two for f16 caches.
//   staging   the K rows and the V rows of a tile (one kv head, 64 positions) are each fetched by ONE tiled TMA copy through a
//             tensor map of the cache (x = row bytes, y = position in page, z = page) into a ring of half-tile slots,
//             completion counted on mbarriers; rows keep their cache format in shared memory.  The warp that is last to
//             finish with a slot issues its refill.  f16 rows go through a rank-4 map with the 128-byte swizzle.  Ragged
//             last tiles and pages under 64 rows are staged row by row through registers instead.
//   QK^T      warp w owns keys 16w..16w+15 of the tile: keys on the MMA M axis, the slot's 6 * q_len query rows on N
//             (all GQA heads and verify rows share one pass over the KV bytes).  int8 / nibbles are widened to f16
//             exactly in registers (byte permute + one f16x2 subtract), products accumulate in fp32 on the tensor
//             cores (mma.sync m16n8k16), the per-32 block scale multiplies the fp32 partial sums.
//   softmax   online, per row, base 2, against a reference maximum that all warps share and that may trail the true
//             maximum by 2^7: a tile whose scores stay under it needs one block barrier (P to shared memory as f16, then
//             P V); only a tile that outgrows it makes the warps exchange maxima, redo P and rescale O.
//   PV        warp w owns output dims 64w..64w+63: V^T tiles on M, rows on N, fp32 accumulators in registers.
//   partials  each unit writes unnormalised (O, m, l); a merge kernel combines a row's chunks in a fixed order, applies
//             the optional sigmoid gate and normalises (reference formula: dec2_combine_k, src/fast/attn_dec2.cu:430-450).
// The chunk grid is fixed by absolute key index, and a chunk's arithmetic never depends on the other rows of the call:
// a row's result is a function of its own keys and of chunk_keys only (row t of a T-row call == the 1-row call).
//
// Batched calls that let the library choose the split (chunk_keys < 0) cut the batch evenly over the CTAs that fit the GPU
// (decode_split_k; one plan per model step when the caller declares the step, b200_attn_step_begin).  There q8_0 caches
// with two to four rows per slot run on a second kernel, decode_tc_k (decode_tc.cuh): tcgen05 MMAs with K in tensor
// memory and V as an f16 image in shared memory, one CTA per SM.  Everything else, and every fixed-chunk call, runs on
// the kernel described above.
//
// Reference counterpart: dec2_k / attn_decode2 (src/fast/attn_dec2.cu:210-530), fp32 FFMA on sm_60.
#include "umma.cuh"

#include <dlfcn.h>
#include <cuda.h>   // CUtensorMap and its enums only: the encoder is looked up at run time, nothing links against libcuda
#include <algorithm>
#include <atomic>
#include <cstring>
#include <cstdlib>
#include <mutex>

namespace b200 {
namespace {

constexpr int TILE = 64;              // keys per tile
constexpr int NWARP = 4, NTHR = NWARP * 32;
constexpr int PGS = 64;               // page-table entries of a chunk kept in shared memory
constexpr int HDR = 1024;             // shared-memory header: barriers, counters, page entries; the slots start 1024-aligned
#ifndef DEC_CTAS
#define DEC_CTAS 4
#endif
constexpr int CTAS_Q = DEC_CTAS;      // CTAs per SM the quantised kernels are compiled for (register budget 65536 / (128 * CTAS_Q))
// fewer query rows need fewer accumulator registers: one row tile (q_len 1) runs six CTAs per SM, two run five
template <uint32_t KT, int NT> constexpr int ctas_per_sm() { return KT == B200_KV_F16 ? 2 : NT == 1 ? CTAS_Q + 2 : NT == 2 ? CTAS_Q + 1 : CTAS_Q; }
constexpr int QSTR = 576;             // bytes per Q row in shared memory (256 f16 + 64: rows g, g+1 on different bank halves)
constexpr int PSTR = 144;             // bytes per P row (64 f16 + 16)
constexpr int SDSTR = 132;            // bytes per V-scale row (64 f16 + 4)
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr float PSHIFT = 8.0f;        // P (and l) are kept times 2^8 inside the kernels
constexpr float REF_GAP = 7.0f;       // a row's reference maximum may trail its true maximum by this much (log2 units)

template <uint32_t KT> struct traits {
    static constexpr int HB = head_bytes(KT);                       // bytes of a head row in the cache
    static constexpr int SROW = HB;                                 // bytes per key row in shared memory
    static constexpr int SLOT = TILE * SROW;                        // one ring slot: the K rows or the V rows of a tile
    static constexpr bool SCALED = KT != B200_KV_F16;
};
// Verify calls on quantised caches (two or three row tiles) keep 32 or 48 output accumulators per thread, which are idle
// during Q K^T and the softmax: there they are parked in tensor memory (tcgen05.st / tcgen05.ld, this warp's own 32 lanes),
// so the compiler has those registers for loads in flight.  PARK_COLS columns are allocated per CTA.
#ifndef DEC_PARK
#define DEC_PARK 1
#endif

template <uint32_t KT, int NT> constexpr bool parks() { return DEC_PARK && KT != B200_KV_F16 && NT >= 2; }
constexpr uint32_t PARK_COLS = 64;

// f16 slots hold four sub-tiles [64 rows][128 B] (dims 64 c .. 64 c + 63) with the 128-byte swizzle of the TMA unit: the
// 16-byte chunk j of a sub-tile row sits at chunk j ^ (row & 7), which keeps 16-byte and ldmatrix accesses of eight
// different rows on different banks.  chunk16 = 16-byte chunk of the 512-byte head row.
__device__ __forceinline__ int f16_slot_off(int row, int chunk16) {
    return (chunk16 >> 3) * (TILE * 128) + row * 128 + (((chunk16 & 7) ^ (row & 7)) << 4);
}

// M-row (0..7) -> key of the warp's 16-key group, chosen so that the A-fragment loads of a phase hit distinct banks
template <uint32_t KT> __device__ __forceinline__ int key_perm(int g) {
    if constexpr (KT == B200_KV_F16) return (g >> 1) + 4 * (g & 1);       // 16-byte loads: lanes of a phase 4 keys apart
    else if constexpr (KT == B200_KV_Q8_0) return 2 * (g & 3) + (g >> 2); // 8-byte loads: 2 keys apart
    else return g;
}
// position of head dim d inside the shared-memory Q row, so that lane t of a quad reads dims of block b for both
// k-steps of the block with one 16-byte load at 64 b + 16 t
template <uint32_t KT> __device__ __forceinline__ int q_slot(int d) {
    if constexpr (KT == B200_KV_Q4_0) {
        const int b = d >> 5, i = d & 31;          // nibble order: byte j = dims j | j + 16
        return b * 32 + ((i & 15) >> 2) * 8 + (i >> 4) * 4 + (i & 3);
    } else return d;
}

struct dec_args {
    const float * q;
    kv_view g;
    float * po; float * pm; float * pl;   // partials [unit][R][256], [unit][R], [unit][R]
    const int32_t * pos;                  // per-row positions (device) or nullptr
    const int32_t * p0p;                  // device first position or nullptr
    int p0;
    int q_len, n_slots, Hq;
    float qscale;                         // softmax scale * log2(e)
    int CH, max_chunks;
    unsigned * status;
    int n_ctx;                            // rows of a contiguous cache
    int tiled;                            // set by the launcher: whole tiles are fetched through the tensor maps
    const int2 * units;                   // work list written by decode_plan_k: (slot, chunk), longest first; nullptr = the
    const int * n_units;                  // grid itself enumerates (slot, chunk) and units past a slot's end exit
    // even split (decode_split_k): the batch's 64-key tiles, slot after slot, are cut into one contiguous run per CTA
    const int4 * segs;                    // (slot, first key, end key, 0) in CTA order; a run that crosses a slot boundary has several
    const int * cta_seg;                  // [n_cta + 1] first segment of each CTA
    const int2 * slot_seg;                // [n_slots] (first segment, segments) of each slot
    const int * n_cta;                    // CTAs (per kv head) that hold work
};

// keys of a slot that the call may touch: 1 + its largest row position, held to the caller's max_n (the grid and the
// partials are sized for max_chunks chunks) and to n_ctx for a contiguous cache.  A position beyond the limit is recorded
// in the status word and its keys past the limit are left out.
__device__ __forceinline__ int key_limit(const dec_args & a) {
    const long long lim = (long long) a.max_chunks * a.CH;
    const int l = (int) (lim < 0x7fffffffLL ? lim : 0x7fffffffLL);
    return a.g.pt ? l : min(l, a.n_ctx);
}

// One tiled copy (TMA unit) of a box of a rank-3 tensor into shared memory, completion counted in bytes on an mbarrier.
// x is in 16-bit elements and x * 2 must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_box3(void * dst, const CUtensorMap * map, int x, int y, int z, uint64_t * bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ int row_pos(const dec_args & a, int slot, int j) {
    const int r = slot * a.q_len + j;
    if (a.pos) return a.pos[r];
    return (a.p0p ? *a.p0p : a.p0) + r;
}

// two int8 (already offset by 128) at bytes (2 * HI, 2 * HI + 1) of u -> f16x2
template <int HI> __device__ __forceinline__ uint32_t cvt_i8x2(uint32_t u) {
    return hsub2_u32(__byte_perm(u, 0x64646464u, HI ? 0x7362 : 0x5140), 0x64806480u);
}
// bytes holding values 0..15 (+8 bias) at bytes (2 * HI, 2 * HI + 1) -> f16x2 of (value - 8)
template <int HI> __device__ __forceinline__ uint32_t cvt_n4x2(uint32_t u) {
    return hsub2_u32(__byte_perm(u, 0x64646464u, HI ? 0x7362 : 0x5140), 0x64086408u);
}

__device__ __forceinline__ void tma_box4(void * dst, const CUtensorMap * map, int x, int y, int z, int w, uint64_t * bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar)) : "memory");
}

// One unit of work: the keys k_lo .. k_cap-1 (as far as the slot has them) of one slot and kv head, all its query rows;
// writes the unnormalised partial (O, m, l) number `unit`.  Called by all threads of the CTA.  A CTA that runs several units
// keeps its ring of copy slots, their barriers and the arrival counters going from one unit to the next: tiles_before is the
// number of tiles its earlier units walked (two ring items each); the function returns this unit's tile count.
// t_base: tensor-memory base of the parked accumulators.
template <uint32_t KT, int NT>
__device__ __forceinline__ int decode_unit(const dec_args & a, const int nslot, const CUtensorMap & mapK, const CUtensorMap & mapV,
                                           unsigned char * smem, const int hk, const int slot, const int k_lo, const int k_cap,
                                           const size_t unit, const int tiles_before, const uint32_t t_base) {
    using TR = traits<KT>;
    constexpr int HB = TR::HB, SROW = TR::SROW;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, t = lane & 3;
    const int R = a.q_len * GQA;

    // visible keys of the slot = 1 + the largest row position
    int n_slot = 0;
    for (int j = 0; j < a.q_len; ++j) n_slot = max(n_slot, row_pos(a, slot, j) + 1);
    {
        const int lim = key_limit(a);
        if (n_slot > lim) { if (tid == 0) atomicOr(a.status, ST_BAD_POS); n_slot = lim; }
    }
    if (k_lo >= n_slot) return 0;
    const int k_hi = min(k_cap, n_slot);
    const int ntiles = (k_hi - k_lo + TILE - 1) / TILE;
    const int ring0 = (2 * tiles_before) % nslot;                       // ring slot of this unit's first item
    const uint32_t ring0_par = (uint32_t) ((2 * tiles_before) / nslot) & 1u;   // and the parity of that slot's use count

    // shared memory carve-up
    uint64_t * full = reinterpret_cast<uint64_t *>(smem);                    // [nslot]
    int * done = reinterpret_cast<int *>(smem + 96);                         // warps that finished Q K^T / P V (two counters)
    int * flag = reinterpret_cast<int *>(smem + 104);                        // [3] "some warp's scores outgrew the references"
    int * pgs = reinterpret_cast<int *>(smem + 128);                         // [PGS] page-table entries of the chunk's pages
    unsigned char * stg = smem + HDR;                                        // nslot * SLOT
    unsigned char * Qs = stg + (size_t) nslot * TR::SLOT;                    // [NT*8][QSTR]
    unsigned char * Ps = Qs + NT * 8 * QSTR;                                 // [NT*8][PSTR]
    unsigned char * Sd = Ps + NT * 8 * PSTR;                                 // [8][SDSTR]  V block scales, transposed
    float * wmax = reinterpret_cast<float *>(Sd + 8 * SDSTR);                // [NWARP][NT*8]
    float * wl = wmax + NWARP * NT * 8;                                      // [NWARP][NT*8]
    float4 * Qb = reinterpret_cast<float4 *>(wl + NWARP * NT * 8);           // [NBLK][NT][4] block sums of Q (quantised caches)

    const int32_t * tab = a.g.pt ? a.g.pt + (a.g.rtab ? a.g.rtab[slot * a.q_len] : 0) : nullptr;
    const unsigned long long hoff = (unsigned long long) hk * HB;
    // the chunk's page-table entries are staged in shared memory when there are at most PGS of them, so that a refill does
    // not wait for a global load
    const int pg0 = tab ? k_lo >> a.g.psh : 0;
    const bool pg_staged = tab && ((k_hi - 1) >> a.g.psh) - pg0 < PGS;

    // staging: the K rows and the V rows of the tiles form one sequence q = 2 * tile (K), 2 * tile + 1 (V) that walks a ring
    // of nslot half-tile slots.  The warp that is last to finish the Q K^T (P V) of a tile refills that tile's K (V) slot with
    // item q + nslot, so a copy is in flight while the other half of the tile is being computed.  A tile that lies inside
    // the slot's keys is one tiled copy through the cache's tensor map (box = 64 rows of this head, inside one page);
    // otherwise the warp moves the 64 rows one by one, rows past the slot's last key replaced by that last key (always
    // readable and finite, and masked in the softmax).
    auto page_of = [&](int p, bool first) { return pg_staged && !first ? pgs[(p >> a.g.psh) - pg0] : tab[p >> a.g.psh]; };
    auto issue = [&](int q, int s, bool first) {   // s = q mod nslot; called by one whole warp
        if (q >= 2 * ntiles) return;
        const int it = q >> 1;
        unsigned char * dst = stg + (size_t) s * TR::SLOT;
        const char * base = (q & 1) ? a.g.v : a.g.k;
        const int p_t = k_lo + it * TILE;
        if (a.tiled && p_t + TILE <= n_slot) {
            if (lane == 0) {
                int y = p_t, z = 0;
                if (tab) {
                    z = page_of(p_t, first);
                    y = p_t & ((1 << a.g.psh) - 1);
                    if (z < 0) { atomicOr(a.status, ST_BAD_PAGE); z = 0; }
                }
                mbar_expect_tx(&full[s], (uint32_t) TILE * HB);
                if constexpr (KT == B200_KV_F16) tma_box4(dst, (q & 1) ? &mapV : &mapK, 0, y, 4 * hk, z, &full[s]);
                else tma_box3(dst, (q & 1) ? &mapV : &mapK, hk * (HB / 2), y, z, &full[s]);
            }
            __syncwarp();
            return;
        }
        // row by row through registers, 16 bytes per lane and step; the slot is published by a plain arrival
        constexpr int CPR = HB / 16;
#pragma unroll 4
        for (int idx = lane; idx < TILE * CPR; idx += 32) {
            const int row = idx / CPR, c = idx - row * CPR;
            const int p = min(p_t + row, n_slot - 1);
            unsigned long long off;
            if (tab) {
                const int pg = page_of(p, first);
                if (pg < 0) { atomicOr(a.status, ST_BAD_PAGE); off = 0; }
                else off = (unsigned long long) pg * a.g.pstride + (unsigned long long) (p & ((1 << a.g.psh) - 1)) * a.g.rowb;
            } else off = (unsigned long long) p * a.g.rowb;
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(base + off + hoff) + c);
            const int o = KT == B200_KV_F16 ? f16_slot_off(row, c) : row * SROW + c * 16;
            *reinterpret_cast<uint4 *>(dst + o) = v;
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full[s])) : "memory");
    };
    // warp 0 starts the first copies before anything else, so that they fly while Q is staged
    if (w == 0) {   // every slot is free at the start of a unit: all items of the earlier units have been consumed
        int s = ring0;
        for (int q0 = 0; q0 < nslot; ++q0) {
            issue(q0, s, true);
            if (++s == nslot) s = 0;
        }
    }
    constexpr bool PARK = parks<KT, NT>();
    if (pg_staged)
        for (int j = tid; j <= ((k_hi - 1) >> a.g.psh) - pg0; j += NTHR) pgs[j] = tab[pg0 + j];
    // Q rows -> shared memory as f16, scaled; row r = j * 6 + hh (verify row j, head hh of the group).  For the quantised
    // caches the middle two of every four dims are swapped (d0 d2 d1 d3): a 32-bit word of cache bytes then splits into the
    // f16 pairs (byte 0, byte 2) and (byte 1, byte 3) with one mask and one byte permute (see the Q K^T loop).
    for (int i = tid; i < NT * 8 * (DH / 4); i += NTHR) {
        const int r = i / (DH / 4), d4 = (i - r * (DH / 4)) * 4;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (r < R) {
            const int j = r / GQA, hh = r - j * GQA;
            v = *reinterpret_cast<const float4 *>(a.q + ((size_t) (slot * a.q_len + j) * a.Hq + hk * GQA + hh) * DH + d4);
        }
        // four consecutive dims stay together under q_slot (it permutes groups of four): one 8-byte store
        uint2 pk;
        if constexpr (TR::SCALED) pk = make_uint2(pack_h2(v.x * a.qscale, v.z * a.qscale), pack_h2(v.y * a.qscale, v.w * a.qscale));
        else pk = make_uint2(pack_h2(v.x * a.qscale, v.y * a.qscale), pack_h2(v.z * a.qscale, v.w * a.qscale));
        *reinterpret_cast<uint2 *>(Qs + r * QSTR + q_slot<KT>(d4) * 2) = pk;
    }
    __syncthreads();
    if constexpr (TR::SCALED) {
        // The cache integers enter the tensor cores as f16 subnormals u * 2^-24 with u = q + 128 (q8_0) or the nibble itself
        // (q4_0, value = nibble - 8).  The offset is taken out again through the accumulator's starting value: for block b and
        // row r it is -OFFS * 2^-24 * (sum of the block's 32 scaled f16 query values), kept per (block, row tile, lane quad
        // position) in the order of an accumulator fragment {row 2t, row 2t+1, row 2t, row 2t+1}.
        constexpr float OFFS = KT == B200_KV_Q8_0 ? 128.0f : 8.0f;
        for (int i = tid; i < NBLK * NT * 8; i += NTHR) {
            const int b = i / (NT * 8), r = i - b * (NT * 8);
            const __half2 * src = reinterpret_cast<const __half2 *>(Qs + r * QSTR + b * 64);   // a block's dims stay inside its 64 bytes
            float sum = 0.0f;
#pragma unroll
            for (int e = 0; e < 16; ++e) { const float2 f = __half22float2(src[e]); sum += f.x + f.y; }
            const float v = -OFFS * 5.9604644775390625e-8f * sum;
            float * dst = reinterpret_cast<float *>(Qb + (b * NT + (r >> 3)) * 4 + ((r & 7) >> 1));
            dst[r & 1] = v; dst[2 + (r & 1)] = v;
        }
    }
    __syncthreads();

    // arrive(c): this warp is done with the K (c = 0) or V (c = 1) item of the tile; lane 0 learns whether it was the last of
    // the four warps.  refill_if_last: that warp refills the slot.  The two are apart in the instruction stream so that the
    // round trip of the shared-memory atomic is covered by other work.
    auto arrive = [&](int c) {
        asm volatile("" ::: "memory");   // the item's shared-memory reads stay above this point
        int last = 0;
        if (lane == 0) last = (atomicAdd(&done[c], 1) & (NWARP - 1)) == NWARP - 1;
        return last;
    };
    auto refill_if_last = [&](int last, int q, int s) {
        if (__shfl_sync(0xffffffffu, last, 0)) issue(q + nslot, s, false);
    };

    // per-lane row bookkeeping: this lane's score / output columns are rows 8i + 2t and 8i + 2t + 1
    int rpos[NT][2];
    float m_run[NT][2], l_run[NT][2];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int r = 8 * i + 2 * t + e;
            rpos[i][e] = r < R ? row_pos(a, slot, r / GQA) : -1;
            m_run[i][e] = B200_NEG_INF;
            l_run[i][e] = 0.0f;
        }
    float O[4][NT][4];
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) O[mt][i][e] = 0.0f;
    // parked accumulators: 16 * NT columns of this warp's 32 tensor-memory lanes
    uint32_t t_O = 0;
    auto park = [&]() {
        const float * o = &O[0][0][0];
#pragma unroll
        for (int c = 0; c < NT; ++c) {
            uint32_t r[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) r[e] = __float_as_uint(o[16 * c + e]);
            umma::tmem_st16(t_O + 16 * c, r);
        }
        umma::tmem_st_wait();
    };
    auto unpark = [&]() {
        float * o = &O[0][0][0];
#pragma unroll
        for (int c = 0; c < NT; ++c) {
            uint32_t r[16];
            umma::tmem_ld16(t_O + 16 * c, r);
#pragma unroll
            for (int e = 0; e < 16; ++e) o[16 * c + e] = __uint_as_float(r[e]);
        }
        umma::tmem_ld_wait();
    };
    if constexpr (PARK) {
        t_O = t_base + ((uint32_t) (32 * w) << 16);
        park();
    }

    const int kA = 16 * w + key_perm<KT>(g), kB = kA + 8;   // this lane's two keys (tile-relative) in the QK phase
    int rmin = 0x7fffffff;   // the mask is only evaluated in tiles that reach past some row's last key or the chunk's end
    for (int j = 0; j < a.q_len; ++j) rmin = min(rmin, row_pos(a, slot, j));
    const int mask_from = min(k_hi, rmin + 1);

    // ring position of the tile's K item (2 it) and V item (2 it + 1): slot index and the parity of its use count
    int last_v = 0, sv_prev = 0;
    int sk = ring0, sv = ring0 + 1;
    uint32_t phk = ring0_par, phv = ring0_par;
    if (sv >= nslot) { sv -= nslot; phv ^= 1u; }
    for (int it = 0; it < ntiles; ++it) {
        const unsigned char * Ks = stg + (size_t) sk * TR::SLOT;
        const unsigned char * Vs = stg + (size_t) sv * TR::SLOT;
        uint64_t * const bar_k = &full[sk], * const bar_v = &full[sv];
        const uint32_t par_k = phk, par_v = phv;
        const int sk_now = sk, sv_now = sv;
        sk += 2; if (sk >= nslot) { sk -= nslot; phk ^= 1u; }
        sv += 2; if (sv >= nslot) { sv -= nslot; phv ^= 1u; }
        mbar_wait(bar_k, par_k, a.status);
        if (it > 0) refill_if_last(last_v, 2 * it - 1, sv_prev);   // the V slot of the previous tile

        // ---------------- S = K Q^T for the warp's 16 keys ----------------
        float S[NT][4];
#pragma unroll
        for (int i = 0; i < NT; ++i) { S[i][0] = S[i][1] = S[i][2] = S[i][3] = 0.0f; }
        const unsigned char * rowA = Ks + kA * SROW, * rowB = Ks + kB * SROW;
        if constexpr (KT == B200_KV_F16) {
#pragma unroll
            for (int b = 0; b < NBLK; ++b) {
                const uint4 wa = *reinterpret_cast<const uint4 *>(Ks + f16_slot_off(kA, 4 * b + t));
                const uint4 wb = *reinterpret_cast<const uint4 *>(Ks + f16_slot_off(kB, 4 * b + t));
                const uint32_t a0[4] = {wa.x, wb.x, wa.y, wb.y}, a1[4] = {wa.z, wb.z, wa.w, wb.w};
#pragma unroll
                for (int i = 0; i < NT; ++i) {
                    const uint4 qv = *reinterpret_cast<const uint4 *>(Qs + (8 * i + g) * QSTR + 64 * b + 16 * t);
                    mma16816(S[i], a0, qv.x, qv.y);
                    mma16816(S[i], a1, qv.z, qv.w);
                }
            }
        } else {
            // Integers -> f16 without arithmetic: a 16-bit lane holding a value u in 0..255 in its low byte IS the f16
            // subnormal u * 2^-24, and the tensor cores take subnormal operands at full rate.  A word of four cache bytes
            // gives the pairs (byte 0, byte 2) by a mask and (byte 1, byte 3) by one byte permute; the query dims are
            // stored in the matching order.  The sign offset (q8_0: u = q + 128 after flipping the top bits; q4_0: the
            // nibble carries +8) comes out through the accumulator's starting value Qb, the factor 2^24 through the scale.
            constexpr float UNSUB = 16777216.0f;
            uint4 sA, sB;   // the 8 block scales of each key (q8_0); q4_0 reads them block by block
            if constexpr (KT == B200_KV_Q8_0) {
                sA = *reinterpret_cast<const uint4 *>(rowA);
                sB = *reinterpret_cast<const uint4 *>(rowB);
            }
#pragma unroll
            for (int b = 0; b < NBLK; ++b) {
                uint32_t a0[4], a1[4];
                float dA, dB;
                if constexpr (KT == B200_KV_Q8_0) {
                    const uint2 wa = *reinterpret_cast<const uint2 *>(rowA + 16 + 32 * b + 8 * t);
                    const uint2 wb = *reinterpret_cast<const uint2 *>(rowB + 16 + 32 * b + 8 * t);
                    const uint32_t ax = wa.x ^ 0x80808080u, ay = wa.y ^ 0x80808080u;
                    const uint32_t bx = wb.x ^ 0x80808080u, by = wb.y ^ 0x80808080u;
                    a0[0] = ax & 0x00ff00ffu; a0[1] = bx & 0x00ff00ffu; a0[2] = __byte_perm(ax, 0u, 0x4341); a0[3] = __byte_perm(bx, 0u, 0x4341);
                    a1[0] = ay & 0x00ff00ffu; a1[1] = by & 0x00ff00ffu; a1[2] = __byte_perm(ay, 0u, 0x4341); a1[3] = __byte_perm(by, 0u, 0x4341);
                    const uint32_t swA = (&sA.x)[b >> 1], swB = (&sB.x)[b >> 1];
                    dA = __half2float(__ushort_as_half((unsigned short) ((b & 1) ? swA >> 16 : swA & 0xffffu))) * UNSUB;
                    dB = __half2float(__ushort_as_half((unsigned short) ((b & 1) ? swB >> 16 : swB & 0xffffu))) * UNSUB;
                } else {
                    // block at byte 18 b: f16 d, then 16 bytes; this lane takes bytes 4t..4t+3 (dims 4t.. low nibbles,
                    // 16+4t.. high nibbles).  The 16 bytes start on a 2-byte boundary for even b.
                    uint32_t qa, qb;
                    if ((b & 1) == 0) {
                        const uint32_t * pa = reinterpret_cast<const uint32_t *>(rowA + 18 * b + 4 * t);
                        const uint32_t * pb = reinterpret_cast<const uint32_t *>(rowB + 18 * b + 4 * t);
                        qa = __funnelshift_r(pa[0], pa[1], 16);
                        qb = __funnelshift_r(pb[0], pb[1], 16);
                    } else {
                        qa = *reinterpret_cast<const uint32_t *>(rowA + 18 * b + 2 + 4 * t);
                        qb = *reinterpret_cast<const uint32_t *>(rowB + 18 * b + 2 + 4 * t);
                    }
                    // nibble pairs: low nibbles of bytes (0, 2) and (1, 3) feed the first k-step, the high nibbles the second
                    a0[0] = qa & 0x000f000fu; a0[1] = qb & 0x000f000fu; a0[2] = (qa >> 8) & 0x000f000fu; a0[3] = (qb >> 8) & 0x000f000fu;
                    a1[0] = (qa >> 4) & 0x000f000fu; a1[1] = (qb >> 4) & 0x000f000fu; a1[2] = (qa >> 12) & 0x000f000fu; a1[3] = (qb >> 12) & 0x000f000fu;
                    dA = __half2float(*reinterpret_cast<const __half *>(rowA + 18 * b)) * UNSUB;
                    dB = __half2float(*reinterpret_cast<const __half *>(rowB + 18 * b)) * UNSUB;
                }
#pragma unroll
                for (int i = 0; i < NT; ++i) {
                    const uint4 qv = *reinterpret_cast<const uint4 *>(Qs + (8 * i + g) * QSTR + 64 * b + 16 * t);
                    float c[4];
                    mma16816_from(c, Qb[(b * NT + i) * 4 + t], a0, qv.x, qv.y);
                    mma16816(c, a1, qv.z, qv.w);
                    S[i][0] = fmaf(dA, c[0], S[i][0]); S[i][1] = fmaf(dA, c[1], S[i][1]);
                    S[i][2] = fmaf(dB, c[2], S[i][2]); S[i][3] = fmaf(dB, c[3], S[i][3]);
                }
            }
        }
        const int last_k = arrive(0);
        // causal / chunk mask, warp-level row maxima
        const int keyA = k_lo + it * TILE + kA, keyB = keyA + 8;
        if (k_lo + (it + 1) * TILE > mask_from) {
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    if (keyA > rpos[i][e] || keyA >= k_hi) S[i][e] = B200_NEG_INF;
                    if (keyB > rpos[i][e] || keyB >= k_hi) S[i][2 + e] = B200_NEG_INF;
                }
        }
        // ---------------- online softmax, P -> shared memory ----------------
        // Every row has a reference maximum m_run, the same in all four warps, that trails its true maximum by at most
        // REF_GAP (P = 2^(S - m_run + PSHIFT) <= 2^15 stays inside f16).  A warp whose keys stay under m_run + REF_GAP needs
        // nothing from the other warps: it writes P at once.  Only when some warp of the CTA sees a larger score (always on
        // the first tile) do the warps exchange their maxima after the barrier, move the references, redo P and rescale O.
        bool grow = false;
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int e = 0; e < 2; ++e) grow = grow || fmaxf(S[i][e], S[i][2 + e]) > m_run[i][e] + REF_GAP;
        const int ph = (tiles_before + it) % 3;   // three flags in turn: the one of the next tile is cleared two barriers after its last reader
        if (__any_sync(0xffffffffu, grow) && lane == 0) flag[ph] = 1;
        if (tid == 0) flag[ph == 2 ? 0 : ph + 1] = 0;
        refill_if_last(last_k, 2 * it, sk_now);
        // P and the V scales of this tile replace those of the previous tile: every warp must be done with its P V
        if (it > 0) {
            int spins = 0;
            while (*reinterpret_cast<volatile int *>(&done[1]) < NWARP * (tiles_before + it))
                if (++spins > (1 << 24)) { atomicOr(a.status, ST_WAIT_TIMEOUT); break; }
        }
        float lsum[NT][2];
        auto write_p = [&]() {   // P carries a factor 2^PSHIFT (numerator and denominator alike): keeps small weights out of
                                 // the f16 subnormal range; 2^(-inf) = 0 for a masked key
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int r = 8 * i + 2 * t + e;
                    const float msafe = m_run[i][e] == B200_NEG_INF ? 0.0f : m_run[i][e];
                    const __half pa = __float2half_rn(ex2f(S[i][e] - msafe + PSHIFT));
                    const __half pb = __float2half_rn(ex2f(S[i][2 + e] - msafe + PSHIFT));
                    lsum[i][e] = __half2float(pa) + __half2float(pb);
                    *reinterpret_cast<__half *>(Ps + r * PSTR + kA * 2) = pa;
                    *reinterpret_cast<__half *>(Ps + r * PSTR + kB * 2) = pb;
                }
        };
        write_p();
        mbar_wait(bar_v, par_v, a.status);   // this tile's V rows
        if constexpr (TR::SCALED) {   // V block scales, transposed to [block][key]
            const int key = tid >> 1, b0 = (tid & 1) * 4;
#pragma unroll
            for (int b = b0; b < b0 + 4; ++b) {
                const unsigned char * src = KT == B200_KV_Q8_0 ? Vs + key * SROW + 2 * b : Vs + key * SROW + 18 * b;
                *reinterpret_cast<uint16_t *>(Sd + b * SDSTR + key * 2) = *reinterpret_cast<const uint16_t *>(src);
            }
        }
        __syncthreads();   // P, the V scales, the warps' maxima and the flag are visible
        if constexpr (PARK) unpark();
        if (flag[ph]) {
            // the warps' row maxima over their 16 keys, exchanged through shared memory
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float mx = fmaxf(S[i][e], S[i][2 + e]);
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    if (g == 0) wmax[w * NT * 8 + 8 * i + 2 * t + e] = mx;
                }
            __syncthreads();
            float fsc[NT][2];
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int r = 8 * i + 2 * t + e;
                    const float mx = fmaxf(fmaxf(wmax[r], wmax[NT * 8 + r]), fmaxf(wmax[2 * NT * 8 + r], wmax[3 * NT * 8 + r]));
                    const float mnew = mx > m_run[i][e] + REF_GAP ? mx : m_run[i][e];
                    fsc[i][e] = ex2f(m_run[i][e] - (mnew == B200_NEG_INF ? 0.0f : mnew));
                    m_run[i][e] = mnew;
                }
            write_p();   // rows whose reference stayed get the same bits again
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int e = 0; e < 2; ++e) l_run[i][e] = fmaf(l_run[i][e], fsc[i][e], lsum[i][e]);
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                for (int i = 0; i < NT; ++i) {
                    O[mt][i][0] *= fsc[i][0]; O[mt][i][1] *= fsc[i][1];
                    O[mt][i][2] *= fsc[i][0]; O[mt][i][3] *= fsc[i][1];
                }
            __syncthreads();   // the rewritten P is visible
        } else {
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int e = 0; e < 2; ++e) l_run[i][e] += lsum[i][e];
        }

        // ---------------- O^T += V^T P^T for the warp's 64 output dims ----------------
#pragma unroll
        for (int u = 0; u < TILE / 16; ++u) {
            uint32_t pw[NT][2];
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                pw[i][0] = *reinterpret_cast<const uint32_t *>(Ps + (8 * i + g) * PSTR + (16 * u + 2 * t) * 2);
                pw[i][1] = *reinterpret_cast<const uint32_t *>(Ps + (8 * i + g) * PSTR + (16 * u + 2 * t + 8) * 2);
            }
            if constexpr (KT == B200_KV_F16) {
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) {
                    // four 8x8 tiles, transposed on load: (keys 0-7 | 8-15) x (dims 0-7 | 8-15) of this m-tile
                    const int mj = lane >> 3, mr = lane & 7;
                    const unsigned char * p = Vs + f16_slot_off(16 * u + (mj >> 1) * 8 + mr, 8 * w + 2 * mt + (mj & 1));
                    uint32_t av[4];
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(av[0]), "=r"(av[1]), "=r"(av[2]), "=r"(av[3]) : "r"(smem_u32(p)));
#pragma unroll
                    for (int i = 0; i < NT; ++i) mma16816(O[mt][i], av, pw[i][0], pw[i][1]);
                }
            } else {
                const unsigned char * v0 = Vs + (16 * u + 2 * t) * SROW, * v1 = v0 + SROW, * v2 = v0 + 8 * SROW, * v3 = v2 + SROW;
#pragma unroll
                for (int y = 0; y < 2; ++y) {
                    const int blk = 2 * w + y;
                    uint32_t ax[4], ay[4];   // m-tiles X and Y of this block
                    if constexpr (KT == B200_KV_Q8_0) {
                        const int col = 16 + 32 * blk + 4 * g;
                        const uint32_t w0 = *reinterpret_cast<const uint32_t *>(v0 + col) ^ 0x80808080u;
                        const uint32_t w1 = *reinterpret_cast<const uint32_t *>(v1 + col) ^ 0x80808080u;
                        const uint32_t w2 = *reinterpret_cast<const uint32_t *>(v2 + col) ^ 0x80808080u;
                        const uint32_t w3 = *reinterpret_cast<const uint32_t *>(v3 + col) ^ 0x80808080u;
                        // interleave key pairs: e01 = (k0.d0, k1.d0, k0.d1, k1.d1), f01 = (k0.d2, k1.d2, k0.d3, k1.d3)
                        const uint32_t e01 = __byte_perm(w0, w1, 0x5140), f01 = __byte_perm(w0, w1, 0x7362);
                        const uint32_t e23 = __byte_perm(w2, w3, 0x5140), f23 = __byte_perm(w2, w3, 0x7362);
                        ax[0] = cvt_i8x2<0>(e01); ax[1] = cvt_i8x2<1>(e01); ax[2] = cvt_i8x2<0>(e23); ax[3] = cvt_i8x2<1>(e23);
                        ay[0] = cvt_i8x2<0>(f01); ay[1] = cvt_i8x2<1>(f01); ay[2] = cvt_i8x2<0>(f23); ay[3] = cvt_i8x2<1>(f23);
                    } else {
                        const int col = 18 * blk + 2 + 2 * g;   // bytes 2g, 2g+1 of the block: dims 2g, 2g+1 | 16+2g, 17+2g
                        const uint32_t h0 = *reinterpret_cast<const uint16_t *>(v0 + col), h1 = *reinterpret_cast<const uint16_t *>(v1 + col);
                        const uint32_t h2 = *reinterpret_cast<const uint16_t *>(v2 + col), h3 = *reinterpret_cast<const uint16_t *>(v3 + col);
                        const uint32_t w01 = h0 | (h1 << 16), w23 = h2 | (h3 << 16);   // bytes (k0.B0, k0.B1, k1.B0, k1.B1)
                        const uint32_t l01 = w01 & 0x0f0f0f0fu, u01 = (w01 >> 4) & 0x0f0f0f0fu;
                        const uint32_t l23 = w23 & 0x0f0f0f0fu, u23 = (w23 >> 4) & 0x0f0f0f0fu;
                        // (k0.x, k1.x) pairs: bytes 0 and 2 -> dim 2g (+16), bytes 1 and 3 -> dim 2g+1 (+16)
                        ax[0] = hsub2_u32(__byte_perm(l01, 0x64646464u, 0x6240), 0x64086408u);
                        ax[1] = hsub2_u32(__byte_perm(l01, 0x64646464u, 0x7351), 0x64086408u);
                        ax[2] = hsub2_u32(__byte_perm(l23, 0x64646464u, 0x6240), 0x64086408u);
                        ax[3] = hsub2_u32(__byte_perm(l23, 0x64646464u, 0x7351), 0x64086408u);
                        ay[0] = hsub2_u32(__byte_perm(u01, 0x64646464u, 0x6240), 0x64086408u);
                        ay[1] = hsub2_u32(__byte_perm(u01, 0x64646464u, 0x7351), 0x64086408u);
                        ay[2] = hsub2_u32(__byte_perm(u23, 0x64646464u, 0x6240), 0x64086408u);
                        ay[3] = hsub2_u32(__byte_perm(u23, 0x64646464u, 0x7351), 0x64086408u);
                    }
                    const uint32_t sd0 = *reinterpret_cast<const uint32_t *>(Sd + blk * SDSTR + (16 * u + 2 * t) * 2);
                    const uint32_t sd1 = *reinterpret_cast<const uint32_t *>(Sd + blk * SDSTR + (16 * u + 2 * t + 8) * 2);
                    // block scale of each key pair folded into V (f16 product of an exact integer and the f16 scale)
                    ax[0] = hmul2_u32(ax[0], sd0); ax[1] = hmul2_u32(ax[1], sd0); ax[2] = hmul2_u32(ax[2], sd1); ax[3] = hmul2_u32(ax[3], sd1);
                    ay[0] = hmul2_u32(ay[0], sd0); ay[1] = hmul2_u32(ay[1], sd0); ay[2] = hmul2_u32(ay[2], sd1); ay[3] = hmul2_u32(ay[3], sd1);
#pragma unroll
                    for (int i = 0; i < NT; ++i) {
                        mma16816(O[2 * y][i], ax, pw[i][0], pw[i][1]);
                        mma16816(O[2 * y + 1][i], ay, pw[i][0], pw[i][1]);
                    }
                }
            }
        }
        last_v = arrive(1);
        sv_prev = sv_now;
        if constexpr (PARK) park();
    }
    if constexpr (PARK) unpark();

    // ---------------- write the unit's partial ----------------
    // l: sum over the lanes that share this row pair (same t), then over the warps
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float l = l_run[i][e];
            l += __shfl_xor_sync(0xffffffffu, l, 4);
            l += __shfl_xor_sync(0xffffffffu, l, 8);
            l += __shfl_xor_sync(0xffffffffu, l, 16);
            if (g == 0) wl[w * NT * 8 + 8 * i + 2 * t + e] = l;
        }
    __syncthreads();
    if (w == 0 && g == 0) {
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int r = 8 * i + 2 * t + e;
                if (r < R) {
                    a.pm[unit * R + r] = m_run[i][e];
                    a.pl[unit * R + r] = (wl[r] + wl[NT * 8 + r]) + (wl[2 * NT * 8 + r] + wl[3 * NT * 8 + r]);
                }
            }
    }
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int r = 8 * i + 2 * t + e;
            if (r >= R) continue;
            float * dst = a.po + (unit * R + r) * DH;
            if constexpr (KT == B200_KV_F16) {
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) {
                    dst[64 * w + 16 * mt + g] = O[mt][i][e];
                    dst[64 * w + 16 * mt + g + 8] = O[mt][i][2 + e];
                }
            } else if constexpr (KT == B200_KV_Q8_0) {
#pragma unroll
                for (int y = 0; y < 2; ++y)
                    *reinterpret_cast<float4 *>(dst + 64 * w + 32 * y + 4 * g) =
                        make_float4(O[2 * y][i][e], O[2 * y][i][2 + e], O[2 * y + 1][i][e], O[2 * y + 1][i][2 + e]);
            } else {
#pragma unroll
                for (int y = 0; y < 2; ++y) {
                    *reinterpret_cast<float2 *>(dst + 64 * w + 32 * y + 2 * g) = make_float2(O[2 * y][i][e], O[2 * y][i][2 + e]);
                    *reinterpret_cast<float2 *>(dst + 64 * w + 32 * y + 16 + 2 * g) = make_float2(O[2 * y + 1][i][e], O[2 * y + 1][i][2 + e]);
                }
            }
        }
    return ntiles;
}

#include "decode_tc.cuh"

// The kernel: one unit per CTA (the grid enumerates (slot, chunk), directly or through the work list), or, with the even
// split, every segment of the CTA's run one after the other.
template <uint32_t KT, int NT>
__global__ void __launch_bounds__(NTHR, ctas_per_sm<KT, NT>())
decode_part_k(const dec_args a, const int nslot, const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV) {
    extern __shared__ __align__(1024) unsigned char smem[];
    // blockIdx.x = unit * Hkv + kv head: the heads of one (slot, key range) are neighbours in launch order, so the four
    // head rows of a position are fetched close together in time
    const int hk = (int) (blockIdx.x % (unsigned) a.g.Hkv), ui = (int) (blockIdx.x / (unsigned) a.g.Hkv);
    int s0 = 0, s1 = 1, slot = 0, k_lo = 0, k_cap = 0;
    size_t unit = 0;
    if (a.segs) {
        if (ui >= *a.n_cta) return;
        s0 = a.cta_seg[ui]; s1 = a.cta_seg[ui + 1];
        if (s0 >= s1) return;
    } else {
        int chunk;
        if (a.units) {
            if (ui >= *a.n_units) return;
            const int2 u = a.units[ui];
            slot = u.x; chunk = u.y;
        } else {
            slot = ui / a.max_chunks; chunk = ui - slot * a.max_chunks;
        }
        int n = 0;
        for (int j = 0; j < a.q_len; ++j) n = max(n, row_pos(a, slot, j) + 1);
        k_lo = chunk * a.CH;
        if (k_lo >= min(n, key_limit(a))) return;   // the chunk lies past the slot's keys
        k_cap = k_lo + a.CH;
        unit = ((size_t) slot * a.g.Hkv + hk) * a.max_chunks + chunk;
    }
    // barriers of the copy ring, arrival counters and flags: made once per CTA
    if (threadIdx.x == 0) {
        uint64_t * full = reinterpret_cast<uint64_t *>(smem);
        for (int s = 0; s < nslot; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
        int * cnt = reinterpret_cast<int *>(smem + 96);   // done[2], flag[3]
        cnt[0] = cnt[1] = cnt[2] = cnt[3] = cnt[4] = 0;
    }
    uint32_t t_base = 0;
    uint32_t * t_slot = reinterpret_cast<uint32_t *>(smem + 120);
    if constexpr (parks<KT, NT>()) {
        if (threadIdx.x >= 32 && threadIdx.x < 64) umma::tmem_alloc(t_slot, PARK_COLS);
        umma::fence_before_sync();
    }
    __syncthreads();
    if constexpr (parks<KT, NT>()) {
        umma::fence_after_sync();
        t_base = *t_slot;
    }
    int tiles = 0;
    for (int sg = s0; sg < s1; ++sg) {
        if (a.segs) {
            const int4 e = a.segs[sg];
            slot = e.x; k_lo = e.y; k_cap = e.z;
            unit = (size_t) sg * a.g.Hkv + hk;
        }
        if (sg > s0) __syncthreads();   // the previous segment's shared memory is no longer read
        tiles += decode_unit<KT, NT>(a, nslot, mapK, mapV, smem, hk, slot, k_lo, k_cap, unit, tiles, t_base);
    }
    if constexpr (parks<KT, NT>()) {
        umma::fence_before_sync();
        __syncthreads();
        if (threadIdx.x >= 32 && threadIdx.x < 64) {
            umma::fence_after_sync();
            umma::tmem_dealloc(t_base, PARK_COLS);
        }
    }
}

// Merge a row's chunk partials.  grid (rows, Hq), MERGE_GROUPS groups of 64 threads (one float4 of the head each): group w
// sums the chunks w, w + G, .. in ascending order, the group sums are added in group order: a fixed order for a given number
// of chunks, so a row's result does not depend on the rest of the call (the fixed-chunk modes run four groups).
//   out != nullptr : out = num / den (* sigmoid(gate)); rows that saw no key give zeros
//   fo  != nullptr : unnormalised num, max in natural-log units, den (for a cross-GPU merge)
// The even split leaves one to a few partials per row (one per CTA run that crosses the slot): there one group of 64 threads
// per (row, head) keeps the launch to little more than one wave of small blocks.
template <int MERGE_GROUPS>
__global__ void __launch_bounds__(64 * MERGE_GROUPS) decode_merge_k(const dec_args a, const float * __restrict__ gate, float * __restrict__ out,
                                                     float * __restrict__ fo, float * __restrict__ fm, float * __restrict__ fl,
                                                     __half2 * __restrict__ qbuf) {
    __shared__ float4 gnum[MERGE_GROUPS > 1 ? MERGE_GROUPS - 1 : 1][64];
    __shared__ float gden[MERGE_GROUPS > 1 ? MERGE_GROUPS - 1 : 1];
    const int lane4 = threadIdx.x & 63, grp = threadIdx.x >> 6;
    const int h = blockIdx.y, row = blockIdx.x, slot = row / a.q_len, j = row - slot * a.q_len;
    const int hk = h / GQA, hh = h - hk * GQA, r = j * GQA + hh, R = a.q_len * GQA;
    const int pos = min(row_pos(a, slot, j), key_limit(a) - 1);   // a row past the limit merges the chunks that exist
    // partials of the row's kv head: consecutive units of stride ustr from unit0 (a segment the row does not reach holds m = -inf)
    int nch;
    size_t unit0, ustr;
    if (a.segs) {
        const int2 sg = a.slot_seg[slot];
        nch = pos < 0 ? 0 : sg.y;
        unit0 = (size_t) sg.x * a.g.Hkv + hk; ustr = a.g.Hkv;
    } else {
        nch = pos < 0 ? 0 : pos / a.CH + 1;
        unit0 = ((size_t) slot * a.g.Hkv + hk) * a.max_chunks; ustr = 1;
    }
    float M = B200_NEG_INF;
    for (int c = 0; c < nch; ++c) M = fmaxf(M, a.pm[(unit0 + c * ustr) * R + r]);
    float den = 0.0f;
    float4 num = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 4
    for (int c = grp; c < nch; c += MERGE_GROUPS) {   // no early continue: the loads of several chunks are in flight together
        const size_t u = unit0 + c * ustr;
        const float ms = a.pm[u * R + r];
        const float f = ms == B200_NEG_INF ? 0.0f : ex2f(ms - M);   // a chunk the row did not see holds zeros: adds nothing
        den = fmaf(f, a.pl[u * R + r], den);
        const float4 o = reinterpret_cast<const float4 *>(a.po + (u * R + r) * DH)[lane4];
        num.x = fmaf(f, o.x, num.x); num.y = fmaf(f, o.y, num.y); num.z = fmaf(f, o.z, num.z); num.w = fmaf(f, o.w, num.w);
    }
    if constexpr (MERGE_GROUPS > 1) {
        if (grp > 0) {
            gnum[grp - 1][lane4] = num;
            if (lane4 == 0) gden[grp - 1] = den;
        }
        __syncthreads();
        if (grp > 0) return;
#pragma unroll
        for (int w = 0; w < MERGE_GROUPS - 1; ++w) {
            const float4 o = gnum[w][lane4];
            num.x += o.x; num.y += o.y; num.z += o.z; num.w += o.w;
            den += gden[w];
        }
    }
    const size_t oi = ((size_t) row * a.Hq + h) * (DH / 4) + lane4;
    if (fo) {   // public partials are plain sums: take the internal 2^PSHIFT out (exact)
        constexpr float U = 1.0f / 256.0f;
        static_assert(PSHIFT == 8.0f, "U must be 2^-PSHIFT");
        reinterpret_cast<float4 *>(fo)[oi] = make_float4(num.x * U, num.y * U, num.z * U, num.w * U);
        if (lane4 == 0) { fm[(size_t) row * a.Hq + h] = M * LN2; fl[(size_t) row * a.Hq + h] = den * U; }
    }
    if (out) {
        float4 y = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (den > 0.0f) {
            const float inv = 1.0f / den;
            y = make_float4(num.x * inv, num.y * inv, num.z * inv, num.w * inv);
            if (gate) {
                const float4 gv = reinterpret_cast<const float4 *>(gate)[oi];
                y.x *= 1.0f / (1.0f + expf(-gv.x)); y.y *= 1.0f / (1.0f + expf(-gv.y));
                y.z *= 1.0f / (1.0f + expf(-gv.z)); y.w *= 1.0f / (1.0f + expf(-gv.w));
            }
        }
        reinterpret_cast<float4 *>(out)[oi] = y;
        // the projection that follows attention reads its input in the a16 format: emitted here, from registers
        if (qbuf) a16_store_lanes8(y, qbuf, (size_t) row * (a.Hq * (DH / 32)) + h * (DH / 32) + (lane4 >> 3),
                                   (size_t) gridDim.x * (a.Hq * (DH / 32)), true);
    }
}

// Merge of caller-provided partials (cross-GPU sequence split): part s has O [R][D] at po + s * so, m (natural log) [R] at
// pm + s * sm and l [R] at pl + s * sm (strides in floats); one block per row, D/4 threads.
__global__ void merge_parts_k(const float * __restrict__ po, const float * __restrict__ pm, const float * __restrict__ pl,
                              int nparts, int R, int D, const float * __restrict__ gate, float * __restrict__ out, size_t so,
                              size_t sm, __half2 * __restrict__ qbuf) {
    const int r = blockIdx.x, i = threadIdx.x;
    float M = B200_NEG_INF;
    for (int s = 0; s < nparts; ++s) M = fmaxf(M, pm[s * sm + r]);
    float den = 0.0f;
    float4 num = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s = 0; s < nparts; ++s) {
        const float ms = pm[s * sm + r];
        if (ms == B200_NEG_INF) continue;
        const float f = ex2f((ms - M) * LOG2E);
        den = fmaf(f, pl[s * sm + r], den);
        const float4 o = reinterpret_cast<const float4 *>(po + s * so + (size_t) r * D)[i];
        num.x = fmaf(f, o.x, num.x); num.y = fmaf(f, o.y, num.y); num.z = fmaf(f, o.z, num.z); num.w = fmaf(f, o.w, num.w);
    }
    float4 y = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (den > 0.0f) {
        const float inv = 1.0f / den;
        y = make_float4(num.x * inv, num.y * inv, num.z * inv, num.w * inv);
        if (gate) {
            const float4 gv = reinterpret_cast<const float4 *>(gate + (size_t) r * D)[i];
            y.x *= 1.0f / (1.0f + expf(-gv.x)); y.y *= 1.0f / (1.0f + expf(-gv.y));
            y.z *= 1.0f / (1.0f + expf(-gv.z)); y.w *= 1.0f / (1.0f + expf(-gv.w));
        }
    }
    reinterpret_cast<float4 *>(out + (size_t) r * D)[i] = y;
    // a16 copy of the gated output (rows of row_len = heads * D values): group index = float index / 32
    if (qbuf) a16_store_lanes8(y, qbuf, ((size_t) r * D + 4 * i) / 32, (size_t) R * D / 32, true);
}

// The same merge with the shards' partials read in place: shard s of a sequence split keeps its partial [O (R*D) | m (R) | l (R)]
// in a buffer that its peers have mapped (part[s]: this GPU's own buffer for s == me, a peer mapping otherwise) and a row of
// flag words flag[s][0..n_seq) that shard j writes at index j.  A call with epoch e (1, 2, .. in step on all shards)
//   1. tells every peer "my partial of call e is complete" (the kernel that wrote it ran before this one on the stream),
//   2. waits, bounded, until every peer has said the same,
//   3. merges in shard order, reading the peers' rows over NVLink with plain loads that bypass L1.
// The caller alternates two partial buffers by the parity of e: a peer that announces call e + 1 has finished reading the
// buffer of call e, and this shard passes step 2 of call e + 1 before the kernel that rewrites that buffer (call e + 2)
// can start.  One block per row, D/4 threads; the first four blocks announce, every block waits by itself.
constexpr int MAX_PEERS = 8;
struct peer_parts { const float * part[MAX_PEERS]; unsigned * flag[MAX_PEERS]; };

__device__ __forceinline__ float4 ld_sys_f4(const float * p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ld_sys_f(const float * p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

__global__ void merge_peers_k(const peer_parts pp, int n_seq, int me, unsigned epoch, int R, int D, const float * __restrict__ gate,
                              float * __restrict__ out, __half2 * __restrict__ qbuf, unsigned * __restrict__ status) {
    const int r = blockIdx.x, i = threadIdx.x;
    // the first blocks of the grid announce (any one would do; a few, so that the announcement does not hang on one block's
    // turn); every block waits by itself
    if (r < 4 && i < n_seq && i != me)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pp.flag[i] + me), "r"(epoch) : "memory");
    if (i < n_seq && i != me) {
        const unsigned * f = pp.flag[me] + i;
        unsigned v;
        const unsigned long long t0 = globaltimer_ns();
        for (int it = 0;; ++it) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if ((int) (v - epoch) >= 0) break;
            if ((it & 63) == 63 && globaltimer_ns() - t0 > 2000000000ull) { atomicOr(status, ST_WAIT_TIMEOUT); break; }
        }
    }
    __syncthreads();
    const size_t om = (size_t) R * D, ol = om + R;
    float ms[MAX_PEERS];
    float M = B200_NEG_INF;
#pragma unroll
    for (int s = 0; s < MAX_PEERS; ++s) {
        ms[s] = B200_NEG_INF;
        if (s < n_seq) ms[s] = s == me ? pp.part[s][om + r] : ld_sys_f(pp.part[s] + om + r);
        M = fmaxf(M, ms[s]);
    }
    float den = 0.0f;
    float4 num = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int s = 0; s < MAX_PEERS; ++s) {
        if (s >= n_seq || ms[s] == B200_NEG_INF) continue;
        const float f = ex2f((ms[s] - M) * LOG2E);
        const float * po = pp.part[s] + (size_t) r * D + 4 * i;
        const float l = s == me ? pp.part[s][ol + r] : ld_sys_f(pp.part[s] + ol + r);
        const float4 o = s == me ? *reinterpret_cast<const float4 *>(po) : ld_sys_f4(po);
        den = fmaf(f, l, den);
        num.x = fmaf(f, o.x, num.x); num.y = fmaf(f, o.y, num.y); num.z = fmaf(f, o.z, num.z); num.w = fmaf(f, o.w, num.w);
    }
    float4 y = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (den > 0.0f) {
        const float inv = 1.0f / den;
        y = make_float4(num.x * inv, num.y * inv, num.z * inv, num.w * inv);
        if (gate) {
            const float4 gv = reinterpret_cast<const float4 *>(gate + (size_t) r * D)[i];
            y.x *= 1.0f / (1.0f + expf(-gv.x)); y.y *= 1.0f / (1.0f + expf(-gv.y));
            y.z *= 1.0f / (1.0f + expf(-gv.z)); y.w *= 1.0f / (1.0f + expf(-gv.w));
        }
    }
    reinterpret_cast<float4 *>(out + (size_t) r * D)[i] = y;
    if (qbuf) a16_store_lanes8(y, qbuf, ((size_t) r * D + 4 * i) / 32, (size_t) R * D / 32, true);
}

// Work list of a batched call: every (slot, chunk) that holds at least one visible key, longest first.  Whole chunks
// come first (all the same length), then the slots' last, shorter chunks in descending order of their tile count, so the
// tail of the launch is made of the shortest units.  One block; writes units[] and *n_units.  The order of equal-length
// units depends on the order of the atomics and does not affect any result (units are independent).
constexpr int PLAN_THR = 256, PLAN_BUCKETS = 256;
__global__ void __launch_bounds__(PLAN_THR) decode_plan_k(const dec_args a, int2 * __restrict__ units, int * __restrict__ n_units) {
    __shared__ int hist[PLAN_BUCKETS], total_full, cur_full;
    const int tid = threadIdx.x;
    const int tiles_per_chunk = a.CH / TILE;
    for (int i = tid; i < PLAN_BUCKETS; i += PLAN_THR) hist[i] = 0;
    if (tid == 0) { total_full = 0; cur_full = 0; }
    __syncthreads();
    const int lim = key_limit(a);
    auto slot_keys = [&](int s) {
        int n = 0;
        for (int j = 0; j < a.q_len; ++j) n = max(n, row_pos(a, s, j) + 1);
        return min(n, lim);
    };
    // bucket of a last chunk: its tile count scaled into PLAN_BUCKETS classes, descending (bucket 0 = longest)
    auto bucket_of = [&](int tail_keys) {
        const int tiles = (tail_keys + TILE - 1) / TILE;   // 1 .. tiles_per_chunk - 1 (a whole chunk is not a tail) or tiles_per_chunk
        const long long cls = (long long) (tiles_per_chunk - tiles) * PLAN_BUCKETS / max(tiles_per_chunk, 1);
        return (int) min((long long) PLAN_BUCKETS - 1, max(0LL, cls));
    };
    for (int s = tid; s < a.n_slots; s += PLAN_THR) {
        const int n = slot_keys(s), nfull = n / a.CH, tail = n - nfull * a.CH;
        if (nfull) atomicAdd(&total_full, nfull);
        if (tail) atomicAdd(&hist[bucket_of(tail)], 1);
    }
    __syncthreads();
    if (tid == 0) {   // exclusive scan of the tail classes, placed after the whole chunks
        int run = total_full;
        for (int i = 0; i < PLAN_BUCKETS; ++i) { const int c = hist[i]; hist[i] = run; run += c; }
        *n_units = run;
    }
    __syncthreads();
    for (int s = tid; s < a.n_slots; s += PLAN_THR) {
        const int n = slot_keys(s), nfull = n / a.CH, tail = n - nfull * a.CH;
        if (nfull) {
            const int base = atomicAdd(&cur_full, nfull);
            for (int c = 0; c < nfull; ++c) units[base + c] = make_int2(s, c);
        }
        if (tail) units[atomicAdd(&hist[bucket_of(tail)], 1)] = make_int2(s, nfull);
    }
}

// Even split of a batch over the resident CTAs (used when the chunk is chosen from the batch).  The 64-key tiles of all
// slots, slot after slot, form one sequence per kv head; CTA c of n_cta takes tiles [c W / n_cta, (c + 1) W / n_cta), so
// every CTA has the same work to within one tile however ragged the contexts are, and all CTAs fit the machine at once.  A
// run that crosses slot boundaries becomes several segments; each segment yields one partial.  n_cta = min(max_cta, W /
// SPLIT_MIN_TILES) keeps runs from getting so short that start-up and the merge dominate.  One block; n_slots <= SPLIT_MAX_SLOTS.
constexpr int SPLIT_THR = 1024, SPLIT_MAX_SLOTS = 2048, SPLIT_MAX_CTA = 1024, SPLIT_MIN_TILES = 4;
__global__ void __launch_bounds__(SPLIT_THR) decode_split_k(const dec_args a, int max_cta, int4 * __restrict__ segs, int * __restrict__ cta_seg,
                                                            int2 * __restrict__ slot_seg, int * __restrict__ n_cta_out) {
    __shared__ int pre[SPLIT_MAX_SLOTS + 1];     // tiles before slot s
    __shared__ int cseg[SPLIT_MAX_CTA + 1];      // segments before CTA c
    __shared__ int first_slot[SPLIT_MAX_CTA];
    const int tid = threadIdx.x, lim = key_limit(a);
    auto slot_keys = [&](int s) {
        int n = 0;
        for (int j = 0; j < a.q_len; ++j) n = max(n, row_pos(a, s, j) + 1);
        return min(n, lim);
    };
    for (int s = tid; s < a.n_slots; s += SPLIT_THR) pre[s + 1] = (slot_keys(s) + TILE - 1) / TILE;
    if (tid == 0) pre[0] = 0;
    __syncthreads();
    if (tid < 32) {   // inclusive scan of pre[1..n_slots], 32 entries at a time with a running carry
        int carry = 0;
        for (int base = 1; base <= a.n_slots; base += 32) {
            const int i = base + tid;
            int v = i <= a.n_slots ? pre[i] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, v, o); if (tid >= o) v += u; }
            if (i <= a.n_slots) pre[i] = v + carry;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
    const long long W = pre[a.n_slots];
    const int n_cta = (int) max(1LL, min((long long) min(max_cta, SPLIT_MAX_CTA), W / SPLIT_MIN_TILES));
    auto cut = [&](int c) { return (int) (W * c / n_cta); };
    // segments per CTA: the slots its run intersects
    int my_first = 0, my_cnt = 0;
    if (tid < n_cta) {
        const int lo = cut(tid), hi = cut(tid + 1);
        if (hi > lo) {
            int l = 0, r = a.n_slots;               // last slot with pre[s] <= lo
            while (r - l > 1) { const int m = (l + r) >> 1; if (pre[m] <= lo) l = m; else r = m; }
            while (pre[l + 1] <= lo) ++l;           // skip empty slots
            my_first = l;
            int e = l;
            while (e < a.n_slots && pre[e] < hi) { if (pre[e + 1] > pre[e] && pre[e + 1] > lo) ++my_cnt; ++e; }
        }
        first_slot[tid] = my_first;
        cseg[tid + 1] = my_cnt;
    }
    if (tid == 0) cseg[0] = 0;
    __syncthreads();
    if (tid < 32) {
        int carry = 0;
        for (int base = 1; base <= n_cta; base += 32) {
            const int i = base + tid;
            int v = i <= n_cta ? cseg[i] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, v, o); if (tid >= o) v += u; }
            if (i <= n_cta) cseg[i] = v + carry;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
    if (tid <= n_cta) cta_seg[tid] = cseg[tid];
    if (tid == 0) *n_cta_out = W > 0 ? n_cta : 0;
    if (tid < n_cta && my_cnt > 0) {
        const int lo = cut(tid), hi = cut(tid + 1);
        int o = cseg[tid];
        for (int s = my_first; s < a.n_slots && pre[s] < hi; ++s) {
            if (pre[s + 1] <= pre[s] || pre[s + 1] <= lo) continue;
            const int t0 = max(lo, pre[s]) - pre[s], t1 = min(hi, pre[s + 1]) - pre[s];
            segs[o++] = make_int4(s, t0 * TILE, t1 * TILE, 0);
        }
    }
    // the segments of a slot are consecutive: from the CTA that holds its first tile to the one that holds its last
    for (int s = tid; s < a.n_slots; s += SPLIT_THR) {
        if (pre[s + 1] <= pre[s]) { slot_seg[s] = make_int2(0, 0); continue; }
        auto cta_of = [&](int tile) {
            int c = (int) min((long long) n_cta - 1, ((long long) tile * n_cta) / max(W, 1LL));
            while (c > 0 && cut(c) > tile) --c;
            while (c + 1 < n_cta && cut(c + 1) <= tile) ++c;
            return c;
        };
        const int c0 = cta_of(pre[s]), c1 = cta_of(pre[s + 1] - 1);
        // inside CTA c0 the slot's segment comes after those of the non-empty slots first_slot[c0] .. s-1
        int before = 0;
        for (int z = first_slot[c0]; z < s; ++z) if (pre[z + 1] > pre[z] && pre[z + 1] > cut(c0)) ++before;
        slot_seg[s] = make_int2(cseg[c0] + before, c1 - c0 + 1);
    }
}

// ------------------------------------------------------------------------------------------------ host side ----
constexpr int DEFAULT_CHUNK = 512;
constexpr int MAX_DEFAULT_CHUNKS = 256;   // the default chunk grows with n_ctx so that a context never has more chunks than this
int g_chunk = 0;            // 0 = not read yet; else B200ATTN_CHUNK or DEFAULT_CHUNK
bool g_chunk_from_env = false;
int g_nsplit_override = 0;  // set_nsplit: chunks per full context

int round_tile(long long v) { return (int) ((std::max<long long>(v, TILE) + TILE - 1) / TILE * TILE); }
int env_chunk(bool * from_env) {
    const char * e = getenv("B200ATTN_CHUNK");
    const bool have = e && *e && atoi(e) > 0;
    if (from_env) *from_env = have;
    return round_tile(have ? atoi(e) : DEFAULT_CHUNK);
}
int default_chunk() {
    if (!g_chunk) g_chunk = env_chunk(&g_chunk_from_env);
    return g_chunk;
}
// The chunk of a call that asks for the library default: a function of the cache's capacity only, so that a row's bits do
// not depend on the batch it is decoded in.  set_nsplit(n) pins n chunks per full context; B200ATTN_CHUNK pins the keys.
int fixed_chunk(int n_ctx) {
    const int base = default_chunk();
    if (g_nsplit_override > 0) return round_tile(((long long) std::max(n_ctx, 1) + g_nsplit_override - 1) / g_nsplit_override);
    if (g_chunk_from_env) return base;
    return std::max(base, round_tile(((long long) std::max(n_ctx, 1) + MAX_DEFAULT_CHUNKS - 1) / MAX_DEFAULT_CHUNKS));
}

// Split partials and the work list live in one library-owned buffer per (device, stream), as in the reference
// (src/fast/attn_dec2.cu:452-464,503-517): sized on the first call or by b200_attn_reserve, and from then on calls that
// fit neither allocate nor synchronise, and the pointer does not move (recorded work stays valid).  A call that needs more
// gets a new, larger buffer; the old one is kept allocated until the process exits, so nothing that was recorded against
// it ever reads freed memory, and no stream is synchronised.
// The even split of a batch depends on the rows' positions only, which a model step does not change from layer to layer.
// Between b200_attn_step_begin(stream, positions, bytes) and the next one (or b200_attn_step_end) the plan that the first
// batched call of a given shape, with its positions inside the declared array, leaves in the stream's scratch is used again by
// the following calls of the same shape instead of being recomputed: what identifies the plan is kept here, and any other
// call on the stream drops it.
struct plan_key {
    const void * scr = nullptr, * pos = nullptr, * p0p = nullptr;
    int p0 = 0, n_slots = 0, q_len = 0, max_chunks = 0, max_cta = 0, Hkv = 0, n_ctx = 0, paged = 0;
    size_t part_floats = 0;
    bool operator==(const plan_key & o) const {
        return scr == o.scr && pos == o.pos && p0p == o.p0p && p0 == o.p0 && n_slots == o.n_slots && q_len == o.q_len &&
               max_chunks == o.max_chunks && max_cta == o.max_cta && Hkv == o.Hkv && n_ctx == o.n_ctx && paged == o.paged &&
               part_floats == o.part_floats;
    }
};
struct scratch {
    int dev = -1; cudaStream_t s = nullptr; float * p = nullptr; size_t cap = 0;
    bool step_mode = false, plan_valid = false;
    const char * step_lo = nullptr, * step_hi = nullptr;   // the position array the caller declared fixed for the step
    plan_key key;
};
scratch g_scr[64];
int g_nscr = 0;
std::mutex g_mu;

scratch * scratch_entry(cudaStream_t s, size_t floats, size_t floats_hint) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(g_mu);
    scratch * e = nullptr;
    for (int i = 0; i < g_nscr; ++i) if (g_scr[i].dev == dev && g_scr[i].s == s) e = &g_scr[i];
    if (!e) {
        if (g_nscr == 64) return nullptr;
        e = &g_scr[g_nscr++];
        e->dev = dev; e->s = s;
    }
    if (floats > e->cap) {
        const size_t want = std::max(std::max(floats, floats_hint), std::max(e->cap + e->cap / 2, (size_t) 1 << 20));
        float * p = nullptr;
        if (cudaMalloc(&p, want * sizeof(float)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        e->p = p;      // the previous buffer, if any, stays allocated (see above)
        e->cap = want;
        e->plan_valid = false;
    }
    return e;
}
float * scratch_for(cudaStream_t s, size_t floats, size_t floats_hint) {
    scratch * e = scratch_entry(s, floats, floats_hint);
    return e ? e->p : nullptr;
}

// ---- tensor maps of the cache ----------------------------------------------------------------------------------
// K and V as rank-3 tensors of 16-bit elements: x = the row of one position (all kv heads), y = position inside a page
// (or in the whole cache when it is contiguous), z = page.  The box is one head's bytes of 64 consecutive positions.
// f16 rows (512 B per head) are wider than a box may be, and their shared-memory image is swizzled: rank 4 with x = 64
// elements (128 B), y = position, z = 128-byte chunk of the row, w = page; box = 64 x 64 x 4 chunks, 128-byte swizzle.
using encode_tiled_fn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                     const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_tiled_fn tensor_map_encoder() {
    static encode_tiled_fn fn = [] {
        void * p = nullptr;
        cudaDriverEntryPointQueryResult r;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &r) != cudaSuccess || r != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            p = nullptr;
        }
        return (encode_tiled_fn) p;
    }();
    return fn;
}
// Encoding a map is pure host arithmetic on (base, geometry); the last few are kept, since a serving loop calls with the
// same caches (one K and one V per layer) every step.
struct map_entry { const char * base; unsigned long long rowb, pstride, rows; int HB; bool paged; CUtensorMap m; };
constexpr int MAP_CACHE = 256;
map_entry g_maps[MAP_CACHE];
int g_nmaps = 0, g_map_next = 0;
std::mutex g_map_mu;

bool make_cache_map(CUtensorMap * m, const char * base, const dec_args & a, int HB) {
    encode_tiled_fn enc = tensor_map_encoder();
    if (!enc) return false;
    const bool paged = a.g.pt != nullptr;
    const cuuint64_t rows = paged ? (cuuint64_t) 1 << a.g.psh : (cuuint64_t) a.n_ctx;
    const unsigned long long pstr = paged ? a.g.pstride : 0;
    {
        std::lock_guard<std::mutex> lk(g_map_mu);
        for (int i = 0; i < g_nmaps; ++i) {
            const map_entry & e = g_maps[i];
            if (e.base == base && e.rowb == a.g.rowb && e.pstride == pstr && e.rows == rows && e.HB == HB && e.paged == paged) {
                *m = e.m;
                return true;
            }
        }
    }
    const cuuint64_t npages = paged ? (cuuint64_t) 0x7fffffff : 1, pbytes = paged ? a.g.pstride : a.g.rowb * rows;
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult rc;
    if (HB == head_bytes(B200_KV_F16)) {
        const cuuint64_t gdim[4] = {64, rows, a.g.rowb / 128, npages};
        const cuuint64_t gstr[3] = {a.g.rowb, 128, pbytes};
        const cuuint32_t box[4] = {64, (cuuint32_t) TILE, 4, 1};
        rc = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, (void *) base, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        const cuuint64_t gdim[3] = {a.g.rowb / 2, rows, npages};
        const cuuint64_t gstr[2] = {a.g.rowb, pbytes};
        const cuuint32_t box[3] = {(cuuint32_t) HB / 2, (cuuint32_t) TILE, 1};
        rc = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, (void *) base, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (rc != CUDA_SUCCESS) return false;
    std::lock_guard<std::mutex> lk(g_map_mu);
    map_entry & e = g_maps[g_map_next];
    g_map_next = (g_map_next + 1) % MAP_CACHE;
    if (g_nmaps < MAP_CACHE) ++g_nmaps;
    e.base = base; e.rowb = a.g.rowb; e.pstride = pstr; e.rows = rows; e.HB = HB; e.paged = paged; e.m = *m;
    return true;
}

template <uint32_t KT, int NT> size_t smem_bytes(int nslot) {
    return HDR + (size_t) nslot * traits<KT>::SLOT + NT * 8 * (QSTR + PSTR) + 8 * SDSTR + 2 * NWARP * NT * 8 * sizeof(float) +
           (traits<KT>::SCALED ? NBLK * NT * 4 * sizeof(float4) : 0);
}

template <uint32_t KT, int NT>
int launch_part(const dec_args & a_in, unsigned blocks, cudaStream_t s) {
    dec_args a = a_in;
    CUtensorMap mapK, mapV;
    memset(&mapK, 0, sizeof mapK);
    memset(&mapV, 0, sizeof mapV);
    // tiled copies need a tile inside one page (pages of at least 64 rows), 16-byte row strides and a contiguous cache short
    // enough for the stride field; anything else keeps the row-by-row copies
    a.tiled = 0;
    if ((!a.g.pt || a.g.psh >= 6) && a.g.rowb % 16 == 0 &&
        (a.g.pt ? a.g.pstride < ((unsigned long long) 1 << 40) : (a.n_ctx >= 1 && a.g.rowb * (unsigned long long) a.n_ctx < ((unsigned long long) 1 << 40))))
        a.tiled = make_cache_map(&mapK, a.g.k, a, traits<KT>::HB) && make_cache_map(&mapV, a.g.v, a, traits<KT>::HB);
    // as many CTAs per SM as the kernel is compiled for, if a ring of two half-tile slots fits that often into the 227 KB of
    // an SM; then the deepest ring (up to 8 slots) that still fits
    auto fits = [](int n, int ctas) { return (size_t) ctas * (smem_bytes<KT, NT>(n) + 1024) <= (size_t) 227 * 1024; };
    int ctas = ctas_per_sm<KT, NT>();
    while (ctas > 1 && !fits(2, ctas)) --ctas;
    int nslot = 2;
    while (nslot < 8 && fits(nslot + 1, ctas)) ++nslot;
    const size_t sm = smem_bytes<KT, NT>(nslot);
    static std::atomic<bool> attr_done[64];   // per instantiation and device; setting the attribute twice is harmless
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(decode_part_k<KT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sm) != cudaSuccess)
            return launch_status("attn_decode (shared memory attribute)");
        cudaFuncSetAttribute(decode_part_k<KT, NT>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        attr_done[dev & 63].store(true, std::memory_order_release);
    }
    decode_part_k<KT, NT><<<blocks, NTHR, sm, s>>>(a, nslot, mapK, mapV);
    return B200_OK;
}

template <uint32_t KT>
int launch_part_nt(const dec_args & a, unsigned blocks, cudaStream_t s) {
    const int nt = (a.q_len * GQA + 7) / 8;
    return nt == 1 ? launch_part<KT, 1>(a, blocks, s) : nt == 2 ? launch_part<KT, 2>(a, blocks, s) : launch_part<KT, 3>(a, blocks, s);
}

// whole tiles can be fetched through tensor maps: pages of at least 64 rows, 16-byte row strides, strides inside the map's fields
bool cache_tiles(const kv_view & g, int n_ctx) {
    return (!g.pt || g.psh >= 6) && g.rowb % 16 == 0 &&
           (g.pt ? g.pstride < ((unsigned long long) 1 << 40) : (n_ctx >= 1 && g.rowb * (unsigned long long) n_ctx < ((unsigned long long) 1 << 40)));
}
// The tensor-core kernel serves the even split of q8_0 caches that can be tiled, for two to four rows per slot (one row
// per slot and q4_0 are faster on the mma.sync kernel: their tiles cost fewer instructions there); B200ATTN_TC=0 keeps the
// mma.sync kernel everywhere.
int g_tc = -1;   // -1 = not read yet
bool tc_enabled() {
    if (g_tc < 0) { const char * e = getenv("B200ATTN_TC"); g_tc = (e && *e == '0') ? 0 : 1; }
    return g_tc != 0;
}
bool tc_eligible(const b200_kv_cache & c, int q_len) {
    return tc_enabled() && c.type == B200_KV_Q8_0 && q_len >= 2 && cache_tiles(view_of(c), c.n_ctx) && tensor_map_encoder() != nullptr;
}

template <int NC>
int launch_tc(const dec_args & a_in, unsigned blocks, cudaStream_t s) {
    dec_args a = a_in;
    CUtensorMap mapK, mapV;
    memset(&mapK, 0, sizeof mapK);
    memset(&mapV, 0, sizeof mapV);
    if (!make_cache_map(&mapK, a.g.k, a, TC_HB) || !make_cache_map(&mapV, a.g.v, a, TC_HB))
        B200_REFUSE(B200_ERR_CUDA, "attn_decode: the cache's tensor map could not be encoded");
    a.tiled = 1;
    const size_t sm = tc_smem_bytes();
    static std::atomic<bool> attr_done[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(decode_tc_k<NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sm) != cudaSuccess)
            return launch_status("attn_decode (shared memory attribute)");
        attr_done[dev & 63].store(true, std::memory_order_release);
    }
    decode_tc_k<NC><<<blocks, TC_THR, sm, s>>>(a, mapK, mapV);
    return B200_OK;
}
int launch_tc_nc(const dec_args & a, unsigned blocks, cudaStream_t s) {
    return a.q_len <= 2 ? launch_tc<16>(a, blocks, s) : launch_tc<32>(a, blocks, s);
}

int sm_count() {
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

// CTAs of decode_part_k<type, row tiles> that fit an SM at once (the same rule as launch_part)
template <uint32_t KT, int NT> int ctas_fitting() {
    int ctas = ctas_per_sm<KT, NT>();
    while (ctas > 1 && (size_t) ctas * (smem_bytes<KT, NT>(2) + 1024) > (size_t) 227 * 1024) --ctas;
    return ctas;
}
template <uint32_t KT> int ctas_fitting_nt(int nt) { return nt == 1 ? ctas_fitting<KT, 1>() : nt == 2 ? ctas_fitting<KT, 2>() : ctas_fitting<KT, 3>(); }
int resident_ctas(uint32_t type, int q_len) {
    const int nt = (q_len * GQA + 7) / 8;
    const int per_sm = type == B200_KV_F16 ? ctas_fitting_nt<B200_KV_F16>(nt) : type == B200_KV_Q8_0 ? ctas_fitting_nt<B200_KV_Q8_0>(nt)
                                                                                                 : ctas_fitting_nt<B200_KV_Q4_0>(nt);
    return per_sm * sm_count();
}

int auto_chunk(long long total_keys, int Hkv) {
    // enough units for several waves over the SMs, chunks between 256 and 4096 keys
    const long long units = 8LL * sm_count();
    long long ch = total_keys * Hkv / units;
    int c = 256;
    while (c < 4096 && c < ch) c *= 2;
    return c;
}

// geometry of a call: chunk, chunks per slot, partial floats, work-list ints
//   split   (chunk chosen from the batch, up to SPLIT_MAX_SLOTS slots): one contiguous run of tiles per resident CTA
//   planned (fixed chunk, more units than a wave): the grid's units ordered longest first through a work list
//   else    the grid enumerates (slot, chunk)
struct dec_geom { int CH, max_chunks, R, max_cta; size_t units, part_floats, list_ints; bool planned, split, tc; };

bool decode_geometry(dec_geom & g, uint32_t type, int n_slots, int q_len, int max_n, int n_ctx, int Hkv, int chunk_keys, bool tc = false) {
    if (max_n < 1) max_n = 1;
    g.tc = false;
    g.R = q_len * GQA;
    g.split = chunk_keys < 0 && n_slots > 1 && n_slots <= SPLIT_MAX_SLOTS;   // one sequence is even as it is: no plan launch
    g.planned = false;
    g.max_cta = 0;
    if (g.split) {
        g.CH = TILE;
        g.max_chunks = (max_n + TILE - 1) / TILE;
        g.tc = tc && type == B200_KV_Q8_0 && q_len >= 2;   // the tensor-core kernel: one CTA per SM
        g.max_cta = std::max(1, std::min(SPLIT_MAX_CTA, (g.tc ? sm_count() : resident_ctas(type, q_len)) / Hkv));
        const size_t nseg = (size_t) g.max_cta + n_slots;
        g.units = nseg * Hkv;
        g.part_floats = g.units * g.R * (DH + 2);
        g.list_ints = 4 * nseg + 2 * (size_t) n_slots + g.max_cta + 2;
        g.list_ints = (g.list_ints + 3) & ~(size_t) 3;
        return true;
    }
    g.CH = chunk_keys > 0 ? round_tile(chunk_keys) : chunk_keys < 0 ? auto_chunk((long long) n_slots * max_n / 2, Hkv) : fixed_chunk(n_ctx);
    g.max_chunks = (max_n + g.CH - 1) / g.CH;
    g.units = (size_t) n_slots * Hkv * g.max_chunks;
    if (g.units >= ((size_t) 1 << 31) || (size_t) n_slots * g.max_chunks >= ((size_t) 1 << 30)) return false;
    g.part_floats = g.units * g.R * (DH + 2);
    // a work list pays once the launch is longer than one wave of resident CTAs; shorter launches enumerate the grid
    g.planned = n_slots > 1 && g.units > (size_t) 2 * sm_count();
    g.list_ints = g.planned ? 2 * (size_t) n_slots * g.max_chunks + 4 : 0;
    return true;
}

int decode_check(const float * q, const b200_kv_cache * c, const float * out, const float * gate, int n_slots, int q_len, int Hq,
                 const char * who) {
    if (!c || !q || !c->k || !c->v) B200_REFUSE(B200_ERR_SHAPE, "%s: null argument", who);
    if (c->D != DH || Hq != GQA * c->Hkv || c->Hkv <= 0) B200_REFUSE(B200_ERR_SHAPE, "%s: unsupported shape (D=%d Hq=%d Hkv=%d)", who, c->D, Hq, c->Hkv);
    if (c->type != B200_KV_F16 && c->type != B200_KV_Q8_0 && c->type != B200_KV_Q4_0) B200_REFUSE(B200_ERR_SHAPE, "%s: unsupported cache type %u", who, c->type);
    if (n_slots < 1 || n_slots > 65535 || q_len < 1 || q_len > B200_MAX_QLEN) B200_REFUSE(B200_ERR_SHAPE, "%s: unsupported rows (slots=%d q_len=%d)", who, n_slots, q_len);
    if (!aligned16(c->k) || !aligned16(c->v) || !aligned16(q) || (out && !aligned16(out)) || (gate && !aligned16(gate)) ||
        (c->pt && c->pstride % 16))
        B200_REFUSE(B200_ERR_SHAPE, "%s: cache base, page stride, q, out and gate must be 16-byte aligned", who);
    if (c->pt && (c->psh < 0 || c->psh > 30)) B200_REFUSE(B200_ERR_SHAPE, "%s: bad page shift %d", who, c->psh);
    return B200_OK;
}

struct merge_out { float * out; const float * gate; float * fo, * fm, * fl; void * qbuf; };

// the kernels of one call, partials and work list in `scr`
int decode_launch(const float * q, const b200_kv_cache * c, const merge_out & mo, int n_slots, int q_len, const int32_t * pos,
                  const int32_t * p0p, int p0, int Hq, float scale, const dec_geom & gm, float * scr, unsigned * st, cudaStream_t s,
                  const char * who, bool reuse_plan = false) {
    dec_args a;
    a.q = q; a.g = view_of(*c);
    a.po = scr; a.pm = scr + gm.units * gm.R * DH; a.pl = a.pm + gm.units * gm.R;
    a.pos = pos; a.p0p = p0p; a.p0 = p0;
    a.q_len = q_len; a.n_slots = n_slots; a.Hq = Hq;
    a.qscale = scale * LOG2E;
    a.CH = gm.CH; a.max_chunks = gm.max_chunks; a.status = st;
    a.n_ctx = c->n_ctx; a.tiled = 0;
    a.units = nullptr; a.n_units = nullptr;
    a.segs = nullptr; a.cta_seg = nullptr; a.slot_seg = nullptr; a.n_cta = nullptr;
    int launches = 2;
    unsigned blocks = (unsigned) gm.units;
    if (gm.split) {
        int * list = reinterpret_cast<int *>(scr + gm.part_floats);
        const size_t nseg = (size_t) gm.max_cta + n_slots;
        int4 * segs = reinterpret_cast<int4 *>(list);
        int2 * slot_seg = reinterpret_cast<int2 *>(list + 4 * nseg);
        int * cta_seg = list + 4 * nseg + 2 * (size_t) n_slots;
        int * n_cta = cta_seg + gm.max_cta + 1;
        a.segs = segs; a.cta_seg = cta_seg; a.slot_seg = slot_seg; a.n_cta = n_cta;
        if (!reuse_plan) {   // else the lists of an earlier call of this step, same shape, same positions, are still there
            decode_split_k<<<1, SPLIT_THR, 0, s>>>(a, gm.max_cta, segs, cta_seg, slot_seg, n_cta);
            ++launches;
        }
        blocks = (unsigned) gm.max_cta * (unsigned) c->Hkv;
    } else if (gm.planned) {
        int * list = reinterpret_cast<int *>(scr + gm.part_floats);
        a.n_units = list;
        a.units = reinterpret_cast<const int2 *>(list + 4);
        decode_plan_k<<<1, PLAN_THR, 0, s>>>(a, reinterpret_cast<int2 *>(list + 4), list);
        ++launches;
    }
    int rc;
    if (gm.split && gm.tc) rc = launch_tc_nc(a, blocks, s);
    else if (c->type == B200_KV_F16) rc = launch_part_nt<B200_KV_F16>(a, blocks, s);
    else if (c->type == B200_KV_Q8_0) rc = launch_part_nt<B200_KV_Q8_0>(a, blocks, s);
    else rc = launch_part_nt<B200_KV_Q4_0>(a, blocks, s);
    if (rc != B200_OK) return rc;
    if (gm.split) decode_merge_k<1><<<dim3(n_slots * q_len, Hq), 64, 0, s>>>(a, mo.gate, mo.out, mo.fo, mo.fm, mo.fl, (__half2 *) mo.qbuf);
    else decode_merge_k<4><<<dim3(n_slots * q_len, Hq), 256, 0, s>>>(a, mo.gate, mo.out, mo.fo, mo.fm, mo.fl, (__half2 *) mo.qbuf);
    count_launch(launches);
    return launch_status(who);
}

}  // namespace

// q [rows][Hq][256]; rows = n_slots * q_len. Exactly one of (pos), (p0p), (p0) gives the positions.
// hint_floats: size the library scratch for at least this much when it has to be (re)allocated.
int decode_impl(const float * q, const b200_kv_cache * c, const merge_out & mo, int n_slots, int q_len, const int32_t * pos,
                const int32_t * p0p, int p0, int max_n, int Hq, float scale, int chunk_keys, cudaStream_t s, const char * who,
                size_t hint_floats = 0) {
    const int chk = decode_check(q, c, mo.out, mo.gate, n_slots, q_len, Hq, who);
    if (chk != B200_OK) return chk;
    if (mo.qbuf && (!mo.out || ((uintptr_t) mo.qbuf & 3))) B200_REFUSE(B200_ERR_SHAPE, "%s: the a16 buffer needs out and 4-byte alignment", who);
    dec_geom gm;
    if (!decode_geometry(gm, c->type, n_slots, q_len, max_n, c->n_ctx, c->Hkv, chunk_keys, tc_eligible(*c, q_len))) B200_REFUSE(B200_ERR_SHAPE, "%s: too many chunks", who);
    const size_t need = gm.part_floats + gm.list_ints;
    scratch * e = scratch_entry(s, need, hint_floats);
    if (!e || !e->p) B200_REFUSE(B200_ERR_ALLOC, "%s: split scratch (%zu floats) could not be allocated", who, need);
    float * scr = e->p;
    unsigned * st = device_status_word();
    if (!st) return B200_ERR_CUDA;
    plan_key k;
    k.scr = scr; k.pos = pos; k.p0p = p0p; k.p0 = p0; k.n_slots = n_slots; k.q_len = q_len; k.max_chunks = gm.max_chunks;
    k.max_cta = gm.max_cta; k.Hkv = c->Hkv; k.n_ctx = c->n_ctx; k.paged = c->pt != nullptr; k.part_floats = gm.part_floats;
    const bool in_step = e->step_mode && pos && (const char *) pos >= e->step_lo && (const char *) pos < e->step_hi;
    const bool reuse = gm.split && in_step && e->plan_valid && k == e->key;
    const int rc = decode_launch(q, c, mo, n_slots, q_len, pos, p0p, p0, Hq, scale, gm, scr, st, s, who, reuse);
    e->plan_valid = gm.split && in_step && rc == B200_OK;   // any other call on the stream rewrites the scratch
    e->key = k;
    return rc;
}

// ---- decode / verify without any allocation --------------------------------------------------------------------
// Same kernels as decode_impl, but the split partials live in a fixed array inside the library image instead of a
// buffer obtained from cudaMalloc.  Every GPU that loads the library carries the array (NOALLOC_BYTES) until the
// process exits.
constexpr size_t NOALLOC_FLOATS = (size_t) 4 << 20;                 // 16 MiB of partials
constexpr size_t NOALLOC_BYTES = NOALLOC_FLOATS * sizeof(float);
static __device__ __align__(256) float g_noalloc_partials[NOALLOC_FLOATS];
static __device__ __align__(256) unsigned g_noalloc_status[64];
struct noalloc_dev { bool ready = false; float * partials = nullptr; unsigned * status = nullptr; };
noalloc_dev g_noalloc[64];
std::mutex g_noalloc_mu;

// In host code the two array names above are host-side handles, not device addresses: the addresses the kernels need are
// looked up once per device, with that device current.
int noalloc_setup(noalloc_dev & out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return B200_ERR_CUDA; }
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    noalloc_dev & e = g_noalloc[dev & 63];
    if (!e.ready) {
        void * p = nullptr, * st = nullptr;
        cudaError_t rc = cudaGetSymbolAddress(&p, g_noalloc_partials);
        if (rc == cudaSuccess) rc = cudaGetSymbolAddress(&st, g_noalloc_status);
        if (rc != cudaSuccess) {
            cudaGetLastError();
            fprintf(stderr, "b200attn: attn_decode_slots_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(rc));
            return B200_ERR_CUDA;
        }
        e.partials = (float *) p;
        e.status = (unsigned *) st;
        e.ready = true;
    }
    out = e;
    return B200_OK;
}

int decode_noalloc_impl(const float * q, const b200_kv_cache * c, float * out, const float * gate, int n_slots, int q_len,
                        const int32_t * pos, int max_n, int Hq, float scale, int chunk_keys, cudaStream_t s) {
    const char * who = "attn_decode_slots_noalloc";
    if (!out || !pos) B200_REFUSE(B200_ERR_SHAPE, "%s: null argument", who);
    const int chk = decode_check(q, c, out, gate, n_slots, q_len, Hq, who);
    if (chk != B200_OK) return chk;
    dec_geom gm;
    const bool ok = decode_geometry(gm, c->type, n_slots, q_len, max_n, c->n_ctx, c->Hkv, chunk_keys, tc_eligible(*c, q_len));
    const size_t need = ok ? gm.part_floats + gm.list_ints : 0;
    if (!ok || need > NOALLOC_FLOATS)
        B200_REFUSE(B200_ERR_SCRATCH, "%s: %zu bytes of split partials needed (slots %d x kv heads %d x chunks %d x rows %d), the built-in array holds %zu; "
                    "use a larger chunk_keys or attn_decode_slots", who, need * sizeof(float), n_slots, c->Hkv, ok ? gm.max_chunks : -1, q_len * GQA, NOALLOC_BYTES);
    noalloc_dev e;
    const int src = noalloc_setup(e);
    if (src != B200_OK) return src;
    const merge_out mo = {out, gate, nullptr, nullptr, nullptr, nullptr};
    return decode_launch(q, c, mo, n_slots, q_len, pos, nullptr, 0, Hq, scale, gm, e.partials, e.status, s, who);
}

}  // namespace b200

using namespace b200;

extern "C" {

// Batched decode / verify for callers that must not allocate device memory.  See include/b200attn.h.
int b200_attn_decode_slots_noalloc(const float * q, const b200_kv_cache * c, float * out, const float * gate, int n_slots,
                                   int q_len, const int32_t * pos, int max_n, int Hq, float scale, int chunk_keys, void * stream) {
    return decode_noalloc_impl(q, c, out, gate, n_slots, q_len, pos, max_n, Hq, scale, chunk_keys, (cudaStream_t) stream);
}

// Status word of the allocation-free entry point on the current device: synchronises the stream, reads the word with a
// symbol copy and clears it with another (neither allocates).  0 = no kernel of that entry point recorded an error.
int b200_noalloc_device_status(void * stream) {
    if (cudaStreamSynchronize((cudaStream_t) stream) != cudaSuccess) return -1;
    unsigned h = 0;
    if (cudaMemcpyFromSymbol(&h, g_noalloc_status, sizeof h) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (h) {
        const unsigned z = 0;
        if (cudaMemcpyToSymbol(g_noalloc_status, &z, sizeof z) != cudaSuccess) { cudaGetLastError(); return -1; }
    }
    return (int) h;
}

int b200_attn_chunk_keys(void) { return default_chunk(); }
int b200_attn_fixed_chunk(int n_ctx) { return fixed_chunk(n_ctx); }

int b200_attn_dec2_nsplit(int Hkv) {
    (void) Hkv;   // the reference derives its stream count from the SM count and Hkv; here the split follows the context
    return g_nsplit_override > 0 ? g_nsplit_override : MAX_DEFAULT_CHUNKS;
}
void b200_attn_dec2_set_nsplit(int n) { g_nsplit_override = n > 0 ? n : 0; }
int b200_attn_step_begin(void * stream, const int32_t * positions, size_t bytes) {
    if (!positions || !bytes) B200_REFUSE(B200_ERR_SHAPE, "attn_step_begin: null position array");
    scratch * e = scratch_entry((cudaStream_t) stream, 0, 0);
    if (!e) B200_REFUSE(B200_ERR_ALLOC, "attn_step_begin: too many (device, stream) pairs");
    e->step_mode = true;
    e->plan_valid = false;
    e->step_lo = (const char *) positions;
    e->step_hi = e->step_lo + bytes;
    return B200_OK;
}
int b200_attn_step_end(void * stream) {
    scratch * e = scratch_entry((cudaStream_t) stream, 0, 0);
    if (!e) return B200_OK;
    e->step_mode = false;
    e->plan_valid = false;
    e->step_lo = e->step_hi = nullptr;
    return B200_OK;
}
int b200_attn_dec_tc(void) { return tc_enabled() ? 1 : 0; }
void b200_attn_dec_set_tc(int on) { g_tc = on < 0 ? -1 : on ? 1 : 0; }
int b200_attn_dec2_reload_env(void) {
    const int before = default_chunk();
    const bool before_env = g_chunk_from_env;
    g_chunk = env_chunk(&g_chunk_from_env);
    return (g_chunk != before || g_chunk_from_env != before_env) ? 1 : 0;
}

int b200_attn_reserve(uint32_t kv_type, int max_slots, int q_len, int max_n, int n_ctx, int Hkv, int chunk_keys, void * stream) {
    if (max_slots < 1 || max_slots > 65535 || q_len < 1 || q_len > B200_MAX_QLEN || max_n < 1 || Hkv < 1 ||
        (kv_type != B200_KV_F16 && kv_type != B200_KV_Q8_0 && kv_type != B200_KV_Q4_0))
        B200_REFUSE(B200_ERR_SHAPE, "attn_reserve: unsupported arguments");
    dec_geom gm;
    if (!decode_geometry(gm, kv_type, max_slots, q_len, max_n, n_ctx > 0 ? n_ctx : max_n, Hkv, chunk_keys)) B200_REFUSE(B200_ERR_SHAPE, "attn_reserve: too many chunks");
    size_t need = gm.part_floats + std::max(gm.list_ints, 2 * (size_t) max_slots * gm.max_chunks + 4);
    if (chunk_keys < 0 && !gm.split) {
        // a fixed chunk chosen from the batch: smaller batches take smaller chunks; their unit count stays under this bound
        const size_t u = 2 * 8 * (size_t) sm_count() + (size_t) max_slots * Hkv;
        need = std::max(need, u * q_len * GQA * (DH + 2) + 2 * u + 4);
    }
    if (!scratch_for((cudaStream_t) stream, need, 0)) B200_REFUSE(B200_ERR_ALLOC, "attn_reserve: %zu floats could not be allocated", need);
    return B200_OK;
}

int b200_attn_decode2(const float * q, const b200_kv_cache * c, float * out, int T, int p0, const int32_t * p0_dev, int Hq,
                      float scale, void * stream, const int32_t * pos_rows) {
    if (T < 1 || T > B200_ATTN_MAX_ROWS) B200_REFUSE(B200_ERR_SHAPE, "attn_decode: unsupported row count %d", T);
    if (!out) B200_REFUSE(B200_ERR_SHAPE, "attn_decode: out is null");
    const int n_ctx = c ? std::max(c->n_ctx, 1) : 1;
    // the grid covers the rows' keys when the host knows them, else the cache's capacity
    const int max_n = (!p0_dev && !pos_rows && p0 >= 0) ? std::min(std::max(p0 + T, 1), c && !c->pt ? n_ctx : 0x7fffffff) : n_ctx;
    // the first call per (device, stream) sizes the scratch for the largest call these entry points accept on this cache
    // (B200_ATTN_MAX_ROWS rows over n_ctx keys), as the reference does (src/fast/attn_dec2.cu:503-517)
    size_t hint = 0;
    if (c && c->Hkv > 0) {
        dec_geom gm;
        if (decode_geometry(gm, c->type, B200_ATTN_MAX_ROWS, 1, n_ctx, n_ctx, c->Hkv, 0)) hint = gm.part_floats + gm.list_ints;
    }
    const merge_out mo = {out, nullptr, nullptr, nullptr, nullptr, nullptr};
    // rows of one sequence at consecutive positions share the pass over its KV (up to 4 rows per slot)
    if (!pos_rows && T <= B200_MAX_QLEN)
        return decode_impl(q, c, mo, 1, T, nullptr, p0_dev, p0, max_n, Hq, scale, 0, (cudaStream_t) stream, "attn_decode", hint);
    return decode_impl(q, c, mo, T, 1, pos_rows, p0_dev, p0, max_n, Hq, scale, 0, (cudaStream_t) stream, "attn_decode", hint);
}

int b200_attn_decode(const float * q, const b200_kv_cache * c, float * out, int T, int p0, int Hq, float scale, void * stream) {
    if (c && !c->pt && (p0 < 0 || p0 + T > c->n_ctx)) B200_REFUSE(B200_ERR_SHAPE, "attn_decode: rows %d..%d outside n_ctx %d", p0, p0 + T - 1, c->n_ctx);
    return b200_attn_decode2(q, c, out, T, p0, nullptr, Hq, scale, stream, nullptr);
}
int b200_attn_decode_dev(const float * q, const b200_kv_cache * c, float * out, int T, const int32_t * p0_dev, int max_n, int Hq,
                         float scale, void * stream) {
    if (!p0_dev) B200_REFUSE(B200_ERR_SHAPE, "attn_decode_dev: p0_dev is null");
    if (T < 1 || T > B200_ATTN_MAX_ROWS) B200_REFUSE(B200_ERR_SHAPE, "attn_decode: unsupported row count %d", T);
    if (!out) B200_REFUSE(B200_ERR_SHAPE, "attn_decode_dev: out is null");
    const int n_ctx = c ? std::max(c->n_ctx, 1) : 1;
    if (max_n < 1 || (c && !c->pt && max_n > n_ctx)) max_n = n_ctx;   // the caller's bound on *p0_dev + T sizes the grid
    size_t hint = 0;
    if (c && c->Hkv > 0) {
        dec_geom gm;
        if (decode_geometry(gm, c->type, B200_ATTN_MAX_ROWS, 1, n_ctx, n_ctx, c->Hkv, 0)) hint = gm.part_floats + gm.list_ints;
    }
    const merge_out mo = {out, nullptr, nullptr, nullptr, nullptr, nullptr};
    if (T <= B200_MAX_QLEN)
        return decode_impl(q, c, mo, 1, T, nullptr, p0_dev, 0, max_n, Hq, scale, 0, (cudaStream_t) stream, "attn_decode_dev", hint);
    return decode_impl(q, c, mo, T, 1, nullptr, p0_dev, 0, max_n, Hq, scale, 0, (cudaStream_t) stream, "attn_decode_dev", hint);
}
int b200_attn_decode_rows(const float * q, const b200_kv_cache * c, float * out, int T, const int32_t * pos, int Hq, float scale,
                          void * stream) {
    if (!pos) B200_REFUSE(B200_ERR_SHAPE, "attn_decode_rows: pos is null");
    return b200_attn_decode2(q, c, out, T, 0, nullptr, Hq, scale, stream, pos);
}

int b200_attn_decode_slots(const float * q, const b200_kv_cache * c, float * out, const float * gate, int n_slots, int q_len,
                           const int32_t * pos, int max_n, int Hq, float scale, int chunk_keys, void * stream) {
    if (!pos || !out) B200_REFUSE(B200_ERR_SHAPE, "attn_decode_slots: pos / out is null");
    const merge_out mo = {out, gate, nullptr, nullptr, nullptr, nullptr};
    return decode_impl(q, c, mo, n_slots, q_len, pos, nullptr, 0, max_n, Hq, scale, chunk_keys, (cudaStream_t) stream, "attn_decode_slots");
}

int b200_attn_decode_slots_a16(const float * q, const b200_kv_cache * c, float * out, const float * gate, void * qbuf, int n_slots,
                               int q_len, const int32_t * pos, int max_n, int Hq, float scale, int chunk_keys, void * stream) {
    if (!pos || !out || !qbuf) B200_REFUSE(B200_ERR_SHAPE, "attn_decode_slots_a16: pos / out / qbuf is null");
    const merge_out mo = {out, gate, nullptr, nullptr, nullptr, qbuf};
    return decode_impl(q, c, mo, n_slots, q_len, pos, nullptr, 0, max_n, Hq, scale, chunk_keys, (cudaStream_t) stream, "attn_decode_slots_a16");
}

int b200_attn_decode_slots_partial(const float * q, const b200_kv_cache * c, float * part_o, float * part_m, float * part_l,
                                   int n_slots, int q_len, const int32_t * pos, int max_n, int Hq, float scale, int chunk_keys,
                                   void * stream) {
    if (!pos || !part_o || !part_m || !part_l) B200_REFUSE(B200_ERR_SHAPE, "attn_decode_slots_partial: null argument");
    if (!aligned16(part_o)) B200_REFUSE(B200_ERR_SHAPE, "attn_decode_slots_partial: part_o must be 16-byte aligned");
    const merge_out mo = {nullptr, nullptr, part_o, part_m, part_l, nullptr};
    return decode_impl(q, c, mo, n_slots, q_len, pos, nullptr, 0, max_n, Hq, scale, chunk_keys, (cudaStream_t) stream,
                       "attn_decode_slots_partial");
}

int b200_attn_merge_gate(const float * part_o, const float * part_m, const float * part_l, int nparts, int R, int D,
                         const float * gate, float * out, void * stream) {
    if (!part_o || !part_m || !part_l || !out || nparts < 1 || R < 1 || D % 4 || D < 4 || D > 4096 || !aligned16(part_o) ||
        !aligned16(out) || (gate && !aligned16(gate)))
        B200_REFUSE(B200_ERR_SHAPE, "attn_merge_gate: unsupported arguments");
    merge_parts_k<<<R, D / 4, 0, (cudaStream_t) stream>>>(part_o, part_m, part_l, nparts, R, D, gate, out, (size_t) R * D, (size_t) R,
                                                          nullptr);
    count_launch();
    return launch_status("attn_merge_gate");
}

// shared by the two exchange entries: optional all-gather over the caller's communicator, then the merge
static int seq_exchange_impl(void * nccl_comm, int n_seq, const float * send, float * recv, int R, int D, const float * gate,
                             float * out, void * qbuf, void * stream, const char * who) {
    using allgather_fn = int (*)(const void *, void *, size_t, int, void *, cudaStream_t);
    static allgather_fn allgather = [] {
        void * f = dlsym(RTLD_DEFAULT, "ncclAllGather");
        if (!f) {
            void * h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
            if (h) f = dlsym(h, "ncclAllGather");
        }
        return (allgather_fn) f;
    }();
    const size_t part = (size_t) R * (D + 2);
    if (!send || !recv || !out || n_seq < 1 || R < 1 || D % 4 || D < 4 || D > 4096 || part % 4 || !aligned16(send) || !aligned16(recv) ||
        !aligned16(out) || (gate && !aligned16(gate)))
        B200_REFUSE(B200_ERR_SHAPE, "%s: unsupported arguments (R * (D + 2) must be a multiple of 4, buffers 16-byte aligned)", who);
    if (qbuf && (D % 128 || ((uintptr_t) qbuf & 3)))
        B200_REFUSE(B200_ERR_SHAPE, "%s: the a16 buffer needs D %% 128 == 0 and 4-byte alignment", who);
    cudaStream_t s = (cudaStream_t) stream;
    const float * parts = n_seq > 1 ? recv : send;
    if (n_seq > 1 && nccl_comm) {   // without a communicator the caller has gathered the parts into recv already
        if (!allgather) B200_REFUSE(B200_ERR_CUDA, "%s: no NCCL library is loaded in this process", who);
        const int rc = allgather(send, recv, part, 7 /* ncclFloat32 */, nccl_comm, s);
        if (rc != 0) B200_REFUSE(B200_ERR_CUDA, "%s: ncclAllGather returned %d", who, rc);
    }
    merge_parts_k<<<R, D / 4, 0, s>>>(parts, parts + (size_t) R * D, parts + (size_t) R * D + R, n_seq, R, D, gate, out, part, part,
                                      (__half2 *) qbuf);
    count_launch();
    return launch_status(who);
}

// The exchange step of the sequence split for a host that drives NCCL itself.  ncclAllGather is taken from the NCCL library
// the process has already loaded (the host's own, or the one bundled with its framework), so the communicator and the
// function come from the same library; nothing here links NCCL.
int b200_seq_exchange_merge(void * nccl_comm, int n_seq, const float * send, float * recv, int R, int D, const float * gate,
                            float * out, void * stream) {
    return seq_exchange_impl(nccl_comm, n_seq, send, recv, R, D, gate, out, nullptr, stream, "seq_exchange_merge");
}
int b200_seq_exchange_merge_a16(void * nccl_comm, int n_seq, const float * send, float * recv, int R, int D, const float * gate,
                                float * out, void * qbuf, void * stream) {
    if (!qbuf) B200_REFUSE(B200_ERR_SHAPE, "seq_exchange_merge_a16: qbuf is null");
    return seq_exchange_impl(nccl_comm, n_seq, send, recv, R, D, gate, out, qbuf, stream, "seq_exchange_merge_a16");
}

// ---- sequence split over peer-mapped buffers ------------------------------------------------------------------
// A buffer other processes of the node can map (cudaMalloc + cudaIpcGetMemHandle): the host passes the 64-byte handle to the
// peers by whatever means it has, they map it with b200_peer_open.  Zero-filled.
int b200_peer_alloc(size_t bytes, void ** ptr, unsigned char * handle) {
    if (!ptr || !handle || !bytes) B200_REFUSE(B200_ERR_SHAPE, "peer_alloc: null argument");
    void * p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); B200_REFUSE(B200_ERR_ALLOC, "peer_alloc: cudaMalloc(%zu) failed", bytes); }
    cudaIpcMemHandle_t h;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess || cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        const cudaError_t e = cudaGetLastError();
        cudaFree(p);
        B200_REFUSE(B200_ERR_CUDA, "peer_alloc: %s", cudaGetErrorString(e));
    }
    static_assert(sizeof h == 64, "handle size");
    memcpy(handle, &h, 64);
    *ptr = p;
    return B200_OK;
}
int b200_peer_open(const unsigned char * handle, void ** ptr) {
    if (!ptr || !handle) B200_REFUSE(B200_ERR_SHAPE, "peer_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void * p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { cudaGetLastError(); B200_REFUSE(B200_ERR_CUDA, "peer_open: %s", cudaGetErrorString(e)); }
    *ptr = p;
    return B200_OK;
}
int b200_peer_close(void * ptr) { return ptr && cudaIpcCloseMemHandle(ptr) != cudaSuccess ? (cudaGetLastError(), B200_ERR_CUDA) : B200_OK; }
int b200_peer_free(void * ptr) { return ptr && cudaFree(ptr) != cudaSuccess ? (cudaGetLastError(), B200_ERR_CUDA) : B200_OK; }

static int seq_merge_peers_impl(const void * const * parts, void * const * flags, int n_seq, int me, unsigned epoch, int R, int D,
                                const float * gate, float * out, void * qbuf, void * stream, const char * who) {
    if (!parts || !flags || !out || n_seq < 1 || n_seq > MAX_PEERS || me < 0 || me >= n_seq || R < 1 || D % 4 || D < 4 * MAX_PEERS || D > 4096 ||
        !aligned16(out) || (gate && !aligned16(gate)))
        B200_REFUSE(B200_ERR_SHAPE, "%s: unsupported arguments", who);
    if (qbuf && (D % 128 || ((uintptr_t) qbuf & 3))) B200_REFUSE(B200_ERR_SHAPE, "%s: the a16 buffer needs D %% 128 == 0 and 4-byte alignment", who);
    peer_parts pp;
    for (int s = 0; s < MAX_PEERS; ++s) {
        pp.part[s] = s < n_seq ? (const float *) parts[s] : nullptr;
        pp.flag[s] = s < n_seq ? (unsigned *) flags[s] : nullptr;
        if (s < n_seq && (!pp.part[s] || !pp.flag[s] || !aligned16(pp.part[s]) || ((uintptr_t) pp.flag[s] & 3)))
            B200_REFUSE(B200_ERR_SHAPE, "%s: shard %d: buffers must be mapped and 16-byte aligned", who, s);
    }
    unsigned * st = device_status_word();
    if (!st) return B200_ERR_CUDA;
    merge_peers_k<<<R, D / 4, 0, (cudaStream_t) stream>>>(pp, n_seq, me, epoch, R, D, gate, out, (__half2 *) qbuf, st);
    count_launch();
    return launch_status(who);
}
int b200_seq_merge_peers(const void * const * parts, void * const * flags, int n_seq, int me, unsigned epoch, int R, int D,
                         const float * gate, float * out, void * stream) {
    return seq_merge_peers_impl(parts, flags, n_seq, me, epoch, R, D, gate, out, nullptr, stream, "seq_merge_peers");
}
int b200_seq_merge_peers_a16(const void * const * parts, void * const * flags, int n_seq, int me, unsigned epoch, int R, int D,
                             const float * gate, float * out, void * qbuf, void * stream) {
    if (!qbuf) B200_REFUSE(B200_ERR_SHAPE, "seq_merge_peers_a16: qbuf is null");
    return seq_merge_peers_impl(parts, flags, n_seq, me, epoch, R, D, gate, out, qbuf, stream, "seq_merge_peers_a16");
}

}  // extern "C"
