/*
 * b200attn — C ABI of the B200 (sm_100a) paged-KV full-attention library.
 *
 * Drop-in for the attention entry points of the reference engine's kernel library (namespace p100e::fast):
 * every function below names the reference declaration it replaces (paths relative to the reference project).
 * Same argument meaning, same cache layouts, same error convention: a call either enqueues its kernels on the given
 * stream and returns B200_OK, or launches nothing and returns a non-zero status after printing one line to stderr
 * (the reference returns bool false, src/fast/attn.cuh:40-43).  Nothing throws, nothing synchronises the stream.
 *
 * All pointers are device pointers unless marked "host".  `stream` is a cudaStream_t passed as void*.
 * Shapes: D == 256 and Hq == 6 * Hkv for the attention kernels (the reference's limits, src/fast/attn_dec2.cu:493).
 * There is no CPU fallback: without a CUDA device every launch entry point returns B200_ERR_CUDA.
 */
#ifndef B200ATTN_H
#define B200ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* KV storage types == ggml type ids (src/fast/attn.cuh:14-16). */
#define B200_KV_F16 1u
#define B200_KV_Q4_0 2u
#define B200_KV_Q8_0 8u
/* rows per call of the reference-compatible row entry points (src/fast/attn.cuh:66) */
#define B200_ATTN_MAX_ROWS 8
/* query rows per slot of the batched entry points (1 real token + 3 drafted ones) */
#define B200_MAX_QLEN 4

enum {
    B200_OK = 0,
    B200_ERR_SHAPE = 1,   /* unsupported shape / type / alignment: nothing launched */
    B200_ERR_ALLOC = 2,   /* library-owned scratch could not be allocated */
    B200_ERR_CUDA = 3,    /* no device, or a launch was rejected by the runtime */
    B200_ERR_SCRATCH = 4, /* caller-provided scratch too small */
    B200_ERR_DEVICE = 5,  /* a kernel recorded an error in the status word (see b200_last_device_status) */
    B200_ERR_FORMAT = 6,  /* a sequence file is not what it should be (magic, fingerprint, header, short file) */
    B200_ERR_IO = 7       /* a read or write on a file descriptor failed */
};

/* One layer's K and V as the kernels see them: field for field the reference's view (src/fast/attn.cuh:18-32).
 * Position p of query row t lives at  k + pt[(rtab ? rtab[t] : 0) + (p >> psh)] * pstride + (p & (2^psh-1)) * rowb
 * with rowb = b200_kv_row_bytes(type, Hkv, D); pt == NULL means contiguous [n_ctx][rowb] (src/fast/kv_page.cuh:20-31).
 * Head row formats (src/fast/attn.cuh:3-7, src/fast/kv_q8.cuh:1-5):
 *   f16   256 halves (512 B)
 *   q8_0  8 f16 block scales, then 256 int8 (272 B); value = q * d
 *   q4_0  8 x {f16 d, 16 bytes}, byte i = value i | value i+16 << 4 (144 B); value = (nibble - 8) * d
 * Offsets may exceed 4 GiB: all addressing is 64-bit (the reference is limited to 32-bit offsets per region). */
typedef struct b200_kv_cache {
    uint32_t type;
    int32_t n_ctx, Hkv, D;
    void *k;
    void *v;
    const int32_t *pt;
    const int32_t *rtab;
    int32_t psh;
    size_t pstride;
} b200_kv_cache;

/* Interleaved M-RoPE positions (src/fast/mrope.cuh:16-21); p == NULL selects plain NEOX. */
typedef struct b200_mrope_pos {
    const int32_t *p; /* device [3][stride]: t, h, w streams */
    int32_t stride;
    int32_t s0, s1, s2;
    int32_t sect;
} b200_mrope_pos;

/* ---------------------------------------------------------------- cache helpers (src/fast/attn.cuh:34-36) ---- */
size_t b200_kv_row_bytes(uint32_t type, int Hkv, int D);                       /* kv_row_bytes, attn.cu:501 */
int b200_kv_alloc(b200_kv_cache *out, uint32_t type, int n_ctx, int Hkv, int D); /* kv_alloc, attn.cu:505 (contiguous) */
void b200_kv_free(b200_kv_cache *c);                                           /* kv_free, attn.cu:517 */
/* kv_fill_random (attn.cuh:68-70, attn.cu:559-581): finite pseudo-random rows at positions p0..p1-1 (benchmarks) */
int b200_kv_fill_random(const b200_kv_cache *c, int p0, int p1, uint32_t seed, void *stream);
/* Benchmark filler for a paged pool (new): slot s owns len[s] (device) local positions through the table row
 * pt + s * table_stride.  The bytes depend on (seed, slot, global position, global kv head) only, so differently sharded
 * pools hold the same values: head0 = global index of this cache's head 0; with the pages of a sequence dealt
 * round-robin over n_seq sequence shards, local page j of shard seq_rank is global page j * n_seq + seq_rank. */
int b200_kv_fill_slots(const b200_kv_cache *c, int n_slots, const int32_t *len, int table_stride, uint32_t seed,
                       int head0, int n_seq, int seq_rank, void *stream);

/* ---------------------------------------------------------------- KV append ---------------------------------- */
/* kv_append (attn.cuh:36, attn.cu:583): k, v [T][Hkv][D] f32 -> positions p0..p0+T-1, converted / quantised.
 * Bytes written are identical to the reference quantiser's for the same inputs. */
int b200_kv_append(const b200_kv_cache *c, const float *k, const float *v, int p0, int T, void *stream);
/* kv_append_dev (attn.cuh:58, attn.cu:587): first position read from *p0_dev when the kernel runs */
int b200_kv_append_dev(const b200_kv_cache *c, const float *k, const float *v, const int32_t *p0_dev, int T, void *stream);
/* attn_prep (src/fast/fused.cuh:101-113, fused.cu:677-721): per token split q|gate, RMSNorm(q)*q_norm,
 * RMSNorm(k)*k_norm, partial NEOX RoPE on the first n_rot dims (angle from pos[t]), K and V quantised straight into
 * cache row p0+t (p0 >= 0) or pos[t] (p0 < 0).  ldq/ldk/ldv: row strides in floats (0 = dense).  mr may be NULL.
 * qg == NULL (then q and gate may be NULL too): only K and V are produced and stored, with the same bytes: the KV-only
 * catch-up of the MTP draft head (the reference runs norm + rope + kv_append for it, src/tp_model.cu:1705-1730). */
int b200_attn_prep(const float *qg, const float *k, const float *v, const float *q_norm, const float *k_norm,
                   const int32_t *pos, float *q, float *gate, const b200_kv_cache *c, int p0, int T, int Hq, int Hkv,
                   int D, int n_rot, float freq_base, float eps, void *stream, int ldq, int ldk, int ldv,
                   const b200_mrope_pos *mr);
/* attn_prep with the rotary position and the cache row given separately (new; needed when a sequence's pages are split
 * over two GPUs: the rotary angle uses the global position rope_pos[t], the row lands at cache_row[t] of this GPU's
 * compacted sequence, and cache_row[t] < 0 means another GPU owns the row: q and gate are produced, K/V are not stored).
 * Same arithmetic and bytes as b200_attn_prep. */
int b200_attn_prep_rows(const float *qg, const float *k, const float *v, const float *q_norm, const float *k_norm,
                        const int32_t *rope_pos, const int32_t *cache_row, float *q, float *gate, const b200_kv_cache *c,
                        int T, int Hq, int Hkv, int D, int n_rot, float freq_base, float eps, void *stream);
/* Prefill form of the append for bf16 activations: k, v [T][Hkv][D] bf16 (raw bits), partial NEOX RoPE applied to K
 * (no norm), quantised into rows p0+t; q [T][Hq][D] bf16 is roped in fp32 and written to q_out [T][Hq][D] f32.
 * No counterpart with bf16 inputs in the reference (its prefill runs k::rope_neox + kv_append on f32,
 * src/tp_model.cu:2899-2908); the arithmetic after widening to f32 is the same. q / q_out may be NULL. */
int b200_rope_append_bf16(const uint16_t *q, const uint16_t *k, const uint16_t *v, float *q_out,
                          const b200_kv_cache *c, int p0, int T, int Hq, int Hkv, int D, int n_rot, float freq_base,
                          void *stream);

/* The same with the cache row and the rotary position given separately (a sequence shard stores token t at its local row
 * row0 + t while the angle comes from the global position rope0 + t); k == v == NULL: only q is rotated. */
int b200_rope_append_bf16_at(const uint16_t *q, const uint16_t *k, const uint16_t *v, float *q_out,
                             const b200_kv_cache *c, int row0, int rope0, int T, int Hq, int Hkv, int D, int n_rot,
                             float freq_base, void *stream);

/* ---------------------------------------------------------------- decode / MTP verify ------------------------ */
/* attn_decode (attn.cuh:44, attn.cu:638): q, out [T][Hq][D] f32, row t at position p0+t sees keys 0..p0+t. T <= 8. */
int b200_attn_decode(const float *q, const b200_kv_cache *c, float *out, int T, int p0, int Hq, float scale, void *stream);
/* attn_decode_dev (attn.cuh:59, attn.cu:654): p0 read from *p0_dev on the device; grid sized for p0+T <= max_n
 * (max_n <= 0: the cache's n_ctx).  A position beyond max_n is reported through the status word (value 8) and the keys
 * past the limit are left out; nothing is read out of bounds. */
int b200_attn_decode_dev(const float *q, const b200_kv_cache *c, float *out, int T, const int32_t *p0_dev, int max_n,
                         int Hq, float scale, void *stream);
/* attn_decode_rows (attn.cuh:64-66, attn.cu:649): row t at pos[t] (device) of its own sequence (pt + rtab[t]) */
int b200_attn_decode_rows(const float *q, const b200_kv_cache *c, float *out, int T, const int32_t *pos, int Hq,
                          float scale, void *stream);
/* attn_decode2 (src/fast/attn_dec2.cuh:17-18): the dispatcher behind the three calls above */
int b200_attn_decode2(const float *q, const b200_kv_cache *c, float *out, int T, int p0, const int32_t *p0_dev, int Hq,
                      float scale, void *stream, const int32_t *pos_rows);
/* attn_dec2_nsplit / attn_dec2_set_nsplit / attn_dec2_reload_env (attn_dec2.cuh:19-21).  The reference splits the keys
 * into a fixed number of interleaved streams; this library splits them into consecutive chunks whose length depends on
 * the cache's capacity only: b200_attn_fixed_chunk(n_ctx) = max(b200_attn_chunk_keys(), n_ctx / 256 rounded up to 64), so
 * a full context has at most 256 chunks.  set_nsplit(n > 0) pins n chunks per full context instead (chunk = n_ctx / n
 * rounded up to 64; 0 restores the default), nsplit reports that number (256 by default), reload_env re-reads
 * B200ATTN_CHUNK (a fixed chunk in keys, for every n_ctx) and returns 1 if the setting changed. */
int b200_attn_dec2_nsplit(int Hkv);
void b200_attn_dec2_set_nsplit(int n);
int b200_attn_dec2_reload_env(void);
int b200_attn_chunk_keys(void);        /* the smallest default chunk (keys): B200ATTN_CHUNK or 512 */
int b200_attn_fixed_chunk(int n_ctx);  /* the chunk the entry points above use for a cache of n_ctx positions */
/* Kernel choice of the batched entry points with chunk_keys = -1 (even split of the batch): q8_0 caches whose tiles can be
 * fetched through tensor maps (pages of at least 64 positions), with two to four rows per slot, run on the tcgen05 kernel
 * (one CTA per SM, K widened into tensor memory, V into an f16 image in shared memory); everything else on the mma.sync
 * kernel.  set_tc(0) keeps the mma.sync kernel everywhere, set_tc(1) restores the default, set_tc(-1) re-reads
 * B200ATTN_TC (0 = off); tc() reports the setting.  Both kernels meet the same tolerance; their results are not bitwise
 * equal. */
/* A model step does not change the rows' positions from layer to layer, and the even split of a batch (chunk_keys = -1)
 * depends on nothing else.  b200_attn_step_begin(stream, positions, bytes) declares that the device array `positions`
 * (`bytes` long) stays as it is until the next step_begin / step_end on that stream.  Until then the batched entry points
 * called on the stream with a `pos` argument inside that array reuse the split that the first call of a given shape (position
 * pointer, slots, q_len, max_n, cache geometry) left in the stream's scratch instead of recomputing it per call; any call
 * of another shape on the stream drops it.  Without step_begin every call computes its own split.  b200_pool_step
 * declares its step descriptor this way on its stream, b200_pool_destroy ends the step. */
int b200_attn_step_begin(void *stream, const int32_t *positions, size_t bytes);
int b200_attn_step_end(void *stream);
int b200_attn_dec_tc(void);
void b200_attn_dec_set_tc(int on);

/* Library-owned scratch of the decode entry points (split partials and the work list), one buffer per (device, stream)
 * like the reference's (attn_dec2.cu:452-464,503-517).  The reference-compatible entry points size it on their first call
 * for the largest call they accept on that cache (B200_ATTN_MAX_ROWS rows over n_ctx keys); for the batched entry points
 * call b200_attn_reserve once with the largest batch (n_ctx = the caches' capacity; it only matters for chunk_keys == 0).
 * Afterwards calls that fit allocate nothing, synchronise nothing, and the buffer does not move, so recorded work stays
 * valid.  A call that needs more than was reserved gets a new, larger buffer (cudaMalloc, no synchronisation); the old one
 * stays allocated until the process exits, so earlier recorded work never reads freed memory.  Two calls on the same
 * (device, stream) are stream-ordered and may share the buffer; calls on different streams use different buffers. */
int b200_attn_reserve(uint32_t kv_type, int max_slots, int q_len, int max_n, int n_ctx, int Hkv, int chunk_keys,
                      void *stream);

/* Batched decode / verify, any number of slots (new; the reference stops at 8 rows per call, attn.cuh:66).
 * n_slots sequences, q_len (1..4) query rows each; row r = slot * q_len + j sits at pos[r] (device) and sees keys
 * 0..pos[r] of its slot (pos[r] < 0: the row sees nothing and its output is zero); the slot's page table is
 * pt + rtab[slot * q_len] (rtab == NULL: one table for all).  The q_len rows of a slot share one pass over its KV.
 * gate != NULL: out = attn * sigmoid(gate) fused into the split merge (ew_quant(EW_SIGMOID_MUL), fused.cu:479-496;
 * k::sigmoid_mul, src/kernels.cu:85-93).  max_n: upper bound of pos[r] + 1 over the call (sizes the grid).
 * chunk_keys: keys per split (multiple of 64); 0 = the library default (a function of the cache's capacity); -1 = an even
 * split of the whole batch: the batch's 64-key tiles, slot after slot, are cut into one contiguous run per resident CTA, so
 * ragged contexts load every SM equally (up to 2048 slots; larger batches take a chunk chosen from the batch size).
 * With chunk_keys >= 0 each row's result depends only on its own keys and on the chunk, never on the other rows of the call
 * (bitwise); with -1 the split points depend on the batch, so results of different batches agree to rounding only. */
int b200_attn_decode_slots(const float *q, const b200_kv_cache *c, float *out, const float *gate, int n_slots,
                           int q_len, const int32_t *pos, int max_n, int Hq, float scale, int chunk_keys, void *stream);
/* b200_attn_decode_slots for callers that cannot allocate device memory (no counterpart in the reference, whose decode
 * path always owns a cudaMalloc'ed scratch, src/fast/attn_dec2.cu:503-517).  Some hosts of this library run where
 * cudaMalloc is off the table: inside a memory pool that already owns the whole GPU, or in a real-time loop that forbids
 * allocator calls after start-up.  This entry point calls no cudaMalloc, cudaFree or
 * other allocating routine, ever: the split partials go to a fixed 16 MiB array that is part of the library image on
 * every GPU that loads it.  Arguments, results and bits are those of b200_attn_decode_slots.
 *   - Limit: n_slots * Hkv * ceil(max_n / chunk) * 6 * q_len * 258 floats must fit in 16 MiB; beyond that the call returns
 *     B200_ERR_SCRATCH with nothing launched (raise chunk_keys, or use b200_attn_decode_slots).
 *   - The first call on each device looks up the array's device address (with that device current); make that first call
 *     before any stream capture begins.
 *   - All calls on a device share the one array, which keeps the previous call's partials: nothing in it needs clearing
 *     (each call writes every partial it later reads), but two calls that overlap on the GPU (for instance on
 *     different streams) race on it.  Serialise them.
 *   - A kernel-side status (bad page id, timed-out wait, position beyond max_n) of this entry point is kept in a word of
 *     its own inside the library image; b200_noalloc_device_status reads and clears it (it allocates nothing either). */
int b200_attn_decode_slots_noalloc(const float *q, const b200_kv_cache *c, float *out, const float *gate, int n_slots,
                                   int q_len, const int32_t *pos, int max_n, int Hq, float scale, int chunk_keys,
                                   void *stream);
int b200_noalloc_device_status(void *stream);
/* b200_attn_decode_slots that also writes the gated output in the a16 activation format the engine's next projection
 * reads (src/fast/a16q.cuh:4-10; the reference fuses the same quantiser into its gate kernel, ew_quant with qbuf,
 * fused.cu:479-496,657-675, consumer matvec_prequantized src/tp_model.cu:1394-1398): qbuf holds, for the rows x Hq*D
 * output, [rows * Hq*D/32][16] half2 scaled values followed by [rows * Hq*D/32] half2 (amax, sum) pairs, byte-identical
 * to ew_quant(EW_SIGMOID_MUL, ..., qbuf) applied to the same attention output. */
int b200_attn_decode_slots_a16(const float *q, const b200_kv_cache *c, float *out, const float *gate, void *qbuf,
                               int n_slots, int q_len, const int32_t *pos, int max_n, int Hq, float scale, int chunk_keys,
                               void *stream);
/* Same pass, but the merged result is left unnormalised for a cross-GPU sequence split:
 * part_o [rows][Hq][D] = sum exp(s - m) v, part_m / part_l [rows][Hq] the running max (natural-log units, -inf if
 * the row saw no key) and the sum.  The formula of the reference's split partials (attn_dec2.cu:404-424). */
int b200_attn_decode_slots_partial(const float *q, const b200_kv_cache *c, float *part_o, float *part_m, float *part_l,
                                   int n_slots, int q_len, const int32_t *pos, int max_n, int Hq, float scale,
                                   int chunk_keys, void *stream);
/* Merge nparts partial results in part order (dec2_combine_k, attn_dec2.cu:430-450), optional sigmoid gate:
 * part_o [nparts][R][D], part_m / part_l [nparts][R], gate / out [R][D]. */
int b200_attn_merge_gate(const float *part_o, const float *part_m, const float *part_l, int nparts, int R, int D,
                         const float *gate, float *out, void *stream);
/* The exchange + merge step of the sequence split for a host that drives NCCL itself.  The reference has no sequence split
 * and no NCCL (its tensor-parallel ranks exchange through its own transports), so this entry has no reference twin.
 * send = this shard's partial as one flat buffer [O (R*D) | m (R) | l (R)] (the three outputs of
 * b200_attn_decode_slots_partial placed back to back), recv = n_seq such buffers.  ncclAllGather over `nccl_comm`
 * (an ncclComm_t of the n_seq shards, rank order = shard order) on `stream`, then the merge of b200_attn_merge_gate.
 * n_seq == 1 merges `send` alone; nccl_comm == NULL with n_seq > 1 means the caller has already gathered the n_seq
 * buffers into recv (some other transport) and only the merge runs.  NCCL is not linked: the symbol is taken from the
 * NCCL library already loaded.  The _a16 form also writes the a16 copy of the gated output (D % 128 == 0). */
int b200_seq_exchange_merge(void *nccl_comm, int n_seq, const float *send, float *recv, int R, int D, const float *gate,
                            float *out, void *stream);
int b200_seq_exchange_merge_a16(void *nccl_comm, int n_seq, const float *send, float *recv, int R, int D,
                                const float *gate, float *out, void *qbuf, void *stream);

/* The same step without a collective: every shard keeps its partial in a buffer that the other shards of its group have
 * mapped (one process per GPU on one node: b200_peer_alloc gives the buffer and a 64-byte handle, b200_peer_open maps a
 * peer's handle; cudaMalloc / cudaIpcGetMemHandle / cudaIpcOpenMemHandle underneath).  parts[s], flags[s] (host arrays of
 * n_seq <= 8 device addresses, in shard order): shard s's partial [O (R*D) | m (R) | l (R)] and its row of n_seq flag
 * words, as seen from this process (own buffer for s == me).  One kernel announces "my partial of call `epoch` is complete"
 * in every peer's flag row, waits (bounded: 2 s, then the status word gets code 1) for the peers' announcements, and merges
 * in shard order reading the peers' rows over NVLink.  epoch = 1, 2, 3, .. in step on all shards of the group; the caller
 * alternates two partial buffers by the parity of the epoch (a shard rewrites a buffer two calls after it was merged, when
 * every peer has moved past it), and the flag rows start zeroed.  Results equal b200_seq_exchange_merge bit for bit. */
int b200_peer_alloc(size_t bytes, void **ptr, unsigned char *handle64);
int b200_peer_open(const unsigned char *handle64, void **ptr);
int b200_peer_close(void *ptr);
int b200_peer_free(void *ptr);
int b200_seq_merge_peers(const void *const *parts, void *const *flags, int n_seq, int me, unsigned epoch, int R, int D,
                         const float *gate, float *out, void *stream);
int b200_seq_merge_peers_a16(const void *const *parts, void *const *flags, int n_seq, int me, unsigned epoch, int R, int D,
                             const float *gate, float *out, void *qbuf, void *stream);


/* ---------------------------------------------------------------- prefill ------------------------------------ */
/* attn_prefill / attn_prefill_variant (attn.cuh:46-53, attn.cu:457-499): any T >= 1, query t at p0+t sees 0..p0+t;
 * the cache must already hold 0..p0+T-1.  Uses library scratch: one buffer per (device, stream), allocated on first use,
 * at most 256 MiB of tile images per pass plus 8 bytes per row and head; a longer context takes several passes; a call that
 * needs more than earlier ones gets a new buffer and the old one stays allocated (nothing is freed or synchronised). */
int b200_attn_prefill(const float *q, const b200_kv_cache *c, float *out, int T, int p0, int Hq, float scale, void *stream);
int b200_attn_prefill_variant(const float *q, const b200_kv_cache *c, float *out, int T, int p0, int Hq, float scale,
                              void *stream, int variant);
/* attn_fold_scratch_bytes / attn_fold (src/fast/attn_fold.cuh:19-26): tensor-core prefill with caller scratch.  The
 * scratch holds the keys of one pass as f16 tile images (1 KiB per key and kv head) plus 8 bytes per row and head; the
 * visible context is walked in as many passes as that takes, the running (O, max, sum) of a row tile carried from pass to
 * pass in `out`, so any scratch from one 128-key step upwards works and p0 does not enter the size: the engine's fixed
 * w_scratch (src/tp_model.cu:2905-2920) serves every depth.  scratch_bytes(T, Hkv, chunk, nsplit): bytes for passes of
 * `chunk` keys (chunk <= 0: 8192); attn_fold's chunk > 0 caps the keys per pass; nsplit is accepted and has no meaning. */
size_t b200_attn_fold_scratch_bytes(int T, int Hkv, int chunk, int nsplit);
int b200_attn_fold(const float *q, const b200_kv_cache *c, float *out, int T, int p0, int Hq, float scale,
                   void *scratch, size_t scratch_bytes, void *stream, int chunk, int nsplit);
/* Prefill with the sigmoid gate fused into the epilogue (new): gate [T][Hq*D] may be NULL; scratch NULL = library scratch.
 * _a16 also writes the a16 copy of the gated output for the next projection (layout: see b200_attn_decode_slots_a16). */
int b200_attn_prefill_gated(const float *q, const b200_kv_cache *c, float *out, const float *gate, int T, int p0,
                            int Hq, float scale, void *scratch, size_t scratch_bytes, void *stream);
int b200_attn_prefill_gated_a16(const float *q, const b200_kv_cache *c, float *out, const float *gate, void *qbuf, int T,
                                int p0, int Hq, float scale, void *scratch, size_t scratch_bytes, void *stream);
/* The whole prefill attention step of one layer on bf16 activations (new; the reference's prefill runs k::rope_neox +
 * kv_append + attn_fold + sigmoid_mul on f32 buffers, src/tp_model.cu:2899-2925): k, v [T][Hkv][D] and q [T][Hq][D] bf16
 * (raw bits) as the projections wrote them.  K is rotated (partial NEOX, n_rot = 64, angle from p0 + t), K and V are
 * quantised into rows p0 + t, and attention runs over rows 0 .. p0+T-1 with q rotated on the fly while it is converted for
 * the tensor cores (no fp32 copy of q goes through memory).  Gate: gate_f32 or gate_bf16 [T][Hq*D] or both NULL.  Result:
 * out_f32 and / or out_bf16 [T][Hq][D] (at least one), qbuf optional (a16 copy).  The arithmetic equals
 * b200_rope_append_bf16 followed by b200_attn_prefill_gated.  scratch (required, 256-byte aligned): at least
 * b200_attn_prefill_bf16_scratch_bytes(T, Hkv, pass_keys, out_f32 == NULL), pass_keys as for attn_fold. */
size_t b200_attn_prefill_bf16_scratch_bytes(int T, int Hkv, int pass_keys, int out_is_bf16);
int b200_attn_prefill_bf16(const uint16_t *q, const uint16_t *k, const uint16_t *v, const float *gate_f32,
                           const uint16_t *gate_bf16, float *out_f32, uint16_t *out_bf16, void *qbuf,
                           const b200_kv_cache *c, int p0, int T, int Hq, int n_rot, float freq_base, float scale,
                           void *scratch, size_t scratch_bytes, void *stream);
/* Prefill over one sequence shard (new; for a sequence split across GPUs): row t sees this cache's keys 0 .. last_key[t]
 * (device; -1 = none; must not decrease with t), max_keys = a host bound on last_key[T-1] + 1.  Leaves the unnormalised
 * part_o [T][Hq][D] with part_m (natural-log units, -inf for a row without keys) and part_l [T*Hq], the inputs of
 * b200_attn_merge_gate / b200_seq_exchange_merge, like b200_attn_decode_slots_partial. */
int b200_attn_prefill_partial(const float *q, const b200_kv_cache *c, float *part_o, float *part_m, float *part_l,
                              const int32_t *last_key, int max_keys, int T, int Hq, float scale, void *scratch,
                              size_t scratch_bytes, void *stream);

/* ---------------------------------------------------------------- gate --------------------------------------- */
/* sigmoid_mul (fused.cuh:24, fused.cu:744-748; k::sigmoid_mul kernels.cu:85-93): x *= 1/(1+expf(-g)) */
int b200_sigmoid_mul(float *x, const float *g, int64_t n, void *stream);
/* ew_quant (fused.cuh:93-99, fused.cu:657-675) with op 1 = EW_SIGMOID_MUL (y = a * sigmoid(b)) and
 * op 0 = EW_SILU_MUL (y = silu(a) * b); qbuf != NULL also writes the a16-quantised activation (src/fast/a16q.cuh). */
int b200_ew_quant(int op, const float *a, const float *b, float *y, void *qbuf, int T, int n, void *stream, int lda,
                  int ldb);

/* ---------------------------------------------------------------- pool, block tables, steps, persistence ---- */
/* The caller-side structures the kernels index, kept by the reference inside tp_model (src/tp_model.cu): one pool per GPU
 * laid out [K|V][kv layer][page][2^psh positions][row] (alloc_pool :3880-3966), a page table ptab[max_slots][max_pages]
 * fed from a free list with stream-ordered uploads of new entries from pinned memory (ensure_pages :3358-3384), the per-step
 * descriptor of row positions and table offsets (forward_batch_ids :3999-4022) and the cache views kv_seq / kv_rows
 * (:3327-3337).  Offsets are 64-bit, a step holds up to max_rows rows, and a pool may be shard seq_rank of n_seq sequence
 * shards (logical page g of a sequence lives on shard g mod n_seq as local page g / n_seq): positions passed in are global.
 * device >= 0: pool and tables in that GPU's memory; device < 0: everything in host memory (tools, tests).
 * seed != 0 hands pages out in a seeded random order.  All calls come from one host thread (as in the reference). */
typedef struct b200_pool b200_pool;
b200_pool *b200_pool_create(uint32_t kv_type, int Hkv, int D, int n_layers, int n_pages, int psh, int max_slots,
                            int max_pages, int max_rows, uint32_t seed, int n_seq, int seq_rank, int device);
void b200_pool_destroy(b200_pool *p);
size_t b200_pool_bytes(const b200_pool *p);
void *b200_pool_base(const b200_pool *p);
/* raw pool bytes [offset, offset + nbytes) -> dst (host or device memory), asynchronous on the stream */
int b200_pool_read(const b200_pool *p, size_t offset, void *dst, size_t nbytes, void *stream);
int b200_pool_free_pages(const b200_pool *p);
int b200_pool_slot_pages(const b200_pool *p, int slot);
const int32_t *b200_pool_table_host(const b200_pool *p);          /* host copy of ptab[max_slots][max_pages], -1 = unset */
int b200_pool_local_length(const b200_pool *p, int n_positions);  /* positions of a sequence of n that live on this shard */
/* ensure_pages: positions [0, n_positions) of the slot become addressable; B200_ERR_ALLOC when the pool is full and
 * B200_ERR_SHAPE when the sequence would exceed max_pages (nothing changes in either case) */
int b200_pool_ensure(b200_pool *p, int slot, int n_positions, void *stream);
int b200_pool_release(b200_pool *p, int slot, void *stream);
/* kv_seq (slot >= 0: pt = that slot's table row, rtab = NULL) or kv_rows (slot < 0: pt = the table, rtab = the step's) */
int b200_pool_view(const b200_pool *p, int layer, int slot, b200_kv_cache *out);
/* Step descriptor: row r = i * q_len + j is token j of slots[i] at global position n_past[i] + j (host arrays, n
 * sequences).  Uploads per row (stream-ordered, pinned staging): the rotary position, the local position of the last key
 * this shard holds for the row (-1 = none: what b200_attn_decode_slots takes as pos), the local cache row of the row's own
 * K/V (-1 = another shard's page: what b200_attn_prep_rows takes as cache_row) and rtab.  grow != 0 first makes the new
 * positions addressable.  The device arrays stay valid until the next b200_pool_step on the same stream order. */
int b200_pool_step(b200_pool *p, const int32_t *slots, const int32_t *n_past, int n, int q_len, int grow, void *stream);
const int32_t *b200_pool_step_rope_pos(const b200_pool *p);
const int32_t *b200_pool_step_last_key(const b200_pool *p);
const int32_t *b200_pool_step_cache_row(const b200_pool *p);
const int32_t *b200_pool_step_rtab(const b200_pool *p);
int b200_pool_step_rows(const b200_pool *p);
int b200_pool_step_max_n(const b200_pool *p);   /* host bound of last_key + 1 over the step (max_n of the decode calls) */
/* Page offload (seq_offload :3432-3481, pages_out :3676-3686): pages first..first+n-1 of the slot to / from host memory in
 * the layout [page][K|V][kv layer][2^psh rows x row bytes], b200_pool_page_bytes() per page, two 2-D copies per page,
 * asynchronous on the stream.  pages_in takes pages from the free list as needed. */
size_t b200_pool_page_bytes(const b200_pool *p);
int b200_pool_pages_out(const b200_pool *p, int slot, int first, int n, void *dst_host, void *stream);
int b200_pool_pages_in(b200_pool *p, int slot, int first, int n, const void *src_host, void *stream);
/* Sequence file (seq_write / seq_read :3738-3862): "P100ESQ2" | 15 x u64 fingerprint | i32 n_past, n_tok, pages | tokens |
 * per GPU: its pages in the offload layout, then its recurrent state (opaque bytes of the caller).  The header and each
 * GPU's block are written / read separately, in rank order, on a POSIX file descriptor.  read_header checks the magic
 * (a "P100ESQ1" file is refused as such), every fingerprint field against `want` (*bad_field = index of the first
 * difference, 7 = GPU count / split) and the header (n_tok == n_past <= max_ctx, pages <= max_pages and enough for n_past). */
int b200_session_write_header(int fd, const uint64_t *fingerprint, int n_past, const int32_t *tokens, int n_tok, int pages);
int b200_session_write_rank(int fd, const b200_pool *p, int slot, int pages, const void *state, size_t state_bytes,
                            void *stream);
int b200_session_read_header(int fd, const uint64_t *want, int max_ctx, int max_pages, int psh, int *n_past, int *n_tok,
                             int *pages, int32_t *tokens, int tok_cap, int *bad_field);
int b200_session_read_rank(int fd, b200_pool *p, int slot, int pages, void *state, size_t state_bytes, void *stream);

/* ---------------------------------------------------------------- diagnostics -------------------------------- */
/* Kernels never trap or spin without a limit: a wait that runs out, or an address check that fails, records a code
 * in a device status word and the kernel returns.  This reads (and clears) that word for the current device after
 * synchronising the given stream; 0 = no error.  Codes (or-ed): 1 a bounded wait gave up, 2 a negative page-table entry,
 * 4 a misaligned address, 8 a row position beyond max_n / n_ctx; 0x100 << k names the wait of the tcgen05 verify kernel
 * that gave up (k = 0 K operand, 1 P, 2 K rows, 3 V rows, 4 previous P V, 5 scores, 6 last P V, 7 a free staging buffer). */
int b200_last_device_status(void *stream);
/* launches of this library's kernels since load (all devices), for benchmark bookkeeping */
uint64_t b200_launch_count(void);
const char *b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H */
