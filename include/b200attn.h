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
    B200_ERR_DEVICE = 5   /* a kernel recorded an error in the status word (see b200_last_device_status) */
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

/* ---------------------------------------------------------------- KV append ---------------------------------- */
/* kv_append (attn.cuh:36, attn.cu:583): k, v [T][Hkv][D] f32 -> positions p0..p0+T-1, converted / quantised.
 * Bytes written are identical to the reference quantiser's for the same inputs. */
int b200_kv_append(const b200_kv_cache *c, const float *k, const float *v, int p0, int T, void *stream);
/* kv_append_dev (attn.cuh:58, attn.cu:587): first position read from *p0_dev when the kernel runs */
int b200_kv_append_dev(const b200_kv_cache *c, const float *k, const float *v, const int32_t *p0_dev, int T, void *stream);
/* attn_prep (src/fast/fused.cuh:101-113, fused.cu:677-721): per token split q|gate, RMSNorm(q)*q_norm,
 * RMSNorm(k)*k_norm, partial NEOX RoPE on the first n_rot dims (angle from pos[t]), K and V quantised straight into
 * cache row p0+t (p0 >= 0) or pos[t] (p0 < 0).  ldq/ldk/ldv: row strides in floats (0 = dense).  mr may be NULL. */
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

/* ---------------------------------------------------------------- decode / MTP verify ------------------------ */
/* attn_decode (attn.cuh:44, attn.cu:638): q, out [T][Hq][D] f32, row t at position p0+t sees keys 0..p0+t. T <= 8. */
int b200_attn_decode(const float *q, const b200_kv_cache *c, float *out, int T, int p0, int Hq, float scale, void *stream);
/* attn_decode_dev (attn.cuh:59, attn.cu:654): p0 read from *p0_dev on the device; grid sized for p0+T <= max_n */
int b200_attn_decode_dev(const float *q, const b200_kv_cache *c, float *out, int T, const int32_t *p0_dev, int max_n,
                         int Hq, float scale, void *stream);
/* attn_decode_rows (attn.cuh:64-66, attn.cu:649): row t at pos[t] (device) of its own sequence (pt + rtab[t]) */
int b200_attn_decode_rows(const float *q, const b200_kv_cache *c, float *out, int T, const int32_t *pos, int Hq,
                          float scale, void *stream);
/* attn_decode2 (src/fast/attn_dec2.cuh:17-18): the dispatcher behind the three calls above */
int b200_attn_decode2(const float *q, const b200_kv_cache *c, float *out, int T, int p0, const int32_t *p0_dev, int Hq,
                      float scale, void *stream, const int32_t *pos_rows);
/* attn_dec2_nsplit / attn_dec2_set_nsplit / attn_dec2_reload_env (attn_dec2.cuh:19-21).  This library splits the
 * keys into fixed chunks of b200_attn_chunk_keys() positions instead of a fixed number of interleaved streams;
 * nsplit reports how many chunks a full n_ctx context has, set_nsplit(n > 0) pins the chunk so that n_ctx/n keys
 * fall in each (0 = default); reload_env re-reads B200ATTN_CHUNK and returns 1 if the chunk changed. */
int b200_attn_dec2_nsplit(int Hkv);
void b200_attn_dec2_set_nsplit(int n);
int b200_attn_dec2_reload_env(void);

/* Batched decode / verify, any number of slots (new; the reference stops at 8 rows per call, attn.cuh:66).
 * n_slots sequences, q_len (1..4) query rows each; row r = slot * q_len + j sits at pos[r] (device) and sees keys
 * 0..pos[r] of its slot (pos[r] < 0: the row sees nothing and its output is zero); the slot's page table is
 * pt + rtab[slot * q_len] (rtab == NULL: one table for all).  The q_len rows of a slot share one pass over its KV.
 * gate != NULL: out = attn * sigmoid(gate) fused into the split merge (ew_quant(EW_SIGMOID_MUL), fused.cu:479-496;
 * k::sigmoid_mul, src/kernels.cu:85-93).  max_n: upper bound of pos[r] + 1 over the call (sizes the grid).
 * chunk_keys: keys per split (multiple of 64); 0 = the library default, -1 = chosen from the batch size.
 * Each row's result depends only on its own keys and on chunk_keys, never on the other rows of the call. */
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
 *   - A kernel-side status (bad page id, timed-out wait) of this entry point is kept in a word of its own and is not
 *     reported by b200_last_device_status. */
int b200_attn_decode_slots_noalloc(const float *q, const b200_kv_cache *c, float *out, const float *gate, int n_slots,
                                   int q_len, const int32_t *pos, int max_n, int Hq, float scale, int chunk_keys,
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
/* The exchange + merge step of the sequence split for a host that drives NCCL itself (the reference links NCCL for its
 * tensor-parallel all-reduce, src/tp_model.cu:41 `#include <nccl.h>`; it has no sequence split, so this entry has no
 * reference twin).  send = this shard's partial as one flat buffer [O (R*D) | m (R) | l (R)] (the three outputs of
 * b200_attn_decode_slots_partial placed back to back), recv = n_seq such buffers.  ncclAllGather over `nccl_comm`
 * (an ncclComm_t of the n_seq shards, rank order = shard order) on `stream`, then the merge of b200_attn_merge_gate.
 * n_seq == 1 merges `send` alone; nccl_comm == NULL with n_seq > 1 means the caller has already gathered the n_seq
 * buffers into recv (some other transport) and only the merge runs.  NCCL is not linked: the symbol is taken from the
 * NCCL library already loaded. */
int b200_seq_exchange_merge(void *nccl_comm, int n_seq, const float *send, float *recv, int R, int D, const float *gate,
                            float *out, void *stream);
int b200_attn_chunk_keys(void); /* the default chunk (keys) used by the reference-compatible entry points */

/* ---------------------------------------------------------------- prefill ------------------------------------ */
/* attn_prefill / attn_prefill_variant (attn.cuh:46-53, attn.cu:457-499): any T >= 1, query t at p0+t sees 0..p0+t;
 * the cache must already hold 0..p0+T-1.  Needs library scratch (allocated on first use per device). */
int b200_attn_prefill(const float *q, const b200_kv_cache *c, float *out, int T, int p0, int Hq, float scale, void *stream);
int b200_attn_prefill_variant(const float *q, const b200_kv_cache *c, float *out, int T, int p0, int Hq, float scale,
                              void *stream, int variant);
/* attn_fold_scratch_bytes / attn_fold (src/fast/attn_fold.cuh:19-26): tensor-core prefill with caller scratch */
size_t b200_attn_fold_scratch_bytes(int T, int Hkv, int chunk, int nsplit);
int b200_attn_fold(const float *q, const b200_kv_cache *c, float *out, int T, int p0, int Hq, float scale,
                   void *scratch, size_t scratch_bytes, void *stream, int chunk, int nsplit);
/* Prefill with the sigmoid gate fused into the epilogue (new): gate [T][Hq*D] may be NULL. */
int b200_attn_prefill_gated(const float *q, const b200_kv_cache *c, float *out, const float *gate, int T, int p0,
                            int Hq, float scale, void *scratch, size_t scratch_bytes, void *stream);

/* ---------------------------------------------------------------- gate --------------------------------------- */
/* sigmoid_mul (fused.cuh:24, fused.cu:744-748; k::sigmoid_mul kernels.cu:85-93): x *= 1/(1+expf(-g)) */
int b200_sigmoid_mul(float *x, const float *g, int64_t n, void *stream);
/* ew_quant (fused.cuh:93-99, fused.cu:657-675) with op 1 = EW_SIGMOID_MUL (y = a * sigmoid(b)) and
 * op 0 = EW_SILU_MUL (y = silu(a) * b); qbuf != NULL also writes the a16-quantised activation (src/fast/a16q.cuh). */
int b200_ew_quant(int op, const float *a, const float *b, float *y, void *qbuf, int T, int n, void *stream, int lda,
                  int ldb);

/* ---------------------------------------------------------------- diagnostics -------------------------------- */
/* Kernels never trap or spin without a limit: a wait that runs out, or an address check that fails, records a code
 * in a device status word and the kernel returns.  This reads (and clears) that word for the current device after
 * synchronising the given stream; 0 = no error. */
int b200_last_device_status(void *stream);
/* launches of this library's kernels since load (all devices), for benchmark bookkeeping */
uint64_t b200_launch_count(void);
const char *b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H */
