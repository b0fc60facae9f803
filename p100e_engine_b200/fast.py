"""Host-side mirror of the reference's `p100e::fast` attention interface (src/fast/attn.cuh, attn_dec2.cuh,
attn_fold.cuh, fused.cuh in the reference project) over torch CUDA tensors.

Same names, same argument order and meaning, same error behaviour: a call returns True after enqueuing its kernels on
the stream, or False with nothing launched (the library prints one line to stderr).  Every call goes through the C ABI
of libb200attn.so; there is no other implementation behind these functions.
"""
import ctypes as C

import torch

from . import lib as L

KV_F16, KV_Q4_0, KV_Q8_0 = L.KV_F16, L.KV_Q4_0, L.KV_Q8_0
ATTN_MAX_ROWS = L.ATTN_MAX_ROWS
EW_SILU_MUL, EW_SIGMOID_MUL = 0, 1


class kv_cache:
    """View of one layer's K and V (reference struct kv_cache, src/fast/attn.cuh:18-32).

    k, v: uint8 CUDA tensors (or raw device addresses) of the K / V region; pt / rtab: int32 CUDA tensors or None.
    """

    def __init__(self, type=KV_F16, n_ctx=0, Hkv=0, D=0, k=None, v=None, pt=None, rtab=None, psh=0, pstride=0):
        self.type, self.n_ctx, self.Hkv, self.D = type, n_ctx, Hkv, D
        self.k, self.v, self.pt, self.rtab, self.psh, self.pstride = k, v, pt, rtab, psh, pstride

    def c(self):
        s = L.KvCache()
        s.type, s.n_ctx, s.Hkv, s.D = self.type, self.n_ctx, self.Hkv, self.D
        s.k, s.v, s.pt, s.rtab = L.ptr(self.k), L.ptr(self.v), L.ptr(self.pt), L.ptr(self.rtab)
        s.psh, s.pstride = self.psh, self.pstride
        return s


def _stream(s):
    if s is None:
        return torch.cuda.current_stream().cuda_stream
    return s.cuda_stream if hasattr(s, "cuda_stream") else s


def kv_row_bytes(type, Hkv, D):
    return L.load().b200_kv_row_bytes(type, Hkv, D)


def kv_alloc(type, n_ctx, Hkv, D, device="cuda"):
    """Contiguous cache [n_ctx][row] for K and V (zero-filled torch allocations; k is None on failure)."""
    c = kv_cache(type, n_ctx, Hkv, D)
    if type not in (KV_F16, KV_Q4_0, KV_Q8_0) or (type != KV_F16 and D % 32):
        return c
    n = kv_row_bytes(type, Hkv, D) * n_ctx
    c.k = torch.zeros(n, dtype=torch.uint8, device=device)
    c.v = torch.zeros(n, dtype=torch.uint8, device=device)
    return c


def kv_free(c):
    c.k = c.v = None


def kv_append(c, k, v, p0, T, s=None):
    return L.load().b200_kv_append(C.byref(c.c()), L.ptr(k), L.ptr(v), p0, T, _stream(s)) == L.OK


def kv_append_dev(c, k, v, p0_dev, T, s=None):
    return L.load().b200_kv_append_dev(C.byref(c.c()), L.ptr(k), L.ptr(v), L.ptr(p0_dev), T, _stream(s)) == L.OK


def attn_decode(q, c, out, T, p0, Hq, scale, s=None):
    return L.load().b200_attn_decode(L.ptr(q), C.byref(c.c()), L.ptr(out), T, p0, Hq, scale, _stream(s)) == L.OK


def attn_decode_dev(q, c, out, T, p0_dev, max_n, Hq, scale, s=None):
    return L.load().b200_attn_decode_dev(L.ptr(q), C.byref(c.c()), L.ptr(out), T, L.ptr(p0_dev), max_n, Hq, scale,
                                         _stream(s)) == L.OK


def attn_decode_rows(q, c, out, T, pos, Hq, scale, s=None):
    return L.load().b200_attn_decode_rows(L.ptr(q), C.byref(c.c()), L.ptr(out), T, L.ptr(pos), Hq, scale,
                                          _stream(s)) == L.OK


def attn_decode2(q, c, out, T, p0, p0_dev, Hq, scale, s=None, pos_rows=None):
    return L.load().b200_attn_decode2(L.ptr(q), C.byref(c.c()), L.ptr(out), T, p0, L.ptr(p0_dev), Hq, scale, _stream(s),
                                      L.ptr(pos_rows)) == L.OK


def attn_decode_slots(q, c, out, gate, n_slots, q_len, pos, max_n, Hq, scale, chunk_keys=0, s=None):
    """Batched decode / verify with the fused sigmoid gate (no row limit; see include/b200attn.h)."""
    return L.load().b200_attn_decode_slots(L.ptr(q), C.byref(c.c()), L.ptr(out), L.ptr(gate), n_slots, q_len, L.ptr(pos),
                                           max_n, Hq, scale, chunk_keys, _stream(s)) == L.OK


def attn_decode_slots_a16(q, c, out, gate, qbuf, n_slots, q_len, pos, max_n, Hq, scale, chunk_keys=0, s=None):
    """attn_decode_slots that also emits the a16 copy of the gated output (input format of the next projection)"""
    return L.load().b200_attn_decode_slots_a16(L.ptr(q), C.byref(c.c()), L.ptr(out), L.ptr(gate), L.ptr(qbuf), n_slots, q_len,
                                               L.ptr(pos), max_n, Hq, scale, chunk_keys, _stream(s)) == L.OK


def attn_decode_slots_noalloc(q, c, out, gate, n_slots, q_len, pos, max_n, Hq, scale, chunk_keys=0, s=None):
    return L.load().b200_attn_decode_slots_noalloc(L.ptr(q), C.byref(c.c()), L.ptr(out), L.ptr(gate), n_slots, q_len, L.ptr(pos),
                                                   max_n, Hq, scale, chunk_keys, _stream(s))


def attn_reserve(kv_type, max_slots, q_len, max_n, n_ctx, Hkv, chunk_keys=0, s=None):
    return L.load().b200_attn_reserve(kv_type, max_slots, q_len, max_n, n_ctx, Hkv, chunk_keys, _stream(s)) == L.OK


def attn_decode_slots_partial(q, c, part_o, part_m, part_l, n_slots, q_len, pos, max_n, Hq, scale, chunk_keys=0, s=None):
    return L.load().b200_attn_decode_slots_partial(L.ptr(q), C.byref(c.c()), L.ptr(part_o), L.ptr(part_m), L.ptr(part_l),
                                                   n_slots, q_len, L.ptr(pos), max_n, Hq, scale, chunk_keys,
                                                   _stream(s)) == L.OK


def attn_merge_gate(part_o, part_m, part_l, nparts, R, D, gate, out, s=None):
    return L.load().b200_attn_merge_gate(L.ptr(part_o), L.ptr(part_m), L.ptr(part_l), nparts, R, D, L.ptr(gate),
                                         L.ptr(out), _stream(s)) == L.OK


def seq_exchange_merge(nccl_comm, n_seq, send, recv, R, D, gate, out, s=None):
    """all-gather of the shards' flat partials over the caller's ncclComm_t (an integer address) + merge + gate"""
    return L.load().b200_seq_exchange_merge(C.c_void_p(nccl_comm), n_seq, L.ptr(send), L.ptr(recv), R, D, L.ptr(gate),
                                            L.ptr(out), _stream(s)) == L.OK


def seq_exchange_merge_a16(nccl_comm, n_seq, send, recv, R, D, gate, out, qbuf, s=None):
    return L.load().b200_seq_exchange_merge_a16(C.c_void_p(nccl_comm), n_seq, L.ptr(send), L.ptr(recv), R, D, L.ptr(gate),
                                                L.ptr(out), L.ptr(qbuf), _stream(s)) == L.OK


def attn_step_begin(positions, nbytes=None, s=None):
    """the device array `positions` stays as it is until the next call: batched calls on the stream whose pos argument lies
    inside it reuse the even split within the step"""
    if nbytes is None:
        nbytes = positions.numel() * positions.element_size()
    return L.load().b200_attn_step_begin(_stream(s), L.ptr(positions), nbytes) == L.OK


def attn_step_end(s=None):
    return L.load().b200_attn_step_end(_stream(s)) == L.OK


def peer_alloc(nbytes):
    """(device address, 64-byte handle) of a zero-filled buffer that other processes of the node can map"""
    p, h = C.c_void_p(), (C.c_ubyte * 64)()
    L.check("b200_peer_alloc", L.load().b200_peer_alloc(nbytes, C.byref(p), h))
    return p.value, bytes(h)


def peer_open(handle):
    """device address of a peer's buffer in this process"""
    p, h = C.c_void_p(), (C.c_ubyte * 64).from_buffer_copy(handle)
    L.check("b200_peer_open", L.load().b200_peer_open(h, C.byref(p)))
    return p.value


def peer_close(ptr):
    return L.load().b200_peer_close(C.c_void_p(ptr)) == L.OK


def peer_free(ptr):
    return L.load().b200_peer_free(C.c_void_p(ptr)) == L.OK


def seq_merge_peers(parts, flags, me, epoch, R, D, gate, out, qbuf=None, s=None):
    """merge of the shards' partials read in place over peer mappings; parts / flags: device addresses in shard order"""
    n = len(parts)
    pa, fa = (C.c_void_p * n)(*parts), (C.c_void_p * n)(*flags)
    lib = L.load()
    if qbuf is None:
        return lib.b200_seq_merge_peers(pa, fa, n, me, epoch, R, D, L.ptr(gate), L.ptr(out), _stream(s)) == L.OK
    return lib.b200_seq_merge_peers_a16(pa, fa, n, me, epoch, R, D, L.ptr(gate), L.ptr(out), L.ptr(qbuf), _stream(s)) == L.OK


def attn_prefill(q, c, out, T, p0, Hq, scale, s=None):
    return L.load().b200_attn_prefill(L.ptr(q), C.byref(c.c()), L.ptr(out), T, p0, Hq, scale, _stream(s)) == L.OK


def attn_fold_scratch_bytes(T, Hkv, chunk=0, nsplit=0):
    return L.load().b200_attn_fold_scratch_bytes(T, Hkv, chunk, nsplit)


def attn_fold(q, c, out, T, p0, Hq, scale, scratch, scratch_bytes, s=None, chunk=0, nsplit=0):
    return L.load().b200_attn_fold(L.ptr(q), C.byref(c.c()), L.ptr(out), T, p0, Hq, scale, L.ptr(scratch), scratch_bytes,
                                   _stream(s), chunk, nsplit) == L.OK


def attn_prefill_gated(q, c, out, gate, T, p0, Hq, scale, scratch, scratch_bytes, s=None):
    return L.load().b200_attn_prefill_gated(L.ptr(q), C.byref(c.c()), L.ptr(out), L.ptr(gate), T, p0, Hq, scale,
                                            L.ptr(scratch), scratch_bytes, _stream(s)) == L.OK


def attn_prefill_gated_a16(q, c, out, gate, qbuf, T, p0, Hq, scale, scratch, scratch_bytes, s=None):
    return L.load().b200_attn_prefill_gated_a16(L.ptr(q), C.byref(c.c()), L.ptr(out), L.ptr(gate), L.ptr(qbuf), T, p0, Hq, scale,
                                                L.ptr(scratch), scratch_bytes, _stream(s)) == L.OK


def attn_prefill_bf16_scratch_bytes(T, Hkv, pass_keys=0, out_is_bf16=False):
    return L.load().b200_attn_prefill_bf16_scratch_bytes(T, Hkv, pass_keys, 1 if out_is_bf16 else 0)


def attn_prefill_bf16(q, k, v, gate_f32, gate_bf16, out_f32, out_bf16, qbuf, c, p0, T, Hq, n_rot, freq_base, scale, scratch,
                      scratch_bytes, s=None):
    """rope + quantise + append of K/V and gated causal attention over bf16 q in one call (see include/b200attn.h)"""
    return L.load().b200_attn_prefill_bf16(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(gate_f32), L.ptr(gate_bf16), L.ptr(out_f32),
                                           L.ptr(out_bf16), L.ptr(qbuf), C.byref(c.c()), p0, T, Hq, n_rot, freq_base, scale,
                                           L.ptr(scratch), scratch_bytes, _stream(s)) == L.OK


def attn_prefill_partial(q, c, part_o, part_m, part_l, last_key, max_keys, T, Hq, scale, scratch, scratch_bytes, s=None):
    return L.load().b200_attn_prefill_partial(L.ptr(q), C.byref(c.c()), L.ptr(part_o), L.ptr(part_m), L.ptr(part_l),
                                              L.ptr(last_key), max_keys, T, Hq, scale, L.ptr(scratch), scratch_bytes,
                                              _stream(s)) == L.OK


def attn_prep(qg, k, v, q_norm, k_norm, pos, q, gate, c, p0, T, Hq, Hkv, D, n_rot, freq_base, eps, s=None, ldq=0, ldk=0,
              ldv=0, mr=None):
    m = None
    if mr is not None:
        m = L.MropePos(L.ptr(mr["p"]), mr["stride"], mr["s0"], mr["s1"], mr["s2"], mr["sect"])
    return L.load().b200_attn_prep(L.ptr(qg), L.ptr(k), L.ptr(v), L.ptr(q_norm), L.ptr(k_norm), L.ptr(pos), L.ptr(q),
                                   L.ptr(gate), C.byref(c.c()), p0, T, Hq, Hkv, D, n_rot, freq_base, eps, _stream(s), ldq,
                                   ldk, ldv, C.byref(m) if m is not None else None) == L.OK


def attn_prep_rows(qg, k, v, q_norm, k_norm, rope_pos, cache_row, q, gate, c, T, Hq, Hkv, D, n_rot, freq_base, eps, s=None):
    """attn_prep with separate rotary positions and cache rows (cache_row < 0: row owned by another GPU)"""
    return L.load().b200_attn_prep_rows(L.ptr(qg), L.ptr(k), L.ptr(v), L.ptr(q_norm), L.ptr(k_norm), L.ptr(rope_pos),
                                        L.ptr(cache_row), L.ptr(q), L.ptr(gate), C.byref(c.c()), T, Hq, Hkv, D, n_rot,
                                        freq_base, eps, _stream(s)) == L.OK


def rope_append_bf16(q, k, v, q_out, c, p0, T, Hq, Hkv, D, n_rot, freq_base, s=None):
    return L.load().b200_rope_append_bf16(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(q_out), C.byref(c.c()), p0, T, Hq, Hkv, D,
                                          n_rot, freq_base, _stream(s)) == L.OK


def rope_append_bf16_at(q, k, v, q_out, c, row0, rope0, T, Hq, Hkv, D, n_rot, freq_base, s=None):
    """rope_append_bf16 with separate cache row / rotary position (sequence shards); k = v = None rotates q only"""
    return L.load().b200_rope_append_bf16_at(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(q_out), C.byref(c.c()), row0, rope0, T, Hq, Hkv, D,
                                             n_rot, freq_base, _stream(s)) == L.OK


def sigmoid_mul(x, g, n, s=None):
    return L.load().b200_sigmoid_mul(L.ptr(x), L.ptr(g), n, _stream(s)) == L.OK


def ew_quant(op, a, b, y, qbuf, T, n, s=None, lda=0, ldb=0):
    return L.load().b200_ew_quant(op, L.ptr(a), L.ptr(b), L.ptr(y), L.ptr(qbuf), T, n, _stream(s), lda, ldb) == L.OK


def kv_fill_random(c, p0, p1, seed, s=None):
    return L.load().b200_kv_fill_random(C.byref(c.c()), p0, p1, seed, _stream(s)) == L.OK


def kv_fill_slots(c, n_slots, lens, table_stride, seed, head0=0, n_seq=1, seq_rank=0, s=None):
    return L.load().b200_kv_fill_slots(C.byref(c.c()), n_slots, L.ptr(lens), table_stride, seed, head0, n_seq, seq_rank,
                                       _stream(s)) == L.OK


def noalloc_device_status(s=None):
    return L.load().b200_noalloc_device_status(_stream(s))


def device_status(s=None):
    """Status word of the current device after synchronising the stream (0 = no kernel recorded an error)."""
    return L.load().b200_last_device_status(_stream(s))
