"""Python mirror of the library's paged-KV pool (b200_pool_* / b200_session_* in include/b200attn.h).

The pool, its page tables, the step descriptor, the page offload layout and the sequence file format are host C++ inside
libb200attn.so (csrc/kv_pool.cu), standing for what the reference engine keeps in tp_model (reference src/tp_model.cu:
alloc_pool :3880-3966, ensure_pages :3358-3384, forward_batch_ids :3999-4022, kv_seq / kv_rows :3327-3337, seq_offload
:3432-3481, seq_write / seq_read :3738-3862).  This module only forwards to it; `device=-1` keeps a pool in host memory,
which is how the CPU tests drive the same code.
"""
import ctypes as C

import numpy as np

from . import lib as L

HEAD_BYTES = {L.KV_F16: 512, L.KV_Q8_0: 272, L.KV_Q4_0: 144}   # D = 256


def row_bytes(kv_type, hkv, d=256):
    return L.load().b200_kv_row_bytes(kv_type, hkv, d)


def _i32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32))


class Pool:
    """One GPU's (or, with device=-1, a host-memory) pool [K|V][layer][page][2^psh][row] with its page table."""

    def __init__(self, kv_type, hkv, n_layers, n_pages, psh=8, d=256, max_slots=1, max_pages=1, max_rows=1, seed=0, n_seq=1,
                 seq_rank=0, device=-1):
        self.lib = L.load()
        self.h = self.lib.b200_pool_create(kv_type, hkv, d, n_layers, n_pages, psh, max_slots, max_pages, max_rows, seed, n_seq,
                                           seq_rank, device)
        if not self.h:
            raise RuntimeError("b200_pool_create refused")
        self.kv_type, self.hkv, self.d, self.n_layers, self.n_pages, self.psh = kv_type, hkv, d, n_layers, n_pages, psh
        self.max_slots, self.max_pages, self.max_rows, self.device = max_slots, max_pages, max_rows, device
        self.rowb = row_bytes(kv_type, hkv, d)
        self.pstride = self.rowb << psh
        self.total_bytes = self.lib.b200_pool_bytes(self.h)
        self.page_bytes = self.lib.b200_pool_page_bytes(self.h)

    def close(self):
        if self.h:
            self.lib.b200_pool_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- tables
    def table(self):
        """host copy of ptab[max_slots][max_pages] (a view of the library's pinned memory; -1 = unset)"""
        p = self.lib.b200_pool_table_host(self.h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_int32)), shape=(self.max_slots, self.max_pages))

    def free_pages(self):
        return self.lib.b200_pool_free_pages(self.h)

    def slot_pages(self, slot):
        return self.lib.b200_pool_slot_pages(self.h, slot)

    def local_length(self, n):
        return self.lib.b200_pool_local_length(self.h, n)

    def ensure(self, slot, n_positions, stream=None):
        return self.lib.b200_pool_ensure(self.h, slot, n_positions, stream)

    def release(self, slot, stream=None):
        return self.lib.b200_pool_release(self.h, slot, stream)

    def view(self, layer, slot=-1):
        """b200_kv_cache of one layer: slot >= 0 = that sequence (kv_seq), slot < 0 = all rows of the last step (kv_rows)"""
        c = L.KvCache()
        L.check("b200_pool_view", self.lib.b200_pool_view(self.h, layer, slot, C.byref(c)))
        return c

    # ---- step descriptor
    def step(self, slots, n_past, q_len, grow=True, stream=None):
        s, n = _i32(slots), _i32(n_past)
        return self.lib.b200_pool_step(self.h, s.ctypes.data, n.ctypes.data, len(s), q_len, 1 if grow else 0, stream)

    def step_arrays(self):
        """device (or host, for a host pool) addresses: rotary position, last visible local key, own cache row, rtab"""
        f = self.lib
        return (f.b200_pool_step_rope_pos(self.h), f.b200_pool_step_last_key(self.h), f.b200_pool_step_cache_row(self.h),
                f.b200_pool_step_rtab(self.h))

    def step_rows(self):
        return self.lib.b200_pool_step_rows(self.h)

    def step_max_n(self):
        return self.lib.b200_pool_step_max_n(self.h)

    def step_host(self):
        """the four step arrays of a host-memory pool as numpy arrays (tests)"""
        assert self.device < 0
        r = self.step_rows()
        return [np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_int32)), shape=(r,)).copy() for p in self.step_arrays()]

    # ---- offload / files
    def pages_out(self, slot, first, n, dst, stream=None):
        return self.lib.b200_pool_pages_out(self.h, slot, first, n, L.ptr(dst), stream)

    def pages_in(self, slot, first, n, src, stream=None):
        return self.lib.b200_pool_pages_in(self.h, slot, first, n, L.ptr(src), stream)

    def base_host(self):
        """the pool bytes of a host-memory pool as a numpy view (tests)"""
        assert self.device < 0
        p = self.lib.b200_pool_base(self.h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(self.total_bytes,))

    def base(self):
        return self.lib.b200_pool_base(self.h)

    def read(self, offset, dst, nbytes, stream=None):
        """raw pool bytes -> dst (tensor, array or address; host or device memory), asynchronous on the stream"""
        return self.lib.b200_pool_read(self.h, offset, L.ptr(dst), nbytes, stream)


def session_write(fd, fingerprint, n_past, tokens, pools_slots, states=None, stream=None):
    """one sequence file: header, then every (pool, slot) block in rank order with its opaque state bytes"""
    lib = L.load()
    fp = np.ascontiguousarray(np.asarray(fingerprint, dtype=np.uint64))
    assert fp.shape == (15,)
    tok = _i32(tokens)
    pages = pools_slots[0][0].slot_pages(pools_slots[0][1])
    rc = lib.b200_session_write_header(fd, fp.ctypes.data, n_past, tok.ctypes.data, len(tok), pages)
    for i, (pool, slot) in enumerate(pools_slots):
        if rc != L.OK:
            break
        st = states[i] if states else b""
        rc = lib.b200_session_write_rank(fd, pool.h, slot, pool.slot_pages(slot), C.c_char_p(st) if st else None, len(st), stream)
    return rc


def session_read(fd, fingerprint, max_ctx, pools_slots, state_bytes=None, stream=None):
    """reads a sequence file into the given (pool, free slot) pairs; returns (status, n_past, tokens, states, bad_field)"""
    lib = L.load()
    fp = np.ascontiguousarray(np.asarray(fingerprint, dtype=np.uint64))
    pool0 = pools_slots[0][0]
    n_past, n_tok, pages, bad = C.c_int(), C.c_int(), C.c_int(), C.c_int(-1)
    tok = np.zeros(max(max_ctx, 1), np.int32)
    rc = lib.b200_session_read_header(fd, fp.ctypes.data, max_ctx, pool0.max_pages, pool0.psh, C.byref(n_past), C.byref(n_tok),
                                      C.byref(pages), tok.ctypes.data, len(tok), C.byref(bad))
    states = []
    for i, (pool, slot) in enumerate(pools_slots):
        if rc != L.OK:
            break
        nb = state_bytes[i] if state_bytes else 0
        buf = C.create_string_buffer(nb) if nb else None
        rc = lib.b200_session_read_rank(fd, pool.h, slot, pages.value, buf, nb, stream)
        states.append(buf.raw if buf else b"")
    return rc, n_past.value, tok[:n_tok.value].copy(), states, bad.value
