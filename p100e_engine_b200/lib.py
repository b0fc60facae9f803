"""ctypes binding of libb200attn.so — the C ABI declared in include/b200attn.h, nothing else.

The library is loaded from this directory (built in-tree by p100e_engine_b200.build).  There is no fallback: if the
shared object is missing or a call is refused, an exception is raised.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("B200ATTN_LIB") or os.path.join(HERE, "libb200attn.so")   # B200ATTN_LIB: another build of the same ABI

KV_F16, KV_Q4_0, KV_Q8_0 = 1, 2, 8
ATTN_MAX_ROWS = 8
MAX_QLEN = 4
OK, ERR_SHAPE, ERR_ALLOC, ERR_CUDA, ERR_SCRATCH, ERR_DEVICE, ERR_FORMAT, ERR_IO = range(8)


class KvCache(C.Structure):
    """b200_kv_cache (include/b200attn.h) == p100e::fast::kv_cache (reference src/fast/attn.cuh:18-32)."""
    _fields_ = [("type", C.c_uint32), ("n_ctx", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32),
                ("k", C.c_void_p), ("v", C.c_void_p), ("pt", C.c_void_p), ("rtab", C.c_void_p),
                ("psh", C.c_int32), ("pstride", C.c_size_t)]

    def c(self):   # the host-side mirror's kv_cache objects convert themselves with c(); a struct is already one
        return self


class MropePos(C.Structure):
    _fields_ = [("p", C.c_void_p), ("stride", C.c_int32), ("s0", C.c_int32), ("s1", C.c_int32), ("s2", C.c_int32),
                ("sect", C.c_int32)]


class B200Error(RuntimeError):
    def __init__(self, what, code):
        super().__init__("%s refused (status %d)" % (what, code))
        self.code = code


P, I, F, U32, SZ, I64 = C.c_void_p, C.c_int, C.c_float, C.c_uint32, C.c_size_t, C.c_int64
KVP = C.POINTER(KvCache)

# name -> (restype, argtypes); every symbol include/b200attn.h declares
SIGNATURES = {
    "b200_kv_row_bytes": (SZ, [U32, I, I]),
    "b200_kv_alloc": (I, [KVP, U32, I, I, I]),
    "b200_kv_free": (None, [KVP]),
    "b200_kv_fill_random": (I, [KVP, I, I, U32, P]),
    "b200_kv_fill_slots": (I, [KVP, I, P, I, U32, I, I, I, P]),
    "b200_kv_append": (I, [KVP, P, P, I, I, P]),
    "b200_kv_append_dev": (I, [KVP, P, P, P, I, P]),
    "b200_attn_prep": (I, [P, P, P, P, P, P, P, P, KVP, I, I, I, I, I, I, F, F, P, I, I, I, C.POINTER(MropePos)]),
    "b200_attn_prep_rows": (I, [P, P, P, P, P, P, P, P, P, KVP, I, I, I, I, I, F, F, P]),
    "b200_rope_append_bf16": (I, [P, P, P, P, KVP, I, I, I, I, I, I, F, P]),
    "b200_rope_append_bf16_at": (I, [P, P, P, P, KVP, I, I, I, I, I, I, I, F, P]),
    "b200_attn_decode": (I, [P, KVP, P, I, I, I, F, P]),
    "b200_attn_decode_dev": (I, [P, KVP, P, I, P, I, I, F, P]),
    "b200_attn_decode_rows": (I, [P, KVP, P, I, P, I, F, P]),
    "b200_attn_decode2": (I, [P, KVP, P, I, I, P, I, F, P, P]),
    "b200_attn_dec2_nsplit": (I, [I]),
    "b200_attn_dec2_set_nsplit": (None, [I]),
    "b200_attn_step_begin": (I, [P, P, SZ]),
    "b200_attn_step_end": (I, [P]),
    "b200_attn_dec_tc": (I, []),
    "b200_attn_dec_set_tc": (None, [I]),
    "b200_attn_dec2_reload_env": (I, []),
    "b200_attn_fixed_chunk": (I, [I]),
    "b200_attn_reserve": (I, [U32, I, I, I, I, I, I, P]),
    "b200_attn_decode_slots": (I, [P, KVP, P, P, I, I, P, I, I, F, I, P]),
    "b200_attn_decode_slots_a16": (I, [P, KVP, P, P, P, I, I, P, I, I, F, I, P]),
    "b200_noalloc_device_status": (I, [P]),
    "b200_attn_decode_slots_noalloc": (I, [P, KVP, P, P, I, I, P, I, I, F, I, P]),
    "b200_attn_decode_slots_partial": (I, [P, KVP, P, P, P, I, I, P, I, I, F, I, P]),
    "b200_attn_merge_gate": (I, [P, P, P, I, I, I, P, P, P]),
    "b200_seq_exchange_merge": (I, [P, I, P, P, I, I, P, P, P]),
    "b200_seq_exchange_merge_a16": (I, [P, I, P, P, I, I, P, P, P, P]),
    "b200_peer_alloc": (I, [SZ, P, P]),
    "b200_peer_open": (I, [P, P]),
    "b200_peer_close": (I, [P]),
    "b200_peer_free": (I, [P]),
    "b200_seq_merge_peers": (I, [P, P, I, I, U32, I, I, P, P, P]),
    "b200_seq_merge_peers_a16": (I, [P, P, I, I, U32, I, I, P, P, P, P]),
    "b200_attn_chunk_keys": (I, []),
    "b200_attn_prefill": (I, [P, KVP, P, I, I, I, F, P]),
    "b200_attn_prefill_variant": (I, [P, KVP, P, I, I, I, F, P, I]),
    "b200_attn_fold_scratch_bytes": (SZ, [I, I, I, I]),
    "b200_attn_fold": (I, [P, KVP, P, I, I, I, F, P, SZ, P, I, I]),
    "b200_attn_prefill_gated": (I, [P, KVP, P, P, I, I, I, F, P, SZ, P]),
    "b200_attn_prefill_gated_a16": (I, [P, KVP, P, P, P, I, I, I, F, P, SZ, P]),
    "b200_attn_prefill_bf16_scratch_bytes": (SZ, [I, I, I, I]),
    "b200_attn_prefill_bf16": (I, [P, P, P, P, P, P, P, P, KVP, I, I, I, I, F, F, P, SZ, P]),
    "b200_attn_prefill_partial": (I, [P, KVP, P, P, P, P, I, I, I, F, P, SZ, P]),
    "b200_sigmoid_mul": (I, [P, P, I64, P]),
    "b200_ew_quant": (I, [I, P, P, P, P, I, I, P, I, I]),
    "b200_pool_create": (P, [U32, I, I, I, I, I, I, I, I, U32, I, I, I]),
    "b200_pool_destroy": (None, [P]),
    "b200_pool_bytes": (SZ, [P]),
    "b200_pool_base": (P, [P]),
    "b200_pool_read": (I, [P, SZ, P, SZ, P]),
    "b200_pool_free_pages": (I, [P]),
    "b200_pool_slot_pages": (I, [P, I]),
    "b200_pool_table_host": (P, [P]),
    "b200_pool_local_length": (I, [P, I]),
    "b200_pool_ensure": (I, [P, I, I, P]),
    "b200_pool_release": (I, [P, I, P]),
    "b200_pool_view": (I, [P, I, I, KVP]),
    "b200_pool_step": (I, [P, P, P, I, I, I, P]),
    "b200_pool_step_rope_pos": (P, [P]),
    "b200_pool_step_last_key": (P, [P]),
    "b200_pool_step_cache_row": (P, [P]),
    "b200_pool_step_rtab": (P, [P]),
    "b200_pool_step_rows": (I, [P]),
    "b200_pool_step_max_n": (I, [P]),
    "b200_pool_page_bytes": (SZ, [P]),
    "b200_pool_pages_out": (I, [P, I, I, I, P, P]),
    "b200_pool_pages_in": (I, [P, I, I, I, P, P]),
    "b200_session_write_header": (I, [I, P, I, P, I, I]),
    "b200_session_write_rank": (I, [I, P, I, I, P, SZ, P]),
    "b200_session_read_header": (I, [I, P, I, I, I, P, P, P, P, I, P]),
    "b200_session_read_rank": (I, [I, P, I, I, P, SZ, P]),
    "b200_last_device_status": (I, [P]),
    "b200_launch_count": (C.c_uint64, []),
    "b200_version": (C.c_char_p, []),
}

_lib = None


def load():
    """dlopen libb200attn.so and set the prototypes. Raises if the library has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError("%s is missing: run `python -m p100e_engine_b200.build`" % LIB_PATH)
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def ptr(x):
    """device (or host) address of a torch tensor / numpy array / int / None"""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    return x.ctypes.data


def check(what, code):
    if code != OK:
        raise B200Error(what, code)
