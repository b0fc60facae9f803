"""ctypes access to the checkers under oracle/ (TEST INFRASTRUCTURE: imported by tests/, the smoke check and the
benchmark's CPU-baseline leg only — never by the product package).

  liboracle.so            CPU restatement (oracle.c), built on demand with gcc
  _ref/libggml_ref.so     the reference's vendored ggml CPU backend (flash_attn_ext, *_ref quantisers), prebuilt by
                          `make -C oracle ref` where the reference checkout exists
  _ref/libp100e_ref.so    the reference's own CUDA kernels compiled for sm_100a (needs a GPU to run)
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
KV_F16, KV_Q4_0, KV_Q8_0 = 1, 2, 8


class OrcKv(C.Structure):
    _fields_ = [("type", C.c_uint32), ("n_ctx", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32),
                ("k", C.c_void_p), ("v", C.c_void_p), ("pt", C.c_void_p), ("rtab", C.c_void_p),
                ("psh", C.c_int32), ("pstride", C.c_size_t)]


def build_oracle():
    subprocess.check_call(["make", "-s", "-C", HERE, "oracle"])


_o = None


def lib():
    global _o
    if _o is None:
        p = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(p) or os.path.getmtime(p) < os.path.getmtime(os.path.join(HERE, "oracle.c")):
            build_oracle()
        o = C.CDLL(p)
        P, I, F = C.c_void_p, C.c_int, C.c_float
        o.orc_f32_to_f16.restype = C.c_uint16
        o.orc_f32_to_f16.argtypes = [F]
        o.orc_f16_to_f32.restype = F
        o.orc_f16_to_f32.argtypes = [C.c_uint16]
        o.orc_kv_row_bytes.restype = C.c_size_t
        o.orc_kv_row_bytes.argtypes = [C.c_uint32, I, I]
        o.orc_kv_off.restype = C.c_size_t
        o.orc_kv_off.argtypes = [C.POINTER(OrcKv), I, I]
        for n in ("orc_quant_q8_0_head", "orc_quant_q4_0_head", "orc_f16_head", "orc_q8_head_to_ggml", "orc_q8_ggml_to_head"):
            getattr(o, n).restype = None
            getattr(o, n).argtypes = [P, P, I]
        o.orc_dequant_head.restype = None
        o.orc_dequant_head.argtypes = [P, C.c_uint32, I, P]
        o.orc_kv_append.restype = None
        o.orc_kv_append.argtypes = [C.POINTER(OrcKv), P, P, I, P, I, I, I]
        o.orc_attn_prep.restype = None
        o.orc_attn_prep.argtypes = [P, P, P, P, P, P, P, P, C.POINTER(OrcKv), I, I, I, I, I, I, F, F, I, I, I, P]
        o.orc_rope_neox.restype = None
        o.orc_rope_neox.argtypes = [P, P, I, I, I, I, F]
        o.orc_attention.restype = None
        o.orc_attention.argtypes = [P, C.POINTER(OrcKv), P, I, I, P, I, F, P, I, I, P, P, P]
        o.orc_merge.restype = None
        o.orc_merge.argtypes = [P, P, P, I, I, I, P, P]
        o.orc_sigmoid_mul.restype = None
        o.orc_sigmoid_mul.argtypes = [P, P, C.c_int64]
        _o = o
    return _o


def _p(a):
    return None if a is None else a.ctypes.data


def row_bytes(type, Hkv, D):
    return lib().orc_kv_row_bytes(type, Hkv, D)


class Cache:
    """Host-memory cache view for the oracle: numpy uint8 K / V regions + optional int32 page table / row offsets."""

    def __init__(self, type, n_ctx, Hkv, D, k, v, pt=None, rtab=None, psh=0, pstride=0):
        self.type, self.n_ctx, self.Hkv, self.D = type, n_ctx, Hkv, D
        self.k, self.v, self.pt, self.rtab, self.psh, self.pstride = k, v, pt, rtab, psh, pstride

    @classmethod
    def contiguous(cls, type, n_ctx, Hkv, D):
        n = row_bytes(type, Hkv, D) * n_ctx
        return cls(type, n_ctx, Hkv, D, np.zeros(n, np.uint8), np.zeros(n, np.uint8))

    def c(self):
        s = OrcKv()
        s.type, s.n_ctx, s.Hkv, s.D = self.type, self.n_ctx, self.Hkv, self.D
        s.k, s.v, s.pt, s.rtab = _p(self.k), _p(self.v), _p(self.pt), _p(self.rtab)
        s.psh, s.pstride = self.psh, self.pstride
        return s


def quant_head(type, x):
    """x: float32 [D] -> uint8 head row in the cache format"""
    x = np.ascontiguousarray(x, np.float32)
    D = x.size
    out = np.zeros(row_bytes(type, 1, D), np.uint8)
    fn = {KV_F16: "orc_f16_head", KV_Q8_0: "orc_quant_q8_0_head", KV_Q4_0: "orc_quant_q4_0_head"}[type]
    getattr(lib(), fn)(_p(x), _p(out), D)
    return out


def dequant_head(type, head, D):
    out = np.zeros(D, np.float32)
    lib().orc_dequant_head(_p(np.ascontiguousarray(head)), type, D, _p(out))
    return out


def kv_append(c, k, v, p0, T, pos=None, ldk=0, ldv=0):
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    pos = None if pos is None else np.ascontiguousarray(pos, np.int32)
    lib().orc_kv_append(C.byref(c.c()), _p(k), _p(v), p0, _p(pos), T, ldk, ldv)


def attn_prep(qg, k, v, q_norm, k_norm, pos, c, p0, T, Hq, Hkv, D, n_rot, freq_base, eps, want_kpre=False):
    qg = np.ascontiguousarray(qg, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    pos = np.ascontiguousarray(pos, np.int32)
    q = np.zeros((T, Hq, D), np.float32)
    gate = np.zeros((T, Hq * D), np.float32)
    kpre = np.zeros((T, Hkv, D), np.float32) if want_kpre else None
    lib().orc_attn_prep(_p(qg), _p(k), _p(v), _p(q_norm), _p(k_norm), _p(pos), _p(q), _p(gate), C.byref(c.c()), p0, T, Hq,
                        Hkv, D, n_rot, freq_base, eps, 0, 0, 0, _p(kpre))
    return (q, gate, kpre) if want_kpre else (q, gate)


def rope_neox(x, pos, n_rot, freq_base):
    x = np.array(x, np.float32, copy=True)
    T, H, D = x.shape
    lib().orc_rope_neox(_p(x), _p(np.ascontiguousarray(pos, np.int32)), T, H, D, n_rot, freq_base)
    return x


def attention(q, c, T, Hq, scale, p0=0, pos=None, gate=None, k_lo=0, k_hi=0, partial=False):
    """fp64 attention of T rows over the cache; returns out [T][Hq][D] (and (oacc, m, l) when partial=True)."""
    q = np.ascontiguousarray(q, np.float32)
    pos = None if pos is None else np.ascontiguousarray(pos, np.int32)
    gate = None if gate is None else np.ascontiguousarray(gate, np.float32)
    D = c.D
    out = np.zeros((T, Hq, D), np.float32)
    oacc = om = ol = None
    if partial:
        oacc = np.zeros((T, Hq, D), np.float32)
        om = np.zeros((T, Hq), np.float32)
        ol = np.zeros((T, Hq), np.float32)
    lib().orc_attention(_p(q), C.byref(c.c()), _p(out), T, p0, _p(pos), Hq, scale, _p(gate), k_lo, k_hi, _p(oacc), _p(om),
                        _p(ol))
    return (out, oacc, om, ol) if partial else out


def merge(oacc, om, ol, gate=None):
    oacc = np.ascontiguousarray(oacc, np.float32)
    nparts, R, D = oacc.shape
    out = np.zeros((R, D), np.float32)
    lib().orc_merge(_p(oacc), _p(np.ascontiguousarray(om, np.float32)), _p(np.ascontiguousarray(ol, np.float32)), nparts, R,
                    D, _p(None if gate is None else np.ascontiguousarray(gate, np.float32)), _p(out))
    return out


def sigmoid_mul(x, g):
    x = np.array(x, np.float32, copy=True)
    lib().orc_sigmoid_mul(_p(x), _p(np.ascontiguousarray(g, np.float32)), x.size)
    return x


def q8_head_to_ggml(head, D=256):
    out = np.zeros(D // 32 * 34, np.uint8)
    lib().orc_q8_head_to_ggml(_p(np.ascontiguousarray(head)), _p(out), D)
    return out


# ---------------------------------------------------------------------------------------------- reference libs ----
_g = None


def ggml_ref():
    """The reference's vendored ggml CPU backend, or None when it was not prebuilt."""
    global _g
    if _g is None:
        p = os.path.join(HERE, "_ref", "libggml_ref.so")
        if not os.path.exists(p):
            return None
        g = C.CDLL(p)
        P, I, F = C.c_void_p, C.c_int, C.c_float
        g.ggml_ref_quantize_q8_0.argtypes = [P, P, C.c_int64]
        g.ggml_ref_quantize_q4_0.argtypes = [P, P, C.c_int64]
        g.ggml_ref_fp32_to_fp16.restype = C.c_uint16
        g.ggml_ref_fp32_to_fp16.argtypes = [F]
        g.ggml_ref_fp16_to_fp32.restype = F
        g.ggml_ref_fp16_to_fp32.argtypes = [C.c_uint16]
        g.ggml_ref_flash_attn.restype = I
        g.ggml_ref_flash_attn.argtypes = [P, P, P, I, I, I, I, I, I, F, I, I, P]
        _g = g
    return _g


def ggml_flash_attn(q, k_rows, v_rows, type, n_kv, q_len, Hq, Hkv, D, scale, n_threads, reps=1):
    """q [q_len][Hq][D] f32; k_rows / v_rows: uint8 [n_kv][Hkv][head bytes] in ggml block layout. Returns out [q_len][Hq][D]."""
    g = ggml_ref()
    q = np.ascontiguousarray(q, np.float32)
    out = np.zeros((q_len, Hq, D), np.float32)
    rc = g.ggml_ref_flash_attn(_p(q), _p(k_rows), _p(v_rows), type, n_kv, q_len, Hq, Hkv, D, scale, n_threads, reps, _p(out))
    if rc:
        raise RuntimeError("ggml_ref_flash_attn failed (%d)" % rc)
    return out


_r = None


def p100e_ref():
    """The reference's own CUDA kernels compiled for sm_100a (ctypes handle), or None when not prebuilt."""
    global _r
    if _r is None:
        p = os.path.join(HERE, "_ref", "libp100e_ref.so")
        if not os.path.exists(p):
            return None
        r = C.CDLL(p)
        P, I, F = C.c_void_p, C.c_int, C.c_float
        KP = C.POINTER(OrcKv)
        r.ref_kv_row_bytes.restype = C.c_size_t
        r.ref_kv_row_bytes.argtypes = [C.c_uint32, I, I]
        r.ref_kv_append.restype = None
        r.ref_kv_append.argtypes = [KP, P, P, I, I, P]
        r.ref_kv_append_dev.restype = None
        r.ref_kv_append_dev.argtypes = [KP, P, P, P, I, P]
        r.ref_attn_decode.argtypes = [P, KP, P, I, I, I, F, P]
        r.ref_attn_decode_dev.argtypes = [P, KP, P, I, P, I, I, F, P]
        r.ref_attn_decode_rows.argtypes = [P, KP, P, I, P, I, F, P]
        r.ref_attn_prefill.argtypes = [P, KP, P, I, I, I, F, P]
        r.ref_attn_fold_scratch_bytes.restype = C.c_size_t
        r.ref_attn_fold_scratch_bytes.argtypes = [I, I, I, I]
        r.ref_attn_fold.argtypes = [P, KP, P, I, I, I, F, P, C.c_size_t, P]
        r.ref_attn_prep.argtypes = [P, P, P, P, P, P, P, P, KP, I, I, I, I, I, I, F, F, P]
        r.ref_attn_prep_mrope.argtypes = [P, P, P, P, P, P, P, P, KP, I, I, I, I, I, I, F, F, P, P, I, I, I, I, I]
        r.ref_sigmoid_mul.restype = None
        r.ref_sigmoid_mul.argtypes = [P, P, C.c_int64, P]
        r.ref_k_sigmoid_mul.restype = None
        r.ref_k_sigmoid_mul.argtypes = [P, P, C.c_int64, P]
        r.ref_ew_quant.argtypes = [I, P, P, P, P, I, I, P]
        r.ref_k_rope_neox.restype = None
        r.ref_k_rope_neox.argtypes = [P, P, I, I, I, I, F, P]
        r.ref_k_attention.restype = None
        r.ref_k_attention.argtypes = [P, P, P, P, I, I, I, I, I, F, P]
        r.ref_attn_dec2_nsplit.argtypes = [I]
        _r = r
    return _r
