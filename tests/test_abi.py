"""The C-ABI library loads and exports exactly what include/b200attn.h declares (no GPU needed: no compute calls)."""
import os
import re

from p100e_engine_b200 import lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "b200attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    syms = header_symbols()
    assert len(syms) >= 25
    for s in syms:
        assert hasattr(lib, s), "library does not export %s" % s


def test_binding_covers_header():
    assert sorted(L.SIGNATURES) == header_symbols()


def test_shim_header_compiles_reference_call_sites():
    """include/p100e_fast_shim.h keeps the reference's C++ signatures and defaults: a translation unit with the call forms
    of the reference's callers (tests/cabi/shim_callsites.cpp) must compile against it"""
    import shutil
    import subprocess
    cuda_inc = None
    for cand in ("/usr/local/cuda/include", os.path.join(os.path.dirname(os.path.dirname(shutil.which("nvcc") or "/x/y")), "include")):
        if os.path.exists(os.path.join(cand, "cuda_runtime.h")):
            cuda_inc = cand
            break
    assert cuda_inc, "cuda_runtime.h not found"
    r = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", cuda_inc,
                        os.path.join(ROOT, "tests", "cabi", "shim_callsites.cpp")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_row_bytes(lib):
    # reference kv_row_bytes (src/fast/attn.cu:501-503): f16 2 B/value, q8_0 34 B and q4_0 18 B per 32 values
    assert lib.b200_kv_row_bytes(L.KV_F16, 4, 256) == 2048
    assert lib.b200_kv_row_bytes(L.KV_Q8_0, 4, 256) == 1088
    assert lib.b200_kv_row_bytes(L.KV_Q4_0, 4, 256) == 576
    assert lib.b200_version().startswith(b"b200attn")


def test_struct_layout():
    # b200_kv_cache must be field-for-field the reference's kv_cache (src/fast/attn.cuh:18-32) on LP64
    import ctypes as C
    assert C.sizeof(L.KvCache) == 64
    assert L.KvCache.k.offset == 16 and L.KvCache.pt.offset == 32 and L.KvCache.psh.offset == 48
    assert L.KvCache.pstride.offset == 56


def test_refusals_without_launch(lib):
    # argument checks happen before any CUDA call: refused calls return a status and launch nothing
    import ctypes as C
    c = L.KvCache()
    c.type, c.n_ctx, c.Hkv, c.D = 99, 8, 4, 256
    n0 = lib.b200_launch_count()
    assert lib.b200_kv_append(C.byref(c), None, None, 0, 1, None) == L.ERR_SHAPE
    assert lib.b200_attn_decode(None, C.byref(c), None, 1, 0, 24, 0.0625, None) == L.ERR_SHAPE
    assert lib.b200_attn_decode_rows(None, C.byref(c), None, 1, None, 24, 0.0625, None) == L.ERR_SHAPE
    # the peer merge: null tables, more shards than the kernel takes, a shard index outside the group
    two = (C.c_void_p * 2)(0, 0)
    assert lib.b200_seq_merge_peers(None, None, 2, 0, 1, 24, 256, None, None, None) == L.ERR_SHAPE
    assert lib.b200_seq_merge_peers(two, two, 9, 0, 1, 24, 256, None, C.c_void_p(16), None) == L.ERR_SHAPE
    assert lib.b200_seq_merge_peers(two, two, 2, 2, 1, 24, 256, None, C.c_void_p(16), None) == L.ERR_SHAPE
    assert lib.b200_seq_merge_peers(two, two, 2, 0, 1, 24, 256, None, C.c_void_p(16), None) == L.ERR_SHAPE   # unmapped shards
    assert lib.b200_peer_open(None, None) == L.ERR_SHAPE and lib.b200_peer_alloc(0, None, None) == L.ERR_SHAPE
    assert lib.b200_launch_count() == n0
