"""Shared helpers of the parity tests: seeded inputs, paged pools, tolerances, host<->device cache mirrors."""
import numpy as np

from oracle import orc

HQ, HKV, D = 24, 4, 256
SCALE = 1.0 / 16.0
TYPES = {"f16": 1, "q4_0": 2, "q8_0": 8}

# Tolerance for fp32-accumulated attention outputs (the bar "max-abs 2e-3 / rel 1e-2"), measured the way the
# reference's own tests measure: largest absolute error relative to the largest reference magnitude
# (max_abs <= 2e-3 * max|ref|, tests/fast_attn_test.cu:70-78 in the reference project) and relative RMS error
# (rel-RMS <= 1e-2, tests/fast_attn_fold_test.cu:82).
TOL_ABS, TOL_REL = 2e-3, 1e-2


def check_close(a, ref, what="", tol_abs=TOL_ABS, tol_rel=TOL_REL):
    a = np.asarray(a, np.float64)
    ref = np.asarray(ref, np.float64)
    assert a.shape == ref.shape, (what, a.shape, ref.shape)
    assert np.isfinite(a).all(), "%s: non-finite output" % what
    mx = max(np.abs(ref).max(), 1e-30)
    err = np.abs(a - ref)
    ma = err.max()
    rms = np.sqrt((err ** 2).sum() / max((ref ** 2).sum(), 1e-60))
    assert ma <= tol_abs * mx, "%s: max_abs %.3e > %.1e * %.3e" % (what, ma, tol_abs, mx)
    assert rms <= tol_rel, "%s: rel-RMS %.3e > %.1e" % (what, rms, tol_rel)
    return ma / mx, rms


def rng_normal(seed, shape):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


class PagedPool:
    """A pool laid out like the reference engine's ([K|V][layer][page][2^psh positions][row], reference
    src/tp_model.cu:3875-3942) or, with interleave=True, like its paging test (page-major with other layers in
    between, tests/fast_sessions_test.cu:69-92): host numpy mirror + page tables."""

    def __init__(self, type, n_pages, psh=8, hkv=HKV, d=D, n_layers=1, layer=0, interleave=False, seed=0, slack=0):
        self.type, self.psh, self.hkv, self.d = type, psh, hkv, d
        self.ps = 1 << psh
        self.rowb = orc.row_bytes(type, hkv, d)
        self.n_pages = n_pages
        pblk = self.ps * self.rowb
        if interleave:
            self.pstride = n_layers * 2 * pblk
            self.koff = layer * 2 * pblk
            self.voff = self.koff + pblk
            self.bytes = n_pages * self.pstride
        else:
            self.pstride = pblk
            self.koff = layer * n_pages * pblk
            self.voff = (n_layers + layer) * n_pages * pblk
            self.bytes = 2 * n_layers * n_pages * pblk
        self.host = np.zeros(self.bytes + slack, np.uint8)
        self.perm = np.random.default_rng(seed).permutation(n_pages).astype(np.int32)
        self.used = 0

    def take(self, n_positions, max_pages):
        """page-table row for a sequence of n_positions (unused entries -1)"""
        need = (n_positions + self.ps - 1) // self.ps
        assert self.used + need <= self.n_pages and need <= max_pages
        row = np.full(max_pages, -1, np.int32)
        row[:need] = self.perm[self.used:self.used + need]
        self.used += need
        return row

    def host_cache(self, pt, rtab=None, n_ctx=None):
        k = self.host[self.koff:]
        v = self.host[self.voff:]
        return orc.Cache(self.type, n_ctx or (len(pt) << self.psh), self.hkv, self.d, k, v, pt, rtab, self.psh, self.pstride)


def to_dev(a, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def dev_cache(pool_t, pool, pt_t=None, rtab_t=None, n_ctx=0):
    """device kv_cache view over a torch uint8 copy of a PagedPool"""
    from p100e_engine_b200 import fast
    return fast.kv_cache(pool.type, n_ctx, pool.hkv, pool.d, pool_t.data_ptr() + pool.koff, pool_t.data_ptr() + pool.voff,
                         pt_t, rtab_t, pool.psh, pool.pstride)


def orc_kv_of(c, dev_k=None, dev_v=None):
    """OrcKv struct for the reference CUDA library from a fast.kv_cache (same fields)"""
    from p100e_engine_b200 import lib as L
    s = orc.OrcKv()
    s.type, s.n_ctx, s.Hkv, s.D = c.type, c.n_ctx, c.Hkv, c.D
    s.k, s.v, s.pt, s.rtab = L.ptr(c.k), L.ptr(c.v), L.ptr(c.pt), L.ptr(c.rtab)
    s.psh, s.pstride = c.psh, c.pstride
    return s
