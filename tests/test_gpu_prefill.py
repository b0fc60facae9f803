"""Chunked causal prefill attention on the GPU (tcgen05 kernel) against the CPU oracle and the reference's own prefill
kernels, restating tests/fast_attn_test.cu:205-220 ((p0, T) = (0,37), (1000,300), (3700,396)),
tests/fast_attn_fold_test.cu:37-92 (fold vs fp32 prefill) and tests/fast_sessions_test.cu (paged == contiguous)."""
import ctypes as C

import numpy as np
import pytest

from oracle import orc
from tests import util
from tests.util import D, HKV, HQ, SCALE, TYPES

pytestmark = pytest.mark.gpu


def _filled(kt, n, cuda, seed, hkv=HKV):
    import torch
    from p100e_engine_b200 import fast
    k = util.rng_normal(seed, (n, hkv, D))
    v = util.rng_normal(seed + 1, (n, hkv, D))
    c = fast.kv_alloc(kt, n, hkv, D)
    assert fast.kv_append(c, util.to_dev(k, cuda), util.to_dev(v, cuda), 0, n)
    torch.cuda.synchronize()
    return c, orc.Cache(kt, n, hkv, D, c.k.cpu().numpy(), c.v.cpu().numpy())


@pytest.mark.parametrize("tname", ["q8_0", "f16", "q4_0"])
@pytest.mark.parametrize("p0,T", [(0, 37), (1000, 300), (3700, 396), (0, 1), (63, 2), (64, 130)])
def test_prefill_vs_oracle(cuda, lib, tname, p0, T):
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    c, oc = _filled(kt, p0 + T, cuda, 100 + p0)
    q = util.rng_normal(7 + T, (T, HQ, D))
    out = torch.full((T, HQ, D), float("nan"), device=cuda)
    assert fast.attn_prefill(util.to_dev(q, cuda), c, out, T, p0, HQ, SCALE)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    ref = orc.attention(q, oc, T, HQ, SCALE, p0=p0)
    util.check_close(out.cpu().numpy(), ref, "prefill %s p0=%d T=%d" % (tname, p0, T))


@pytest.mark.parametrize("tname", ["q8_0", "f16", "q4_0"])
def test_prefill_one_kv_head_shard(cuda, lib, tname):
    """the shape one GPU of a 4-GPU run holds: one kv head, 6 query heads; odd number of 64-key images (a last half step)"""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    p0, T, hq = 130, 250, 6
    c, oc = _filled(kt, p0 + T, cuda, 55, hkv=1)
    q = util.rng_normal(56, (T, hq, D))
    out = torch.full((T, hq, D), float("nan"), device=cuda)
    assert fast.attn_prefill(util.to_dev(q, cuda), c, out, T, p0, hq, SCALE)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    ref = orc.attention(q, oc, T, hq, SCALE, p0=p0)
    util.check_close(out.cpu().numpy(), ref, "prefill one head %s" % tname)


@pytest.mark.parametrize("tname", ["q8_0", "q4_0"])
def test_prefill_gated_paged_vs_oracle_and_reference(cuda, lib, tname):
    """paged cache (seeded permutation), caller scratch, fused gate; against the oracle and the reference's fp32
    attn_prefill + k::sigmoid_mul and its attn_fold"""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    p0, T = 700, 520
    n = p0 + T
    pool = util.PagedPool(kt, 8, psh=8, seed=2)
    pt = pool.take(n, 8)
    pool_t = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    pt_t = util.to_dev(pt, cuda)
    dc = util.dev_cache(pool_t, pool, pt_t, None, 8 << 8)
    assert fast.kv_append(dc, util.to_dev(util.rng_normal(1, (n, HKV, D)), cuda), util.to_dev(util.rng_normal(2, (n, HKV, D)), cuda), 0, n)
    torch.cuda.synchronize()
    pool.host[:pool.bytes] = pool_t.cpu().numpy()
    q = util.rng_normal(3, (T, HQ, D))
    gate = util.rng_normal(4, (T, HQ * D))
    qd, gd = util.to_dev(q, cuda), util.to_dev(gate, cuda)
    nb = fast.attn_fold_scratch_bytes(T, HKV, n)
    scratch = torch.empty(nb, dtype=torch.uint8, device=cuda)
    out = torch.zeros(T, HQ, D, device=cuda)
    assert fast.attn_prefill_gated(qd, dc, out, gd, T, p0, HQ, SCALE, scratch, nb)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    ref = orc.attention(q, pool.host_cache(pt), T, HQ, SCALE, p0=p0, gate=gate)
    util.check_close(out.cpu().numpy(), ref, "gated paged prefill " + tname)
    # too little scratch is refused with nothing launched
    n0 = lib.b200_launch_count()
    assert not fast.attn_fold(qd, dc, out, T, p0, HQ, SCALE, scratch, 1024)
    assert lib.b200_launch_count() == n0
    r = orc.p100e_ref()
    if r is not None:
        rc = util.orc_kv_of(dc)
        o_ref = torch.zeros(T, HQ, D, device=cuda)
        assert r.ref_attn_prefill(qd.data_ptr(), C.byref(rc), o_ref.data_ptr(), T, p0, HQ, SCALE, None) == 0
        r.ref_k_sigmoid_mul(o_ref.data_ptr(), gd.data_ptr(), T * HQ * D, None)
        torch.cuda.synchronize()
        util.check_close(out.cpu().numpy(), o_ref.cpu().numpy(), "vs reference attn_prefill " + tname)
        # the reference's own tensor-free fold path is held to 3e-2 / 1e-2 RMS against its fp32 kernel
        # (tests/fast_attn_fold_test.cu:82); ours must sit inside the same band
        o_fold = torch.zeros(T, HQ, D, device=cuda)
        ws = torch.empty(256 << 20, dtype=torch.uint8, device=cuda)
        assert r.ref_attn_fold(qd.data_ptr(), C.byref(rc), o_fold.data_ptr(), T, p0, HQ, SCALE, ws.data_ptr(), 256 << 20, None) == 0
        r.ref_k_sigmoid_mul(o_fold.data_ptr(), gd.data_ptr(), T * HQ * D, None)
        torch.cuda.synchronize()
        util.check_close(o_fold.cpu().numpy(), o_ref.cpu().numpy(), "reference fold vs reference fp32", 3e-2, 1e-2)


def test_prefill_equals_looped_decode(cuda, lib):
    """prefill rows agree with the decode kernel row by row (reference relation tests/fast_prefill_test.cu:383-429)"""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES["q8_0"]
    p0, T = 300, 70
    c, _ = _filled(kt, p0 + T, cuda, 55)
    q = util.to_dev(util.rng_normal(56, (T, HQ, D)), cuda)
    o_pf = torch.zeros(T, HQ, D, device=cuda)
    o_dec = torch.zeros(T, HQ, D, device=cuda)
    assert fast.attn_prefill(q, c, o_pf, T, p0, HQ, SCALE)
    for t in range(0, T, 4):
        tt = min(4, T - t)
        assert fast.attn_decode(q[t:t + tt], c, o_dec[t:t + tt], tt, p0 + t, HQ, SCALE)
    torch.cuda.synchronize()
    util.check_close(o_pf.cpu().numpy(), o_dec.cpu().numpy(), "prefill vs looped decode")


def test_prefill_linearity_in_v_full_size(cuda, lib):
    """Chunked-prefill shape at full size (T = 8192, p0 = 0, q8_0, 32 pages): too large for the oracle, so checked through
    size-independent properties: rows of a chunked call (4 x 2048 with growing p0) equal the single call, and the
    first rows equal a short prefix run"""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES["q8_0"]
    T = 8192
    pool = util.PagedPool(kt, 32, psh=8, seed=3)
    pt = pool.take(T, 32)
    pool_t = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    dc = util.dev_cache(pool_t, pool, util.to_dev(pt, cuda), None, T)
    g = torch.Generator(device="cpu").manual_seed(5)
    k = torch.randn(T, HKV, D, generator=g).to(torch.bfloat16)
    v = torch.randn(T, HKV, D, generator=g).to(torch.bfloat16)
    q = torch.randn(T, HQ, D, generator=g).to(torch.bfloat16)
    qr = torch.zeros(T, HQ, D, device=cuda)
    assert fast.rope_append_bf16(q.to(cuda), k.to(cuda), v.to(cuda), qr, dc, 0, T, HQ, HKV, D, 64, 1e7)
    gate = torch.randn(T, HQ * D, generator=g).to(cuda)
    o_full = torch.zeros(T, HQ, D, device=cuda)
    assert fast.attn_prefill_gated(qr, dc, o_full, gate, T, 0, HQ, SCALE, None, 0)
    o_chunk = torch.zeros(T, HQ, D, device=cuda)
    for p0 in range(0, T, 2048):
        assert fast.attn_prefill_gated(qr[p0:p0 + 2048], dc, o_chunk[p0:p0 + 2048], gate[p0:p0 + 2048], 2048, p0, HQ, SCALE, None, 0)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    assert torch.isfinite(o_full).all()
    util.check_close(o_chunk.cpu().numpy(), o_full.cpu().numpy(), "chunked vs single call", 1e-3, 1e-3)
    # prefix against the oracle (first 40 rows only)
    pool.host[:pool.bytes] = pool_t.cpu().numpy()
    ref = orc.attention(qr[:40].cpu().numpy(), pool.host_cache(pt), 40, HQ, SCALE, p0=0, gate=gate[:40].cpu().numpy())
    util.check_close(o_full[:40].cpu().numpy(), ref, "config 3 prefix vs oracle")
