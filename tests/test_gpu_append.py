"""KV append and attention input prep on the GPU: bytes against the CPU oracle (bit-exact) and against the reference's
own kernels compiled for sm_100a (memcmp), following the reference tests tests/fast_attn_test.cu:105-128,
tests/fast_sessions_test.cu:69-128 and tests/fast_fusion_test.cu:212-253."""
import ctypes as C

import numpy as np
import pytest

from oracle import orc
from tests import util
from tests.util import D, HKV, HQ, TYPES

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tname", ["f16", "q8_0", "q4_0"])
def test_append_contiguous_bitexact(cuda, lib, tname):
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    T, p0, n_ctx = 37, 3, 64
    k = util.rng_normal(1, (T, HKV, D))
    v = util.rng_normal(2, (T, HKV, D)) * 2.0
    # edge rows: all zeros, ties in magnitude with opposite signs, one huge value, negative extreme
    k[0] = 0.0
    v[1, 0, :32] = np.tile(np.array([1.5, -1.5], np.float32), 16)
    v[1, 1, :32] = np.tile(np.array([-1.5, 1.5], np.float32), 16)
    k[2, 0, 5] = 60000.0
    k[2, 1, 7] = -3.25
    c = fast.kv_alloc(kt, n_ctx, HKV, D)
    assert fast.kv_append(c, util.to_dev(k, cuda), util.to_dev(v, cuda), p0, T)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    oc = orc.Cache.contiguous(kt, n_ctx, HKV, D)
    orc.kv_append(oc, k, v, p0, T)
    assert np.array_equal(c.k.cpu().numpy(), oc.k)
    assert np.array_equal(c.v.cpu().numpy(), oc.v)
    # device-resident first position (graph replay form) writes the same bytes
    c2 = fast.kv_alloc(kt, n_ctx, HKV, D)
    p0_dev = torch.tensor([p0], dtype=torch.int32, device=cuda)
    assert fast.kv_append_dev(c2, util.to_dev(k, cuda), util.to_dev(v, cuda), p0_dev, T)
    assert torch.equal(c2.k, c.k) and torch.equal(c2.v, c.v)
    # block round trip limits of the reference test (tests/fast_attn_test.cu:122)
    rowb = orc.row_bytes(kt, HKV, D)
    hb = rowb // HKV
    lim = {"f16": 1e-3, "q8_0": 0.005, "q4_0": 0.126}[tname]
    vb = c.v.cpu().numpy()
    for t in range(3, T):
        for h in range(HKV):
            deq = orc.dequant_head(kt, vb[(p0 + t) * rowb + h * hb:(p0 + t) * rowb + (h + 1) * hb], D)
            for b in range(D // 32):
                x = v[t, h, b * 32:(b + 1) * 32]
                assert np.abs(x - deq[b * 32:(b + 1) * 32]).max() / np.abs(x).max() < lim


@pytest.mark.parametrize("tname", ["f16", "q8_0", "q4_0"])
@pytest.mark.parametrize("interleave", [False, True])
def test_append_paged_equals_contiguous(cuda, lib, tname, interleave):
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    lens = [700, 1100, 300]
    maxp = 8
    pool = util.PagedPool(kt, 16, psh=8, n_layers=2, layer=1, interleave=interleave, seed=5)
    pts = np.stack([pool.take(n, maxp) for n in lens])
    pool_t = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    pt_t = util.to_dev(pts.reshape(-1), cuda)
    for s, n in enumerate(lens):
        k = util.rng_normal(10 + s, (n, HKV, D))
        v = util.rng_normal(20 + s, (n, HKV, D))
        hc = pool.host_cache(pts[s])
        dc = util.dev_cache(pool_t, pool, pt_t[s * maxp:(s + 1) * maxp], None, maxp << 8)
        for p in range(0, n, 64):
            T = min(64, n - p)
            orc.kv_append(hc, k[p:p + T], v[p:p + T], p, T)
            assert fast.kv_append(dc, util.to_dev(k[p:p + T], cuda), util.to_dev(v[p:p + T], cuda), p, T)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    assert np.array_equal(pool_t.cpu().numpy(), pool.host[:pool.bytes])


@pytest.mark.parametrize("tname", ["f16", "q8_0", "q4_0"])
def test_append_matches_reference_kernels(cuda, lib, tname):
    """same bytes as the reference's kv_append compiled for this GPU (src/fast/attn.cu:583)"""
    import torch
    from p100e_engine_b200 import fast
    ref = orc.p100e_ref()
    if ref is None:
        pytest.skip("reference kernels not prebuilt (oracle/_ref/libp100e_ref.so)")
    kt = TYPES[tname]
    T, p0, n_ctx = 130, 7, 256
    k = util.to_dev(util.rng_normal(3, (T, HKV, D)), cuda)
    v = util.to_dev(util.rng_normal(4, (T, HKV, D)) * 3.0, cuda)
    a = fast.kv_alloc(kt, n_ctx, HKV, D)
    b = fast.kv_alloc(kt, n_ctx, HKV, D)
    assert fast.kv_append(a, k, v, p0, T)
    rb = util.orc_kv_of(b)
    ref.ref_kv_append(C.byref(rb), k.data_ptr(), v.data_ptr(), p0, T, None)
    torch.cuda.synchronize()
    assert torch.equal(a.k, b.k) and torch.equal(a.v, b.v)


def _prep_inputs(T, Hq, Hkv, seed):
    qg = util.rng_normal(seed, (T, Hq, 2 * D))
    k = util.rng_normal(seed + 1, (T, Hkv, D))
    v = util.rng_normal(seed + 2, (T, Hkv, D))
    rng = np.random.default_rng(seed + 3)
    qn = (0.2 + rng.random(D)).astype(np.float32)
    kn = (0.2 + rng.random(D)).astype(np.float32)
    return qg, k, v, qn, kn


@pytest.mark.parametrize("tname", ["f16", "q8_0", "q4_0"])
@pytest.mark.parametrize("T,row0,pos0", [(1, 0, 0), (4, 77, 77), (3, 10, 100000)])
def test_attn_prep_matches_reference_kernels(cuda, lib, tname, T, row0, pos0):
    """q, gate and cache bytes identical to the reference's attn_prep (tests/fast_fusion_test.cu:212-253): cache rows
    from the host (p0 + t) and from the device positions (p0 = -1)"""
    import torch
    from p100e_engine_b200 import fast
    ref = orc.p100e_ref()
    if ref is None:
        pytest.skip("reference kernels not prebuilt (oracle/_ref/libp100e_ref.so)")
    kt = TYPES[tname]
    Hq, Hkv, n_rot, base, eps, n_ctx = 12, 2, 64, 1e7, 1e-6, 256
    qg, k, v, qn, kn = [util.to_dev(x, cuda) for x in _prep_inputs(T, Hq, Hkv, 40)]
    pos = torch.arange(pos0, pos0 + T, dtype=torch.int32, device=cuda)
    for pp in ([row0, -1] if row0 == pos0 else [row0]):
        outs = []
        for impl in ("new", "ref"):
            c = fast.kv_alloc(kt, n_ctx, Hkv, D)
            q = torch.zeros(T, Hq, D, device=cuda)
            gate = torch.zeros(T, Hq * D, device=cuda)
            if impl == "new":
                assert fast.attn_prep(qg, k, v, qn, kn, pos, q, gate, c, pp, T, Hq, Hkv, D, n_rot, base, eps)
            else:
                rc = util.orc_kv_of(c)
                assert ref.ref_attn_prep(qg.data_ptr(), k.data_ptr(), v.data_ptr(), qn.data_ptr(), kn.data_ptr(),
                                         pos.data_ptr(), q.data_ptr(), gate.data_ptr(), C.byref(rc), pp, T, Hq, Hkv, D, n_rot,
                                         base, eps, None) == 0
            torch.cuda.synchronize()
            outs.append((q, gate, c.k.clone(), c.v.clone()))
        for a_, b_, name in zip(outs[0], outs[1], ("q", "gate", "K bytes", "V bytes")):
            assert torch.equal(a_, b_), "%s differs from the reference (%s, p0=%d)" % (name, tname, pp)
    assert fast.device_status() == 0


@pytest.mark.parametrize("tname", ["q8_0", "q4_0", "f16"])
def test_attn_prep_vs_oracle(cuda, lib, tname):
    """against the CPU restatement: gate exact, q within a few ulp (host libm), cache bytes equal except where the
    last-ulp difference of the rotated value crosses a rounding boundary (bounded fraction, one quantisation step)"""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    T, p0, n_rot, base, eps = 5, 1000, 64, 1e7, 1e-6
    qg, k, v, qn, kn = _prep_inputs(T, HQ, HKV, 50)
    pos = np.arange(p0, p0 + T, dtype=np.int32)
    n_ctx = 2048
    oc = orc.Cache.contiguous(kt, n_ctx, HKV, D)
    q_o, gate_o = orc.attn_prep(qg, k, v, qn, kn, pos, oc, p0, T, HQ, HKV, D, n_rot, base, eps)
    c = fast.kv_alloc(kt, n_ctx, HKV, D)
    q = torch.zeros(T, HQ, D, device=cuda)
    gate = torch.zeros(T, HQ * D, device=cuda)
    assert fast.attn_prep(util.to_dev(qg, cuda), util.to_dev(k, cuda), util.to_dev(v, cuda), util.to_dev(qn, cuda),
                          util.to_dev(kn, cuda), util.to_dev(pos, cuda), q, gate, c, p0, T, HQ, HKV, D, n_rot, base, eps)
    torch.cuda.synchronize()
    assert np.array_equal(gate.cpu().numpy(), gate_o)
    # host and device powf differ in the last ulp, which the position multiplies: the reference's own rotary test
    # allows 2e-4 + 1.2e-7 * pos (tests/mrope_test.cu:62-169)
    np.testing.assert_allclose(q.cpu().numpy(), q_o, rtol=1e-5, atol=2e-4 + 1.2e-7 * (p0 + T))
    assert np.array_equal(c.v.cpu().numpy(), oc.v)          # V: no libm on the way, bit-exact
    kb, ko = c.k.cpu().numpy(), oc.k
    assert (kb != ko).mean() < 1e-2
    rowb = orc.row_bytes(kt, HKV, D)
    hb = rowb // HKV
    for t in range(T):
        for h in range(HKV):
            o = (p0 + t) * rowb + h * hb
            a = orc.dequant_head(kt, kb[o:o + hb], D)
            b = orc.dequant_head(kt, ko[o:o + hb], D)
            step = {"f16": 1e-3, "q8_0": 1.0 / 127, "q4_0": 1.0 / 7}[tname] * np.abs(b).max()
            assert np.abs(a - b).max() <= 1.01 * step


def test_rope_append_bf16_vs_oracle(cuda, lib):
    """prefill form: bf16 K/V, rotation only; bytes against the oracle fed with the widened values"""
    import torch
    from p100e_engine_b200 import fast
    T, p0, n_rot, base = 300, 0, 64, 1e7
    kt = TYPES["q8_0"]
    q = torch.from_numpy(util.rng_normal(60, (T, HQ, D))).to(torch.bfloat16)
    k = torch.from_numpy(util.rng_normal(61, (T, HKV, D))).to(torch.bfloat16)
    v = torch.from_numpy(util.rng_normal(62, (T, HKV, D))).to(torch.bfloat16)
    pos = np.arange(p0, p0 + T, dtype=np.int32)
    kr = orc.rope_neox(k.float().numpy(), pos, n_rot, base)
    qr = orc.rope_neox(q.float().numpy(), pos, n_rot, base)
    oc = orc.Cache.contiguous(kt, 512, HKV, D)
    orc.kv_append(oc, kr, v.float().numpy(), p0, T)
    c = fast.kv_alloc(kt, 512, HKV, D)
    q_out = torch.zeros(T, HQ, D, device=cuda)
    assert fast.rope_append_bf16(q.to(cuda), k.to(cuda), v.to(cuda), q_out, c, p0, T, HQ, HKV, D, n_rot, base)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    assert np.array_equal(c.v.cpu().numpy(), oc.v)
    assert (c.k.cpu().numpy() != oc.k).mean() < 1e-2
    np.testing.assert_allclose(q_out.cpu().numpy(), qr, rtol=1e-5, atol=2e-4 + 1.2e-7 * (p0 + T))


@pytest.mark.parametrize("tname", ["f16", "q8_0", "q4_0"])
def test_rope_append_bf16_row_kernel_equals_head_kernel(cuda, lib, tname):
    """16-byte aligned inputs are read with 16-byte loads, inputs shifted by one element value by value: the cache bytes
    and the rotated q must be identical"""
    import torch
    from p100e_engine_b200 import fast
    T, p0, n_rot, base = 257, 1000, 64, 1e7
    kt = TYPES[tname]
    outs = []
    for shift in (0, 1):
        bufs = []
        for seed, heads in ((70, HQ), (71, HKV), (72, HKV)):
            x = torch.from_numpy(util.rng_normal(seed, (T, heads, D))).to(torch.bfloat16)
            flat = torch.zeros(x.numel() + 8, dtype=torch.bfloat16, device=cuda)
            flat[shift:shift + x.numel()] = x.reshape(-1).to(cuda)
            bufs.append(flat[shift:shift + x.numel()].view(T, heads, D))
        assert (bufs[0].data_ptr() % 16 == 0) == (shift == 0)
        c = fast.kv_alloc(kt, 2048, HKV, D)
        q_out = torch.zeros(T, HQ, D, device=cuda)
        assert fast.rope_append_bf16(bufs[0], bufs[1], bufs[2], q_out, c, p0, T, HQ, HKV, D, n_rot, base)
        torch.cuda.synchronize()
        assert fast.device_status() == 0
        rowb = orc.row_bytes(kt, HKV, D)   # only the appended rows are defined
        rows = slice(p0 * rowb, (p0 + T) * rowb)
        outs.append((c.k.cpu().numpy().reshape(-1)[rows].copy(), c.v.cpu().numpy().reshape(-1)[rows].copy(), q_out.cpu().numpy().copy()))
    for a, b in zip(outs[0], outs[1]):
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8))
