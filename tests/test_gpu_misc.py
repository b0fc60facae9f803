"""Further GPU parity cases: interleaved M-RoPE in attn_prep (reference tests/mrope_test.cu:62-117), the gate / a16
epilogue (tests/fast_fusion_test.cu:161-178, tests/fast_fused_test.cu:100), offsets beyond 4 GiB (the reference's 32-bit
limit, src/fast/attn_dec2.cu:495), the long-context q4_0 batch at full size (16 slots x 131072 keys, q4_0), and the two-GPU
sequence split through NCCL when two GPUs are present."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import orc
from tests import util
from tests.util import D, HKV, HQ, SCALE, TYPES

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("tname", ["q8_0", "q4_0", "f16"])
def test_attn_prep_mrope_matches_reference(cuda, lib, tname):
    import torch
    from p100e_engine_b200 import fast
    ref = orc.p100e_ref()
    if ref is None:
        pytest.skip("reference kernels not prebuilt")
    kt = TYPES[tname]
    Hq, Hkv, n_rot, base, eps, n_ctx, stride, T = 12, 2, 64, 1e7, 1e-6, 512, 64, 24
    P0, nx = 40, 6      # image rows: t = P, h = P + i / nx, w = P + i % nx
    mp = np.zeros((3, stride), np.int32)
    i = np.arange(T)
    mp[0, :T], mp[1, :T], mp[2, :T] = P0, P0 + i // nx, P0 + i % nx
    rows = np.arange(300, 300 + T, dtype=np.int32)     # cache rows differ from the rotary positions
    rng = np.random.default_rng(3)
    qg = util.to_dev(util.rng_normal(1, (T, Hq, 2 * D)), cuda)
    k = util.to_dev(util.rng_normal(2, (T, Hkv, D)), cuda)
    v = util.to_dev(util.rng_normal(3, (T, Hkv, D)), cuda)
    qn = util.to_dev((0.2 + rng.random(D)).astype(np.float32), cuda)
    kn = util.to_dev((0.2 + rng.random(D)).astype(np.float32), cuda)
    pos, mpd = util.to_dev(rows, cuda), util.to_dev(mp, cuda)
    outs = []
    for impl in ("new", "ref"):
        c = fast.kv_alloc(kt, n_ctx, Hkv, D)
        q = torch.zeros(T, Hq, D, device=cuda)
        gate = torch.zeros(T, Hq * D, device=cuda)
        if impl == "new":
            assert fast.attn_prep(qg, k, v, qn, kn, pos, q, gate, c, -1, T, Hq, Hkv, D, n_rot, base, eps,
                                  mr={"p": mpd, "stride": stride, "s0": 11, "s1": 11, "s2": 10, "sect": 32})
        else:
            rc = util.orc_kv_of(c)
            assert ref.ref_attn_prep_mrope(qg.data_ptr(), k.data_ptr(), v.data_ptr(), qn.data_ptr(), kn.data_ptr(), pos.data_ptr(),
                                           q.data_ptr(), gate.data_ptr(), C.byref(rc), -1, T, Hq, Hkv, D, n_rot, base, eps, None,
                                           mpd.data_ptr(), stride, 11, 11, 10, 32) == 0
        torch.cuda.synchronize()
        outs.append((q, gate, c.k.clone(), c.v.clone()))
    for a, b, name in zip(outs[0], outs[1], ("q", "gate", "K bytes", "V bytes")):
        assert torch.equal(a, b), name + " differs from the reference under M-RoPE"


def test_gate_and_a16_epilogue_match_reference(cuda, lib):
    import torch
    from p100e_engine_b200 import fast
    ref = orc.p100e_ref()
    if ref is None:
        pytest.skip("reference kernels not prebuilt")
    T, n = 4, HQ * D
    a = util.to_dev(util.rng_normal(1, (T, n)), cuda)
    b = util.to_dev(util.rng_normal(2, (T, n)) * 3.0, cuda)
    qb = T * (n // 32) * 17 * 4      # 16 half2 per group + one (amax, sum) half2 per group
    for op in (fast.EW_SIGMOID_MUL, fast.EW_SILU_MUL):
        y1, y2 = torch.zeros(T, n, device=cuda), torch.zeros(T, n, device=cuda)
        q1 = torch.zeros(qb, dtype=torch.uint8, device=cuda)
        q2 = torch.zeros(qb, dtype=torch.uint8, device=cuda)
        assert fast.ew_quant(op, a, b, y1, q1, T, n)
        assert ref.ref_ew_quant(op, a.data_ptr(), b.data_ptr(), y2.data_ptr(), q2.data_ptr(), T, n, None) == 0
        torch.cuda.synchronize()
        assert torch.equal(y1, y2) and torch.equal(q1, q2), "ew_quant op %d differs from the reference" % op
    x1, x2 = a.clone(), a.clone()
    assert fast.sigmoid_mul(x1, b, T * n)
    ref.ref_k_sigmoid_mul(x2.data_ptr(), b.data_ptr(), T * n, None)
    torch.cuda.synchronize()
    assert torch.equal(x1, x2)


def test_offsets_beyond_4gib(cuda, lib):
    """a page whose byte offset exceeds 2^32 (the reference refuses such pools): same bits as the same rows placed low"""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES["q8_0"]
    rowb = orc.row_bytes(kt, HKV, D)
    pstride = 256 * rowb
    hi_page = (5 << 30) // pstride + 3                      # > 4 GiB into the K region
    pool_bytes = (hi_page + 1) * pstride
    kpool = torch.empty(pool_bytes, dtype=torch.uint8, device=cuda)
    vpool = torch.empty(pool_bytes, dtype=torch.uint8, device=cuda)
    n = 400
    k = util.to_dev(util.rng_normal(1, (n, HKV, D)), cuda)
    v = util.to_dev(util.rng_normal(2, (n, HKV, D)), cuda)
    q = util.to_dev(util.rng_normal(3, (4, HQ, D)), cuda)
    outs = []
    for pages in ([1, 0], [hi_page, hi_page - 1]):
        pt = torch.tensor(pages, dtype=torch.int32, device=cuda)
        c = fast.kv_cache(kt, 512, HKV, D, kpool, vpool, pt, None, 8, pstride)
        assert fast.kv_append(c, k, v, 0, n)
        out = torch.zeros(4, HQ, D, device=cuda)
        assert fast.attn_decode(q, c, out, 4, n - 4, HQ, SCALE)
        o2 = torch.zeros(4, HQ, D, device=cuda)
        assert fast.attn_prefill(q, c, o2, 4, n - 4, HQ, SCALE)
        torch.cuda.synchronize()
        outs.append((out, o2))
    assert fast.device_status() == 0
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    lo = kpool[pstride:pstride + 256 * rowb]
    hi = kpool[hi_page * pstride:hi_page * pstride + 256 * rowb]
    assert torch.equal(lo, hi)


def test_config4_full_size_q4_0(cuda, lib):
    """Long-context batch: 16 slots x 131072 keys, q4_0, 512 pages per slot in a seeded permutation of an 8192-page pool.
    Two slots are checked against the oracle; all slots through chunk independence (two chunk sizes agree)."""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES["q4_0"]
    slots, n, maxp = 16, 131072, 512
    pool = util.PagedPool(kt, slots * maxp + 8, psh=8, seed=11)
    pts = np.stack([pool.take(n, maxp) for _ in range(slots)])
    pool_t = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    pt_t = util.to_dev(pts.reshape(-1), cuda)
    g = torch.Generator(device="cpu").manual_seed(7)
    for s in range(slots):
        pc = util.dev_cache(pool_t, pool, pt_t[s * maxp:(s + 1) * maxp], None, n)
        for p in range(0, n, 32768):
            kk = torch.randn(32768, HKV, D, generator=g).to(cuda)
            vv = torch.randn(32768, HKV, D, generator=g).to(cuda)
            assert fast.kv_append(pc, kk, vv, p, 32768)
    pos = torch.full((slots,), n - 1, dtype=torch.int32, device=cuda)
    rtab = torch.arange(slots, dtype=torch.int32, device=cuda) * maxp
    q = util.rng_normal(5, (slots, HQ, D))
    qd = util.to_dev(q, cuda)
    c = util.dev_cache(pool_t, pool, pt_t, rtab, n)
    o1 = torch.zeros(slots, HQ, D, device=cuda)
    o2 = torch.zeros(slots, HQ, D, device=cuda)
    assert fast.attn_decode_slots(qd, c, o1, None, slots, 1, pos, n, HQ, SCALE, 2048)
    assert fast.attn_decode_slots(qd, c, o2, None, slots, 1, pos, n, HQ, SCALE, 8192)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    util.check_close(o1.cpu().numpy(), o2.cpu().numpy(), "chunk 2048 vs 8192", 1e-3, 1e-3)
    host = pool_t.cpu().numpy()
    for s in (0, 15):
        hc = orc.Cache(kt, n, HKV, D, host[pool.koff:], host[pool.voff:], pts[s], None, 8, pool.pstride)
        ref = orc.attention(q[s:s + 1], hc, 1, HQ, SCALE, p0=n - 1)
        util.check_close(o1[s:s + 1].cpu().numpy(), ref, "config 4 slot %d vs oracle" % s)


def test_two_gpu_sequence_split_nccl(cuda, lib):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", "29533", os.path.join(ROOT, "tests", "nccl_seq_split_worker.py")],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.count("OK") == 2, r.stdout + r.stderr


def test_peer_merge_on_one_gpu_and_a_wait_that_runs_out(cuda, lib):
    """the peer merge with both "shards" on one GPU: the peer's flag row is written by hand, so the kernel's wait finds
    it set and the merge equals attn_merge_gate over the two parts; then a call whose announcement never comes: the wait
    gives up after its limit, the status word says so, and the context stays usable"""
    import time
    import torch
    from p100e_engine_b200 import fast
    R, Dm = 24, 256
    rng = np.random.default_rng(6)
    part_floats = R * (Dm + 2)
    # one buffer per shard: [partial | flag row of 64 words]
    bufs = [torch.zeros(part_floats + 64, device=cuda) for _ in range(2)]
    po = torch.from_numpy(rng.standard_normal((2, R, Dm)).astype(np.float32)).to(cuda)
    pm = torch.from_numpy(rng.standard_normal((2, R)).astype(np.float32)).to(cuda)
    pl = torch.from_numpy((rng.random((2, R)) + 0.5).astype(np.float32)).to(cuda)
    for s in range(2):
        bufs[s][:part_floats] = torch.cat([po[s].reshape(-1), pm[s], pl[s]])
    gate = torch.from_numpy(rng.standard_normal((R, Dm)).astype(np.float32)).to(cuda)
    parts = [b.data_ptr() for b in bufs]
    flags = [b.data_ptr() + 4 * part_floats for b in bufs]
    want = torch.zeros(R, Dm, device=cuda)
    assert fast.attn_merge_gate(po, pm, pl, 2, R, Dm, gate, want)
    # shard 0's view: shard 1 has announced call 1 (word 1 of shard 0's flag row)
    bufs[0][part_floats:].view(torch.int32)[1] = 1
    out = torch.zeros(R, Dm, device=cuda)
    assert fast.seq_merge_peers(parts, flags, 0, 1, R, Dm, gate, out)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    assert torch.equal(out, want)
    assert int(bufs[1][part_floats:].view(torch.int32)[0]) == 1   # and shard 0 announced itself in shard 1's row
    # call 2 is never announced by shard 1
    t0 = time.time()
    assert fast.seq_merge_peers(parts, flags, 0, 2, R, Dm, gate, out)
    torch.cuda.synchronize()
    assert 1.0 < time.time() - t0 < 30.0
    assert fast.device_status() & 1
    assert fast.attn_merge_gate(po, pm, pl, 2, R, Dm, gate, out)   # the context still works
    torch.cuda.synchronize()
    assert fast.device_status() == 0 and torch.equal(out, want)


def test_seq_exchange_merge_single_shard(cuda, lib):
    """with one sequence shard the exchange entry point needs no communicator: it normalises and gates the flat partial
    exactly as attn_merge_gate does with one part"""
    import torch
    from p100e_engine_b200 import fast
    R, Dm = 24, 256
    rng = np.random.default_rng(5)
    po = torch.from_numpy(rng.standard_normal((R, Dm)).astype(np.float32)).to(cuda)
    pm = torch.from_numpy(rng.standard_normal(R).astype(np.float32)).to(cuda)
    pl = torch.from_numpy((rng.random(R) + 0.5).astype(np.float32)).to(cuda)
    pm[3] = float("-inf")   # a row that saw no key
    pl[3] = 0.0
    gate = torch.from_numpy(rng.standard_normal((R, Dm)).astype(np.float32)).to(cuda)
    send = torch.cat([po.reshape(-1), pm, pl]).contiguous()
    recv = torch.zeros_like(send)
    o1 = torch.zeros(R, Dm, device=cuda)
    o2 = torch.zeros(R, Dm, device=cuda)
    assert fast.attn_merge_gate(po, pm, pl, 1, R, Dm, gate, o1)
    assert fast.seq_exchange_merge(0, 1, send, recv, R, Dm, gate, o2)
    torch.cuda.synchronize()
    assert torch.equal(o1, o2)
    assert torch.all(o2[3] == 0)
    with np.errstate(divide="ignore", invalid="ignore"):
        want = po.cpu().numpy() / pl.cpu().numpy()[:, None] / (1.0 + np.exp(-gate.cpu().numpy()))
    want[3] = 0
    np.testing.assert_allclose(o2.cpu().numpy(), want, rtol=2e-5, atol=1e-6)
    # two shards gathered by the caller (no communicator): the same part twice merges to the same rows
    recv2 = torch.cat([send, send]).contiguous()
    assert fast.seq_exchange_merge(0, 2, send, recv2, R, Dm, gate, o2)
    torch.cuda.synchronize()
    np.testing.assert_allclose(o2.cpu().numpy(), want, rtol=2e-5, atol=1e-6)
