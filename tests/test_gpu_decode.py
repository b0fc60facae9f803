"""Decode / MTP-verify attention on the GPU against the CPU oracle (fp64) and the reference's own kernels, restating
the reference tests: tests/fast_attn_test.cu:130-295 (depths, T = 1..4, three cache types, device p0),
tests/fast_tinv_test.cu (row t of a T-row call == the 1-row call, bitwise), tests/fast_sessions_test.cu:130-230
(paged == contiguous, per-row sequences)."""
import ctypes as C

import numpy as np
import pytest

from oracle import orc
from tests import util
from tests.util import D, HKV, HQ, SCALE, TYPES

pytestmark = pytest.mark.gpu


def _filled(kt, n, cuda, seed=7, hkv=HKV):
    """contiguous cache of n positions filled through kv_append on the device + its host mirror for the oracle"""
    import torch
    from p100e_engine_b200 import fast
    k = util.rng_normal(seed, (n, hkv, D))
    v = util.rng_normal(seed + 1, (n, hkv, D))
    c = fast.kv_alloc(kt, n, hkv, D)
    for p in range(0, n, 4096):
        T = min(4096, n - p)
        assert fast.kv_append(c, util.to_dev(k[p:p + T], cuda), util.to_dev(v[p:p + T], cuda), p, T)
    torch.cuda.synchronize()
    oc = orc.Cache(kt, n, hkv, D, c.k.cpu().numpy(), c.v.cpu().numpy())
    return c, oc


@pytest.mark.parametrize("tname", ["q8_0", "f16", "q4_0"])
def test_decode_vs_oracle_depths(cuda, lib, tname):
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    n = 4500
    c, oc = _filled(kt, n, cuda)
    q = util.rng_normal(11, (4, HQ, D)) * 1.5
    qd = util.to_dev(q, cuda)
    out = torch.zeros(4, HQ, D, device=cuda)
    for T in (1, 2, 3, 4):
        for p0 in (0, 1, 31, 63, 64, 127, 128, 255, 256, 257, 511, 512, 600, 1023, 1024, 4095, 4096, n - T):
            if p0 + T > n:
                continue
            out.fill_(float("nan"))
            assert fast.attn_decode(qd, c, out, T, p0, HQ, SCALE)
            torch.cuda.synchronize()
            ref = orc.attention(q[:T], oc, T, HQ, SCALE, p0=p0)
            util.check_close(out[:T].cpu().numpy(), ref, "%s T=%d p0=%d" % (tname, T, p0))
    assert fast.device_status() == 0


@pytest.mark.parametrize("tname", ["q8_0", "f16", "q4_0"])
def test_one_kv_head_shard_vs_oracle(cuda, lib, tname):
    """the shape one GPU of a 4- or 8-GPU run holds: a single kv head (rows of 272 / 512 / 144 bytes), 6 query heads"""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    n, hq = 1500, 6
    c, oc = _filled(kt, n, cuda, seed=31, hkv=1)
    q = util.rng_normal(33, (4, hq, D))
    qd = util.to_dev(q, cuda)
    out = torch.zeros(4, hq, D, device=cuda)
    for T in (1, 4):
        for p0 in (0, 63, 64, 700, n - T):
            out.fill_(float("nan"))
            assert fast.attn_decode(qd, c, out, T, p0, hq, SCALE)
            torch.cuda.synchronize()
            ref = orc.attention(q[:T], oc, T, hq, SCALE, p0=p0)
            util.check_close(out[:T].cpu().numpy(), ref, "%s one head T=%d p0=%d" % (tname, T, p0))
    assert fast.device_status() == 0


@pytest.mark.parametrize("tname", ["q8_0", "f16", "q4_0"])
def test_decode_config1_vs_oracle_and_reference(cuda, lib, tname):
    """Single-sequence decode shape: one slot, q_len 1, context 4096, 16 pages of 256 in a seeded permutation, sigmoid gate;
    also against the reference's attn_decode on the same paged cache"""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    n = 4096
    pool = util.PagedPool(kt, 16, psh=8, seed=1)
    pt = pool.take(n, 16)
    k = util.rng_normal(21, (n, HKV, D))
    v = util.rng_normal(22, (n, HKV, D))
    q = util.rng_normal(23, (1, HQ, D))
    gate = util.rng_normal(24, (1, HQ * D))
    pool_t = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    pt_t = util.to_dev(pt, cuda)
    dc = util.dev_cache(pool_t, pool, pt_t, None, n)
    assert fast.kv_append(dc, util.to_dev(k, cuda), util.to_dev(v, cuda), 0, n)
    torch.cuda.synchronize()
    pool.host[:pool.bytes] = pool_t.cpu().numpy()
    hc = pool.host_cache(pt)
    ref = orc.attention(q, hc, 1, HQ, SCALE, p0=n - 1)
    out = torch.zeros(1, HQ, D, device=cuda)
    qd = util.to_dev(q, cuda)
    assert fast.attn_decode(qd, dc, out, 1, n - 1, HQ, SCALE)
    torch.cuda.synchronize()
    util.check_close(out.cpu().numpy(), ref, "config 1 " + tname)
    # fused gate through the batched entry point
    pos = torch.tensor([n - 1], dtype=torch.int32, device=cuda)
    outg = torch.zeros(1, HQ, D, device=cuda)
    assert fast.attn_decode_slots(qd, dc, outg, util.to_dev(gate, cuda), 1, 1, pos, n, HQ, SCALE)
    torch.cuda.synchronize()
    refg = orc.attention(q, hc, 1, HQ, SCALE, p0=n - 1, gate=gate)
    util.check_close(outg.cpu().numpy(), refg, "config 1 gated " + tname)
    r = orc.p100e_ref()
    if r is not None:
        outr = torch.zeros(1, HQ, D, device=cuda)
        rc = util.orc_kv_of(dc)
        assert r.ref_attn_decode(qd.data_ptr(), C.byref(rc), outr.data_ptr(), 1, n - 1, HQ, SCALE, None) == 0
        torch.cuda.synchronize()
        util.check_close(out.cpu().numpy(), outr.cpu().numpy(), "config 1 vs reference kernel " + tname)
        util.check_close(outr.cpu().numpy(), ref, "reference kernel vs oracle " + tname)
    assert fast.device_status() == 0


@pytest.mark.parametrize("tname", ["q8_0", "f16", "q4_0"])
def test_t_invariance_and_device_p0(cuda, lib, tname):
    """row t of a T-row call is bitwise the 1-row call at p0 + t; device-p0 calls are bitwise the host-p0 calls
    (reference tests/fast_attn_test.cu:130-204, tests/fast_tinv_test.cu:41-61)"""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    n = 2200
    c, _ = _filled(kt, n, cuda, seed=31)
    q = util.to_dev(util.rng_normal(32, (4, HQ, D)), cuda)
    out4 = torch.zeros(4, HQ, D, device=cuda)
    out1 = torch.zeros(1, HQ, D, device=cuda)
    outd = torch.zeros(4, HQ, D, device=cuda)
    p0_dev = torch.zeros(1, dtype=torch.int32, device=cuda)
    for T in (2, 3, 4):
        for p0 in (0, 5, 61, 62, 63, 64, 509, 510, 511, 512, 1023, 1500, n - T):
            assert fast.attn_decode(q, c, out4, T, p0, HQ, SCALE)
            p0_dev.fill_(p0)
            assert fast.attn_decode_dev(q, c, outd, T, p0_dev, n, HQ, SCALE)
            torch.cuda.synchronize()
            assert torch.equal(out4[:T], outd[:T]), "device p0 differs (T=%d p0=%d)" % (T, p0)
            for t in range(T):
                assert fast.attn_decode(q[t:t + 1], c, out1, 1, p0 + t, HQ, SCALE)
                torch.cuda.synchronize()
                assert torch.equal(out1[0], out4[t]), "row %d of T=%d at p0=%d differs from the 1-row call" % (t, T, p0)
    assert fast.device_status() == 0


@pytest.mark.parametrize("tname", ["q8_0", "f16", "q4_0"])
@pytest.mark.parametrize("interleave", [False, True])
def test_paged_equals_contiguous_and_rows(cuda, lib, tname, interleave):
    """three sequences in a shared pool (random page permutation, other layers in between): decode T = 1..4 bitwise
    equal to the contiguous cache; attn_decode_rows over rows of different sequences == per-row calls"""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    Hkv, Hq = 2, 12
    lens = [700, 3000, 300]
    maxp = 16
    pool = util.PagedPool(kt, 24, psh=8, hkv=Hkv, n_layers=2, layer=1, interleave=interleave, seed=9)
    pts = np.stack([pool.take(n, maxp) for n in lens])
    pool_t = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    pt_t = util.to_dev(pts.reshape(-1), cuda)
    cont, paged = [], []
    for s, n in enumerate(lens):
        k = util.to_dev(util.rng_normal(40 + s, (n, Hkv, D)), cuda)
        v = util.to_dev(util.rng_normal(50 + s, (n, Hkv, D)), cuda)
        cc = fast.kv_alloc(kt, maxp << 8, Hkv, D)
        pc = util.dev_cache(pool_t, pool, pt_t[s * maxp:(s + 1) * maxp], None, maxp << 8)
        assert fast.kv_append(cc, k, v, 0, n) and fast.kv_append(pc, k, v, 0, n)
        cont.append(cc)
        paged.append(pc)
    q = util.to_dev(util.rng_normal(60, (8, Hq, D)), cuda)
    o1 = torch.zeros(8, Hq, D, device=cuda)
    o2 = torch.zeros(8, Hq, D, device=cuda)
    for s, n in enumerate(lens):
        for T in (1, 2, 3, 4):
            for p0 in (0, 1, 255, 256, 257, 511, 600, 2047, 2048, n - T):
                if p0 < 0 or p0 + T > n:
                    continue
                assert fast.attn_decode(q, cont[s], o1, T, p0, Hq, SCALE)
                assert fast.attn_decode(q, paged[s], o2, T, p0, Hq, SCALE)
                torch.cuda.synchronize()
                assert torch.equal(o1[:T], o2[:T]), "paged differs (seq %d T=%d p0=%d)" % (s, T, p0)
    # rows of different sequences in one call
    rows = [(0, 699), (1, 2999), (2, 0), (1, 1234), (0, 255), (2, 299), (1, 256), (0, 1)]
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device=cuda)
    rtab = torch.tensor([s * maxp for s, _ in rows], dtype=torch.int32, device=cuda)
    allc = util.dev_cache(pool_t, pool, pt_t, rtab, maxp << 8)
    assert fast.attn_decode_rows(q, allc, o1, 8, pos, Hq, SCALE)
    torch.cuda.synchronize()
    for i, (s, p) in enumerate(rows):
        assert fast.attn_decode(q[i:i + 1], paged[s], o2[:1], 1, p, Hq, SCALE)
        torch.cuda.synchronize()
        assert torch.equal(o1[i], o2[0]), "row %d (seq %d pos %d) differs from its own call" % (i, s, p)
    assert fast.device_status() == 0


@pytest.mark.parametrize("tname", ["q8_0", "f16", "q4_0"])
def test_small_pages_take_the_row_copies(cuda, lib, tname):
    """pages of 16 rows cannot hold a 64-row box, so such a pool is staged row by row through registers instead of by
    tiled copies: the result must equal the contiguous cache (tiled copies) bitwise"""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    Hkv, Hq, n, psh, maxp = 2, 12, 1000, 4, 64
    pool = util.PagedPool(kt, 80, psh=psh, hkv=Hkv, seed=21)
    pt_t = util.to_dev(pool.take(n, maxp), cuda)
    pool_t = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    k = util.to_dev(util.rng_normal(81, (n, Hkv, D)), cuda)
    v = util.to_dev(util.rng_normal(82, (n, Hkv, D)), cuda)
    cc = fast.kv_alloc(kt, maxp << psh, Hkv, D)
    pc = util.dev_cache(pool_t, pool, pt_t, None, maxp << psh)
    assert fast.kv_append(cc, k, v, 0, n) and fast.kv_append(pc, k, v, 0, n)
    q = util.to_dev(util.rng_normal(83, (4, Hq, D)), cuda)
    o1 = torch.zeros(4, Hq, D, device=cuda)
    o2 = torch.zeros(4, Hq, D, device=cuda)
    for T in (1, 4):
        for p0 in (0, 15, 16, 63, 64, 500, n - T):
            assert fast.attn_decode(q, cc, o1, T, p0, Hq, SCALE)
            assert fast.attn_decode(q, pc, o2, T, p0, Hq, SCALE)
            torch.cuda.synchronize()
            assert torch.equal(o1[:T], o2[:T]), "small pages differ (T=%d p0=%d)" % (T, p0)
    assert fast.device_status() == 0


def _verify_batch(cuda, kt, n_slots, q_len, lens, seed, chunk_keys, gate_on=True, psh=8):
    """config-2 style batch: slots with their own contexts in a shared pool; returns (got, oracle)"""
    import torch
    from p100e_engine_b200 import fast
    pg = 1 << psh
    maxp = (max(lens) + pg - 1) // pg
    total = sum((n + pg - 1) // pg for n in lens)
    pool = util.PagedPool(kt, total + 3, psh=psh, seed=seed)
    pts = np.stack([pool.take(n, maxp) for n in lens])
    pool_t = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    pt_t = util.to_dev(pts.reshape(-1), cuda)
    for s, n in enumerate(lens):
        k = util.to_dev(util.rng_normal(seed * 100 + 2 * s, (n, HKV, D)), cuda)
        v = util.to_dev(util.rng_normal(seed * 100 + 2 * s + 1, (n, HKV, D)), cuda)
        pc = util.dev_cache(pool_t, pool, pt_t[s * maxp:(s + 1) * maxp], None, maxp << psh)
        for p in range(0, n, 8192):
            T = min(8192, n - p)
            assert fast.kv_append(pc, k[p:p + T], v[p:p + T], p, T)
    torch.cuda.synchronize()
    pool.host[:pool.bytes] = pool_t.cpu().numpy()
    rows = n_slots * q_len
    pos = np.array([lens[s] - q_len + j for s in range(n_slots) for j in range(q_len)], np.int32)
    rtab = np.array([s * maxp for s in range(n_slots) for _ in range(q_len)], np.int32)
    q = util.rng_normal(seed + 1, (rows, HQ, D))
    gate = util.rng_normal(seed + 2, (rows, HQ * D)) if gate_on else None
    c = util.dev_cache(pool_t, pool, pt_t, util.to_dev(rtab, cuda), maxp << psh)
    out = torch.zeros(rows, HQ, D, device=cuda)
    assert fast.attn_decode_slots(util.to_dev(q, cuda), c, out, None if gate is None else util.to_dev(gate, cuda), n_slots,
                                  q_len, util.to_dev(pos, cuda), max(lens), HQ, SCALE, chunk_keys)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    hc = pool.host_cache(pts.reshape(-1), rtab, maxp << psh)
    ref = orc.attention(q, hc, rows, HQ, SCALE, pos=pos, gate=gate)
    return out.cpu().numpy(), ref, (q, gate, pos, rtab, c, pool, pool_t, pt_t)


@pytest.mark.parametrize("tname", ["q8_0", "f16", "q4_0"])
@pytest.mark.parametrize("chunk", [0, 256, -1])
def test_verify_batch_vs_oracle(cuda, lib, tname, chunk):
    """MTP-verify batch shape at oracle-friendly sizes: 8 slots x q_len 4, ragged contexts, shared pool, gate"""
    lens = [1024, 3000, 257, 4, 640, 2049, 1500, 511]
    got, ref, _ = _verify_batch(cuda, TYPES[tname], 8, 4, lens, 3, chunk)
    util.check_close(got, ref, "verify batch %s chunk=%d" % (tname, chunk))


@pytest.mark.parametrize("tname", ["q8_0"])
@pytest.mark.parametrize("q_len", [2, 3, 4])
def test_even_split_kernels_agree(cuda, lib, tname, q_len):
    """the even split runs q8_0 verify batches (two to four rows per slot) on the tcgen05 kernel; the mma.sync kernel
    (set_tc(0)) must give the same result within the tolerance, and both must match the oracle, for every row count and
    ragged contexts"""
    lens = [5000, 130, 64, 4, 2049, 767, 128, 1]
    lens = [max(n, q_len) for n in lens]
    assert lib.b200_attn_dec_tc() == 1
    got_tc, ref, _ = _verify_batch(cuda, TYPES[tname], len(lens), q_len, lens, 11 + q_len, -1)
    try:
        lib.b200_attn_dec_set_tc(0)
        assert lib.b200_attn_dec_tc() == 0
        got_mma, _, _ = _verify_batch(cuda, TYPES[tname], len(lens), q_len, lens, 11 + q_len, -1)
    finally:
        lib.b200_attn_dec_set_tc(1)
    util.check_close(got_tc, ref, "even split, tcgen05 kernel (%s, q_len %d)" % (tname, q_len))
    util.check_close(got_mma, ref, "even split, mma.sync kernel (%s, q_len %d)" % (tname, q_len))
    util.check_close(got_tc, got_mma, "tcgen05 vs mma.sync (%s, q_len %d)" % (tname, q_len))


def test_even_split_64_row_pages_and_long_page_lists(cuda, lib):
    """the tcgen05 kernel fetches 64-position boxes: pages of exactly 64 rows, a run with more pages than the kernel keeps
    in shared memory (a 20,000-key slot = 313 pages), a slot that ends one key into a page"""
    lens = [20000, 300, 65, 4097]
    got, ref, _ = _verify_batch(cuda, TYPES["q8_0"], len(lens), 4, lens, 23, -1, psh=6)
    util.check_close(got, ref, "even split, 64-row pages")


def test_even_split_many_short_slots(cuda, lib):
    """a wide batch of short sequences: every CTA of the tcgen05 kernel walks many one- and two-tile runs, so the staging
    ring, the tensor-memory buffers and the barrier phases carry over from run to run dozens of times"""
    rng = np.random.default_rng(31)
    lens = [int(x) for x in rng.integers(3, 400, size=150)]
    got, ref, _ = _verify_batch(cuda, TYPES["q8_0"], len(lens), 3, lens, 29, -1)
    util.check_close(got, ref, "even split, 150 short slots")


def test_split_plan_is_shared_inside_a_declared_step(cuda, lib):
    """between attn_step_begin(positions) and step_end the batched calls of one shape launch the split kernel once; the
    results are the same bits; a call of another shape, a position array outside the declared one, or step_end bring
    the per-call split back"""
    import torch
    from p100e_engine_b200 import fast
    lens = [1500, 300, 2049, 77, 900]
    q_len = 4
    got, ref, (q, gate, pos, rtab, c, pool, pool_t, pt_t) = _verify_batch(cuda, TYPES["q8_0"], len(lens), q_len, lens, 41, -1)
    util.check_close(got, ref, "reference call")
    qd, gd, pos_t = util.to_dev(q, cuda), util.to_dev(gate, cuda), util.to_dev(pos, cuda)
    out = torch.zeros(len(lens) * q_len, HQ, D, device=cuda)

    def call(p=pos_t, ql=q_len, n=len(lens)):
        n0 = lib.b200_launch_count()
        assert fast.attn_decode_slots(qd[:n * ql], c, out[:n * ql], gd[:n * ql], n, ql, p, max(lens), HQ, SCALE, -1)
        torch.cuda.synchronize()
        assert fast.device_status() == 0
        return lib.b200_launch_count() - n0

    assert call() == 3                        # no step declared: split + attention + merge
    assert fast.attn_step_begin(pos_t)
    try:
        assert call() == 3 and np.array_equal(out.cpu().numpy(), got)
        assert call() == 2 and np.array_equal(out.cpu().numpy(), got)      # the split of the first call serves the second
        assert call() == 2
        other = pos_t.clone()
        assert call(other) == 3               # positions outside the declared array
        assert call() == 3                    # that call took the scratch: the plan is computed again ...
        assert call() == 2                    # ... and shared from then on
        assert fast.attn_step_begin(pos_t)    # a new step
        assert call() == 3 and call() == 2
    finally:
        assert fast.attn_step_end()
    assert call() == 3
    assert np.array_equal(out.cpu().numpy(), got)


def test_even_split_contiguous_cache_several_row_groups(cuda, lib):
    """the batched entry point on a contiguous cache: three row groups at different depths of one sequence, chosen split"""
    import torch
    from p100e_engine_b200 import fast
    n, q_len = 5000, 4
    c, oc = _filled(TYPES["q8_0"], n, cuda, seed=91)
    starts = [n - q_len, 1900, 130]
    pos = np.array([s0 + j for s0 in starts for j in range(q_len)], np.int32)
    rows = len(pos)
    q = util.rng_normal(92, (rows, HQ, D))
    out = torch.zeros(rows, HQ, D, device=cuda)
    assert fast.attn_decode_slots(util.to_dev(q, cuda), c, out, None, len(starts), q_len, util.to_dev(pos, cuda), n, HQ, SCALE, -1)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    ref = orc.attention(q, oc, rows, HQ, SCALE, pos=pos)
    util.check_close(out.cpu().numpy(), ref, "even split, contiguous cache")


def test_slot_rows_independent_of_batch(cuda, lib):
    """a slot's rows are bitwise the same whether it is decoded alone or inside a batch (same chunk)"""
    import torch
    from p100e_engine_b200 import fast
    lens = [900, 2500, 300]
    got, _, (q, gate, pos, rtab, c, pool, pool_t, pt_t) = _verify_batch(cuda, TYPES["q8_0"], 3, 4, lens, 4, 512)
    maxp = (max(lens) + 255) // 256
    for s in range(3):
        sl = slice(4 * s, 4 * s + 4)
        cs = util.dev_cache(pool_t, pool, pt_t[s * maxp:(s + 1) * maxp], None, maxp << 8)
        out = torch.zeros(4, HQ, D, device=cuda)
        assert fast.attn_decode_slots(util.to_dev(q[sl], cuda), cs, out, util.to_dev(gate[sl], cuda), 1, 4,
                                      util.to_dev(pos[sl], cuda), lens[s], HQ, SCALE, 512)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), got[sl])


@pytest.mark.parametrize("tname", ["q8_0", "q4_0"])
def test_partial_and_merge_two_sequence_shards(cuda, lib, tname):
    """sequence split as used across two GPUs: each shard attends to its own pages, the (O, m, l) partials are merged in
    shard order with the gate; equals the unsplit result and the oracle's merge"""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    n, q_len = 3000, 4
    c, oc = _filled(kt, n, cuda, seed=71)
    q = util.rng_normal(72, (q_len, HQ, D))
    gate = util.rng_normal(73, (q_len, HQ * D))
    pos = np.arange(n - q_len, n, dtype=np.int32)
    rowb = orc.row_bytes(kt, HKV, D)
    # shard r owns pages r, r+2, ... of 256 positions: build its compacted local cache and local positions
    po = torch.zeros(2, q_len, HQ, D, device=cuda)
    pm = torch.zeros(2, q_len, HQ, device=cuda)
    pl = torch.zeros(2, q_len, HQ, device=cuda)
    kh, vh = c.k.cpu().numpy().reshape(n, rowb), c.v.cpu().numpy().reshape(n, rowb)
    for r in range(2):
        own = np.array([p for p in range(n) if (p >> 8) % 2 == r])
        lk, lv = util.to_dev(kh[own].reshape(-1), cuda), util.to_dev(vh[own].reshape(-1), cuda)
        lc = fast.kv_cache(kt, len(own), HKV, D, lk, lv)
        lpos = np.array([np.searchsorted(own, p, side="right") - 1 for p in pos], np.int32)
        assert fast.attn_decode_slots_partial(util.to_dev(q, cuda), lc, po[r], pm[r], pl[r], 1, q_len,
                                              util.to_dev(lpos, cuda), len(own), HQ, SCALE)
    out = torch.zeros(q_len, HQ, D, device=cuda)
    R = q_len * HQ
    assert fast.attn_merge_gate(po, pm, pl, 2, R, D, util.to_dev(gate, cuda), out)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    ref = orc.attention(q, oc, q_len, HQ, SCALE, pos=pos, gate=gate)
    util.check_close(out.cpu().numpy(), ref, "two-shard merge " + tname)
    om = orc.merge(po.cpu().numpy().reshape(2, R, D), pm.cpu().numpy().reshape(2, R), pl.cpu().numpy().reshape(2, R),
                   gate.reshape(R, D))
    util.check_close(out.cpu().numpy().reshape(R, D), om, "merge kernel vs oracle merge", 1e-5, 1e-4)


def test_empty_rows_and_refusals(cuda, lib):
    import torch
    from p100e_engine_b200 import fast
    c, _ = _filled(TYPES["q8_0"], 300, cuda, seed=81)
    q = util.to_dev(util.rng_normal(82, (2, HQ, D)), cuda)
    out = torch.full((2, HQ, D), 7.0, device=cuda)
    pos = torch.tensor([-1, 5], dtype=torch.int32, device=cuda)
    assert fast.attn_decode_slots(q, c, out, None, 2, 1, pos, 300, HQ, SCALE)
    torch.cuda.synchronize()
    assert (out[0] == 0).all() and torch.isfinite(out[1]).all() and (out[1] != 7.0).any()
    # unsupported shapes are refused with nothing launched (reference: attn.cuh:40-43)
    n0 = lib.b200_launch_count()
    assert not fast.attn_decode(q, c, out, 9, 0, HQ, SCALE)
    assert not fast.attn_decode(q, c, out, 1, 0, HQ + 1, SCALE)
    bad = fast.kv_cache(3, 300, HKV, D, c.k, c.v)
    assert not fast.attn_decode(q, bad, out, 1, 0, HQ, SCALE)
    assert lib.b200_launch_count() == n0
