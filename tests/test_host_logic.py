"""Host-side logic of the path without a GPU: pool layout and page tables, step descriptors, shard plans, local
positions of a sequence split, and the multi-rank exchange + merge over a 2-process gloo group."""
import os
import subprocess
import sys

import numpy as np

from p100e_engine_b200 import dist as Dm
from p100e_engine_b200 import pool as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_pool_layout_matches_reference_engine_layout(lib):
    # [K|V][layer][page][256][row] with pstride = 256 * rowb (reference src/tp_model.cu:3934-3942)
    pl = P.Pool(8, 4, 16, 100, 8, max_slots=2, max_pages=4, max_rows=8)
    assert pl.rowb == 1088 and pl.pstride == 256 * 1088
    assert pl.total_bytes == 2 * 16 * 100 * pl.pstride
    assert pl.page_bytes == 2 * 16 * pl.pstride           # offload block of one page: [K|V][layer][256 rows]
    base = pl.base()
    c3, c0 = pl.view(3, 0), pl.view(0, -1)
    assert c3.k - base == 3 * 100 * pl.pstride and c3.v - base == (16 + 3) * 100 * pl.pstride
    assert c0.v - base == 16 * 100 * pl.pstride and c0.pstride == pl.pstride and c0.psh == 8
    assert c3.rtab is None and c0.rtab is not None        # kv_seq: the slot's own table row; kv_rows: per-row offsets
    assert c3.n_ctx == 4 * 256 and (c3.type, c3.Hkv, c3.D) == (8, 4, 256)
    assert P.row_bytes(1, 4) == 2048 and P.row_bytes(2, 4) == 576
    pl.close()


def test_page_table_and_descriptor(lib):
    from p100e_engine_b200 import lib as L
    tb = P.Pool(8, 1, 1, 10, 8, max_slots=3, max_pages=4, max_rows=16, seed=1)
    assert tb.ensure(0, 700) == L.OK and tb.slot_pages(0) == 3
    assert tb.ensure(1, 1024) == L.OK and tb.slot_pages(1) == 4
    assert tb.ensure(2, 1025) == L.ERR_SHAPE and tb.slot_pages(2) == 0      # more pages than a slot may hold
    assert tb.ensure(2, 512) == L.OK
    tab = tb.table()
    used = tab[tab >= 0]
    assert len(set(used.tolist())) == len(used) == 9 and tb.free_pages() == 1
    assert tb.ensure(0, 1024) == L.OK and tb.free_pages() == 0
    assert tb.ensure(2, 700) == L.ERR_ALLOC and tb.slot_pages(2) == 2       # pool full: nothing changes
    assert tb.release(1) == L.OK
    assert (tb.table()[1] == -1).all() and tb.free_pages() == 4
    assert tb.step([2, 0], [500, 10], 4, grow=False) == L.OK
    pos, last, crow, rtab = tb.step_host()
    assert pos.tolist() == [500, 501, 502, 503, 10, 11, 12, 13]
    assert last.tolist() == pos.tolist() and crow.tolist() == pos.tolist()   # one shard: local == global
    assert rtab.tolist() == [8, 8, 8, 8, 0, 0, 0, 0]
    assert tb.step_rows() == 8 and tb.step_max_n() == 504
    assert tb.step([0] * 5, [0] * 5, 4, grow=False) == L.ERR_SHAPE           # 20 rows > max_rows
    tb.close()


def test_local_positions_sequence_split(lib):
    for n_seq in (1, 2, 4):
        pools = [P.Pool(8, 1, 1, 64, 8, max_slots=1, max_pages=32, max_rows=4, n_seq=n_seq, seq_rank=r) for r in range(n_seq)]
        for n in (1, 5, 255, 256, 257, 511, 512, 513, 1000, 4096):
            owner = (np.arange(n) >> 8) % n_seq
            tot = 0
            for r in range(n_seq):
                own = np.nonzero(owner == r)[0]
                assert Dm.seq_local_length(n, n_seq, r) == len(own) == pools[r].local_length(n)
                tot += len(own)
                ps = [0, n // 2, n - 1]
                assert pools[r].step([0] * 3, ps, 1, grow=False) == 0
                _, last, crow, _ = pools[r].step_host()
                for i, p in enumerate(ps):
                    want = np.searchsorted(own, p, side="right") - 1
                    assert Dm.seq_local_positions([p], n_seq, r)[0] == want == last[i]
                    assert crow[i] == (want if owner[p] == r else -1)      # the row's own K/V lands on the owner only
            assert tot == n
        for pl in pools:
            pl.close()
    assert Dm.seq_local_positions([-1], 2, 0)[0] == -1


def test_page_offload_layout_and_restore(lib):
    """pages_out writes [page][K|V][layer][rows] (reference seq_offload, src/tp_model.cu:3462-3466); pages_in into another
    pool with another page placement restores the same logical bytes"""
    rng = np.random.default_rng(5)
    a = P.Pool(8, 2, 3, 12, 5, max_slots=2, max_pages=6, max_rows=4, seed=7)
    assert a.ensure(1, 100) == 0 and a.slot_pages(1) == 4
    a.base_host()[:] = rng.integers(0, 256, a.total_bytes, dtype=np.uint8)
    buf = np.zeros(4 * a.page_bytes, np.uint8)
    assert a.pages_out(1, 0, 4, buf) == 0
    pblk, region, tab = a.pstride, 12 * a.pstride, a.table()[1]
    img = a.base_host()
    for i in range(4):
        for kv in range(2):
            for l in range(3):
                src = img[(kv * 3 + l) * region + tab[i] * pblk:][:pblk]
                dst = buf[i * a.page_bytes + (kv * 3 + l) * pblk:][:pblk]
                assert np.array_equal(src, dst)
    b = P.Pool(8, 2, 3, 9, 5, max_slots=3, max_pages=6, max_rows=4, seed=99)
    assert b.ensure(0, 40) == 0                     # other sequences hold pages already: another placement
    assert b.pages_in(2, 0, 4, buf) == 0 and b.slot_pages(2) == 4
    back = np.zeros_like(buf)
    assert b.pages_out(2, 0, 4, back) == 0
    assert np.array_equal(back, buf)
    assert b.pages_in(2, 5, 1, buf) != 0            # pages arrive in order
    a.close()
    b.close()


def test_sequence_file_round_trip(lib, tmp_path):
    """writer and reader of the reference's sequence file layout (src/tp_model.cu:3688-3695,3738-3862): magic, 15 x u64
    fingerprint, header, tokens, per GPU pages + state; the reader's refusals"""
    from p100e_engine_b200 import lib as L
    rng = np.random.default_rng(11)
    fp = rng.integers(1, 1 << 60, 15, dtype=np.uint64)
    pools = [P.Pool(2, 1, 2, 8, 5, max_slots=2, max_pages=4, max_rows=4, seed=3 + r) for r in range(2)]   # two "GPUs"
    n_past = 70
    toks = rng.integers(0, 1000, n_past).astype(np.int32)
    states = [bytes(rng.integers(0, 256, 13 + r, dtype=np.uint8)) for r in range(2)]
    for pl in pools:
        assert pl.ensure(1, n_past) == 0
        pl.base_host()[:] = rng.integers(0, 256, pl.total_bytes, dtype=np.uint8)
    path = str(tmp_path / "seq.bin")
    fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_TRUNC)
    assert P.session_write(fd, fp, n_past, toks, [(pools[0], 1), (pools[1], 1)], states) == L.OK
    os.close(fd)
    raw = open(path, "rb").read()
    np_pages = pools[0].slot_pages(1)
    assert raw[:8] == b"P100ESQ2" and np.array_equal(np.frombuffer(raw[8:128], np.uint64), fp)
    assert np.frombuffer(raw[128:140], np.int32).tolist() == [n_past, n_past, np_pages]
    assert np.array_equal(np.frombuffer(raw[140:140 + 4 * n_past], np.int32), toks)
    assert len(raw) == 140 + 4 * n_past + sum(np_pages * pl.page_bytes for pl in pools) + 13 + 14
    ref_pages = []
    for pl in pools:
        b = np.zeros(np_pages * pl.page_bytes, np.uint8)
        assert pl.pages_out(1, 0, np_pages, b) == 0
        ref_pages.append(b)
    off = 140 + 4 * n_past
    assert raw[off:off + len(ref_pages[0])] == ref_pages[0].tobytes() and raw[off + len(ref_pages[0]):][:13] == states[0]
    # read into fresh pools
    fresh = [P.Pool(2, 1, 2, 8, 5, max_slots=2, max_pages=4, max_rows=4, seed=50 + r) for r in range(2)]
    fd = os.open(path, os.O_RDONLY)
    rc, got_past, got_toks, got_states, bad = P.session_read(fd, fp, 128, [(fresh[0], 0), (fresh[1], 0)], [13, 14])
    os.close(fd)
    assert rc == L.OK and got_past == n_past and np.array_equal(got_toks, toks) and got_states == states and bad == -1
    for pl, want in zip(fresh, ref_pages):
        b = np.zeros_like(want)
        assert pl.pages_out(0, 0, np_pages, b) == 0 and np.array_equal(b, want)
    # refusals: another fingerprint (field 7 = GPU count / split), an old-format file, a foreign file, a short file
    fp2 = fp.copy()
    fp2[7] += 1
    fd = os.open(path, os.O_RDONLY)
    rc, *_, bad = P.session_read(fd, fp2, 128, [(fresh[0], 1)], [13])
    os.close(fd)
    assert rc == L.ERR_FORMAT and bad == 7
    for blob in (b"P100ESQ1" + raw[8:], b"NOTAFILE" + raw[8:], raw[:100]):
        open(path, "wb").write(blob)
        fd = os.open(path, os.O_RDONLY)
        rc, *_ = P.session_read(fd, fp, 128, [(fresh[0], 1)], [13])
        os.close(fd)
        assert rc == L.ERR_FORMAT
    open(path, "wb").write(raw)
    fd = os.open(path, os.O_RDONLY)
    rc, *_ = P.session_read(fd, fp, 64, [(fresh[0], 1)], [13])      # n_past 70 exceeds this engine's context
    os.close(fd)
    assert rc == L.ERR_FORMAT
    for pl in pools + fresh:
        pl.close()


def test_shard_plan():
    for world in (1, 2, 4, 8):
        seen = set()
        for rank in range(world):
            pl = Dm.ShardPlan(world, rank, 4, 6)
            assert pl.hq_local == 6 * pl.hkv_local
            assert pl.n_head_shards * pl.n_seq == world
            seen.add((pl.kv_head0, pl.seq_rank))
            assert rank in pl.merge_group_ranks()
        assert len(seen) == world
    p8 = Dm.ShardPlan(8, 5, 4, 6)
    assert (p8.n_head_shards, p8.n_seq, p8.head_rank, p8.seq_rank, p8.hkv_local) == (4, 2, 2, 1, 1)
    assert p8.merge_group_ranks() == [4, 5]
    assert Dm.ShardPlan(8, 0).all_merge_groups() == [[0, 1], [2, 3], [4, 5], [6, 7]]


def test_two_rank_sequence_split_merge_gloo():
    """two CPU ranks (gloo): each computes the oracle's partial over its own pages, all-gathers (O, m, l) and merges in
    rank order; both ranks end with the unsplit result"""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29517", PYTHONPATH=ROOT)
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "gloo_seq_split_worker.py"), str(r), "2"], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
        assert "OK" in o, o


def _run_peer_workers(fail_rank, port):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), PYTHONPATH=ROOT)
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "gloo_peer_merge_worker.py"), str(r), "2", str(fail_rank)],
                              env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
    return outs


def test_peer_merge_host_protocol_gloo():
    """two CPU ranks (gloo), device calls recorded instead of made: the shards map each other's buffers in shard order,
    alternate the two partial buffers, count the calls alike; when one shard cannot map its peer, both give up"""
    for o in _run_peer_workers(-1, 29518):
        assert "OK" in o, o
    for o in _run_peer_workers(1, 29519):
        assert "REFUSED" in o, o
