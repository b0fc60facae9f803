"""Host-side logic of the path without a GPU: pool layout and page tables, step descriptors, shard plans, local
positions of a sequence split, and the multi-rank exchange + merge over a 2-process gloo group."""
import os
import subprocess
import sys

import numpy as np

from p100e_engine_b200 import dist as Dm
from p100e_engine_b200 import pool as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_pool_layout_matches_reference_engine_layout():
    # [K|V][layer][page][256][row] with pstride = 256 * rowb (reference src/tp_model.cu:3934-3942)
    lay = P.PoolLayout(8, 4, 16, 100, 8)
    assert lay.rowb == 1088 and lay.pstride == 256 * 1088
    assert lay.k_offset(3) == 3 * 100 * lay.pstride
    assert lay.v_offset(0) == 16 * 100 * lay.pstride
    assert lay.total_bytes == 2 * 16 * 100 * lay.pstride
    assert P.row_bytes(1, 4) == 2048 and P.row_bytes(2, 4) == 576


def test_page_table_and_descriptor():
    tb = P.PageTable(10, 3, 4, 8, seed=1)
    assert tb.ensure_pages(0, 700) and tb.n_alloc[0] == 3
    assert tb.ensure_pages(1, 1024) and tb.n_alloc[1] == 4
    assert not tb.ensure_pages(2, 1025)          # more pages than a slot may hold
    assert tb.ensure_pages(2, 512)
    used = tb.ptab[tb.ptab >= 0]
    assert len(set(used.tolist())) == len(used) == 9
    assert not tb.ensure_pages(0, 1024) or len(tb.free) == 0
    tb.release(1)
    assert (tb.ptab[1] == -1).all() and len(tb.free) >= 4
    pos, rtab = P.step_descriptor([2, 0], [500, 10], 4, 4)
    assert pos.tolist() == [500, 501, 502, 503, 10, 11, 12, 13]
    assert rtab.tolist() == [8, 8, 8, 8, 0, 0, 0, 0]


def test_local_positions_sequence_split():
    for n_seq in (1, 2, 4):
        for n in (1, 5, 255, 256, 257, 511, 512, 513, 1000, 4096):
            owner = (np.arange(n) >> 8) % n_seq
            tot = 0
            for r in range(n_seq):
                own = np.nonzero(owner == r)[0]
                assert P.local_length(n, n_seq, r) == len(own)
                tot += len(own)
                for p in (0, n // 2, n - 1):
                    want = np.searchsorted(own, p, side="right") - 1
                    assert P.local_positions([p], n_seq, r)[0] == want
            assert tot == n
    assert P.local_positions([-1], 2, 0)[0] == -1


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
