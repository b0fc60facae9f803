"""Worker of tests/test_host_logic.py::test_two_rank_sequence_split_merge_gloo (one CPU rank of a gloo group)."""
import sys

import numpy as np
import torch
import torch.distributed as dist

from oracle import orc
from p100e_engine_b200 import dist as Dm
from tests import util


def main():
    rank, world = int(sys.argv[1]), int(sys.argv[2])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    plan = Dm.ShardPlan(world * 4, rank, 4, 6)      # 4 head shards x `world` sequence shards; this worker plays head shard 0
    plan.n_seq, plan.seq_rank = world, rank
    kt, n, q_len, hq, hkv = orc.KV_Q8_0, 1500, 4, 6, 1
    k = util.rng_normal(1, (n, hkv, 256))
    v = util.rng_normal(2, (n, hkv, 256))
    q = util.rng_normal(3, (q_len, hq, 256))
    gate = util.rng_normal(4, (q_len, hq * 256))
    pos = np.arange(n - q_len, n, dtype=np.int32)
    full = orc.Cache.contiguous(kt, n, hkv, 256)
    orc.kv_append(full, k, v, 0, n)
    want = orc.attention(q, full, q_len, hq, util.SCALE, pos=pos, gate=gate)
    own = np.nonzero((np.arange(n) >> 8) % world == rank)[0]
    loc = orc.Cache.contiguous(kt, len(own), hkv, 256)
    orc.kv_append(loc, k[own], v[own], 0, len(own))
    lpos = plan.local_positions(pos)
    _, oacc, om, ol = orc.attention(q, loc, q_len, hq, util.SCALE, pos=lpos, partial=True)
    R = q_len * hq
    send = torch.from_numpy(np.concatenate([oacc.reshape(-1), om.reshape(-1), ol.reshape(-1)]))
    recv = [torch.zeros_like(send) for _ in range(world)]
    dist.all_gather(recv, send)
    parts = [r.numpy() for r in recv]
    po = np.stack([p[:R * 256].reshape(R, 256) for p in parts])
    pm = np.stack([p[R * 256:R * 256 + R] for p in parts])
    pl = np.stack([p[R * 256 + R:] for p in parts])
    got = orc.merge(po, pm, pl, gate.reshape(R, 256)).reshape(q_len, hq, 256)
    util.check_close(got, want, "rank %d merged" % rank, 1e-5, 1e-5)
    host = Dm.merge_partials_host(po, pm, pl) * (1.0 / (1.0 + np.exp(-gate.reshape(R, 256).astype(np.float64))))
    util.check_close(host.reshape(q_len, hq, 256), want, "host merge", 1e-5, 1e-5)
    dist.barrier()
    dist.destroy_process_group()
    print("OK rank", rank)


if __name__ == "__main__":
    main()
