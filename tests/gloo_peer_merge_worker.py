"""Worker of tests/test_host_logic.py::test_peer_merge_host_protocol_gloo (one CPU rank of a gloo group).

The device calls behind PeerMerge (b200_peer_alloc / open / close / free, b200_seq_merge_peers) are replaced by
recorders: what is checked is the host protocol around them: every shard maps every other shard's buffer in shard order,
the two partial buffers alternate with the call number, every shard passes the same epoch, and a shard whose mapping fails
makes the whole group give up together (so that a caller can fall back to NCCL on all ranks alike)."""
import sys

import torch.distributed as dist

from p100e_engine_b200 import dist as Dm, fast


def main():
    rank, world, fail_rank = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    plan = Dm.ShardPlan(world * 4, rank, 4, 6)
    plan.n_seq, plan.seq_rank = world, rank
    calls, closed = [], []
    own_addr = 0x10000000 * (rank + 1)

    def peer_alloc(nbytes):
        return own_addr, bytes([rank]) * 64

    def peer_open(handle):
        src = handle[0]
        assert handle == bytes([src]) * 64
        if rank == fail_rank:
            raise RuntimeError("mapping refused (test)")
        return 0x10000000 * (src + 1) + 0x1000     # where this process sees shard src's buffer

    fast.peer_alloc, fast.peer_open = peer_alloc, peer_open
    fast.peer_close = lambda p: closed.append(p) or True
    fast.peer_free = lambda p: closed.append(p) or True
    fast.seq_merge_peers = lambda parts, flags, me, epoch, R, D, gate, out, qbuf=None, s=None: calls.append((list(parts), list(flags), me, epoch, R, D)) or True
    rows, hq = 8, 6
    try:
        mg = Dm.PeerMerge(plan, rows, hq, 256, None, None)
    except RuntimeError as e:
        assert fail_rank >= 0, e
        dist.barrier()
        print("REFUSED rank", rank, "freed", len(closed))
        dist.destroy_process_group()
        return
    assert fail_rank < 0
    R = rows * hq
    part = (R * 258 * 4 + 255) // 256 * 256
    for call in range(1, 4):
        po, pm, pl = mg.views()
        par = call & 1
        assert po == own_addr + par * part and pm == po + R * 256 * 4 and pl == pm + R * 4
        mg.exchange_and_merge(0, 0)
        parts, flags, me, epoch, r_, d_ = calls[-1]
        assert (me, epoch, r_, d_) == (rank, call, R, 256)
        for s in range(world):
            base = own_addr if s == rank else 0x10000000 * (s + 1) + 0x1000
            assert parts[s] == base + par * part and flags[s] == base + 2 * part
    dist.barrier()
    dist.destroy_process_group()
    print("OK rank", rank)


if __name__ == "__main__":
    main()
