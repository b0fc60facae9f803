"""Worker of tests/test_gpu_misc.py::test_two_gpu_sequence_split_nccl: two GPUs hold alternate pages of every slot, compute
partial (O, m, l) with the library, all-gather them over NCCL and merge; rank results must equal the oracle; then the same
merge over peer-mapped buffers (no collective) must give the same bits."""
import os

import numpy as np
import torch
import torch.distributed as dist

from oracle import orc
from p100e_engine_b200 import dist as Dm, fast
from tests import util


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    plan = Dm.ShardPlan(world, rank, 1, 6)          # one kv head, `world` sequence shards
    kt, hq, hkv, q_len = orc.KV_Q8_0, 6, 1, 4
    lens = [1500, 300, 2049]
    rows = len(lens) * q_len
    pos = np.array([n - q_len + j for n in lens for j in range(q_len)], np.int32)
    q = util.rng_normal(3, (rows, hq, 256))
    gate = util.rng_normal(4, (rows, hq * 256))
    want = np.zeros((rows, hq, 256), np.float32)
    maxp = 5
    ptab = np.full((len(lens), maxp), -1, np.int32)
    rowb = orc.row_bytes(kt, hkv, 256)
    pool_k = torch.zeros(16 * 256 * rowb, dtype=torch.uint8, device=dev)
    pool_v = torch.zeros_like(pool_k)
    nextp = 0
    for s, n in enumerate(lens):
        k = util.rng_normal(10 + s, (n, hkv, 256))
        v = util.rng_normal(20 + s, (n, hkv, 256))
        full = orc.Cache.contiguous(kt, n, hkv, 256)
        orc.kv_append(full, k, v, 0, n)
        sl = slice(s * q_len, (s + 1) * q_len)
        want[sl] = orc.attention(q[sl], full, q_len, hq, util.SCALE, pos=pos[sl], gate=gate[sl])
        own = np.nonzero((np.arange(n) >> 8) % world == rank)[0]
        npg = (len(own) + 255) // 256
        ptab[s, :npg] = np.arange(nextp, nextp + npg)
        nextp += npg
        c = fast.kv_cache(kt, maxp << 8, hkv, 256, pool_k, pool_v, util.to_dev(ptab[s], dev), None, 8, 256 * rowb)
        if len(own):
            assert fast.kv_append(c, util.to_dev(k[own], dev), util.to_dev(v[own], dev), 0, len(own))
    lpos = plan.local_positions(pos)
    rtab = np.repeat(np.arange(len(lens)) * maxp, q_len).astype(np.int32)
    c = fast.kv_cache(kt, maxp << 8, hkv, 256, pool_k, pool_v, util.to_dev(ptab.reshape(-1), dev), util.to_dev(rtab, dev), 8, 256 * rowb)
    mg = Dm.SeqMerge(plan, rows, hq, 256, dev, None)
    po, pm, pl = mg.views()
    assert fast.attn_decode_slots_partial(util.to_dev(q, dev), c, po, pm, pl, len(lens), q_len, util.to_dev(lpos, dev), 2049, hq, util.SCALE)
    out = torch.zeros(rows * hq, 256, device=dev)
    mg.exchange_and_merge(util.to_dev(gate, dev), out)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    util.check_close(out.cpu().numpy().reshape(rows, hq, 256), want, "rank %d" % rank)
    # the same step through the C entry point with a raw ncclComm_t, as a C++ host would drive it
    import ctypes as C
    path = [ln.split()[-1] for ln in open("/proc/self/maps") if "libnccl" in ln][0]
    nccl = C.CDLL(path)

    class UniqueId(C.Structure):
        _fields_ = [("internal", C.c_byte * 128)]

    uid = UniqueId()
    if rank == 0:
        assert nccl.ncclGetUniqueId(C.byref(uid)) == 0
    t = torch.frombuffer(bytearray(bytes(uid)), dtype=torch.uint8).to(dev)
    dist.broadcast(t, 0)
    C.memmove(C.byref(uid), bytes(t.cpu().numpy().tobytes()), 128)
    comm = C.c_void_p()
    nccl.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
    assert nccl.ncclCommInitRank(C.byref(comm), world, uid, rank) == 0
    recv = torch.zeros(world, mg.send.numel(), device=dev)
    out2 = torch.zeros_like(out)
    assert fast.seq_exchange_merge(comm.value, world, mg.send, recv, rows * hq, 256, util.to_dev(gate, dev), out2)
    torch.cuda.synchronize()
    assert torch.equal(out, out2), "C exchange differs from the torch.distributed exchange"
    nccl.ncclCommDestroy.argtypes = [C.c_void_p]
    nccl.ncclCommDestroy(comm)
    # the same merge without a collective: partials read in place over peer-mapped buffers, three calls in a row (the two
    # buffers alternate; the second call sees other queries, so a stale read of the first would show)
    pm_ = Dm.PeerMerge(plan, rows, hq, 256, dev, None)
    for call in range(3):
        qq = q if call != 1 else q[::-1].copy()
        a_o, a_m, a_l = pm_.views()
        assert fast.attn_decode_slots_partial(util.to_dev(qq, dev), c, a_o, a_m, a_l, len(lens), q_len, util.to_dev(lpos, dev), 2049, hq,
                                              util.SCALE)
        out3 = torch.zeros_like(out)
        pm_.exchange_and_merge(util.to_dev(gate, dev), out3)
        torch.cuda.synchronize()
        assert fast.device_status() == 0
        if call != 1:
            assert torch.equal(out, out3), "peer-mapped merge differs from the NCCL exchange (call %d)" % call
        else:
            assert not torch.equal(out, out3)
    dist.barrier()
    dist.destroy_process_group()
    print("OK rank", rank)


if __name__ == "__main__":
    main()
