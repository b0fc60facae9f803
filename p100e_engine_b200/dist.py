"""Multi-GPU wrapper of the attention path: one process per GPU.

Sharding follows the reference's tensor parallelism — whole KV-head groups per rank (a KV head and its 6 query heads,
reference src/tp_split.h:45,209-215; per-rank caches sized by the local head count, src/tp_model.cu:3886-3891) — so at
2 and 4 GPUs attention needs no exchange at all.  With 4 KV heads and 8 GPUs the heads split 4 ways and each sequence's
pages split 2 ways: the two sequence shards of a head compute unnormalised (O, m, l) over their own keys, all-gather
them over NCCL (NVLink / NVSwitch) and merge them in shard order with the formula of the reference's split combine
(dec2_combine_k, src/fast/attn_dec2.cu:430-450), fused with the sigmoid gate.  The received partials land in local
memory before the merge kernel reads them.

torch.distributed is used for the process group and the all-gather only; all arithmetic runs in libb200attn.so.
"""
import numpy as np


def seq_local_positions(pos, n_seq, seq_rank, psh=8):
    """Global row positions -> positions in shard seq_rank's compacted sequence (the mapping the library's pool applies in
    b200_pool_step).  The pages of a sequence are dealt round-robin: shard r keeps logical pages r, r + n_seq, ... back to
    back, so global position p (page g = p >> psh, offset o) sits at local page g // n_seq, offset o, if g % n_seq == r.
    A row at global position P sees global keys 0..P; on this shard these are the local positions 0..local(P'), P' being
    the last owned position <= P.  Returns that last visible local position per row, -1 when the shard owns none."""
    pos = np.asarray(pos, np.int64)
    ps = 1 << psh
    g = pos >> psh
    o = pos & (ps - 1)
    full_before = np.maximum((g - seq_rank + n_seq - 1) // n_seq, 0)   # owned pages with index < g
    owns = (g % n_seq) == seq_rank
    loc = np.where(owns, full_before * ps + o, full_before * ps - 1)
    return np.where(pos < 0, -1, loc).astype(np.int32)


def seq_local_length(n, n_seq, seq_rank, psh=8):
    """number of positions of a sequence of n positions that live on shard seq_rank"""
    return 0 if n <= 0 else int(seq_local_positions(np.array([n - 1]), n_seq, seq_rank, psh)[0]) + 1


class ShardPlan:
    """Which KV heads and which sequence shard a rank owns.

    world 1: everything.  world 2 / 4: heads split, n_seq = 1.  world 8 (more ranks than KV heads): head shards =
    n_kv_heads, the remaining factor splits the sequence; ranks sharing a head group form one merge group.
    """

    def __init__(self, world, rank, n_kv_heads=4, gqa=6, n_seq=None):
        if world < 1 or rank < 0 or rank >= world:
            raise ValueError("bad world / rank")
        self.world, self.rank = world, rank
        # n_seq forces the number of sequence shards (the default uses them only when the ranks outnumber the kv heads)
        self.n_head_shards = min(world, n_kv_heads) if not n_seq else world // n_seq
        if self.n_head_shards < 1 or n_kv_heads % self.n_head_shards or world % self.n_head_shards:
            raise ValueError("world size %d does not tile %d kv heads" % (world, n_kv_heads))
        self.n_seq = world // self.n_head_shards
        self.head_rank = rank // self.n_seq
        self.seq_rank = rank % self.n_seq
        self.hkv_local = n_kv_heads // self.n_head_shards
        self.hq_local = self.hkv_local * gqa
        self.kv_head0 = self.head_rank * self.hkv_local
        self.q_head0 = self.kv_head0 * gqa

    def merge_group_ranks(self):
        """global ranks of the sequence shards that share this rank's heads, in merge order"""
        return [self.head_rank * self.n_seq + s for s in range(self.n_seq)]

    def all_merge_groups(self):
        return [[h * self.n_seq + s for s in range(self.n_seq)] for h in range(self.n_head_shards)]

    def local_positions(self, pos, psh=8):
        return seq_local_positions(pos, self.n_seq, self.seq_rank, psh)

    def local_length(self, n, psh=8):
        return seq_local_length(n, self.n_seq, self.seq_rank, psh)


class NcclComm:
    """A raw ncclComm_t over `ranks` (global ranks, in shard order), made with the NCCL library that torch has loaded: the
    library's exchange entry point and plain all-gathers are then enqueued straight on the caller's stream, without the
    process group's own stream and the two event hops around every collective.  Collective: every rank of `ranks` constructs
    it at the same point; the unique id travels over the torch process group `group` (the same ranks)."""

    def __init__(self, ranks, group, device):
        import ctypes as C
        import torch
        import torch.distributed as dist
        paths = [ln.split()[-1] for ln in open("/proc/self/maps") if "libnccl" in ln]
        if not paths:
            raise RuntimeError("no NCCL library is loaded in this process")
        self.nccl = C.CDLL(paths[0])

        class UniqueId(C.Structure):
            _fields_ = [("internal", C.c_byte * 128)]

        uid = UniqueId()
        me = dist.get_rank()
        if me == ranks[0] and self.nccl.ncclGetUniqueId(C.byref(uid)) != 0:
            raise RuntimeError("ncclGetUniqueId failed")
        t = torch.frombuffer(bytearray(bytes(uid)), dtype=torch.uint8).to(device)
        dist.broadcast(t, ranks[0], group=group)
        C.memmove(C.byref(uid), t.cpu().numpy().tobytes(), 128)
        self.comm = C.c_void_p()
        self.nccl.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
        if self.nccl.ncclCommInitRank(C.byref(self.comm), len(ranks), uid, ranks.index(me)) != 0:
            raise RuntimeError("ncclCommInitRank failed")
        self.nccl.ncclAllGather.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p]
        self.nccl.ncclCommDestroy.argtypes = [C.c_void_p]
        self.rank, self.size = ranks.index(me), len(ranks)

    @property
    def handle(self):
        return self.comm.value

    def all_gather_f32(self, buf, stream=None):
        """in-place all-gather of a float32 tensor [size][n]: this rank's row is its contribution (on the current stream)"""
        import torch
        n = buf.numel() // self.size
        st = (stream or torch.cuda.current_stream()).cuda_stream
        rc = self.nccl.ncclAllGather(buf.data_ptr() + 4 * n * self.rank, buf.data_ptr(), n, 7, self.comm, st)
        if rc != 0:
            raise RuntimeError("ncclAllGather returned %d" % rc)

    def close(self):
        if self.comm:
            self.nccl.ncclCommDestroy(self.comm)
            self.comm = None


class SeqMerge:
    """All-gather + merge of sequence-shard partials inside one merge group (used only when plan.n_seq > 1)."""

    def __init__(self, plan, rows, hq_local, d=256, device=None, group=None, comm=None):
        """group: torch process group of the shards (the exchange then runs through torch.distributed); comm: a NcclComm of
        the shards (the exchange and the merge are then one library call on the current stream)"""
        import torch
        self.plan, self.rows, self.hq, self.d, self.group, self.comm = plan, rows, hq_local, d, group, comm
        R = rows * hq_local
        self.R = R
        # one flat send buffer per rank: [O (R*d) | m (R) | l (R)], gathered into [n_seq][R*(d+2)]
        self.send = torch.zeros(R * (d + 2), dtype=torch.float32, device=device)
        self.recv = torch.zeros(plan.n_seq, R * (d + 2), dtype=torch.float32, device=device)

    def views(self):
        """(part_o, part_m, part_l) views of the send buffer for b200_attn_decode_slots_partial"""
        R, d = self.R, self.d
        return self.send[:R * d], self.send[R * d:R * d + R], self.send[R * d + R:]

    def exchange_and_merge(self, gate, out):
        import torch.distributed as dist
        from . import fast
        R, d = self.R, self.d
        if self.comm is not None:
            if not fast.seq_exchange_merge(self.comm.handle, self.plan.n_seq, self.send, self.recv, R, d, gate, out):
                raise RuntimeError("seq_exchange_merge refused")
            return
        dist.all_gather_into_tensor(self.recv.view(-1), self.send, group=self.group)
        # the merge reads the gathered flat buffers in place (no communicator: the gather above was the exchange)
        if not fast.seq_exchange_merge(0, self.plan.n_seq, self.send, self.recv, R, d, gate, out):
            raise RuntimeError("seq_exchange_merge refused")


class PeerMerge:
    """Merge of sequence-shard partials read in place over peer-mapped buffers (one process per GPU on one node): no
    collective in the path.  Every shard owns two partial buffers (used alternately) and a row of flag words in one
    buffer from b200_peer_alloc; the handles go round the group once, at construction.  Same interface as SeqMerge."""

    def __init__(self, plan, rows, hq_local, d=256, device=None, group=None):
        import torch
        import torch.distributed as dist
        from . import fast
        self.plan, self.rows, self.hq, self.d = plan, rows, hq_local, d
        R = rows * hq_local
        self.R = R
        self.part_bytes = (R * (d + 2) * 4 + 255) // 256 * 256
        self.flag_off = 2 * self.part_bytes
        n, me = plan.n_seq, plan.seq_rank
        # every shard runs the same collectives whatever happens locally, and all of them learn whether all mappings exist
        err = None
        try:
            self.own, handle = fast.peer_alloc(self.flag_off + 256)
        except Exception as e:   # noqa: BLE001 - reported to the whole group below
            self.own, handle, err = 0, b"", e
        handles = [None] * n
        dist.all_gather_object(handles, handle, group=group)
        self.base = []
        for s in range(n):
            try:
                self.base.append(self.own if s == me else fast.peer_open(handles[s]) if (err is None and handles[s]) else 0)
            except Exception as e:   # noqa: BLE001
                self.base.append(0)
                err = err or e
        ok = torch.tensor([0 if (err is not None or 0 in self.base) else 1], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)   # also: every flag row is zeroed and mapped before the first call
        if int(ok.item()) == 0:
            self.close()
            raise RuntimeError("peer-mapped buffers are not available in this group: %r" % (err,))
        self.me, self.epoch, self.torch, self.device = me, 0, torch, device

    def close(self):
        from . import fast
        for s, b in enumerate(getattr(self, "base", [])):
            if b and b != self.own:
                fast.peer_close(b)
        if getattr(self, "own", 0):
            fast.peer_free(self.own)
        self.base, self.own = [], 0

    def _views(self, parity):
        """(part_o, part_m, part_l) device addresses of this shard's buffer of the given parity"""
        R, d = self.R, self.d
        b = self.own + parity * self.part_bytes
        return b, b + R * d * 4, b + (R * d + R) * 4

    def views(self):
        """where the next call's partial goes (b200_attn_decode_slots_partial takes the addresses)"""
        return self._views((self.epoch + 1) & 1)

    def exchange_and_merge(self, gate, out, qbuf=None):
        from . import fast
        self.epoch += 1
        par = self.epoch & 1
        parts = [b + par * self.part_bytes for b in self.base]
        flags = [b + self.flag_off for b in self.base]
        if not fast.seq_merge_peers(parts, flags, self.me, self.epoch, self.R, self.d, gate, out, qbuf):
            raise RuntimeError("seq_merge_peers refused")


def merge_partials_host(parts_o, parts_m, parts_l):
    """numpy statement of the merge (for CPU tests of the exchange logic): parts_* [n][R][D] / [n][R] -> [R][D]"""
    parts_o = np.asarray(parts_o, np.float64)
    parts_m = np.asarray(parts_m, np.float64)
    parts_l = np.asarray(parts_l, np.float64)
    M = parts_m.max(axis=0)
    w = np.where(np.isneginf(parts_m), 0.0, np.exp(parts_m - np.where(np.isneginf(M), 0.0, M)[None, :]))
    den = (w * parts_l).sum(axis=0)
    num = (w[:, :, None] * parts_o).sum(axis=0)
    return np.where(den[:, None] > 0, num / np.where(den > 0, den, 1.0)[:, None], 0.0)
