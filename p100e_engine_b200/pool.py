"""Paged KV pool, block tables and step descriptors — the caller-side structures the attention kernels index.

Mirrors what the reference engine keeps in tp_model (reference src/tp_model.cu): one allocation per GPU laid out
[K|V][kv layer][page][2^psh positions][row] (alloc_pool, :3875-3966), a page table ptab[max_slots][max_pages] of int32
page ids filled from a free list (ensure_pages, :3358-3384), and per step a descriptor of row positions and per-row
table offsets rtab[row] = slot * max_pages (forward_batch_ids, :3999-4022).  Differences: offsets are 64-bit (a layer
region may exceed 4 GiB), a step may hold any number of rows, and a sequence-shard map says which GPU of a pair owns
each page when the KV sequence is split across two GPUs.

Pure host logic (numpy); device buffers are attached by the caller (torch tensors), so this module runs without a GPU.
"""
import numpy as np

from . import lib as L

HEAD_BYTES = {L.KV_F16: 512, L.KV_Q8_0: 272, L.KV_Q4_0: 144}   # D = 256


def row_bytes(kv_type, hkv, d=256):
    per32 = {L.KV_F16: 64, L.KV_Q8_0: 34, L.KV_Q4_0: 18}[kv_type]
    return hkv * (d // 32) * per32


class PoolLayout:
    """Byte layout of one GPU's pool: [K|V][layer][page][2^psh][row]."""

    def __init__(self, kv_type, hkv, n_layers, n_pages, psh=8, d=256):
        self.kv_type, self.hkv, self.d, self.n_layers, self.n_pages, self.psh = kv_type, hkv, d, n_layers, n_pages, psh
        self.page_positions = 1 << psh
        self.rowb = row_bytes(kv_type, hkv, d)
        self.pstride = self.page_positions * self.rowb          # bytes between consecutive pages of one layer's K
        self.layer_bytes = n_pages * self.pstride
        self.total_bytes = 2 * n_layers * self.layer_bytes

    def k_offset(self, layer):
        return layer * self.layer_bytes

    def v_offset(self, layer):
        return (self.n_layers + layer) * self.layer_bytes


class PageTable:
    """ptab[max_slots][max_pages] with a free list; pages are handed out in a seeded random order so that physical
    placement is scattered the way a long-running server's is."""

    def __init__(self, n_pages, max_slots, max_pages, psh=8, seed=0):
        self.psh, self.max_slots, self.max_pages = psh, max_slots, max_pages
        self.ptab = np.full((max_slots, max_pages), -1, np.int32)
        self.n_alloc = np.zeros(max_slots, np.int32)
        self.free = list(np.random.default_rng(seed).permutation(n_pages).astype(np.int32))[::-1]

    def ensure_pages(self, slot, n_positions):
        """make positions [0, n_positions) of the slot addressable; returns False when the pool is exhausted"""
        need = (n_positions + (1 << self.psh) - 1) >> self.psh
        if need > self.max_pages:
            return False
        while self.n_alloc[slot] < need:
            if not self.free:
                return False
            self.ptab[slot, self.n_alloc[slot]] = self.free.pop()
            self.n_alloc[slot] += 1
        return True

    def release(self, slot):
        for i in range(self.n_alloc[slot]):
            self.free.append(self.ptab[slot, i])
        self.ptab[slot, :] = -1
        self.n_alloc[slot] = 0


def step_descriptor(slots, n_past, q_len, max_pages):
    """Rows of one decode / verify step, slot-major: row r = i * q_len + j is token j of slots[i] at position
    n_past[i] + j and reads the table at rtab[r] = slots[i] * max_pages.  Returns (pos, rtab) int32 arrays."""
    slots = np.asarray(slots, np.int64)
    n_past = np.asarray(n_past, np.int64)
    j = np.arange(q_len, dtype=np.int64)
    pos = (n_past[:, None] + j[None, :]).reshape(-1).astype(np.int32)
    rtab = np.repeat(slots * max_pages, q_len).astype(np.int32)
    return pos, rtab


# ---- sequence sharding over a pair of GPUs ----------------------------------------------------------------------
def seq_shard_owner(page_index, n_seq):
    """which of the n_seq sequence shards owns logical page `page_index` of a sequence: pages are dealt round-robin,
    so the shards stay balanced at every depth and an appended token lands on the shard that owns its page"""
    return page_index % n_seq


def local_positions(pos, n_seq, seq_rank, psh=8):
    """Global row positions -> positions in shard seq_rank's compacted sequence.

    Shard r keeps logical pages r, r + n_seq, ... back to back, so global position p (page g = p >> psh, offset o)
    sits at local page g // n_seq, offset o, if g % n_seq == r.  A row at global position P sees global keys 0..P; on
    this shard these are the local positions 0..local(P'), P' being the last owned position <= P.  Returns the local
    position of that last visible key per row, -1 when the shard owns no visible key."""
    pos = np.asarray(pos, np.int64)
    ps = 1 << psh
    g = pos >> psh
    o = pos & (ps - 1)
    full_before = (g - seq_rank + n_seq - 1) // n_seq            # owned pages with index < g
    full_before = np.maximum(full_before, 0)
    owns = (g % n_seq) == seq_rank
    loc = np.where(owns, full_before * ps + o, full_before * ps - 1)
    loc = np.where(pos < 0, -1, loc)
    return loc.astype(np.int32)


def local_length(n, n_seq, seq_rank, psh=8):
    """number of positions of a sequence of n positions that live on shard seq_rank"""
    if n <= 0:
        return 0
    return int(local_positions(np.array([n - 1]), n_seq, seq_rank, psh)[0]) + 1
