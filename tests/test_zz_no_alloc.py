"""The allocation-free decode entry point (b200_attn_decode_slots_noalloc): for callers that may not call cudaMalloc
(a pool that owns the whole GPU, a no-allocation real-time loop), the split partials live in a fixed array inside the
library.  Checked through the C ABI against the regular entry point on two calls in a row (the array is shared and keeps
the previous call's contents), plus the size limit.  Collected last on purpose: it runs after every other test."""
import ctypes as C

import numpy as np
import pytest

from tests import util
from tests.util import D, HKV, HQ, SCALE, TYPES

pytestmark = pytest.mark.gpu


def _case(cuda, lib, kt, lens, q_len, seed):
    import torch
    from p100e_engine_b200 import fast, lib as L
    n_slots = len(lens)
    maxp = (max(lens) + 255) // 256
    pool = util.PagedPool(kt, sum((n + 255) // 256 for n in lens) + 1, psh=8, seed=seed)
    pts = np.stack([pool.take(n, maxp) for n in lens])
    pool_t = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    pt_t = util.to_dev(pts.reshape(-1), cuda)
    for s, n in enumerate(lens):
        pc = util.dev_cache(pool_t, pool, pt_t[s * maxp:(s + 1) * maxp], None, maxp << 8)
        assert fast.kv_append(pc, util.to_dev(util.rng_normal(seed + 2 * s, (n, HKV, D)), cuda),
                              util.to_dev(util.rng_normal(seed + 2 * s + 1, (n, HKV, D)), cuda), 0, n)
    rows = n_slots * q_len
    pos = util.to_dev(np.array([lens[s] - q_len + j for s in range(n_slots) for j in range(q_len)], np.int32), cuda)
    rtab = util.to_dev(np.array([s * maxp for s in range(n_slots) for _ in range(q_len)], np.int32), cuda)
    q = util.to_dev(util.rng_normal(seed + 50, (rows, HQ, D)), cuda)
    gate = util.to_dev(util.rng_normal(seed + 51, (rows, HQ * D)), cuda)
    c = util.dev_cache(pool_t, pool, pt_t, rtab, maxp << 8)
    cs = c.c()
    want = torch.zeros(rows, HQ, D, device=cuda)
    got = torch.full((rows, HQ, D), float("nan"), device=cuda)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.b200_attn_decode_slots(q.data_ptr(), C.byref(cs), want.data_ptr(), gate.data_ptr(), n_slots, q_len, pos.data_ptr(),
                                      max(lens), HQ, SCALE, 512, stream) == L.OK
    assert lib.b200_attn_decode_slots_noalloc(q.data_ptr(), C.byref(cs), got.data_ptr(), gate.data_ptr(), n_slots, q_len,
                                              pos.data_ptr(), max(lens), HQ, SCALE, 512, stream) == L.OK
    torch.cuda.synchronize()
    util.check_close(got.cpu().numpy(), want.cpu().numpy(), "no-alloc entry vs regular entry")
    assert torch.equal(got, want)      # same kernels, same chunking: the bits agree as well
    return (q, cs, gate, pos, n_slots, q_len, max(lens), c, pool_t, pt_t, rtab)


def test_noalloc_matches_regular_entry_twice(cuda, lib):
    import torch
    # two different calls back to back: the second one reuses the array with the first one's partials still in it
    _case(cuda, lib, TYPES["q8_0"], [1500, 300, 2049], 4, 11)
    keep = _case(cuda, lib, TYPES["q4_0"], [700, 64], 1, 12)
    # once the kernels are loaded, a further call leaves the device's free memory where it was, and so does reading the
    # entry point's own status word
    q, cs, gate, pos, n_slots, q_len, max_n = keep[:7]
    out = torch.zeros(n_slots * q_len, HQ, D, device=cuda)
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    assert lib.b200_attn_decode_slots_noalloc(q.data_ptr(), C.byref(cs), out.data_ptr(), gate.data_ptr(), n_slots, q_len,
                                              pos.data_ptr(), max_n, HQ, SCALE, 512, stream) == 0
    assert lib.b200_noalloc_device_status(stream) == 0
    assert torch.cuda.mem_get_info()[0] == free0


def test_noalloc_status_word_is_readable(cuda, lib):
    """a position beyond max_n through this entry point lands in its own status word (bit 8), which
    b200_noalloc_device_status returns and clears; the regular status word stays clean"""
    import torch
    keep = _case(cuda, lib, TYPES["q8_0"], [900], 4, 14)
    q, cs, gate, pos, n_slots, q_len, max_n = keep[:7]
    out = torch.full((q_len, HQ, D), float("nan"), device=cuda)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.b200_attn_decode_slots_noalloc(q.data_ptr(), C.byref(cs), out.data_ptr(), gate.data_ptr(), n_slots, q_len,
                                              pos.data_ptr(), 256, HQ, SCALE, 256, stream) == 0      # claims 256 keys of 900
    assert lib.b200_noalloc_device_status(stream) == 8
    assert lib.b200_noalloc_device_status(stream) == 0
    assert lib.b200_last_device_status(stream) == 0
    assert torch.isfinite(out).all()


def test_noalloc_rejects_oversize(cuda, lib):
    import torch
    from p100e_engine_b200 import lib as L
    keep = _case(cuda, lib, TYPES["q8_0"], [600], 4, 13)
    q, cs, gate, pos, n_slots, q_len, max_n = keep[:7]
    out = torch.zeros(q_len, HQ, D, device=cuda)
    n0 = lib.b200_launch_count()
    # 64-key chunks over a claimed 4M-key context need far more than the built-in array: refused, nothing launched
    rc = lib.b200_attn_decode_slots_noalloc(q.data_ptr(), C.byref(cs), out.data_ptr(), gate.data_ptr(), n_slots, q_len,
                                            pos.data_ptr(), 1 << 22, HQ, SCALE, 64, torch.cuda.current_stream().cuda_stream)
    assert rc == L.ERR_SCRATCH
    assert lib.b200_launch_count() == n0
