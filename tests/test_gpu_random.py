"""Seeded random shapes: batched decode / verify and gated prefill against the oracle, and the same call repeated must give
the same bits (a race between warps or CTAs would show up as a difference between runs)."""
import numpy as np
import pytest

from oracle import orc
from tests import util
from tests.test_gpu_decode import TYPES, _verify_batch
from tests.test_gpu_prefill import _filled

pytestmark = pytest.mark.gpu
HQ, D, SCALE = util.HQ, util.D, util.SCALE


def test_random_decode_batches(cuda, lib):
    import torch
    from p100e_engine_b200 import fast
    rng = np.random.default_rng(12345)
    for trial in range(15):
        tname = ["q8_0", "q4_0", "f16"][trial % 3]
        q_len = int(rng.integers(1, 5))
        n_slots = int(rng.integers(1, 7))
        lens = [int(max(q_len, rng.integers(1, 5000))) for _ in range(n_slots)]
        chunk = int(rng.choice([0, 64, 128, 256, 512, 1024, -1]))
        got, ref, (q, gate, pos, rtab, c, pool, pool_t, pt_t) = _verify_batch(cuda, TYPES[tname], n_slots, q_len, lens,
                                                                              50 + trial, chunk)
        util.check_close(got, ref, "random decode %d: %s q_len %d lens %s chunk %d" % (trial, tname, q_len, lens, chunk))
        again = torch.zeros(n_slots * q_len, HQ, D, device=cuda)
        for _ in range(2):
            assert fast.attn_decode_slots(util.to_dev(q, cuda), c, again, util.to_dev(gate, cuda), n_slots, q_len,
                                          util.to_dev(pos, cuda), max(lens), HQ, SCALE, chunk)
            torch.cuda.synchronize()
            assert np.array_equal(again.cpu().numpy(), got), "run-to-run difference in trial %d" % trial
    assert fast.device_status() == 0


def test_random_gated_prefills(cuda, lib):
    import torch
    from p100e_engine_b200 import fast
    rng = np.random.default_rng(777)
    for trial in range(9):
        tname = ["q8_0", "q4_0", "f16"][trial % 3]
        T, p0 = int(rng.integers(1, 700)), int(rng.integers(0, 2500))
        c, oc = _filled(TYPES[tname], p0 + T, cuda, 200 + trial)
        q = util.rng_normal(300 + trial, (T, HQ, D))
        gate = util.rng_normal(400 + trial, (T, HQ * D))
        out = torch.full((T, HQ, D), float("nan"), device=cuda)
        assert fast.attn_prefill_gated(util.to_dev(q, cuda), c, out, util.to_dev(gate, cuda), T, p0, HQ, SCALE, None, 0)
        torch.cuda.synchronize()
        ref = orc.attention(q, oc, T, HQ, SCALE, p0=p0, gate=gate)
        util.check_close(out.cpu().numpy(), ref, "random prefill %d: %s T %d p0 %d" % (trial, tname, T, p0))
        again = torch.zeros_like(out)
        assert fast.attn_prefill_gated(util.to_dev(q, cuda), c, again, util.to_dev(gate, cuda), T, p0, HQ, SCALE, None, 0)
        torch.cuda.synchronize()
        assert torch.equal(again, out), "run-to-run difference in trial %d" % trial
    assert fast.device_status() == 0
