"""The baseline's configurations at their real sizes against the reference's own kernels on the same GPU
(oracle/_ref/libp100e_ref.so: the reference's .cu files compiled unmodified for sm_100a).

  config 2   MTP verify, 8 slots x q_len 4, contexts ~U{1024..32768}, q8_0 pages, sigmoid gate
  config 5   one layer of the whole-box decode: 64 slots x q_len 4, contexts ~U{512..65536}, q8_0 and f16, chunk chosen
             from the batch (chunk_keys = -1, what the benchmark runs)
  config 3   chunked causal prefill, T = 8192, p0 = 0, bf16 inputs, partial RoPE, q8_0 pages: every row against the
             reference's fp32 attn_prefill

The reference takes at most 8 rows per call (src/fast/attn.cuh:64-66) and pool views under 4 GiB (src/fast/attn_dec2.cu:495):
it is called in 8-row groups, and for the f16 pool (more than 4 GiB per K region) the slots are split in two groups whose
pages come from separate halves of the pool, each half handed to the reference as its own view.  The caches hold N(0,1)
keys and values quantised by this library's kv_append, whose bytes other tests hold equal to the reference quantiser's.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import orc
from tests import util
from tests.util import D, HKV, HQ, SCALE, TYPES

pytestmark = pytest.mark.gpu


def _verify_case(cuda, kt, lens, q_len, seed, chunk, groups=1):
    import torch
    from p100e_engine_b200 import fast
    ref = orc.p100e_ref()
    if ref is None:
        pytest.skip("reference kernels not prebuilt")
    n_slots = len(lens)
    maxp = (max(lens) + 255) // 256
    rowb = orc.row_bytes(kt, HKV, D)
    pstride = 256 * rowb
    need = [(n + 255) // 256 for n in lens]
    # slots are dealt to `groups` page ranges; inside a range the pages are a seeded permutation
    grp = [s * groups // n_slots for s in range(n_slots)]
    g_pages = [sum(need[s] for s in range(n_slots) if grp[s] == g) + 1 for g in range(groups)]
    g_base = np.concatenate([[0], np.cumsum(g_pages)])[:groups]
    n_pages = int(sum(g_pages))
    rng = np.random.default_rng(seed)
    perms = [rng.permutation(g_pages[g]).astype(np.int32) for g in range(groups)]
    used = [0] * groups
    pt_abs = np.full((n_slots, maxp), -1, np.int32)      # page ids in the whole pool (this library's view)
    pt_rel = np.full((n_slots, maxp), -1, np.int32)      # page ids inside the slot's group range (the reference's views)
    for s in range(n_slots):
        g = grp[s]
        ids = perms[g][used[g]:used[g] + need[s]]
        used[g] += need[s]
        pt_rel[s, :need[s]] = ids
        pt_abs[s, :need[s]] = ids + g_base[g]
    kpool = torch.zeros(n_pages * pstride, dtype=torch.uint8, device=cuda)
    vpool = torch.zeros(n_pages * pstride, dtype=torch.uint8, device=cuda)
    pt_t = util.to_dev(pt_abs.reshape(-1), cuda)
    ptr_t = util.to_dev(pt_rel.reshape(-1), cuda)
    gen = torch.Generator(device=cuda)
    for s, n in enumerate(lens):
        gen.manual_seed(seed * 1000 + s)
        cs = fast.kv_cache(kt, maxp << 8, HKV, D, kpool, vpool, pt_t[s * maxp:(s + 1) * maxp], None, 8, pstride)
        for p in range(0, n, 16384):
            T = min(16384, n - p)
            k = torch.randn(T, HKV, D, generator=gen, device=cuda)
            v = torch.randn(T, HKV, D, generator=gen, device=cuda)
            assert fast.kv_append(cs, k, v, p, T)
    rows = n_slots * q_len
    pos = np.array([lens[s] - q_len + j for s in range(n_slots) for j in range(q_len)], np.int32)
    rtab = np.array([s * maxp for s in range(n_slots) for _ in range(q_len)], np.int32)
    pos_t, rtab_t = util.to_dev(pos, cuda), util.to_dev(rtab, cuda)
    gen.manual_seed(seed + 77)
    q = torch.randn(rows, HQ, D, generator=gen, device=cuda)
    gate = torch.randn(rows, HQ * D, generator=gen, device=cuda)
    c = fast.kv_cache(kt, maxp << 8, HKV, D, kpool, vpool, pt_t, rtab_t, 8, pstride)
    out = torch.full((rows, HQ, D), float("nan"), device=cuda)
    assert fast.attn_decode_slots(q, c, out, gate, n_slots, q_len, pos_t, max(lens), HQ, SCALE, chunk)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    # the reference: 8 rows per call, each group through its own (< 4 GiB) view of the pool, then its gate kernel
    want = torch.zeros(rows, HQ, D, device=cuda)
    for g in range(groups):
        assert g_pages[g] * pstride < (1 << 32)
        kv = orc.OrcKv()
        kv.type, kv.n_ctx, kv.Hkv, kv.D = kt, maxp << 8, HKV, D
        kv.k = kpool.data_ptr() + int(g_base[g]) * pstride
        kv.v = vpool.data_ptr() + int(g_base[g]) * pstride
        kv.pt, kv.psh, kv.pstride = ptr_t.data_ptr(), 8, pstride
        r_rows = [r for r in range(rows) if grp[r // q_len] == g]
        for i in range(0, len(r_rows), 8):
            r0, nr = r_rows[i], min(8, len(r_rows) - i)
            assert r_rows[i + nr - 1] == r0 + nr - 1          # a group's rows are consecutive
            kv.rtab = rtab_t.data_ptr() + 4 * r0
            assert ref.ref_attn_decode_rows(q.data_ptr() + 4 * r0 * HQ * D, C.byref(kv), want.data_ptr() + 4 * r0 * HQ * D, nr,
                                            pos_t.data_ptr() + 4 * r0, HQ, SCALE, None) == 0
    ref.ref_k_sigmoid_mul(want.data_ptr(), gate.data_ptr(), rows * HQ * D, None)
    torch.cuda.synchronize()
    return out.cpu().numpy(), want.cpu().numpy()


def test_config2_verify_batch_vs_reference_kernels(cuda, lib):
    lens = np.random.default_rng(0xB202).integers(1024, 32769, size=8).tolist()
    for chunk in (-1, 0):
        got, want = _verify_case(cuda, TYPES["q8_0"], lens, 4, 2, chunk)
        util.check_close(got, want, "config 2 (8 slots x q_len 4, contexts %s, chunk %d)" % (lens, chunk))


@pytest.mark.parametrize("tname", ["q8_0", "f16"])
def test_config5_one_layer_vs_reference_kernels(cuda, lib, tname):
    lens = np.random.default_rng(0xB205).integers(512, 65537, size=64).tolist()
    got, want = _verify_case(cuda, TYPES[tname], lens, 4, 5, -1, groups=2 if tname == "f16" else 1)
    util.check_close(got, want, "config 5, one layer, %s (64 slots x q_len 4, %d keys)" % (tname, sum(lens)))
    # slot by slot as well: a short slot's error must not hide behind the batch's largest magnitude
    for s in range(64):
        util.check_close(got[4 * s:4 * s + 4], want[4 * s:4 * s + 4], "config 5 %s slot %d (%d keys)" % (tname, s, lens[s]))


def test_config3_prefill_every_row_vs_reference_fp32(cuda, lib):
    import torch
    from p100e_engine_b200 import fast
    ref = orc.p100e_ref()
    if ref is None:
        pytest.skip("reference kernels not prebuilt")
    kt, T = TYPES["q8_0"], 8192
    pool = util.PagedPool(kt, 32, psh=8, seed=3)
    pt = pool.take(T, 32)
    pool_t = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    dc = util.dev_cache(pool_t, pool, util.to_dev(pt, cuda), None, T)
    g = torch.Generator(device="cpu").manual_seed(0xB203)
    k = torch.randn(T, HKV, D, generator=g).to(torch.bfloat16).to(cuda)
    v = torch.randn(T, HKV, D, generator=g).to(torch.bfloat16).to(cuda)
    q = torch.randn(T, HQ, D, generator=g).to(torch.bfloat16).to(cuda)
    gate = torch.randn(T, HQ * D, generator=g).to(cuda)
    qr = torch.zeros(T, HQ, D, device=cuda)
    assert fast.rope_append_bf16(q, k, v, qr, dc, 0, T, HQ, HKV, D, 64, 1e7)
    out = torch.zeros(T, HQ, D, device=cuda)
    assert fast.attn_prefill_gated(qr, dc, out, gate, T, 0, HQ, SCALE, None, 0)
    want = torch.zeros(T, HQ, D, device=cuda)
    assert ref.ref_attn_prefill(qr.data_ptr(), C.byref(util.orc_kv_of(dc)), want.data_ptr(), T, 0, HQ, SCALE, None) == 0
    ref.ref_k_sigmoid_mul(want.data_ptr(), gate.data_ptr(), T * HQ * D, None)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    got, want = out.cpu().numpy(), want.cpu().numpy()
    util.check_close(got, want, "config 3, all 8192 rows vs the reference's fp32 attn_prefill")
    for t0 in range(0, T, 512):      # and per 512-row band, the deepest ones included
        util.check_close(got[t0:t0 + 512], want[t0:t0 + 512], "config 3 rows %d..%d" % (t0, t0 + 511))
    # the one-call bf16 entry point (rotation inside the attention kernel) gives the same bits as the two calls
    pool2_t = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    dc2 = util.dev_cache(pool2_t, pool, util.to_dev(pt, cuda), None, T)
    nb = fast.attn_prefill_bf16_scratch_bytes(T, HKV, T)
    scratch = torch.empty(nb, dtype=torch.uint8, device=cuda)
    out2 = torch.zeros(T, HQ, D, device=cuda)
    assert fast.attn_prefill_bf16(q, k, v, gate, None, out2, None, None, dc2, 0, T, HQ, 64, 1e7, SCALE, scratch, nb)
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    assert torch.equal(pool2_t, pool_t), "cache bytes of the one-call prefill differ"
    assert torch.equal(out2, out), "one-call bf16 prefill differs from rope_append_bf16 + attn_prefill_gated"
