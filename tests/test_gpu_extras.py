"""The parts of the path around the attention kernels, on the GPU: the a16 copy emitted from the attention epilogues, the
MTP draft-head protocol (KV-only catch-up, verify, rollback), prefill in several passes over a fixed scratch, prefill
over sequence shards with the (O, m, l) merge, the position guard, the scratch reservation, the device pool with its step
descriptor and page offload, and the sharding-independent cache filler."""
import ctypes as C

import numpy as np
import pytest

from oracle import orc
from tests import util
from tests.util import D, HKV, HQ, SCALE, TYPES

pytestmark = pytest.mark.gpu

N_ROT, BASE, EPS = 64, 1e7, 1e-6


def _paged_batch(cuda, kt, lens, seed, hkv=HKV):
    """paged pool with one sequence per slot filled through kv_append; returns (cache over all rows, pool tensor, tables)"""
    import torch
    from p100e_engine_b200 import fast
    maxp = (max(lens) + 255) // 256
    pool = util.PagedPool(kt, sum((n + 255) // 256 for n in lens) + 1, psh=8, seed=seed, hkv=hkv)
    pts = np.stack([pool.take(n, maxp) for n in lens])
    pool_t = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    pt_t = util.to_dev(pts.reshape(-1), cuda)
    for s, n in enumerate(lens):
        pc = util.dev_cache(pool_t, pool, pt_t[s * maxp:(s + 1) * maxp], None, maxp << 8)
        assert fast.kv_append(pc, util.to_dev(util.rng_normal(seed + 2 * s, (n, hkv, D)), cuda),
                              util.to_dev(util.rng_normal(seed + 2 * s + 1, (n, hkv, D)), cuda), 0, n)
    return pool, pool_t, pt_t, maxp


def _qbuf_bytes(rows, n):
    return rows * (n // 32) * 17 * 4      # 16 half2 per 32-value group + one (amax, sum) half2 per group


def test_decode_epilogue_emits_a16_like_the_reference_gate_kernel(cuda, lib):
    """b200_attn_decode_slots_a16: out equals the plain entry point bitwise, and the a16 buffer equals what the reference's
    ew_quant(EW_SIGMOID_MUL, ..., qbuf) writes for the same ungated attention output and gate"""
    import torch
    from p100e_engine_b200 import fast
    ref = orc.p100e_ref()
    if ref is None:
        pytest.skip("reference kernels not prebuilt")
    kt, lens, q_len = TYPES["q8_0"], [900, 70, 2100], 4
    pool, pool_t, pt_t, maxp = _paged_batch(cuda, kt, lens, 21)
    rows, n = len(lens) * q_len, HQ * D
    pos = util.to_dev(np.array([lens[s] - q_len + j for s in range(len(lens)) for j in range(q_len)], np.int32), cuda)
    rtab = util.to_dev(np.array([s * maxp for s in range(len(lens)) for _ in range(q_len)], np.int32), cuda)
    c = util.dev_cache(pool_t, pool, pt_t, rtab, maxp << 8)
    q = util.to_dev(util.rng_normal(5, (rows, HQ, D)), cuda)
    gate = util.to_dev(util.rng_normal(6, (rows, n)) * 2.0, cuda)
    raw = torch.zeros(rows, HQ, D, device=cuda)
    plain = torch.zeros(rows, HQ, D, device=cuda)
    fused = torch.zeros(rows, HQ, D, device=cuda)
    qb = torch.zeros(_qbuf_bytes(rows, n), dtype=torch.uint8, device=cuda)
    assert fast.attn_decode_slots(q, c, raw, None, len(lens), q_len, pos, max(lens), HQ, SCALE, 256)
    assert fast.attn_decode_slots(q, c, plain, gate, len(lens), q_len, pos, max(lens), HQ, SCALE, 256)
    assert fast.attn_decode_slots_a16(q, c, fused, gate, qb, len(lens), q_len, pos, max(lens), HQ, SCALE, 256)
    y_ref = torch.zeros(rows, n, device=cuda)
    qb_ref = torch.zeros_like(qb)
    assert ref.ref_ew_quant(1, raw.data_ptr(), gate.data_ptr(), y_ref.data_ptr(), qb_ref.data_ptr(), rows, n, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(fused, plain)
    # the fused gate uses the same expression as the reference's kernel on the same ungated value
    assert torch.equal(fused.view(rows, n), y_ref)
    assert torch.equal(qb, qb_ref), "a16 bytes of the fused epilogue differ from the reference's ew_quant"
    assert fast.device_status() == 0


def test_prefill_and_shard_merge_epilogues_emit_a16(cuda, lib):
    import torch
    from p100e_engine_b200 import fast
    kt, p0, T = TYPES["q8_0"], 130, 200
    pool, pool_t, pt_t, maxp = _paged_batch(cuda, kt, [p0 + T], 31)
    c = util.dev_cache(pool_t, pool, pt_t, None, maxp << 8)
    n = HQ * D
    q = util.to_dev(util.rng_normal(7, (T, HQ, D)), cuda)
    gate = util.to_dev(util.rng_normal(8, (T, n)), cuda)
    out1, out2 = torch.zeros(T, HQ, D, device=cuda), torch.zeros(T, HQ, D, device=cuda)
    qb = torch.zeros(_qbuf_bytes(T, n), dtype=torch.uint8, device=cuda)
    assert fast.attn_prefill_gated(q, c, out1, gate, T, p0, HQ, SCALE, None, 0)
    assert fast.attn_prefill_gated_a16(q, c, out2, gate, qb, T, p0, HQ, SCALE, None, 0)
    # the stand-alone quantiser (held byte-equal to the reference's kernel in test_gpu_misc) applied to the same values:
    # op 1 with gate logits of +inf-like size multiplies by exactly 1
    ones = torch.full((T, n), 1e4, device=cuda)
    y = torch.zeros(T, n, device=cuda)
    qb_want = torch.zeros_like(qb)
    assert fast.ew_quant(fast.EW_SIGMOID_MUL, out1.view(T, n), ones, y, qb_want, T, n)
    torch.cuda.synchronize()
    assert torch.equal(out1, out2) and torch.equal(y, out1.view(T, n))
    assert torch.equal(qb, qb_want), "a16 bytes of the prefill epilogue differ from the stand-alone quantiser"
    # sequence-shard merge with the a16 copy: two artificial parts of the same rows
    R = 8 * HQ
    po = util.to_dev(util.rng_normal(9, (2, R, D)), cuda)
    pm = util.to_dev(util.rng_normal(10, (2, R)), cuda)
    pl = util.to_dev(np.abs(util.rng_normal(11, (2, R))) + 0.5, cuda)
    recv = torch.cat([torch.cat([po[i].reshape(-1), pm[i], pl[i]]) for i in range(2)]).contiguous()
    g2 = util.to_dev(util.rng_normal(12, (R, D)), cuda)
    o_a, o_b = torch.zeros(R, D, device=cuda), torch.zeros(R, D, device=cuda)
    qb2 = torch.zeros(_qbuf_bytes(8, n), dtype=torch.uint8, device=cuda)
    assert fast.seq_exchange_merge(0, 2, recv, recv, R, D, g2, o_a)
    assert fast.seq_exchange_merge_a16(0, 2, recv, recv, R, D, g2, o_b, qb2)
    qb2_want = torch.zeros_like(qb2)
    y2 = torch.zeros(8, n, device=cuda)
    assert fast.ew_quant(fast.EW_SIGMOID_MUL, o_a.view(8, n), torch.full((8, n), 1e4, device=cuda), y2, qb2_want, 8, n)
    torch.cuda.synchronize()
    assert torch.equal(o_a, o_b) and torch.equal(qb2, qb2_want)
    assert fast.device_status() == 0


@pytest.mark.parametrize("tname", ["q8_0", "q4_0", "f16"])
def test_mtp_draft_head_catch_up_verify_rollback(cuda, lib, tname):
    """The draft head keeps one more KV layer (reference src/tp_mtp.cu:427-447,535-558,592-611).  Its prompt catch-up
    stores K/V only (src/tp_model.cu:1705-1730); a verify step appends 1 + 3 rows and attends with q_len 4; when only k
    of the drafts are accepted the rows are rolled back by position (src/tp_model.cu:3172-3180) and the next step
    overwrites them.  Bits that must hold: KV-only catch-up == the full prep's cache bytes; every verify row == the
    single-row decode at its position; after a rollback and re-append the accepted history decodes as if nothing had
    been drafted."""
    import torch
    from p100e_engine_b200 import fast
    kt = TYPES[tname]
    n0, n_ctx = 300, 1024
    rng = np.random.default_rng(41)
    qn = util.to_dev((0.5 + rng.random(D)).astype(np.float32), cuda)
    kn = util.to_dev((0.5 + rng.random(D)).astype(np.float32), cuda)

    def acts(T, seed):
        return (util.to_dev(util.rng_normal(seed, (T, HQ, 2 * D)), cuda), util.to_dev(util.rng_normal(seed + 1, (T, HKV, D)), cuda),
                util.to_dev(util.rng_normal(seed + 2, (T, HKV, D)), cuda))

    def prep(c, qg, k, v, p0, T, q, gate):
        pos = torch.arange(p0, p0 + T, dtype=torch.int32, device=cuda)
        assert fast.attn_prep(qg, k, v, qn, kn, pos, q, gate, c, p0, T, HQ, HKV, D, N_ROT, BASE, EPS)

    # prompt: one cache filled by the full prep, one by the KV-only catch-up
    qg0, k0, v0 = acts(n0, 100)
    full, kvonly = fast.kv_alloc(kt, n_ctx, HKV, D), fast.kv_alloc(kt, n_ctx, HKV, D)
    q = torch.zeros(n0, HQ, D, device=cuda)
    gate = torch.zeros(n0, HQ * D, device=cuda)
    prep(full, qg0, k0, v0, 0, n0, q, gate)
    prep(kvonly, None, k0, v0, 0, n0, None, None)
    torch.cuda.synchronize()
    assert torch.equal(full.k, kvonly.k) and torch.equal(full.v, kvonly.v), "KV-only catch-up bytes differ"

    # verify step: the last sampled token + 3 drafts at positions n0 .. n0+3
    qg1, k1, v1 = acts(4, 200)
    q4 = torch.zeros(4, HQ, D, device=cuda)
    g4 = torch.zeros(4, HQ * D, device=cuda)
    prep(kvonly, qg1, k1, v1, n0, 4, q4, g4)
    ver = torch.zeros(4, HQ, D, device=cuda)
    pos4 = torch.arange(n0, n0 + 4, dtype=torch.int32, device=cuda)
    assert fast.attn_decode_slots(q4, kvonly, ver, g4, 1, 4, pos4, n0 + 4, HQ, SCALE, 0)
    one = torch.zeros(4, HQ, D, device=cuda)
    for t in range(4):
        assert fast.attn_decode_slots(q4[t:t + 1], kvonly, one[t:t + 1], g4[t:t + 1], 1, 1, pos4[t:t + 1], n0 + t + 1, HQ, SCALE, 0)
    torch.cuda.synchronize()
    assert torch.equal(ver, one), "a verify row differs from the single-row decode at its position"

    # two drafts rejected: the history ends at n0 + 2; the next step re-appends from there with other tokens
    keep = 2
    qg2, k2, v2 = acts(4, 300)
    prep(kvonly, qg2, k2, v2, n0 + keep, 4, q4, g4)
    after = torch.zeros(4, HQ, D, device=cuda)
    posb = torch.arange(n0 + keep, n0 + keep + 4, dtype=torch.int32, device=cuda)
    assert fast.attn_decode_slots(q4, kvonly, after, g4, 1, 4, posb, n0 + keep + 4, HQ, SCALE, 0)
    # the same history built without ever drafting
    clean = fast.kv_alloc(kt, n_ctx, HKV, D)
    prep(clean, None, k0, v0, 0, n0, None, None)
    qt, gt = torch.zeros(keep, HQ, D, device=cuda), torch.zeros(keep, HQ * D, device=cuda)
    prep(clean, qg1[:keep], k1[:keep], v1[:keep], n0, keep, qt, gt)
    qc, gc = torch.zeros(4, HQ, D, device=cuda), torch.zeros(4, HQ * D, device=cuda)
    prep(clean, qg2, k2, v2, n0 + keep, 4, qc, gc)
    want = torch.zeros(4, HQ, D, device=cuda)
    assert fast.attn_decode_slots(qc, clean, want, gc, 1, 4, posb, n0 + keep + 4, HQ, SCALE, 0)
    torch.cuda.synchronize()
    rowb = orc.row_bytes(kt, HKV, D)
    used = (n0 + keep + 4) * rowb
    assert torch.equal(kvonly.k[:used], clean.k[:used]) and torch.equal(kvonly.v[:used], clean.v[:used])
    assert torch.equal(after, want), "decode after a rollback differs from the never-drafted history"
    assert fast.device_status() == 0


@pytest.mark.parametrize("tname", ["q8_0", "f16"])
def test_prefill_passes_over_a_small_scratch(cuda, lib, tname):
    """attn_fold with a scratch that holds 256 keys at a time: the context is walked in passes with the running
    (O, max, sum) carried in `out`; result against the single-pass call and the oracle.  The reference call form
    attn_fold_scratch_bytes(T, Hkv, 0, 0) gives a scratch that serves any depth."""
    import torch
    from p100e_engine_b200 import fast
    kt, p0, T = TYPES[tname], 1100, 150
    pool, pool_t, pt_t, maxp = _paged_batch(cuda, kt, [p0 + T], 51)
    c = util.dev_cache(pool_t, pool, pt_t, None, maxp << 8)
    q = util.to_dev(util.rng_normal(52, (T, HQ, D)), cuda)
    single = torch.zeros(T, HQ, D, device=cuda)
    assert fast.attn_prefill(q, c, single, T, p0, HQ, SCALE)
    nb = fast.attn_fold_scratch_bytes(T, HKV, 256)
    assert nb < fast.attn_fold_scratch_bytes(T, HKV, p0 + T)
    scratch = torch.empty(nb, dtype=torch.uint8, device=cuda)
    multi = torch.full((T, HQ, D), float("nan"), device=cuda)
    n0 = lib.b200_launch_count()
    assert fast.attn_fold(q, c, multi, T, p0, HQ, SCALE, scratch, nb)
    assert lib.b200_launch_count() - n0 == 2 * 5          # ceil(1250 / 256) passes of two kernels
    big = torch.empty(fast.attn_fold_scratch_bytes(T, HKV), dtype=torch.uint8, device=cuda)   # the reference's call form
    capped = torch.full((T, HQ, D), float("nan"), device=cuda)
    assert fast.attn_fold(q, c, capped, T, p0, HQ, SCALE, big, big.numel(), chunk=512)        # chunk caps the pass
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    pool.host[:pool.bytes] = pool_t.cpu().numpy()
    ref = orc.attention(q.cpu().numpy(), pool.host_cache(pt_t.cpu().numpy()), T, HQ, SCALE, p0=p0)
    util.check_close(single.cpu().numpy(), ref, "single pass vs oracle " + tname)
    util.check_close(multi.cpu().numpy(), ref, "5 passes vs oracle " + tname)
    util.check_close(capped.cpu().numpy(), ref, "3 passes vs oracle " + tname)
    util.check_close(multi.cpu().numpy(), single.cpu().numpy(), "passes vs single pass " + tname, 1e-3, 1e-3)


def test_prefill_bf16_entry_outputs_and_passes(cuda, lib):
    """the one-call bf16 prefill: a prompt chunk, then a deeper chunk with a bf16 gate, a bf16 result and a scratch that holds
    256 keys at a time (several passes; the running O then lives in the scratch), against the f32 two-call path"""
    import torch
    from p100e_engine_b200 import fast
    kt, n1, T = TYPES["q8_0"], 2000, 100
    pool = util.PagedPool(kt, 10, psh=8, seed=61)
    pt = util.to_dev(pool.take(n1 + T, 9), cuda)
    g = torch.Generator(device="cpu").manual_seed(62)

    def bf(*shape):
        return torch.randn(*shape, generator=g).to(torch.bfloat16).to(cuda)

    pa, pb = torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda), torch.zeros(pool.bytes, dtype=torch.uint8, device=cuda)
    ca, cb = util.dev_cache(pa, pool, pt, None, 9 * 256), util.dev_cache(pb, pool, pt, None, 9 * 256)
    big = torch.empty(fast.attn_prefill_bf16_scratch_bytes(n1, HKV, n1 + T), dtype=torch.uint8, device=cuda)
    for p0, n in ((0, n1), (n1, T)):
        k, v, q, gate = bf(n, HKV, D), bf(n, HKV, D), bf(n, HQ, D), bf(n, HQ * D)
        qr = torch.zeros(n, HQ, D, device=cuda)
        want = torch.zeros(n, HQ, D, device=cuda)
        assert fast.rope_append_bf16(q, k, v, qr, ca, p0, n, HQ, HKV, D, N_ROT, BASE)
        assert fast.attn_prefill_gated(qr, ca, want, gate.float(), n, p0, HQ, SCALE, None, 0)
        if p0 == 0:
            got = torch.zeros(n, HQ, D, device=cuda)
            assert fast.attn_prefill_bf16(q, k, v, None, gate, got, None, None, cb, p0, n, HQ, N_ROT, BASE, SCALE, big, big.numel())
            torch.cuda.synchronize()
            assert torch.equal(got, want), "f32 result of the one-call path differs (bf16 gate widened exactly)"
        else:
            nb = fast.attn_prefill_bf16_scratch_bytes(n, HKV, 256, True)
            small = torch.empty(nb, dtype=torch.uint8, device=cuda)
            got = torch.zeros(n, HQ, D, dtype=torch.bfloat16, device=cuda)
            qb = torch.zeros(_qbuf_bytes(n, HQ * D), dtype=torch.uint8, device=cuda)
            n0 = lib.b200_launch_count()
            assert fast.attn_prefill_bf16(q, k, v, None, gate, None, got, qb, cb, p0, n, HQ, N_ROT, BASE, SCALE, small, nb)
            assert lib.b200_launch_count() - n0 == 1 + 2 * 9      # append + ceil(2100 / 256) passes
            torch.cuda.synchronize()
            util.check_close(got.float().cpu().numpy(), want.cpu().numpy(), "bf16 result over 9 passes", 6e-3, 1e-2)
            assert not fast.attn_prefill_bf16(q, k, v, None, gate, None, got, None, cb, p0, n, HQ, 32, BASE, SCALE, small, nb)   # n_rot 64 only
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    assert torch.equal(pa, pb)


def test_prefill_over_sequence_shards_merges_to_the_unsplit_result(cuda, lib):
    """two sequence shards (pages dealt round-robin) each run b200_attn_prefill_partial over their own keys; the merge of
    the two (O, m, l) with the gate equals the unsplit gated prefill"""
    import torch
    from p100e_engine_b200 import dist as Dm, fast
    kt, p0, T = TYPES["q8_0"], 600, 300
    n = p0 + T
    k = util.rng_normal(71, (n, HKV, D))
    v = util.rng_normal(72, (n, HKV, D))
    q = util.to_dev(util.rng_normal(73, (T, HQ, D)), cuda)
    gate = util.to_dev(util.rng_normal(74, (T, HQ * D)), cuda)
    whole = fast.kv_alloc(kt, n, HKV, D)
    assert fast.kv_append(whole, util.to_dev(k, cuda), util.to_dev(v, cuda), 0, n)
    want = torch.zeros(T, HQ, D, device=cuda)
    assert fast.attn_prefill_gated(q, whole, want, gate, T, p0, HQ, SCALE, None, 0)
    R = T * HQ
    recv = torch.zeros(2, R * (D + 2), device=cuda)
    for r in range(2):
        own = np.nonzero((np.arange(n) >> 8) % 2 == r)[0]
        shard = fast.kv_alloc(kt, len(own), HKV, D)
        assert fast.kv_append(shard, util.to_dev(k[own], cuda), util.to_dev(v[own], cuda), 0, len(own))
        last = Dm.seq_local_positions(np.arange(p0, p0 + T), 2, r)
        buf = recv[r]
        assert fast.attn_prefill_partial(q, shard, buf[:R * D], buf[R * D:R * D + R], buf[R * D + R:], util.to_dev(last, cuda),
                                         int(last.max()) + 1, T, HQ, SCALE, None, 0)
    got = torch.zeros(T, HQ, D, device=cuda)
    assert fast.seq_exchange_merge(0, 2, recv, recv, R, D, gate.view(R, D), got.view(R, D))
    torch.cuda.synchronize()
    assert fast.device_status() == 0
    util.check_close(got.cpu().numpy(), want.cpu().numpy(), "sequence-shard prefill merge", 1e-3, 1e-3)
    # a shard that holds nothing yet gives the empty partial: zero O, m = -inf, l = 0
    empty = fast.kv_alloc(kt, 64, HKV, D)
    buf = torch.full((R * (D + 2),), float("nan"), device=cuda)
    none = torch.full((T,), -1, dtype=torch.int32, device=cuda)
    assert fast.attn_prefill_partial(q, empty, buf[:R * D], buf[R * D:R * D + R], buf[R * D + R:], none, 0, T, HQ, SCALE, None, 0)
    torch.cuda.synchronize()
    assert (buf[:R * D] == 0).all() and torch.isneginf(buf[R * D:R * D + R]).all() and (buf[R * D + R:] == 0).all()


def test_position_beyond_max_n_is_reported_not_read(cuda, lib):
    """a caller that understates max_n: the keys past the limit are left out, the output stays finite and the status word
    carries the position bit (8); the contiguous cache's n_ctx limits a device position the same way"""
    import torch
    from p100e_engine_b200 import fast
    kt, n = TYPES["q8_0"], 3000
    c = fast.kv_alloc(kt, n, HKV, D)
    assert fast.kv_append(c, util.to_dev(util.rng_normal(1, (n, HKV, D)), cuda), util.to_dev(util.rng_normal(2, (n, HKV, D)), cuda), 0, n)
    q = util.to_dev(util.rng_normal(3, (4, HQ, D)), cuda)
    pos = torch.arange(n - 4, n, dtype=torch.int32, device=cuda)
    out = torch.full((4, HQ, D), float("nan"), device=cuda)
    assert fast.attn_decode_slots(q, c, out, None, 1, 4, pos, 1000, HQ, SCALE, 256)      # claims 1000 keys, rows sit at ~3000
    torch.cuda.synchronize()
    assert fast.device_status() == 8
    assert torch.isfinite(out).all()
    # what it computed is attention over the first 1024 keys (4 chunks of 256 cover max_n = 1000)
    hc = orc.Cache(kt, n, HKV, D, c.k.cpu().numpy(), c.v.cpu().numpy())
    ref = orc.attention(q.cpu().numpy(), hc, 4, HQ, SCALE, pos=np.full(4, 1023, np.int32))
    util.check_close(out.cpu().numpy(), ref, "clamped to the chunks that exist")
    p0 = torch.tensor([n + 500], dtype=torch.int32, device=cuda)                       # beyond the cache itself
    assert fast.attn_decode_dev(q, c, out, 1, p0, n, HQ, SCALE)
    torch.cuda.synchronize()
    assert fast.device_status() == 8 and torch.isfinite(out[:1]).all()
    assert fast.device_status() == 0


def test_reserve_then_calls_allocate_nothing(cuda, lib):
    import torch
    from p100e_engine_b200 import fast
    kt, lens = TYPES["q8_0"], [5000, 800, 2500, 64]
    pool, pool_t, pt_t, maxp = _paged_batch(cuda, kt, lens, 81)
    rows = len(lens) * 4
    pos = util.to_dev(np.array([lens[s] - 4 + j for s in range(len(lens)) for j in range(4)], np.int32), cuda)
    rtab = util.to_dev(np.array([s * maxp for s in range(len(lens)) for _ in range(4)], np.int32), cuda)
    c = util.dev_cache(pool_t, pool, pt_t, rtab, maxp << 8)
    q = util.to_dev(util.rng_normal(5, (rows, HQ, D)), cuda)
    out = torch.zeros(rows, HQ, D, device=cuda)
    assert fast.attn_decode_slots(q, c, out, None, len(lens), 4, pos, max(lens), HQ, SCALE, 64)   # kernels loaded, attributes set
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        assert fast.attn_reserve(kt, 8, 4, 8192, maxp << 8, HKV, 64)
        torch.cuda.synchronize()
        free0 = torch.cuda.mem_get_info()[0]
        for chunk in (64, 256, 1024):
            assert fast.attn_decode_slots(q, c, out, None, len(lens), 4, pos, max(lens), HQ, SCALE, chunk)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0, "a call within the reservation allocated device memory"
    assert fast.device_status() == 0


def test_nsplit_setting_moves_the_default_chunk(cuda, lib):
    import torch
    from p100e_engine_b200 import fast
    assert lib.b200_attn_dec2_nsplit(4) == 256 and lib.b200_attn_fixed_chunk(4096) == lib.b200_attn_chunk_keys()
    assert lib.b200_attn_fixed_chunk(1 << 20) == 4096
    kt, n = TYPES["q8_0"], 4096
    c = fast.kv_alloc(kt, n, HKV, D)
    assert fast.kv_append(c, util.to_dev(util.rng_normal(1, (n, HKV, D)), cuda), util.to_dev(util.rng_normal(2, (n, HKV, D)), cuda), 0, n)
    q = util.to_dev(util.rng_normal(3, (1, HQ, D)), cuda)
    a, b = torch.zeros(1, HQ, D, device=cuda), torch.zeros(1, HQ, D, device=cuda)
    assert fast.attn_decode(q, c, a, 1, n - 1, HQ, SCALE)
    try:
        lib.b200_attn_dec2_set_nsplit(4)
        assert lib.b200_attn_dec2_nsplit(4) == 4 and lib.b200_attn_fixed_chunk(n) == 1024
        n0 = lib.b200_launch_count()
        assert fast.attn_decode(q, c, b, 1, n - 1, HQ, SCALE)
        assert lib.b200_launch_count() - n0 == 2
    finally:
        lib.b200_attn_dec2_set_nsplit(0)
    torch.cuda.synchronize()
    assert lib.b200_attn_fixed_chunk(n) == lib.b200_attn_chunk_keys()
    util.check_close(b.cpu().numpy(), a.cpu().numpy(), "4 chunks vs the default split", 1e-3, 1e-3)


def test_device_pool_step_views_and_offload(cuda, lib):
    """the library's pool on the GPU: pages, step descriptor and views drive attn_prep_rows + attn_decode_slots to the same
    bits as hand-built tables; pages_out / pages_in move a sequence to another slot with the same result"""
    import torch
    from p100e_engine_b200 import fast, lib as L, pool as P
    kt, lens, q_len = TYPES["q8_0"], [700, 300, 1200], 4
    pl = P.Pool(kt, HKV, 2, 24, 8, max_slots=4, max_pages=8, max_rows=16, seed=9, device=0)
    rng = np.random.default_rng(91)
    qn = util.to_dev((0.5 + rng.random(D)).astype(np.float32), cuda)
    kn = util.to_dev((0.5 + rng.random(D)).astype(np.float32), cuda)
    layer = 1
    # history of every slot through the sequence view (kv_seq) and kv_append
    for s, n in enumerate(lens):
        assert pl.ensure(s, n - q_len) == L.OK
        cs = pl.view(layer, s)
        assert fast.kv_append(cs, util.to_dev(util.rng_normal(100 + s, (n - q_len, HKV, D)), cuda),
                              util.to_dev(util.rng_normal(200 + s, (n - q_len, HKV, D)), cuda), 0, n - q_len)
    rows = len(lens) * q_len
    assert pl.step([0, 1, 2], [n - q_len for n in lens], q_len, grow=True) == L.OK
    rope_pos, last_key, cache_row, _ = pl.step_arrays()
    assert pl.step_rows() == rows and pl.step_max_n() == max(lens)
    qg = util.to_dev(util.rng_normal(7, (rows, HQ, 2 * D)), cuda)
    k = util.to_dev(util.rng_normal(8, (rows, HKV, D)), cuda)
    v = util.to_dev(util.rng_normal(9, (rows, HKV, D)), cuda)
    q, gate = torch.zeros(rows, HQ, D, device=cuda), torch.zeros(rows, HQ * D, device=cuda)
    cr = pl.view(layer, -1)
    assert fast.attn_prep_rows(qg, k, v, qn, kn, rope_pos, cache_row, q, gate, cr, rows, HQ, HKV, D, N_ROT, BASE, EPS)
    out = torch.zeros(rows, HQ, D, device=cuda)
    assert fast.attn_decode_slots(q, cr, out, gate, len(lens), q_len, last_key, pl.step_max_n(), HQ, SCALE, 256)
    torch.cuda.synchronize()
    # the same through hand-built tensors over the pool's memory
    tab = util.to_dev(pl.table().reshape(-1).copy(), cuda)
    pos = util.to_dev(np.array([lens[s] - q_len + j for s in range(3) for j in range(q_len)], np.int32), cuda)
    rtab = util.to_dev(np.array([s * 8 for s in range(3) for _ in range(q_len)], np.int32), cuda)
    hand = fast.kv_cache(kt, 8 << 8, HKV, D, cr.k, cr.v, tab, rtab, 8, pl.pstride)
    out2 = torch.zeros(rows, HQ, D, device=cuda)
    assert fast.attn_decode_slots(q, hand, out2, gate, len(lens), q_len, pos, max(lens), HQ, SCALE, 256)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    # offload slot 2 to pinned host memory, release it, bring it back into slot 3 (other pages), decode again
    npg = pl.slot_pages(2)
    host = torch.empty(npg * pl.page_bytes, dtype=torch.uint8).pin_memory()
    assert pl.pages_out(2, 0, npg, host) == L.OK
    torch.cuda.synchronize()
    assert pl.release(2) == L.OK
    assert pl.ensure(1, 300 + 256) == L.OK            # another sequence grabs a page in between
    assert pl.pages_in(3, 0, npg, host) == L.OK and pl.slot_pages(3) == npg
    assert pl.step([0, 1, 3], [n - q_len for n in lens], q_len, grow=False) == L.OK
    _, last_key, _, _ = pl.step_arrays()
    out3 = torch.zeros(rows, HQ, D, device=cuda)
    assert fast.attn_decode_slots(q, pl.view(layer, -1), out3, gate, len(lens), q_len, last_key, pl.step_max_n(), HQ, SCALE, 256)
    torch.cuda.synchronize()
    assert torch.equal(out3, out), "a sequence restored from its offloaded pages decodes differently"
    assert fast.device_status() == 0
    pl.close()


@pytest.mark.parametrize("tname", ["q8_0", "f16", "q4_0"])
def test_fill_slots_does_not_depend_on_the_sharding(cuda, lib, tname):
    """b200_kv_fill_slots: the same (slot, position, head) holds the same bytes in an unsharded pool and in a pool that
    holds kv heads 2..3 of sequence shard 1 of 2"""
    import torch
    from p100e_engine_b200 import fast, pool as P
    kt, lens = TYPES[tname], [700, 1300]
    hb = orc.row_bytes(kt, 1, D)
    whole = P.Pool(kt, 4, 1, 12, 8, max_slots=2, max_pages=8, max_rows=4, seed=3, device=0)
    part = P.Pool(kt, 2, 1, 8, 8, max_slots=2, max_pages=4, max_rows=4, seed=4, n_seq=2, seq_rank=1, device=0)
    for s, n in enumerate(lens):
        assert whole.ensure(s, n) == 0 and part.ensure(s, n) == 0
    lw = util.to_dev(np.array(lens, np.int32), cuda)
    lp = util.to_dev(np.array([part.local_length(n) for n in lens], np.int32), cuda)
    assert fast.kv_fill_slots(whole.view(0, -1), 2, lw, 8, 77, 0, 1, 0)
    assert fast.kv_fill_slots(part.view(0, -1), 2, lp, 4, 77, 2, 2, 1)
    torch.cuda.synchronize()

    def slot_rows(pl, s):   # the slot's pages in the offload layout [page][K|V][row][row bytes] (one layer)
        npg = pl.slot_pages(s)
        buf = np.zeros(npg * pl.page_bytes, np.uint8)
        assert pl.pages_out(s, 0, npg, buf) == 0
        torch.cuda.synchronize()
        return buf.reshape(npg, 2, 256, pl.rowb)

    for s, n in enumerate(lens):
        rw, rp = slot_rows(whole, s), slot_rows(part, s)
        checked = 0
        for gpos in (0, 255, 256, 300, 511, 512, 700, n - 1):
            page = gpos >> 8
            if gpos >= n or page % 2 != 1:
                continue
            lpos = ((page // 2) << 8) + (gpos & 255)
            for kv in range(2):
                assert np.array_equal(rw[page, kv, gpos & 255, 2 * hb:4 * hb], rp[lpos >> 8, kv, lpos & 255, :]), (s, gpos, kv)
            checked += 1
        assert checked >= 2
    whole.close()
    part.close()
