"""Generates the committed golden vectors from the REFERENCE's own code.

  python tests/golden/make_golden.py cpu    quantiser vectors from the reference's vendored ggml *_ref quantisers
                                            (oracle/_ref/libggml_ref.so, built by `make -C oracle ref` where the reference
                                            checkout exists) -> tests/golden/quant_ref.npz
  python tests/golden/make_golden.py gpu    attention / attn_prep outputs of the reference's CUDA kernels compiled for
                                            sm_100a (oracle/_ref/libp100e_ref.so), run on a GPU
                                            -> <out dir>/attn_ref_gpu.npz (copy it to tests/golden/)
Inputs are seeded and small; the .npz files hold inputs and outputs so the tests need neither the reference nor a GPU.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
HERE = os.path.dirname(os.path.abspath(__file__))


def quant_inputs():
    rng = np.random.default_rng(20261125)
    rows = [rng.standard_normal(256).astype(np.float32) * s for s in (1.0, 1e-3, 37.0, 1e4)]
    rows += [rng.uniform(-1, 1, 256).astype(np.float32) for _ in range(4)]
    z = np.zeros(256, np.float32)
    rows.append(z.copy())                                      # all zero: d = 0
    t = z.copy(); t[::2] = 1.5; t[1::2] = -1.5; rows.append(t)  # ties: first maximum (positive) wins
    t = z.copy(); t[::2] = -1.5; t[1::2] = 1.5; rows.append(t)  # ties: first maximum (negative) wins
    t = rng.standard_normal(256).astype(np.float32); t[5] = 60000.0; t[40] = -65000.0; rows.append(t)
    t = rng.standard_normal(256).astype(np.float32) * 1e-7; rows.append(t)   # scales in the f16 subnormal range
    t = (rng.integers(-127, 128, 256) / 127.0).astype(np.float32); rows.append(t)   # exact grid points and .5 cases
    t = (np.arange(256) % 32 - 15.5).astype(np.float32) / 8.0; rows.append(t)
    return np.stack(rows)


def make_cpu():
    from oracle import orc
    g = orc.ggml_ref()
    assert g is not None, "build oracle/_ref/libggml_ref.so first (make -C oracle ref)"
    x = quant_inputs()
    n = x.shape[0]
    q8 = np.zeros((n, 8 * 34), np.uint8)
    q4 = np.zeros((n, 8 * 18), np.uint8)
    f16 = np.zeros((n, 256), np.uint16)
    for i in range(n):
        g.ggml_ref_quantize_q8_0(x[i].ctypes.data, q8[i].ctypes.data, 256)
        g.ggml_ref_quantize_q4_0(x[i].ctypes.data, q4[i].ctypes.data, 256)
        f16[i] = [g.ggml_ref_fp32_to_fp16(float(v)) for v in x[i]]
    np.savez_compressed(os.path.join(HERE, "quant_ref.npz"), x=x, q8_ggml_blocks=q8, q4_ggml_blocks=q4, f16=f16)
    print("wrote quant_ref.npz", x.shape)


def make_gpu(outdir):
    import torch
    from oracle import orc
    from tests import util
    r = orc.p100e_ref()
    assert r is not None and torch.cuda.is_available()
    dev = torch.device("cuda:0")
    Hq, Hkv, D, scale = 12, 2, 256, 1.0 / 16.0      # the per-rank shape of a 2-GPU split (reference tests/fast_tinv_test.cu:14)
    out = {}
    n = 120
    k = util.rng_normal(1, (n, Hkv, D))
    v = util.rng_normal(2, (n, Hkv, D))
    q = util.rng_normal(3, (4, Hq, D))
    qp = util.rng_normal(4, (12, Hq, D))
    out.update({"k": k, "v": v, "q": q, "qp": qp})
    for tname, kt in util.TYPES.items():
        rowb = orc.row_bytes(kt, Hkv, D)
        kc = torch.zeros(n * rowb, dtype=torch.uint8, device=dev)
        vc = torch.zeros(n * rowb, dtype=torch.uint8, device=dev)
        c = orc.OrcKv()
        c.type, c.n_ctx, c.Hkv, c.D, c.k, c.v = kt, n, Hkv, D, kc.data_ptr(), vc.data_ptr()
        kd, vd, qd = util.to_dev(k, dev), util.to_dev(v, dev), util.to_dev(q, dev)
        r.ref_kv_append(C.byref(c), kd.data_ptr(), vd.data_ptr(), 0, n, None)
        o = torch.zeros(4, Hq, D, device=dev)
        for T, p0 in ((1, 0), (1, 59), (4, 60), (3, 116)):
            assert r.ref_attn_decode(qd.data_ptr(), C.byref(c), o.data_ptr(), T, p0, Hq, scale, None) == 0
            torch.cuda.synchronize()
            out["%s_dec_%d_%d" % (tname, T, p0)] = o[:T].cpu().numpy().copy()
        op = torch.zeros(12, Hq, D, device=dev)
        assert r.ref_attn_prefill(util.to_dev(qp, dev).data_ptr(), C.byref(c), op.data_ptr(), 12, 108, Hq, scale, None) == 0
        torch.cuda.synchronize()
        out.update({tname + "_kc": kc.cpu().numpy(), tname + "_vc": vc.cpu().numpy(), tname + "_prefill_12_108": op.cpu().numpy()})
    Hq, Hkv = 6, 1
    # attn_prep (norm + RoPE + quantise): q, gate, K/V bytes
    T, n_rot, base, eps = 3, 64, 1e7, 1e-6
    qg = util.rng_normal(11, (T, Hq, 2 * D))
    k = util.rng_normal(12, (T, Hkv, D))
    v = util.rng_normal(13, (T, Hkv, D))
    rng = np.random.default_rng(14)
    qn = (0.2 + rng.random(D)).astype(np.float32)
    kn = (0.2 + rng.random(D)).astype(np.float32)
    pos = np.array([5, 6, 7], np.int32)
    kt = 8
    rowb = orc.row_bytes(kt, Hkv, D)
    kc = torch.zeros(16 * rowb, dtype=torch.uint8, device=dev)
    vc = torch.zeros(16 * rowb, dtype=torch.uint8, device=dev)
    c = orc.OrcKv()
    c.type, c.n_ctx, c.Hkv, c.D, c.k, c.v = kt, 16, Hkv, D, kc.data_ptr(), vc.data_ptr()
    qo = torch.zeros(T, Hq, D, device=dev)
    go = torch.zeros(T, Hq * D, device=dev)
    a = [util.to_dev(x, dev) for x in (qg, k, v, qn, kn, pos)]
    assert r.ref_attn_prep(a[0].data_ptr(), a[1].data_ptr(), a[2].data_ptr(), a[3].data_ptr(), a[4].data_ptr(), a[5].data_ptr(),
                           qo.data_ptr(), go.data_ptr(), C.byref(c), -1, T, Hq, Hkv, D, n_rot, base, eps, None) == 0
    torch.cuda.synchronize()
    out.update({"prep_qg": qg, "prep_k": k, "prep_v": v, "prep_qn": qn, "prep_kn": kn, "prep_pos": pos, "prep_q": qo.cpu().numpy(),
                "prep_gate": go.cpu().numpy(), "prep_kc": kc.cpu().numpy(), "prep_vc": vc.cpu().numpy()})
    os.makedirs(outdir, exist_ok=True)
    np.savez_compressed(os.path.join(outdir, "attn_ref_gpu.npz"), **out)
    print("wrote", os.path.join(outdir, "attn_ref_gpu.npz"))


if __name__ == "__main__":
    if sys.argv[1] == "cpu":
        make_cpu()
    else:
        make_gpu(sys.argv[2] if len(sys.argv) > 2 else os.path.join(ROOT, "tests", "golden"))
