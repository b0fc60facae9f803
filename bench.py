#!/usr/bin/env python
"""Benchmark of the paged-KV decode / MTP-verify attention path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME] [--kv TYPE]

Workloads (synthetic, seeded; shapes of the configurations the baseline names):
  whole_box   64 slots x q_len 4, contexts ~U{512..65536}, 16 full-attention layers, paged pool with a seeded page
              permutation (default; the configuration the 1/2/4/8-GPU scaling is defined on)
  verify8     8 slots x q_len 4, contexts ~U{1024..32768}, one layer
  long_q4     16 slots x q_len 1, context 131072 each, q4_0, one layer
  long_q8     the same with a q8_0 cache (plain decode: one query row per slot)
  decode1     1 slot x q_len 1, context 4096, one layer (latency-bound)
  prefill8k   one sequence, 8192 new tokens, no prior context: bf16 Q/K/V -> partial RoPE + quantise + append (q8_0
              pages), tensor-core causal attention over the quantised cache, sigmoid gate; metric = attention
              TFLOP/s with FLOPs = 4 * D * Hq * T^2 / 2 (the reference's count, tests/fast_attn_fold_test.cu:83)
A step = for every layer: attn_prep of the step's rows (norm + partial RoPE + quantise + append into the pages) and
the split-KV attention of all slots with the fused sigmoid gate.  metric = KV bytes read per second, counted once per
slot and layer: sum_slots n_ctx * Hkv * 2 * head_bytes (the reference's own definition, tests/fast_attn_test.cu:277
in the reference project).  Multi-GPU: KV heads sharded over min(N, 4) ranks, pages of each sequence dealt over the
remaining factor with an NCCL (O, m, l) merge; the total workload is fixed (strong scaling).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HQ, HKV, D, PSH = 24, 4, 256, 8
SCALE = 1.0 / 16.0
N_ROT, ROPE_BASE, EPS = 64, 1e7, 1e-6
KV_TYPES = {"f16": 1, "q4_0": 2, "q8_0": 8}
HEAD_BYTES = {1: 512, 2: 144, 8: 272}

# DRAM traffic figures taken from the ncu captures summarised under profiles/ (static: a profiler never runs inside a timed
# bench).  Decode: traffic per algorithmic KV byte on the verify8 capture; it grows in proportion to the keys of a launch.
DRAM_PER_ALGORITHMIC_BYTE = 408.5 / 362.5
PREFILL8K_DRAM_BYTES = 640.1e6

WORKLOADS = {
    # name: (slots, q_len, ctx_lo, ctx_hi, layers, default kv)
    "whole_box": (64, 4, 512, 65536, 16, "q8_0"),
    "verify8": (8, 4, 1024, 32768, 1, "q8_0"),
    "long_q4": (16, 1, 131072, 131072, 1, "q4_0"),
    "long_q8": (16, 1, 131072, 131072, 1, "q8_0"),
    "decode1": (1, 1, 4096, 4096, 1, "q8_0"),
    # chunked causal prefill: one sequence, T new tokens, p0 = 0 (slots, q_len unused; ctx = T)
    "prefill8k": (1, 0, 8192, 8192, 1, "q8_0"),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="whole_box", choices=sorted(WORKLOADS))
    ap.add_argument("--kv", default=None, choices=sorted(KV_TYPES))
    ap.add_argument("--layers", type=int, default=0, help="override the workload's layer count")
    ap.add_argument("--chunk", type=int, default=-1, help="keys per split (-1 = chosen from the batch)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--q-len", type=int, default=0, help="override the workload's query rows per slot (1..4)")
    ap.add_argument("--seed", type=int, default=0xB200)
    return ap.parse_args()


def contexts(args):
    slots, q_len, lo, hi, layers, kv = WORKLOADS[args.workload]
    rng = np.random.default_rng(args.seed)
    n = rng.integers(lo, hi + 1, size=slots).astype(np.int64) if hi > lo else np.full(slots, lo, np.int64)
    return slots, (args.q_len or q_len), n, (args.layers or layers), KV_TYPES[args.kv or kv]


# ------------------------------------------------------------------------------------------------ clocks ----
class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs (read-only queries)"""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        self.th.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, val in zip(names, f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def clocks_under_load(index, clocks, run_steps, ms_total, steps):
    """A timed region shorter than nvidia-smi's start-up yields no sample: the same steps are then repeated, untimed, for
    about a second with the sampler running, and those samples are reported (marked as taken on a repeat).  The decision
    and the number of repeats follow from the (rank-reduced) time of the timed region, so every rank does the same."""
    if ms_total >= 350.0 or clocks.get("reasons") == ["unavailable"]:
        return clocks
    import torch
    reps = min(20000, int(1200.0 / max(ms_total / max(steps, 1), 1e-3)) + 1)
    clk = ClockSampler(index)
    clk.start()
    time.sleep(0.15)
    for _ in range(reps):
        run_steps()
    torch.cuda.synchronize()
    out = clk.stop()
    out["window"] = "repeat of the timed steps for about a second (the timed region was too short to sample)"
    return out if out.get("samples", 0) > 0 else clocks


# ---------------------------------------------------------------------------------------------- CPU baseline ----
class CpuSample:
    """A bounded sample of the workload for the reference's CPU attention path (the vendored ggml CPU backend's
    flash_attn_ext, prebuilt in oracle/_ref): the largest slots of one layer up to ~200k keys, cache contents
    synthetic in ggml block layout (values do not change the cost)."""

    def __init__(self, args, n_ctx, q_len, kt):
        from oracle import orc
        self.orc, self.kt, self.q_len = orc, kt, q_len
        self.ok = orc.ggml_ref() is not None
        if not self.ok:
            return
        rng = np.random.default_rng(args.seed + 1)
        hb = HEAD_BYTES[kt]
        pick, tot = [], 0
        for s in np.argsort(-n_ctx):
            pick.append(int(s))
            tot += int(n_ctx[s])
            if tot >= 200_000:
                break
        self.caches = []
        for s in pick:
            n = int(n_ctx[s])
            if kt == 1:
                kv = rng.standard_normal((2, n, HKV, D)).astype(np.float16).view(np.uint8).reshape(2, n, HKV, hb)
            else:
                nb = D // 32
                kv = rng.integers(0, 256, size=(2, n, HKV, nb, hb // nb), dtype=np.uint8)
                sc = np.frombuffer(np.float16(1.0 / 127.0 if kt == 8 else 0.125).tobytes(), np.uint8)
                kv[..., 0] = sc[0]
                kv[..., 1] = sc[1]
                kv = kv.reshape(2, n, HKV, hb)
            q = rng.standard_normal((q_len, HQ, D)).astype(np.float32)
            self.caches.append((n, np.ascontiguousarray(kv[0]), np.ascontiguousarray(kv[1]), q))
        self.keys = tot
        self.nbytes = tot * HKV * 2 * hb
        self.desc = "%d largest slots of one layer (%d keys, q_len %d), vendored ggml CPU flash_attn_ext" % (len(pick), tot, q_len)

    def one_pass(self, threads):
        t0 = time.perf_counter()
        for n, k, v, q in self.caches:
            self.orc.ggml_flash_attn(q, k, v, self.kt, n, self.q_len, HQ, HKV, D, SCALE, threads)
        return time.perf_counter() - t0


def base_line(args, slots, q_len, layers):
    return {"metric": "decode_attn_kv_bandwidth", "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "data": "synthetic",
            "config": {"workload": args.workload, "kv": args.kv or WORKLOADS[args.workload][5], "slots": slots,
                       "q_len": q_len, "layers": layers, "heads": "24q/4kv", "head_dim": D, "page": 1 << PSH}}


def run_reference(args):
    """--impl reference: the reference's CPU implementation of the path on this box's host cores (rank 0 only); each
    step is one pass over a bounded sample of the workload."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    slots, q_len, n_ctx, layers, kt = contexts(args)
    threads = os.cpu_count() or 1
    smp = CpuSample(args, n_ctx, q_len, kt)
    if not smp.ok:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libggml_ref.so was not prebuilt"}))
        return
    for _ in range(args.warmup):
        smp.one_pass(threads)
    ts = [smp.one_pass(threads) for _ in range(args.steps)]
    ms = 1e3 * float(np.mean(ts))
    val = smp.nbytes / (ms * 1e-3) / 1e9
    line = base_line(args, slots, q_len, layers)
    line["config"]["step"] = "bounded sample: " + smp.desc
    line.update({"impl": "reference", "value": val, "ms_per_step": ms, "dtype": "q8_0 x q8_0 dot, fp32 accumulate (ggml)",
                 "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "reference", "sample": smp.desc},
                 "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------ GPU arm ----
class Workload:
    """This rank's share of the workload: its KV heads, its pages of every slot, per-layer activations."""

    def __init__(self, args, plan, dev):
        import torch
        from p100e_engine_b200 import fast, pool as P
        self.torch, self.fast = torch, fast
        self.plan, self.dev = plan, dev
        slots, q_len, n_ctx, layers, kt = contexts(args)
        self.slots, self.q_len, self.n_ctx, self.layers, self.kt = slots, q_len, n_ctx, layers, kt
        self.rows = slots * q_len
        hkv, hq = plan.hkv_local, plan.hq_local
        self.hkv, self.hq = hkv, hq
        # global step descriptor: the q_len rows of a slot are its last q_len positions (appended by this step)
        pos_g, rtab = P.step_descriptor(np.arange(slots), n_ctx - q_len, q_len, 0)
        n_loc = np.array([plan.local_length(int(n), PSH) for n in n_ctx], np.int64)
        self.max_pages = int(((n_loc.max() + (1 << PSH) - 1) >> PSH) + 1)
        n_pages = int((((n_loc + (1 << PSH) - 1) >> PSH)).sum() + 4)
        self.layout = P.PoolLayout(kt, hkv, layers, n_pages, PSH, D)
        self.table = P.PageTable(n_pages, slots, self.max_pages, PSH, seed=args.seed + 7)
        for s in range(slots):
            assert self.table.ensure_pages(s, int(n_loc[s]))
        rtab = np.repeat(np.arange(slots) * self.max_pages, q_len).astype(np.int32)
        pos_l = plan.local_positions(pos_g, PSH)                 # last visible local key per row (-1: none here)
        own = (pos_g >> PSH) % plan.n_seq == plan.seq_rank       # rows whose page this rank owns
        crow = np.where(own, pos_l, -1).astype(np.int32)
        self.max_n = int(max(n_loc.max(), 1))
        self.pool = torch.empty(self.layout.total_bytes, dtype=torch.uint8, device=dev)
        self.ptab = torch.from_numpy(self.table.ptab.reshape(-1).copy()).to(dev)
        self.rtab = torch.from_numpy(rtab).to(dev)
        self.pos_g = torch.from_numpy(pos_g).to(dev)
        self.pos_l = torch.from_numpy(pos_l).to(dev)
        self.crow = torch.from_numpy(crow).to(dev)
        self.local_keys = int(n_loc.sum())
        self.kv_bytes_layer = self.local_keys * hkv * 2 * HEAD_BYTES[kt]
        self.total_kv_bytes_layer = int(n_ctx.sum()) * HKV * 2 * HEAD_BYTES[kt]
        # activations (this rank's heads), one set per layer, on the device and in pinned host memory
        g = torch.Generator(device="cpu").manual_seed(args.seed + 100 * plan.rank)
        self.h_qg = [torch.randn(self.rows, hq, 2 * D, generator=g).pin_memory() for _ in range(layers)]
        self.h_k = [torch.randn(self.rows, hkv, D, generator=g).pin_memory() for _ in range(layers)]
        self.h_v = [torch.randn(self.rows, hkv, D, generator=g).pin_memory() for _ in range(layers)]
        self.d_qg = [x.to(dev) for x in self.h_qg]
        self.d_k = [x.to(dev) for x in self.h_k]
        self.d_v = [x.to(dev) for x in self.h_v]
        self.h_out = [torch.empty(self.rows, hq, D).pin_memory() for _ in range(layers)]
        self.qn = (0.5 + torch.rand(D, generator=g)).to(dev)
        self.kn = (0.5 + torch.rand(D, generator=g)).to(dev)
        self.q = torch.empty(self.rows, hq, D, device=dev)
        self.gate = torch.empty(self.rows, hq * D, device=dev)
        self.out = torch.empty(self.rows, hq, D, device=dev)
        # staging buffers for the end-to-end loop (double-buffered by layer parity)
        self.s_qg = [torch.empty_like(self.d_qg[0]) for _ in range(2)]
        self.s_k = [torch.empty_like(self.d_k[0]) for _ in range(2)]
        self.s_v = [torch.empty_like(self.d_v[0]) for _ in range(2)]
        self.chunk = args.chunk
        self.caches = [self.cache(l) for l in range(layers)]
        for l in range(layers):      # finite pseudo-random pages (cost does not depend on the values)
            flat = fast.kv_cache(kt, n_pages << PSH, hkv, D, self.pool.data_ptr() + self.layout.k_offset(l),
                                 self.pool.data_ptr() + self.layout.v_offset(l))
            assert fast.kv_fill_random(flat, 0, n_pages << PSH, args.seed + l)
        self.merge = None
        if plan.n_seq > 1:
            from p100e_engine_b200 import dist as Dm
            import torch.distributed as dist
            groups = [dist.new_group(r) for r in plan.all_merge_groups()]
            self.merge = Dm.SeqMerge(plan, self.rows, hq, D, dev, groups[plan.head_rank])
        torch.cuda.synchronize()

    def cache(self, layer):
        return self.fast.kv_cache(self.kt, self.max_pages << PSH, self.hkv, D, self.pool.data_ptr() + self.layout.k_offset(layer),
                                  self.pool.data_ptr() + self.layout.v_offset(layer), self.ptab, self.rtab, PSH,
                                  self.layout.pstride)

    def layer(self, l, qg, k, v, ev=None):
        """one layer of the step on the current stream: prep (append) + attention + gate"""
        fast, c = self.fast, self.caches[l]
        ok = fast.attn_prep_rows(qg, k, v, self.qn, self.kn, self.pos_g, self.crow, self.q, self.gate, c, self.rows, self.hq,
                                 self.hkv, D, N_ROT, ROPE_BASE, EPS)
        if ev is not None:
            ev[0].record()
        if self.merge is None:
            ok = ok and fast.attn_decode_slots(self.q, c, self.out, self.gate, self.slots, self.q_len, self.pos_l, self.max_n,
                                               self.hq, SCALE, self.chunk)
            if ev is not None:
                ev[1].record()
        else:
            po, pm, pl = self.merge.views()
            ok = ok and fast.attn_decode_slots_partial(self.q, c, po, pm, pl, self.slots, self.q_len, self.pos_l, self.max_n,
                                                       self.hq, SCALE, self.chunk)
            if ev is not None:
                ev[1].record()
            self.merge.exchange_and_merge(self.gate, self.out.view(self.rows * self.hq, D))
        if not ok:
            raise RuntimeError("a library call was refused")

    def step(self, events=None):
        for l in range(self.layers):
            self.layer(l, self.d_qg[l], self.d_k[l], self.d_v[l], None if events is None else events[l])

    def step_e2e(self):
        """the same step with this step's activations coming from pinned host memory and every layer's result read
        back to the host.  Copies run on their own streams, double-buffered by layer parity, so the upload of layer l+1 and
        the read-back of layer l-1 overlap the kernels of layer l; the timed region still contains all of them."""
        torch = self.torch
        main = torch.cuda.current_stream()
        if not hasattr(self, "h2d_stream"):
            self.h2d_stream, self.d2h_stream = torch.cuda.Stream(), torch.cuda.Stream()
            self.ev_in = [torch.cuda.Event() for _ in range(2)]      # staging b uploaded
            self.ev_used = [torch.cuda.Event() for _ in range(2)]    # staging b consumed by its layer
            self.ev_out = [torch.cuda.Event() for _ in range(2)]     # out b written by its layer
            self.ev_read = [torch.cuda.Event() for _ in range(2)]    # out b copied to the host
            self.out2 = [self.out, torch.empty_like(self.out)]
        self.h2d_stream.wait_stream(main)
        self.d2h_stream.wait_stream(main)
        for l in range(self.layers):
            b = l & 1
            with torch.cuda.stream(self.h2d_stream):
                if l >= 2:
                    self.h2d_stream.wait_event(self.ev_used[b])
                self.s_qg[b].copy_(self.h_qg[l], non_blocking=True)
                self.s_k[b].copy_(self.h_k[l], non_blocking=True)
                self.s_v[b].copy_(self.h_v[l], non_blocking=True)
                self.ev_in[b].record(self.h2d_stream)
            main.wait_event(self.ev_in[b])
            if l >= 2:
                main.wait_event(self.ev_read[b])
            self.out = self.out2[b]
            self.layer(l, self.s_qg[b], self.s_k[b], self.s_v[b])
            self.ev_used[b].record(main)
            self.ev_out[b].record(main)
            with torch.cuda.stream(self.d2h_stream):
                self.d2h_stream.wait_event(self.ev_out[b])
                self.h_out[l].copy_(self.out2[b], non_blocking=True)
                self.ev_read[b].record(self.d2h_stream)
        main.wait_stream(self.h2d_stream)
        main.wait_stream(self.d2h_stream)
        self.out = self.out2[0]

    def e2e_bytes(self):
        h2d = sum(x.numel() * 4 for x in (self.h_qg[0], self.h_k[0], self.h_v[0])) * self.layers
        d2h = self.h_out[0].numel() * 4 * self.layers
        return h2d, d2h


def run_b200(args):
    import torch
    import torch.distributed as dist
    from p100e_engine_b200 import dist as Dm, lib as L

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (this path has no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = L.load()
    plan = Dm.ShardPlan(world, rank, HKV, 6)
    wl = Workload(args, plan, dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, events=None):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(steps):
            fn(None if events is None else events[i])
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        wl.step()
    barrier()
    # ---- device-resident timing (inputs in HBM), with per-call events around the attention launches ----
    events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(wl.layers)]
              for _ in range(args.steps)]
    clk = ClockSampler(local)
    clk.start()
    n0 = lib.b200_launch_count()
    ms_total = timed(lambda ev: wl.step(ev), args.steps, events)
    launches = lib.b200_launch_count() - n0
    clocks = clocks_under_load(local, clk.stop(), lambda: wl.step(None), ms_total, args.steps)
    att_ms = [e0.elapsed_time(e1) for st in events for (e0, e1) in st]
    att_ms_avg = float(np.mean(att_ms))
    # ---- end to end: host buffers in, host results out ----
    for _ in range(3):
        wl.step_e2e()
    ms_e2e = timed(lambda ev: wl.step_e2e(), args.steps)
    status = lib.b200_last_device_status(None)
    if status:
        raise SystemExit("bench.py: a kernel recorded device status %d" % status)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    ms_step = ms_total / args.steps
    total_bytes = wl.total_kv_bytes_layer * wl.layers
    value = total_bytes / (ms_step * 1e-3) / 1e9
    e2e_ms = ms_e2e / args.steps
    h2d, d2h = wl.e2e_bytes()
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = wl.kv_bytes_layer / (att_ms_avg * 1e-3) / 1e9
    line = base_line(args, wl.slots, wl.q_len, wl.layers)
    line["config"].update({"parallelism": "kv-head shards %d x sequence shards %d" % (plan.n_head_shards, plan.n_seq),
                           "keys_per_layer": int(wl.n_ctx.sum()), "chunk_keys": args.chunk,
                           "l2": "inputs larger than L2 (%.1f GB of KV per step per GPU)" % (wl.kv_bytes_layer * wl.layers / 1e9),
                           "step": "per layer: attn_prep (norm+RoPE+quantise+append) + split-KV attention + sigmoid gate"})
    line.update({"value": value, "ms_per_step": ms_step, "dtype": "f16 operands, fp32 accumulate",
                 "clocks": clocks, "gpu_launches": int(launches),
                 "e2e": {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                         "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
                 "roofline": {"bound": "hbm", "kernel": "decode_part_k (+ merge) per layer call", "achieved": achieved,
                              "peak": peak, "peak_source": "measured" if peaks else "fallback", "unit": "GB/s",
                              "frac": achieved / peak, "traffic": int(DRAM_PER_ALGORITHMIC_BYTE * wl.kv_bytes_layer),
                              "traffic_source": "dram read + write of one ncu capture of decode_part_k on verify8 (408.5 MB for 362.5 MB "
                                                "of KV rows), scaled by the KV bytes of this launch",
                              "avg_launch_ms": att_ms_avg, "algorithmic_bytes_per_launch": int(wl.kv_bytes_layer)}})
    if not args.no_cpu_baseline:
        smp = CpuSample(args, wl.n_ctx, wl.q_len, wl.kt)
        if smp.ok:
            threads = os.cpu_count() or 1
            smp.one_pass(threads)
            reps, t = 0, 0.0
            while reps < 3 or (t < 5.0 and reps < 50):
                t += smp.one_pass(threads)
                reps += 1
            line["cpu_baseline"] = {"value": smp.nbytes / (t / reps) / 1e9, "unit": "GB/s", "cores": threads,
                                    "kind": "reference", "sample": smp.desc + ", %d passes" % reps}
        else:
            line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": 0, "kind": "reference",
                                    "sample": "oracle/_ref/libggml_ref.so was not prebuilt"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_prefill(args):
    """prefill8k on one GPU (N > 1: every rank runs its KV-head shard of the same sequence)"""
    import torch
    import torch.distributed as dist
    from p100e_engine_b200 import dist as Dm, fast, lib as L
    from p100e_engine_b200 import pool as P
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (this path has no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = L.load()
    nshard = min(world, HKV)
    if world > HKV:
        raise SystemExit("bench.py: prefill8k shards KV heads only (N <= 4)")
    hkv, hq = HKV // nshard, HQ // nshard
    T = WORKLOADS[args.workload][2]
    kt = KV_TYPES[args.kv or WORKLOADS[args.workload][5]]
    n_pages = T >> PSH
    layout = P.PoolLayout(kt, hkv, 1, n_pages, PSH, D)
    pool = torch.zeros(layout.total_bytes, dtype=torch.uint8, device=dev)
    pt = torch.from_numpy(np.random.default_rng(args.seed).permutation(n_pages).astype(np.int32)).to(dev)
    c = fast.kv_cache(kt, T, hkv, D, pool.data_ptr() + layout.k_offset(0), pool.data_ptr() + layout.v_offset(0), pt, None, PSH,
                      layout.pstride)
    g = torch.Generator(device="cpu").manual_seed(args.seed + rank)
    h_q = torch.randn(T, hq, D, generator=g).to(torch.bfloat16).pin_memory()
    h_k = torch.randn(T, hkv, D, generator=g).to(torch.bfloat16).pin_memory()
    h_v = torch.randn(T, hkv, D, generator=g).to(torch.bfloat16).pin_memory()
    h_g = torch.randn(T, hq * D, generator=g).pin_memory()
    h_o = torch.empty(T, hq, D).pin_memory()
    d_q, d_k, d_v, d_g = h_q.to(dev), h_k.to(dev), h_v.to(dev), h_g.to(dev)
    s_q, s_k, s_v, s_g = [torch.empty_like(x) for x in (d_q, d_k, d_v, d_g)]
    qr = torch.empty(T, hq, D, device=dev)
    out = torch.empty(T, hq, D, device=dev)
    nb = fast.attn_fold_scratch_bytes(T, hkv, T)
    scratch = torch.empty(nb, dtype=torch.uint8, device=dev)

    def step(q, k, v, gt, ev=None):
        ok = fast.rope_append_bf16(q, k, v, qr, c, 0, T, hq, hkv, D, N_ROT, ROPE_BASE)
        if ev is not None:
            ev[0].record()
        ok = ok and fast.attn_prefill_gated(qr, c, out, gt, T, 0, hq, SCALE, scratch, nb)
        if ev is not None:
            ev[1].record()
        if not ok:
            raise RuntimeError("a library call was refused")

    def step_e2e():
        s_q.copy_(h_q, non_blocking=True); s_k.copy_(h_k, non_blocking=True)
        s_v.copy_(h_v, non_blocking=True); s_g.copy_(h_g, non_blocking=True)
        step(s_q, s_k, s_v, s_g)
        h_o.copy_(out, non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(steps):
            fn(i)
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        step(d_q, d_k, d_v, d_g)
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    clk = ClockSampler(local)
    clk.start()
    n0 = lib.b200_launch_count()
    ms_total = timed(lambda i: step(d_q, d_k, d_v, d_g, events[i]), args.steps)
    launches = lib.b200_launch_count() - n0
    clocks = clocks_under_load(local, clk.stop(), lambda: step(d_q, d_k, d_v, d_g), ms_total, args.steps)
    att_ms = float(np.mean([e0.elapsed_time(e1) for e0, e1 in events]))
    for _ in range(3):
        step_e2e()
    ms_e2e = timed(lambda i: step_e2e(), args.steps)
    if lib.b200_last_device_status(None):
        raise SystemExit("bench.py: a kernel recorded a device status")
    if rank == 0:
        flops = 4.0 * D * HQ * (T * T / 2.0)
        ms_step = ms_total / args.steps
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak = float(peaks.get("bf16_tflops", 1590.0))
        ach = flops / nshard / (att_ms * 1e-3) / 1e12
        line = {"metric": "prefill_attn_tflops", "value": flops / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f16 operands, fp32 accumulate", "data": "synthetic",
                "config": {"workload": args.workload, "kv": args.kv or "q8_0", "T": T, "p0": 0, "heads": "24q/4kv", "head_dim": D,
                           "page": 1 << PSH, "parallelism": "kv-head shards %d" % nshard,
                           "l2": "K/V tile images (%.1f MB) and Q/out (%.0f MB) exceed no cache assumption: inputs larger than L2" % (nb / 1e6, 2 * T * hq * D * 4 / 1e6),
                           "step": "rope_append_bf16 (RoPE + quantise + append) + attn_prefill_gated (dequantise to f16 tiles + tcgen05 attention + gate)"},
                "clocks": clocks, "gpu_launches": int(launches),
                "e2e": {"value": flops / (ms_e2e / args.steps * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e / args.steps,
                        "h2d_bytes_per_step": int(sum(x.numel() * x.element_size() for x in (h_q, h_k, h_v, h_g))),
                        "d2h_bytes_per_step": int(h_o.numel() * 4)},
                "roofline": {"bound": "tensor", "kernel": "kv_tiles_k + prefill_k", "achieved": ach, "peak": peak,
                             "peak_source": "measured burst" if peaks else "fallback", "unit": "TFLOP/s", "frac": ach / peak,
                             "traffic": int(PREFILL8K_DRAM_BYTES) if (T == 8192 and nshard == 1) else None,
                             "traffic_source": "dram read + write of one ncu capture of prefill_k at T = 8192 (bytes)",
                             "avg_launch_ms": att_ms, "algorithmic_flops_per_launch": flops / nshard}}
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                                    "sample": "not timed for prefill: see the decode workloads for the CPU attention baseline"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "prefill8k":
        run_prefill(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
