#!/usr/bin/env python
"""Benchmark of the paged-KV decode / MTP-verify attention path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME] [--kv TYPE]

Workloads (synthetic, seeded; shapes of the configurations the baseline names):
  whole_box   64 slots x q_len 4, contexts ~U{512..65536}, 16 full-attention layers, paged pool with a seeded page
              permutation (default; the configuration the 1/2/4/8-GPU scaling is defined on).  --kv f16 --layers 8 runs
              the f16 variant half the layers at a time (all 16 layers of f16 pages are 139 GB)
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

Every input is a function of (seed, layer, slot, position, global head) only, so the runs at 1, 2, 4 and 8 GPUs solve the
same problem: `out_fingerprint` (64 fixed samples of layer 0's gated output) must agree between them.  The default line
also carries a `prefill` record (the prefill8k workload measured in the same process after the decode region).
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


def rank_of(plan):
    return plan.rank


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="whole_box", choices=sorted(WORKLOADS))
    ap.add_argument("--kv", default=None, choices=sorted(KV_TYPES))
    ap.add_argument("--layers", type=int, default=0, help="override the workload's layer count")
    ap.add_argument("--slots", type=int, default=0, help="override the workload's slot count")
    ap.add_argument("--chunk", type=int, default=-1, help="keys per split (-1 = chosen from the batch)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="leave the prefill record out of the decode line")
    ap.add_argument("--breakdown", action="store_true", help="add per-layer times of the step's parts (an extra eager pass)")
    ap.add_argument("--q-len", type=int, default=0, help="override the workload's query rows per slot (1..4)")
    ap.add_argument("--seq-shards", type=int, default=0, help="force the number of sequence shards (default: only when N > 4)")
    ap.add_argument("--sub-batches", type=int, default=1, help="with sequence shards: the slots go in this many groups on as many streams")
    ap.add_argument("--exchange", default="peers", choices=["peers", "nccl"],
                    help="with sequence shards: partials read in place over peer-mapped buffers (one kernel), or ncclAllGather + merge")
    ap.add_argument("--seed", type=int, default=0xB200)
    return ap.parse_args()


def contexts(args):
    slots, q_len, lo, hi, layers, kv = WORKLOADS[args.workload]
    slots = args.slots or slots
    rng = np.random.default_rng(args.seed)
    n = rng.integers(lo, hi + 1, size=slots).astype(np.int64) if hi > lo else np.full(slots, lo, np.int64)
    return slots, (args.q_len or q_len), n, (args.layers or layers), KV_TYPES[args.kv or kv]


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        return {}


def traffic_ratios():
    """DRAM traffic per algorithmic unit, from the ncu captures summarised under profiles/ (a profiler never runs inside a
    timed bench): profiles/traffic.json names the capture each figure comes from"""
    try:
        return json.load(open(os.path.join(ROOT, "profiles", "traffic.json")))
    except (OSError, ValueError):
        return {}


def usable_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


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
def ggml_rows(rows, kt):
    """cache head rows [n][Hkv][head bytes] -> the same values in ggml block layout (q8_0: the reference keeps a head's 8
    scales first, ggml interleaves {scale, 32 quants}; f16 and q4_0 rows are ggml's layout already)"""
    if kt != 8:
        return np.ascontiguousarray(rows)
    n, h, _ = rows.shape
    sc = rows[:, :, :16].reshape(n, h, 8, 2)
    qs = rows[:, :, 16:].reshape(n, h, 8, 32)
    return np.ascontiguousarray(np.concatenate([sc, qs], axis=3).reshape(n, h, 8 * 34))


class CpuSample:
    """A bounded sample of the workload for the reference's CPU attention path (the vendored ggml CPU backend's
    flash_attn_ext, prebuilt in oracle/_ref): the largest slots of one layer up to ~200k keys.  `fetch(slot)` returns that
    slot's (n, K rows, V rows, q rows) as the workload holds them; without it (the --impl reference arm has no GPU pool)
    the rows are synthetic bytes of the same format."""

    def __init__(self, args, n_ctx, q_len, kt, fetch=None, budget_keys=200_000):
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
            if tot >= budget_keys:
                break
        self.caches = []
        for s in pick:
            n = int(n_ctx[s])
            if fetch is not None:
                n, k, v, q = fetch(s)
                self.caches.append((n, ggml_rows(k, kt), ggml_rows(v, kt), np.ascontiguousarray(q, np.float32)))
                continue
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
        self.desc = "%d largest slots of one layer (%d keys, q_len %d), vendored ggml CPU flash_attn_ext over %s" % (
            len(pick), tot, q_len, "the workload's own quantised rows re-packed to ggml blocks" if fetch is not None
            else "synthetic rows in ggml block layout")

    def one_pass(self, threads, first_only=False):
        t0 = time.perf_counter()
        for n, k, v, q in self.caches[:1] if first_only else self.caches:
            self.orc.ggml_flash_attn(q, k, v, self.kt, n, self.q_len, HQ, HKV, D, SCALE, threads)
        return time.perf_counter() - t0

    def first_bytes(self):
        return self.caches[0][0] * HKV * 2 * HEAD_BYTES[self.kt]


def base_line(args, slots, q_len, layers):
    return {"metric": "decode_attn_kv_bandwidth", "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "data": "synthetic",
            "config": {"workload": args.workload, "kv": args.kv or WORKLOADS[args.workload][5], "slots": slots,
                       "q_len": q_len, "layers": layers, "heads": "24q/4kv", "head_dim": D, "page": 1 << PSH, "seed": args.seed}}


def run_reference(args):
    """--impl reference: the reference's CPU implementation of the path on this box's host cores (rank 0 only); each
    step is one pass over a bounded sample of the workload."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    threads = usable_cores()
    if args.workload == "prefill8k":
        smp = PrefillCpuSample(args)
        if not smp.ok:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libggml_ref.so was not prebuilt"}))
            return
        for _ in range(args.warmup):
            smp.one_pass(threads)
        ms = 1e3 * float(np.mean([smp.one_pass(threads) for _ in range(args.steps)]))
        val = smp.flops / (ms * 1e-3) / 1e12
        line = prefill_base_line(args, 1)
        line["config"]["step"] = "bounded sample: " + smp.desc
        line.update({"impl": "reference", "value": val, "ms_per_step": ms, "dtype": "q8_0 x q8_0 dot, fp32 accumulate (ggml)",
                     "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "reference", "sample": smp.desc},
                     "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        print(json.dumps(line))
        return
    slots, q_len, n_ctx, layers, kt = contexts(args)
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
def dist_setup():
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (this path has no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    return world, rank, local, dev


class Workload:
    """This rank's share of the workload: its KV heads, its pages of every slot, per-layer activations."""

    def __init__(self, args, plan, dev, local):
        import torch
        from p100e_engine_b200 import fast, pool as P
        self.torch, self.fast = torch, fast
        self.plan, self.dev, self.args = plan, dev, args
        slots, q_len, n_ctx, layers, kt = contexts(args)
        self.slots, self.q_len, self.n_ctx, self.layers, self.kt = slots, q_len, n_ctx, layers, kt
        self.rows = slots * q_len
        hkv, hq = plan.hkv_local, plan.hq_local
        self.hkv, self.hq = hkv, hq
        n_loc = np.array([plan.local_length(int(n), PSH) for n in n_ctx], np.int64)
        self.max_pages = int(((n_loc.max() + (1 << PSH) - 1) >> PSH) + 1)
        n_pages = int((((n_loc + (1 << PSH) - 1) >> PSH)).sum() + 4)
        # the pool, its page tables and the step descriptor are the library's (C++): pages handed out in a seeded random order
        self.pool = P.Pool(kt, hkv, layers, n_pages, PSH, D, max_slots=slots, max_pages=self.max_pages, max_rows=self.rows,
                           seed=args.seed + 7 + plan.rank, n_seq=plan.n_seq, seq_rank=plan.seq_rank, device=local)
        for s in range(slots):
            if self.pool.ensure(s, int(n_ctx[s])) != 0:
                raise RuntimeError("pool_ensure refused")
        # one step: the q_len rows of a slot are its last q_len positions (appended by this step)
        if self.pool.step(np.arange(slots), n_ctx - q_len, q_len, grow=False) != 0:
            raise RuntimeError("pool_step refused")
        self.rope_pos, self.last_key, self.cache_row, self.rtab = self.pool.step_arrays()
        self.max_n = self.pool.step_max_n()
        self.local_keys = int(n_loc.sum())
        self.kv_bytes_layer = self.local_keys * hkv * 2 * HEAD_BYTES[kt]
        self.total_kv_bytes_layer = int(n_ctx.sum()) * HKV * 2 * HEAD_BYTES[kt]
        self.caches = [self.pool.view(l, -1) for l in range(layers)]
        lens = torch.from_numpy(n_loc.astype(np.int32)).to(dev)
        for l in range(layers):      # finite pseudo-random pages, a function of (layer, slot, global position, global head)
            assert fast.kv_fill_slots(self.caches[l], slots, lens, self.max_pages, args.seed + 1000 * l, plan.kv_head0, plan.n_seq,
                                      plan.seq_rank)
        # activations of this rank's heads, one set per layer (generated for all heads, then sliced: the same numbers at every N)
        self.h_qg, self.h_k, self.h_v = [], [], []
        q0, k0 = plan.q_head0, plan.kv_head0
        for l in range(layers):
            g = torch.Generator(device="cpu").manual_seed(args.seed * 1000 + l)
            qg = torch.randn(self.rows, HQ, 2 * D, generator=g)
            k = torch.randn(self.rows, HKV, D, generator=g)
            v = torch.randn(self.rows, HKV, D, generator=g)
            self.h_qg.append(qg[:, q0:q0 + hq].contiguous().pin_memory())
            self.h_k.append(k[:, k0:k0 + hkv].contiguous().pin_memory())
            self.h_v.append(v[:, k0:k0 + hkv].contiguous().pin_memory())
        g = torch.Generator(device="cpu").manual_seed(args.seed + 5)
        self.qn = (0.5 + torch.rand(D, generator=g)).to(dev)
        self.kn = (0.5 + torch.rand(D, generator=g)).to(dev)
        self.d_qg = [x.to(dev) for x in self.h_qg]
        self.d_k = [x.to(dev) for x in self.h_k]
        self.d_v = [x.to(dev) for x in self.h_v]
        self.q = torch.empty(self.rows, hq, D, device=dev)
        self.gate = torch.empty(self.rows, hq * D, device=dev)
        self.out = torch.empty(self.rows, hq, D, device=dev)
        self.chunk = args.chunk
        # sequence shards: the shards' partials are merged in place over peer-mapped buffers (one kernel per layer; NCCL
        # all-gather + merge if the mapping is not available or --exchange nccl).  --sub-batches n > 1 puts the slots in n
        # groups on n streams, so that the exchange of one group runs beside the attention of another (inside a layer;
        # layers stay in order)
        self.merge = None
        self.in_group = None
        if plan.n_seq > 1:
            from p100e_engine_b200 import dist as Dm
            import torch.distributed as dist
            groups = [dist.new_group(r) for r in plan.all_merge_groups()]
            group, ranks = groups[plan.head_rank], plan.merge_group_ranks()
            self.nsub = max(1, min(args.sub_batches, slots))
            cut = [slots * i // self.nsub for i in range(self.nsub + 1)]
            self.sub = [(cut[i], cut[i + 1]) for i in range(self.nsub)]
            # one raw NCCL communicator per stream that exchanges (the two sub-batch streams, the upload stream): the
            # collectives are enqueued on those streams themselves
            self.peers = args.exchange == "peers"
            self.comms = [Dm.NcclComm(ranks, group, dev) for _ in range((0 if self.peers else self.nsub) + 1)]
            self.in_comm = self.comms[-1]
            self.group = group
            if self.peers:
                try:
                    self.merge = [Dm.PeerMerge(plan, (b - a) * q_len, hq, D, dev, group) for a, b in self.sub]
                except RuntimeError as e:   # raised on every shard of the group alike
                    if rank_of(plan) == 0:
                        sys.stderr.write("bench.py: %s; exchanging through NCCL instead\n" % e)
                    self.peers = False
                    self.comms = [Dm.NcclComm(ranks, group, dev) for _ in range(self.nsub)] + self.comms
            if not self.peers:
                self.merge = [Dm.SeqMerge(plan, (b - a) * q_len, hq, D, dev, group, self.comms[i]) for i, (a, b) in enumerate(self.sub)]
            self.sub_streams = [torch.cuda.Stream() for _ in range(self.nsub)]
            self.ev_prep = torch.cuda.Event()
            self.ev_sub = [torch.cuda.Event() for _ in range(self.nsub)]
        # scratch of the decode calls sized once for the largest call on every stream that issues them
        streams = [torch.cuda.current_stream()] if self.merge is None else self.sub_streams
        for st in streams:
            with torch.cuda.stream(st):
                assert fast.attn_reserve(kt, slots, q_len, self.max_n, self.max_pages << PSH, hkv, self.chunk)
        torch.cuda.synchronize()

    def sub_cache(self, l, a):
        """the layer's cache view for the rows of slots a..: per-row table offsets start at that sub-batch's first row"""
        import ctypes as C
        from p100e_engine_b200 import lib as L
        c = self.caches[l]
        s = L.KvCache()
        C.memmove(C.byref(s), C.byref(c), C.sizeof(L.KvCache))
        s.rtab = self.rtab + 4 * a * self.q_len
        return s

    def layer(self, l, qg, k, v, ev=None, out=None, halves=None):
        """one layer of the step on the current stream: prep (append) + attention + gate.  halves: the activations arrive as
        n_seq row blocks (each sequence shard uploaded one and they were exchanged), one prep launch per block"""
        fast, c, torch = self.fast, self.caches[l], self.torch
        out = self.out if out is None else out
        if halves is None:
            ok = fast.attn_prep_rows(qg, k, v, self.qn, self.kn, self.rope_pos, self.cache_row, self.q, self.gate, c, self.rows,
                                     self.hq, self.hkv, D, N_ROT, ROPE_BASE, EPS)
        else:
            ok = True
            for (r0, r1), (qg_b, k_b, v_b) in halves:
                cb = self.sub_cache(l, 0)
                cb.rtab = self.rtab + 4 * r0
                ok = ok and fast.attn_prep_rows(qg_b, k_b, v_b, self.qn, self.kn, self.rope_pos + 4 * r0, self.cache_row + 4 * r0,
                                                self.q[r0:r1], self.gate[r0:r1], cb, r1 - r0, self.hq, self.hkv, D, N_ROT, ROPE_BASE, EPS)
        if ev is not None:
            ev[0].record()
        if self.merge is None:
            ok = ok and fast.attn_decode_slots(self.q, c, out, self.gate, self.slots, self.q_len, self.last_key, self.max_n,
                                               self.hq, SCALE, self.chunk)
            if ev is not None:
                ev[1].record()
        else:
            main = torch.cuda.current_stream()
            self.ev_prep.record(main)
            for i, (a, b) in enumerate(self.sub):
                r0, r1 = a * self.q_len, b * self.q_len
                with torch.cuda.stream(self.sub_streams[i]):
                    self.sub_streams[i].wait_event(self.ev_prep)
                    po, pm, pl = self.merge[i].views()
                    ok = ok and fast.attn_decode_slots_partial(self.q[r0:r1], self.sub_cache(l, a), po, pm, pl, b - a, self.q_len,
                                                               self.last_key + 4 * r0, self.max_n, self.hq, SCALE, self.chunk)
                    if ev is not None and i == self.nsub - 1:
                        ev[1].record(self.sub_streams[i])
                    self.merge[i].exchange_and_merge(self.gate[r0:r1], out[r0:r1].view((r1 - r0) * self.hq, D))
                    self.ev_sub[i].record(self.sub_streams[i])
            for e in self.ev_sub:
                main.wait_event(e)
        if not ok:
            raise RuntimeError("a library call was refused")

    def begin_step(self):
        """the rows' positions are those of a model step: the same for every layer (the library then computes the split of
        the batch once per step and stream instead of once per layer call)"""
        nbytes = 4 * self.rows
        if self.merge is None:
            self.fast.attn_step_begin(self.last_key, nbytes)
        else:
            for st in self.sub_streams:
                self.fast.attn_step_begin(self.last_key, nbytes, st)

    def step(self, events=None):
        self.begin_step()
        for l in range(self.layers):
            self.layer(l, self.d_qg[l], self.d_k[l], self.d_v[l], None if events is None else events[l])

    # ---- end to end: host buffers in, host results out
    def e2e_setup(self):
        torch = self.torch
        n_seq, r = self.plan.n_seq, self.plan.seq_rank
        # with sequence shards the pair shares the rows: each uploads and reads back one block, the blocks are exchanged
        cut = [self.rows * i // n_seq for i in range(n_seq + 1)]
        self.blocks = [(cut[i], cut[i + 1]) for i in range(n_seq)]
        self.my = self.blocks[r]
        self.h2d_stream, self.d2h_stream = torch.cuda.Stream(), torch.cuda.Stream()
        self.ev_in = [torch.cuda.Event() for _ in range(2)]      # staging b uploaded (and exchanged)
        self.ev_used = [torch.cuda.Event() for _ in range(2)]    # staging b consumed by its layer
        self.ev_out = [torch.cuda.Event() for _ in range(2)]     # out b written by its layer
        self.ev_read = [torch.cuda.Event() for _ in range(2)]    # out b copied to the host
        self.out2 = [self.out, torch.empty_like(self.out)]
        per_row = self.hq * 2 * D + 2 * self.hkv * D
        nb = self.blocks[0][1] - self.blocks[0][0]
        assert all(b - a == nb for a, b in self.blocks), "rows must split evenly over the sequence shards"
        # staging [parity][shard block][rows of the block x (qg | k | v)]: a block is contiguous, so it is one all-gather unit
        self.stage = [torch.empty(n_seq, nb * per_row, device=self.dev) for _ in range(2)]
        self.h_in = []
        a, b = self.my
        for l in range(self.layers):
            flat = torch.cat([self.h_qg[l][a:b].reshape(-1), self.h_k[l][a:b].reshape(-1), self.h_v[l][a:b].reshape(-1)])
            self.h_in.append(flat.pin_memory())
        self.h_out = [torch.empty(b - a, self.hq, D).pin_memory() for _ in range(self.layers)]
        self.nb = nb

    def block_views(self, stage):
        nb, hq, hkv = self.nb, self.hq, self.hkv
        out = []
        for i, rng in enumerate(self.blocks):
            f = stage[i]
            o1 = nb * hq * 2 * D
            o2 = o1 + nb * hkv * D
            out.append((rng, (f[:o1].view(nb, hq, 2 * D), f[o1:o2].view(nb, hkv, D), f[o2:].view(nb, hkv, D))))
        return out

    def step_e2e(self):
        """the same step with this step's activations coming from pinned host memory and every layer's result read
        back to the host.  Copies run on their own streams, double-buffered by layer parity, so the upload of layer l+1 and
        the read-back of layer l-1 overlap the kernels of layer l; the timed region still contains all of them."""
        torch = self.torch
        import torch.distributed as dist
        main = torch.cuda.current_stream()
        if not hasattr(self, "h2d_stream"):
            self.e2e_setup()
        self.h2d_stream.wait_stream(main)
        self.d2h_stream.wait_stream(main)
        self.begin_step()
        r = self.plan.seq_rank
        a, b_ = self.my
        for l in range(self.layers):
            b = l & 1
            with torch.cuda.stream(self.h2d_stream):
                if l >= 2:
                    self.h2d_stream.wait_event(self.ev_used[b])
                self.stage[b][r].copy_(self.h_in[l], non_blocking=True)
                if self.plan.n_seq > 1:
                    self.in_comm.all_gather_f32(self.stage[b], self.h2d_stream)
                self.ev_in[b].record(self.h2d_stream)
            main.wait_event(self.ev_in[b])
            if l >= 2:
                main.wait_event(self.ev_read[b])
            self.layer(l, None, None, None, out=self.out2[b], halves=self.block_views(self.stage[b]))
            self.ev_used[b].record(main)
            self.ev_out[b].record(main)
            with torch.cuda.stream(self.d2h_stream):
                self.d2h_stream.wait_event(self.ev_out[b])
                self.h_out[l].copy_(self.out2[b][a:b_], non_blocking=True)
                self.ev_read[b].record(self.d2h_stream)
        main.wait_stream(self.h2d_stream)
        main.wait_stream(self.d2h_stream)

    def e2e_bytes(self):
        return self.h_in[0].numel() * 4 * self.layers, self.h_out[0].numel() * 4 * self.layers

    def breakdown(self, steps):
        """per-layer device times of the step's parts from CUDA events on this rank (eager launches, the slots in one batch, no
        overlap between parts), and the host's time to issue a layer"""
        torch, fast = self.torch, self.fast
        names = ["attn_prep", "split plan / work list + attention kernel + merge of the partials"]
        if self.merge is not None:
            import torch.distributed as dist
            from p100e_engine_b200 import dist as Dm
            if self.peers:
                names += ["merge of the shards over peer-mapped partials + gate (one kernel, includes the wait for the peer)"]
                if not hasattr(self, "bd_merge"):
                    self.bd_merge = Dm.PeerMerge(self.plan, self.rows, self.hq, D, self.dev, self.group)
            else:
                names += ["copy into place + all-gather of (O, m, l) in the pair (NCCL)", "merge of the shards + gate"]
                if not hasattr(self, "bd_merge"):
                    self.bd_merge = Dm.SeqMerge(self.plan, self.rows, self.hq, D, self.dev, self.group, self.comms[0])
            mg = self.bd_merge
        acc = np.zeros(len(names))
        host = 0.0
        for it in range(steps + 1):
            ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)] for _ in range(self.layers)]
            torch.cuda.synchronize()
            fast.attn_step_begin(self.last_key, 4 * self.rows)
            t0 = time.perf_counter()
            for l in range(self.layers):
                c = self.caches[l]
                ev[l][0].record()
                ok = fast.attn_prep_rows(self.d_qg[l], self.d_k[l], self.d_v[l], self.qn, self.kn, self.rope_pos, self.cache_row, self.q,
                                         self.gate, c, self.rows, self.hq, self.hkv, D, N_ROT, ROPE_BASE, EPS)
                ev[l][1].record()
                if self.merge is None:
                    ok = ok and fast.attn_decode_slots(self.q, c, self.out, self.gate, self.slots, self.q_len, self.last_key, self.max_n,
                                                       self.hq, SCALE, self.chunk)
                    ev[l][2].record()
                else:
                    po, pm, pl = mg.views()
                    ok = ok and fast.attn_decode_slots_partial(self.q, c, po, pm, pl, self.slots, self.q_len, self.last_key, self.max_n,
                                                               self.hq, SCALE, self.chunk)
                    ev[l][2].record()
                    if self.peers:
                        mg.exchange_and_merge(self.gate, self.out.view(mg.R, D))
                        ev[l][3].record()
                    else:
                        mg.recv[self.plan.seq_rank].copy_(mg.send)
                        mg.comm.all_gather_f32(mg.recv)
                        ev[l][3].record()
                        ok = ok and fast.seq_exchange_merge(0, self.plan.n_seq, mg.send, mg.recv, mg.R, D, self.gate, self.out.view(mg.R, D))
                        ev[l][4].record()
                assert ok
            t1 = time.perf_counter()
            torch.cuda.synchronize()
            if it == 0:
                continue      # warm-up (scratch of this stream, the extra merge buffers)
            host += (t1 - t0) / self.layers
            for l in range(self.layers):
                for i in range(len(names)):
                    acc[i] += ev[l][i].elapsed_time(ev[l][i + 1])
        per = acc / (steps * self.layers) * 1e3
        return {"unit": "us per layer", "parts": {n: round(float(v), 2) for n, v in zip(names, per)},
                "sum": round(float(per.sum()), 2), "host_issue": round(host / steps * 1e6, 2)}

    # ---- checks and samples
    def fingerprint(self, world):
        """64 fixed (row, global head, dim) samples of layer 0's gated output, each taken on the rank that owns the head"""
        torch = self.torch
        self.layer(0, self.d_qg[0], self.d_k[0], self.d_v[0])
        torch.cuda.synchronize()
        rng = np.random.default_rng(self.args.seed + 99)
        rows = rng.integers(0, self.rows, 64)
        heads = rng.integers(0, HQ, 64)
        dims = rng.integers(0, D, 64)
        fp = torch.zeros(64, dtype=torch.float64, device=self.dev)
        o = self.out.double()
        for i in range(64):
            h = int(heads[i]) - self.plan.q_head0
            if 0 <= h < self.hq and self.plan.seq_rank == 0:
                fp[i] = o[int(rows[i]), h, int(dims[i])]
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(fp)
        return [float("%.6g" % x) for x in fp.cpu().tolist()]

    def fetch_slot(self, s):
        """layer 0's K / V rows of slot s as the pool holds them and its q rows after prep (the CPU baseline's input);
        only meaningful on an unsharded rank"""
        torch = self.torch
        n = int(self.n_ctx[s])
        rowb = self.pool.rowb
        tab = self.pool.table()[s]
        npg = (n + 255) >> 8
        buf = torch.empty(2, npg, 256 * rowb, dtype=torch.uint8, device=self.dev)
        region = self.pool.n_pages * self.pool.pstride
        for kv in range(2):
            for i in range(npg):
                assert self.pool.read(kv * self.layers * region + int(tab[i]) * self.pool.pstride, buf[kv, i], 256 * rowb) == 0
        torch.cuda.synchronize()
        rows = buf.cpu().numpy().reshape(2, npg * 256, self.hkv, rowb // self.hkv)[:, :n]
        q = self.q[s * self.q_len:(s + 1) * self.q_len].cpu().numpy()
        return n, rows[0], rows[1], q


def run_b200(args):
    import torch
    import torch.distributed as dist
    from p100e_engine_b200 import dist as Dm, lib as L

    world, rank, local, dev = dist_setup()
    lib = L.load()
    plan = Dm.ShardPlan(world, rank, HKV, 6, args.seq_shards or None)
    wl = Workload(args, plan, dev, local)

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
    barrier()
    ms_e2e = timed(lambda ev: wl.step_e2e(), args.steps)
    status = lib.b200_last_device_status(None)
    if status:
        raise SystemExit("bench.py: a kernel recorded device status %d" % status)
    fingerprint = wl.fingerprint(world)
    bd = wl.breakdown(max(3, min(args.steps, 10))) if args.breakdown else None

    prefill = None
    if args.workload == "whole_box" and not args.no_prefill:
        prefill = prefill_measure(args, world, rank, local, dev, steps=max(3, min(args.steps, 10)), warmup=3,
                                  cpu=not args.no_cpu_baseline)
    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    ms_step = ms_total / args.steps
    total_bytes = wl.total_kv_bytes_layer * wl.layers
    value = total_bytes / (ms_step * 1e-3) / 1e9
    e2e_ms = ms_e2e / args.steps
    h2d, d2h = wl.e2e_bytes()
    peaks = measured_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = wl.kv_bytes_layer / (att_ms_avg * 1e-3) / 1e9
    # the attention kernel of this call: the even split of a q8_0 verify batch runs on the tcgen05 kernel
    tc = bool(L.load().b200_attn_dec_tc()) and args.chunk < 0 and wl.slots > 1 and wl.kt == KV_TYPES["q8_0"] and wl.q_len >= 2
    kname = "decode_tc_k" if tc else "decode_part_k"
    tr = traffic_ratios().get(kname, {})
    line = base_line(args, wl.slots, wl.q_len, wl.layers)
    if plan.n_seq > 1:
        line["config"]["exchange"] = ("partials merged in place over peer-mapped buffers" if wl.peers else "ncclAllGather of the partials + merge") + \
            ", %d sub-batch(es)" % wl.nsub
    line["config"].update({"parallelism": "kv-head shards %d x sequence shards %d" % (plan.n_head_shards, plan.n_seq),
                           "keys_per_layer": int(wl.n_ctx.sum()), "chunk_keys": args.chunk,
                           "l2": "inputs larger than L2 (%.1f GB of KV per step per GPU)" % (wl.kv_bytes_layer * wl.layers / 1e9),
                           "step": "per layer: attn_prep (norm+RoPE+quantise+append) + split-KV attention + sigmoid gate"})
    line.update({"value": value, "ms_per_step": ms_step, "dtype": "f16 operands, fp32 accumulate",
                 "clocks": clocks, "gpu_launches": int(launches), "out_fingerprint": fingerprint,
                 "e2e": {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                         "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
                 "roofline": {"bound": "hbm", "kernel": kname + " (+ split plan / work list, merge of the partials) per layer call", "achieved": achieved,
                              "peak": peak, "peak_source": "measured" if peaks else "fallback", "unit": "GB/s",
                              "frac": achieved / peak,
                              "traffic": int(tr["dram_bytes_per_kv_byte"] * wl.kv_bytes_layer) if tr else None,
                              "traffic_source": tr.get("source"),
                              "avg_launch_ms": att_ms_avg, "algorithmic_bytes_per_launch": int(wl.kv_bytes_layer),
                              "timing": "CUDA events around each layer's attention call on the launching stream, inside the timed region"}})
    if bd is not None:
        line["breakdown"] = bd
    if prefill is not None:
        line["prefill"] = prefill
    if not args.no_cpu_baseline:
        threads = usable_cores()
        smp = CpuSample(args, wl.n_ctx, wl.q_len, wl.kt, fetch=wl.fetch_slot if world == 1 else None)
        if smp.ok:
            smp.one_pass(threads)
            reps, t = 0, 0.0
            while reps < 3 or (t < 5.0 and reps < 50):
                t += smp.one_pass(threads)
                reps += 1
            t1 = smp.one_pass(1, first_only=True)
            line["cpu_baseline"] = {"value": smp.nbytes / (t / reps) / 1e9, "unit": "GB/s", "cores": threads,
                                    "kind": "reference", "sample": smp.desc + ", %d passes" % reps,
                                    "one_thread": {"value": smp.first_bytes() / t1 / 1e9, "unit": "GB/s",
                                                   "sample": "the largest slot alone (%d keys), one pass" % smp.caches[0][0]}}
        else:
            line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": 0, "kind": "reference",
                                    "sample": "oracle/_ref/libggml_ref.so was not prebuilt"}
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------ prefill ----
def prefill_base_line(args, nshard, n_seq=1):
    T = WORKLOADS["prefill8k"][2]
    return {"metric": "prefill_attn_tflops", "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "data": "synthetic",
            "config": {"workload": "prefill8k", "kv": "q8_0", "T": T, "p0": 0, "heads": "24q/4kv", "head_dim": D, "page": 1 << PSH,
                       "parallelism": "kv-head shards %d x sequence shards %d" % (nshard, n_seq), "seed": args.seed}}


class PrefillCpuSample:
    """Bounded CPU sample of the prefill: the last 64 query rows of the sequence (depth 8128..8191, causal among themselves)
    through the vendored ggml flash_attn_ext over the sequence's q8_0 rows; FLOPs by the reference's formula for those rows"""

    def __init__(self, args, k_rows=None, v_rows=None, q=None):
        from oracle import orc
        self.orc = orc
        self.ok = orc.ggml_ref() is not None
        if not self.ok:
            return
        T, self.rows = WORKLOADS["prefill8k"][2], 64
        rng = np.random.default_rng(args.seed + 3)
        if k_rows is None:
            kv = rng.integers(0, 256, size=(2, T, HKV, 8, 34), dtype=np.uint8)
            sc = np.frombuffer(np.float16(1.0 / 127.0).tobytes(), np.uint8)
            kv[..., 0], kv[..., 1] = sc[0], sc[1]
            self.k, self.v = np.ascontiguousarray(kv[0].reshape(T, HKV, 272)), np.ascontiguousarray(kv[1].reshape(T, HKV, 272))
            self.q = rng.standard_normal((self.rows, HQ, D)).astype(np.float32)
            src = "synthetic rows in ggml block layout"
        else:
            self.k, self.v, self.q = ggml_rows(k_rows, 8), ggml_rows(v_rows, 8), np.ascontiguousarray(q, np.float32)
            src = "the sequence's own q8_0 rows re-packed to ggml blocks"
        self.T = T
        self.flops = 4.0 * D * HQ * float(sum(range(T - self.rows + 1, T + 1)))
        self.desc = "the last %d of %d query rows (%.1f GFLOP), vendored ggml CPU flash_attn_ext over %s" % (self.rows, T, self.flops / 1e9, src)

    def one_pass(self, threads):
        t0 = time.perf_counter()
        self.orc.ggml_flash_attn(self.q, self.k, self.v, 8, self.T, self.rows, HQ, HKV, D, SCALE, threads)
        return time.perf_counter() - t0


def prefill_measure(args, world, rank, local, dev, steps, warmup, cpu=True):
    """prefill8k on this rank's shard; returns the record (rank 0) or None.  N <= 4: KV-head shards of the same sequence, the
    one-call bf16 entry point.  N = 8: 4 head shards x 2 sequence shards; each shard appends the pages it owns, computes the
    unnormalised (O, m, l) over its keys, the pair all-gathers them over NCCL and merges with the gate."""
    import torch
    import torch.distributed as dist
    from p100e_engine_b200 import dist as Dm, fast, lib as L, pool as P
    lib = L.load()
    plan = Dm.ShardPlan(world, rank, HKV, 6, args.seq_shards or None)
    hkv, hq, n_seq = plan.hkv_local, plan.hq_local, plan.n_seq
    T = WORKLOADS["prefill8k"][2]
    kt = KV_TYPES["q8_0"]
    n_loc = plan.local_length(T, PSH)
    n_pages = ((n_loc + 255) >> PSH) + 1
    pool = P.Pool(kt, hkv, 1, n_pages, PSH, D, max_slots=1, max_pages=n_pages, max_rows=4, seed=args.seed + 11, n_seq=n_seq,
                  seq_rank=plan.seq_rank, device=local)
    assert pool.ensure(0, T) == 0
    c = pool.view(0, 0)
    g = torch.Generator(device="cpu").manual_seed(args.seed + 17)
    q_all = torch.randn(T, HQ, D, generator=g).to(torch.bfloat16)
    k_all = torch.randn(T, HKV, D, generator=g).to(torch.bfloat16)
    v_all = torch.randn(T, HKV, D, generator=g).to(torch.bfloat16)
    g_all = torch.randn(T, HQ, D, generator=g).to(torch.bfloat16)
    q0, k0 = plan.q_head0, plan.kv_head0
    h_q = q_all[:, q0:q0 + hq].contiguous().pin_memory()
    h_k = k_all[:, k0:k0 + hkv].contiguous().pin_memory()
    h_v = v_all[:, k0:k0 + hkv].contiguous().pin_memory()
    h_g = g_all[:, q0:q0 + hq].contiguous().view(T, hq * D).pin_memory()
    d_q, d_k, d_v, d_g = h_q.to(dev), h_k.to(dev), h_v.to(dev), h_g.to(dev)
    out = torch.empty(T, hq, D, dtype=torch.bfloat16, device=dev)
    nb = fast.attn_prefill_bf16_scratch_bytes(T, hkv, T, True)
    scratch = torch.empty(nb, dtype=torch.uint8, device=dev)
    group = None
    if n_seq > 1:
        groups = [dist.new_group(r) for r in plan.all_merge_groups()]
        group = groups[plan.head_rank]
        comm = Dm.NcclComm(plan.merge_group_ranks(), group, dev)
        qr = torch.empty(T, hq, D, device=dev)
        R = T * hq
        send = torch.empty(R * (D + 2), device=dev)
        recv = torch.empty(n_seq, R * (D + 2), device=dev)
        out32 = torch.empty(T, hq, D, device=dev)
        gate32 = torch.empty(T, hq * D, device=dev)
        last = torch.from_numpy(plan.local_positions(np.arange(T), PSH)).to(dev)
        own_pages = [p for p in range(T >> PSH) if p % n_seq == plan.seq_rank]

    def step(q, k, v, gt, ev=None):
        if n_seq == 1:
            ok = fast.attn_prefill_bf16(q, k, v, None, gt, None, out, None, c, 0, T, hq, N_ROT, ROPE_BASE, SCALE, scratch, nb)
            if ev is not None:
                ev[0].record()
                ev[1].record()
        else:
            ok = fast.rope_append_bf16_at(q, None, None, qr, c, 0, 0, T, hq, hkv, D, N_ROT, ROPE_BASE)
            for p in own_pages:      # the pages this shard owns: local rows, global angles
                t0 = p << PSH
                ok = ok and fast.rope_append_bf16_at(None, k[t0:t0 + 256], v[t0:t0 + 256], None, c, (p // n_seq) << PSH, t0, 256, hq, hkv,
                                                     D, N_ROT, ROPE_BASE)
            if ev is not None:
                ev[0].record()
            ok = ok and fast.attn_prefill_partial(qr, c, send[:R * D], send[R * D:R * D + R], send[R * D + R:], last, n_loc, T, hq, SCALE,
                                                  scratch, nb)
            if ev is not None:
                ev[1].record()
            gate32.copy_(gt)
            ok = ok and fast.seq_exchange_merge(comm.handle, n_seq, send, recv, R, D, gate32.view(R, D), out32.view(R, D))
            out.copy_(out32)
        if not ok:
            raise RuntimeError("a library call was refused")

    # end to end: the next step's inputs upload while this step computes, the previous result reads back meanwhile
    s_in = [[torch.empty_like(x) for x in (d_q, d_k, d_v, d_g)] for _ in range(2)]
    o2 = [torch.empty_like(out) for _ in range(2)]
    h_o = torch.empty(T, hq, D, dtype=torch.bfloat16).pin_memory()
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    ev_up = [torch.cuda.Event() for _ in range(2)]
    ev_used = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_read = [torch.cuda.Event() for _ in range(2)]
    state = {"i": 0}

    def upload(b):
        with torch.cuda.stream(up):
            up.wait_event(ev_used[b])
            for dst, src in zip(s_in[b], (h_q, h_k, h_v, h_g)):
                dst.copy_(src, non_blocking=True)
            ev_up[b].record(up)

    def step_e2e():
        """step i: inputs of step i were uploaded during step i-1 (the first one up front); its result reads back during i+1"""
        main = torch.cuda.current_stream()
        i = state["i"]
        b = i & 1
        if i == 0:
            ev_used[0].record(main)
            ev_used[1].record(main)
            ev_read[0].record(main)
            ev_read[1].record(main)
            upload(0)
        upload(b ^ 1)                      # the next step's inputs, while this one computes
        main.wait_event(ev_up[b])
        main.wait_event(ev_read[b])        # o2[b] was read back
        step(*s_in[b])
        o2[b].copy_(out)
        ev_used[b].record(main)
        ev_done[b].record(main)
        with torch.cuda.stream(down):
            down.wait_event(ev_done[b])
            h_o.copy_(o2[b], non_blocking=True)
            ev_read[b].record(down)
        state["i"] = i + 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):
            fn(i)
        b.record()
        torch.cuda.current_stream().wait_stream(down)
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(warmup, 3)):
        step(d_q, d_k, d_v, d_g)
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    kern_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    clk = ClockSampler(local)
    clk.start()
    n0 = lib.b200_launch_count()

    def timed_step(i):
        kern_ev[i][0].record()
        step(d_q, d_k, d_v, d_g, events[i])
        kern_ev[i][1].record()

    ms_total = timed(timed_step, steps)
    launches = lib.b200_launch_count() - n0
    clocks = clocks_under_load(local, clk.stop(), lambda: step(d_q, d_k, d_v, d_g), ms_total, steps)
    # the attention part of a step: from the end of the append to the end of the attention kernel (N = 8) or, for the
    # one-call entry, the whole call less a separately timed append
    if n_seq > 1:
        att_ms = float(np.mean([e0.elapsed_time(e1) for e0, e1 in events]))
    else:
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(5):
            fast.rope_append_bf16_at(None, d_k, d_v, None, c, 0, 0, T, hq, hkv, D, N_ROT, ROPE_BASE)
        a1.record()
        torch.cuda.synchronize()
        app_ms = a0.elapsed_time(a1) / 5
        att_ms = float(np.mean([e0.elapsed_time(e1) for e0, e1 in kern_ev])) - app_ms
    for _ in range(3):
        step_e2e()
    ms_e2e = timed(lambda i: step_e2e(), steps)
    if lib.b200_last_device_status(None):
        raise SystemExit("bench.py: a prefill kernel recorded a device status")
    cpu_rec = None
    if rank == 0 and cpu:
        k_rows = v_rows = q_rot = None
        if world == 1:   # the CPU path reads the very rows the GPU attended over, and the rotated, unscaled query rows
            rowb = pool.rowb
            tab = pool.table()[0]
            buf = torch.empty(2, T >> PSH, 256 * rowb, dtype=torch.uint8, device=dev)
            region = pool.n_pages * pool.pstride
            for kv in range(2):
                for i in range(T >> PSH):
                    assert pool.read(kv * region + int(tab[i]) * pool.pstride, buf[kv, i], 256 * rowb) == 0
            torch.cuda.synchronize()
            rows = buf.cpu().numpy().reshape(2, T, hkv, rowb // hkv)
            k_rows, v_rows = rows[0], rows[1]
            qr_s = torch.empty(64, hq, D, device=dev)
            assert fast.rope_append_bf16_at(d_q[T - 64:], None, None, qr_s, c, 0, T - 64, 64, hq, hkv, D, N_ROT, ROPE_BASE)
            q_rot = qr_s.cpu().numpy()
        smp = PrefillCpuSample(args, k_rows, v_rows, q_rot)
        if smp.ok:
            threads = usable_cores()
            smp.one_pass(threads)
            reps, t = 0, 0.0
            while reps < 3 or (t < 3.0 and reps < 30):
                t += smp.one_pass(threads)
                reps += 1
            t1 = smp.one_pass(1)
            cpu_rec = {"value": smp.flops / (t / reps) / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "reference",
                       "sample": smp.desc + ", %d passes" % reps,
                       "one_thread": {"value": smp.flops / t1 / 1e12, "unit": "TFLOP/s", "sample": "the same sample, one pass"}}
        else:
            cpu_rec = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "reference", "sample": "oracle/_ref/libggml_ref.so was not prebuilt"}
    pool.close()
    if rank != 0:
        return None
    flops = 4.0 * D * HQ * (T * T / 2.0)
    ms_step = ms_total / steps
    peaks = measured_peaks()
    peak = float(peaks.get("bf16_tflops", 1590.0))
    nshard = plan.n_head_shards
    ach = flops / (nshard * n_seq) / (att_ms * 1e-3) / 1e12
    tr = traffic_ratios().get("prefill_k", {})
    h2d = int(sum(x.numel() * x.element_size() for x in (h_q, h_k, h_v, h_g)))
    rec = {"metric": "prefill_attn_tflops", "unit": "TFLOP/s", "value": flops / (ms_step * 1e-3) / 1e12, "ms_per_step": ms_step,
           "steps": steps, "warmup": warmup, "dtype": "f16 operands, fp32 accumulate",
           "config": {"workload": "prefill8k", "kv": "q8_0", "T": T, "p0": 0,
                      "parallelism": "kv-head shards %d x sequence shards %d" % (nshard, n_seq),
                      "l2": "K/V tile images (%.0f MB) and the bf16 q / gate / result rows (%.0f MB) per GPU: inputs larger than L2" % (
                          T * hkv * 1024 / 1e6, 3 * T * hq * D * 2 / 1e6),
                      "step": ("b200_attn_prefill_bf16: RoPE + quantise + append of K/V, dequantise to f16 tiles, tcgen05 attention with "
                               "in-kernel q rotation, sigmoid gate, bf16 result") if n_seq == 1 else
                              ("per shard: q rotation, append of the owned pages, b200_attn_prefill_partial; NCCL all-gather of (O, m, l) "
                               "inside the pair; merge + gate")},
           "clocks": clocks, "gpu_launches": int(launches),
           "e2e": {"value": flops / (ms_e2e / steps * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e / steps,
                   "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(h_o.numel() * 2),
                   "pcie_bound": "%.0f MB in + %.0f MB out per step cross PCIe; at ~50 GB/s per direction that is %.1f ms, against %.2f ms of kernels: "
                                 "copies are double-buffered and overlap the kernels, the link sets the end-to-end rate" % (
                                     h2d / 1e6, h_o.numel() * 2 / 1e6, h2d / 50e6, ms_step)},
           "roofline": {"bound": "tensor", "kernel": "kv_tiles_k + prefill_k", "achieved": ach, "peak": peak,
                        "peak_source": "measured burst" if peaks else "fallback", "unit": "TFLOP/s", "frac": ach / peak,
                        "traffic": int(tr["dram_bytes"]) if (tr and nshard == 1 and n_seq == 1) else None,
                        "traffic_source": tr.get("source") if tr else None,
                        "avg_launch_ms": att_ms, "algorithmic_flops_per_launch": flops / (nshard * n_seq)}}
    if cpu_rec is not None:
        rec["cpu_baseline"] = cpu_rec
    return rec


def run_prefill(args):
    import torch.distributed as dist
    world, rank, local, dev = dist_setup()
    rec = prefill_measure(args, world, rank, local, dev, steps=args.steps, warmup=args.warmup, cpu=not args.no_cpu_baseline)
    if rank == 0:
        line = prefill_base_line(args, min(world, HKV), max(1, world // HKV))
        line["config"].update(rec.pop("config"))
        line.update(rec)
        line["steps"], line["warmup"] = args.steps, args.warmup
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
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
