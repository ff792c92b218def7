#!/usr/bin/env python
"""Benchmark of the hot path: paged compressed-KV decode attention (+ fused KV encode).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg3] [--impl ours|reference]

One "step" is one decode step of the whole model shape: for every layer, one
paged decode-attention call over that layer's own compressed KV pool (distinct
pools, so every byte comes from HBM; a layer's pool is far larger than L2).
`value` is whole-job packed-KV bandwidth: algorithmic bytes of all ranks / the
slowest rank's device time.  Under torchrun every rank owns its own batch of
sequences (sequence sharding, no data-path collective; weak scaling).  With
more than one rank the line also carries two strong-scaling sub-records:
`head_sharded` (configuration 4: KV heads split over the ranks, NCCL all-gather
of the outputs inside the timed region) and `ragged_lpt` (configuration 5: ONE
ragged batch of 256 sequences split over the ranks by token count).

After the timed regions the decode output of sampled sequences is compared with
the CPU oracle (`parity`); the oracle is never on the timed path.

--impl reference times the CPU arm: the oracle's restatement of the reference's
unfused path on the host cores (OpenMP over all cores), on a bounded sample of
the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "tq_paged_decode_attn_hbm_gbs"
UNIT = "GB/s"

# Benchmark configurations 2..5 (configuration 1 is the CPU-runnable parity case, not a bench line).
WORKLOADS = {
    # name: layers, B, ctx, Hq, Hkv, D, bits_k, bits_v, ragged
    "cfg2": dict(desc="qwen2.5-0.5b-shaped decode, K3V3", layers=24, B=32, ctx=4096, Hq=14, Hkv=2,
                 D=64, bk=3, bv=3, ragged=False),
    "cfg3": dict(desc="llama-3-8b-shaped decode, K4V4", layers=32, B=64, ctx=8192, Hq=32, Hkv=8,
                 D=128, bk=4, bv=4, ragged=False),
    "cfg4": dict(desc="long-context decode, K3V3, KV heads sharded", layers=32, B=4, ctx=131072,
                 Hq=64, Hkv=8, D=128, bk=3, bv=3, ragged=False),
    "cfg5": dict(desc="mixed-bit ragged serving batch, K4V2", layers=4, B=256, ctx=32768, Hq=16,
                 Hkv=8, D=256, bk=4, bv=2, ragged=True),
}


def packed_dim(d, bits):
    return d * bits // 8


def decode_bytes(seq_lens, Hq, Hkv, D, bk, bv):
    """Algorithmic bytes of one layer's decode call: packed K/V + fp16 norms once per KV head,
    page ids, q in, out (bf16)."""
    tok_head = packed_dim(D, bk) + 2 + packed_dim(D, bv) + 2
    kv = int(sum(int(s) for s in seq_lens)) * Hkv * tok_head
    pages = int(sum((int(s) + 15) // 16 for s in seq_lens)) * 4
    qo = 2 * len(seq_lens) * Hq * D * 2
    return kv + pages + qo


def encode_bytes(n_vec, D, bits, in_bytes=2):
    return n_vec * (D * in_bytes + packed_dim(D, bits) + 2)


class ClockSampler:
    """nvidia-smi clock / throttle-reason sampler running beside the timed regions (read-only)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), f[5:9]):
                if val.lower() == "active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)),
                "reasons": sorted(reasons), "samples": len(sm)}


def make_seq_lens(w, gen):
    if not w["ragged"]:
        return np.full(w["B"], w["ctx"], np.int32)
    # config 5: log-uniform context lengths in [128, 32768]
    u = torch.rand(w["B"], generator=gen).numpy()
    return np.floor(np.exp(math.log(128) + u * (math.log(32768) - math.log(128)))).astype(np.int32)


def synth_kv(n_tok, Hkv, D, cfg_name, gen_dev, device):
    """Synthetic K or V [n_tok, Hkv, D] bf16 with the value distribution the config names."""
    x = torch.randn(n_tok, Hkv, D, device=device, generator=gen_dev, dtype=torch.float32)
    if cfg_name == "cfg2":      # per-head lognormal(0, 0.5) channel scales
        sc = torch.exp(0.5 * torch.randn(Hkv, D, device=device, generator=gen_dev))
        x = x * sc
    elif cfg_name == "cfg3":    # 1% of channels x10
        mask = torch.rand(Hkv, D, device=device, generator=gen_dev) < 0.01
        x = torch.where(mask, x * 10.0, x)
    elif cfg_name == "cfg5":    # Student-t(nu=5)
        chi = torch.randn(5, n_tok, Hkv, D, device=device, generator=gen_dev).pow(2).sum(0) / 5.0
        x = x / chi.sqrt()
    return x.to(torch.bfloat16)


def build_pool(w, cfg_name, seq_lens, layers, Hkv_local, device, seed):
    """Allocate and fill the per-layer pools through the library's own fused store."""
    from fused_turboquant_b200 import PagedKVPool

    B = len(seq_lens)
    max_blocks = int((int(seq_lens.max()) + 15) // 16)
    num_blocks = int(sum((int(s) + 15) // 16 for s in seq_lens))
    pool = PagedKVPool(num_blocks, Hkv_local, w["D"], w["bk"], w["bv"], n_layers=layers,
                       device=device)
    gcpu = torch.Generator("cpu").manual_seed(seed)
    perm = torch.randperm(num_blocks, generator=gcpu).numpy().astype(np.int32)
    bt = np.zeros((B, max_blocks), np.int32)
    pos = 0
    for b in range(B):
        nb = (int(seq_lens[b]) + 15) // 16
        bt[b, :nb] = perm[pos:pos + nb]
        pos += nb
    bt_dev = torch.from_numpy(bt).to(device)
    gdev = torch.Generator(device=device).manual_seed(seed + 1)
    # fill sequence by sequence group so the fp32 staging tensors stay small
    tok_budget = 1 << 17
    for layer in range(layers):
        b0 = 0
        while b0 < B:
            b1, ntok = b0, 0
            while b1 < B and (ntok == 0 or ntok + int(seq_lens[b1]) <= tok_budget):
                ntok += int(seq_lens[b1]); b1 += 1
            slots = torch.cat([
                bt_dev[b, torch.arange(int(seq_lens[b]), device=device) // 16].long() * 16 +
                torch.arange(int(seq_lens[b]), device=device) % 16 for b in range(b0, b1)])
            k = synth_kv(ntok, Hkv_local, w["D"], cfg_name, gdev, device)
            v = synth_kv(ntok, Hkv_local, w["D"], cfg_name, gdev, device)
            pool.store(k, v, slots, layer=layer)
            del k, v
            b0 = b1
    return pool, bt_dev


def cpu_arm(w, seconds_target: float, threads: int):
    """Time the oracle's unfused decode attention on a bounded sample of the workload.

    Returns (GB/s on the same algorithmic bytes, description of the sample)."""
    from fused_turboquant_b200 import codebook
    from oracle import oracle as orc

    orc.set_threads(threads)
    D, bk, bv, Hq, Hkv = w["D"], w["bk"], w["bv"], w["Hq"], w["Hkv"]
    ctx = min(w["ctx"], 8192)
    rng = np.random.default_rng(0)
    signs = codebook.rht_signs(D, 42)
    _, lk = codebook.codebook_f32(D, bk)
    _, lv = codebook.codebook_f32(D, bv)

    def run(B):
        k_idx = rng.integers(0, 256, (B, Hkv, ctx, packed_dim(D, bk)), dtype=np.uint8)
        v_idx = rng.integers(0, 256, (B, Hkv, ctx, packed_dim(D, bv)), dtype=np.uint8)
        k_n = (rng.random((B, Hkv, ctx)) * 4 + 9).astype(np.float16)
        v_n = (rng.random((B, Hkv, ctx)) * 4 + 9).astype(np.float16)
        q = rng.standard_normal((B, Hq, D)).astype(np.float32)
        t = time.perf_counter()
        orc.decode_attn(q, k_idx, k_n, v_idx, v_n, lk, lv, signs, D ** -0.5, bk, bv)
        dt = time.perf_counter() - t
        return dt, decode_bytes([ctx] * B, Hq, Hkv, D, bk, bv)

    dt, nbytes = run(1)                       # calibration (also the warm-up)
    B = int(max(1, min(64, seconds_target / max(dt, 1e-3))))
    dt, nbytes = run(B)
    sample = (f"1 layer, {B} sequences x {Hkv} KV heads x ctx {ctx} of the workload shape, "
              f"oracle decode_attn, {dt:.2f} s")
    return nbytes / dt / 1e9, sample


def cpu_encode_arm(w, seconds_target: float, threads: int):
    """Time the oracle's encode (the reference's _encode_unfused restated) on a bounded sample:
    returns (tokens/s for K and V of all KV heads, sample description)."""
    from fused_turboquant_b200 import codebook
    from oracle import oracle as orc

    orc.set_threads(threads)
    D, Hkv = w["D"], w["Hkv"]
    signs = codebook.rht_signs(D, 42)
    bk_, _ = codebook.codebook_f32(D, w["bk"])
    bv_, _ = codebook.codebook_f32(D, w["bv"])
    rng = np.random.default_rng(1)
    n_tok = 4096
    while True:
        x = rng.standard_normal((n_tok * Hkv, D)).astype(np.float32)
        t = time.perf_counter()
        orc.encode(x, signs, bk_, w["bk"])
        orc.encode(x, signs, bv_, w["bv"])
        dt = time.perf_counter() - t
        if dt >= min(seconds_target, 1.0) or n_tok >= (1 << 18):
            break
        n_tok *= 4
    return n_tok / dt, f"{n_tok} tokens x {Hkv} KV heads, K and V, oracle encode, {dt:.2f} s"


def workload_config(name, w, B, max_seq, layers_per_call, sharding):
    return {"workload": f"{name}: {w['desc']}", "layers": w["layers"], "batch_per_gpu": B,
            "ctx": int(max_seq), "q_heads": w["Hq"], "kv_heads": w["Hkv"], "head_dim": w["D"],
            "key_bits": w["bk"], "value_bits": w["bv"], "page_tokens": 16, "activations": "bf16",
            "sharding": sharding, "layers_per_call": layers_per_call,
            "l2": "inputs larger than L2 (distinct pool per layer)"}


def run_reference_arm(args, w, rank):
    """CPU arm: the oracle's restatement of the reference's unfused CPU path, all host cores,
    every step a bounded sample of the workload (rank 0 only; other ranks exit)."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    vals, times = [], []
    sample = ""
    per_step = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        t = time.perf_counter()
        v, sample = cpu_arm(w, per_step, threads)
        if i >= args.warmup:
            vals.append(v)
            times.append(time.perf_counter() - t)
    value = float(np.mean(vals))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * float(np.mean(times)),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(args.workload, w, w["B"], w["ctx"], 1, "sequences"),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def parity_probe(pool, bt, seq_lens, q_layer0, out_layer0, w, sample_ids):
    """Compare the decode output of sampled sequences of layer 0 with the CPU oracle (outside
    every timed region).  out is bf16: elements outside 1e-3 + 2e-3 |ref| are counted, and how
    many of them differ from the bf16 rounding of the oracle's value by at most one bf16 step."""
    from oracle import oracle as orc

    D, bk, bv = w["D"], w["bk"], w["bv"]
    checked = viol = flips = 0
    max_err = 0.0
    for b in sample_ids:
        S = int(seq_lens[b])
        if S == 0:
            continue
        kc, kn, vc, vn = pool.gather_sequence(0, bt[b], S)
        ref = orc.decode_attn(q_layer0[b:b + 1].float().cpu().numpy(), kc[None].cpu().numpy(),
                              kn[None].cpu().numpy(), vc[None].cpu().numpy(), vn[None].cpu().numpy(),
                              pool.levels_k, pool.levels_v, pool.signs, D ** -0.5, bk, bv)
        got16 = out_layer0[b:b + 1]
        got = got16.float().cpu().numpy()
        bad = np.abs(got - ref) > 1e-3 + 2e-3 * np.abs(ref)
        ref16 = torch.from_numpy(ref).to(torch.bfloat16)
        ulp = (got16.cpu().view(torch.int16).int() - ref16.view(torch.int16).int()).abs().numpy()
        checked += got.size
        viol += int(bad.sum())
        flips += int((bad & (ulp <= 1)).sum())
        max_err = max(max_err, float(np.abs(got - ref).max()))
    return {"checked_elems": checked, "violations": viol, "violations_within_1_bf16_step": flips,
            "max_abs_err": max_err, "gate": "1e-3 + 2e-3*|ref|, bf16 output vs fp32 oracle",
            "sequences": [int(b) for b in sample_ids], "layer": 0}


class Setup:
    """One workload resident on this rank: pools, page table, queries, workspace."""

    def __init__(self, name, w, seq_lens, Hkv_local, Hq_local, device, seed, gen,
                 force_per_layer=False, force_one_call=False):
        self.name, self.w, self.seq_lens, self.device = name, w, seq_lens, device
        self.Hkv, self.Hq, self.L, self.D = Hkv_local, Hq_local, w["layers"], w["D"]
        self.B = len(seq_lens)
        self.max_seq = int(seq_lens.max()) if self.B else 0
        self.pool, self.bt = build_pool(w, name, seq_lens, self.L, Hkv_local, device, seed)
        self.sl = torch.from_numpy(seq_lens).to(device)
        self.q_host = torch.randn(self.L, self.B, Hq_local, self.D, generator=gen) \
            .to(torch.bfloat16).pin_memory()
        self.out_host = torch.empty_like(self.q_host).pin_memory()
        self.q_dev = self.q_host.to(device)
        self.out_dev = torch.empty_like(self.q_dev)
        self.bytes_layer = decode_bytes(seq_lens, Hq_local, Hkv_local, self.D, w["bk"], w["bv"])
        # A layer that moves less than 64 MB is launch-bound on its own: such workloads run all
        # layers in ONE call (layer is a dimension of the kernel's work items).  Larger layers
        # get one call per layer, as an inference engine would issue them.
        # (force_one_call: the record that gathers once per step runs the step as one call at
        # every rank count, not only where a rank's share of a layer is small)
        self.layers_per_call = self.L if (force_one_call or (self.bytes_layer < (64 << 20)
                                                              and not force_per_layer)) else 1
        self.n_calls = self.L // self.layers_per_call
        self.ws = torch.empty(self.pool.workspace_bytes(self.B, Hq_local, self.max_seq,
                                                        self.layers_per_call),
                              dtype=torch.uint8, device=device)

    def call(self, i, qd=None, od=None):
        qd = self.q_dev if qd is None else qd
        od = self.out_dev if od is None else od
        if self.layers_per_call == 1:
            self.pool.decode_attention(qd[i], self.bt, self.sl, self.max_seq, layer=i, out=od[i],
                                       workspace=self.ws)
        else:
            self.pool.decode_attention(qd, self.bt, self.sl, self.max_seq, layer=None, out=od,
                                       workspace=self.ws)

    def step(self, post=None, post_each=None):
        for i in range(self.n_calls):
            self.call(i)
            if post_each is not None:
                post_each(self.out_dev[i] if self.layers_per_call == 1 else self.out_dev)
        return post(self.out_dev) if post is not None else self.out_dev


def device_barrier(world):
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def time_regions(setup, steps, regions, world, post=None, post_each=None):
    """`regions` timed regions of exactly `steps` steps each (barrier + synchronize on both sides,
    CUDA events on the launching stream); returns the per-region milliseconds of this rank."""
    out = []
    for _ in range(regions):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        device_barrier(world)
        e0.record()
        for _ in range(steps):
            setup.step(post, post_each)
        e1.record()
        device_barrier(world)
        out.append(e0.elapsed_time(e1))
    return out


def time_calls(setup, reps):
    """Mean CUDA-event duration of one decode call (all the nodes the call puts into the stream)."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(setup.n_calls)]
    ms = []
    for _ in range(reps):
        for i in range(setup.n_calls):
            evs[i][0].record()
            setup.call(i)
            evs[i][1].record()
        torch.cuda.synchronize()
        ms += [a.elapsed_time(b) for a, b in evs]
    return float(np.mean(ms))


def time_e2e(setup, steps, world, gather=None):
    """The same steps through the public API with HOST buffers: q copied in from pinned memory
    and the outputs copied back inside the timed region."""
    device = setup.device
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    overlap = setup.layers_per_call == 1 and gather is None
    if overlap:
        # One call per layer: the query of layer i+1 is copied in (and the output of layer i-1
        # copied out) on side streams while layer i computes.  Every byte still crosses PCIe inside
        # the timed region, and a step only ends when its last output is in host memory.
        main = torch.cuda.current_stream(device)
        s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        ev_in = [torch.cuda.Event() for _ in range(setup.n_calls)]
        ev_done = [torch.cuda.Event() for _ in range(setup.n_calls)]
        s_in.wait_stream(main)
        s_out.wait_stream(main)
    device_barrier(world)
    e2.record()
    for it in range(steps):
        if overlap:
            for i in range(setup.n_calls):
                with torch.cuda.stream(s_in):
                    if it > 0:
                        s_in.wait_event(ev_done[i])   # last step's layer i no longer reads q_dev[i]
                    setup.q_dev[i].copy_(setup.q_host[i], non_blocking=True)
                    ev_in[i].record(s_in)
            for i in range(setup.n_calls):
                main.wait_event(ev_in[i])
                setup.call(i)
                ev_done[i].record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[i])
                    setup.out_host[i].copy_(setup.out_dev[i], non_blocking=True)
            main.wait_stream(s_out)                   # the step's result is on the host
            continue
        setup.q_dev.copy_(setup.q_host, non_blocking=True)
        res = setup.step(gather)
        if gather is not None:
            res.to("cpu", non_blocking=True)
        else:
            setup.out_host.copy_(res, non_blocking=True)
    e3.record()
    device_barrier(world)
    return e2.elapsed_time(e3), ("per layer on side streams, overlapped with the other layers' compute"
                                 if overlap else "before / after the step on the compute stream")


def reduce_max_sum(vals_max, vals_sum, device, world):
    import torch.distributed as dist
    a = torch.tensor(vals_max, dtype=torch.float64, device=device)
    b = torch.tensor(vals_sum, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(a, op=dist.ReduceOp.MAX)
        dist.all_reduce(b, op=dist.ReduceOp.SUM)
    return [float(x) for x in a], [float(x) for x in b]


def load_peaks():
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        pass
    return float(peaks.get("hbm_gbs", 6650.0)), ("measured" if "hbm_gbs" in peaks else "fallback")


def load_traffic(name, layers_per_call):
    """DRAM read + write bytes of one decode call from the ncu capture recorded for this workload
    (profiles/traffic.json); None when no capture exists for it."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            tab = json.load(f)
        e = tab.get(f"{name}/layers_per_call={layers_per_call}")
        return (float(e["dram_bytes_per_call"]), e["source"]) if e else (None, None)
    except Exception:
        return None, None


def side_workload(name, device, steps, world, gen_seed):
    """A short single-GPU measurement of another configuration (default run only)."""
    w = dict(WORKLOADS[name])
    gen = torch.Generator("cpu").manual_seed(gen_seed)
    seq_lens = make_seq_lens(w, gen)
    s = Setup(name, w, seq_lens, w["Hkv"], w["Hq"], device, seed=31, gen=gen)
    for _ in range(3):
        s.step()
    regs = time_regions(s, steps, 3, world)
    call_ms = time_calls(s, 3)
    peak, _ = load_peaks()
    ms_step = float(np.median(regs)) / steps
    bytes_call = s.bytes_layer * s.layers_per_call
    traffic, src = load_traffic(name, s.layers_per_call)
    rec = {"workload": f"{name}: {w['desc']}", "value": s.bytes_layer * s.L / (ms_step * 1e-3) / 1e9,
           "unit": UNIT, "ms_per_step": ms_step, "steps": steps, "layers_per_call": s.layers_per_call,
           "roofline": {"achieved": bytes_call / (call_ms * 1e-3) / 1e9, "peak": peak,
                        "frac": bytes_call / (call_ms * 1e-3) / 1e9 / peak,
                        "bytes_per_launch": bytes_call, "ms_per_launch": call_ms,
                        "traffic": traffic, "traffic_source": src},
           "parity": parity_probe(s.pool, s.bt, seq_lens, s.q_dev[0], s.out_dev[0], w,
                                  sorted({0, int(seq_lens.argmin())}))}
    del s
    torch.cuda.empty_cache()
    return rec


def head_sharded_record(device, rank, world, steps):
    """Configuration 4 as stated: KV heads split over the ranks (Hkv / world each, with the query
    heads of those groups), every rank holds all four 131 072-token sequences of its heads, and
    the outputs are all-gathered along the head axis over NCCL inside the timed region -- once per
    step (all layers in one call, their outputs in one collective) and, second figure, once per
    layer (one call and one collective per layer: what a model with dependent layers has to do).  Strong scaling: the total work is fixed."""
    from fused_turboquant_b200 import sharding

    w = dict(WORKLOADS["cfg4"])
    if w["Hkv"] % world:
        return {"skipped": f"kv_heads {w['Hkv']} not divisible by {world} ranks"}
    kvr, qr = sharding.shard_kv_heads(w["Hkv"], w["Hq"], world, rank)
    gen = torch.Generator("cpu").manual_seed(20254 + 1000 * rank)
    seq_lens = make_seq_lens(w, gen)
    out = {"workload": f"cfg4: {w['desc']}", "scaling": "strong", "kv_heads_per_rank": len(kvr),
           "q_heads_per_rank": len(qr), "layers": w["layers"], "steps": steps,
           "allgather_bytes_per_rank_per_layer": int(w["B"] * len(qr) * w["D"] * 2)}
    total_bytes_step = decode_bytes(seq_lens, w["Hq"], w["Hkv"], w["D"], w["bk"], w["bv"]) * w["layers"]
    for mode in ("per_step", "per_layer"):
        s = Setup("cfg4", w, seq_lens, len(kvr), len(qr), device, seed=41 + rank, gen=gen,
                  force_per_layer=(mode == "per_layer"), force_one_call=(mode == "per_step"))
        gather = sharding.all_gather_heads
        post, post_each = (gather, None) if mode == "per_step" else (None, gather)
        for _ in range(3):
            s.step(post, post_each)
        regs = time_regions(s, steps, 3, world, post, post_each)          # kernel + all-gather
        regs_k = time_regions(s, steps, 3, world)                         # kernels alone
        (ms, ms_k), _ = reduce_max_sum([float(np.median(regs)), float(np.median(regs_k))], [0.0],
                                       device, world)
        # the collective alone, same message sizes
        n_coll = 1 if mode == "per_step" else s.n_calls
        msg = s.out_dev if mode == "per_step" else s.out_dev[0]
        device_barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps * n_coll):
            gather(msg)
        e1.record()
        device_barrier(world)
        (ms_g,), _ = reduce_max_sum([e0.elapsed_time(e1)], [0.0], device, world)
        out[mode] = {"value": total_bytes_step / (ms / steps * 1e-3) / 1e9, "unit": UNIT,
                     "ms_per_step": ms / steps, "kernel_ms_per_step_max_rank": ms_k / steps,
                     "allgather_ms_per_step_alone": ms_g / steps, "collectives_per_step": n_coll,
                     "layers_per_call": s.layers_per_call,
                     "per_gpu_frac_of_peak": total_bytes_step / world / (ms / steps * 1e-3) / 1e9
                     / load_peaks()[0]}
        del s
        torch.cuda.empty_cache()
    return out


def ragged_lpt_record(device, rank, world, steps):
    """Configuration 5 as stated: ONE ragged batch of 256 sequences (the same draw on every rank)
    split over the ranks by token count (longest-processing-time first); no collective on the
    data path.  Strong scaling; reports the slowest and the fastest rank."""
    import torch.distributed as dist
    from fused_turboquant_b200 import sharding

    w = dict(WORKLOADS["cfg5"])
    gen = torch.Generator("cpu").manual_seed(20255)
    all_lens = make_seq_lens(w, gen)
    owned = sharding.shard_sequences_lpt(all_lens.tolist(), world)[rank]
    seq_lens = all_lens[owned]
    genq = torch.Generator("cpu").manual_seed(77 + rank)
    s = Setup("cfg5", w, seq_lens, w["Hkv"], w["Hq"], device, seed=51 + rank, gen=genq)
    for _ in range(3):
        s.step()
    regs = time_regions(s, steps, 3, world)
    ms_local = float(np.median(regs))
    t = torch.tensor([ms_local, -ms_local, float(seq_lens.sum()), -float(seq_lens.sum())],
                     dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_bytes_step = decode_bytes(all_lens, w["Hq"], w["Hkv"], w["D"], w["bk"], w["bv"]) * w["layers"]
    rec = {"workload": f"cfg5: {w['desc']}", "scaling": "strong", "sequences": int(len(all_lens)),
           "steps": steps, "value": total_bytes_step / (float(t[0]) / steps * 1e-3) / 1e9,
           "unit": UNIT, "ms_per_step_max_rank": float(t[0]) / steps,
           "ms_per_step_min_rank": -float(t[1]) / steps, "tokens_max_rank": int(t[2]),
           "tokens_min_rank": int(-float(t[3])), "partition": "lpt on token counts",
           "per_gpu_frac_of_peak": total_bytes_step / world / (float(t[0]) / steps * 1e-3) / 1e9
           / load_peaks()[0]}
    del s
    torch.cuda.empty_cache()
    return rec


# vLLM-v1 slot-format shapes (--workload tq_*): single GPU, all layer caches in one allocation
TQ_SHAPES = {
    "tq_qwen": dict(desc="slot format, qwen2.5-0.5b shape, K3V3, value rotation", Hq=14, Hkv=2, D=64,
                    kb=3, vb=3, B=32, ctx=4096, layers=24, v_rotate=True),
    "tq_llama": dict(desc="slot format, llama-3-8b shape, K4V4", Hq=32, Hkv=8, D=128, kb=4, vb=4,
                     B=64, ctx=8192, layers=4, v_rotate=False),
    "tq_llama_k8v4": dict(desc="slot format, llama-3-8b shape, FP8 keys, 4-bit values", Hq=32, Hkv=8,
                          D=128, kb=8, vb=4, B=64, ctx=8192, layers=4, v_rotate=False),
}


def run_tq_workload(args):
    """The vLLM-v1 slot-format path (fused store, split-KV decode) on one GPU.  A step decodes
    every layer; layers smaller than 64 MB go through ONE ftq_tq_decode_layers call, larger
    ones one call per layer.  Bytes counted: the slot bytes in use (codes, norm, scale, zero;
    padding excluded) of every attended (token, KV head), block ids, queries and outputs."""
    from fused_turboquant_b200 import tq_v1

    w = TQ_SHAPES[args.workload]
    Hq, Hkv, D, kb, vb, B, ctx, L = (w[k] for k in ("Hq", "Hkv", "D", "kb", "vb", "B", "ctx", "layers"))
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev).manual_seed(20252)
    cfg = tq_v1.TurboQuantSlotConfig(D, kb, vb, norm_correction=True)
    slot, bs = cfg.slot_size_aligned, 16
    blocks_per_seq = ctx // bs
    nb = B * blocks_per_seq
    cent = torch.sort(torch.randn(1 << min(kb, 4), generator=gen, device=dev) / D ** 0.5).values
    cent, mids = tq_v1.midpoints_of(cent)
    caches = torch.zeros((L, nb, bs, Hkv, slot), dtype=torch.uint8, device=dev)
    bt = torch.randperm(nb, generator=gen, device=dev).view(B, blocks_per_seq).to(torch.int32)
    pos = torch.arange(ctx, device=dev)
    slots = (bt.long()[:, pos // bs] * bs + pos % bs).reshape(-1)
    n_tok = B * ctx
    store_ms = []
    for layer in range(L):
        k = torch.randn((n_tok, Hkv, D), generator=gen, device=dev).bfloat16()
        v = torch.randn((n_tok, Hkv, D), generator=gen, device=dev).bfloat16()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        tq_v1.launch_store(k, v, caches[layer], slots, mids, cfg, v_rotate=w["v_rotate"])
        e1.record()
        torch.cuda.synchronize()
        store_ms.append(e0.elapsed_time(e1))
        del k, v
    seq_lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    q = torch.randn((L, B, Hq, D), generator=gen, device=dev).bfloat16()
    used = cfg.slot_size
    layer_bytes = B * ctx * Hkv * used + B * blocks_per_seq * 4 + 2 * B * Hq * D * 2
    batched = layer_bytes < (64 << 20)
    rows = L if batched else 1
    # split count with the lowest modelled cost: waves of (row, KV head, split) items over the
    # persistent CTAs x (pages of an item + the fixed cost of an item, ~15 / 30 pages for a
    # 16- / 8-warp CTA), as the paged path plans its chunks
    per_sm = 1 if 4 in (kb, vb) else 2
    cta_slots = torch.cuda.get_device_properties(dev).multi_processor_count * per_sm
    best = (float("inf"), 1)
    for sp in range(1, 33):
        items = rows * B * Hkv * sp
        cost = -(-items // cta_slots) * (blocks_per_seq / sp + (15.0 if per_sm == 1 else 30.0))
        if cost < best[0] * (1 - 1e-9):
            best = (cost, sp)
    splits = best[1]
    mid_o = torch.empty((rows * B, Hq, splits, D + 1), dtype=torch.float32, device=dev)
    out = torch.empty((L, B, Hq, D), dtype=torch.bfloat16, device=dev)

    def step():
        if batched:
            tq_v1.decode_attention(q, caches, bt, seq_lens, cent, cfg, D ** -0.5, num_kv_splits=splits,
                                   v_rotate=w["v_rotate"], mid_o=mid_o, output=out)
        else:
            for layer in range(L):
                tq_v1.decode_attention(q[layer], caches[layer], bt, seq_lens, cent, cfg, D ** -0.5,
                                       num_kv_splits=splits, v_rotate=w["v_rotate"], mid_o=mid_o,
                                       output=out[layer])

    for _ in range(max(3, args.warmup)):
        step()
    regs = []
    for _ in range(max(1, args.regions)):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        regs.append(e0.elapsed_time(e1))
    ms = float(np.median(regs)) / args.steps
    peak, peak_src = load_peaks()
    value = L * layer_bytes / ms / 1e6
    best_store = min(store_ms[1:]) if L > 1 else store_ms[0]
    store_bytes = n_tok * Hkv * (2 * D * 2 + used)
    print(json.dumps({
        "metric": "tq_v1_decode_attn_hbm_gbs", "value": value, "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "timed_regions_ms": regs,
        "config": {"workload": f"{args.workload}: {w['desc']}", **{k: v for k, v in w.items() if k != "desc"},
                   "splits": splits, "slot_bytes": slot, "layers_per_call": rows,
                   "l2": "distinct layer caches, each step reads all of them"},
        "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": "GB/s",
                     "frac": value / peak, "traffic": None, "peak_source": peak_src},
        "store": {"tokens_per_s": n_tok / best_store * 1e3, "ms": best_store,
                  "gbs": store_bytes / best_store / 1e6},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS) + sorted(TQ_SHAPES))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debug)")
    ap.add_argument("--regions", type=int, default=5,
                    help="timed regions of --steps steps each (the median is reported)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--no-encode", action="store_true", help="skip the encode measurement")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the other workloads (1 GPU) / the strong-scaling sub-records (N GPUs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.workload in TQ_SHAPES:
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the CPU arm times the configuration-2..5 "
                              "workloads only"}), flush=True)
            return
        if not torch.cuda.is_available():
            raise RuntimeError("bench.py needs a CUDA device (no CPU fallback in the product path)")
        run_tq_workload(args)
        return
    w = dict(WORKLOADS[args.workload])
    if args.layers:
        w["layers"] = args.layers
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, w, rank)
        return

    import torch.distributed as dist
    from fused_turboquant_b200 import _lib, sharding

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (no CPU fallback in the product path)")
    _lib.load()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    # ---- main workload: every rank owns its own batch (sequence sharding, weak scaling); with
    # --workload cfg4 on several ranks the KV heads are sharded instead (strong scaling)
    head_sharded = args.workload == "cfg4" and world > 1
    Hkv_local, Hq_local = w["Hkv"], w["Hq"]
    if head_sharded:
        kvr, qr = sharding.shard_kv_heads(w["Hkv"], w["Hq"], world, rank)
        Hkv_local, Hq_local = len(kvr), len(qr)
    gen = torch.Generator("cpu").manual_seed(20250 + int(args.workload[-1]) + 1000 * rank)
    seq_lens = make_seq_lens(w, gen)
    s = Setup(args.workload, w, seq_lens, Hkv_local, Hq_local, device, seed=7 + rank, gen=gen)
    gather = sharding.all_gather_heads if head_sharded else None
    bytes_step = s.bytes_layer * s.L

    for _ in range(args.warmup):
        s.step(gather)
    device_barrier(world)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    torch.cuda.profiler.start()   # ncu --profile-from-start off captures from here
    regions = time_regions(s, args.steps, max(1, args.regions), world, gather)
    call_ms = time_calls(s, min(args.steps, 5))
    torch.cuda.profiler.stop()
    ms_e2e, copies = time_e2e(s, args.steps, world, gather)
    clocks = sampler.stop() if rank == 0 else None

    (ms_total, ms_e2e), (total_bytes_step,) = reduce_max_sum(
        [float(np.median(regions)), ms_e2e], [float(bytes_step)], device, world)

    # ---- parity of what was just timed (rank 0, outside the timed regions)
    parity = None
    if rank == 0 and not head_sharded:
        s.step()
        torch.cuda.synchronize()
        parity = parity_probe(s.pool, s.bt, seq_lens, s.q_dev[0], s.out_dev[0], w,
                              sorted({0, s.B - 1} if not w["ragged"] else
                                     {int(seq_lens.argmin()), int(np.argsort(seq_lens)[len(seq_lens) // 2])}))

    # ---- encode throughput (prefill encode of the same shape), rank-local, summed over ranks
    enc = None
    if not args.no_encode:
        from fused_turboquant_b200 import PagedKVPool
        n_tok = min(int(seq_lens.sum()), 1 << 19)
        gdev = torch.Generator(device=device).manual_seed(99)
        k = synth_kv(n_tok, Hkv_local, s.D, args.workload, gdev, device)
        v = synth_kv(n_tok, Hkv_local, s.D, args.workload, gdev, device)
        nblk = (n_tok + 15) // 16
        epool = PagedKVPool(nblk, Hkv_local, s.D, w["bk"], w["bv"], n_layers=1, device=device)
        slots = torch.randperm(nblk, device=device).repeat_interleave(16)[:n_tok] * 16 + \
            torch.arange(n_tok, device=device) % 16
        for _ in range(3):
            epool.store(k, v, slots, layer=0)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        device_barrier(world)
        a.record()
        for _ in range(reps):
            epool.store(k, v, slots, layer=0)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / reps
        eb = encode_bytes(n_tok * Hkv_local, s.D, w["bk"]) + encode_bytes(n_tok * Hkv_local, s.D, w["bv"])
        (ms,), (tok_total,) = reduce_max_sum([ms], [float(n_tok)], device, world)
        peak, _ = load_peaks()
        enc = {"tokens_per_s": tok_total / (ms * 1e-3), "ms": ms, "tokens": int(tok_total),
               "vectors_per_token": 2 * Hkv_local, "bytes_per_gpu": eb,
               "gbs_per_gpu": eb / (ms * 1e-3) / 1e9, "frac_of_peak": eb / (ms * 1e-3) / 1e9 / peak,
               "launches": 2}
        del k, v, epool

    peak, peak_src = load_peaks()
    line = None
    if rank == 0:
        ms_step = ms_total / args.steps
        value = total_bytes_step / (ms_step * 1e-3) / 1e9
        bytes_call = s.bytes_layer * s.layers_per_call
        traffic, traffic_src = load_traffic(args.workload, s.layers_per_call)
        # 4-bit keys with a GQA group of at most 4 run the streaming kernel (merge and counter
        # reset inside the kernel); the other configurations run attn_mma_kernel behind a memset
        # node, followed by the merge kernel
        fused = w["bk"] == 4 and w["Hq"] // w["Hkv"] <= 4
        # Duration of the dominant kernel's launch.  Where a call is this one kernel and a step is
        # nothing but such calls back to back, it is the timed region divided by its launches
        # (gaps between launches included).  Otherwise (several nodes per call, or a collective
        # inside the step) it is the event-timed duration of one call, timed call by call.
        launch_ms = call_ms
        if fused and gather is None:
            launch_ms = float(np.median(regions)) / (args.steps * s.n_calls)
        achieved = bytes_call / (launch_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if head_sharded else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": workload_config(args.workload, w, s.B, s.max_seq, s.layers_per_call,
                                      "kv-heads+allgather" if head_sharded else "sequences"),
            "timed_regions_ms": regions, "timed_region": f"median of {len(regions)} regions of "
                                                         f"{args.steps} steps each",
            "pct_of_nominal_8000": 100.0 * value / world / 8000.0,
            "decode_tokens_per_s": s.B * world / (ms_step * 1e-3),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_src,
                         "peak_source": peak_src, "frac_of_nominal_8000": achieved / 8000.0,
                         "kernel": ("attn_stream_kernel (one ftq_paged_decode_attn call = this one "
                                    "kernel)" if fused else
                                    "attn_mma_kernel + attn_merge_kernel behind one memset node "
                                    "(one ftq_paged_decode_attn call)")
                                   + ", %d layer(s)" % s.layers_per_call,
                         "bytes_per_launch": bytes_call, "ms_per_launch": launch_ms,
                         "ms_per_call_timed_alone": call_ms},
            "e2e": {"value": total_bytes_step / (ms_e2e / args.steps * 1e-3) / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": int(s.q_host.numel() * 2),
                    "d2h_bytes_per_step": int(s.q_host.numel() * 2 * (world if head_sharded else 1)),
                    "ms_per_step": ms_e2e / args.steps, "copies": copies},
            "gpu_launches": int(args.steps * len(regions) * s.n_calls * (1 if fused else 2)),
            "memset_nodes": 0 if fused else int(args.steps * len(regions) * s.n_calls),
            "clocks": clocks, "parity": parity, "encode": enc,
        }
    del s
    torch.cuda.empty_cache()

    if not args.no_extra:
        if world == 1:
            others = {}
            for name in ("cfg2", "cfg5"):
                if name != args.workload and args.workload == "cfg3" and not args.layers:
                    others[name] = side_workload(name, device, min(args.steps, 10), world,
                                                 20250 + int(name[-1]))
            if rank == 0 and others:
                line["other_workloads"] = others
        elif not head_sharded:
            hs = head_sharded_record(device, rank, world, min(args.steps, 5))
            rl = ragged_lpt_record(device, rank, world, min(args.steps, 5))
            if rank == 0:
                line["head_sharded"] = hs
                line["ragged_lpt"] = rl

    if rank == 0:
        if world == 1 and not args.no_cpu:
            cores = os.cpu_count() or 1
            v, sample = cpu_arm(w, 12.0, cores)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": sample}
            if enc is not None:
                tps, esample = cpu_encode_arm(w, 4.0, cores)
                line["encode"]["cpu_baseline"] = {"tokens_per_s": tps, "cores": cores,
                                                  "kind": "port", "sample": esample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
