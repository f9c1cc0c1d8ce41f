#!/usr/bin/env python
"""Benchmark of the LSH ordering + hierarchical gated-delta forward on B200.

One step = one pass of the hot path over one synthetic 60k-hit event:
  E2LSH bucket ids (3 rounds x 8 hashes) -> 24 stable row sorts -> gather of the hit rows by the
  layer's ordering -> hierarchical (Fenwick-level) chunkwise gated-delta forward (T = 60000 padded
  to 61440, H = 8, K = V = 64, L = 17, bf16) -> scatter of the mixer output back to hit order.
Each rank owns one event (event sharding, no data-path collective).

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # CPU restatement of the reference path

Prints one JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_HITS = 60000
T_PAD = 61440
H, K, V, LEVELS = 8, 64, 64, 17
ROUNDS, HEADS = 3, 8
METRIC = "hits/sec, 60k-hit event LSH+hier. gated-delta fwd"
WORKLOAD = ("config 3 + config 2: E2LSH ids (3x8) + 24 stable sorts + row gather, then hierarchical "
            "gated-delta fwd T=60000 (padded 61440) H=8 K=V=64 L=17 bf16, output scattered back")


def set_event_size(n_hits: int) -> None:
    """Scale the event down (profiler captures, quick checks); the default is the 60k-hit workload."""
    global N_HITS, T_PAD, WORKLOAD
    N_HITS = n_hits
    T_PAD = (n_hits + 1023) // 1024 * 1024
    WORKLOAD = WORKLOAD.replace("T=60000 (padded 61440)", f"T={N_HITS} (padded {T_PAD})") + " [reduced event]"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def make_event(seed: int):
    from lampa_b200 import synth
    inp = synth.gdn_inputs(seed, T_PAD, H, K, V, L=LEVELS, g_shift=2.0)
    for key in ("k", "v", "beta", "g", "lam"):          # padded tokens are inert
        inp[key][:, N_HITS:] = 0
    inp["lam"] = inp["lam"].to(torch.bfloat16)
    hits = synth.detector_hits(seed + 1000, N_HITS)
    alpha, beta = synth.lsh_params(seed + 2000, heads=HEADS, dim=6, rounds=ROUNDS)
    return dict(inp, hits=hits, alpha=alpha, lsh_beta=beta)


# ---- clocks sampler (read-only NVML) ----------------------------------------------------------------
class ClockSampler(threading.Thread):
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag, self.ok = index, [], False, False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.max_sm = None

    def run(self):
        while self.ok and not self.stop_flag:
            try:
                sm = self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)
                rs = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.samples.append((time.perf_counter(), sm, rs))
            except Exception:
                pass
            time.sleep(0.01)

    def summary(self, t0: float, t1: float):
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "NVML unavailable"}
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples[-3:]
        mask = 0
        for s in inside:
            mask |= s[2]
        reasons = [n for b, n in self.REASONS.items() if mask & b and n != "gpu_idle"]
        return {"sm_mhz": float(np.median([s[1] for s in inside])) if inside else None,
                "sm_max_mhz": float(self.max_sm), "reasons": reasons, "samples": len(inside)}


# ---- CPU restatement of the reference path (checker code, timed as the baseline) ---------------------
def cpu_pass(ev, n_tokens: int):
    """One pass of the path over the first n_tokens hits on the host cores; returns seconds."""
    from oracle import oracle
    oracle.set_threads(os.cpu_count() or 1)      # launchers such as torchrun export OMP_NUM_THREADS=1
    a = [ev[k][0, :n_tokens].float().numpy() for k in ("q", "k", "v", "g", "beta", "lam")]
    hits = ev["hits"][:n_tokens].numpy()
    t0 = time.perf_counter()
    ids = oracle.lsh_ids(hits, ev["alpha"].numpy(), ev["lsh_beta"].numpy(), 1.0)
    perms = [oracle.segsort(np.ascontiguousarray(ids[r, h])) for r in range(ROUNDS) for h in range(HEADS)]
    oracle.permute_rows(hits, perms[0])
    o, _, _ = oracle.hgdn(*a, use_l2norm=True)
    oracle.permute_rows(o.reshape(n_tokens, -1), oracle.invert_perm(perms[0]))
    return time.perf_counter() - t0


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ev = make_event(20252)
    cores = os.cpu_count() or 1
    probe_n = 2048
    probe = cpu_pass(ev, probe_n)
    budget = 150.0 / max(1, args.steps + args.warmup)
    n = int(min(N_HITS, max(512, probe_n * budget / max(probe, 1e-6) * 0.6)))
    n = max(64, n // 64 * 64) if n < N_HITS else N_HITS
    for _ in range(args.warmup):
        cpu_pass(ev, n)
    t = [cpu_pass(ev, n) for _ in range(args.steps)]
    tot = float(np.sum(t))
    val = n * args.steps / tot
    sample = (f"first {n} of {N_HITS} hits of the event per step (fewer hits => fewer Fenwick levels, so this "
              f"flatters the CPU); C restatement of the reference's token recurrence, OpenMP over heads")
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "hits/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * tot / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": WORKLOAD},
            "cpu_baseline": {"value": val, "unit": "hits/s", "cores": min(cores, H), "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "hits/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---- this library ------------------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist
    import lampa_b200
    from lampa_b200 import _lib as L

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path in this library)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    ev = make_event(20252 + rank)
    d = {k: v.to(dev) for k, v in ev.items()}
    pinned = {k: v.pin_memory() for k, v in ev.items() if k not in ("alpha", "lsh_beta")}
    stage = {k: torch.empty_like(v, device=dev) for k, v in pinned.items()}
    o_host = torch.empty(N_HITS, H * V, dtype=torch.bfloat16).pin_memory()
    perm_host = torch.empty(N_HITS, dtype=torch.int64).pin_memory()

    def step(t):
        ids = lampa_b200.lsh_hash(t["hits"], d["alpha"], d["lsh_beta"], 1.0)["ids"]
        perm = lampa_b200.segmented_sort(ids, nseg=ROUNDS * HEADS).view(ROUNDS, HEADS, N_HITS)
        order = perm[0, 0]
        lampa_b200.permute_rows(t["hits"], order)
        o, _ = lampa_b200.chunk_h_gated_delta_rule(t["q"], t["k"], t["v"], t["g"], t["lam"], t["beta"],
                                                   use_qk_l2norm_in_kernel=True)
        out = lampa_b200.permute_rows(o[0, :N_HITS].reshape(N_HITS, H * V), order, scatter=True)
        return out, order

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        t1 = time.perf_counter()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), t0, t1

    # End-to-end leg: host buffers in, host buffers out, every step.  Copies run on their own
    # streams and are double-buffered so that step i+1's upload and step i-1's download overlap
    # step i's kernels; all three are inside the timed region.
    stages = [stage, {k: torch.empty_like(v) for k, v in stage.items()}]
    outs_host = [(o_host, perm_host),
                 (torch.empty_like(o_host).pin_memory(), torch.empty_like(perm_host).pin_memory())]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    e2e_count = [0]

    def e2e_step():
        i = e2e_count[0]
        b = i & 1
        e2e_count[0] += 1
        cur = torch.cuda.current_stream(dev)
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_free[b])          # kernels of step i-2 no longer read this buffer set
            for kk, hv in pinned.items():
                stages[b][kk].copy_(hv, non_blocking=True)
            ev_in[b].record(s_in)
        cur.wait_event(ev_in[b])
        out, order = step(stages[b])
        ev_free[b].record(cur)
        ev_done[b].record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[b])
            if i >= 2:
                pass                                 # host buffer b was filled two steps ago on this same stream
            outs_host[b][0].copy_(out, non_blocking=True)
            outs_host[b][1].copy_(order, non_blocking=True)
            out.record_stream(s_out)
            order.record_stream(s_out)
            ev_out[b].record(s_out)

    def e2e_drain():
        torch.cuda.current_stream(dev).wait_stream(s_out)

    # Device-resident leg.  Events are independent, so `--streams S` keeps S of them in flight, each on its own
    # stream with its own inputs and its own intermediates: kernels that cannot fill the GPU alone (the 120-CTA
    # sort, the 40-CTA level scan, the second, partly empty round of the output pass) overlap with the other
    # event's kernels.  S = 1 is the plain back-to-back sequence and is always reported beside it.
    n_streams = max(1, args.streams)
    streams = [torch.cuda.Stream(dev) for _ in range(n_streams)]
    inputs = [d] + [{k: v.to(dev) for k, v in make_event(20252 + rank + 1000 * s).items()} for s in range(1, n_streams)]
    step_no = [0]

    graphs = [None] * n_streams

    def step_concurrent():
        k = step_no[0] % n_streams
        step_no[0] += 1
        with torch.cuda.stream(streams[k]):
            if graphs[k] is not None:
                graphs[k].replay()
                return None
            return step(inputs[k])

    def capture_graphs():
        # one CUDA graph per stream: the nine launches and their scratch allocations of a step, replayed
        for k in range(n_streams):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(streams[k]):
                with torch.cuda.graph(g, stream=streams[k]):
                    keep.append(step(inputs[k]))
            graphs[k] = g
        torch.cuda.synchronize()

    keep = []

    def timed_concurrent(steps):
        barrier()
        main = torch.cuda.current_stream(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(main)
        for st_ in streams:
            st_.wait_event(e0)
        for _ in range(steps):
            step_concurrent()
        for st_ in streams:
            main.wait_stream(st_)
        e1.record(main)
        barrier()
        t1 = time.perf_counter()
        ms_ = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms_, op=dist.ReduceOp.MAX)
        return float(ms_.item()), t0, t1

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step(d)
    ms_single, t0, t1 = timed(lambda: step(d), args.steps)
    if n_streams > 1 or not args.no_graph:
        for _ in range(max(args.warmup, 3)):
            step_concurrent()
        torch.cuda.synchronize()
        if not args.no_graph:
            capture_graphs()
            for _ in range(max(args.warmup, 3)):
                step_concurrent()
            torch.cuda.synchronize()
        ms, t0, t1 = timed_concurrent(args.steps)
        L.check_status(dev)
    else:
        ms = ms_single
    clocks = sampler.summary(t0, t1)
    L.check_status(dev)

    e2e_steps = max(3, min(args.steps, 50))
    ms_e2e = None
    if not args.no_e2e:
        for _ in range(4):
            e2e_step()
        e2e_drain()

        def e2e_run():
            e2e_step()

        barrier()
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ea.record()
        for _ in range(e2e_steps):
            e2e_run()
        e2e_drain()                                  # the last download is inside the timed region
        eb.record()
        barrier()
        t_e2e = torch.tensor([ea.elapsed_time(eb)], device=dev)
        if world > 1:
            dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
        ms_e2e = float(t_e2e.item())
    sampler.stop_flag = True

    # per-kernel durations (CUDA events recorded by the library around each of its launches)
    prof_steps = max(3, min(args.steps, 20))
    torch.cuda.synchronize()
    L.profile_enable(True)
    for _ in range(prof_steps):
        step(d)
    torch.cuda.synchronize()
    prof = L.profile_read()
    L.profile_enable(False)
    L.check_status(dev)

    if rank == 0:
        pk = peaks()
        per_kernel = {n: {"ms_per_launch": r["ms"] / r["launches"], "launches_per_step": r["launches"] / prof_steps,
                          "ms_per_step": r["ms"] / prof_steps} for n, r in prof.items()}
        tot_k = sum(v["ms_per_step"] for v in per_kernel.values())
        for v in per_kernel.values():
            v["share"] = v["ms_per_step"] / tot_k
        dom = max(per_kernel, key=lambda n: per_kernel[n]["ms_per_step"])
        n_chunks = T_PAD // 64
        n_lev = max(1, (n_chunks - 1).bit_length())
        alg = {   # algorithmic cost of one launch of each kernel on this workload
            "gdn_prep_hier": ("tensor", H * n_chunks * (7 * 524288 + 2 * 174763)),
            "gdn_out_hier": ("tensor", H * n_chunks * (n_lev * 2.5 * 524288)),
            "gdn_out_hier_umma": ("tensor", H * n_chunks * (n_lev * 2.5 * 524288)),
            "gdn_compose": ("tensor", H * n_chunks * 2 * 2 * 64 ** 3),
            "gdn_level_hier": ("tensor", H * (n_chunks // 32) * 5 * 2 * 64 ** 3),
            "lsh_hash": ("hbm", N_HITS * 120),
            "segsort": ("hbm", N_HITS * ROUNDS * HEADS * 68),
            "permute_rows": ("hbm", N_HITS * (16 + 2 * (96 + H * V * 2)) / 2),
            "gdn_plan": ("hbm", 64),
        }
        # DRAM bytes (read + write) per launch on the default workload, from the committed ncu capture
        # profiles/kernels_bench_60k_hier.md
        ncu_traffic = {"gdn_prep_hier": 493.3e6, "gdn_out_hier_umma": 421.4e6, "gdn_compose": 192.3e6,
                       "gdn_level_hier": 6.6e6, "segsort": 5.8e6, "lsh_hash": 5.8e6, "permute_rows": 43.3e6}
        bound, units = alg.get(dom, ("hbm", 0))
        dur_s = per_kernel[dom]["ms_per_launch"] * 1e-3
        if bound == "tensor":
            achieved, peak, unit = units / dur_s / 1e12, pk["bf16_tflops"], "TFLOP/s"
        else:
            achieved, peak, unit = units / dur_s / 1e9, pk["hbm_gbs"], "GB/s"
        h2d = int(sum(v.numel() * v.element_size() for v in pinned.values()))
        d2h = int(o_host.numel() * o_host.element_size() + perm_host.numel() * 8)
        line = {
            "metric": METRIC, "value": world * N_HITS * args.steps / (ms * 1e-3), "unit": "hits/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sharding": "one event per rank, no collective",
                       "streams": n_streams, "cuda_graphs": not args.no_graph,
                       "l2": "inputs (~215 MB/step) and intermediates (~375 MB) exceed the 126 MB L2"},
            "clocks": clocks,
            "e2e": None if ms_e2e is None else {
                "value": world * N_HITS * e2e_steps / (ms_e2e * 1e-3), "unit": "hits/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps},
            "gpu_launches": int(round(sum(v["launches_per_step"] for v in per_kernel.values()) * args.steps)),
            "roofline": {"kernel": dom, "bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                         "frac": achieved / peak,
                         "traffic": ncu_traffic.get(dom) if N_HITS == 60000 else None, "peak_source": pk["source"],
                         "whole_step_hbm_gbs": N_HITS * 4432 / (ms / args.steps * 1e-3) / 1e9},
            "kernels": per_kernel,
            "single_stream": {"value": world * N_HITS * args.steps / (ms_single * 1e-3), "unit": "hits/s",
                              "ms_per_step": ms_single / args.steps},
        }
        if world == 1 and not args.no_cpu:
            cores = os.cpu_count() or 1
            n = N_HITS if not args.cpu_sample else args.cpu_sample
            sec = cpu_pass(ev, n)
            line["cpu_baseline"] = {"value": n / sec, "unit": "hits/s", "cores": min(cores, H), "kind": "port",
                                    "sample": f"one pass over {n} of {N_HITS} hits of the same event ({sec:.1f} s); "
                                              "C restatement of the reference's token recurrence, OpenMP over heads"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_plain(args):
    """Configuration 1 on one GPU: timing of the plain chunkwise rule (not the headline metric)."""
    import lampa_b200
    from lampa_b200 import _lib as L, synth
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    T = 65536
    d = {k: v.to(dev) for k, v in synth.gdn_inputs(20251, T, H, K, V, g_shift=2.0, h0=True).items()}

    def step():
        return lampa_b200.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"],
                                                 output_final_state=True, use_qk_l2norm_in_kernel=True)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    L.profile_enable(True)
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    prof = L.profile_read()
    L.profile_enable(False)
    L.check_status(dev)
    print(json.dumps({
        "metric": "tokens/sec, plain chunkwise gated-delta fwd", "value": T * args.steps / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "config 1: chunk_gated_delta_rule T=65536 H=8 K=V=64 bf16, h0 + final state"},
        "hbm_gbs_algorithmic": T * 4160 / (ms / args.steps * 1e-3) / 1e9,
        "kernels": {n: {"ms_per_launch": r["ms"] / r["launches"]} for n, r in prof.items()}}), flush=True)


def run_layer(args):
    """The layer's elementwise producers / consumers at the benchmark shape (not the headline metric): short
    convolution on a [T, H*K] projection, gate inputs (g, beta, lambda) and the gated RMS norm of the output.
    Each is timed alone with CUDA events, L2 flushed between launches; GB/s over the algorithmic bytes."""
    from lampa_b200 import _lib as L
    from lampa_b200.layer import ShortConvolution, gate_inputs, rms_norm_gated
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    T, Lv, dt = 61440, 17, torch.bfloat16
    gen = torch.Generator().manual_seed(20259)
    rnd = lambda *shape: torch.randn(*shape, generator=gen).to(dt).to(dev)
    x = rnd(1, T, H * K)
    conv = ShortConvolution(H * K, 4).to(dev).to(dt)
    a, b, dl = rnd(1, T, H), rnd(1, T, H), rnd(1, T, H * Lv)
    A_log, dtb, Lp = torch.zeros(H, device=dev), torch.zeros(H, device=dev), torch.ones(H, Lv, device=dev)
    o, g, w = rnd(1, T, H, V), rnd(1, T, H, V), torch.ones(V, device=dev).to(dt)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ops = {
        "short_conv_fwd": (lambda: conv(x), 2 * x.numel() * 2),
        "gate_inputs": (lambda: gate_inputs(a, b, dl, A_log, dtb, Lp, "positive"),
                        a.numel() * (2 + 2 + 4 + 2) + dl.numel() * (2 + 2)),
        "rmsnorm_gate": (lambda: rms_norm_gated(o, g, w, None, "swish", eps=1e-5), 3 * o.numel() * 2),
    }
    out = {}
    for name, (fn, nbytes) in ops.items():
        for _ in range(max(args.warmup, 3)):
            fn()
        L.profile_enable(True)
        for _ in range(args.steps):
            flush.zero_()
            fn()
        torch.cuda.synchronize()
        prof = L.profile_read()
        L.profile_enable(False)
        ms = prof[name]["ms"] / prof[name]["launches"]
        out[name] = {"us_per_launch": ms * 1e3, "algorithmic_bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9,
                     "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / peaks()["hbm_gbs"]}
    print(json.dumps({"metric": "GB/s, layer producers/consumers", "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                      "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": f"ShortConvolution [T={T}, D={H * K}, W=4] + gate inputs (H={H}, L={Lv}) + "
                                             f"FusedRMSNormGated [{T * H} rows of {V}], L2 flushed between launches"},
                      "kernels": out}), flush=True)


def run_hept(args):
    """The HEPT bucket attention at the 60k-hit event shape (not the headline metric): 3 rounds x 8 heads,
    buckets of 100 hits, 24 value features and 24 + 6 query / key features, random bucket orders; the fused
    gather + attention + scatter kernel and the combination over rounds, timed with CUDA events, L2 flushed
    between launches.  TFLOP/s over the useful fp32 work (bucket^2 x (dq + dv) x 2 per bucket), GB/s over the
    algorithmic bytes (q, k, v rows and positions read once, so and denom written once per round, head, hit)."""
    from lampa_b200 import _lib as L
    from lampa_b200.bucket_attn import assume_zero_padded, hept_bucket_attention
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    n, heads, rounds, bucket, dq, dv = N_HITS, 8, 3, 100, 30, 24
    gen = torch.Generator().manual_seed(20261)
    ldq = (dq + 3) // 4 * 4
    q = torch.zeros(heads, n, ldq)
    k = torch.zeros(heads, n, ldq)
    q[..., :dq] = torch.randn(heads, n, dq, generator=gen) * (2.0 / dq ** 0.5)
    k[..., :dq] = q[..., :dq] + torch.randn(heads, n, dq, generator=gen) / dq ** 0.5
    v = torch.randn(heads, n, dv, generator=gen)
    pos = lambda: torch.stack([torch.stack([torch.randperm(n, generator=gen) for _ in range(heads)])
                               for _ in range(rounds)])
    qp, kp = pos().to(dev), pos().to(dev)
    q, k, v = q.to(dev)[..., :dq], k.to(dev)[..., :dq], v.to(dev)       # rows padded with zeros to whole 16-byte pieces
    assume_zero_padded(q)
    assume_zero_padded(k)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(max(args.warmup, 3)):
        hept_bucket_attention(q, k, v, qp, kp, bucket)
    L.profile_enable(True)
    for _ in range(args.steps):
        flush.zero_()
        hept_bucket_attention(q, k, v, qp, kp, bucket)
    torch.cuda.synchronize()
    prof = L.profile_read()
    L.profile_enable(False)
    units = rounds * heads * n
    flops = units * bucket * (dq + dv) * 2
    nbytes = {"bucket_rbf_attn": units * (2 * dq * 4 + dv * 4 + 16 + dv * 4 + 4),
              "bucket_attn_combine": units * (dv * 4 + 4) + heads * n * dv * 4}
    out = {}
    for name in ("bucket_rbf_attn", "bucket_attn_combine"):
        ms = prof[name]["ms"] / prof[name]["launches"]
        out[name] = {"us_per_launch": ms * 1e3, "algorithmic_bytes": nbytes[name],
                     "gbs": nbytes[name] / (ms * 1e-3) / 1e9}
    ms = out["bucket_rbf_attn"]["us_per_launch"] * 1e-3
    out["bucket_rbf_attn"]["fp32_tflops"] = flops / (ms * 1e-3) / 1e12
    total_ms = sum(o["us_per_launch"] for o in out.values()) * 1e-3
    # fp32 FMA bound: no measured fp32 peak is written by the driver, so the denominator is the nominal
    # 148 SMs x 128 FMA lanes x 2 flop x the maximum SM clock reported by NVML (1965 MHz on this pool)
    try:
        import pynvml
        pynvml.nvmlInit()
        mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(pynvml.nvmlDeviceGetHandleByIndex(dev.index or 0),
                                                     pynvml.NVML_CLOCK_SM))
    except Exception:
        mhz = 1965.0
    peak = 148 * 128 * 2 * mhz * 1e6 / 1e12
    roof = {"kernel": "bucket_rbf_attn", "bound": "fp32-fma", "achieved": out["bucket_rbf_attn"]["fp32_tflops"],
            "peak": peak, "unit": "TFLOP/s", "frac": out["bucket_rbf_attn"]["fp32_tflops"] / peak,
            "peak_source": "nominal (SMs x lanes x 2 x max SM clock)", "traffic": 310.0e6 if n == 60000 else None}
    print(json.dumps({"metric": "hits/sec, HEPT bucket attention", "value": n / (total_ms * 1e-3), "unit": "hits/s",
                      "roofline": roof,
                      "n_gpus": 1, "steps": args.steps, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": f"bucket attention N={n} rounds={rounds} heads={heads} bucket={bucket} "
                                             f"dq={dq} dv={dv}, random bucket orders, L2 flushed between launches"},
                      "kernels": out}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-sample", type=int, default=0, help="hits in the CPU baseline pass (default: all)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer (end-to-end) leg")
    ap.add_argument("--hits", type=int, default=N_HITS, help="hits of the event (default: the 60k-hit workload)")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying "
                                                            "one captured CUDA graph per stream")
    ap.add_argument("--streams", type=int, default=3,
                    help="independent events kept in flight in the device-resident leg (1: strictly back to back)")
    ap.add_argument("--workload", default="event", choices=["event", "plain", "layer", "hept"],
                    help="event: the headline LSH + hierarchical step; plain: configuration 1 "
                         "(chunk_gated_delta_rule, T=65536, H=8, K=V=64, initial and final state), device-resident only; "
                         "layer: the elementwise kernels around the op (short convolution, gate inputs, gated norm); "
                         "hept: the bucket attention of the HEPT layer at the event shape")
    args = ap.parse_args()
    if args.hits != N_HITS:
        set_event_size(args.hits)
    if args.workload == "plain":
        run_plain(args)
    elif args.workload == "hept":
        run_hept(args)
    elif args.workload == "layer":
        run_layer(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
