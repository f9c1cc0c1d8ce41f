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
DEFAULT_N_HITS = N_HITS
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


def profile_traffic():
    """DRAM bytes (read + write) per launch of each kernel on the default workload, read from the table in the
    committed profiler summary (rows `| kernel | ... | dram_bytes_per_launch |`); {} when it is absent."""
    import re
    path = os.path.join(ROOT, "profiles", "dram_traffic_bench_60k_hier.md")
    out = {}
    if os.path.exists(path):
        for line in open(path):
            m = re.match(r"\|\s*`?([a-z_0-9]+)`?\s*\|.*\|\s*([0-9.]+e[0-9]+|[0-9]+)\s*\|\s*$", line)
            if m:
                out[m.group(1)] = float(m.group(2))
    return out


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
    """The CPU arm: the C restatement of the reference's token recurrence (plus the hash, the 24 sorts and the two
    row moves) over the WHOLE event, all host cores, exactly `--steps` timed passes after `--warmup` untimed ones
    (about 8 s per pass on 8 cores)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ev = make_event(20252)
    cores = os.cpu_count() or 1
    for _ in range(args.warmup):
        cpu_pass(ev, N_HITS)
    t = [cpu_pass(ev, N_HITS) for _ in range(args.steps)]
    tot = float(np.sum(t))
    val = N_HITS * args.steps / tot
    sample = (f"the whole {N_HITS}-hit event per step, {args.steps} timed passes (median {np.median(t):.2f} s); C "
              f"restatement of the reference's token recurrence, OpenMP over heads")
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
        # the output rows go straight to their hits' positions: the un-ordering is folded into the output pass's store
        o, _ = lampa_b200.chunk_h_gated_delta_rule(t["q"], t["k"], t["v"], t["g"], t["lam"], t["beta"],
                                                   use_qk_l2norm_in_kernel=True, out_perm=order)
        out = o[0, :N_HITS].reshape(N_HITS, H * V)
        return out, order

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(vals):
        t = torch.tensor(vals, device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def timed(fn, steps):
        """Exactly `steps` steps on the current stream between two barriers; an event after every step gives the
        per-step times as well.  Returns (total ms, per-step ms list, t0, t1), max over ranks."""
        barrier()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        t0 = time.perf_counter()
        evs[0].record()
        for i in range(steps):
            fn()
            evs[i + 1].record()
        barrier()
        t1 = time.perf_counter()
        per = max_over_ranks([evs[i].elapsed_time(evs[i + 1]) for i in range(steps)])
        tot = max_over_ranks([evs[0].elapsed_time(evs[steps])])[0]
        return tot, per, t0, t1

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

    def timed_concurrent(steps, rounds):
        """`rounds` back-to-back repetitions of the timed region (exactly `steps` steps each, the streams joined at
        its two ends), each timed by its own pair of events; no host synchronisation in between.  Returns the
        per-round ms (max over ranks) and the host times around all of them."""
        barrier()
        main = torch.cuda.current_stream(dev)
        pairs = []
        t0 = time.perf_counter()
        for _ in range(rounds):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(main)
            for st_ in streams:
                st_.wait_event(e0)
            for _ in range(steps):
                step_concurrent()
            for st_ in streams:
                main.wait_stream(st_)
            e1.record(main)
            pairs.append((e0, e1))
        barrier()
        t1 = time.perf_counter()
        return max_over_ranks([a.elapsed_time(b) for a, b in pairs]), t0, t1

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step(d)
    ms_single, per_single, t0, t1 = timed(lambda: step(d), args.steps)
    rounds = 1
    if n_streams > 1 or not args.no_graph:
        for _ in range(max(args.warmup, 3)):
            step_concurrent()
        torch.cuda.synchronize()
        if not args.no_graph:
            capture_graphs()
            for _ in range(max(args.warmup, 3)):
                step_concurrent()
            torch.cuda.synchronize()
        probe_ms, _, _ = timed_concurrent(args.steps, 1)
        # the timed region (exactly --steps steps) is repeated until the repetitions cover about 0.6 s, so that the
        # clock sampler sees the GPU under load more than once; the line reports the median repetition
        rounds = int(min(400, max(3, np.ceil(600.0 / max(probe_ms[0], 1e-3)))))
        round_ms, t0, t1 = timed_concurrent(args.steps, rounds)
        ms = float(np.median(round_ms))
        L.check_status(dev)
    else:
        round_ms = [ms_single]
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

    # configuration 4 beside the headline: the packed 64-event model forward with the SAME 64 events split over
    # the ranks (strong scaling) and the NCCL gather of the outputs inside its timed region
    model_res = None
    if not args.no_model and N_HITS == 60000:
        model_res = model_measure(model_setup(dev, rank, world), dev, rank, world, max(3, min(args.steps, 5)), 3,
                                  e2e=not args.no_e2e)

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
        import ctypes
        lay = (ctypes.c_size_t * 12)()
        desc = L.GdnDesc(B=1, T=T_PAD, H=H, K=K, V=V, L=LEVELS, nseq=0, qkv_dtype=L.LAMPA_BF16, gb_dtype=L.LAMPA_F32,
                         lam_dtype=L.LAMPA_BF16, use_l2norm=1, scale=1.0)
        L.check(L.lib().lampa_gdn_workspace_layout(ctypes.byref(desc), lay), "lampa_gdn_workspace_layout")
        rec_bytes = int(lay[1])    # one (chunk, head) record: four 8 KB bf16 tiles + the chunk-level lambda rows, 1024-aligned
        in_bytes = H * (2 * K + V) * 2 + 2 * H * 4 + H * LEVELS * 2     # q, k, v bf16 + g, beta fp32 + lambda bf16 per token
        alg = {   # cost of one launch of each kernel on this workload against the roofline that bounds it
            # preparation: 57 flop per byte moved, far below the ridge (~250): HBM-bound.  Bytes = the inputs it must
            # read + the records this design makes it write (its compulsory traffic; the records are intermediates)
            "gdn_prep_hier": ("hbm", T_PAD * in_bytes + H * n_chunks * rec_bytes),
            "gdn_out_hier": ("tensor", H * n_chunks * (n_lev * 2.5 * 524288)),
            "gdn_out_hier_umma": ("tensor", H * n_chunks * (n_lev * 2.5 * 524288)),
            "gdn_compose": ("tensor", H * n_chunks * 2 * 2 * 64 ** 3),
            "gdn_level_hier": ("tensor", H * (n_chunks // 32) * 5 * 2 * 64 ** 3),
            "lsh_hash": ("hbm", N_HITS * 120),
            "segsort": ("hbm", N_HITS * ROUNDS * HEADS * 68),
            "permute_rows": ("hbm", N_HITS * (8 + 2 * 96)),
        }
        ncu_traffic = profile_traffic() if N_HITS == 60000 else {}
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
                         "traffic": ncu_traffic.get(dom), "peak_source": pk["source"],
                         "note": ("bytes = inputs read (%d B/token) + records written (%d B per chunk-head); inputs alone: %.0f GB/s; "
                                  "as dense flops (nine 64^3 products + the blockwise inverse = 4.02 MFLOP per chunk-head): %.0f TFLOP/s"
                                  % (in_bytes, rec_bytes, T_PAD * in_bytes / dur_s / 1e9,
                                     H * n_chunks * (7 * 524288 + 2 * 174763) / dur_s / 1e12)) if dom == "gdn_prep_hier" else None,
                         "whole_step_hbm_gbs": N_HITS * 4432 / (ms / args.steps * 1e-3) / 1e9},
            "kernels": per_kernel,
            "single_stream": {"value": world * N_HITS * args.steps / (ms_single * 1e-3), "unit": "hits/s",
                              "ms_per_step": ms_single / args.steps,
                              "ms_per_step_median": float(np.median(per_single)), "steps_timed": len(per_single)},
            "config4": model_res,
            "timed_rounds": {"rounds": rounds, "steps_per_round": args.steps, "reported": "median round",
                             "ms_per_step_min": float(np.min(round_ms)) / args.steps,
                             "ms_per_step_max": float(np.max(round_ms)) / args.steps},
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


# ---- configuration 4: packed, event-sharded model forward -----------------------------------------------
MODEL_EVENTS = 64
MODEL_WORKLOAD = ("config 4: lshgd-style model forward, 64 events of U(6000, 60000) hits packed by cu_seqlens: "
                  "Linear 24->128, 4 x [RMSNorm, E2LSH order (3 x 8 hashes, round b mod 3), hierarchical gated-delta "
                  "mixer H=4 K=V=32 bf16 (short conv, gates, gated norm), un-order, MLP 128->512->128 GELU], Linear "
                  "128->24; events split over the ranks by hit count (LPT), outputs all-gathered over NCCL")


def model_setup(dev, rank, world, n_events=MODEL_EVENTS):
    """This rank's share of the events (host rows, pinned), the model, the plan."""
    from lampa_b200 import sharding, synth
    from lampa_b200.model import LSHGatedDelta
    lengths = synth.event_sizes(20254, n_events).tolist()
    plan = sharding.lpt_assign(lengths, world)
    owned = plan[rank]
    rows = [synth.detector_hits(20254 + e, lengths[e]) for e in owned]
    local = torch.cat(rows) if rows else torch.zeros(0, 24)
    cu, _ = sharding.pack_events(lengths, owned)
    torch.manual_seed(20254)
    model = LSHGatedDelta(max_hits_per_event=60000).to(dev)
    return {"lengths": lengths, "plan": plan, "owned": owned, "hits_host": local.pin_memory(), "cu": cu.to(dev),
            "model": model, "imbalance": sharding.imbalance(lengths, plan)}


def model_measure(ms_, dev, rank, world, steps, warmup, e2e=True, profile=True):
    """Device-resident and host-to-host timing of the sharded forward; returns a dict (rank 0's is printed)."""
    import torch.distributed as dist
    from lampa_b200 import _lib as L, sharding
    model, cu, lengths, plan = ms_["model"], ms_["cu"], ms_["lengths"], ms_["plan"]
    hits_dev = ms_["hits_host"].to(dev)
    total_hits = int(sum(lengths))
    side = torch.cuda.Stream(dev, priority=-1)      # the gather's copies and NCCL kernels go ahead of the next step's launches
    gather_us = []

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # The forward of a fixed batch is captured once and replayed (the host otherwise needs ~20 us per library call,
    # 255 of them per step, which is what bounds a step once eight ranks have cut the GPU work to 7 ms); the NCCL
    # gather stays outside the graph.  `static_in` is the graph's input buffer.
    static_in = hits_dev.clone()
    graph, static_out = None, None
    if not ms_.get("no_graph", False):
        try:
            for _ in range(2):
                model(static_in, cu)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):     # NCCL's watchdog thread may touch CUDA meanwhile
                static_out = model(static_in, cu)
            graph = g
        except Exception as exc:      # capture is an optimisation of the measurement loop, not a requirement
            sys.stderr.write(f"model forward not captured ({type(exc).__name__}: {exc}); launching eagerly\n")
            graph = None
            torch.cuda.synchronize()

    def forward(hits):
        if graph is None:
            return model(hits, cu)
        if hits.data_ptr() != static_in.data_ptr():
            static_in.copy_(hits, non_blocking=True)
        graph.replay()
        return static_out

    def step(hits):
        out = forward(hits)
        if world > 1:       # the path's only collective, on a side stream, inside the timed region
            cur = torch.cuda.current_stream(dev)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                out.record_stream(side)
                g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                g0.record(side)
                full = sharding.gather_event_outputs(out, lengths, plan)
                g1.record(side)
                gather_us.append((g0, g1))
            return out, full
        return out, out

    def run(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(warmup, 3)):
        step(static_in)
    gather_us.clear()
    ms = run(lambda: step(static_in), steps)
    g_us = float(np.median([a.elapsed_time(b) for a, b in gather_us])) * 1e3 if gather_us else 0.0
    L.check_status(dev)
    res = {"metric": "hits/sec, packed 64-event model forward", "value": total_hits * steps / (ms * 1e-3),
           "unit": "hits/s", "n_gpus": world, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms / steps,
           "scaling": "strong", "dtype": "bf16", "data": "synthetic",
           "config": {"workload": MODEL_WORKLOAD, "events": len(lengths), "hits": total_hits,
                      "sharding": "events by LPT on hit count; all_gather of [hits, 24] fp32 outputs on a side stream",
                      "lpt_imbalance": ms_["imbalance"], "gather_us": g_us, "cuda_graphs": graph is not None,
                      "l2": "activations of one block (hundreds of MB per tensor) exceed the 126 MB L2"}}
    if e2e:
        out_host = torch.empty(hits_dev.shape[0], 24).pin_memory()
        stage = static_in                      # the upload lands in the forward's input buffer

        def e2e_step():
            stage.copy_(ms_["hits_host"], non_blocking=True)
            out, _ = step(stage)
            out_host.copy_(out, non_blocking=True)

        for _ in range(2):
            e2e_step()
        n = max(3, min(steps, 10))
        ms_e = run(e2e_step, n)
        res["e2e"] = {"value": total_hits * n / (ms_e * 1e-3), "unit": "hits/s", "steps": n,
                      "h2d_bytes_per_step": int(hits_dev.numel() * 4), "d2h_bytes_per_step": int(out_host.numel() * 4)}
    if profile:
        torch.cuda.synchronize()
        L.profile_enable(True)
        n = 3
        for _ in range(n):
            model(hits_dev, cu)
        torch.cuda.synchronize()
        prof = L.profile_read()
        L.profile_enable(False)
        per = {k: {"ms_per_step": r["ms"] / n, "launches_per_step": r["launches"] / n} for k, r in prof.items()}
        ours = sum(v["ms_per_step"] for v in per.values())
        res["kernels"] = per
        res["library_kernels_ms_per_step"] = ours
        res["gpu_launches"] = int(round(sum(v["launches_per_step"] for v in per.values()) * steps))
        # dominant library kernel against its bound (tensor pipe for the mixer's preparation and output passes)
        if per:
            dom = max(per, key=lambda k: per[k]["ms_per_step"])
            own_hits = int(hits_dev.shape[0])
            chunks = sum((lengths[e] + 63) // 64 for e in ms_["owned"])
            nlev = 10
            alg = {"gdn_prep_hier": ("tensor", 4 * 4 * chunks * (7 * 2 * 64 * 64 * 32 + 2 * 174763)),
                   "gdn_out_hier": ("tensor", 4 * 4 * chunks * nlev * 2.5 * 2 * 64 * 32 * 32)}
            pk = peaks()
            if dom in alg:
                units = alg[dom][1]
                dur = per[dom]["ms_per_step"] * 1e-3
                res["roofline"] = {"kernel": dom, "bound": "tensor", "achieved": units / dur / 1e12,
                                   "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                                   "frac": units / dur / 1e12 / pk["bf16_tflops_sustained"], "traffic": None,
                                   "peak_source": pk["source"] + " (sustained: timed inside a long step)",
                                   "note": f"{own_hits} hits on this rank, 4 blocks"}
    return res


def model_cpu_baseline(n_hits=6000):
    """The CPU statement of the model (tests/model_oracle.py over the CPU checker) on one small event."""
    from lampa_b200 import synth
    from lampa_b200.model import LSHGatedDelta
    from oracle import oracle
    from tests import model_oracle
    oracle.set_threads(os.cpu_count() or 1)
    torch.manual_seed(20254)
    m = LSHGatedDelta(max_hits_per_event=60000)
    hits = synth.detector_hits(1, n_hits)
    cu = torch.tensor([0, n_hits], dtype=torch.int64)
    t0 = time.perf_counter()
    model_oracle.forward(m, hits, cu)
    sec = time.perf_counter() - t0
    return {"value": n_hits / sec, "unit": "hits/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"one event of {n_hits} hits ({sec:.1f} s): torch CPU layers + C token recurrence of the mixer"}


def run_model(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sampler = ClockSampler(local)
    sampler.start()
    t0 = time.perf_counter()
    setup = model_setup(dev, rank, world)
    setup["no_graph"] = args.no_graph
    res = model_measure(setup, dev, rank, world, args.steps, args.warmup, e2e=not args.no_e2e)
    res["clocks"] = sampler.summary(t0, time.perf_counter())
    sampler.stop_flag = True
    res.update({"higher_is_better": True, "vs_baseline": None})
    if rank == 0:
        if world == 1 and not args.no_cpu:
            res["cpu_baseline"] = model_cpu_baseline()
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_plain(args):
    """Configurations 1 and 0 on one GPU: timing of the plain chunkwise rule (not the headline metric).
    plain: T = 65536, H = 8, random initial state; config0: T = 6144, H = 4, zero initial state, with the CPU
    restatement of the token recurrence timed beside it on the same inputs."""
    import lampa_b200
    from lampa_b200 import _lib as L, synth
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    cfg0 = args.workload == "config0"
    T = (6144 if cfg0 else 65536) if args.hits == DEFAULT_N_HITS else args.hits   # --hits shrinks the case for a profiler capture
    nh = 4 if cfg0 else H                                  # heads
    host = synth.gdn_inputs(20250 if cfg0 else 20251, T, nh, K, V, g_shift=2.0, h0=True)
    if cfg0:
        host["h0"].zero_()
    d = {k: v.to(dev) for k, v in host.items()}

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
    # HBM roofline of each pass: the bytes it has to move by this design (inputs, records, block composites, output)
    pk = peaks()
    n_ch = (T + 63) // 64
    rec = 4 * 8192                                        # M, Q~, B^T, O_local: bf16 [64][64] each
    alg = {"gdn_prep_plain": T * (nh * (2 * K + V) * 2 + 2 * nh * 4) + nh * n_ch * rec,
           "gdn_compose": nh * n_ch * 3 * 8192,
           "gdn_out_plain_umma": nh * n_ch * rec + T * nh * V * 2,
           "gdn_out_plain": nh * n_ch * rec + T * nh * V * 2}
    kernels = {}
    for n, r in prof.items():
        per = r["ms"] / r["launches"]
        kernels[n] = {"ms_per_launch": per}
        if n in alg:
            kernels[n]["hbm_gbs"] = alg[n] / (per * 1e-3) / 1e9
            kernels[n]["hbm_frac"] = kernels[n]["hbm_gbs"] / pk["hbm_gbs"]
    dom = max(kernels, key=lambda n: kernels[n]["ms_per_launch"])
    cpu_line = None
    if cfg0 and not args.no_cpu:
        from oracle import oracle
        cores = os.cpu_count() or 1
        oracle.set_threads(cores)
        a = [host[k][0].float().numpy() for k in ("q", "k", "v", "g", "beta")]
        oracle.gdn_plain(*a, h0=host["h0"].numpy(), use_l2norm=True)                  # warm-up
        t0 = time.perf_counter()
        oracle.gdn_plain(*a, h0=host["h0"].numpy(), use_l2norm=True)
        sec = time.perf_counter() - t0
        cpu_line = {"value": T / sec, "unit": "tokens/s", "cores": min(cores, nh), "kind": "port",
                    "sample": f"one pass over all {T} tokens ({sec * 1e3:.0f} ms); C restatement of the reference's token "
                              "recurrence, OpenMP over heads"}
    print(json.dumps({
        "roofline": {"kernel": dom, "bound": "hbm", "achieved": kernels[dom].get("hbm_gbs"), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": kernels[dom].get("hbm_frac"), "traffic": None, "peak_source": pk["source"]},
        "metric": "tokens/sec, plain chunkwise gated-delta fwd", "value": T * args.steps / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"config {0 if cfg0 else 1}: chunk_gated_delta_rule T={T} H={nh} K=V=64 bf16, "
                               f"{'zero' if cfg0 else 'random'} initial state + final state"},
        "cpu_baseline": cpu_line,
        "hbm_gbs_algorithmic": T * 4160 / (ms / args.steps * 1e-3) / 1e9,
        "kernels": kernels}), flush=True)


def run_heads(args):
    """One 60k-hit event split by HEAD over the ranks (strong scaling of a single event): rank r hashes and sorts the
    three rounds of its heads, runs the hierarchical rule on them and the [hits, H/N, V] outputs are all-gathered over
    NCCL on a side stream, under the next event's kernels.  Device-resident; not the headline metric."""
    import torch.distributed as dist
    import lampa_b200
    from lampa_b200 import _lib as L, sharding
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ev = make_event(20252)                                      # the same event on every rank
    h0, h1 = sharding.head_slice(H, rank, world)
    d = {k: ev[k][:, :, h0:h1].contiguous().to(dev) for k in ("q", "k", "v", "g", "beta", "lam")}
    hits = ev["hits"].to(dev)
    alpha, lsh_beta = ev["alpha"][h0:h1].contiguous().to(dev), ev["lsh_beta"].to(dev)
    hl = h1 - h0
    side = torch.cuda.Stream(dev, priority=-1)
    done = torch.cuda.Event()

    def step():
        ids = lampa_b200.lsh_hash(hits, alpha, lsh_beta, 1.0)["ids"]
        perm = lampa_b200.segmented_sort(ids, nseg=ROUNDS * hl).view(ROUNDS, hl, N_HITS)
        order = perm[0, 0]
        lampa_b200.permute_rows(hits, order)
        o, _ = lampa_b200.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"],
                                                   use_qk_l2norm_in_kernel=True, out_perm=order)
        out = o[0, :N_HITS].reshape(N_HITS, hl * V)
        if world == 1:
            return out
        done.record()
        with torch.cuda.stream(side):
            side.wait_event(done)
            full = sharding.gather_heads(out.view(N_HITS, hl, V))
            out.record_stream(side)
        return full

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    torch.cuda.current_stream().wait_stream(side)
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    L.check_status(dev)
    if rank == 0:
        print(json.dumps({
            "metric": "hits/sec, one 60k-hit event split by head", "value": N_HITS * args.steps / (ms * 1e-3), "unit": "hits/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sharding": f"heads: {hl} of {H} per rank, ids and sorts of those heads only; "
                       "all_gather of [hits, H/N, V] bf16 outputs on a side stream"}}), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
    ap.add_argument("--no-model", action="store_true", help="skip the configuration-4 sub-measurement of the default run")
    ap.add_argument("--streams", type=int, default=4,
                    help="independent events kept in flight in the device-resident leg (1: strictly back to back)")
    ap.add_argument("--workload", default="event", choices=["event", "model", "plain", "config0", "layer", "hept", "heads"],
                    help="event: the headline LSH + hierarchical step; model: configuration 4, the packed 64-event "
                         "model forward, events split over the ranks (strong scaling) with an NCCL gather; plain: configuration 1 "
                         "(chunk_gated_delta_rule, T=65536, H=8, K=V=64, initial and final state), device-resident only; "
                         "config0: configuration 0's shape (T=6144, H=4) on the same op, with the CPU restatement beside it; "
                         "layer: the elementwise kernels around the op (short convolution, gate inputs, gated norm); "
                         "hept: the bucket attention of the HEPT layer at the event shape; heads: one event split by head over the "
                         "ranks, outputs all-gathered over NCCL")
    args = ap.parse_args()
    if args.hits != N_HITS:
        set_event_size(args.hits)
    if args.workload in ("plain", "config0"):
        run_plain(args)
    elif args.workload == "model" and args.impl != "reference":
        run_model(args)
    elif args.workload == "hept":
        run_hept(args)
    elif args.workload == "heads":
        run_heads(args)
    elif args.workload == "layer":
        run_layer(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
