#!/usr/bin/env python
"""Benchmark of the TW-Marlin W4A16 GEMM path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1 (default): the Qwen2-7B-shaped decode GEMM set, M = 1, one layer's four GEMMs x 28 distinct
layers (fused QKV 3584x4608, o 3584x3584, gate+up 3584x37888, down 18944x3584), Q4 group-128
weights, FP16 activations/outputs.  One step = the 112 GEMMs once, enqueued through the C ABI and
replayed as one CUDA graph.  Metric: algorithmic bytes (each operand once) / time, in GB/s.
Synthetic seeded data of those shapes; every step streams 3.37 GB, far more than the 126 MB L2.

`--impl reference` times the reference's CPU route for the same GEMMs (dequantise, multiply,
FP32 accumulate; restated in C because the reference's Rust cannot be compiled here) on the host
cores, on a bounded sample per step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYERS = 28
GROUP = 128
# (name, K, N) of one Qwen2-7B-shaped layer, decode order
LAYER_GEMMS = [("qkv", 3584, 4608), ("o", 3584, 3584), ("gate_up", 3584, 37888), ("down", 18944, 3584)]
METRIC = "w4a16_gemm_hbm_gbs_m1"
UNIT = "GB/s"


def algorithmic_bytes(m: int, n: int, k: int, group: int, a_bytes: int = 2, c_bytes: int = 2) -> int:
    """Each operand touched once: packed nibbles + fp16 scales + activations + outputs."""
    return k * n // 2 + (k // group) * n * 2 + m * k * a_bytes + m * n * c_bytes


def layer_bytes(m: int = 1) -> int:
    return sum(algorithmic_bytes(m, n, k, GROUP) for _, k, n in LAYER_GEMMS)


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# ------------------------------------------------------------------ ours --

def build_weights(torch, q, device, layers):
    """Seeded synthetic weights W[K,N] ~ N(0, 0.02^2), quantised and packed on the device."""
    out = []
    for layer in range(layers):
        mats = []
        for pid, (_, k, n) in enumerate(LAYER_GEMMS):
            gen = torch.Generator(device=device).manual_seed(1000 * layer + pid)
            w = torch.randn((k, n), generator=gen, device=device, dtype=torch.float32) * 0.02
            mats.append(q.quantize_f32_to_tw_marlin(w, k, n, GROUP))
            del w
        out.append(mats)
    torch.cuda.synchronize()
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    from tensorwarp_b200 import _lib
    from tensorwarp_b200 import quantize as q

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    m = 1
    weights = build_weights(torch, q, device, LAYERS)
    # activations: FP16 N(0,1), CPU generator seed 0, one vector per GEMM, all in one pinned host buffer
    a_sizes = [k for _ in range(LAYERS) for _, k, _ in LAYER_GEMMS]
    c_sizes = [n for _ in range(LAYERS) for _, _, n in LAYER_GEMMS]
    host_a = torch.randn(sum(a_sizes), generator=torch.Generator().manual_seed(0)).to(torch.float16).pin_memory()
    host_c = torch.empty(sum(c_sizes), dtype=torch.float16).pin_memory()
    dev_a = host_a.to(device)
    dev_c = torch.zeros(sum(c_sizes), dtype=torch.float16, device=device)
    ws = q.Workspace.for_shapes([(m, n, k, GROUP) for _, k, n in LAYER_GEMMS], device)

    stream = torch.cuda.Stream(device)
    flags = _lib.TWM_FLAG_PDL        # weights are constants: let each GEMM prefetch them early

    gemm_list = [(weights[layer][pid], k, n) for layer in range(LAYERS) for pid, (_, k, n) in enumerate(LAYER_GEMMS)]

    def enqueue_all(extra_flags=0, hint=True, a_buf=None, c_buf=None):
        # every GEMM names its successor (the step's first GEMM follows its last one in the next replay),
        # so the successor's first weights are on their way into L2 while this GEMM's grid drains
        a_buf = dev_a if a_buf is None else a_buf
        c_buf = dev_c if c_buf is None else c_buf
        ao = co = 0
        for i, ((p, s), k, n) in enumerate(gemm_list):
            (np_, ns_), nk, nn = gemm_list[(i + 1) % len(gemm_list)]
            q.gemm_tw_marlin_m1(a_buf[ao:ao + k], p, s, c_buf[co:co + n], n, k, group_size=GROUP,
                                workspace=ws, flags=flags | extra_flags,
                                next_gemm=(np_, ns_, m, nn, nk, GROUP) if hint else None)
            ao += k
            co += n

    with torch.cuda.stream(stream):
        enqueue_all()                                   # eager once: initialises per-device state
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            enqueue_all()
        launches_per_step = LAYERS * len(LAYER_GEMMS)

        for _ in range(args.warmup):
            graph.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            e0.record(stream)
            for _ in range(args.steps):
                graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            dist.barrier()
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())

        # end to end: host activations -> device, the 112 GEMMs, outputs -> host, every step
        for _ in range(2):
            dev_a.copy_(host_a, non_blocking=True)
            graph.replay()
            host_c.copy_(dev_c, non_blocking=True)
        torch.cuda.synchronize()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(args.steps):
            dev_a.copy_(host_a, non_blocking=True)
            graph.replay()
            host_c.copy_(dev_c, non_blocking=True)
        f1.record(stream)
        torch.cuda.synchronize()
        e2e_serial_ms = f0.elapsed_time(f1)
        # The same end to end, pipelined: two sets of device buffers and two captured graphs used in turn,
        # the copies on streams of their own, so that step i+1's activations come in and step i-1's
        # outputs go out while step i's GEMMs run.  Every step still copies its inputs in and its results out.
        dev_a2, dev_c2 = torch.empty_like(dev_a), torch.zeros_like(dev_c)
        host_c2 = torch.empty_like(host_c).pin_memory()
        graph2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph2, stream=stream):
            enqueue_all(a_buf=dev_a2, c_buf=dev_c2)
        torch.cuda.synchronize()
        s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        sets = [(dev_a, dev_c, host_c, graph), (dev_a2, dev_c2, host_c2, graph2)]
        ev_in = [torch.cuda.Event() for _ in sets]
        ev_comp = [torch.cuda.Event() for _ in sets]
        ev_out = [torch.cuda.Event() for _ in sets]

        def pipelined(steps):
            for i in range(steps):
                j = i & 1
                a_j, c_j, h_j, g_j = sets[j]
                if i >= 2:
                    s_in.wait_event(ev_comp[j])            # the GEMMs that read this set's activations are done
                with torch.cuda.stream(s_in):
                    a_j.copy_(host_a, non_blocking=True)
                    ev_in[j].record(s_in)
                stream.wait_event(ev_in[j])
                if i >= 2:
                    stream.wait_event(ev_out[j])           # this set's previous outputs have left
                g_j.replay()
                ev_comp[j].record(stream)
                s_out.wait_event(ev_comp[j])
                with torch.cuda.stream(s_out):
                    h_j.copy_(c_j, non_blocking=True)
                    ev_out[j].record(s_out)
            for j in range(min(steps, 2)):
                stream.wait_event(ev_out[j])

        s_in.wait_stream(stream); s_out.wait_stream(stream)
        pipelined(4)
        torch.cuda.synchronize()
        same_pipe = bool(torch.equal(host_c, host_c2))
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record(stream)
        pipelined(args.steps)
        p1.record(stream)
        torch.cuda.synchronize()
        e2e_ms = p0.elapsed_time(p1)
        del graph2
        if world > 1:
            t = torch.tensor([e2e_ms, e2e_serial_ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms, e2e_serial_ms = float(t[0].item()), float(t[1].item())
    # Diagnostic, not the headline: the same 112 GEMMs (each has its own activation and output
    # slice, so they ARE independent) launched with TWM_FLAG_INDEPENDENT, i.e. without the wait
    # for the launch before that a decode step needs.  The difference to `value` is what the
    # dependency between consecutive launches costs.
    independent = None
    if rank == 0:
        with torch.cuda.stream(stream):
            ref_c = dev_c.clone()
            dev_c.zero_()
            graph_i = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_i, stream=stream):
                enqueue_all(_lib.TWM_FLAG_INDEPENDENT)
            for _ in range(args.warmup):
                graph_i.replay()
            torch.cuda.synchronize()
            same = bool(torch.equal(dev_c, ref_c))
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record(stream)
            for _ in range(args.steps):
                graph_i.replay()
            g1.record(stream)
            torch.cuda.synchronize()
            ind_ms = g0.elapsed_time(g1) / args.steps
        independent = {"ms_per_step": round(ind_ms, 4), "same_bits_as_dependent_run": same}
        del graph_i
        # Diagnostic: the headline's launches without the hint that names each GEMM's successor
        with torch.cuda.stream(stream):
            dev_c.zero_()
            graph_n = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_n, stream=stream):
                enqueue_all(hint=False)
            for _ in range(args.warmup):
                graph_n.replay()
            torch.cuda.synchronize()
            same_n = bool(torch.equal(dev_c, ref_c))
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record(stream)
            for _ in range(args.steps):
                graph_n.replay()
            g1.record(stream)
            torch.cuda.synchronize()
            independent["without_next_hint"] = {"ms_per_step": round(g0.elapsed_time(g1) / args.steps, 4), "same_bits": same_n}
        del graph_n
    err = q.device_error(stream)
    if err:
        raise RuntimeError(f"device error word {err:#x}")
    extras = {}
    if rank == 0:
        extras["per_gemm_us"] = per_gemm_us(torch, q, _lib, weights, device, stream)
        extras["chain"] = chain_figures(torch, q, _lib, weights, dev_a, dev_c, stream, args)
        extras["simt_f32_drop_in"] = simt_drop_in(torch, q, _lib, weights, device, stream, args)
        extras["ref_cuda"] = ref_cuda_figures(torch, weights, device, stream, args)
        err = q.device_error(stream)
        if err:
            raise RuntimeError(f"device error word {err:#x} (side measurements)")
    decode = None
    sweep = None
    config0 = None
    tp1 = None
    if not args.no_decode and rank == 0:
        del weights, graph
        torch.cuda.empty_cache()
        sweep = m_sweep(torch, q, device)
        torch.cuda.empty_cache()
        config0 = config0_gemv(torch, q, device)
        torch.cuda.empty_cache()
        decode = decode_tok_s(torch, device)
        torch.cuda.empty_cache()
        tp1 = tp1_anchor(torch, device)

    step_bytes = LAYERS * layer_bytes(m)
    ms_per_step = ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = world * step_bytes / (e2e_ms / args.steps * 1e-3) / 1e9
    peak, peak_kind = measured_peak_gbs()
    per_launch_bytes = step_bytes / launches_per_step
    per_launch_us = ms_per_step * 1e3 / launches_per_step
    achieved = per_launch_bytes / (per_launch_us * 1e-6) / 1e9
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
        "config": {"workload": "configs[1]: Qwen2-7B-shaped decode GEMM set, M=1, 4 GEMMs x 28 layers, Q4 group-128",
                   "l2": "inputs larger than L2: 3.37 GB of distinct weights streamed per step",
                   "launch": "one CUDA graph of 112 GEMM launches on one stream, programmatic dependent launch",
                   "parallelism": "replicas only" if world > 1 else "single GPU"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "peak_kind": peak_kind,
                     "kernel": "twm::mma::gemv_kernel<1,2>",
                     "avg_launch_us": round(per_launch_us, 3), "avg_launch_bytes": int(per_launch_bytes),
                     "traffic": TRAFFIC_PER_LAUNCH},
        "e2e": {"value": round(e2e_value, 1), "unit": UNIT, "h2d_bytes_per_step": int(host_a.numel() * 2),
                "d2h_bytes_per_step": int(host_c.numel() * 2),
                "serial_value": round(world * step_bytes / (e2e_serial_ms / args.steps * 1e-3) / 1e9, 1),
                "same_outputs_in_both_buffer_sets": same_pipe,
                "note": "value: every step copies its activations in from pinned host memory and its outputs back, on copy "
                        "streams, two buffer sets in turn, so the copies overlap the neighbouring steps' GEMMs; "
                        "serial_value: the same on one stream, nothing overlapped"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks.summary(),
    }
    if independent is not None:
        ind_gbs = step_bytes / (independent["ms_per_step"] * 1e-3) / 1e9
        independent.update({"gbs": round(ind_gbs, 1), "hbm_frac": round(ind_gbs / peak, 4),
                            "note": "same GEMM set without the wait for the preceding launch (TWM_FLAG_INDEPENDENT); diagnostic"})
        line["without_next_hint"] = independent.pop("without_next_hint")
        line["independent_launches"] = independent
    if decode is not None:
        line["decode"] = decode
    if sweep is not None:
        line["m_sweep"] = sweep
    if config0 is not None:
        line["config0"] = config0
    if tp1 is not None:
        line["tp1"] = tp1
    line.update(extras)
    if rank == 0:
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(target_seconds=12.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _time_graph(torch, stream, enqueue, steps, warm=3):
    """Milliseconds per replay of `enqueue` captured as one CUDA graph (CUDA events on `stream`)."""
    with torch.cuda.stream(stream):
        enqueue()                                        # eager once
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            enqueue()
        for _ in range(warm):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def per_gemm_us(torch, q, _lib, weights, device, stream):
    """Microseconds per GEMM of each configs[1] shape: 28 launches of the same shape (28 distinct
    weight sets, each launch waiting for the one before) in one graph."""
    peak, _ = measured_peak_gbs()
    out = {}
    for pid, (name, k, n) in enumerate(LAYER_GEMMS):
        a = torch.randn(k, generator=torch.Generator(device=device).manual_seed(40 + pid), device=device).half()
        c = torch.empty(n, dtype=torch.float16, device=device)
        ws = q.Workspace(q.workspace_bytes(1, n, k, GROUP), device)

        def enqueue():
            for layer in range(len(weights)):
                p_, s_ = weights[layer][pid]
                q.gemm_tw_marlin_m1(a, p_, s_, c, n, k, group_size=GROUP, workspace=ws, flags=_lib.TWM_FLAG_PDL)

        us = _time_graph(torch, stream, enqueue, 10) * 1e3 / len(weights)
        b = algorithmic_bytes(1, n, k, GROUP)
        out[name] = {"us": round(us, 2), "hbm_frac": round(b / us / 1e3 / peak, 3)}
    return out


def chain_figures(torch, q, _lib, weights, dev_a, dev_c, stream, args):
    """The same 112 GEMMs as ONE persistent launch (twm_chain_*): every GEMM waits for the one before
    through a counter in device memory while the next GEMM's weights are already streaming; and the
    same list with no waits at all.  Reported beside the headline, which stays the reference's
    calling pattern (one launch per GEMM)."""
    peak, _ = measured_peak_gbs()
    step_bytes = LAYERS * layer_bytes(1)
    out = {}
    for key, fl in (("dependent", 0), ("independent", _lib.TWM_FLAG_INDEPENDENT)):
        ch = q.GemmChain()
        ao = co = 0
        for layer in range(LAYERS):
            for pid, (_, k, n) in enumerate(LAYER_GEMMS):
                p_, s_ = weights[layer][pid]
                ch.add(dev_a[ao:ao + k], p_, s_, dev_c[co:co + n], 1, n, k, group_size=GROUP, flags=fl)
                ao += k
                co += n
        ch.build()
        ms = _time_graph(torch, stream, lambda: ch.launch(stream), args.steps)
        out[key] = {"ms_per_step": round(ms, 4), "gbs": round(step_bytes / ms / 1e6, 1),
                    "hbm_frac": round(step_bytes / ms / 1e6 / peak, 4), "launches_per_step": 1}
        info = ch.info
        out["grid"], out["split_tiles"], out["device_bytes"] = info.grid, info.split_tiles, int(info.device_bytes)
        ch.close()
    return out


def simt_drop_in(torch, q, _lib, weights, device, stream, args):
    """The reference's own signature: FP32 activations in, FP32 out (quantize.rs:1304-1307), which runs
    on the FP32-FMA streaming kernel; same 112 GEMMs, same graph and dependency as the headline."""
    peak, _ = measured_peak_gbs()
    a_sizes = [k for _ in range(LAYERS) for _, k, _ in LAYER_GEMMS]
    c_sizes = [n for _ in range(LAYERS) for _, _, n in LAYER_GEMMS]
    a32 = torch.randn(sum(a_sizes), generator=torch.Generator(device=device).manual_seed(1), device=device)
    c32 = torch.zeros(sum(c_sizes), device=device)
    ws = q.Workspace.for_shapes([(1, n, k, GROUP) for _, k, n in LAYER_GEMMS], device)

    def enqueue():
        ao = co = 0
        for layer in range(LAYERS):
            for pid, (_, k, n) in enumerate(LAYER_GEMMS):
                p_, s_ = weights[layer][pid]
                q.gemm_tw_marlin_m1(a32[ao:ao + k], p_, s_, c32[co:co + n], n, k, group_size=GROUP, workspace=ws,
                                    flags=_lib.TWM_FLAG_PDL)
                ao += k
                co += n

    ms = _time_graph(torch, stream, enqueue, args.steps)
    step_bytes = LAYERS * sum(algorithmic_bytes(1, n, k, GROUP, 4, 4) for _, k, n in LAYER_GEMMS)
    return {"ms_per_step": round(ms, 4), "gbs": round(step_bytes / ms / 1e6, 1),
            "hbm_frac": round(step_bytes / ms / 1e6 / peak, 4), "kernel": "twm::simt::gemv_kernel"}


def ref_cuda_figures(torch, weights, device, stream, args):
    """The kernel to beat: the reference's own warp_gemm_tw_marlin_m1(_direct) (quantize.rs:1186-1298),
    compiled unchanged for sm_100a into oracle/_ref, run through its own launcher logic (split
    heuristic, memset, launch; quantize.rs:1311-1357) on the same 112 GEMMs in one CUDA graph.  It
    takes FP32 activations and one scale per 32-block, so the group-128 scales are shown to it with
    every row repeated four times (identical weights).  This leg is a measurement of the reference,
    not part of the product path."""
    from oracle import ref as oref
    if not oref.available():
        return {"unavailable": "oracle/_ref/libtwm_ref.so not built (needs the reference tree at build time)"}
    peak, _ = measured_peak_gbs()
    a_sizes = [k for _ in range(LAYERS) for _, k, _ in LAYER_GEMMS]
    c_sizes = [n for _ in range(LAYERS) for _, _, n in LAYER_GEMMS]
    a32 = torch.randn(sum(a_sizes), generator=torch.Generator(device=device).manual_seed(1), device=device)
    c32 = torch.zeros(sum(c_sizes), device=device)
    scales32 = [[s_.repeat_interleave(GROUP // 32, dim=0).contiguous() for _, s_ in mats] for mats in weights]
    sp = stream.cuda_stream

    def enqueue(only=None):
        ao = co = 0
        for layer in range(LAYERS):
            for pid, (_, k, n) in enumerate(LAYER_GEMMS):
                if only is None or only == pid:
                    oref.gemm_tw_marlin_m1(c32[co:co + n].data_ptr(), a32[ao:ao + k].data_ptr(), weights[layer][pid][0].data_ptr(),
                                           scales32[layer][pid].data_ptr(), n, k, stream=sp)
                ao += k
                co += n

    ms = _time_graph(torch, stream, enqueue, max(3, args.steps // 4))
    step_bytes = LAYERS * layer_bytes(1)
    out = {"ms_per_step": round(ms, 4), "gbs_on_the_same_algorithmic_bytes": round(step_bytes / ms / 1e6, 1),
           "hbm_frac": round(step_bytes / ms / 1e6 / peak, 4), "per_gemm_us": {}}
    for pid, (name, _, _) in enumerate(LAYER_GEMMS):
        us = _time_graph(torch, stream, lambda: enqueue(pid), 3) * 1e3 / LAYERS
        out["per_gemm_us"][name] = round(us, 2)
    return out


def tp1_anchor(torch, device, steps: int = 5):
    """configs[4] on ONE GPU: the Llama-3-70B-shaped 80-layer decode stack (35 GB of Q4 weights), M=1,
    KV 4096, the same stack bench.py --gpus N runs tensor-parallel: the tp=1 point of that curve."""
    from tensorwarp_b200 import tensor_parallel as tp
    peak, _ = measured_peak_gbs()
    kv_len = 4096
    base = tp.LLAMA3_70B
    cfg = type(base)(**{**base.__dict__, "max_seq": kv_len + 128})
    spec = tp.shard_spec(cfg, 1, 0)
    layers = [tp.random_shard_layer(cfg, spec, li, device) for li in range(cfg.layers)]
    stack = tp.TPDecodeStack(cfg, spec, layers, 1, device, all_reduce=lambda t: None, comm=None)
    stack.prefill_random_kv(kv_len, seed=2)
    stack.x.copy_(torch.randn((1, cfg.hidden), generator=torch.Generator().manual_seed(7)))
    stream = torch.cuda.Stream(device)
    ms = _time_graph(torch, stream, lambda: stack.forward(stream.cuda_stream), steps)
    hd = cfg.head_dim
    gemms = [(cfg.hidden, spec.n_qkv), (cfg.num_heads * hd, cfg.hidden), (cfg.hidden, spec.n_gu), (spec.n_gu // 2, cfg.hidden)]
    nbytes = cfg.layers * sum(algorithmic_bytes(1, n, k, cfg.group_size, 2, 4 if n == cfg.hidden else 2) for k, n in gemms)
    finite = bool(torch.isfinite(stack.x).all().item())
    del stack, layers
    torch.cuda.empty_cache()
    return {"workload": "configs[4] at tp=1: Llama-3-70B-shaped 80-layer Q4 decode stack, M=1, KV 4096, one GPU",
            "ms_per_step": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "hbm_frac": round(nbytes / ms / 1e6 / peak, 4),
            "finite": finite}


def config0_gemv(torch, q, device):
    """configs[0]: the Qwen2-0.5B gate+up GEMV (M=1, K=896, N=9728, G=128, FP16), 64 distinct weight
    sets per graph (279 MB, larger than L2), programmatic dependent launch."""
    from tensorwarp_b200 import _lib
    k, n, copies = 896, 9728, 64
    peak, _ = measured_peak_gbs()
    ws = []
    for i in range(copies):
        w = torch.randn((k, n), generator=torch.Generator(device=device).manual_seed(300 + i), device=device) * 0.02
        ws.append(q.quantize_f32_to_tw_marlin(w, k, n, GROUP))
        del w
    a = torch.randn((1, k), generator=torch.Generator(device=device).manual_seed(0), device=device).half()
    c = torch.empty((1, n), dtype=torch.float16, device=device)
    wsb = q.Workspace(q.workspace_bytes(1, n, k, GROUP), device)
    stream = torch.cuda.Stream(device)

    def enqueue():
        for p_, s_ in ws:
            q.gemm_tw_marlin(a, p_, s_, c, 1, n, k, group_size=GROUP, workspace=wsb, flags=_lib.TWM_FLAG_PDL)

    with torch.cuda.stream(stream):
        enqueue()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            enqueue()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(10):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (10 * copies)
    b = algorithmic_bytes(1, n, k, GROUP)
    return {"workload": "configs[0]: M=1, K=896, N=9728, G=128, FP16", "us": round(us, 2),
            "gbs": round(b / us / 1e3, 1), "hbm_frac": round(b / us / 1e3 / peak, 3)}


def m_sweep(torch, q, device):
    """configs[2]: the 7B gate+up shape (K=3584, N=37888, G=128, FP16) at M = 1..256, eight distinct
    weight sets per graph (568 MB, larger than L2), programmatic dependent launch, every GEMM naming the
    next one (`next_gemm`, as the decode engines do); microseconds per
    GEMM (for M above one launch's rows: all its launches), the kernel the heuristic chose, HBM and
    tensor fractions of the measured peaks."""
    from tensorwarp_b200 import _lib
    k, n, copies = 3584, 37888, 8
    names = {_lib.TWM_KERNEL_SIMT: "simt", _lib.TWM_KERNEL_TC: "tcgen05", _lib.TWM_KERNEL_MMA: "mma", _lib.TWM_KERNEL_TCW: "tcgen05-wide", _lib.TWM_KERNEL_TCR: "tcgen05-256col-f16w"}
    peak, _ = measured_peak_gbs()
    tf_peak = 1629.9
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            tf_peak = float(json.load(f).get("bf16_tflops", tf_peak))
    except (OSError, ValueError):
        pass
    ws = []
    for i in range(copies):
        w = torch.randn((k, n), generator=torch.Generator(device=device).manual_seed(200 + i), device=device) * 0.02
        ws.append(q.quantize_f32_to_tw_marlin(w, k, n, GROUP))
        del w
    out = []
    for m in (1, 2, 4, 8, 16, 32, 64, 128, 256):
        a = torch.randn((m, k), generator=torch.Generator(device=device).manual_seed(m), device=device).half()
        c = torch.empty((m, n), dtype=torch.float16, device=device)
        wsb = q.Workspace(q.workspace_bytes(m, n, k, GROUP), device)
        stream = torch.cuda.Stream(device)

        def enqueue():
            for i, (p_, s_) in enumerate(ws):
                nxt = ws[(i + 1) % copies]               # as a decode step does: each GEMM names its successor (L2 hint)
                q.gemm_tw_marlin(a, p_, s_, c, m, n, k, group_size=GROUP, workspace=wsb, flags=_lib.TWM_FLAG_PDL,
                                 next_gemm=(nxt[0], nxt[1], m, n, k, GROUP))

        with torch.cuda.stream(stream):
            enqueue()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                enqueue()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(5):
                graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (5 * copies)
        b = algorithmic_bytes(m, n, k, GROUP)
        kern = q.plan(m, n, k, GROUP).kernel
        out.append({"m": m, "us": round(us, 2), "kernel": names.get(kern, str(kern)),
                    "hbm_frac": round(b / us / 1e3 / peak, 3), "tensor_frac": round(2.0 * m * k * n / us / 1e6 / tf_peak, 4)})
        del graph
    return out


def decode_tok_s(torch, device, new_tokens: int = 64, kv_len: int = 2048):
    """configs[3]: full Qwen2-7B-shaped Q4 decode step (28 layers, FP16 KV prefilled to 2048 tokens of
    N(0,1), FP16 LM head, greedy) replayed as one CUDA graph; the token never leaves the device.
    Also timed, as a side figure: the same step with the LM head as a TW-Marlin GEMM (the reference's
    forward_lm_head_tw_marlin option)."""
    from tensorwarp_b200 import generate as gen
    cfg = gen.QWEN2_7B
    model = gen.Q4Model(cfg, device=device, seed=0)
    first = int(torch.randint(0, cfg.vocab, (1,), generator=torch.Generator().manual_seed(3)).item())

    def run(q4_lm_head):
        eng = gen.QuantizedGenerationEngine(model, q4_lm_head=q4_lm_head)
        eng.prefill_random_kv(kv_len, seed=2)
        eng.capture()
        eng.set_token(first)
        for _ in range(3):
            eng.replay()
        torch.cuda.synchronize()
        eng.prefill_random_kv(kv_len, seed=2)          # back to position 2048
        eng.buf.step.zero_()
        eng.set_token(first)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(eng.stream):
            e0.record(eng.stream)
            for _ in range(new_tokens):
                eng.replay()
            e1.record(eng.stream)
        torch.cuda.synchronize()
        toks = eng.buf.history[:new_tokens].tolist()
        prof = None
        if not q4_lm_head:
            eng.prefill_random_kv(kv_len, seed=2)
            eng.set_token(first)
            prof = eng.profile_decode_tw_marlin(steps=2)      # eager, one CUDA-event pair per operation
        return e0.elapsed_time(e1), eng.launches_per_step, bool(all(0 <= t < cfg.vocab for t in toks)), prof

    ms, launches, in_vocab, prof = run(False)
    q4_bytes = cfg.layers * layer_bytes(1)
    kv_bytes = cfg.layers * 2 * (kv_len + new_tokens // 2) * cfg.kv_dim * 2
    step_bytes = q4_bytes + cfg.vocab * cfg.hidden * 2 + kv_bytes
    out = {"tok_s": round(new_tokens / (ms * 1e-3), 1), "ms_per_token": round(ms / new_tokens, 4),
           "workload": f"configs[3]: Qwen2-7B-shaped Q4 decode, KV {kv_len} FP16, {new_tokens} greedy tokens, one CUDA graph per token",
           "launches_per_token": launches, "bytes_per_token": int(step_bytes),
           "hbm_gbs": round(step_bytes / (ms / new_tokens * 1e-3) / 1e9, 1), "tokens_in_vocab": in_vocab}
    if prof is not None:
        out["eager_profile_per_step"] = {"note": "eager launches with an event pair around every operation (no graph, so launch "
                                                 "gaps count); the shares, not the absolute total, carry over to the graph",
                                         "total_us": prof["total_us"], "gemm_us": prof["gemm_us"], "non_gemm_us": prof["non_gemm_us"],
                                         "us_per_layer": {k: v["us_per_layer"] for k, v in prof["ops"].items() if v["us_per_layer"] is not None},
                                         "lm_head_us": prof["ops"]["lm_head"]["us"]}
    ms4, _, in_vocab4, _ = run(True)
    step_bytes4 = q4_bytes + algorithmic_bytes(1, cfg.vocab, cfg.hidden, GROUP, 2, 4) + kv_bytes
    out["q4_lm_head"] = {"tok_s": round(new_tokens / (ms4 * 1e-3), 1), "ms_per_token": round(ms4 / new_tokens, 4),
                         "bytes_per_token": int(step_bytes4), "tokens_in_vocab": in_vocab4}
    return out


# ------------------------------------------------------------- tensor parallel --

def run_tp(args):
    """N > 1: configs[4], the Llama-3-70B-shaped Q4 decode layer stack (80 layers), tensor-parallel over
    the N GPUs of one box.  QKV and gate+up column-sharded, o and down row-sharded with an all-reduce of
    the FP32 partials after each; KV length 4096; M = 1 (headline) and M = 32.  One step = the 80-layer
    stack once, one CUDA graph per rank.  Strong scaling: the model is fixed, each rank holds 1/N of it.

    Whatever goes wrong on any rank is caught, gathered over a host-side (gloo) group and printed by
    rank 0 in the JSON line together with the timings taken so far; the exit code is then non-zero."""
    import datetime

    import torch
    import torch.distributed as dist

    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=180))
    host_group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=300))
    state = {"phase": "start", "results": {}, "checks": {}, "clocks": None, "launches": 0}
    error = None
    try:
        _tp_body(args, torch, dist, world, rank, local_rank, device, state)
    except BaseException as exc:                       # noqa: BLE001 - reported, then the exit code says so
        error = f"rank {rank} in phase '{state['phase']}': {type(exc).__name__}: {exc}"
    errors = [None] * world
    try:
        dist.all_gather_object(errors, error, group=host_group)
    except BaseException as exc:                       # noqa: BLE001
        errors = [error or f"rank {rank}: error gather failed: {exc}"]
    failed = [e for e in errors if e]
    if rank == 0:
        print(json.dumps(_tp_line(args, world, state, failed)), flush=True)
    try:
        dist.destroy_process_group()
    except BaseException:                              # noqa: BLE001
        pass
    if failed:
        sys.exit(1)


def _tp_cfg():
    from tensorwarp_b200 import tensor_parallel as tp
    kv_len = 4096
    base = tp.LLAMA3_70B
    return type(base)(**{**base.__dict__, "max_seq": kv_len + 128}), kv_len


def _tp_stack_bytes(cfg, spec, m):
    hd = cfg.head_dim
    gemms = [(cfg.hidden, spec.n_qkv), ((spec.q_heads[1] - spec.q_heads[0]) * hd, cfg.hidden),
             (cfg.hidden, spec.n_gu), (spec.n_gu // 2, cfg.hidden)]
    return cfg.layers * sum(algorithmic_bytes(m, n, k, cfg.group_size, 2, 4 if n == cfg.hidden else 2) for k, n in gemms)


def _tp_body(args, torch, dist, world, rank, local_rank, device, state):
    from tensorwarp_b200 import quantize as q
    from tensorwarp_b200 import tensor_parallel as tp

    cfg, kv_len = _tp_cfg()
    spec = tp.shard_spec(cfg, world, rank)
    state["phase"] = "building the rank's weights"
    layers = [tp.random_shard_layer(cfg, spec, li, device) for li in range(cfg.layers)]
    torch.cuda.synchronize()
    state["stack_bytes_m1"] = _tp_stack_bytes(cfg, spec, 1)
    tiny = torch.zeros(8, device=device)

    def check_all_ranks(what, stream=None):
        """The device error word of every rank, decided together so that all ranks raise or none."""
        w = torch.tensor([q.device_error(stream)], device=device, dtype=torch.int32)
        dist.all_reduce(w, op=dist.ReduceOp.MAX)
        if int(w.item()):
            raise RuntimeError(f"device error word {int(w.item()):#x} on some rank after {what} "
                               "(bit 0 mbarrier wait, bit 1 split-K / chain wait, bit 2 peer-flag wait ran out)")

    # generous limit for the consumer's wait on the peers (the ranks are aligned on the device before
    # every phase; the limit only matters if a rank dies)
    comm = tp.PeerComm.distributed(32 * cfg.hidden, wait_ms=10000.0)

    # ---- exactness of the fused all-reduce: x after the first exchange against the rank-order sum of
    # the gathered partials, bit for bit (the order twm_allreduce_add_rmsnorm adds in)
    state["phase"] = "cross-check of the fused all-reduce"
    x0 = torch.randn((1, cfg.hidden), generator=torch.Generator().manual_seed(7)).to(device)
    sp = torch.cuda.current_stream().cuda_stream
    st_n = tp.TPDecodeStack(cfg, spec, layers[:1], 1, device, all_reduce=lambda t: None, comm=None)
    st_n.prefill_random_kv(kv_len, seed=2)
    st_n.x.copy_(x0)
    st_n.attn_phase(0, sp)
    torch.cuda.synchronize()
    gathered = [torch.zeros_like(st_n.part) for _ in range(world)]
    dist.all_gather(gathered, st_n.part)
    acc = gathered[0].clone()
    for r in range(1, world):
        acc += gathered[r]
    ref_x = x0 + acc
    st_f = tp.TPDecodeStack(cfg, spec, layers[:1], 1, device, all_reduce=lambda t: None, comm=comm)
    st_f.prefill_random_kv(kv_len, seed=2)
    st_f.x.copy_(x0)
    torch.cuda.synchronize()
    dist.barrier()
    dist.all_reduce(tiny)                              # ranks meet on the device before the first peer wait
    st_f.attn_phase(0, sp)
    st_f._join_and_norm(st_f.normed.data_ptr(), layers[0].ffn_norm.data_ptr(), sp)
    torch.cuda.synchronize()
    check_all_ranks("the one-exchange cross-check")
    diff = (st_f.x - ref_x).abs().max() / ref_x.pow(2).mean().sqrt()
    d = torch.tensor([float(diff)], device=device)
    dist.all_reduce(d, op=dist.ReduceOp.MAX)
    state["checks"]["max_rel_diff_vs_rank_order_sum"] = float(d.item())
    if float(d.item()) != 0.0:
        raise RuntimeError(f"fused all-reduce differs from the rank-order sum of the partials: {float(d.item())}")
    del st_n, st_f

    final_x = {}
    # (rows, collective): "fused" = the row-parallel GEMM epilogues store their FP32 partials into every
    # rank's receive buffer over NVLink and the add+RMSNorm kernel sums them (no collective launch);
    # "nccl" = ncclAllReduce between the GEMM and the add+RMSNorm kernel.
    for rows, coll in ((1, "fused"), (1, "nccl"), (32, "fused"), (32, "nccl")):
        key = f"m{rows}_{coll}"
        state["phase"] = f"{key}: set-up"
        stack = tp.TPDecodeStack(cfg, spec, layers, rows, device, all_reduce=lambda t: dist.all_reduce(t),
                                 comm=comm if coll == "fused" else None)
        stack.prefill_random_kv(kv_len, seed=2)
        host_x = torch.randn((rows, cfg.hidden), generator=torch.Generator().manual_seed(7)).pin_memory()
        host_out = torch.empty((rows, cfg.hidden)).pin_memory()
        stream = torch.cuda.Stream(device)
        with torch.cuda.stream(stream):
            stack.x.copy_(host_x, non_blocking=True)
            torch.cuda.synchronize()
            dist.barrier()
            state["phase"] = f"{key}: eager warm-up"
            dist.all_reduce(tiny)                             # on `stream`: the ranks start the forward together
            stack.forward(stream.cuda_stream)                 # eager once (NCCL and kernel warm-up)
            torch.cuda.synchronize()
            check_all_ranks(f"{key} eager warm-up", stream)
            state["phase"] = f"{key}: capture"
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                stack.forward(stream.cuda_stream)
            torch.cuda.synchronize()
            dist.barrier()
            state["phase"] = f"{key}: graph warm-up"
            dist.all_reduce(tiny)
            for _ in range(args.warmup):
                graph.replay()
            torch.cuda.synchronize()
            check_all_ranks(f"{key} graph warm-up", stream)
            dist.barrier()
            torch.cuda.synchronize()
            state["phase"] = f"{key}: timed region"
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with ClockSampler(local_rank) as clocks:
                dist.all_reduce(tiny)
                e0.record(stream)
                for _ in range(args.steps):
                    graph.replay()
                e1.record(stream)
                torch.cuda.synchronize()
            dist.barrier()
            t = torch.tensor([e0.elapsed_time(e1)], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item()) / args.steps
            # end to end, a separately timed loop: activations from pinned host memory in, result back out, every step
            state["phase"] = f"{key}: end-to-end loop"
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.all_reduce(tiny)
            f0.record(stream)
            for _ in range(args.steps):
                stack.x.copy_(host_x, non_blocking=True)
                graph.replay()
                host_out.copy_(stack.x, non_blocking=True)
            f1.record(stream)
            torch.cuda.synchronize()
            t = torch.tensor([f0.elapsed_time(f1)], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item()) / args.steps
            check_all_ranks(f"{key} timed loops", stream)
        total_bytes = world * _tp_stack_bytes(cfg, spec, rows)
        state["phase"] = f"{key}: final step"
        with torch.cuda.stream(stream):                       # one more step from the same input, kept for the comparison below
            dist.barrier()
            stack.x.copy_(host_x, non_blocking=True)
            dist.all_reduce(tiny)
            graph.replay()
            torch.cuda.synchronize()
        final_x[(rows, coll)] = stack.x.clone()
        fin = torch.tensor([1 if bool(torch.isfinite(stack.x).all().item()) else 0], device=device)
        dist.all_reduce(fin, op=dist.ReduceOp.MIN)
        state["results"][key] = {"ms_per_step": round(ms, 4), "gbs": round(total_bytes / (ms * 1e-3) / 1e9, 1),
                                 "e2e_ms_per_step": round(e2e_ms, 4), "e2e_gbs": round(total_bytes / (e2e_ms * 1e-3) / 1e9, 1),
                                 "e2e_note": "separately timed loop with the H2D/D2H copies; run-to-run noise can put it either side of ms_per_step",
                                 "launches": stack.launches, "allreduce_bytes": rows * cfg.hidden * 4,
                                 "allreduces_per_step": 2 * cfg.layers, "h2d": rows * cfg.hidden * 4,
                                 "d2h": rows * cfg.hidden * 4, "finite": bool(int(fin.item()))}
        if key == "m1_fused":
            state["clocks"] = clocks.summary()
        if not int(fin.item()):
            raise RuntimeError(f"{key}: non-finite activations after the stack")
        del stack, graph
        torch.cuda.empty_cache()
    # Informational: the two collectives over all 80 layers.  Both norm kernels take the sum of squares in
    # the same order, so with two ranks (a + b is the same sum either way) the two paths agree bit for
    # bit; with more ranks NCCL adds the partials in its own order and single FP16 roundings may flip.
    state["phase"] = "fused against NCCL over the whole stack"
    ref_x, got_x = final_x[(1, "nccl")], final_x[(1, "fused")]
    d = torch.tensor([float((got_x - ref_x).abs().max() / ref_x.pow(2).mean().sqrt())], device=device)
    dist.all_reduce(d, op=dist.ReduceOp.MAX)
    state["checks"]["max_rel_diff_vs_nccl_80_layers"] = float(d.item())
    dist.barrier()
    comm.close()
    state["phase"] = "done"


def _tp_line(args, world, state, failed):
    peak, peak_kind = measured_peak_gbs()
    res = state["results"]
    r1 = res.get("m1_fused")
    line = {
        "metric": METRIC, "value": r1["gbs"] if r1 else None, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r1["ms_per_step"] if r1 else None, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"configs[4]: Llama-3-70B-shaped Q4 decode layer stack, 80 layers, tensor parallel tp={world}, "
                               "M=1, KV 4096, Q4 group-128 (the tp=1 point of this curve is the `tp1` key of the --gpus 1 line)",
                   "l2": f"inputs larger than L2: {state.get('stack_bytes_m1', 0) / 1e9:.2f} GB of weights streamed per rank per step",
                   "launch": "one CUDA graph per rank; o and down GEMM epilogues push FP32 partials to every rank over "
                             "NVLink peer memory, the add+RMSNorm kernel sums them (one-shot all-reduce, no collective launch)",
                   "parallelism": f"tp{world}"},
        "roofline": {"bound": "hbm", "achieved": round(r1["gbs"] / world, 1) if r1 else None, "peak": peak, "unit": "GB/s",
                     "frac": round(r1["gbs"] / world / peak, 4) if r1 else None, "peak_kind": peak_kind,
                     "kernel": "twm::mma::gemv_kernel<1,2> (per rank, whole step incl. collectives)", "traffic": None},
        "e2e": {"value": r1["e2e_gbs"] if r1 else None, "unit": UNIT, "h2d_bytes_per_step": r1["h2d"] if r1 else 0,
                "d2h_bytes_per_step": r1["d2h"] if r1 else 0},
        "gpu_launches": r1["launches"] * args.steps if r1 else 0,
        "clocks": state["clocks"],
        "tp": dict(res, gemm_launches_per_step=4 * 80, **state["checks"]),
    }
    if failed:
        line["error"] = failed[0]
        line["errors"] = failed
        line["cross_check"] = "failed"
    else:
        line["cross_check"] = "passed"
    return line


# dram__bytes_read.sum + dram__bytes_write.sum per launch, averaged over one layer's four kernels
# (8 588 032 + 6 695 424 + 70 571 264 + 35 111 936 bytes for qkv, o, gate+up, down; one ncu capture per
# shape, summarised in profiles/bench_config1_launch_list.md)
TRAFFIC_PER_LAUNCH = 30241664


# ------------------------------------------------------- CPU baseline arm --

def _cpu_sample_inputs(np, oracle, k, n, seed):
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)
    packed, scales = oracle.quantize_pack(w, k, n, GROUP)
    a = rng.standard_normal((1, k), dtype=np.float32).astype(np.float16).astype(np.float32)
    return a, packed, scales


def cpu_baseline(target_seconds: float):
    """The reference's CPU route (dequantise, multiply, FP32 accumulate) restated in C, all host
    threads, on a bounded sample: the o-projection GEMM (K=3584, N=3584) repeated."""
    import numpy as np

    import oracle
    k, n = 3584, 3584
    a, packed, scales = _cpu_sample_inputs(np, oracle, k, n, 7)
    oracle.w4a16_threaded(a, packed, scales, 1, n, k, GROUP)       # warm
    t0 = time.perf_counter()
    reps = 0
    while True:
        _, used = oracle.w4a16_threaded(a, packed, scales, 1, n, k, GROUP)
        reps += 1
        if time.perf_counter() - t0 > target_seconds or reps >= 2000:
            break
    dt = time.perf_counter() - t0
    value = reps * algorithmic_bytes(1, n, k, GROUP) / dt / 1e9
    return {"value": round(value, 3), "unit": UNIT, "cores": used, "kind": "port",
            "sample": f"o-projection GEMM K={k} N={n} M=1 G={GROUP}, {reps} repetitions, {dt:.1f} s"}


def _random_tw_marlin(np, k, n, seed):
    """Random nibbles and scales of the right shapes: the CPU route's time does not depend on the
    values, and quantising gigabytes of FP32 weights on the host would only delay the run."""
    rng = np.random.default_rng(seed)
    packed = rng.integers(0, 256, size=(k // 32, n, 16), dtype=np.uint8)
    scales = (rng.random((k // GROUP, n), dtype=np.float32) * np.float32(0.01)).astype(np.float16).view(np.uint16)
    a = rng.standard_normal((1, k), dtype=np.float32).astype(np.float16).astype(np.float32)
    return a, packed, scales


def run_reference(args):
    """Reference arm: the reference's own CPU implementation of the path.  Its Rust cannot be built
    here (no cargo/rustc), so this is the C restatement under oracle/ (dequantise, multiply, FP32
    accumulate), on every host core the process may use.

    --gpus 1: one step = the 28-layer configs[1] GEMM set (112 GEMMs, cycling over four weight sets;
    the CPU route is compute-bound at a few GB/s, far below host memory bandwidth).
    --gpus N > 1: the repo arm runs the configs[4] stack; one step here = ONE of its 80 layers at full
    (unsharded) size, labelled as such: a bounded sample, both sides are bytes per second."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np

    import oracle
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cores = len(os.sched_getaffinity(0))
    oracle.set_threads(cores)                          # a launcher may have set OMP_NUM_THREADS=1
    if world == 1:
        sets = 4
        inputs = [[_random_tw_marlin(np, k, n, 100 + 10 * si + i) for i, (_, k, n) in enumerate(LAYER_GEMMS)] for si in range(sets)]
        shapes = [(k, n) for _, k, n in LAYER_GEMMS]
        layers_per_step = LAYERS
        step_bytes = LAYERS * layer_bytes(1)
        workload = ("configs[1]: Qwen2-7B-shaped decode GEMM set, M=1, 4 GEMMs x 28 layers, Q4 group-128, on the host cores "
                    f"(cycling over {sets} weight sets)")
        sample = f"the full step: {LAYERS} layers x 4 GEMMs, {step_bytes} algorithmic bytes"
    else:
        cfg, _ = _tp_cfg()
        shapes = [(cfg.hidden, cfg.q_dim + 2 * cfg.kv_dim), (cfg.q_dim, cfg.hidden), (cfg.hidden, 2 * cfg.ffn), (cfg.ffn, cfg.hidden)]
        inputs = [[_random_tw_marlin(np, k, n, 200 + i) for i, (k, n) in enumerate(shapes)]]
        layers_per_step = 1
        step_bytes = sum(algorithmic_bytes(1, n, k, GROUP, 2, 4 if n == cfg.hidden else 2) for k, n in shapes)
        workload = ("configs[4]: Llama-3-70B-shaped Q4 decode layer stack, M=1, Q4 group-128, on the host cores; "
                    "one step = ONE of the 80 layers at full size (a bounded sample)")
        sample = f"one of 80 layers per step (4 GEMMs, {step_bytes} algorithmic bytes)"
    used = 1

    def step():
        nonlocal used
        for layer in range(layers_per_step):
            for (a, packed, scales), (k, n) in zip(inputs[layer % len(inputs)], shapes):
                _, used = oracle.w4a16_threaded(a, packed, scales, 1, n, k, GROUP)

    warm = min(args.warmup, 1)
    for _ in range(warm):
        step()
    steps = args.steps
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    value = steps * step_bytes / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT,
        "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": round(dt / steps * 1e3, 3), "higher_is_better": True, "scaling": "weak" if world == 1 else "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload},
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": used, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the configs[3] decode tok/s measurement")
    args = ap.parse_args()
    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 5
        args.warmup = args.warmup if args.warmup is not None else 1
        args.steps = min(args.steps, 20)          # each step is about two seconds of CPU work: the run stays under a minute
        run_reference(args)
    else:
        world = int(os.environ.get("WORLD_SIZE", "1"))
        args.warmup = max(args.warmup if args.warmup is not None else 5, 3)
        if world > 1:
            args.steps = args.steps if args.steps is not None else 20
            run_tp(args)
        else:
            args.steps = args.steps if args.steps is not None else 50
            run_ours(args)


if __name__ == "__main__":
    main()
