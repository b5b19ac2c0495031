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

    def enqueue_all(extra_flags=0):
        ao = co = 0
        for layer in range(LAYERS):
            for pid, (_, k, n) in enumerate(LAYER_GEMMS):
                p, s = weights[layer][pid]
                q.gemm_tw_marlin_m1(dev_a[ao:ao + k], p, s, dev_c[co:co + n], n, k, group_size=GROUP,
                                    workspace=ws, flags=flags | extra_flags)
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
        e2e_ms = f0.elapsed_time(f1)
        if world > 1:
            t = torch.tensor([e2e_ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
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
    err = q.device_error(stream)
    if err:
        raise RuntimeError(f"device error word {err:#x}")
    decode = None
    sweep = None
    config0 = None
    if not args.no_decode and rank == 0:
        del weights, graph
        torch.cuda.empty_cache()
        sweep = m_sweep(torch, q, device)
        torch.cuda.empty_cache()
        config0 = config0_gemv(torch, q, device)
        torch.cuda.empty_cache()
        decode = decode_tok_s(torch, device)

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
                "d2h_bytes_per_step": int(host_c.numel() * 2)},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks.summary(),
    }
    if independent is not None:
        ind_gbs = step_bytes / (independent["ms_per_step"] * 1e-3) / 1e9
        independent.update({"gbs": round(ind_gbs, 1), "hbm_frac": round(ind_gbs / peak, 4),
                            "note": "same GEMM set without the wait for the preceding launch (TWM_FLAG_INDEPENDENT); diagnostic"})
        line["independent_launches"] = independent
    if decode is not None:
        line["decode"] = decode
    if sweep is not None:
        line["m_sweep"] = sweep
    if config0 is not None:
        line["config0"] = config0
    if rank == 0:
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(target_seconds=12.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
    weight sets per graph (568 MB, larger than L2), programmatic dependent launch; microseconds per
    GEMM (for M above one launch's rows: all its launches), the kernel the heuristic chose, HBM and
    tensor fractions of the measured peaks."""
    from tensorwarp_b200 import _lib
    k, n, copies = 3584, 37888, 8
    names = {_lib.TWM_KERNEL_SIMT: "simt", _lib.TWM_KERNEL_TC: "tcgen05", _lib.TWM_KERNEL_MMA: "mma"}
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
            for p_, s_ in ws:
                q.gemm_tw_marlin(a, p_, s_, c, m, n, k, group_size=GROUP, workspace=wsb, flags=_lib.TWM_FLAG_PDL)

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
        return e0.elapsed_time(e1), eng.launches_per_step, bool(all(0 <= t < cfg.vocab for t in toks))

    ms, launches, in_vocab = run(False)
    q4_bytes = cfg.layers * layer_bytes(1)
    kv_bytes = cfg.layers * 2 * (kv_len + new_tokens // 2) * cfg.kv_dim * 2
    step_bytes = q4_bytes + cfg.vocab * cfg.hidden * 2 + kv_bytes
    out = {"tok_s": round(new_tokens / (ms * 1e-3), 1), "ms_per_token": round(ms / new_tokens, 4),
           "workload": f"configs[3]: Qwen2-7B-shaped Q4 decode, KV {kv_len} FP16, {new_tokens} greedy tokens, one CUDA graph per token",
           "launches_per_token": launches, "bytes_per_token": int(step_bytes),
           "hbm_gbs": round(step_bytes / (ms / new_tokens * 1e-3) / 1e9, 1), "tokens_in_vocab": in_vocab}
    ms4, _, in_vocab4 = run(True)
    step_bytes4 = q4_bytes + algorithmic_bytes(1, cfg.vocab, cfg.hidden, GROUP, 2, 4) + kv_bytes
    out["q4_lm_head"] = {"tok_s": round(new_tokens / (ms4 * 1e-3), 1), "ms_per_token": round(ms4 / new_tokens, 4),
                         "bytes_per_token": int(step_bytes4), "tokens_in_vocab": in_vocab4}
    return out


# ------------------------------------------------------------- tensor parallel --

def run_tp(args):
    """N > 1: configs[4], the Llama-3-70B-shaped Q4 decode layer stack (80 layers), tensor-parallel over
    the N GPUs of one box.  QKV and gate+up column-sharded, o and down row-sharded with an NCCL
    all-reduce (FP32 partials) after each; KV length 4096; M = 1 (headline) and M = 32.  One step =
    the 80-layer stack once, one CUDA graph per rank.  Strong scaling: the model is fixed, each
    rank holds 1/N of it."""
    import torch
    import torch.distributed as dist

    from tensorwarp_b200 import quantize as q
    from tensorwarp_b200 import tensor_parallel as tp

    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)

    kv_len = 4096
    base = tp.LLAMA3_70B
    cfg = type(base)(**{**base.__dict__, "max_seq": kv_len + 128})
    spec = tp.shard_spec(cfg, world, rank)
    layers = [tp.random_shard_layer(cfg, spec, li, device) for li in range(cfg.layers)]
    torch.cuda.synchronize()
    hd = cfg.head_dim
    shard_gemms = [(cfg.hidden, spec.n_qkv), ((spec.q_heads[1] - spec.q_heads[0]) * hd, cfg.hidden),
                   (cfg.hidden, spec.n_gu), (spec.n_gu // 2, cfg.hidden)]

    def stack_bytes(m):
        return cfg.layers * sum(algorithmic_bytes(m, n, k, cfg.group_size, 2, 4 if n == cfg.hidden else 2)
                                for k, n in shard_gemms)

    results = {}
    clocks_summary = None
    comm = tp.PeerComm.distributed(2 * cfg.hidden)
    final_x = {}
    # (rows, collective): "fused" = the row-parallel GEMM epilogues store their FP32 partials into every
    # rank's receive buffer over NVLink and the add+RMSNorm kernel sums them (no collective launch);
    # "nccl" = ncclAllReduce between the GEMM and the add+RMSNorm kernel.
    for rows, coll in ((1, "fused"), (1, "nccl"), (32, "nccl")):
        stack = tp.TPDecodeStack(cfg, spec, layers, rows, device, all_reduce=lambda t: dist.all_reduce(t),
                                 comm=comm if coll == "fused" else None)
        stack.prefill_random_kv(kv_len, seed=2)
        host_x = torch.randn((rows, cfg.hidden), generator=torch.Generator().manual_seed(7)).pin_memory()
        host_out = torch.empty((rows, cfg.hidden)).pin_memory()
        stream = torch.cuda.Stream(device)
        with torch.cuda.stream(stream):
            stack.x.copy_(host_x, non_blocking=True)
            torch.cuda.synchronize()
            dist.barrier()                                    # ranks enter each phase together: device-side waits are bounded
            stack.forward(stream.cuda_stream)                 # eager once (NCCL and kernel warm-up)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                stack.forward(stream.cuda_stream)
            torch.cuda.synchronize()
            dist.barrier()
            for _ in range(args.warmup):
                graph.replay()
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with ClockSampler(local_rank) as clocks:
                e0.record(stream)
                for _ in range(args.steps):
                    graph.replay()
                e1.record(stream)
                torch.cuda.synchronize()
            dist.barrier()
            t = torch.tensor([e0.elapsed_time(e1)], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item()) / args.steps
            # end to end: activations from pinned host memory in, result back out, every step
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
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
        total_bytes = world * stack_bytes(rows)
        with torch.cuda.stream(stream):                       # one more step from the same input, kept for the cross-check
            dist.barrier()
            stack.x.copy_(host_x, non_blocking=True)
            graph.replay()
            torch.cuda.synchronize()
        final_x[(rows, coll)] = stack.x.clone()
        results[(rows, coll)] = {"ms_per_step": round(ms, 4), "gbs": round(total_bytes / (ms * 1e-3) / 1e9, 1),
                         "e2e_gbs": round(total_bytes / (e2e_ms * 1e-3) / 1e9, 1), "launches": stack.launches,
                         "allreduce_bytes": rows * cfg.hidden * 4, "allreduces_per_step": 2 * cfg.layers,
                         "h2d": rows * cfg.hidden * 4, "d2h": rows * cfg.hidden * 4,
                         "finite": bool(torch.isfinite(stack.x).all().item())}
        if (rows, coll) == (1, "fused"):
            clocks_summary = clocks.summary()
        del stack, graph
        torch.cuda.empty_cache()
    # The two collectives must agree.  The sum of squares inside the two norm kernels is taken in a
    # different order, so FP16 roundings of the normed activations can flip; over 80 random layers such
    # flips grow, so the strict comparison is on the first two layers and the full depth is reported.
    ref_x, got_x = final_x[(1, "nccl")], final_x[(1, "fused")]
    rel_full = float((got_x - ref_x).abs().max() / ref_x.pow(2).mean().sqrt())
    short = {}
    for coll in ("fused", "nccl"):
        st2 = tp.TPDecodeStack(cfg, spec, layers[:2], 1, device, all_reduce=lambda t: dist.all_reduce(t),
                               comm=comm if coll == "fused" else None)
        st2.prefill_random_kv(kv_len, seed=2)
        st2.x.copy_(torch.randn((1, cfg.hidden), generator=torch.Generator().manual_seed(7)))
        torch.cuda.synchronize()
        dist.barrier()
        st2.forward(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        short[coll] = st2.x.clone()
        del st2
    rel = float((short["fused"] - short["nccl"]).abs().max() / short["nccl"].pow(2).mean().sqrt())
    # With two ranks both paths add the same two FP32 partials (same bits in every run so far).  With
    # more, NCCL's order of additions is its own while the fused path adds in rank order: the FP32 sums
    # differ in the last bit, an FP16 rounding of a normed activation can flip, and one flip moves the
    # output by about 1e-3 of its RMS (measured 1.2e-3 at four ranks).
    tol = 1e-3 if world == 2 else 1e-2
    if not rel < tol:
        raise RuntimeError(f"fused all-reduce result differs from the NCCL path: {rel}")
    dist.barrier()
    comm.close()
    err = q.device_error()
    if err:
        raise RuntimeError(f"device error word {err:#x}")
    peak, peak_kind = measured_peak_gbs()
    r1 = results[(1, "fused")]
    r1["max_rel_diff_vs_nccl_2_layers"] = rel
    r1["max_rel_diff_vs_nccl_80_layers"] = rel_full
    gemm_launches = 4 * cfg.layers
    line = {
        "metric": METRIC, "value": r1["gbs"], "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": r1["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"configs[4]: Llama-3-70B-shaped Q4 decode layer stack, 80 layers, tensor parallel tp={world}, "
                               "M=1, KV 4096, Q4 group-128",
                   "l2": f"inputs larger than L2: {stack_bytes(1) / 1e9:.2f} GB of weights streamed per rank per step",
                   "launch": "one CUDA graph per rank; o and down GEMM epilogues push FP32 partials to every rank over "
                             "NVLink peer memory, the add+RMSNorm kernel sums them (one-shot all-reduce, no collective launch)",
                   "parallelism": f"tp{world}"},
        "roofline": {"bound": "hbm", "achieved": round(r1["gbs"] / world, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(r1["gbs"] / world / peak, 4), "peak_kind": peak_kind,
                     "kernel": "twm::mma::gemv_kernel<1,2> (per rank, whole step incl. collectives)", "traffic": None},
        "e2e": {"value": r1["e2e_gbs"], "unit": UNIT, "h2d_bytes_per_step": r1["h2d"], "d2h_bytes_per_step": r1["d2h"]},
        "gpu_launches": r1["launches"] * args.steps,
        "clocks": clocks_summary,
        "tp": {"m1_fused": r1, "m1_nccl": results[(1, "nccl")], "m32_nccl": results[(32, "nccl")],
               "gemm_launches_per_step": gemm_launches},
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum per launch, averaged over one layer's four kernels,
# from the ncu capture summarised in profiles/bench_config1_launch_list.md
TRAFFIC_PER_LAUNCH = 30116928


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


def run_reference(args):
    """Reference arm: the reference's own CPU implementation of the path.  Its Rust cannot be built
    here (no cargo/rustc), so this is the C restatement under oracle/, all host threads.  One step =
    one layer's four GEMMs (a bounded sample of the 28-layer workload)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np

    import oracle
    inputs = [_cpu_sample_inputs(np, oracle, k, n, 100 + i) for i, (_, k, n) in enumerate(LAYER_GEMMS)]
    used = 1

    def step():
        nonlocal used
        for (a, packed, scales), (_, k, n) in zip(inputs, LAYER_GEMMS):
            _, used = oracle.w4a16_threaded(a, packed, scales, 1, n, k, GROUP)

    for _ in range(min(args.warmup, 1)):
        step()
    steps = args.steps
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    value = steps * layer_bytes(1) / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT,
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": min(args.warmup, 1),
        "ms_per_step": round(dt / steps * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "configs[1]: Qwen2-7B-shaped decode GEMM set, M=1, Q4 group-128; one step = one layer's "
                               "four GEMMs on the host cores"},
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": used, "kind": "port",
                         "sample": f"{steps} x one layer (4 GEMMs, {layer_bytes(1)} algorithmic bytes)"},
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
        args.steps = min(args.steps, 20)          # each step is seconds of CPU work
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
