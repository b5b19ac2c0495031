"""One W4A16 GEMM shape, a few launches: the command the kernel profiles under profiles/ were taken with.

    python tests/run_one_gemm.py --m 256 --k 3584 --n 37888 --group 128 --kernel tcw --launches 4

Seeded random weights (quantised on the device) and FP16 N(0,1) activations; every launch goes
through tensorwarp_b200.quantize.gemm_tw_marlin with programmatic dependent launch, as in the
benchmarks.  Prints the mean device time per GEMM (CUDA events) and the library's error word.
`--tp-layers L --tp N` instead runs L layers of the tensor-parallel decode stack at degree N
(`--m` rows = sequences decoding in lock step) with every rank emulated on this one GPU (ranks enqueued one after another, so the producers of an
all-reduce have finished before its consumer starts)."""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tensorwarp_b200 import _lib  # noqa: E402
from tensorwarp_b200 import quantize as q  # noqa: E402

KERNELS = {"auto": 0, "simt": _lib.TWM_KERNEL_SIMT, "tc": _lib.TWM_KERNEL_TC, "mma": _lib.TWM_KERNEL_MMA,
           "tcw": _lib.TWM_KERNEL_TCW, "tcr": _lib.TWM_KERNEL_TCR}


def one_gemm(args) -> None:
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(args.seed)
    w = torch.randn((args.k, args.n), generator=gen, device=dev) * 0.02
    packed, scales = q.quantize_f32_to_tw_marlin(w, args.k, args.n, args.group)
    del w
    a_dtype = torch.float32 if args.kernel == "simt" else torch.float16
    a = torch.randn((args.m, args.k), generator=gen, device=dev).to(a_dtype)
    c = torch.empty((args.m, args.n), dtype=a_dtype, device=dev)
    kern = KERNELS[args.kernel]
    ws = q.Workspace(max(q.plan(args.m, args.n, args.k, args.group, kernel_override=kern, splits_override=args.splits).workspace_bytes, 16), dev)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(args.launches + 1):
            if i == 1:
                e0.record(stream)
            q.gemm_tw_marlin(a, packed, scales, c, args.m, args.n, args.k, group_size=args.group, workspace=ws,
                             flags=_lib.TWM_FLAG_PDL, kernel_override=kern, splits_override=args.splits)
        e1.record(stream)
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / max(args.launches, 1)
    pl = q.plan(args.m, args.n, args.k, args.group, kernel_override=kern, splits_override=args.splits)
    print(f"m={args.m} k={args.k} n={args.n} group={args.group} kernel={args.kernel} (plan: kernel {pl.kernel}, {pl.grid_x} tiles x {pl.splits} K slices): {us:.2f} us per GEMM "
          f"(eager launches, cold start included), error word {q.device_error():#x}")


def tp_layers(args) -> None:
    from tensorwarp_b200 import tensor_parallel as tp
    base = tp.LLAMA3_70B
    cfg = type(base)(**{**base.__dict__, "max_seq": args.kv + 8, "layers": args.tp_layers})
    dev = "cuda"
    comms = tp.PeerComm.local_group(args.tp, args.m * cfg.hidden)
    stacks = []
    for r in range(args.tp):
        spec = tp.shard_spec(cfg, args.tp, r)
        layers = [tp.random_shard_layer(cfg, spec, li, dev, args.seed) for li in range(cfg.layers)]
        st = tp.TPDecodeStack(cfg, spec, layers, args.m, dev, all_reduce=lambda t: None, comm=comms[r])
        st.prefill_random_kv(args.kv)
        st.x.copy_(torch.randn((args.m, cfg.hidden), generator=torch.Generator().manual_seed(args.seed)).to(dev))
        stacks.append(st)
    sp = torch.cuda.current_stream().cuda_stream
    for _ in range(2):                       # two passes: the second one is warm
        for li in range(cfg.layers):
            for st in stacks:
                st.attn_phase(li, sp)
            for st in stacks:
                st.ffn_phase(li, sp)
        for st in stacks:
            st.finish(sp)
        torch.cuda.synchronize()
    finite = all(bool(torch.isfinite(st.x).all()) for st in stacks)
    print(f"tp={args.tp}, {cfg.layers} layers, {args.m} row(s), KV {args.kv}: two passes over all ranks on one GPU, "
          f"finite={finite}, error word {q.device_error():#x}")
    for c in comms:
        c.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--k", type=int, default=3584)
    ap.add_argument("--n", type=int, default=37888)
    ap.add_argument("--group", type=int, default=128)
    ap.add_argument("--kernel", default="auto", choices=sorted(KERNELS))
    ap.add_argument("--launches", type=int, default=4)
    ap.add_argument("--splits", type=int, default=0, help="K slices (0 = the plan's choice)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--tp", type=int, default=0)
    ap.add_argument("--tp-layers", type=int, default=3)
    ap.add_argument("--kv", type=int, default=4096)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    if args.tp:
        tp_layers(args)
    else:
        one_gemm(args)


if __name__ == "__main__":
    main()
