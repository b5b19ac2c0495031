"""The tensor-parallel stack as real processes, one per GPU (skipped on boxes with fewer than two):
bench.py under torch.distributed.run.  Its body gathers every rank's partial o output, adds them
in rank order on the host side of NCCL, and requires the fused one-shot all-reduce (GEMM epilogues
storing into the peers' memory over NVLink, add + RMSNorm consumer) to give exactly those bits;
it also runs the 80-layer stack with both collectives and requires finite results and a clean
device error word on every rank.  No GPU is made to fault or hang: every peer wait is bounded."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_bench_cross_checks():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29571", os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "2", "--warmup", "3"]
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert line.get("error") is None and line["cross_check"] == "passed"
    assert line["n_gpus"] == 2 and line["tp"]["max_rel_diff_vs_rank_order_sum"] == 0.0
    assert line["tp"]["max_rel_diff_vs_nccl_80_layers"] == 0.0          # two ranks: a + b is the same sum either way
    for key in ("m1_fused", "m1_nccl", "m32_fused", "m32_nccl"):
        assert line["tp"][key]["finite"] and line["tp"][key]["ms_per_step"] > 0
