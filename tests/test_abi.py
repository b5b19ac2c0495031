"""CPU tests of the boundary: the library builds, loads, exports every symbol the header
declares, and its pure-host entry points behave.  No compute call is made."""
import ctypes as C
import os
import re

import pytest

from tensorwarp_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in sorted(os.listdir(inc)):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names.update(re.findall(r"\b(twm_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_every_declared_symbol_is_exported_and_bound(twm_lib):
    names = _declared_symbols()
    assert "twm_gemm_w4a16" in names and "twm_plan" in names
    for name in names:
        assert hasattr(twm_lib, name), f"{name} declared in twmarlin.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"


def test_version_and_status_strings(twm_lib):
    assert b"sm_100a" in twm_lib.twm_version()
    for code in (0, -1, -2, -3, -4, -5, -6):
        assert len(twm_lib.twm_status_string(code)) > 0


def _plan(lib, *a):
    p = _lib.Plan()
    st = lib.twm_plan(*a, C.byref(p))
    return st, p


def test_plan_benchmark_shapes(twm_lib):
    # gate+up of the 7B shape: 296 tiles fill 148 SMs twice over -> never split
    st, p = _plan(twm_lib, 1, 37888, 3584, 128, 148, 0, 0)
    assert st == 0 and p.splits == 1 and p.grid_x == 296 and p.workspace_bytes == 0
    # the heuristic stays on the split-K kernel for FP16 activations up to eight rows
    assert _plan(twm_lib, 1, 4608, 3584, 128, 148, 0, 0)[1].kernel == _lib.TWM_KERNEL_MMA
    # small-N shapes must split to cover the machine (the reference's k<2048 cut-off is not inherited)
    for (n, k) in ((4608, 3584), (3584, 3584), (3584, 18944), (9728, 896)):
        # M=1 on the streaming MMA kernel: the slices of a tile form a cluster, no workspace
        st, p = _plan(twm_lib, 1, n, k, 128, 148, 0, 0)
        assert st == 0
        assert 1 < p.splits <= 16 and p.cluster_reduce == 1 and p.workspace_bytes == 0, (n, k)
        assert 100 <= p.grid_x * p.grid_y <= 2 * 148, (n, k, p.grid_x, p.grid_y)
        assert p.blocks_per_split * p.splits >= k // 32 > p.blocks_per_split * (p.splits - 1)
        assert p.blocks_per_split % 4 == 0          # whole 128-groups per slice
        # the FP32 kernel (the reference's f32 signature) splits through the workspace
        st, p = _plan(twm_lib, 1, n, k, 128, 148, 0, _lib.TWM_KERNEL_SIMT)
        assert st == 0 and p.splits > 1 and p.cluster_reduce == 0
        assert p.workspace_bytes == 16384 + p.splits * n * 4
        assert twm_lib.twm_workspace_bytes(1, n, k, 128) >= p.workspace_bytes
    # deterministic
    a = _plan(twm_lib, 4, 4608, 3584, 32, 148, 0, 0)[1]
    b = _plan(twm_lib, 4, 4608, 3584, 32, 148, 0, 0)[1]
    assert (a.splits, a.blocks_per_split, a.grid_x) == (b.splits, b.blocks_per_split, b.grid_x)


def test_plan_rows_and_staged_activations(twm_lib):
    """Which kernel the heuristic names by row count, and the workspace a plan asks for: the streaming MMA kernel up
    to 32 rows, with room for the staged rows ([K/32][rows16][64 B] + [K/G][rows16] f32 behind counters and K-slice
    partials) from nine rows on any matrix and from three rows on matrices of 2^26 weights."""
    k, n, g = 3584, 37888, 128
    kinds = [_plan(twm_lib, m, n, k, g, 148, 0, 0)[1].kernel for m in (1, 8, 9, 16, 32, 33, 64, 65, 256)]
    assert kinds == [_lib.TWM_KERNEL_MMA] * 5 + [_lib.TWM_KERNEL_TC] * 2 + [_lib.TWM_KERNEL_TCR] * 2
    for m, rows in ((9, 16), (16, 16), (17, 24), (24, 24), (25, 32), (32, 32)):
        p = _plan(twm_lib, m, n, k, g, 148, 0, _lib.TWM_KERNEL_MMA)[1]
        assert p.splits == 1 and p.cluster_reduce == 0
        assert p.workspace_bytes == 16384 + 256 + (k // 32) * rows * 64 + (k // g) * rows * 4, m
        assert twm_lib.twm_workspace_bytes(m, n, k, g) >= p.workspace_bytes
    # three to eight rows: staged on the large matrix, the CTAs' own stager warps on the small one
    assert _plan(twm_lib, 3, n, k, g, 148, 0, _lib.TWM_KERNEL_MMA)[1].workspace_bytes == 16384 + 256 + (k // 32) * 8 * 64 + (k // g) * 8 * 4
    assert _plan(twm_lib, 2, n, k, g, 148, 0, _lib.TWM_KERNEL_MMA)[1].workspace_bytes == 0
    small = _plan(twm_lib, 4, 4608, k, g, 148, 0, _lib.TWM_KERNEL_MMA)[1]
    assert small.splits > 1 and small.workspace_bytes == 16384 + small.splits * 4 * 4608 * 4
    # ... but a caller may need the staged form there too (a push to tensor-parallel peers): covered by the size query
    assert twm_lib.twm_workspace_bytes(4, 4608, k, g) >= small.workspace_bytes + 256 + (k // 32) * 8 * 64 + (k // g) * 8 * 4
    # more rows than one launch carries: planned for the first launch's 32
    p40 = _plan(twm_lib, 40, 4608, k, g, 148, 0, _lib.TWM_KERNEL_MMA)[1]
    assert p40.workspace_bytes == 16384 + p40.splits * 32 * 4608 * 4 + 256 + (k // 32) * 32 * 64 + (k // g) * 32 * 4
    # a K slice count that needs a second wave of CTAs is not chosen over one wave (70B-sized down projection)
    p = _plan(twm_lib, 1, 8192, 28672, g, 148, 0, 0)[1]
    assert p.grid_x * p.grid_y <= 2 * 148 and p.splits == 4


def test_plan_rejects_bad_shapes(twm_lib):
    assert _plan(twm_lib, 1, 128, 100, 32, 148, 0, 0)[0] == _lib.TWM_EINVAL     # K % 32
    assert _plan(twm_lib, 1, 128, 96, 128, 148, 0, 0)[0] == _lib.TWM_EINVAL     # K % G
    assert _plan(twm_lib, 1, 128, 128, 64, 148, 0, 0)[0] == _lib.TWM_EINVAL     # G not 32/128
    assert _plan(twm_lib, 0, 128, 128, 32, 148, 0, 0)[0] == _lib.TWM_EINVAL
    assert _plan(twm_lib, 1, 0, 128, 32, 148, 0, 0)[0] == _lib.TWM_EINVAL
    assert _plan(twm_lib, 1, 128, 128, 32, 148, 65, 0)[0] == _lib.TWM_EINVAL    # splits_override > 64
    assert twm_lib.twm_plan(1, 128, 128, 32, 148, 0, 0, None) == _lib.TWM_EINVAL


def test_plan_override(twm_lib):
    st, p = _plan(twm_lib, 1, 256, 1024, 32, 148, 5, 0)
    assert st == 0 and p.blocks_per_split == 7 and p.splits == 5    # 32 blocks in 5 slices of <= 7


def test_gemm_argument_errors_need_no_gpu(twm_lib):
    """Null pointers, bad dtypes and misalignment are rejected before any CUDA call."""
    args = _lib.GemmArgs(M=1, N=128, K=128, group_size=32, a_dtype=0, c_dtype=0, a=None, lda=128,
                         packed=0x1000, scales=0x2000, c=0x3000, ldc=128)
    assert twm_lib.twm_gemm_w4a16(C.byref(args), None) == _lib.TWM_EINVAL
    args.a = 0x4000
    args.a_dtype = 7
    assert twm_lib.twm_gemm_w4a16(C.byref(args), None) == _lib.TWM_EINVAL
    args.a_dtype = 0
    args.packed = 0x1008
    assert twm_lib.twm_gemm_w4a16(C.byref(args), None) == _lib.TWM_EALIGN
    args.packed = 0x1000
    args.lda = 64
    assert twm_lib.twm_gemm_w4a16(C.byref(args), None) == _lib.TWM_EINVAL
    assert twm_lib.twm_gemm_w4a16(None, None) == _lib.TWM_EINVAL


def test_slice_k_offsets(twm_lib):
    po, so = C.c_size_t(), C.c_size_t()
    assert twm_lib.twm_slice_k_offsets(8192, 1024, 128, 1024, 1024, C.byref(po), C.byref(so)) == 0
    assert po.value == (1024 // 32) * 1024 * 16 and so.value == (1024 // 128) * 1024
    assert twm_lib.twm_slice_k_offsets(8192, 1024, 128, 32, 1024, C.byref(po), C.byref(so)) == _lib.TWM_EINVAL


def test_host_mirror_rejects_cpu_tensors():
    """There is no CPU path: a host tensor is an error, not a fallback."""
    import torch
    from tensorwarp_b200 import quantize as q
    with pytest.raises(_lib.TwmError):
        q.quantize_f32_to_tw_marlin(torch.zeros(32, 8), 32, 8)
    with pytest.raises(_lib.TwmError):
        q.gemm_tw_marlin_m1(torch.zeros(32), torch.zeros(1, 8, 16, dtype=torch.uint8),
                            torch.zeros(1, 8, dtype=torch.float16), torch.zeros(8), 8, 32)
