"""GPU test of twm_gemm_w4a16_static_ws, the GEMM entry point for hosts that cannot hand this
library a workspace (all device memory is spoken for at start-up, or allocation calls are off
limits while serving).  It must give what twm_gemm_w4a16 gives with a caller-owned workspace,
call after call on the shared built-in scratch array.  Named so that pytest collects it last."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import rel_err_floored, seeded_activations, seeded_weights
from tensorwarp_b200 import _lib
from tensorwarp_b200 import quantize as q

pytestmark = pytest.mark.gpu

TOL_F16 = 1e-2          # the tolerance of the other FP16-output GEMM tests


def _args(a, p, s, c, m, n, k, group, ws=None, splits=0):
    return _lib.GemmArgs(M=m, N=n, K=k, group_size=group, a_dtype=_lib.TWM_F16, c_dtype=_lib.TWM_F16,
                         a=a.data_ptr(), lda=k, packed=p.data_ptr(), scales=s.data_ptr(), c=c.data_ptr(), ldc=n,
                         workspace=ws.ptr if ws is not None else None,
                         workspace_bytes=ws.nbytes if ws is not None else 0, splits_override=splits)


@pytest.mark.parametrize("m,k,n,splits", [(3, 3584, 4608, 0), (4, 2048, 1000, 0), (8, 3584, 1024, 0), (16, 2048, 640, 0),
                                            (3, 2048, 1000, 5)])
def test_static_scratch_matches_caller_workspace(m, k, n, splits):
    """Rows 3-4: the streaming kernel's split-K partials live in the array; rows 8 and 16: the tensor-core
    kernel's pre-pass output and partials; the last case: a split count the caller asked for."""
    lib = _lib.lib()
    group = 128
    w = seeded_weights(k, n, 91)
    packed, scales = oracle.quantize_pack(w, k, n, group)
    a_np = seeded_activations(m, k, 3)
    a = torch.from_numpy(a_np).cuda().half()
    p = torch.from_numpy(packed).cuda()
    s = torch.from_numpy(scales.view(np.float16)).cuda()
    assert q.plan(m, n, k, group, splits_override=splits).workspace_bytes > 0, "the case must exercise the scratch"
    stream = torch.cuda.current_stream().cuda_stream

    # the existing entry point, with a workspace the caller allocated
    ws = q.Workspace(max(q.workspace_bytes(m, n, k, group), q.plan(m, n, k, group, splits_override=splits).workspace_bytes))
    c_ref = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    _lib.check(lib.twm_gemm_w4a16(C.byref(_args(a, p, s, c_ref, m, n, k, group, ws, splits)), stream), "twm_gemm_w4a16")
    torch.cuda.synchronize()
    ref = c_ref.float().cpu().numpy()
    assert rel_err_floored(ref, oracle.w4a16_f64(a_np, packed, scales, m, n, k, group)) < TOL_F16

    # the new entry point, twice in a row on the shared array, no workspace passed
    for call in range(2):
        c_new = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        _lib.check(lib.twm_gemm_w4a16_static_ws(C.byref(_args(a, p, s, c_new, m, n, k, group, None, splits)), stream),
                   "twm_gemm_w4a16_static_ws")
        torch.cuda.synchronize()
        got = c_new.float().cpu().numpy()
        assert not np.isnan(got).any(), f"call {call}: some outputs were never written"
        assert rel_err_floored(got, ref.astype(np.float64)) < TOL_F16, f"call {call}"
    assert q.device_error() == 0


def test_static_scratch_rejects_oversized_plans():
    """A plan that needs more scratch than the array holds is refused before anything is enqueued."""
    lib = _lib.lib()
    cap = lib.twm_static_ws_capacity()
    m, k, n, group = 8, 8192, 65536, 128
    need = q.plan(m, n, k, group, splits_override=8, kernel_override=_lib.TWM_KERNEL_MMA).workspace_bytes
    assert need > cap
    dummy = torch.zeros(64, dtype=torch.uint8, device="cuda")          # never dereferenced: the call fails first
    args = _lib.GemmArgs(M=m, N=n, K=k, group_size=group, a_dtype=_lib.TWM_F16, c_dtype=_lib.TWM_F16,
                         a=dummy.data_ptr(), lda=k, packed=dummy.data_ptr(), scales=dummy.data_ptr(),
                         c=dummy.data_ptr(), ldc=n, splits_override=8)
    st = lib.twm_gemm_w4a16_static_ws(C.byref(args), torch.cuda.current_stream().cuda_stream)
    assert st == _lib.TWM_EWORKSPACE
    msg = lib.twm_last_error().decode()
    # (the size named is that of the plan the call would run: up to eight rows fall back from the staging
    #  pre-pass to the kernel's own stager warps before giving up, which needs the split-K part only)
    named = int(msg.split("needs ")[1].split(" bytes")[0])
    assert str(cap) in msg and cap < named <= need
