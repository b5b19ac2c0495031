"""GPU parity tests of the GEMM chain (twm_chain_*): a list of dependent W4A16 GEMMs as one
persistent launch must give what the same GEMMs give one launch at a time, against the CPU
oracle, bit-identically from run to run, and replay after replay inside a CUDA graph."""
import numpy as np
import pytest
import torch

import oracle
from helpers import rel_err_floored, seeded_activations, seeded_weights
from tensorwarp_b200 import _lib
from tensorwarp_b200 import quantize as q

pytestmark = pytest.mark.gpu

DEV = "cuda"
TOL_F16 = 1e-2          # FP16 output, max relative error per element (floored denominator)
TOL_F32 = 5e-3          # FP32 output of the tensor-core kernels


def _dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).to(DEV)
    return t if dtype is None else t.to(dtype)


def _quantised(k, n, group, seed):
    w = seeded_weights(k, n, seed)
    packed, scales = oracle.quantize_pack(w, k, n, group)
    return packed, scales


def _f16_np(t):
    return t.float().cpu().numpy()


@pytest.mark.parametrize("group", [32, 128])
@pytest.mark.parametrize("m", [1, 2, 3, 8])
def test_dependent_chain_against_oracle(m, group):
    """Three GEMMs, each reading the output of the one before (the last adds into an FP32 buffer):
    every stage is checked against the FP64 oracle fed with the chain's own previous output."""
    dims = [1024, 544, 2048, 328]                       # K0 -> N0 = K1 -> N1 = K2 -> N2
    if group == 128:
        dims = [1024, 512, 2048, 328]
    mats = [_quantised(dims[i], dims[i + 1], group, 100 + i) for i in range(3)]
    a0 = seeded_activations(m, dims[0], 5)
    bufs = [_dev(a0, torch.float16)]
    bufs.append(torch.full((m, dims[1]), float("nan"), dtype=torch.float16, device=DEV))
    bufs.append(torch.full((m, dims[2]), float("nan"), dtype=torch.float16, device=DEV))
    out = torch.ones((m, dims[3]), dtype=torch.float32, device=DEV)
    dev_w = [(_dev(p), _dev(s.view(np.float16))) for p, s in mats]
    ch = q.GemmChain()
    ch.add(bufs[0], *dev_w[0], bufs[1], m, dims[1], dims[0], group_size=group)
    ch.add(bufs[1], *dev_w[1], bufs[2], m, dims[2], dims[1], group_size=group)
    ch.add(bufs[2], *dev_w[2], out, m, dims[3], dims[2], group_size=group, flags=_lib.TWM_FLAG_ACCUMULATE)
    ch.build()
    info = ch.info
    assert info.count == 3 and info.grid >= 148 and info.rows >= m
    ch.launch()
    torch.cuda.synchronize()
    assert q.device_error() == 0
    x = a0
    for i in range(2):
        got = _f16_np(bufs[i + 1])
        assert not np.isnan(got).any()
        ref = oracle.w4a16_f64(x, mats[i][0], mats[i][1], m, dims[i + 1], dims[i], group)
        assert rel_err_floored(got, ref) < TOL_F16, f"stage {i}"
        x = got                                           # the next stage reads what this one stored
    ref = oracle.w4a16_f64(x, mats[2][0], mats[2][1], m, dims[3], dims[2], group) + 1.0
    assert rel_err_floored(out.cpu().numpy(), ref) < TOL_F32
    first = [b.clone() for b in bufs[1:]] + [out.clone()]
    # again: same bits (the accumulating buffer is put back first), counters came back to zero
    out.fill_(1.0)
    ch.launch()
    torch.cuda.synchronize()
    assert q.device_error() == 0
    for b, f in zip(bufs[1:] + [out], first):
        assert torch.equal(b, f)
    ch.close()


def test_chain_matches_single_launches_on_7b_layer_shapes():
    """configs[1]: one layer's four GEMMs (M=1, G=128, FP16) with their own inputs and outputs.
    The chain and the one-launch-per-GEMM path sum K slices in different places, so they agree to
    FP16 rounding, not bit for bit; one shape is also checked against the oracle."""
    group = 128
    shapes = [(3584, 4608), (3584, 3584), (3584, 37888), (18944, 3584)]
    ws = q.Workspace.for_shapes([(1, n, k, group) for k, n in shapes], DEV)
    ch = q.GemmChain()
    keep = []
    for i, (k, n) in enumerate(shapes):
        w = torch.randn((k, n), generator=torch.Generator(device=DEV).manual_seed(2000 + i), device=DEV) * 0.02
        p, s = q.quantize_f32_to_tw_marlin(w, k, n, group)
        del w
        a = _dev(seeded_activations(1, k, i), torch.float16)
        c_chain = torch.full((1, n), float("nan"), dtype=torch.float16, device=DEV)
        c_single = torch.full((1, n), float("nan"), dtype=torch.float16, device=DEV)
        q.gemm_tw_marlin(a, p, s, c_single, 1, n, k, group_size=group, workspace=ws)
        ch.add(a, p, s, c_chain, 1, n, k, group_size=group)
        keep.append((a, p, s, c_chain, c_single))
    ch.build()
    for _ in range(3):
        ch.launch()
    torch.cuda.synchronize()
    assert q.device_error() == 0
    for (k, n), (a, p, s, c_chain, c_single) in zip(shapes, keep):
        got, ref = _f16_np(c_chain), _f16_np(c_single).astype(np.float64)
        assert not np.isnan(got).any()
        assert rel_err_floored(got, ref) < TOL_F16, (k, n)
    k, n = shapes[0]
    a, p, s, c_chain, _ = keep[0]
    ref64 = oracle.w4a16_f64(_f16_np(a), p.cpu().numpy(), s.cpu().numpy().view(np.uint16), 1, n, k, group)
    assert rel_err_floored(_f16_np(c_chain), ref64) < TOL_F16
    ch.close()


@pytest.mark.parametrize("m", [1, 4])
def test_silu_mul_prologue(m):
    """gate+up -> SwiGLU -> down in one chain: the down GEMM reads silu(gate) * up straight from the
    fused gate+up output, and gives the bits of twm_silu_mul followed by the same chain GEMM."""
    group, hidden, ffn = 128, 1024, 2816
    pgu, sgu = _quantised(hidden, 2 * ffn, group, 300)
    pdn, sdn = _quantised(ffn, hidden, group, 301)
    x = _dev(seeded_activations(m, hidden, 9), torch.float16)
    wgu = (_dev(pgu), _dev(sgu.view(np.float16)))
    wdn = (_dev(pdn), _dev(sdn.view(np.float16)))
    gate_up = torch.zeros((m, 2 * ffn), dtype=torch.float16, device=DEV)
    y_fused = torch.full((m, hidden), float("nan"), dtype=torch.float32, device=DEV)
    ch = q.GemmChain()
    ch.add(x, *wgu, gate_up, m, 2 * ffn, hidden, group_size=group)
    ch.add(gate_up, *wdn, y_fused, m, hidden, ffn, group_size=group, silu_mul=True)
    ch.build().launch()
    torch.cuda.synchronize()
    assert q.device_error() == 0
    # unfused: the separate SwiGLU kernel on the same gate_up, then a one-GEMM chain
    act = torch.zeros((m, ffn), dtype=torch.float16, device=DEV)
    _lib.check(_lib.lib().twm_silu_mul(act.data_ptr(), gate_up.data_ptr(), m, ffn, 0,
                                       torch.cuda.current_stream().cuda_stream), "twm_silu_mul")
    y_plain = torch.full((m, hidden), float("nan"), dtype=torch.float32, device=DEV)
    ch2 = q.GemmChain().add(act, *wdn, y_plain, m, hidden, ffn, group_size=group).build()
    ch2.launch()
    torch.cuda.synchronize()
    assert torch.equal(y_fused, y_plain)
    # SwiGLU outputs are small and of mixed magnitude: the tensor core's FP32 accumulator then loses
    # a little more against the FP64 oracle than with N(0,1) activations (1e-5 of the output RMS)
    ref = oracle.w4a16_f64(_f16_np(act), pdn, sdn, m, hidden, ffn, group)
    assert rel_err_floored(y_fused.cpu().numpy(), ref) < 4 * TOL_F32
    assert float(np.max(np.abs(y_fused.cpu().numpy() - ref))) < 1e-4 * float(np.sqrt(np.mean(ref ** 2)))
    ch.close(); ch2.close()


@pytest.mark.parametrize("k,n,group", [(96, 130, 32), (160, 33, 32), (4224, 129, 128), (2560, 1000, 128), (32, 1, 32)])
def test_ragged_shapes_in_a_chain(k, n, group):
    """N not a multiple of 128 or of 8 (scale rows copied by hand, zero-filled tile tails) and a K
    whose last work unit is short."""
    m = 2
    packed, scales = _quantised(k, n, group, 400)
    a = seeded_activations(m, k, 2)
    c = torch.full((m, n + 3), float("nan"), dtype=torch.float32, device=DEV)     # padded rows: ldc > N
    ch = q.GemmChain().add(_dev(a, torch.float16), _dev(packed), _dev(scales.view(np.float16)), c[:, :n], m, n, k,
                           group_size=group).build()
    ch.launch()
    torch.cuda.synchronize()
    assert q.device_error() == 0
    assert rel_err_floored(c[:, :n].cpu().numpy(), oracle.w4a16_f64(a, packed, scales, m, n, k, group)) < TOL_F32
    assert torch.isnan(c[:, n:]).all()                     # the padding is not touched
    ch.close()


def test_chain_in_a_cuda_graph_and_independent_flag():
    """Captured once, replayed: the completion counters are put back by the kernel itself.  GEMMs
    flagged independent do not wait; the dependent GEMM after them still sees all of them."""
    group, k, n = 128, 2048, 1536
    mats = [_quantised(k, n, group, 500 + i) for i in range(3)]
    pk, sk = _quantised(n, 640, group, 510)
    a = [_dev(seeded_activations(1, k, 20 + i), torch.float16) for i in range(3)]
    mid = [torch.zeros((1, n), dtype=torch.float16, device=DEV) for _ in range(3)]
    out = torch.zeros((1, 640), dtype=torch.float32, device=DEV)
    ch = q.GemmChain()
    dev_w = [(_dev(p), _dev(s.view(np.float16))) for p, s in mats]
    for i in range(3):
        ch.add(a[i], *dev_w[i], mid[i], 1, n, k, group_size=group, flags=_lib.TWM_FLAG_INDEPENDENT)
    ch.add(mid[2], _dev(pk), _dev(sk.view(np.float16)), out, 1, 640, n, group_size=group)
    ch.build()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ch.launch(stream)                                  # eager once
        torch.cuda.synchronize()
        eager = [t.clone() for t in mid] + [out.clone()]
        for t in mid + [out]:
            t.zero_()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            ch.launch(stream)
        for _ in range(5):
            graph.replay()
        torch.cuda.synchronize()
    assert q.device_error() == 0
    for got, ref in zip(mid + [out], eager):
        assert torch.equal(got, ref)
    for i in range(3):
        ref = oracle.w4a16_f64(_f16_np(a[i]), mats[i][0], mats[i][1], 1, n, k, group)
        assert rel_err_floored(_f16_np(mid[i]), ref) < TOL_F16
    ref = oracle.w4a16_f64(_f16_np(mid[2]), pk, sk, 1, 640, n, group)
    assert rel_err_floored(out.cpu().numpy(), ref) < TOL_F32
    ch.close()


def test_chain_rejects_what_it_cannot_run():
    p = torch.zeros((4, 128, 16), dtype=torch.uint8, device=DEV)
    s = torch.zeros((1, 128), dtype=torch.float16, device=DEV)
    a = torch.zeros((9, 128), dtype=torch.float16, device=DEV)
    c = torch.zeros((9, 128), dtype=torch.float16, device=DEV)
    with pytest.raises(_lib.TwmError) as e:
        q.GemmChain().add(a, p, s, c, 9, 128, 128, group_size=128).build()        # more than eight rows
    assert e.value.status == _lib.TWM_EINVAL
    with pytest.raises(_lib.TwmError):
        q.GemmChain().add(a.float(), p, s, c, 1, 128, 128, group_size=128)        # FP32 activations
