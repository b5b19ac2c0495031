"""GPU parity tests, through the C ABI: the sm_100a kernels against the CPU oracle and
against the reference's own CUDA kernels (compiled unchanged into oracle/_ref)."""
import numpy as np
import pytest
import torch

import oracle
from oracle import ref as oref
from helpers import raw_rel_violations, rel_err_floored, seeded_activations, seeded_weights
from tensorwarp_b200 import _lib
from tensorwarp_b200 import quantize as q

pytestmark = pytest.mark.gpu

DEV = "cuda"
# north-star tolerance: max relative error per output element, FP16 output
TOL_F16 = 1e-2
# f32 output of the FP32-FMA kernel: only summation order differs from the oracle
TOL_F32 = 1e-3
# f32 output of the tensor-core kernels: the tensor core's FP32 accumulator aligns addends with
# fewer guard bits than an IEEE fused multiply-add chain (about 1e-6 of the output RMS observed);
# still two orders below the FP16 rounding of the final store
TOL_TC_F32 = 5e-3
# Every kernel but the 256-column tcgen05 one multiplies exact weights f32(scale) * (nibble - 8) by the
# activations as they are (that one rounds the weights to FP16: see _tc_ref).
# Absolute bounds in units of the output RMS, on top of the relative test: FP16 output (its own
# rounding), and FP32 output of the tensor-core kernels (the accumulator's truncation adds up
# along K: 6.4e-6 seen at K = 3584 over 200 000 outputs).
TC_ABS_VS_EXACT = 2e-3
TC_ABS_F32 = 2e-5


def _tc_ref(a, packed, scales, m, n, k, group, kernel):
    """The adjudicating oracle for a kernel family: exact weights f32(scale) * (q - 8), except for the
    256-column tcgen05 kernel, whose weights enter the tensor core as f16_rn(scale * (q - 8)), the
    rounding of the reference's own batched route (dequant_q4_to_f16, quantize.rs:534-571)."""
    return oracle.w4a16_f64(a, packed, scales, m, n, k, group, weights_f16=(kernel == _lib.TWM_KERNEL_TCR))


def _abs_err_over_rms(y, ref64):
    rms = float(np.sqrt(np.mean(np.asarray(ref64, dtype=np.float64) ** 2))) + 1e-30
    return float(np.max(np.abs(np.asarray(y, dtype=np.float64) - ref64))) / rms


def _to_dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).to(DEV)
    return t if dtype is None else t.to(dtype)


def _quantised(k, n, group, seed):
    w = seeded_weights(k, n, seed)
    packed, scales = oracle.quantize_pack(w, k, n, group)
    return w, packed, scales


def _run_gemm(a_np, packed, scales, m, n, k, group, a_dtype, c_dtype, ws=None, **kw):
    a = _to_dev(a_np, a_dtype)
    c = torch.full((m, n), float("nan"), dtype=c_dtype, device=DEV)     # poison: every element must be written
    p = _to_dev(packed)
    s = _to_dev(scales.view(np.float16))
    if ws is None:
        ws = q.Workspace(max(q.workspace_bytes(m, n, k, group), 16) + 64 * min(m, 64) * n * 4 + 16384 + 512 + 128 * k)
    q.gemm_tw_marlin(a, p, s, c, m, n, k, group_size=group, workspace=ws, **kw)
    torch.cuda.synchronize()
    assert q.device_error() == 0
    # the kernels hand the tile counters back at zero
    assert int(ws.buf[:16384].view(torch.int32).abs().sum().item()) == 0
    return c.float().cpu().numpy()


# ---------------------------------------------------------------- layout --

@pytest.mark.parametrize("group", [32, 128])
@pytest.mark.parametrize("k,n", [(128, 1), (128, 33), (256, 257), (896, 9728), (3584, 512)])
def test_quantize_pack_bit_exact(k, n, group):
    w = seeded_weights(k, n, 11)
    w[: group, 0] = 0.0                        # an all-zero group
    p_ref, s_ref = oracle.quantize_pack(w, k, n, group)
    p, s = q.quantize_f32_to_tw_marlin(_to_dev(w), k, n, group)
    assert np.array_equal(p.cpu().numpy(), p_ref)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), s_ref)
    p2, s2 = q.cpu_quantize_tw_marlin(_to_dev(np.ascontiguousarray(w.T)), k, n, group)      # [N,K] input
    assert np.array_equal(p2.cpu().numpy(), p_ref)
    assert np.array_equal(s2.cpu().numpy().view(np.uint16), s_ref)


def test_oracle_quantiser_equals_reference_kernel():
    """The reference's warp_quantize_q4_0 (quantize.rs:103-146) on the columns of a matrix
    gives the same nibbles, and an f32 scale whose f16 rounding is the oracle's scale."""
    if not oref.available():
        pytest.skip("oracle/_ref not built")
    k, n = 512, 96
    w = seeded_weights(k, n, 13)
    cols = np.ascontiguousarray(w.T).reshape(-1)                     # column after column = [N,K]
    x = _to_dev(cols)
    out = torch.zeros(cols.size // 32 * 20, dtype=torch.uint8, device=DEV)
    oref.quantize_q4_0(out.data_ptr(), x.data_ptr(), cols.size)
    torch.cuda.synchronize()
    blocks = out.cpu().numpy().reshape(n, k // 32, 20)
    p_ref, s_ref = oracle.quantize_pack(w, k, n, 32)
    assert np.array_equal(blocks[:, :, 4:], np.transpose(p_ref, (1, 0, 2)))
    scale32 = blocks[:, :, :4].copy().view(np.float32).reshape(n, k // 32)
    assert np.array_equal(oracle.f32_to_f16_bits(scale32), s_ref.T)
    # and the reference's dequantise kernel on those blocks equals the oracle's f32-scale round trip
    back = torch.zeros(cols.size, dtype=torch.float32, device=DEV)
    oref.dequantize_q4_0(back.data_ptr(), out.data_ptr(), cols.size)
    torch.cuda.synchronize()
    assert np.array_equal(back.cpu().numpy(), oracle.q4_0_roundtrip(cols))


@pytest.mark.parametrize("group", [32, 128])
@pytest.mark.parametrize("k,n", [(128, 1), (256, 31), (384, 257), (3584, 640)])
def test_dequant_bit_exact(k, n, group):
    _, packed, scales = _quantised(k, n, group, 17)
    p, s = _to_dev(packed), _to_dev(scales.view(np.float16))
    d32 = q.dequant_tw_marlin(p, s, k, n, group, torch.float32).cpu().numpy()
    assert np.array_equal(d32.view(np.uint32), oracle.dequant_f32(packed, scales, k, n, group).view(np.uint32))
    d16 = q.dequant_tw_marlin(p, s, k, n, group, torch.float16).cpu().numpy()
    assert np.array_equal(d16.view(np.uint16), oracle.dequant_f16_bits(packed, scales, k, n, group))


def test_dequant_all_nibbles_and_odd_scales():
    """Every nibble value 0..15 against negative, subnormal and large scales: the decode is
    exact whatever produced the tensors."""
    k, n = 32, 16
    packed = np.zeros((1, n, 16), dtype=np.uint8)
    for col in range(n):
        packed[0, col, :] = [(col + i) % 16 | (((col + i + 5) % 16) << 4) for i in range(16)]
    scales = np.array([[0x3C00, 0xBC00, 0x0001, 0x03FF, 0x7BFF, 0x0000, 0x8000, 0x1234,
                        0x5555, 0x3555, 0x2E66, 0x4900, 0x0400, 0x8400, 0x6000, 0x3800]], dtype=np.uint16)
    p, s = _to_dev(packed), _to_dev(scales.view(np.float16))
    d32 = q.dequant_tw_marlin(p, s, k, n, 32, torch.float32).cpu().numpy()
    assert np.array_equal(d32.view(np.uint32), oracle.dequant_f32(packed, scales, k, n, 32).view(np.uint32))


@pytest.mark.parametrize("group", [32, 128])
def test_fuse_and_slice(group):
    k, ns = 256, [40, 8, 8]
    mats = [oracle.quantize_pack(seeded_weights(k, n_i, 30 + i), k, n_i, group) for i, n_i in enumerate(ns)]
    fp_ref, fs_ref = oracle.fuse_n(mats, k, group)
    dev = [(_to_dev(p), _to_dev(s.view(np.float16))) for p, s in mats]
    fp, fs = q.fuse_tw_marlin_n(dev, k, ns, group)
    assert np.array_equal(fp.cpu().numpy(), fp_ref)
    assert np.array_equal(fs.cpu().numpy().view(np.uint16), fs_ref)
    # slicing is the inverse of fusing
    off = 0
    for (p, s), n_i in zip(mats, ns):
        sp, ss = q.slice_tw_marlin_n(fp, fs, k, sum(ns), off, n_i, group)
        assert np.array_equal(sp.cpu().numpy(), p) and np.array_equal(ss.cpu().numpy().view(np.uint16), s)
        off += n_i
    # a K slice is a contiguous run of block rows
    kp, ks = q.slice_tw_marlin_k(fp, fs, k, sum(ns), 128, 128, group)
    assert np.array_equal(kp.cpu().numpy(), fp_ref[4:8])
    assert np.array_equal(ks.cpu().numpy().view(np.uint16), fs_ref[128 // group: 256 // group])


# ------------------------------------------------------------------ GEMM --

SMALL_SHAPES = [(32, 1), (32, 31), (128, 33), (160, 128), (256, 257), (512, 129), (1024, 1000), (2560, 136)]


@pytest.mark.parametrize("k,n", SMALL_SHAPES)
@pytest.mark.parametrize("splits", [0, 1, 2, 3, 7])
def test_m1_f32_reference_mode(k, n, splits):
    """f32 in / f32 out, G=32: the reference's own signature (quantize.rs:1301-1310)."""
    _, packed, scales = _quantised(k, n, 32, 41)
    a = seeded_activations(1, k, 0)
    y = _run_gemm(a, packed, scales, 1, n, k, 32, torch.float32, torch.float32, splits_override=splits)
    ref64 = oracle.w4a16_f64(a, packed, scales, 1, n, k, 32)
    assert rel_err_floored(y, ref64) < TOL_F32
    ko = oracle.m1_kernel_order(a[0], packed, scales, n, k, 32)
    assert np.max(np.abs(y[0] - ko)) <= 1e-5 * max(1.0, float(np.max(np.abs(ko))))


@pytest.mark.parametrize("kernel", [_lib.TWM_KERNEL_SIMT, _lib.TWM_KERNEL_TC, _lib.TWM_KERNEL_MMA])
@pytest.mark.parametrize("group", [32, 128])
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 13, 16])
@pytest.mark.parametrize("k,n", [(128, 33), (384, 257), (1024, 512), (3584, 264)])
def test_small_m_f16(m, k, n, group, kernel):
    """FP16 activations and output on every kernel family (FP32-FMA, warp-level MMA, tcgen05)."""
    if k % group:
        pytest.skip("K not a multiple of the group")
    _, packed, scales = _quantised(k, n, group, 43)
    a = seeded_activations(m, k, 0)
    y = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float16, kernel_override=kernel)
    ref64 = _tc_ref(a, packed, scales, m, n, k, group, kernel)
    assert rel_err_floored(y, ref64) < TOL_F16
    assert _abs_err_over_rms(y, oracle.w4a16_f64(a, packed, scales, m, n, k, group)) < TC_ABS_VS_EXACT
    # and bit-identical to rounding the f32-output run to f16 (one rounding, at the end)
    y32 = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float32, kernel_override=kernel)
    assert rel_err_floored(y32, ref64) < (TOL_F32 if kernel == _lib.TWM_KERNEL_SIMT else TOL_TC_F32)
    assert np.array_equal(y32.astype(np.float16).astype(np.float32), y)


@pytest.mark.parametrize("kernel", [_lib.TWM_KERNEL_TC, _lib.TWM_KERNEL_MMA])
@pytest.mark.parametrize("splits", [1, 2, 5])
@pytest.mark.parametrize("k,n,group", [(32, 40, 32), (96, 130, 32), (2048, 300, 128), (4224, 129, 128), (8192, 64, 32)])
def test_tc_kernel_slices(k, n, group, splits, kernel):
    """Tensor-core kernels: K slices that start and end inside a scale group (tcgen05 kernel),
    more blocks than TMEM slots, ring stages and staged activation chunks, ragged N."""
    m = 3
    _, packed, scales = _quantised(k, n, group, 45)
    a = seeded_activations(m, k, 1)
    y = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float32,
                  kernel_override=kernel, splits_override=splits)
    assert rel_err_floored(y, _tc_ref(a, packed, scales, m, n, k, group, kernel)) < TOL_TC_F32


@pytest.mark.parametrize("splits", [0, 1, 3])
@pytest.mark.parametrize("m", [33, 64, 128, 129, 200])
@pytest.mark.parametrize("k,n", [(512, 128), (2048, 300), (3584, 1000)])
def test_wide_tensor_core_kernel(m, k, n, splits):
    """The many-row tcgen05 kernel (rows on the MMA's M dimension): a partial last row block, ragged N,
    K slices through the workspace, more rows than one launch carries; FP32 and FP16 outputs."""
    group = 128
    kern = _lib.TWM_KERNEL_TCW
    _, packed, scales = _quantised(k, n, group, 49)
    a = seeded_activations(m, k, 2)
    ref = oracle.w4a16_f64(a, packed, scales, m, n, k, group)
    y32 = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float32, kernel_override=kern, splits_override=splits)
    assert rel_err_floored(y32, ref) < TOL_F16 and _abs_err_over_rms(y32, ref) < TC_ABS_F32
    y16 = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float16, kernel_override=kern, splits_override=splits,
                    flags=_lib.TWM_FLAG_PDL)
    assert np.array_equal(y32.astype(np.float16).astype(np.float32), y16)          # one rounding, at the end
    again = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float32, kernel_override=kern, splits_override=splits)
    assert np.array_equal(again, y32)                                              # fixed summation order
    # the heuristic's choice at these narrow shapes: this kernel for 65 ... 128 rows, the 256-column kernel beyond
    assert q.plan(m, n, k, group).kernel == (_lib.TWM_KERNEL_TCR if m > 128 else (kern if m >= 65 else _lib.TWM_KERNEL_TC))


@pytest.mark.parametrize("kind", ["silu", "geglu"])
@pytest.mark.parametrize("group", [32, 128])
@pytest.mark.parametrize("k,n,splits", [(2816, 1024, 0), (18944, 3584, 0), (512, 300, 1), (1024, 128, 3)])
def test_gated_activation_prologue(k, n, splits, group, kind):
    """twm_gemm_args.a_prologue: the GEMM reads act(gate) * up from the preceding GEMM's [gate | up] row.
    Bit for bit the result of the separate pass (fused_silu_mul, ops.rs:966-977; split_geglu,
    moe_batched_marlin.rs:138-152, restated in the oracle) followed by the plain GEMM."""
    _, packed, scales = _quantised(k, n, group, 57)
    gu = (seeded_activations(1, 2 * k, 6) * 1.5).astype(np.float16).astype(np.float32)
    if kind == "silu":
        g, u = gu[:, :k].astype(np.float32), gu[:, k:].astype(np.float32)
        act_dev = torch.zeros((1, k), dtype=torch.float16, device=DEV)
        _lib.check(_lib.lib().twm_silu_mul(act_dev.data_ptr(), _to_dev(gu, torch.float16).data_ptr(), 1, k, 0,
                                           torch.cuda.current_stream().cuda_stream), "twm_silu_mul")
        act = act_dev.float().cpu().numpy()
        ref_act = (g / (1.0 + np.exp(-g)) * u).astype(np.float16).astype(np.float32)
        assert np.max(np.abs(act - ref_act)) <= 2.0 ** -9 * max(1.0, float(np.abs(ref_act).max()))       # expf's last place
        prologue = _lib.TWM_A_SILU_MUL
    else:
        act = oracle.moe_split_geglu(gu.reshape(1, 2 * k), k).astype(np.float16).astype(np.float32)
        prologue = _lib.TWM_A_GEGLU
    plain = _run_gemm(act, packed, scales, 1, n, k, group, torch.float16, torch.float32, splits_override=splits)
    fused = _run_gemm(gu, packed, scales, 1, n, k, group, torch.float16, torch.float32, splits_override=splits,
                      a_prologue=prologue, flags=_lib.TWM_FLAG_PDL)
    if kind == "silu":
        assert np.array_equal(fused, plain)
    else:       # tanhf on the device against the oracle's: one f16 place of the activation at most
        ref = oracle.w4a16_f64(act, packed, scales, 1, n, k, group)
        assert _abs_err_over_rms(fused, ref) < 2e-3
    # the tensor core's truncating accumulator: the error grows with the number of scale groups added up
    ref = oracle.w4a16_f64(act, packed, scales, 1, n, k, group)
    assert _abs_err_over_rms(plain, ref) < TC_ABS_F32 * max(1.0, k / 3584)


@pytest.mark.parametrize("kind", ["silu", "geglu"])
@pytest.mark.parametrize("m", [2, 5, 16, 24, 32])
@pytest.mark.parametrize("k,n,group", [(512, 300, 32), (2816, 1024, 128)])
def test_gated_activation_prologue_on_several_rows(m, k, n, group, kind):
    """Two to 32 rows: the streaming kernel's staging pre-pass applies the prologue while it stages the rows.
    With one K slice the result is, bit for bit, that of the separate pass followed by the plain GEMM."""
    _, packed, scales = _quantised(k, n, group, 59)
    gu = (seeded_activations(m, 2 * k, 7) * 1.5).astype(np.float16).astype(np.float32)
    if kind == "silu":
        act_dev = torch.zeros((m, k), dtype=torch.float16, device=DEV)
        _lib.check(_lib.lib().twm_silu_mul(act_dev.data_ptr(), _to_dev(gu, torch.float16).data_ptr(), m, k, 0,
                                           torch.cuda.current_stream().cuda_stream), "twm_silu_mul")
        act = act_dev.float().cpu().numpy()
        prologue = _lib.TWM_A_SILU_MUL
    else:
        act = oracle.moe_split_geglu(gu, k).astype(np.float16).astype(np.float32)
        prologue = _lib.TWM_A_GEGLU
    ref = oracle.w4a16_f64(act, packed, scales, m, n, k, group)
    for splits in (1, 0):
        plain = _run_gemm(act, packed, scales, m, n, k, group, torch.float16, torch.float32, splits_override=splits)
        fused = _run_gemm(gu, packed, scales, m, n, k, group, torch.float16, torch.float32, splits_override=splits,
                          a_prologue=prologue, flags=_lib.TWM_FLAG_PDL)
        if kind == "silu" and splits == 1:
            assert np.array_equal(fused, plain)
        # (gated activations are far from N(0,1): a few large products per output, so twice the usual bound
        #  on the accumulator's truncation, still two orders below an FP16 step of the output)
        assert _abs_err_over_rms(fused, ref) < (2e-3 if kind == "geglu" else 2 * TC_ABS_F32)
        assert _abs_err_over_rms(plain, ref) < 2 * TC_ABS_F32


def test_next_gemm_hint_changes_nothing_but_timing():
    """twm_gemm_args.next: the producer warps ask for the head of the following GEMM's weights; the
    result is the same bits with and without it, whatever the successor looks like (another shape, a
    plan with K slices, a successor the library cannot plan: the hint is then dropped)."""
    k, n, group = 3584, 4608, 128
    _, packed, scales = _quantised(k, n, group, 61)
    _, p2, s2 = _quantised(18944, 3584, group, 62)
    a = seeded_activations(1, k, 8)
    plain = _run_gemm(a, packed, scales, 1, n, k, group, torch.float16, torch.float32, flags=_lib.TWM_FLAG_PDL)
    p2d, s2d = _to_dev(p2), _to_dev(s2.view(np.float16))
    pd, sd = _to_dev(packed), _to_dev(scales.view(np.float16))
    for nxt in ((p2d, s2d, 1, 3584, 18944, group), (pd, sd, 1, n, k, group), (p2d, s2d, 64, 3584, 18944, group),
                (p2d, s2d, 1, 3584, 18944 + 32, group)):          # the last one is not a valid shape (K % 128 != 0)
        hinted = _run_gemm(a, packed, scales, 1, n, k, group, torch.float16, torch.float32, flags=_lib.TWM_FLAG_PDL,
                           next_gemm=nxt)
        assert np.array_equal(hinted, plain)


def test_gated_activation_prologue_refusals():
    k, n = 256, 256
    _, packed, scales = _quantised(k, n, 32, 58)
    gu2 = seeded_activations(2, 2 * k)
    gu33 = seeded_activations(33, 2 * k)
    for kw in (dict(m=33, a=gu33, dt=torch.float16), dict(m=1, a=gu2[:1], dt=torch.float32),
               dict(m=2, a=gu2, dt=torch.float16, kernel_override=_lib.TWM_KERNEL_TC),
               dict(m=1, a=gu2[:1], dt=torch.float16, kernel_override=_lib.TWM_KERNEL_SIMT)):
        with pytest.raises(_lib.TwmError) as e:
            extra = {x: kw[x] for x in kw if x not in ("m", "a", "dt")}
            _run_gemm(kw["a"], packed, scales, kw["m"], n, k, 32, kw["dt"], torch.float32, a_prologue=_lib.TWM_A_SILU_MUL, **extra)
        assert e.value.status == _lib.TWM_EINVAL


@pytest.mark.parametrize("m", [65, 100, 128, 129, 256, 300])
@pytest.mark.parametrize("k,n", [(256, 256), (512, 300), (1024, 1000), (3584, 768)])
def test_256_column_tensor_core_kernel(m, k, n):
    """The 256-column tcgen05 kernel (TWM_KERNEL_TCR): weights rounded to FP16 as the reference's batched
    route rounds them, one accumulator over the whole K.  Against the FP16-weight oracle to accumulation
    error, against the exact-weight oracle to the weight rounding; ragged N (a last tile of one half, of
    a partial half), a partial last row block, more rows than one launch carries; FP32 and FP16 outputs."""
    group, kern = 128, _lib.TWM_KERNEL_TCR
    _, packed, scales = _quantised(k, n, group, 53)
    a = seeded_activations(m, k, 4)
    ref16 = oracle.w4a16_f64(a, packed, scales, m, n, k, group, weights_f16=True)
    y32 = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float32, kernel_override=kern)
    # one accumulator over the whole K: the tensor core's truncation adds up over K / 16 chained MMAs
    # (2.4e-5 of the output RMS seen at K = 3584) instead of over the eight of a scale group
    assert _abs_err_over_rms(y32, ref16) < 4 * TC_ABS_F32 * max(1.0, k / 3584) and rel_err_floored(y32, ref16) < TOL_F16
    assert _abs_err_over_rms(y32, oracle.w4a16_f64(a, packed, scales, m, n, k, group)) < TC_ABS_VS_EXACT
    y16 = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float16, kernel_override=kern, flags=_lib.TWM_FLAG_PDL)
    assert np.array_equal(y32.astype(np.float16).astype(np.float32), y16)          # one rounding of the sums, at the end
    again = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float32, kernel_override=kern)
    assert np.array_equal(again, y32)
    with pytest.raises(_lib.TwmError):                                             # it does not split K
        _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float32, kernel_override=kern, splits_override=2)


def test_wide_tensor_core_kernel_refuses_what_it_cannot_do():
    k, n = 256, 256
    _, packed, scales = _quantised(k, n, 32, 46)
    with pytest.raises(_lib.TwmError) as e:                                        # scale group 32
        _run_gemm(seeded_activations(80, k), packed, scales, 80, n, k, 32, torch.float16, torch.float16,
                  kernel_override=_lib.TWM_KERNEL_TCW)
    assert e.value.status == _lib.TWM_EINVAL
    assert q.plan(80, n, k, 32).kernel == _lib.TWM_KERNEL_TC                       # the heuristic keeps such shapes on the narrow kernel


def test_tc_kernel_rejects_f32_activations():
    k, n = 128, 128
    _, packed, scales = _quantised(k, n, 32, 46)
    with pytest.raises(_lib.TwmError) as e:
        _run_gemm(seeded_activations(1, k), packed, scales, 1, n, k, 32, torch.float32, torch.float32,
                  kernel_override=_lib.TWM_KERNEL_TC)
    assert e.value.status == _lib.TWM_EINVAL


@pytest.mark.parametrize("group", [32, 128])
@pytest.mark.parametrize("splits", [0, 1, 3])
@pytest.mark.parametrize("m", [9, 12, 16, 17, 24, 31, 32, 40, 67])
@pytest.mark.parametrize("k,n", [(256, 128), (512, 200), (2048, 1000), (3584, 136)])
def test_streaming_kernel_nine_to_32_rows(m, k, n, splits, group):
    """The warp-level-MMA kernel with its staging pre-pass (16- and 32-row launches, and what is left of
    more rows): ragged N, ragged last ring stage, K slices through the workspace, both outputs."""
    kern = _lib.TWM_KERNEL_MMA
    _, packed, scales = _quantised(k, n, group, 51)
    a = seeded_activations(m, k, 3)
    ref = oracle.w4a16_f64(a, packed, scales, m, n, k, group)
    y32 = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float32, kernel_override=kern, splits_override=splits)
    assert rel_err_floored(y32, ref) < TOL_TC_F32 and _abs_err_over_rms(y32, ref) < TC_ABS_F32
    y16 = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float16, kernel_override=kern, splits_override=splits,
                    flags=_lib.TWM_FLAG_PDL)
    assert np.array_equal(y32.astype(np.float16).astype(np.float32), y16)          # one rounding, at the end
    # every row is computed as in a launch of up to eight rows: same products, same summation order
    rows8 = np.concatenate([_run_gemm(a[m0:m0 + 8], packed, scales, min(8, m - m0), n, k, group, torch.float16, torch.float32,
                                      kernel_override=kern, splits_override=splits)
                            for m0 in range(0, m, 8)])
    if splits != 0:                                                                # (the automatic slice count depends on the rows)
        assert np.array_equal(rows8, y32)
    # the heuristic's choice up to 32 rows
    assert q.plan(min(m, 32), n, k, group).kernel == kern


@pytest.mark.parametrize("m,k,n,group", [(12, 96, 40, 32), (20, 256, 72, 128), (32, 160, 8, 32), (9, 128, 1, 128)])
def test_streaming_kernel_staged_rows_narrower_than_a_tile(m, k, n, group):
    """Fewer columns than one 128-column tile (no tensor map: row-by-row bulk copies, scale rows copied by
    the lanes when they are not 16-byte multiples), K shorter than a ring stage."""
    _, packed, scales = _quantised(k, n, group, 54)
    a = seeded_activations(m, k, 6)
    ref = oracle.w4a16_f64(a, packed, scales, m, n, k, group)
    for splits in (0, 1):
        y = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float32, kernel_override=_lib.TWM_KERNEL_MMA,
                      splits_override=splits)
        assert rel_err_floored(y, ref) < TOL_TC_F32 and _abs_err_over_rms(y, ref) < 2 * TC_ABS_F32


def test_streaming_kernel_staged_rows_on_a_large_matrix():
    """Three to eight rows on a matrix of 2^26 weights or more go through the pre-pass as well; without room
    for the staged rows in the workspace the CTAs' own stager warps do the same work: same bits."""
    k, n, group = 3584, 18944, 128
    _, packed, scales = _quantised(k, n, group, 52)
    for m in (3, 5, 8):
        a = seeded_activations(m, k, 4)
        assert q.plan(m, n, k, group).workspace_bytes >= m * k * 2
        staged = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float32, splits_override=1)
        small = q.Workspace(16384 + 64)                                             # counters only: no room for the rows
        own = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float32, ws=small, splits_override=1)
        assert np.array_equal(staged, own)
        ref = oracle.w4a16_f64(a, packed, scales, m, n, k, group)
        assert rel_err_floored(staged, ref) < TOL_TC_F32 and _abs_err_over_rms(staged, ref) < TC_ABS_F32
    # accumulate into C, and a second call gives the same bits
    a = seeded_activations(12, k, 5)
    base = _run_gemm(a, packed, scales, 12, n, k, group, torch.float16, torch.float32)
    c = torch.ones((12, n), dtype=torch.float32, device=DEV)
    ws = q.Workspace(q.workspace_bytes(12, n, k, group))
    q.gemm_tw_marlin(_to_dev(a, torch.float16), _to_dev(packed), _to_dev(scales.view(np.float16)), c, 12, n, k, group_size=group,
                     workspace=ws, flags=_lib.TWM_FLAG_ACCUMULATE)
    torch.cuda.synchronize()
    assert np.array_equal(c.cpu().numpy(), base + 1.0)
    assert np.array_equal(_run_gemm(a, packed, scales, 12, n, k, group, torch.float16, torch.float32), base)


def test_streaming_kernel_refuses_what_needs_its_own_stagers_beyond_eight_rows():
    k, n, group, m = 512, 256, 128, 12
    _, packed, scales = _quantised(k, n, group, 53)
    a = _to_dev(seeded_activations(m, k, 0), torch.float16)
    c = torch.empty((m, n), dtype=torch.float16, device=DEV)
    p, s = _to_dev(packed), _to_dev(scales.view(np.float16))
    with pytest.raises(_lib.TwmError):                                            # no workspace: nowhere to stage the rows
        q.gemm_tw_marlin(a, p, s, c, m, n, k, group_size=group, kernel_override=_lib.TWM_KERNEL_MMA)
    offs = torch.zeros(1, dtype=torch.int32, device=DEV)
    # per-expert offset tables: the kernel's own stager warps only, so not beyond eight rows
    args_ws = q.Workspace(q.workspace_bytes(m, n, k, group))
    with pytest.raises(_lib.TwmError):
        q.gemm_tw_marlin(a, p, s, c, m, n, k, group_size=group, workspace=args_ws, kernel_override=_lib.TWM_KERNEL_MMA,
                         packed_offsets=offs, scales_offsets=offs, expert_idx=0)


@pytest.mark.parametrize("group", [32, 128])
@pytest.mark.parametrize("m", [9, 16, 19, 32, 33, 64, 70, 130])
def test_m_beyond_eight(m, group):
    """The tcgen05 kernel's two accumulator widths (16, 32 rows) and more rows than one launch carries."""
    k, n = 512, 200
    _, packed, scales = _quantised(k, n, group, 47)
    a = seeded_activations(m, k, 0)
    y = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float16)
    # (130 rows at group 128 run on the 256-column kernel: adjudicated by the FP16-weight oracle)
    assert rel_err_floored(y, _tc_ref(a, packed, scales, m, n, k, group, q.plan(m, n, k, group).kernel)) < TOL_F16
    assert _abs_err_over_rms(y, oracle.w4a16_f64(a, packed, scales, m, n, k, group)) < TC_ABS_VS_EXACT
    # FP32 rows from the FP32-FMA kernel agree too (m > 8 there is served by several launches)
    y32 = _run_gemm(a, packed, scales, m, n, k, group, torch.float32, torch.float32)
    assert rel_err_floored(y32, oracle.w4a16_f64(a, packed, scales, m, n, k, group)) < TOL_F32


@pytest.mark.parametrize("m", [16, 32, 64, 128, 256])
def test_config2_shapes_beyond_eight_rows(m):
    """configs[2] at M = 16 ... 256 on the 7B gate+up shape (K=3584, N=37888), the full launch; a
    384-column slice of it against the oracle, every element for "written" and for linearity."""
    k, n, group = 3584, 37888, 128
    w = torch.randn((k, n), generator=torch.Generator(device=DEV).manual_seed(77), device=DEV) * 0.02
    p, s = q.quantize_f32_to_tw_marlin(w, k, n, group)
    del w
    a = seeded_activations(m, k, 0)
    c = torch.full((m, n), float("nan"), dtype=torch.float16, device=DEV)
    ws = q.Workspace(q.workspace_bytes(m, n, k, group))
    q.gemm_tw_marlin(_to_dev(a, torch.float16), p, s, c, m, n, k, group_size=group, flags=_lib.TWM_FLAG_PDL, workspace=ws)
    torch.cuda.synchronize()
    assert q.device_error() == 0
    # a column slice against the oracle (the whole matrix would take minutes on the CPU)
    cols = slice(12800, 12800 + 384)
    packed = p.cpu().numpy()[:, cols].copy()
    scales = s.cpu().numpy().view(np.uint16)[:, cols].copy()
    chosen = q.plan(m, n, k, group).kernel
    assert chosen == (_lib.TWM_KERNEL_TCR if m >= 65 else (_lib.TWM_KERNEL_TC if m >= 33 else _lib.TWM_KERNEL_MMA))
    ref = _tc_ref(a, packed, scales, m, 384, k, group, chosen)
    assert rel_err_floored(c[:, cols].float().cpu().numpy(), ref) < TOL_F16
    # whichever weights the kernel multiplies, the result is within 2e-3 of the output RMS of the exact-weight product
    assert _abs_err_over_rms(c[:, cols].float().cpu().numpy(), oracle.w4a16_f64(a, packed, scales, m, 384, k, group)) < TC_ABS_VS_EXACT
    # and size-independent properties on the whole output: every element written, linear in the activations
    assert not torch.isnan(c).any()
    c2 = torch.empty_like(c)
    q.gemm_tw_marlin(_to_dev(2.0 * a, torch.float16), p, s, c2, m, n, k, group_size=group, workspace=ws)
    torch.cuda.synchronize()
    # (doubling an activation doubles its products exactly unless an intermediate FP16 value leaves the
    #  normal range, so this is "within one FP16 step", and equal almost everywhere)
    normal = (c.abs() < 30000) & (c.abs() > 1e-3)
    step = (2 * c[normal]).abs().float() * 2.0 ** -10
    assert torch.all((c2[normal].float() - 2 * c[normal].float()).abs() <= step)
    assert (c2[normal] != 2 * c[normal]).float().mean() < 1e-3


@pytest.mark.parametrize("m", [16, 64, 200])
def test_tensor_core_kernel_with_tiny_activation_rows(m):
    """Rows whose activations are tiny (1e-4 ... 1e-3, FP16 subnormals among them) beside ordinary
    rows: the tensor-core kernels multiply the activations as they are by exact nibble operands, so
    such rows are as accurate, relative to their own RMS, as any other row."""
    k, n, group = 2048, 512, 128
    _, packed, scales = _quantised(k, n, group, 91)
    a = seeded_activations(m, k, 3)
    a[1] *= 1e-4
    a[m - 1] *= 1e-3
    a = a.astype(np.float16).astype(np.float32)
    y = _run_gemm(a, packed, scales, m, n, k, group, torch.float16, torch.float32)
    ref = oracle.w4a16_f64(a, packed, scales, m, n, k, group)
    # (200 rows run on the 256-column kernel, whose weights are rounded to FP16: the same relative bound
    #  for every row, tiny or not, only a larger one)
    bound = 2e-3 if q.plan(m, n, k, group).kernel == _lib.TWM_KERNEL_TCR else 1e-4
    for row in (0, 1, m - 1):
        rms = float(np.sqrt(np.mean(ref[row] ** 2)))
        assert float(np.max(np.abs(y[row] - ref[row]))) < bound * rms, row


def test_config0_shape_vs_literal_cpu_path():
    """configs[0]: M=1, K=896, N=9728, G=128, FP16 in/out, against the reference's CPU route
    restated literally (dequantise the matrix, naive matmul, FP32 accumulate)."""
    k, n, group = 896, 9728, 128
    _, packed, scales = _quantised(k, n, group, 0)
    a = seeded_activations(1, k, 0)
    y = _run_gemm(a, packed, scales, 1, n, k, group, torch.float16, torch.float16)
    lit = oracle.w4a16_literal(a, packed, scales, 1, n, k, group)
    ref64 = oracle.w4a16_f64(a, packed, scales, 1, n, k, group)
    assert rel_err_floored(y, ref64) < TOL_F16
    assert rel_err_floored(lit, ref64) < TOL_F16
    bad, worst = raw_rel_violations(y, ref64, TOL_F16)
    rms = float(np.sqrt(np.mean(ref64 ** 2)))
    # raw (unfloored) criterion: any violator must be a near-zero output
    assert bad == 0 or worst < rms * 2.0 ** -5, (bad, worst, rms)


@pytest.mark.parametrize("k,n", [(3584, 4608), (3584, 3584), (3584, 37888), (18944, 3584)])
def test_config1_shapes(k, n):
    """configs[1]: the four Qwen2-7B decode GEMMs at full size, M=1, G=128, FP16."""
    group = 128
    w = torch.randn((k, n), generator=torch.Generator(device=DEV).manual_seed(1000 + n % 7), device=DEV) * 0.02
    p, s = q.quantize_f32_to_tw_marlin(w, k, n, group)
    torch.cuda.synchronize()
    packed, scales = p.cpu().numpy(), s.cpu().numpy().view(np.uint16)
    a = seeded_activations(1, k, 0)
    y = _run_gemm(a, packed, scales, 1, n, k, group, torch.float16, torch.float16, flags=_lib.TWM_FLAG_PDL)
    ref64 = oracle.w4a16_f64(a, packed, scales, 1, n, k, group)
    assert rel_err_floored(y, ref64) < TOL_F16
    # size-independent property: linearity in the activations, C(2a) = 2 C(a) exactly (power of two)
    y2 = _run_gemm(2.0 * a, packed, scales, 1, n, k, group, torch.float16, torch.float16)
    normal = (np.abs(y) < 30000) & (np.abs(y) > 1e-3)      # away from f16 overflow and subnormals
    assert np.array_equal(y2[normal], 2.0 * y[normal])


def test_against_reference_cuda_kernel():
    """The reference's warp_gemm_tw_marlin_m1(_direct) run on this GPU: the oracle's
    kernel-order restatement reproduces the direct kernel bit for bit, the split-K kernel
    (FP32 atomics, any order) within summation error, and the sm_100a kernel agrees with both."""
    if not oref.available():
        pytest.skip("oracle/_ref not built")
    for (k, n, group) in [(896, 9728, 32), (3584, 4608, 128), (3584, 3584, 32), (2048, 300, 32)]:
        _, packed, scales = _quantised(k, n, group, 51)
        a = seeded_activations(1, k, 0)
        s32 = scales if group == 32 else np.repeat(scales, 4, axis=0)      # G=128 shown to a G=32 kernel
        ad, pd, sd = _to_dev(a), _to_dev(packed), _to_dev(np.ascontiguousarray(s32).view(np.float16))
        c_direct = torch.zeros(n, dtype=torch.float32, device=DEV)
        assert oref.gemm_tw_marlin_m1(c_direct.data_ptr(), ad.data_ptr(), pd.data_ptr(), sd.data_ptr(), n, k,
                                      force_splits=1) == 1
        c_auto = torch.zeros(n, dtype=torch.float32, device=DEV)
        used = oref.gemm_tw_marlin_m1(c_auto.data_ptr(), ad.data_ptr(), pd.data_ptr(), sd.data_ptr(), n, k)
        torch.cuda.synchronize()
        assert used == oracle.splitk_plan_ref(n, k)[1]
        ko = oracle.m1_kernel_order(a[0], packed, np.ascontiguousarray(s32), n, k, 32)
        assert np.array_equal(c_direct.cpu().numpy().view(np.uint32), ko.view(np.uint32))
        ref64 = oracle.w4a16_f64(a, packed, scales, 1, n, k, group)
        assert rel_err_floored(c_auto.cpu().numpy()[None], ref64) < TOL_F32
        y = _run_gemm(a, packed, scales, 1, n, k, group, torch.float32, torch.float32)
        assert rel_err_floored(y, c_direct.cpu().numpy()[None].astype(np.float64)) < TOL_F32
        y16 = _run_gemm(a, packed, scales, 1, n, k, group, torch.float16, torch.float16)
        assert rel_err_floored(y16, c_direct.cpu().numpy()[None].astype(np.float64)) < TOL_F16


def test_deterministic_and_split_invariant():
    """Two runs are bit-identical (the reference's split-K is not: FP32 atomics), and the
    result does not depend on which slice arrives last."""
    k, n, group = 3584, 4608, 128
    _, packed, scales = _quantised(k, n, group, 53)
    a = seeded_activations(1, k, 0)
    for kernel in (_lib.TWM_KERNEL_SIMT, _lib.TWM_KERNEL_TC, _lib.TWM_KERNEL_MMA, _lib.TWM_KERNEL_TCW, _lib.TWM_KERNEL_TCR):
        runs = [_run_gemm(a, packed, scales, 1, n, k, group, torch.float16, torch.float32, kernel_override=kernel)
                for _ in range(3)]
        assert np.array_equal(runs[0], runs[1]) and np.array_equal(runs[0], runs[2])


def test_indirect_and_from_buffer():
    """Expert-indexed weights (quantize_indirect.rs:185-253) and host offsets (quantize.rs:1731-1782)."""
    k, n, group, experts = 256, 136, 32, 3
    mats = [_quantised(k, n, group, 60 + e)[1:] for e in range(experts)]
    pbuf = np.concatenate([p.reshape(-1) for p, _ in mats])
    sbuf = np.concatenate([s.reshape(-1) for _, s in mats])
    poff = np.array([e * (k // 32) * n * 16 for e in range(experts)], dtype=np.uint32)
    soff = np.array([e * (k // group) * n for e in range(experts)], dtype=np.uint32)
    a = seeded_activations(1, k, 0)
    ad, pd, sd = _to_dev(a, torch.float32), _to_dev(pbuf), _to_dev(sbuf.view(np.float16))
    po, so = _to_dev(poff.view(np.int32)), _to_dev(soff.view(np.int32))
    for e in range(experts):
        ref64 = oracle.w4a16_f64(a, mats[e][0], mats[e][1], 1, n, k, group)
        c = torch.full((n,), float("nan"), dtype=torch.float32, device=DEV)
        q.gemm_tw_marlin_m1_indirect(ad, pd, po, sd, so, e, c, n, k, flags=_lib.TWM_FLAG_PDL)
        c2 = torch.full((n,), float("nan"), dtype=torch.float32, device=DEV)
        q.gemm_tw_marlin_m1_from_buffer(ad, pd, int(poff[e]), sd, int(soff[e]), c2, n, k)
        torch.cuda.synchronize()
        assert rel_err_floored(c.cpu().numpy()[None], ref64) < TOL_F32
        assert np.array_equal(c.cpu().numpy(), c2.cpu().numpy())


def test_accumulate_flag_and_strides():
    k, n, m, group = 256, 200, 2, 32
    _, packed, scales = _quantised(k, n, group, 70)
    a = seeded_activations(m, k, 0)
    a_wide = torch.zeros((m, k + 64), dtype=torch.float16, device=DEV)
    a_wide[:, :k] = _to_dev(a, torch.float16)
    c_wide = torch.ones((m, n + 8), dtype=torch.float32, device=DEV)
    q.gemm_tw_marlin(a_wide[:, :k], _to_dev(packed), _to_dev(scales.view(np.float16)), c_wide[:, :n], m, n, k,
                     group_size=group, flags=_lib.TWM_FLAG_ACCUMULATE)
    torch.cuda.synchronize()
    ref64 = oracle.w4a16_f64(a, packed, scales, m, n, k, group) + 1.0
    assert rel_err_floored(c_wide[:, :n].cpu().numpy(), ref64) < TOL_F32
    assert torch.all(c_wide[:, n:] == 1.0)        # the padding columns are not touched


def test_errors_are_statuses():
    k, n = 3584, 3584
    a = torch.zeros(k, dtype=torch.float32, device=DEV)
    p = torch.zeros((k // 32, n, 16), dtype=torch.uint8, device=DEV)
    s = torch.zeros((k // 128, n), dtype=torch.float16, device=DEV)
    c = torch.zeros(n, dtype=torch.float32, device=DEV)
    # the reference's own call has no scratch argument: without a workspace the FP32 kernel runs unsplit
    c.fill_(1.0)
    q.gemm_tw_marlin_m1(a, p, s, c, n, k, group_size=128, workspace=None)
    torch.cuda.synchronize()
    assert torch.all(c == 0)
    # a split count the caller asks for needs its scratch
    with pytest.raises(_lib.TwmError) as e:
        q.gemm_tw_marlin_m1(a, p, s, c, n, k, group_size=128, workspace=None, splits_override=4)
    assert e.value.status == _lib.TWM_EWORKSPACE
    with pytest.raises(_lib.TwmError) as e:
        q.gemm_tw_marlin_m1(a, p, s, c, n, k - 16, group_size=128)
    assert e.value.status == _lib.TWM_EINVAL
    # FP16 activations, one row: the slices add up inside a cluster, no workspace needed
    a16 = torch.zeros(k, dtype=torch.float16, device=DEV)
    c16 = torch.ones(n, dtype=torch.float16, device=DEV)
    q.gemm_tw_marlin_m1(a16, p, s, c16, n, k, group_size=128, workspace=None)
    torch.cuda.synchronize()
    assert torch.all(c16 == 0)


def test_independent_launch_flag_same_bits():
    """TWM_FLAG_INDEPENDENT (no wait for the preceding launch): four GEMMs with their own inputs
    and outputs, launched back to back, give the bits of the ordinary launches."""
    shapes = [(3584, 4608), (3584, 3584), (1024, 9728), (2048, 1024)]
    group = 128
    ws = q.Workspace(1 << 24)
    mats, outs = [], {}
    for i, (k, n) in enumerate(shapes):
        _, packed, scales = _quantised(k, n, group, 80 + i)
        mats.append((_to_dev(packed), _to_dev(scales.view(np.float16)), _to_dev(seeded_activations(1, k, i), torch.float16)))
    for flags in (0, _lib.TWM_FLAG_PDL, _lib.TWM_FLAG_PDL | _lib.TWM_FLAG_INDEPENDENT):
        cs = [torch.full((1, n), float("nan"), dtype=torch.float16, device=DEV) for _, n in shapes]
        for rep in range(3):
            for (k, n), (p, s, a), c in zip(shapes, mats, cs):
                q.gemm_tw_marlin(a, p, s, c, 1, n, k, group_size=group, workspace=ws, flags=flags)
        torch.cuda.synchronize()
        outs[flags] = [c.clone() for c in cs]
    for flags in outs:
        for c, ref in zip(outs[flags], outs[0]):
            assert torch.equal(c, ref)
    assert q.device_error() == 0


@pytest.mark.parametrize("k,n", [(8192, 1280), (1024, 8192), (8192, 7168), (3584, 8192), (8192, 2560), (2048, 8192)])
def test_tensor_parallel_shard_shapes(k, n):
    """The per-rank GEMM shapes of the 70B-shaped stack at tp = 8 and tp = 4 (M = 1, G = 128): the plan
    reaches its largest cluster (16 K slices) on the tp = 8 QKV shard."""
    group = 128
    _, packed, scales = _quantised(k, n, group, 90 + (k + n) % 7)
    a = seeded_activations(1, k, 4)
    y = _run_gemm(a, packed, scales, 1, n, k, group, torch.float16, torch.float32, flags=_lib.TWM_FLAG_PDL)
    assert rel_err_floored(y, oracle.w4a16_f64(a, packed, scales, 1, n, k, group)) < TOL_TC_F32
    if (k, n) == (8192, 1280):
        p = q.plan(1, n, k, group)
        assert p.splits == 16 and p.cluster_reduce == 1
