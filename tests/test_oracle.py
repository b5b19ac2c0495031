"""CPU tests of the oracle: known answers, the reference tests' closed-form
inputs, internal consistency.  No GPU."""
import numpy as np
import pytest

import oracle
from helpers import seeded_activations, seeded_weights


def test_f16_conversion_matches_ieee():
    h = np.arange(65536, dtype=np.uint16)
    ref = h.view(np.float16).astype(np.float32)
    ok = ~np.isnan(ref)
    assert np.array_equal(oracle.f16_bits_to_f32(h)[ok].view(np.uint32), ref[ok].view(np.uint32))
    rng = np.random.default_rng(1)
    with np.errstate(over="ignore"):
        for s in (1e-8, 1e-5, 1e-3, 1.0, 100.0, 1e5):
            x = rng.standard_normal(200_000).astype(np.float32) * np.float32(s)
            assert np.array_equal(oracle.f32_to_f16_bits(x), x.astype(np.float16).view(np.uint16))
        # every f32 that sits exactly half way between two f16 (ties to even)
        bits = (np.arange(0, 1 << 19, dtype=np.uint32) << 13) | np.uint32(0x1000)
        x = bits.view(np.float32)
        ok = ~np.isnan(x)
        assert np.array_equal(oracle.f32_to_f16_bits(x)[ok], x.astype(np.float16).view(np.uint16)[ok])


@pytest.mark.parametrize("group", [32, 128])
def test_quantise_known_answers(group):
    k, n = group, 4
    w = np.zeros((k, n), dtype=np.float32)
    w[:, 1] = 0.7                      # every value = +amax  -> nibble 15
    w[:, 2] = -0.7                     # every value = -amax  -> nibble 1
    w[0, 3], w[1, 3], w[2, 3] = 7.0, 0.5, -0.5   # scale 1: +-0.5 are ties, round away from zero
    packed, scales = oracle.quantize_pack(w, k, n, group)
    assert packed.shape == (k // 32, n, 16) and scales.shape == (1, n)
    assert np.all(packed[:, 0, :] == 0x88) and scales[0, 0] == 0            # all-zero group: scale 0, nibble 8
    assert np.all(packed[:, 1, :] == 0xFF)
    assert np.all(packed[:, 2, :] == 0x11)
    assert scales[0, 1] == oracle.f32_to_f16_bits(np.float32(0.7) / np.float32(7.0))
    assert packed[0, 3, 0] == (15 | (9 << 4))       # k=0 -> 7+8=15 low nibble, k=1 -> round(0.5)=1 -> 9 high
    assert packed[0, 3, 1] == (7 | (8 << 4))        # k=2 -> round(-0.5)=-1 -> 7 ; k=3 -> 0 -> 8
    assert scales[0, 3] == 0x3C00                    # 1.0
    d = oracle.dequant_f32(packed, scales, k, n, group)
    assert d[0, 3] == 7.0 and d[1, 3] == 1.0 and d[2, 3] == -1.0 and np.all(d[:, 0] == 0)


def test_nibble_order_matches_kernel_word_view():
    """Byte i low/high nibble == bits 4*(j%8) of little-endian u32 j/8 (quantize.rs:1207-1217)."""
    k, n = 32, 1
    w = (np.arange(32, dtype=np.float32) % 15 - 7).reshape(k, n)   # amax 7 -> scale 1 -> q = v + 8
    packed, _ = oracle.quantize_pack(w, k, n, 32)
    words = packed.reshape(-1).view("<u4")
    for j in range(32):
        assert ((int(words[j // 8]) >> (4 * (j % 8))) & 0xF) - 8 == int(w[j, 0])


def test_layout_nk_equals_kn():
    k, n = 256, 24
    w = seeded_weights(k, n, 3)
    for g in (32, 128):
        p1, s1 = oracle.quantize_pack(w, k, n, g)
        p2, s2 = oracle.quantize_pack(np.ascontiguousarray(w.T), k, n, g, w_is_nk=True)
        assert np.array_equal(p1, p2) and np.array_equal(s1, s2)


def test_reference_roundtrip_closed_form():
    """Input of q4_0_roundtrip_correctness (quantize.rs:3009): quantise+pack+dequantise with the
    f32 scale equals the reference's cpu_q4_0_roundtrip; with the stored f16 scale it differs
    only by the f16 rounding of the scale."""
    n = 1024
    x = np.array([((i * 7 + 3) % 200) * 0.01 - 1.0 for i in range(n)], dtype=np.float32)
    rt = oracle.q4_0_roundtrip(x)
    assert np.max(np.abs(rt - x)) <= np.max(np.abs(x)) / 7.0 / 2 + 1e-6      # half a step
    # the same data as one column of K=1024: nibbles must reproduce rt / scale
    packed, scales = oracle.quantize_pack(x.reshape(n, 1), n, 1, 32)
    d = oracle.dequant_f32(packed, scales, n, 1, 32).reshape(-1)
    s16 = oracle.f16_bits_to_f32(scales).reshape(-1)
    for b in range(n // 32):
        amax = np.max(np.abs(x[b * 32:(b + 1) * 32]))
        s32 = np.float32(amax) / np.float32(7.0)
        q_from_rt = np.round(rt[b * 32:(b + 1) * 32] / s32)
        q_from_d = np.round(d[b * 32:(b + 1) * 32] / s16[b])
        assert np.array_equal(q_from_rt, q_from_d)
        assert abs(s16[b] - s32) <= s32 * 2.0 ** -11


def test_reference_dequant_f16_closed_form():
    """Input of dequant_q4_to_f16_correctness (quantize.rs:3618-3620), K=128, N=64:
    f16 dequant within 0.01 of scale*q, as that test asserts."""
    k, n = 128, 64
    w = np.array([((i * 17 + 3) % 101) * 0.02 - 1.0 for i in range(k * n)], dtype=np.float32).reshape(k, n)
    packed, scales = oracle.quantize_pack(w, k, n, 32)
    d32 = oracle.dequant_f32(packed, scales, k, n, 32)
    d16 = oracle.f16_bits_to_f32(oracle.dequant_f16_bits(packed, scales, k, n, 32))
    assert np.max(np.abs(d16 - d32)) < 0.01
    assert np.max(np.abs(d32 - w)) <= 1.0 / 7.0 / 2 + 2e-3


@pytest.mark.parametrize("group", [32, 128])
def test_gemm_variants_agree(group):
    m, k, n = 3, 512, 40
    w = seeded_weights(k, n, 5)
    a = seeded_activations(m, k, 0)
    packed, scales = oracle.quantize_pack(w, k, n, group)
    lit = oracle.w4a16_literal(a, packed, scales, m, n, k, group)
    thr, used = oracle.w4a16_threaded(a, packed, scales, m, n, k, group)
    assert used >= 1 and np.array_equal(lit, thr)            # same arithmetic, bit for bit
    dense = oracle.dequant_f32(packed, scales, k, n, group)
    assert np.array_equal(lit, oracle.gemm_f32(a, dense, m, n, k))
    f64 = oracle.w4a16_f64(a, packed, scales, m, n, k, group)
    assert np.allclose(lit, f64, rtol=0, atol=1e-4)
    ko = oracle.m1_kernel_order(a[0], packed, scales, n, k, group)
    assert np.allclose(ko, f64[0], rtol=0, atol=1e-4)
    # split ranges of the kernel-order restatement add up to the whole
    parts = sum(oracle.m1_kernel_order(a[0], packed, scales, n, k, group, g0, g0 + 4).astype(np.float64)
                for g0 in range(0, k // 32, 4))
    assert np.allclose(parts, f64[0], rtol=0, atol=1e-4)


def test_group128_equals_repeated_scales():
    """A G=128 tensor fed to G=32 code with every scale row repeated four times gives the same
    weights: how G=128 inputs are shown to the reference's own kernel."""
    k, n = 256, 16
    w = seeded_weights(k, n, 9)
    p, s = oracle.quantize_pack(w, k, n, 128)
    s_rep = np.repeat(s, 4, axis=0)
    assert np.array_equal(oracle.dequant_f32(p, s, k, n, 128), oracle.dequant_f32(p, s_rep, k, n, 32))


def test_splitk_plan_ref_values():
    """The reference heuristic (quantize.rs:1314-1325) at the benchmark shapes."""
    assert oracle.splitk_plan_ref(4608, 3584) == (18, 14, 8)
    assert oracle.splitk_plan_ref(3584, 3584) == (14, 14, 8)
    assert oracle.splitk_plan_ref(37888, 3584) == (148, 1, 112)
    assert oracle.splitk_plan_ref(3584, 18944) == (14, 19, 32)
    assert oracle.splitk_plan_ref(9728, 896) == (38, 1, 28)       # k < 2048 never splits


def test_fuse_n():
    k = 128
    mats = []
    for i, n in enumerate((8, 3, 5)):
        mats.append(oracle.quantize_pack(seeded_weights(k, n, 20 + i), k, n, 32))
    fp, fs = oracle.fuse_n(mats, k, 32)
    assert fp.shape == (4, 16, 16) and fs.shape == (4, 16)
    assert np.array_equal(fp, np.concatenate([p for p, _ in mats], axis=1))
    assert np.array_equal(fs, np.concatenate([s for _, s in mats], axis=1))
    # fusing never changes values: dequant of the fused matrix = concatenation of the dequants
    d = oracle.dequant_f32(fp, fs, k, 16, 32)
    assert np.array_equal(d, np.concatenate([oracle.dequant_f32(p, s, k, p.shape[1], 32) for p, s in mats], axis=1))
