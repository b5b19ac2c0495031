"""CPU tests that pin the oracle against outputs of the reference's own CUDA kernels.

tests/golden/reference_kernels.npz was written by tests/golden/make_golden.py on a B200 from the
kernels in the reference tree, compiled unchanged (oracle/build_ref.py).  No GPU is needed here."""
import os

import numpy as np

import oracle

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernels.npz"))


def test_m1_kernel_restatement_equals_reference_direct_kernel_bit_for_bit():
    """warp_gemm_tw_marlin_m1_direct (quantize.rs:1249-1298)."""
    for tag in ("a", "b", "c"):
        k, n = int(GOLD[f"gemm_{tag}_k"]), int(GOLD[f"gemm_{tag}_n"])
        a, packed, scales = GOLD[f"gemm_{tag}_a"], GOLD[f"gemm_{tag}_packed"], GOLD[f"gemm_{tag}_scales"]
        ours = oracle.m1_kernel_order(a[0], packed, scales, n, k, 32)
        assert np.array_equal(ours.view(np.uint32), GOLD[f"gemm_{tag}_c_direct"].view(np.uint32)), tag


def test_reference_splitk_kernel_and_heuristic():
    """warp_gemm_tw_marlin_m1 + the launcher's split count (quantize.rs:1186-1245, 1317-1325): FP32
    atomics in any order, so agreement is to summation error."""
    for tag in ("a", "b", "c"):
        k, n = int(GOLD[f"gemm_{tag}_k"]), int(GOLD[f"gemm_{tag}_n"])
        a, packed, scales = GOLD[f"gemm_{tag}_a"], GOLD[f"gemm_{tag}_packed"], GOLD[f"gemm_{tag}_scales"]
        assert int(GOLD[f"gemm_{tag}_splits_auto"]) == oracle.splitk_plan_ref(n, k)[1]
        ref64 = oracle.w4a16_f64(a, packed, scales, 1, n, k, 32)[0]
        rms = float(np.sqrt(np.mean(ref64 ** 2)))
        assert np.max(np.abs(GOLD[f"gemm_{tag}_c_auto"] - ref64)) < 1e-5 * rms
        assert np.max(np.abs(oracle.w4a16_literal(a, packed, scales, 1, n, k, 32)[0] - ref64)) < 1e-5 * rms


def test_quantiser_equals_reference_quantise_kernel():
    """warp_quantize_q4_0 / warp_dequantize_q4_0 (quantize.rs:103-175) on the input of the
    reference's q4_0_roundtrip_correctness test (quantize.rs:3009)."""
    x = GOLD["q4_x"]
    blocks = GOLD["q4_blocks"].reshape(-1, 20)
    packed, scales = oracle.quantize_pack(x.reshape(-1, 1), x.size, 1, 32)        # one column of K = 1024
    assert np.array_equal(blocks[:, 4:], packed[:, 0, :])
    scale32 = blocks[:, :4].copy().view(np.float32).reshape(-1)
    assert np.array_equal(oracle.f32_to_f16_bits(scale32), scales[:, 0])
    assert np.array_equal(oracle.q4_0_roundtrip(x).view(np.uint32), GOLD["q4_roundtrip"].view(np.uint32))


def test_decode_order_equals_reference_f16_dequant_and_tile_gemm():
    """warp_dequant_q4_to_f16 and warp_gemm_q4_0 (quantize.rs:534-571, 186-246) on column-block Q4_0:
    the nibble order and `scale * (q - 8)` of the oracle reproduce them."""
    w, a = GOLD["tile_w"], GOLD["tile_a"]
    k, n = w.shape
    blocks = GOLD["tile_blocks"].reshape(n, k // 32, 20)                   # (col * nkb + blk) * 20
    packed, _ = oracle.quantize_pack(w, k, n, 32)
    assert np.array_equal(np.transpose(blocks[:, :, 4:], (1, 0, 2)), packed)
    scale32 = blocks[:, :, :4].copy().view(np.float32).reshape(n, k // 32).T       # [blk][col]
    # decode with the f32 scale the Q4_0 block carries: exact f32 product, f16 rounding of it
    nib = np.zeros((k, n), dtype=np.float32)
    for kk in range(k):
        byte = packed[kk // 32, :, (kk % 32) // 2]
        nib[kk] = ((byte >> 4) if (kk % 2) else (byte & 0x0F)).astype(np.float32) - 8.0
    dense = (np.repeat(scale32, 32, axis=0) * nib).astype(np.float32)
    assert np.array_equal(oracle.f32_to_f16_bits(dense), GOLD["tile_dequant_f16_bits"])
    c = oracle.gemm_f32(a, dense, a.shape[0], n, k)
    assert np.max(np.abs(c - GOLD["tile_c"])) < 1e-4 * float(np.sqrt(np.mean(c.astype(np.float64) ** 2)))


def test_reorder_restatement_on_the_reference_quantisers_blocks():
    """reorder_to_tw_marlin (quantize.rs:912-956) restated: on column-major Q4_0 blocks written by the
    reference's own quantise kernel it gives the oracle quantiser's packed bytes and the FP16 rounding
    of the blocks' FP32 scales; and back again."""
    w = GOLD["tile_w"]
    k, n = w.shape
    packed, scales = oracle.reorder_to_tw_marlin(GOLD["tile_blocks"], k, n)
    p_ref, s_ref = oracle.quantize_pack(w, k, n, 32)
    assert np.array_equal(packed, p_ref) and np.array_equal(scales, s_ref)
    blocks = GOLD["tile_blocks"].reshape(n, k // 32, 20)
    scale32 = blocks[:, :, :4].copy().view(np.float32).reshape(n, k // 32).T
    assert np.array_equal(oracle.f32_to_f16_bits(scale32), scales)
    again = oracle.reorder_to_tw_marlin(oracle.tw_marlin_to_q4_0_blocks(packed, scales, k, n), k, n)
    assert np.array_equal(again[0], packed) and np.array_equal(again[1], scales)


def test_moe_restatement_equals_reference_batched_kernels():
    """batched_marlin_gate_up / split_geglu / down_axpy (moe_batched_marlin.rs:21-152): the gate+up kernel
    bit for bit, GEGLU to the last place of tanhf, the atomicAdd-ed weighted sum to FP32 summation order."""
    hidden, moe_dim, n_experts, top_k, gu_pb, gu_sb, dn_pb, dn_sb = (int(v) for v in GOLD["moe_dims"])
    x, ids, wts = GOLD["moe_x"], GOLD["moe_ids"], GOLD["moe_wts"]
    gu = oracle.moe_gate_up(x, GOLD["moe_gu_packed"], GOLD["moe_gu_scales"], ids, gu_pb, gu_sb, hidden, 2 * moe_dim, 32)
    assert np.array_equal(gu.view(np.uint32), GOLD["moe_gate_up"].view(np.uint32))
    act = oracle.moe_split_geglu(gu, moe_dim)
    assert np.max(np.abs(act - GOLD["moe_act"])) <= 1e-6 * max(1.0, float(np.abs(act).max()))
    acc, acc64 = oracle.moe_down_axpy(GOLD["moe_act"], GOLD["moe_dn_packed"], GOLD["moe_dn_scales"], ids, wts, dn_pb, dn_sb,
                                      moe_dim, hidden, 32)
    rms = float(np.sqrt(np.mean(acc64 ** 2)))
    assert np.max(np.abs(GOLD["moe_acc"] - acc64)) < 1e-5 * rms
    assert np.max(np.abs(acc - acc64)) < 1e-5 * rms
