"""Generates tests/golden/reference_kernels.npz on a machine with a B200.

Runs the REFERENCE'S OWN CUDA kernels (compiled unchanged into oracle/_ref by oracle/build_ref.py:
warp_gemm_tw_marlin_m1_direct, warp_gemm_tw_marlin_m1, warp_quantize_q4_0, warp_dequantize_q4_0,
warp_dequant_q4_to_f16, warp_gemm_q4_0, batched_marlin_gate_up, batched_marlin_split_geglu,
batched_marlin_down_axpy) on small seeded inputs and stores inputs and outputs, so
that the CPU-only tests can pin the oracle against the reference's results.

    python tests/golden/make_golden.py [output.npz]        (default: tests/golden/reference_kernels.npz, in place)
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from oracle import ref as oref  # noqa: E402
from helpers import seeded_activations, seeded_weights  # noqa: E402


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def main(out_path):
    out = {}
    # 1. TW-Marlin M=1 GEMM, direct (one K slice) and split-K (FP32 atomics), reference layout G=32
    for tag, (k, n) in {"a": (896, 384), "b": (2048, 300), "c": (3584, 136)}.items():
        w = seeded_weights(k, n, 100 + k)
        packed, scales = oracle.quantize_pack(w, k, n, 32)         # inputs only; outputs come from the reference
        a = seeded_activations(1, k, 7)
        ad, pd, sd = dev(a), dev(packed), dev(scales.view(np.float16))
        c_direct = torch.zeros(n, dtype=torch.float32, device="cuda")
        oref.gemm_tw_marlin_m1(c_direct.data_ptr(), ad.data_ptr(), pd.data_ptr(), sd.data_ptr(), n, k, force_splits=1)
        c_auto = torch.zeros(n, dtype=torch.float32, device="cuda")
        used = oref.gemm_tw_marlin_m1(c_auto.data_ptr(), ad.data_ptr(), pd.data_ptr(), sd.data_ptr(), n, k)
        torch.cuda.synchronize()
        out[f"gemm_{tag}_k"] = np.int64(k)
        out[f"gemm_{tag}_n"] = np.int64(n)
        out[f"gemm_{tag}_a"] = a
        out[f"gemm_{tag}_packed"] = packed
        out[f"gemm_{tag}_scales"] = scales
        out[f"gemm_{tag}_c_direct"] = c_direct.cpu().numpy()
        out[f"gemm_{tag}_c_auto"] = c_auto.cpu().numpy()
        out[f"gemm_{tag}_splits_auto"] = np.int64(used)
    # 2. Q4_0 quantise / dequantise of a flat array (the closed-form input of q4_0_roundtrip_correctness)
    x = np.array([((i * 7 + 3) % 200) * 0.01 - 1.0 for i in range(1024)], dtype=np.float32)
    xd = dev(x)
    blocks = torch.zeros(1024 // 32 * 20, dtype=torch.uint8, device="cuda")
    oref.quantize_q4_0(blocks.data_ptr(), xd.data_ptr(), 1024)
    back = torch.zeros(1024, dtype=torch.float32, device="cuda")
    oref.dequantize_q4_0(back.data_ptr(), blocks.data_ptr(), 1024)
    torch.cuda.synchronize()
    out["q4_x"] = x
    out["q4_blocks"] = blocks.cpu().numpy()
    out["q4_roundtrip"] = back.cpu().numpy()
    # 3. column-block Q4_0 matrix -> FP16 dequant and the 32x32-tile GEMM (the reference's M>1 kernel)
    k, n, m = 128, 64, 5
    w = np.array([((i * 17 + 3) % 101) * 0.02 - 1.0 for i in range(k * n)], dtype=np.float32).reshape(k, n)
    cols = np.ascontiguousarray(w.T).reshape(-1)
    cb = torch.zeros(cols.size // 32 * 20, dtype=torch.uint8, device="cuda")      # column-major blocks: (col*nkb + blk)*20
    oref.quantize_q4_0(cb.data_ptr(), dev(cols).data_ptr(), cols.size)
    f16 = torch.zeros((k, n), dtype=torch.float16, device="cuda")
    oref.dequant_q4_to_f16(f16.data_ptr(), cb.data_ptr(), k, n)
    a = seeded_activations(m, k, 9)
    c = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    oref.gemm_q4_0(c.data_ptr(), dev(a).data_ptr(), cb.data_ptr(), m, n, k)
    torch.cuda.synchronize()
    out["tile_w"] = w
    out["tile_a"] = a
    out["tile_blocks"] = cb.cpu().numpy()
    out["tile_dequant_f16_bits"] = f16.cpu().numpy().view(np.uint16)
    out["tile_c"] = c.cpu().numpy()
    # 4. batched expert GEMVs (crates/kernels/src/moe_batched_marlin.rs:21-152): gate+up, GEGLU, down + weighted sum
    hidden, moe_dim, n_experts, top_k = 256, 128, 4, 3
    rng = np.random.default_rng(12)
    ids = np.array([2, 0, 3], dtype=np.float32)
    wts = np.array([0.5, 0.3, 0.2], dtype=np.float32)
    x = rng.standard_normal(hidden, dtype=np.float32).astype(np.float16).astype(np.float32)
    gu = [oracle.quantize_pack(seeded_weights(hidden, 2 * moe_dim, 300 + e), hidden, 2 * moe_dim, 32) for e in range(n_experts)]
    dn = [oracle.quantize_pack(seeded_weights(moe_dim, hidden, 400 + e), moe_dim, hidden, 32) for e in range(n_experts)]
    gu_p = np.concatenate([p.reshape(-1) for p, _ in gu]); gu_s = np.concatenate([s.reshape(-1) for _, s in gu])
    dn_p = np.concatenate([p.reshape(-1) for p, _ in dn]); dn_s = np.concatenate([s.reshape(-1) for _, s in dn])
    gu_pb, gu_sb, dn_pb, dn_sb = gu[0][0].size, gu[0][1].size, dn[0][0].size, dn[0][1].size
    xd, idd, wtd = dev(x), dev(ids), dev(wts)
    gu_pd, gu_sd, dn_pd, dn_sd = dev(gu_p), dev(gu_s.view(np.float16)), dev(dn_p), dev(dn_s.view(np.float16))   # kept alive while the kernels run
    c_gu = torch.zeros((top_k, 2 * moe_dim), dtype=torch.float32, device="cuda")
    oref.batched_marlin_gate_up(c_gu.data_ptr(), xd.data_ptr(), gu_pd.data_ptr(), gu_sd.data_ptr(),
                                idd.data_ptr(), gu_pb, gu_sb, 2 * moe_dim, hidden, top_k)
    act = torch.zeros((top_k, moe_dim), dtype=torch.float32, device="cuda")
    oref.batched_marlin_split_geglu(act.data_ptr(), c_gu.data_ptr(), moe_dim, top_k)
    acc = torch.zeros(hidden, dtype=torch.float32, device="cuda")
    oref.batched_marlin_down_axpy(acc.data_ptr(), act.data_ptr(), dn_pd.data_ptr(), dn_sd.data_ptr(),
                                  idd.data_ptr(), wtd.data_ptr(), dn_pb, dn_sb, hidden, moe_dim, top_k)
    torch.cuda.synchronize()
    out.update({"moe_x": x, "moe_ids": ids, "moe_wts": wts, "moe_gu_packed": gu_p, "moe_gu_scales": gu_s, "moe_dn_packed": dn_p,
                "moe_dn_scales": dn_s, "moe_dims": np.array([hidden, moe_dim, n_experts, top_k, gu_pb, gu_sb, dn_pb, dn_sb], dtype=np.int64),
                "moe_gate_up": c_gu.cpu().numpy(), "moe_act": act.cpu().numpy(), "moe_acc": acc.cpu().numpy()})
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k_: getattr(v, "shape", ()) for k_, v in out.items() if k_.endswith(("c_direct", "tile_c"))})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_kernels.npz"))
