"""GPU parity tests of the batched expert GEMVs (twm_moe_gate_up / twm_moe_down_axpy) against the CPU
restatement of the reference's kernels (crates/kernels/src/moe_batched_marlin.rs:21-152) and
against those kernels themselves, compiled unchanged into oracle/_ref; and of the on-device
Q4_0-block -> TW-Marlin reorder (quantize.rs:912-956)."""
import numpy as np
import pytest
import torch

import oracle
from oracle import ref as oref
from helpers import rel_err_floored, seeded_weights
from tensorwarp_b200 import _lib
from tensorwarp_b200 import quantize as q

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).to(DEV)
    return t if dtype is None else t.to(dtype)


def _experts(n_experts, k, n, group, seed):
    """All experts' TW-Marlin tensors in two flat buffers, as the reference's loader lays them out."""
    ps, ss = [], []
    for e in range(n_experts):
        p, s = oracle.quantize_pack(seeded_weights(k, n, seed + e), k, n, group)
        ps.append(p.reshape(-1))
        ss.append(s.reshape(-1))
    return np.concatenate(ps), np.concatenate(ss), ps[0].size, ss[0].size


# (hidden, moe_dim, experts, top_k, group): small; a Gemma-MoE-like shape; shapes whose weighted sum fills a 15- or
# 16-CTA cluster; and twenty slots, more than a cluster holds, so that the sum goes through the workspace
CASES = [(256, 128, 4, 2, 32), (256, 128, 4, 2, 128), (2816, 704, 16, 8, 32), (1024, 2048, 8, 4, 128), (512, 4096, 6, 3, 128),
         (256, 128, 24, 20, 32)]


@pytest.mark.parametrize("hidden,moe_dim,n_experts,top_k,group", CASES)
def test_expert_gemvs_against_oracle(hidden, moe_dim, n_experts, top_k, group):
    rng = np.random.default_rng(hidden + moe_dim)
    ids = rng.permutation(n_experts)[:top_k].astype(np.float32)
    wts = rng.random(top_k, dtype=np.float32)
    wts /= wts.sum()
    x = rng.standard_normal(hidden, dtype=np.float32).astype(np.float16).astype(np.float32)
    gu_p, gu_s, gu_pb, gu_sb = _experts(n_experts, hidden, 2 * moe_dim, group, 700)
    dn_p, dn_s, dn_pb, dn_sb = _experts(n_experts, moe_dim, hidden, group, 800)
    ws = q.Workspace(max(q.moe_workspace_bytes(top_k, 2 * moe_dim, hidden, group), q.moe_workspace_bytes(top_k, hidden, moe_dim, group), 16))
    ids_d, wts_d = _dev(ids), _dev(wts)
    # ---- gate + up: one row per slot
    gate_up = torch.full((top_k, 2 * moe_dim), float("nan"), dtype=torch.float16, device=DEV)
    q.batched_marlin_gate_up(_dev(x, torch.float16), _dev(gu_p), _dev(gu_s.view(np.float16)), ids_d, gate_up, gu_pb, gu_sb,
                             2 * moe_dim, hidden, top_k, group_size=group, workspace=ws)
    torch.cuda.synchronize()
    assert q.device_error() == 0
    ref_gu = oracle.moe_gate_up(x, gu_p, gu_s, ids, gu_pb, gu_sb, hidden, 2 * moe_dim, group)
    got_gu = gate_up.float().cpu().numpy()
    assert not np.isnan(got_gu).any()
    assert rel_err_floored(got_gu, ref_gu.astype(np.float64)) < 1e-2
    # ---- gated activation + down + weighted sum, from the kernel's own FP16 gate_up
    acc = torch.full((hidden,), 0.25, dtype=torch.float32, device=DEV)
    q.batched_marlin_down_axpy(gate_up, _dev(dn_p), _dev(dn_s.view(np.float16)), ids_d, wts_d, acc, dn_pb, dn_sb, hidden,
                               moe_dim, top_k, activation="geglu", group_size=group, workspace=ws,
                               flags=_lib.TWM_FLAG_ACCUMULATE)
    torch.cuda.synchronize()
    assert q.device_error() == 0
    act = oracle.moe_split_geglu(got_gu, moe_dim).astype(np.float16).astype(np.float32)     # the GEMV multiplies FP16 values
    _, ref64 = oracle.moe_down_axpy(act, dn_p, dn_s, ids, wts, dn_pb, dn_sb, moe_dim, hidden, group,
                                    acc=np.full(hidden, 0.25, dtype=np.float32))
    got = acc.cpu().numpy()
    # tanhf on the device and in libm differ in the last place: a few FP16 roundings of the activation may flip
    assert rel_err_floored(got[None], ref64[None]) < 1e-2
    # same bits every run (the reference's atomicAdd order is not fixed), and without ACCUMULATE the row is overwritten
    again = torch.full((hidden,), 0.25, dtype=torch.float32, device=DEV)
    q.batched_marlin_down_axpy(gate_up, _dev(dn_p), _dev(dn_s.view(np.float16)), ids_d, wts_d, again, dn_pb, dn_sb, hidden,
                               moe_dim, top_k, activation="geglu", group_size=group, workspace=ws,
                               flags=_lib.TWM_FLAG_ACCUMULATE)
    plain = torch.full((hidden,), 123.0, dtype=torch.float32, device=DEV)
    q.batched_marlin_down_axpy(gate_up, _dev(dn_p), _dev(dn_s.view(np.float16)), ids_d, wts_d, plain, dn_pb, dn_sb, hidden,
                               moe_dim, top_k, activation="geglu", group_size=group, workspace=ws)
    torch.cuda.synchronize()
    assert torch.equal(again, acc)
    assert rel_err_floored((plain + 0.25).cpu().numpy()[None], ref64[None]) < 1e-2
    assert int(ws.buf[:16384].view(torch.int32).abs().sum().item()) == 0       # counters handed back at zero


def test_expert_gemvs_against_reference_kernels():
    """The reference's own batched kernels on this GPU (F32 activations, group 32, atomicAdd) against
    the oracle restatement and against this library's kernels on the same inputs."""
    if not oref.available():
        pytest.skip("oracle/_ref not built")
    hidden, moe_dim, n_experts, top_k, group = 1024, 512, 8, 4, 32
    rng = np.random.default_rng(5)
    ids = rng.permutation(n_experts)[:top_k].astype(np.float32)
    wts = rng.random(top_k, dtype=np.float32)
    x = rng.standard_normal(hidden, dtype=np.float32).astype(np.float16).astype(np.float32)
    gu_p, gu_s, gu_pb, gu_sb = _experts(n_experts, hidden, 2 * moe_dim, group, 900)
    dn_p, dn_s, dn_pb, dn_sb = _experts(n_experts, moe_dim, hidden, group, 950)
    xd, ids_d, wts_d = _dev(x), _dev(ids), _dev(wts)
    gu_pd, gu_sd = _dev(gu_p), _dev(gu_s.view(np.float16))
    dn_pd, dn_sd = _dev(dn_p), _dev(dn_s.view(np.float16))
    ref_gu = torch.zeros((top_k, 2 * moe_dim), device=DEV)
    oref.batched_marlin_gate_up(ref_gu.data_ptr(), xd.data_ptr(), gu_pd.data_ptr(), gu_sd.data_ptr(), ids_d.data_ptr(), gu_pb,
                                gu_sb, 2 * moe_dim, hidden, top_k)
    ref_act = torch.zeros((top_k, moe_dim), device=DEV)
    oref.batched_marlin_split_geglu(ref_act.data_ptr(), ref_gu.data_ptr(), moe_dim, top_k)
    ref_acc = torch.zeros(hidden, device=DEV)
    oref.batched_marlin_down_axpy(ref_acc.data_ptr(), ref_act.data_ptr(), dn_pd.data_ptr(), dn_sd.data_ptr(), ids_d.data_ptr(),
                                  wts_d.data_ptr(), dn_pb, dn_sb, hidden, moe_dim, top_k)
    torch.cuda.synchronize()
    # the oracle restates the reference kernels: gate+up bit for bit, GEGLU to the last place of tanhf,
    # the weighted sum to FP32 summation order (atomicAdd)
    o_gu = oracle.moe_gate_up(x, gu_p, gu_s, ids, gu_pb, gu_sb, hidden, 2 * moe_dim, group)
    assert np.array_equal(o_gu.view(np.uint32), ref_gu.cpu().numpy().view(np.uint32))
    o_act = oracle.moe_split_geglu(o_gu, moe_dim)
    assert np.max(np.abs(o_act - ref_act.cpu().numpy())) <= 1e-6 * max(1.0, float(np.abs(o_act).max()))
    o_acc, o_acc64 = oracle.moe_down_axpy(ref_act.cpu().numpy(), dn_p, dn_s, ids, wts, dn_pb, dn_sb, moe_dim, hidden, group)
    rms = float(np.sqrt(np.mean(o_acc64 ** 2)))
    assert np.max(np.abs(ref_acc.cpu().numpy() - o_acc64)) < 1e-5 * rms
    # this library on the same inputs (FP16 gate_up in between instead of F32: FP16-level agreement)
    gate_up = torch.zeros((top_k, 2 * moe_dim), dtype=torch.float16, device=DEV)
    q.batched_marlin_gate_up(xd.half(), gu_pd, gu_sd, ids_d, gate_up, gu_pb, gu_sb, 2 * moe_dim, hidden, top_k, group_size=group)
    acc = torch.zeros(hidden, device=DEV)
    q.batched_marlin_down_axpy(gate_up, dn_pd, dn_sd, ids_d, wts_d, acc, dn_pb, dn_sb, hidden, moe_dim, top_k,
                               activation="geglu", group_size=group)
    torch.cuda.synchronize()
    assert q.device_error() == 0
    assert rel_err_floored(gate_up.float().cpu().numpy(), ref_gu.cpu().numpy().astype(np.float64)) < 1e-2
    assert np.max(np.abs(acc.cpu().numpy() - ref_acc.cpu().numpy())) < 2e-2 * float(ref_acc.pow(2).mean().sqrt())


@pytest.mark.parametrize("k,n", [(128, 64), (3584, 520), (32, 1), (2048, 4608)])
def test_reorder_from_q4_0_blocks_bit_exact(k, n):
    """Column-major Q4_0 blocks -> TW-Marlin on the device, bit for bit the oracle's restatement of
    reorder_to_tw_marlin (quantize.rs:912-956)."""
    w = seeded_weights(k, n, 61)
    p0, s0 = oracle.quantize_pack(w, k, n, 32)
    blocks = oracle.tw_marlin_to_q4_0_blocks(p0, s0, k, n)
    # give the blocks scales that are NOT FP16-representable, as a real Q4_0 tensor has (f32 amax / 7)
    b = blocks.reshape(-1, 20).copy()
    sc = b[:, :4].copy().view(np.float32)
    sc *= np.float32(1.0 + 2.0 ** -13)
    b[:, :4] = sc.view(np.uint8)
    blocks = b.reshape(-1)
    p_ref, s_ref = oracle.reorder_to_tw_marlin(blocks, k, n)
    p, s = q.reorder_to_tw_marlin(_dev(blocks), k, n)
    torch.cuda.synchronize()
    assert np.array_equal(p.cpu().numpy(), p_ref)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), s_ref)
    assert np.array_equal(p_ref, p0)


def test_from_quantized_builds_a_layer_that_runs():
    """TWMarlinWeights.from_quantized (quantize.rs:1090-1134) + fuse_projections: the fused tensors equal the
    oracle's fusion of the reordered parts, and a GEMV on them matches the oracle."""
    hidden, kv, ffn = 256, 128, 512
    names = {"wq": (hidden, hidden), "wk": (hidden, kv), "wv": (hidden, kv), "wo": (hidden, hidden),
             "w_gate": (hidden, ffn), "w_up": (hidden, ffn), "w_down": (ffn, hidden)}
    qw, host = {}, {}
    for i, (name, (k, n)) in enumerate(names.items()):
        p, s = oracle.quantize_pack(seeded_weights(k, n, 70 + i), k, n, 32)
        host[name] = (p, s)
        qw[name] = _dev(oracle.tw_marlin_to_q4_0_blocks(p, s, k, n))
    qw["attn_norm"] = torch.ones(hidden, device=DEV)
    qw["ffn_norm"] = torch.ones(hidden, device=DEV)
    lw = q.TWMarlinWeights.from_quantized(qw, hidden, kv, ffn, fuse=True)
    fp, fs = oracle.fuse_n([host["wq"], host["wk"], host["wv"]], hidden, 32)
    assert np.array_equal(lw.wqkv[0].cpu().numpy(), fp) and np.array_equal(lw.wqkv[1].cpu().numpy().view(np.uint16), fs)
    a = np.random.default_rng(1).standard_normal((1, hidden), dtype=np.float32).astype(np.float16).astype(np.float32)
    c = torch.zeros(2 * ffn, dtype=torch.float16, device=DEV)
    q.gemm_tw_marlin_m1(_dev(a, torch.float16), lw.wgu[0], lw.wgu[1], c, 2 * ffn, hidden, group_size=32)
    torch.cuda.synchronize()
    gp, gs = oracle.fuse_n([host["w_gate"], host["w_up"]], hidden, 32)
    assert rel_err_floored(c.float().cpu().numpy()[None], oracle.w4a16_f64(a, gp, gs, 1, 2 * ffn, hidden, 32)) < 1e-2
