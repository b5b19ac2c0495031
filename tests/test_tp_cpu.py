"""CPU tests of the tensor-parallel host logic: shard arithmetic, and a two-process gloo run in
which column/row shards of TW-Marlin tensors plus one all-reduce reproduce the unsharded GEMMs
(computed by the CPU oracle on both sides; no GPU involved)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from helpers import seeded_activations, seeded_weights
from tensorwarp_b200 import tensor_parallel as tp
from tensorwarp_b200.generate import TransformerConfig


def test_shard_spec_covers_everything_once():
    cfg = tp.LLAMA3_70B
    for degree in (1, 2, 4, 8):
        specs = [tp.shard_spec(cfg, degree, r) for r in range(degree)]
        assert specs[0].q_heads[0] == 0 and specs[-1].q_heads[1] == cfg.num_heads
        assert specs[0].ffn[0] == 0 and specs[-1].ffn[1] == cfg.ffn
        for a, b in zip(specs, specs[1:]):
            assert a.q_heads[1] == b.q_heads[0] and a.kv_heads[1] == b.kv_heads[0] and a.ffn[1] == b.ffn[0]
        for s in specs:
            assert s.n_qkv == (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim // degree
            assert s.n_gu == 2 * cfg.ffn // degree
            assert (s.q_cols[1] - s.q_cols[0]) % cfg.group_size == 0       # row shards hold whole scale groups
            # a group of query heads stays with its kv head
            group = cfg.num_heads // cfg.num_kv_heads
            assert s.q_heads[0] // group == s.kv_heads[0] and (s.q_heads[1] - 1) // group == s.kv_heads[1] - 1
    # the sizes the benchmark plan lists for tp = 8
    s = tp.shard_spec(cfg, 8, 0)
    assert (s.n_qkv, s.n_gu) == (1280, 7168)


def test_shard_spec_rejects_bad_degrees():
    cfg = tp.LLAMA3_70B
    with pytest.raises(ValueError):
        tp.shard_spec(cfg, 3, 0)             # 64 heads do not divide by 3
    with pytest.raises(ValueError):
        tp.shard_spec(cfg, 8, 8)
    small = TransformerConfig(hidden=256, num_heads=2, num_kv_heads=2, head_dim=128, ffn=192, vocab=10, layers=1,
                              group_size=128)
    with pytest.raises(ValueError):
        tp.shard_spec(small, 2, 0)           # ffn/2 = 96 is not a whole 128-group


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = TransformerConfig(hidden=256, num_heads=4, num_kv_heads=2, head_dim=128, ffn=512, vocab=10, layers=1,
                            group_size=128, qkv_bias=False)
    spec = tp.shard_spec(cfg, world, rank)
    g = cfg.group_size
    # every rank builds the same full tensors, then keeps only its share
    w_up = seeded_weights(cfg.hidden, cfg.ffn, 1)
    w_down = seeded_weights(cfg.ffn, cfg.hidden, 2)
    pu, su = oracle.quantize_pack(w_up, cfg.hidden, cfg.ffn, g)
    pd, sd = oracle.quantize_pack(w_down, cfg.ffn, cfg.hidden, g)
    x = seeded_activations(3, cfg.hidden, 4)
    # column-parallel: local columns of `up`, no communication
    c0, c1 = spec.ffn
    pu_l, su_l = np.ascontiguousarray(pu[:, c0:c1]), np.ascontiguousarray(su[:, c0:c1])
    act_local = oracle.w4a16_f64(x, pu_l, su_l, 3, c1 - c0, cfg.hidden, g).astype(np.float32)
    act_local = act_local.astype(np.float16).astype(np.float32)              # GEMM output is FP16
    # row-parallel: local K range of `down`, FP32 partial, one all-reduce
    pd_l, sd_l = np.ascontiguousarray(pd[c0 // 32:c1 // 32]), np.ascontiguousarray(sd[c0 // g:c1 // g])
    part = oracle.w4a16_f64(act_local, pd_l, sd_l, 3, cfg.hidden, c1 - c0, g).astype(np.float32)
    t = torch.from_numpy(part)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    # unsharded reference on every rank
    act_full = oracle.w4a16_f64(x, pu, su, 3, cfg.ffn, cfg.hidden, g).astype(np.float32)
    act_full = act_full.astype(np.float16).astype(np.float32)
    ref = oracle.w4a16_f64(act_full, pd, sd, 3, cfg.hidden, cfg.ffn, g)
    assert np.array_equal(act_full[:, c0:c1], act_local)                     # a column shard computes its columns exactly
    err = float(np.max(np.abs(t.numpy() - ref)) / np.sqrt(np.mean(ref ** 2)))
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(f"{err}\n")
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_row_parallel_sum_equals_unsharded(tmp_path):
    oracle.build()
    port = _free_port()
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        err = float(open(tmp_path / f"rank{r}.txt").read())
        assert err < 1e-5, (r, err)
