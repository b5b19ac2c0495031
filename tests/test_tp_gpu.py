"""GPU test of the tensor-parallel layer stack on ONE device: the ranks of a tp=2 (and tp=4) group
are run phase by phase in one process and their partial outputs are summed where NCCL would
all-reduce them; the result must match the unsharded stack (tp=1).  The multi-process NCCL run is
bench.py --gpus N."""
import numpy as np
import pytest
import torch

from tensorwarp_b200 import quantize as q
from tensorwarp_b200 import tensor_parallel as tp
from tensorwarp_b200.generate import TransformerConfig

pytestmark = pytest.mark.gpu

CFG = TransformerConfig(hidden=512, num_heads=8, num_kv_heads=4, head_dim=128, ffn=1024, vocab=10, layers=3,
                        rope_theta=5e5, eps=1e-5, max_seq=256, group_size=128, qkv_bias=False)


def _full_layers(cfg, seed):
    out = []
    dev = "cuda"
    for layer in range(cfg.layers):
        shapes = [(cfg.hidden, cfg.q_dim), (cfg.hidden, cfg.kv_dim), (cfg.hidden, cfg.kv_dim), (cfg.q_dim, cfg.hidden),
                  (cfg.hidden, cfg.ffn), (cfg.hidden, cfg.ffn), (cfg.ffn, cfg.hidden)]
        mats = []
        for pid, (k, n) in enumerate(shapes):
            gen = torch.Generator(device=dev).manual_seed(seed + 1000 * layer + pid)
            w = torch.randn((k, n), generator=gen, device=dev) * 0.02
            mats.append(q.quantize_f32_to_tw_marlin(w, k, n, cfg.group_size))
        out.append(mats)
    return out


def _run(cfg, full, degree, rows, x0, kv_len, fused=False):
    ones = torch.ones(cfg.hidden, device="cuda")
    stacks = []
    comms = tp.PeerComm.local_group(degree, rows * cfg.hidden) if fused else [None] * degree
    for r in range(degree):
        spec = tp.shard_spec(cfg, degree, r)
        layers = [tp.shard_layer(cfg, spec, *mats, ones, ones) for mats in full]
        st = tp.TPDecodeStack(cfg, spec, layers, rows, "cuda", all_reduce=lambda t: None, comm=comms[r])
        stacks.append(st)
    # the same random KV cache for every degree: generate the full cache, hand each rank its kv heads
    gen = torch.Generator(device="cuda").manual_seed(11)
    for li in range(cfg.layers):
        kfull = torch.randn((rows, kv_len, cfg.kv_dim), generator=gen, device="cuda").half()
        vfull = torch.randn((rows, kv_len, cfg.kv_dim), generator=gen, device="cuda").half()
        for st in stacks:
            c0, c1 = st.spec.kv_cols
            st.k_cache[li][:, :kv_len] = kfull[:, :, c0:c1]
            st.v_cache[li][:, :kv_len] = vfull[:, :, c0:c1]
    for st in stacks:
        st.pos.fill_(kv_len)
        st.cache_len.fill_(kv_len + 1)
        st.x.copy_(x0)
    sp = torch.cuda.current_stream().cuda_stream

    def reduce_all():
        if fused:          # the GEMM epilogues already pushed every rank's partial into every rank's buffer
            return
        total = sum(st.part for st in stacks)
        for st in stacks:
            st.part.copy_(total)

    for li in range(cfg.layers):
        for st in stacks:
            st.attn_phase(li, sp)
        reduce_all()
        for st in stacks:
            st.ffn_phase(li, sp)
        reduce_all()
    for st in stacks:
        st.finish(sp)
    torch.cuda.synchronize()
    assert q.device_error() == 0
    out = [st.x.cpu().numpy() for st in stacks]
    for c in comms:
        if c is not None:
            c.close()
    return out


@pytest.mark.parametrize("rows", [1, 2, 3, 9])
def test_sharded_stack_equals_unsharded(rows):
    cfg = CFG
    full = _full_layers(cfg, 21)
    x0 = torch.randn((rows, cfg.hidden), generator=torch.Generator().manual_seed(5)).cuda()
    ref = _run(cfg, full, 1, rows, x0, 100)[0]
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    for degree in (2, 4):
        outs = _run(cfg, full, degree, rows, x0, 100)
        for o in outs[1:]:
            assert np.array_equal(o, outs[0])                 # every rank ends with the same activations
        err = float(np.max(np.abs(outs[0] - ref))) / rms
        assert err < 2e-3, (degree, err)                      # FP32 partials, different summation order only
        # the fused path: GEMM epilogues push into the peers' buffers, add+RMSNorm takes the sum
        fused = _run(cfg, full, degree, rows, x0, 100, fused=True)
        for o in fused[1:]:
            assert np.array_equal(o, fused[0])
        assert float(np.max(np.abs(fused[0] - ref))) / rms < 2e-3, degree


@pytest.mark.parametrize("kernel,rows,n,splits", [(3, 1, 3072, 0), (3, 2, 3072, 0), (3, 1, 8192, 0), (3, 2, 16384, 0), (3, 1, 512, 0),
                                                  (2, 5, 3072, 0), (2, 32, 8192, 0), (2, 64, 512, 0), (2, 32, 3072, 3),
                                                  (3, 3, 3072, 0), (3, 8, 3072, 2), (3, 9, 8192, 0), (3, 16, 3072, 3), (3, 32, 512, 0),
                                                  (3, 17, 3072, 0), (0, 12, 3072, 0), (0, 40, 3072, 0)])
def test_row_parallel_push_and_sum(kernel, rows, n, splits):
    """The row-parallel GEMM with `comm` on the streaming MMA kernel (one or two rows from its cluster leaders,
    three to 32 in its staged-rows form, also with K slices through the workspace), on the narrow tcgen05
    kernel (up to 64), and with the kernel left to the library, then the consumer: every
    rank's x + sum over ranks equals x + the unsharded GEMM, and all ranks hold the same bits.  Run
    twice in a row: the sequence number alternates between the two buffer sets."""
    import ctypes as C
    from tensorwarp_b200 import _lib
    lib = _lib.lib()
    degree, k, group = 2, 2048 if n <= 3072 else 512, 128
    gen = torch.Generator(device="cuda").manual_seed(5)
    w = torch.randn((k, n), generator=gen, device="cuda") * 0.02
    packed, scales = q.quantize_f32_to_tw_marlin(w, k, n, group)
    a = torch.randn((rows, k), generator=gen, device="cuda").half()
    full = torch.zeros((rows, n), device="cuda")
    ws = q.Workspace(64 << 20)
    q.gemm_tw_marlin(a, packed, scales, full, rows, n, k, group_size=group, workspace=ws)
    comms = tp.PeerComm.local_group(degree, rows * n)
    gamma = torch.ones(n, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    kb = k // degree
    shards = []
    for r in range(degree):
        p_r = packed.view(k // 32, n, 16)[r * kb // 32:(r + 1) * kb // 32].contiguous()
        s_r = scales.view(k // group, n)[r * kb // group:(r + 1) * kb // group].contiguous()
        shards.append((p_r, s_r, a[:, r * kb:(r + 1) * kb].contiguous()))
    # each rank's partial as the same kernel stores it without `comm`: what an NCCL all-reduce would add up
    parts = []
    for r in range(degree):
        p_r, s_r, a_r = shards[r]
        part = torch.zeros((rows, n), device="cuda")
        q.gemm_tw_marlin(a_r, p_r, s_r, part, rows, n, kb, group_size=group, kernel_override=kernel, workspace=ws,
                         splits_override=splits)
        parts.append(part)
    for step in range(2):
        xs = [torch.full((rows, n), 0.5 * (step + 1), device="cuda") for _ in range(degree)]
        dummy = torch.zeros((rows, n), device="cuda")
        for r in range(degree):                         # every rank's producer first ...
            p_r, s_r, a_r = shards[r]
            args = _lib.GemmArgs(M=rows, N=n, K=kb, group_size=group, a_dtype=_lib.TWM_F16, c_dtype=_lib.TWM_F32,
                                 a=a_r.data_ptr(), lda=kb, packed=p_r.data_ptr(), scales=s_r.data_ptr(),
                                 c=dummy.data_ptr(), ldc=n, kernel_override=kernel, comm=comms[r].ptr,
                                 workspace=ws.ptr, workspace_bytes=ws.nbytes, splits_override=splits)
            _lib.check(lib.twm_gemm_w4a16(C.byref(args), stream), "twm_gemm_w4a16")
        ys = [torch.zeros((rows, n), device="cuda", dtype=torch.float16) for _ in range(degree)]
        for r in range(degree):                         # ... then every rank's consumer
            _lib.check(lib.twm_allreduce_add_rmsnorm(ys[r].data_ptr(), xs[r].data_ptr(), comms[r].ptr, gamma.data_ptr(),
                                                     rows, n, 1e-5, 0, stream), "twm_allreduce_add_rmsnorm")
        torch.cuda.synchronize()
        assert q.device_error() == 0
        want = full + 0.5 * (step + 1)
        for r in range(degree):
            assert torch.equal(xs[r], xs[0]) and torch.equal(ys[r], ys[0])
        rms = float(want.pow(2).mean().sqrt())
        assert float((xs[0] - want).abs().max()) / rms < 2e-3
        assert torch.all(dummy == 0)                    # with comm the result goes to the peers only
        # the one-CTA add + RMSNorm on the rank-order sum of the partials (the NCCL path's kernel) gives the
        # same bits as the multi-CTA consumer: both take the sum of squares in the same order
        x_ref = torch.full((rows, n), 0.5 * (step + 1), device="cuda")
        y_ref = torch.zeros((rows, n), device="cuda", dtype=torch.float16)
        summed = parts[0] + parts[1]
        _lib.check(lib.twm_add_rmsnorm(y_ref.data_ptr(), x_ref.data_ptr(), summed.data_ptr(), gamma.data_ptr(), rows, n,
                                       1e-5, 0, stream), "twm_add_rmsnorm")
        torch.cuda.synchronize()
        assert torch.equal(xs[0], x_ref) and torch.equal(ys[0], y_ref)
    for c in comms:
        c.close()


def test_consumer_wait_runs_out_without_a_producer():
    """A consumer whose peers never deliver: the bounded wait (50 ms here, a field of twm_comm) expires, the
    kernel returns, the device error word carries bit 2, x is left as it was, and the context stays usable.
    Nothing hangs and nothing faults: the failure is a flag that nobody sets."""
    import ctypes as C
    from tensorwarp_b200 import _lib
    lib = _lib.lib()
    rows, n = 1, 2048
    comms = tp.PeerComm.local_group(2, rows * n, wait_ms=50.0)
    x = torch.full((rows, n), 3.0, device="cuda")
    y = torch.full((rows, n), 7.0, device="cuda", dtype=torch.float16)
    gamma = torch.ones(n, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert q.device_error() == 0
    _lib.check(lib.twm_allreduce_add_rmsnorm(y.data_ptr(), x.data_ptr(), comms[0].ptr, gamma.data_ptr(), rows, n, 1e-5,
                                             0, stream), "twm_allreduce_add_rmsnorm")
    torch.cuda.synchronize()
    word = C.c_uint(0)
    assert lib.twm_device_error(stream, C.byref(word)) == _lib.TWM_ETIMEOUT
    assert word.value & 4
    assert torch.all(x == 3.0) and torch.all(y == 7.0)
    assert q.device_error() == 0                       # reading cleared it
    # the context is alive: an ordinary GEMM still runs
    w = torch.randn((256, 128), device="cuda") * 0.02
    p, s = q.quantize_f32_to_tw_marlin(w, 256, 128, 128)
    c = torch.zeros(128, dtype=torch.float16, device="cuda")
    q.gemm_tw_marlin_m1(torch.ones(256, dtype=torch.float16, device="cuda"), p, s, c, 128, 256, group_size=128)
    torch.cuda.synchronize()
    assert q.device_error() == 0
    for c_ in comms:
        c_.close()
