"""GPU tests of the decode step built from the W4A16 GEMMs and their neighbour kernels, against
the CPU restatement in oracle/decode_ref.py (teacher-forced logits), plus the reference's own
self-consistency checks: graph replay == eager launches, two runs identical
(crates/kernels/src/generate.rs:3811-3841, 3667-3723)."""
import numpy as np
import pytest
import torch

import oracle
from oracle import decode_ref
from tensorwarp_b200 import generate as gen
from tensorwarp_b200 import _lib
from tensorwarp_b200 import quantize as q

pytestmark = pytest.mark.gpu

SMALL = gen.TransformerConfig(hidden=256, num_heads=2, num_kv_heads=1, head_dim=128, ffn=512, vocab=1024, layers=2,
                              rope_theta=1e6, eps=1e-6, max_seq=512, group_size=128, qkv_bias=True)
GQA = gen.TransformerConfig(hidden=512, num_heads=8, num_kv_heads=2, head_dim=128, ffn=1024, vocab=2000, layers=2,
                            rope_theta=1e4, eps=1e-5, max_seq=384, group_size=32, qkv_bias=False)


def _dense_provider(model):
    """Dequantised weights for the oracle, from the packed tensors through the CPU oracle's decode."""
    cfg = model.cfg
    cache = {}

    def dq(w, k, n):
        p = w[0].cpu().numpy()
        s = w[1].cpu().numpy().view(np.uint16)
        return oracle.dequant_f32(p, s, k, n, cfg.group_size)

    def dense(li, name):
        key = (li, name)
        if key in cache:
            return cache[key]
        if li == -1:
            if name == "embed_row":
                val = lambda tok: model.embed[int(tok)].float().cpu().numpy()      # one row at a time: the table is large
            elif name == "final_norm":
                val = model.final_norm.cpu().numpy()
            else:
                val = model.lm_head.float().cpu().numpy()
        else:
            lw = model.layers[li]
            if name == "qkv":
                val = dq(lw.wqkv, cfg.hidden, cfg.q_dim + 2 * cfg.kv_dim)
            elif name == "o":
                val = dq(lw.wo, cfg.q_dim, cfg.hidden)
            elif name == "gu":
                val = dq(lw.wgu, cfg.hidden, 2 * cfg.ffn)
            elif name == "down":
                val = dq(lw.w_down, cfg.ffn, cfg.hidden)
            elif name == "attn_norm":
                val = lw.attn_norm.cpu().numpy()
            elif name == "ffn_norm":
                val = lw.ffn_norm.cpu().numpy()
            else:
                val = lw.bqkv.cpu().numpy() if lw.bqkv is not None else None
        cache[key] = val
        return val

    return dense


@pytest.mark.parametrize("cfg,prefill", [(SMALL, 100), (GQA, 200), (SMALL, 0)])
def test_teacher_forced_logits_match_oracle(cfg, prefill):
    model = gen.Q4Model(cfg, seed=5)
    eng = gen.QuantizedGenerationEngine(model)
    if prefill:
        eng.prefill_random_kv(prefill, seed=2)
    else:
        eng.set_position(0)
    kc = [c.float().cpu().numpy().copy() for c in eng.buf.k_cache]
    vc = [c.float().cpu().numpy().copy() for c in eng.buf.v_cache]
    dense = _dense_provider(model)
    tokens = torch.randint(0, cfg.vocab, (5,), generator=torch.Generator().manual_seed(3)).tolist()
    greedy_agree = 0
    for i, tok in enumerate(tokens):
        eng.set_token(tok)
        eng.step_eager()
        torch.cuda.synchronize()
        logits = eng.buf.logits.cpu().numpy()
        ref = decode_ref.decode_step(cfg, dense, tok, prefill + i, kc, vc)
        rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
        err = float(np.max(np.abs(logits - ref))) / rms
        assert err < 1e-2, (i, err)
        greedy_agree += int(int(eng.buf.token.item()) == int(np.argmax(ref)))
        # the appended cache rows are the oracle's, to FP16 rounding of one unit in the last place
        for li in range(cfg.layers):
            kg = eng.buf.k_cache[li][prefill + i].float().cpu().numpy()
            assert np.max(np.abs(kg - kc[li][prefill + i])) <= 2e-3 * max(1.0, float(np.abs(kc[li][prefill + i]).max()))
    assert int(eng.buf.pos.item()) == prefill + len(tokens)
    assert int(eng.buf.cache_len.item()) == prefill + len(tokens) + 1
    assert greedy_agree >= len(tokens) - 1          # near-flat random logits: one near-tie may flip
    assert q.device_error() == 0


def test_config3_dimensions_two_layers_teacher_forced():
    """configs[3] at its own shape: Qwen2-7B dimensions (hidden 3584, 28 query / 4 KV heads of 128, ffn
    18944, vocabulary 152064, QKV bias), KV cache prefilled to 2048 tokens, FP16 LM head; two of the 28
    layers (the oracle's dense FP32 copy of one layer is 0.9 GB), two teacher-forced steps."""
    cfg = gen.TransformerConfig(hidden=3584, num_heads=28, num_kv_heads=4, head_dim=128, ffn=18944, vocab=152064, layers=2,
                                rope_theta=1e6, eps=1e-6, max_seq=2304, group_size=128, qkv_bias=True)
    prefill = 2048
    model = gen.Q4Model(cfg, seed=0)
    eng = gen.QuantizedGenerationEngine(model)
    eng.prefill_random_kv(prefill, seed=2)
    kc = [c.float().cpu().numpy().copy() for c in eng.buf.k_cache]
    vc = [c.float().cpu().numpy().copy() for c in eng.buf.v_cache]
    dense = _dense_provider(model)
    tokens = torch.randint(0, cfg.vocab, (2,), generator=torch.Generator().manual_seed(3)).tolist()
    for i, tok in enumerate(tokens):
        eng.set_token(tok)
        eng.step_eager()
        torch.cuda.synchronize()
        logits = eng.buf.logits.cpu().numpy()
        ref = decode_ref.decode_step(cfg, dense, tok, prefill + i, kc, vc)
        rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
        err = float(np.max(np.abs(logits - ref))) / rms
        assert err < 1e-2, (i, err)
        # the greedy token is the oracle's, or a near-tie of it (random-init logits are nearly flat)
        tok_gpu = int(eng.buf.token.item())
        assert 0 <= tok_gpu < cfg.vocab
        assert ref[tok_gpu] >= float(ref.max()) - 1e-2 * rms
        for li in range(cfg.layers):
            kg = eng.buf.k_cache[li][prefill + i].float().cpu().numpy()
            assert np.max(np.abs(kg - kc[li][prefill + i])) <= 2e-3 * max(1.0, float(np.abs(kc[li][prefill + i]).max()))
    assert int(eng.buf.cache_len.item()) == prefill + len(tokens) + 1
    assert q.device_error() == 0
    # the same two steps as a captured graph, with the Q4 LM head option: tokens stay inside the vocabulary
    eng2 = gen.QuantizedGenerationEngine(model, q4_lm_head=True)
    eng2.prefill_random_kv(prefill, seed=2)
    toks = eng2.generate_tw_marlin_graph(tokens[0], 2)
    assert all(0 <= t < cfg.vocab for t in toks)
    assert q.device_error() == 0


def test_generate_refuses_to_run_past_the_cache_or_the_token_list():
    """The host checks the bounds the device buffers have (max_seq rows of cache, max_seq token slots);
    at the last position one more token is still fine."""
    cfg = SMALL
    model = gen.Q4Model(cfg, seed=3)
    eng = gen.QuantizedGenerationEngine(model)
    eng.prefill_random_kv(cfg.max_seq - 1, seed=2)
    toks = eng.generate_tw_marlin_graph(1, 1)            # writes row max_seq - 1: the last one
    assert len(toks) == 1 and 0 <= toks[0] < cfg.vocab
    with pytest.raises(_lib.TwmError):
        eng.generate_tw_marlin_graph(1, 1)               # the cache is full now
    eng.prefill_random_kv(10, seed=2)
    eng.buf.step.fill_(cfg.max_seq - 2)
    with pytest.raises(_lib.TwmError):
        eng.generate_tw_marlin_graph(1, 5)               # the token list would overflow
    eng.reset_history()
    assert len(eng.generate_tw_marlin_graph(1, 5)) == 5
    # a replay past the list's end does not write past it (the device-side guard)
    eng.buf.step.fill_(cfg.max_seq)
    guard = eng.buf.history.clone()
    eng.replay()
    torch.cuda.synchronize()
    assert torch.equal(eng.buf.history, guard)
    assert q.device_error() == 0


def test_argmax_of_all_nan_logits_is_token_zero():
    lib = _lib.lib()
    n = 5000
    logits = torch.full((n,), float("nan"), device="cuda")
    tok = torch.full((1,), -5, dtype=torch.int32, device="cuda")
    hist = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    pos, ln, step = (torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(3))
    scratch = torch.zeros(lib.twm_argmax_scratch_bytes(), dtype=torch.uint8, device="cuda")
    _lib.check(lib.twm_argmax_advance(tok.data_ptr(), hist.data_ptr(), 4, pos.data_ptr(), ln.data_ptr(), step.data_ptr(),
                                      logits.data_ptr(), n, scratch.data_ptr(), scratch.numel(), 0,
                                      torch.cuda.current_stream().cuda_stream), "twm_argmax_advance")
    torch.cuda.synchronize()
    assert int(tok.item()) == 0 and hist.tolist() == [0, -1, -1, -1] and int(step.item()) == 1


def test_graph_replay_equals_eager_and_is_deterministic():
    cfg = SMALL
    model = gen.Q4Model(cfg, seed=7)
    runs = []
    for mode in ("eager", "graph", "graph"):
        eng = gen.QuantizedGenerationEngine(model)
        eng.prefill_random_kv(64, seed=2)
        if mode == "eager":
            eng.set_token(17)
            for _ in range(12):
                eng.step_eager()
            torch.cuda.synchronize()
            toks = eng.buf.history[:12].tolist()
        else:
            toks = eng.generate_tw_marlin_graph(17, 12)
        assert all(0 <= t < cfg.vocab for t in toks)
        runs.append(toks)
    assert runs[0] == runs[1] == runs[2]
    assert q.device_error() == 0


def test_without_programmatic_launch_same_tokens():
    cfg = GQA
    model = gen.Q4Model(cfg, seed=9)
    outs = []
    for pdl in (True, False):
        eng = gen.QuantizedGenerationEngine(model, use_pdl=pdl)
        eng.prefill_random_kv(130, seed=2)
        outs.append(eng.generate_tw_marlin_graph(3, 8))
    assert outs[0] == outs[1]


@pytest.mark.parametrize("length", [1, 31, 500, 2049])
@pytest.mark.parametrize("heads,kv_heads,rows", [(28, 4, 1), (8, 8, 2), (16, 2, 3), (28, 4, 3)])
def test_attention_against_float64(length, heads, kv_heads, rows):
    """twm_attn_decode (split-KV chunk kernel + merge kernel) with two cache capacities (the grid
    covers the capacity, the length comes from the device) against a float64 soft-max attention
    on the same cache contents.  The large capacity with several sequences makes the CTAs walk
    several chunks, which runs the tensor-core form of the pass (groups of 1, 7 and 8 q heads)."""
    lib = _lib.lib()
    hd = 128
    g = torch.Generator(device="cuda").manual_seed(length * 31 + heads)
    qv = torch.randn((rows, heads * hd), generator=g, device="cuda").half()
    kv_dim = kv_heads * hd
    kc = torch.randn((rows, length, kv_dim), generator=g, device="cuda").half()
    vc = torch.randn((rows, length, kv_dim), generator=g, device="cuda").half()
    len_buf = torch.tensor([length], dtype=torch.int32, device="cuda")
    outs = []
    for max_seq in (max(length, 2100), 9000):
        k_cache = torch.zeros((rows, max_seq, kv_dim), dtype=torch.float16, device="cuda")
        v_cache = torch.zeros_like(k_cache)
        k_cache[:, :length] = kc
        v_cache[:, :length] = vc
        out = torch.full((rows, heads * hd), float("nan"), dtype=torch.float16, device="cuda")
        scratch = torch.zeros(lib.twm_attn_scratch_bytes(rows, heads, hd, max_seq), dtype=torch.uint8, device="cuda")
        _lib.check(lib.twm_attn_decode(out.data_ptr(), qv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), rows, heads,
                                       kv_heads, hd, len_buf.data_ptr(), max_seq, scratch.data_ptr(), scratch.numel(), 0,
                                       torch.cuda.current_stream().cuda_stream), "twm_attn_decode")
        torch.cuda.synchronize()
        outs.append(out.float().cpu().numpy())
    qn = qv.float().cpu().numpy().astype(np.float64).reshape(rows, heads, hd)
    kn = kc.float().cpu().numpy().astype(np.float64).reshape(rows, length, kv_heads, hd)
    vn = vc.float().cpu().numpy().astype(np.float64).reshape(rows, length, kv_heads, hd)
    group = heads // kv_heads
    ref = np.zeros((rows, heads, hd))
    for r in range(rows):
        for h in range(heads):
            s = kn[r, :, h // group] @ qn[r, h] / np.sqrt(hd)
            p = np.exp(s - s.max())
            ref[r, h] = (p / p.sum()) @ vn[r, :, h // group]
    ref = ref.reshape(rows, heads * hd)
    for o in outs:
        assert np.max(np.abs(o - ref)) < 4e-3          # FP16 output of values of order one
    assert np.max(np.abs(outs[0] - outs[1])) < 2e-3
    assert q.device_error() == 0


@pytest.mark.parametrize("pos,max_seq", [(0, 512), (31, 512), (32, 512), (100, 512), (511, 512), (4000, 9000), (4031, 9000)])
@pytest.mark.parametrize("heads,kv_heads,rows,with_bias", [(28, 4, 1, True), (8, 8, 2, False), (16, 2, 3, True), (28, 4, 3, False)])
def test_attention_with_fused_rope_equals_the_two_passes(pos, max_seq, heads, kv_heads, rows, with_bias):
    """twm_rope_table + twm_attn_decode_rope against twm_rope_append + twm_attn_decode on the same
    fused QKV rows: the attention output and both caches bit for bit (position at the start, at the
    end and in the middle of a 32-token chunk, at the end of the cache, with the length covering the
    new token and one token short of it; the large cache makes each CTA walk several chunks)."""
    lib = _lib.lib()
    hd, base = 128, 1e6
    kv_dim = kv_heads * hd
    g = torch.Generator(device="cuda").manual_seed(pos * 7 + heads)
    qkv = torch.randn((rows, (heads + 2 * kv_heads) * hd), generator=g, device="cuda").half()
    bias = torch.randn((heads + 2 * kv_heads) * hd, generator=g, device="cuda") if with_bias else None
    k0 = torch.randn((rows, max_seq, kv_dim), generator=g, device="cuda").half()
    v0 = torch.randn((rows, max_seq, kv_dim), generator=g, device="cuda").half()
    pos_buf = torch.tensor([pos], dtype=torch.int32, device="cuda")
    sp = torch.cuda.current_stream().cuda_stream
    bias_ptr = bias.data_ptr() if bias is not None else None
    for length in (pos + 1, pos):
        if length < 1:
            continue
        len_buf = torch.tensor([length], dtype=torch.int32, device="cuda")
        scratch = torch.zeros(lib.twm_attn_scratch_bytes(rows, heads, hd, max_seq), dtype=torch.uint8, device="cuda")
        # two passes
        ka, va = k0.clone(), v0.clone()
        qa = torch.zeros((rows, heads * hd), dtype=torch.float16, device="cuda")
        out_a = torch.full((rows, heads * hd), float("nan"), dtype=torch.float16, device="cuda")
        _lib.check(lib.twm_rope_append(qa.data_ptr(), ka.data_ptr(), va.data_ptr(), qkv.data_ptr(), bias_ptr, rows, heads,
                                       kv_heads, hd, pos_buf.data_ptr(), max_seq, base, 0, sp), "twm_rope_append")
        _lib.check(lib.twm_attn_decode(out_a.data_ptr(), qa.data_ptr(), ka.data_ptr(), va.data_ptr(), rows, heads, kv_heads, hd,
                                       len_buf.data_ptr(), max_seq, scratch.data_ptr(), scratch.numel(), 0, sp), "twm_attn_decode")
        # one pass
        kb, vb = k0.clone(), v0.clone()
        table = torch.zeros(hd, dtype=torch.float32, device="cuda")
        out_b = torch.full((rows, heads * hd), float("nan"), dtype=torch.float16, device="cuda")
        _lib.check(lib.twm_rope_table(table.data_ptr(), pos_buf.data_ptr(), hd, base, _lib.TWM_FLAG_PDL, sp), "twm_rope_table")
        _lib.check(lib.twm_attn_decode_rope(out_b.data_ptr(), qkv.data_ptr(), bias_ptr, table.data_ptr(), kb.data_ptr(),
                                            vb.data_ptr(), rows, heads, kv_heads, hd, pos_buf.data_ptr(), len_buf.data_ptr(),
                                            max_seq, scratch.data_ptr(), scratch.numel(), _lib.TWM_FLAG_PDL, sp),
                   "twm_attn_decode_rope")
        torch.cuda.synchronize()
        assert torch.equal(ka, kb) and torch.equal(va, vb)
        assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16))
        assert not torch.equal(ka, k0)                       # the row was appended
    assert q.device_error() == 0


def test_q4_lm_head_option():
    """The LM head as a TW-Marlin GEMM inside the step (forward_lm_head_tw_marlin,
    generate.rs:1750-1761): logits equal the oracle's W4A16 product of the step's final normed
    activations, and the rest of the step is the one the FP16 head sees."""
    cfg = GQA
    model = gen.Q4Model(cfg, seed=11)
    engs = []
    for q4 in (False, True):
        eng = gen.QuantizedGenerationEngine(model, q4_lm_head=q4)
        eng.prefill_random_kv(70, seed=2)
        eng.set_token(5)
        eng.step_eager()
        torch.cuda.synchronize()
        engs.append(eng)
    assert torch.equal(engs[0].buf.normed, engs[1].buf.normed)
    packed, scales = model.lm_head_q4
    normed = engs[1].buf.normed.float().cpu().numpy()[None]
    ref = oracle.w4a16_f64(normed, packed.cpu().numpy(), scales.cpu().numpy().view(np.uint16), 1, cfg.vocab, cfg.hidden,
                           cfg.group_size)
    got = engs[1].buf.logits.cpu().numpy()[None]
    rms = float(np.sqrt(np.mean(ref ** 2)))
    assert float(np.max(np.abs(got - ref))) < 1e-3 * rms
    # the quantised head stays close to the FP16 one (4-bit weights: a few per cent of the logit RMS)
    fp16 = engs[0].buf.logits.cpu().numpy()[None]
    assert float(np.sqrt(np.mean((got - fp16) ** 2))) < 0.2 * float(np.sqrt(np.mean(fp16 ** 2)))
    assert engs[0].launches_per_step == engs[1].launches_per_step
    assert q.device_error() == 0
