"""Host-side mirror of the reference's TW-Marlin decode engine, over the C ABI.

Follows ``QuantizedGenerationEngine::forward_decode_tw_marlin_graph`` and
``generate_tw_marlin_graph`` (crates/kernels/src/generate.rs:2124-2211, 2412-2547): one decode
step is a fixed sequence of kernel launches on one stream, position and cache length live in
device buffers, the step is captured once and replayed.  Differences, all on the data side that
the benchmark configuration asks for: GEMM inputs/outputs, KV cache and LM head are FP16 (the
reference keeps everything F32, generate.rs:1382-1404, kv_cache.rs:76-99), the residual stream
stays F32, and greedy sampling stays on the device (the reference copies the logits to the host
every token, generate.rs:2531-2534).  torch supplies memory and the graph object only.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import _lib
from . import quantize as q
from ._lib import check


@dataclass
class TransformerConfig:
    """The fields of the reference's TransformerConfig that the decode path reads."""
    hidden: int = 3584
    num_heads: int = 28
    num_kv_heads: int = 4
    head_dim: int = 128
    ffn: int = 18944
    vocab: int = 152064
    layers: int = 28
    rope_theta: float = 1e6
    eps: float = 1e-6
    max_seq: int = 4096
    group_size: int = 128
    qkv_bias: bool = True

    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim


QWEN2_7B = TransformerConfig()


class Q4Model:
    """Random-initialised weights of the given shape in TW-Marlin form (quantised on the device),
    FP16 embedding / LM head, F32 norms and biases.  Seeds follow the benchmark plan:
    1000 * layer + projection id (0 q, 1 k, 2 v, 3 o, 4 gate, 5 up, 6 down)."""

    def __init__(self, cfg: TransformerConfig, device="cuda", seed: int = 0):
        self.cfg = cfg
        self.device = torch.device(device)
        g = cfg.group_size
        self.layers: List[q.TWMarlinWeights] = []

        def rand_w(k, n, sd):
            gen = torch.Generator(device=self.device).manual_seed(sd)
            return torch.randn((k, n), generator=gen, device=self.device, dtype=torch.float32) * 0.02

        for layer in range(cfg.layers):
            base = seed + 1000 * layer
            shapes = [(cfg.hidden, cfg.q_dim), (cfg.hidden, cfg.kv_dim), (cfg.hidden, cfg.kv_dim),
                      (cfg.q_dim, cfg.hidden), (cfg.hidden, cfg.ffn), (cfg.hidden, cfg.ffn), (cfg.ffn, cfg.hidden)]
            mats = []
            for pid, (k, n) in enumerate(shapes):
                w = rand_w(k, n, base + pid)
                mats.append(q.quantize_f32_to_tw_marlin(w, k, n, g))
                del w
            bias = None
            if cfg.qkv_bias:
                gen = torch.Generator(device=self.device).manual_seed(base + 500)
                bias = torch.randn(cfg.q_dim + 2 * cfg.kv_dim, generator=gen, device=self.device) * 0.02
            lw = q.TWMarlinWeights(
                hidden=cfg.hidden, kv_dim=cfg.kv_dim, ffn=cfg.ffn, group_size=g,
                attn_norm=torch.ones(cfg.hidden, device=self.device), ffn_norm=torch.ones(cfg.hidden, device=self.device),
                wq=mats[0], wk=mats[1], wv=mats[2], wo=mats[3], w_gate=mats[4], w_up=mats[5], w_down=mats[6])
            # fused QKV and gate+up (TWMarlinWeights::fuse_projections, quantize.rs:1138-1165)
            lw.wqkv = q.fuse_tw_marlin_n([lw.wq, lw.wk, lw.wv], cfg.hidden, [cfg.q_dim, cfg.kv_dim, cfg.kv_dim], g)
            lw.wgu = q.fuse_tw_marlin_n([lw.w_gate, lw.w_up], cfg.hidden, [cfg.ffn, cfg.ffn], g)
            lw.wq = lw.wk = lw.wv = lw.w_gate = lw.w_up = None          # only the fused tensors are kept
            lw.bqkv = bias
            self.layers.append(lw)
        gen = torch.Generator(device=self.device).manual_seed(seed + 900001)
        self.embed = (torch.randn((cfg.vocab, cfg.hidden), generator=gen, device=self.device) * 0.02).half()
        gen = torch.Generator(device=self.device).manual_seed(seed + 900002)
        self.lm_head = (torch.randn((cfg.vocab, cfg.hidden), generator=gen, device=self.device) * 0.02).half()
        self.lm_head_q4 = None          # (packed, scales) of the same matrix, made on demand
        self.final_norm = torch.ones(cfg.hidden, device=self.device)
        torch.cuda.synchronize(self.device)

    def quantize_lm_head(self):
        """The LM head as a TW-Marlin tensor ([vocab, hidden] is already the [N, K] form the quantiser
        takes), for forward_lm_head_tw_marlin (generate.rs:1750-1761)."""
        if self.lm_head_q4 is None:
            cfg = self.cfg
            self.lm_head_q4 = q.quantize_f32_to_tw_marlin(self.lm_head.float().contiguous(), cfg.hidden, cfg.vocab,
                                                          cfg.group_size, w_is_nk=True)
            torch.cuda.synchronize(self.device)
        return self.lm_head_q4


class Q4DecodeBuffers:
    """Every buffer one decode step touches, allocated once (Q4DecodeBuffers::allocate,
    generate.rs:1382-1416)."""

    def __init__(self, cfg: TransformerConfig, device):
        f16, f32, i32 = torch.float16, torch.float32, torch.int32
        dev = device
        self.x = torch.zeros(cfg.hidden, dtype=f32, device=dev)                  # residual stream
        self.normed = torch.zeros(cfg.hidden, dtype=f16, device=dev)
        self.qkv = torch.zeros(cfg.q_dim + 2 * cfg.kv_dim, dtype=f16, device=dev)
        self.rope_table = torch.zeros(cfg.head_dim, dtype=torch.float32, device=dev)      # cos | sin of the step's position
        self.attn = torch.zeros(cfg.q_dim, dtype=f16, device=dev)
        self.gate_up = torch.zeros(2 * cfg.ffn, dtype=f16, device=dev)
        self.logits = torch.zeros(cfg.vocab, dtype=f32, device=dev)
        self.token = torch.zeros(1, dtype=i32, device=dev)
        self.pos = torch.zeros(1, dtype=i32, device=dev)                          # pos_buf (generate.rs:1413)
        self.cache_len = torch.zeros(1, dtype=i32, device=dev)                    # cache_len_buf (generate.rs:1415)
        self.step = torch.zeros(1, dtype=i32, device=dev)
        self.history = torch.zeros(cfg.max_seq, dtype=i32, device=dev)
        self.k_cache = [torch.zeros((cfg.max_seq, cfg.kv_dim), dtype=f16, device=dev) for _ in range(cfg.layers)]
        self.v_cache = [torch.zeros((cfg.max_seq, cfg.kv_dim), dtype=f16, device=dev) for _ in range(cfg.layers)]
        lib = _lib.lib()
        self.attn_scratch = torch.zeros(lib.twm_attn_scratch_bytes(1, cfg.num_heads, cfg.head_dim, cfg.max_seq),
                                        dtype=torch.uint8, device=dev)
        self.argmax_scratch = torch.zeros(lib.twm_argmax_scratch_bytes(), dtype=torch.uint8, device=dev)
        shapes = [(1, cfg.q_dim + 2 * cfg.kv_dim, cfg.hidden, cfg.group_size), (1, cfg.hidden, cfg.q_dim, cfg.group_size),
                  (1, 2 * cfg.ffn, cfg.hidden, cfg.group_size), (1, cfg.hidden, cfg.ffn, cfg.group_size)]
        self.workspace = q.Workspace.for_shapes(shapes, dev)


class QuantizedGenerationEngine:
    """Decode engine on TW-Marlin weights (generate.rs:1191-2547, Q4 + marlin + graph path)."""

    def __init__(self, model: Q4Model, use_pdl: bool = True, q4_lm_head: bool = False):
        self.model = model
        # the reference's graph path keeps the LM head outside the graph in FP32/FP16 (generate.rs:2530-2534)
        # and has a Q4 one as an option (forward_lm_head_tw_marlin, generate.rs:1750-1761): same here
        self.q4_lm_head = q4_lm_head
        if q4_lm_head:
            model.quantize_lm_head()
        self.cfg = model.cfg
        self.buf = Q4DecodeBuffers(model.cfg, model.device)
        self.flags = _lib.TWM_FLAG_PDL if use_pdl else 0
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.stream = torch.cuda.Stream(model.device)
        self.launches_per_step = 0

    # ------------------------------------------------------------------ state --
    def prefill_random_kv(self, length: int, seed: int = 2) -> None:
        """KV cache holding `length` tokens of FP16 N(0,1) (the benchmark's stand-in for a prefill)."""
        gen = torch.Generator(device=self.model.device).manual_seed(seed)
        for kc, vc in zip(self.buf.k_cache, self.buf.v_cache):
            kc[:length] = torch.randn((length, self.cfg.kv_dim), generator=gen, device=self.model.device).half()
            vc[:length] = torch.randn((length, self.cfg.kv_dim), generator=gen, device=self.model.device).half()
        self.set_position(length)

    def set_position(self, pos: int) -> None:
        self.buf.pos.fill_(pos)
        self.buf.cache_len.fill_(pos + 1)       # the step appends one token before attending
        torch.cuda.synchronize(self.model.device)

    def set_token(self, token: int) -> None:
        self.buf.token.fill_(int(token))

    def reset_history(self) -> None:
        """Start the generated-token list over (the step counter indexes it)."""
        self.buf.step.zero_()

    # ------------------------------------------------------------------- step --
    def _step_ops(self, stream_ptr: int):
        """One decode step as an ordered list of (category, launches, enqueue) triples: the launch
        order of generate.rs:2149-2206 with the split/add passes folded into their neighbours.  The
        categories are the rows of the reference's profile table (generate.rs:2380-2396)."""
        lib, cfg, b, fl = _lib.lib(), self.cfg, self.buf, self.flags
        ops = []

        pending = []         # the Q4 GEMMs' arguments in launch order: each one names its successor

        def gemm(a, w, c, n_out, k_in, accumulate=False, silu_mul=False):
            args = _lib.GemmArgs(M=1, N=n_out, K=k_in, group_size=cfg.group_size, a_dtype=_lib.TWM_F16,
                                 c_dtype=_lib.TWM_F32 if c.dtype == torch.float32 else _lib.TWM_F16,
                                 a=a.data_ptr(), lda=2 * k_in if silu_mul else k_in, packed=w[0].data_ptr(),
                                 scales=w[1].data_ptr(), c=c.data_ptr(), ldc=n_out, workspace=b.workspace.ptr,
                                 workspace_bytes=b.workspace.nbytes,
                                 flags=fl | (_lib.TWM_FLAG_ACCUMULATE if accumulate else 0),
                                 a_prologue=_lib.TWM_A_SILU_MUL if silu_mul else _lib.TWM_A_PLAIN)
            if pending:      # the GEMM before this one pulls the head of these weights into L2 while it drains
                pending[-1].next = C.addressof(args)
            pending.append(args)
            return lambda: check(lib.twm_gemm_w4a16(C.byref(args), stream_ptr), "twm_gemm_w4a16")

        # cos/sin of this step's position, once for all layers
        ops.append(("rope_table", 1, lambda: check(lib.twm_rope_table(b.rope_table.data_ptr(), b.pos.data_ptr(), cfg.head_dim,
                                                                      cfg.rope_theta, fl, stream_ptr), "twm_rope_table")))
        ops.append(("embedding", 1, lambda: check(lib.twm_embed(b.x.data_ptr(), self.model.embed.data_ptr(), b.token.data_ptr(),
                                                                 1, cfg.hidden, fl, stream_ptr), "twm_embed")))
        for li, lw in enumerate(self.model.layers):
            ops.append(("attn_rmsnorm", 1, lambda lw=lw: check(lib.twm_rmsnorm(
                b.normed.data_ptr(), b.x.data_ptr(), lw.attn_norm.data_ptr(), 1, cfg.hidden, cfg.eps, fl, stream_ptr), "twm_rmsnorm")))
            ops.append(("qkv_gemm", 1, gemm(b.normed, lw.wqkv, b.qkv, cfg.q_dim + 2 * cfg.kv_dim, cfg.hidden)))
            # bias + RoPE on q and k, the KV append and the attention itself: the attention kernel takes the fused
            # QKV output (fused_bias_rope_append_device_pos + decode_attention_flash_device_len, generate.rs:2164-2178)
            ops.append(("attention", 2, lambda li=li, lw=lw: check(lib.twm_attn_decode_rope(
                b.attn.data_ptr(), b.qkv.data_ptr(), lw.bqkv.data_ptr() if lw.bqkv is not None else None,
                b.rope_table.data_ptr(), b.k_cache[li].data_ptr(), b.v_cache[li].data_ptr(), 1, cfg.num_heads,
                cfg.num_kv_heads, cfg.head_dim, b.pos.data_ptr(), b.cache_len.data_ptr(), cfg.max_seq,
                b.attn_scratch.data_ptr(), b.attn_scratch.numel(), fl, stream_ptr), "twm_attn_decode_rope")))
            ops.append(("out_gemm", 1, gemm(b.attn, lw.wo, b.x, cfg.hidden, cfg.q_dim, accumulate=True)))          # x += o(attn)
            ops.append(("ffn_rmsnorm", 1, lambda lw=lw: check(lib.twm_rmsnorm(
                b.normed.data_ptr(), b.x.data_ptr(), lw.ffn_norm.data_ptr(), 1, cfg.hidden, cfg.eps, fl, stream_ptr), "twm_rmsnorm")))
            ops.append(("gate_up_gemm", 1, gemm(b.normed, lw.wgu, b.gate_up, 2 * cfg.ffn, cfg.hidden)))
            # x += down(silu(gate) * up): the gated activation (fused_silu_mul, ops.rs:966-977) is taken on the fly by
            # the down GEMM's activation reader, bit for bit what the separate pass stored
            ops.append(("down_gemm", 1, gemm(b.gate_up, lw.w_down, b.x, cfg.hidden, cfg.ffn, accumulate=True, silu_mul=True)))
        ops.append(("final_rmsnorm", 1, lambda: check(lib.twm_rmsnorm(b.normed.data_ptr(), b.x.data_ptr(),
                                                                      self.model.final_norm.data_ptr(), 1, cfg.hidden, cfg.eps,
                                                                      fl, stream_ptr), "twm_rmsnorm")))
        if self.q4_lm_head:
            ops.append(("lm_head", 1, gemm(b.normed, self.model.lm_head_q4, b.logits, cfg.vocab, cfg.hidden)))
        else:
            ops.append(("lm_head", 1, lambda: check(lib.twm_lm_head(b.logits.data_ptr(), b.normed.data_ptr(),
                                                                    self.model.lm_head.data_ptr(), cfg.hidden, cfg.vocab, fl,
                                                                    stream_ptr), "twm_lm_head")))
        ops.append(("argmax_advance", 2, lambda: check(lib.twm_argmax_advance(
            b.token.data_ptr(), b.history.data_ptr(), b.history.numel(), b.pos.data_ptr(), b.cache_len.data_ptr(),
            b.step.data_ptr(), b.logits.data_ptr(), cfg.vocab, b.argmax_scratch.data_ptr(), b.argmax_scratch.numel(), fl,
            stream_ptr), "twm_argmax_advance")))
        if len(pending) > 1:
            pending[-1].next = C.addressof(pending[0])       # the next token's first GEMM
        return ops

    def forward_decode_tw_marlin_graph(self, stream_ptr: int) -> int:
        """Enqueue one decode step (embedding .. arg-max) on the stream; returns the number of
        kernel launches (forward_decode_tw_marlin_graph, generate.rs:2124-2211)."""
        n = 0
        for _, launches, enqueue in self._step_ops(stream_ptr):
            enqueue()
            n += launches
        self.launches_per_step = n
        return n

    def profile_decode_tw_marlin(self, steps: int = 3) -> dict:
        """Per-operation time of a decode step (profile_decode_tw_marlin, generate.rs:2216-2408): every
        operation of `steps` eager steps is bracketed by CUDA events on the engine's stream (the
        reference brackets with host synchronisations, which also counts launch latency).  Returns
        {"ops": {category: {"us", "us_per_layer", "pct"}}, "total_us", "gemm_us", "non_gemm_us",
        "embed_us"} per step.  Position and cache length are put back afterwards."""
        b = self.buf
        saved = (b.pos.clone(), b.cache_len.clone(), b.step.clone(), b.token.clone())
        acc: dict = {}
        with torch.cuda.stream(self.stream):
            self.forward_decode_tw_marlin_graph(self.stream.cuda_stream)          # warm
            for _ in range(steps):
                events = []
                for cat, _, enqueue in self._step_ops(self.stream.cuda_stream):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(self.stream)
                    enqueue()
                    e1.record(self.stream)
                    events.append((cat, e0, e1))
                torch.cuda.synchronize()
                for cat, e0, e1 in events:
                    acc[cat] = acc.get(cat, 0.0) + e0.elapsed_time(e1) * 1e3
            b.pos.copy_(saved[0]); b.cache_len.copy_(saved[1]); b.step.copy_(saved[2]); b.token.copy_(saved[3])
            torch.cuda.synchronize()
        per_step = {k: v / steps for k, v in acc.items()}
        total = sum(per_step.values())
        layered = {"attn_rmsnorm", "qkv_gemm", "attention", "out_gemm", "ffn_rmsnorm", "gate_up_gemm", "down_gemm"}
        nl = max(len(self.model.layers), 1)
        table = {k: {"us": round(v, 1), "us_per_layer": round(v / nl, 2) if k in layered else None,
                     "pct": round(100.0 * v / total, 1)} for k, v in per_step.items()}
        gemm_us = sum(v for k, v in per_step.items() if k.endswith("_gemm"))
        return {"ops": table, "total_us": round(total, 1), "gemm_us": round(gemm_us, 1),
                "non_gemm_us": round(total - gemm_us - per_step.get("embedding", 0.0), 1),
                "embed_us": round(per_step.get("embedding", 0.0), 1)}

    def step_eager(self) -> None:
        with torch.cuda.stream(self.stream):
            self.forward_decode_tw_marlin_graph(self.stream.cuda_stream)

    def capture(self) -> None:
        """Capture one step (GraphCapture::record_with_device, cuda_graph.rs:85-111).  One eager
        step runs first (it initialises per-device state), then its effects on the position
        buffers and the cache are undone, as the reference does (generate.rs:2491-2500)."""
        b = self.buf
        saved = (b.pos.clone(), b.cache_len.clone(), b.step.clone(), b.token.clone())
        with torch.cuda.stream(self.stream):
            self.forward_decode_tw_marlin_graph(self.stream.cuda_stream)
            torch.cuda.synchronize()
            b.pos.copy_(saved[0]); b.cache_len.copy_(saved[1]); b.step.copy_(saved[2]); b.token.copy_(saved[3])
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                self.forward_decode_tw_marlin_graph(self.stream.cuda_stream)
        torch.cuda.synchronize()

    def replay(self) -> None:
        self.graph.replay()

    def generate_tw_marlin_graph(self, first_token: int, max_tokens: int) -> List[int]:
        """Greedy decode `max_tokens` tokens from `first_token` by replaying the captured step
        (generate.rs:2512-2536 without the per-token host round trip)."""
        if self.graph is None:
            self.capture()
        self.set_token(first_token)
        start = int(self.buf.step.item())
        pos = int(self.buf.pos.item())
        if pos + max_tokens > self.cfg.max_seq:
            raise _lib.TwmError(_lib.TWM_EINVAL, f"generate_tw_marlin_graph: position {pos} + {max_tokens} tokens runs past "
                                                 f"the cache (max_seq {self.cfg.max_seq})")
        if start + max_tokens > self.buf.history.numel():
            raise _lib.TwmError(_lib.TWM_EINVAL, f"generate_tw_marlin_graph: {start} + {max_tokens} tokens do not fit the "
                                                 f"token list ({self.buf.history.numel()} entries); reset_history() first")
        for _ in range(max_tokens):
            self.graph.replay()
        torch.cuda.synchronize()
        return self.buf.history[start:start + max_tokens].tolist()
