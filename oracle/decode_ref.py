"""CPU restatement of one Q4 decode step (TEST INFRASTRUCTURE ONLY).

Restates forward_decode_tw_marlin_graph (crates/kernels/src/generate.rs:2124-2211) and the
kernels it launches — RMSNorm (ops.rs:302-336), bias + rotate-half RoPE + KV append
(ops.rs:2601-2650), decode attention with 1/sqrt(d) scaling and grouped-query heads
(kv_cache.rs:951-1076), SwiGLU (ops.rs:966-977), LM head (generate.rs:1727-1735) — in numpy
float32, with the storage roundings of the configuration under test: GEMM inputs/outputs, KV
cache and LM-head weights are FP16, the residual stream is FP32.  Weights arrive dequantised
(w = f32(scale) * (nibble - 8), exact), so this file holds no quantisation logic.
"""
from __future__ import annotations

import numpy as np


def _f16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def rmsnorm(x, gamma, eps):
    x = x.astype(np.float32)
    rms = np.float32(1.0) / np.sqrt(np.mean(x * x, dtype=np.float32) + np.float32(eps), dtype=np.float32)
    return _f16(x * rms * gamma.astype(np.float32))


def rope(vec, pos, head_dim, theta):
    """vec: [heads*head_dim]; rotate-half pairs (i, i + head_dim/2); freq = 1/theta^(2i/head_dim)."""
    half = head_dim // 2
    v = vec.reshape(-1, head_dim).astype(np.float32)
    pair = np.arange(half, dtype=np.float32)
    freq = np.float32(1.0) / np.power(np.float32(theta), np.float32(2.0) * pair / np.float32(head_dim), dtype=np.float32)
    ang = np.float32(pos) * freq
    c, s = np.cos(ang, dtype=np.float32), np.sin(ang, dtype=np.float32)
    x0, x1 = v[:, :half], v[:, half:]
    out = np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c], axis=1)
    return out.reshape(-1)


def decode_step(cfg, dense, token, pos, k_cache, v_cache):
    """One step.  `dense(layer, name)` returns the dequantised f32 [K,N] matrix for name in
    {"qkv","o","gu","down"}, the f32 vector for {"attn_norm","ffn_norm","bias"} (bias may be None),
    and for layer = -1: "embed_row" (callable token -> f32 [hidden]), "final_norm", "lm_head"
    (f32 [vocab, hidden]).  k_cache/v_cache: lists of f32 arrays [max_seq, kv_dim], updated in place
    at `pos`.  Returns the logits (f32 [vocab])."""
    h, hd = cfg.hidden, cfg.head_dim
    q_dim, kv_dim = cfg.num_heads * hd, cfg.num_kv_heads * hd
    group = cfg.num_heads // cfg.num_kv_heads
    x = dense(-1, "embed_row")(token).astype(np.float32)
    for li in range(cfg.layers):
        xn = rmsnorm(x, dense(li, "attn_norm"), cfg.eps)
        qkv = _f16(xn @ dense(li, "qkv"))
        bias = dense(li, "bias")
        if bias is not None:
            qkv_b = qkv + bias.astype(np.float32)
        else:
            qkv_b = qkv
        q = _f16(rope(qkv_b[:q_dim], pos, hd, cfg.rope_theta))
        k_cache[li][pos] = _f16(rope(qkv_b[q_dim:q_dim + kv_dim], pos, hd, cfg.rope_theta))
        v_cache[li][pos] = _f16(qkv_b[q_dim + kv_dim:])
        length = pos + 1
        attn = np.zeros(q_dim, dtype=np.float32)
        scale = np.float32(1.0 / np.sqrt(hd))
        for head in range(cfg.num_heads):
            kvh = head // group
            kk = k_cache[li][:length, kvh * hd:(kvh + 1) * hd]
            vv = v_cache[li][:length, kvh * hd:(kvh + 1) * hd]
            s = (kk @ (q[head * hd:(head + 1) * hd] * scale)).astype(np.float32)
            p = np.exp(s - s.max(), dtype=np.float32)
            attn[head * hd:(head + 1) * hd] = (p @ vv) / p.sum(dtype=np.float32)
        attn = _f16(attn)
        x = x + (attn @ dense(li, "o")).astype(np.float32)
        xn = rmsnorm(x, dense(li, "ffn_norm"), cfg.eps)
        gu = _f16(xn @ dense(li, "gu"))
        g, u = gu[:cfg.ffn], gu[cfg.ffn:]
        act = _f16(g / (np.float32(1.0) + np.exp(-g, dtype=np.float32)) * u)
        x = x + (act @ dense(li, "down")).astype(np.float32)
    xn = rmsnorm(x, dense(-1, "final_norm"), cfg.eps)
    return (dense(-1, "lm_head") @ xn).astype(np.float32)
