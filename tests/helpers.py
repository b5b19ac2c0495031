"""Shared pieces of the parity tests: seeded inputs and the error criterion."""
from __future__ import annotations

import numpy as np


def seeded_weights(k: int, n: int, seed: int, std: float = 0.02) -> np.ndarray:
    """[K,N] f32 ~ N(0, std^2): the synthetic weights the benchmark configs name."""
    return (np.random.default_rng(seed).standard_normal((k, n), dtype=np.float32) * np.float32(std))


def seeded_activations(m: int, k: int, seed: int = 0) -> np.ndarray:
    """[M,K] ~ N(0,1), rounded to fp16 and widened back (so f16 and f32 paths see the same numbers)."""
    a = np.random.default_rng(seed).standard_normal((m, k), dtype=np.float32)
    return a.astype(np.float16).astype(np.float32)


def rel_err_floored(y: np.ndarray, ref64: np.ndarray) -> float:
    """max |y - ref| / max(|ref|, 2^-10 * rms(ref)).

    FP32 summation order alone moves an output that happens to be near zero by
    more than 1 % of itself, so the denominator is floored at a thousandth of
    the typical output magnitude; ref64 is the f64-accumulated oracle."""
    ref64 = np.asarray(ref64, dtype=np.float64)
    rms = float(np.sqrt(np.mean(ref64 ** 2))) if ref64.size else 0.0
    den = np.maximum(np.abs(ref64), rms * 2.0 ** -10 + 1e-30)
    return float(np.max(np.abs(np.asarray(y, dtype=np.float64) - ref64) / den)) if ref64.size else 0.0


def raw_rel_violations(y: np.ndarray, ref64: np.ndarray, tol: float = 1e-2):
    """The unfloored criterion: count of outputs with |y-ref|/|ref| > tol and the
    largest |ref| among them (reported, not asserted)."""
    ref64 = np.asarray(ref64, dtype=np.float64)
    rel = np.abs(np.asarray(y, dtype=np.float64) - ref64) / np.maximum(np.abs(ref64), 1e-300)
    bad = rel > tol
    return int(bad.sum()), float(np.abs(ref64[bad]).max()) if bad.any() else 0.0
