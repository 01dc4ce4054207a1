"""Seeded synthetic tensors (codes uniform, scale = bf16(|N(0, 0.02)|), bias = bf16(N(0, 0.01)), activations
bf16(N(0, 1)); GGUF blocks with f16 d, dmin = |N(0, 0.01)|) and the parity metric."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O


def affine_weights(rng: np.random.Generator, n: int, k: int, bits: int = 4, group_size: int = 64,
                   experts: int | None = None):
    """q ~ U{0..2^bits-1} packed low code first; scale = bf16(|N(0,0.02)|), bias = bf16(N(0,0.01))."""
    lead = (n,) if experts is None else (experts, n)
    # 32 uniform random bits per word are 32/bits independent uniform codes
    w = rng.integers(0, 1 << 32, size=lead + (k * bits // 32,), dtype=np.uint32)
    scales = O.f32_to_bf16(np.abs(rng.normal(0, 0.02, size=lead + (k // group_size,))).astype(np.float32))
    biases = O.f32_to_bf16(rng.normal(0, 0.01, size=lead + (k // group_size,)).astype(np.float32))
    return w, scales, biases


def activations(rng: np.random.Generator, m: int, k: int) -> np.ndarray:
    return O.f32_to_bf16(rng.normal(0, 1, size=(m, k)).astype(np.float32))


def gguf_weights(rng: np.random.Generator, fmt: int, rows: int, k: int, experts: int | None = None):
    """Uniform random code/scale bytes with f16 d, dmin = |N(0,0.01)| at the format's offsets."""
    bb = O.BLOCK_BYTES[fmt]
    nb = k // 256
    lead = (rows,) if experts is None else (experts, rows)
    w = rng.integers(0, 256, size=lead + (nb, bb), dtype=np.uint8)
    d = O.f32_to_f16_bits(np.abs(rng.normal(0, 0.01, size=lead + (nb,))).astype(np.float32))
    dmin = O.f32_to_f16_bits(np.abs(rng.normal(0, 0.01, size=lead + (nb,))).astype(np.float32))
    at = 80 if fmt == O.Q2_K else 0
    w[..., at] = d & 0xFF
    w[..., at + 1] = d >> 8
    w[..., at + 2] = dmin & 0xFF
    w[..., at + 3] = dmin >> 8
    return np.ascontiguousarray(w.reshape(lead + (nb * bb,)))


def parity(y: np.ndarray, ref: np.ndarray):
    """max over elements of |y - ref| / max(|ref|, rms(ref)) for f32 arrays, plus rel-L2."""
    y = y.astype(np.float64)
    ref = ref.astype(np.float64)
    rms = float(np.sqrt(np.mean(ref * ref))) or 1.0
    denom = np.maximum(np.abs(ref), rms)
    err = float(np.max(np.abs(y - ref) / denom)) if y.size else 0.0
    l2 = float(np.linalg.norm(y - ref) / (np.linalg.norm(ref) or 1.0))
    return err, l2


def bf16_ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> int:
    """Largest distance in bf16 ULPs (ordered-integer key, as array_ops.rs:1028-1031)."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - (u & 0x7FFF), 0x8000 + u)
    return int(np.max(np.abs(key(a_bits) - key(b_bits)))) if a_bits.size else 0
