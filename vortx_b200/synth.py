"""Seeded synthetic inputs with the shapes and distributions of the benchmark configurations.

numpy's counter-based Philox generator: the same seed gives the same bits on every machine,
so the CPU oracle and the GPU path always see identical inputs.
"""
from __future__ import annotations

import numpy as np


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(seed))


def uniform_matrix(rows: int, cols: int, seed: int) -> np.ndarray:
    """f32 entries i.i.d. uniform in [-1, 1)."""
    return (_rng(seed).random((rows, cols), dtype=np.float32) * np.float32(2.0) - np.float32(1.0))


def normal_matrix(rows: int, cols: int, seed: int, sigma: float = 0.02) -> np.ndarray:
    """f32 entries i.i.d. N(0, sigma^2) — the pre-quantisation weights (sigma = 0.02)."""
    return _rng(seed).standard_normal((rows, cols), dtype=np.float32) * np.float32(sigma)


def normal_vectors(batch: int, length: int, seed: int) -> np.ndarray:
    """`batch` contiguous f32 vectors ~ N(0, 1) — the activations."""
    return _rng(seed).standard_normal((batch, length), dtype=np.float32)
