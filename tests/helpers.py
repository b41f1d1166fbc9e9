"""Seeded synthetic inputs shared by the CPU and GPU tests and the benchmark.

A counter-based generator (splitmix64 of seed and index, Box-Muller in float64, rounded to
bfloat16) so that every program draws identical tensors.  No public dataset or benchmark
item is involved in this path; these shapes and distributions stand in for the GPT-2
activations, weights and gradients the reference trains on.
"""
from __future__ import annotations

import numpy as np
import torch

MASK = (1 << 64) - 1


def splitmix64(x: np.ndarray) -> np.ndarray:
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & np.uint64(MASK)
    z = x
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & np.uint64(MASK)
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & np.uint64(MASK)
    return z ^ (z >> np.uint64(31))


def uniform01(seed: int, n: int, stream: int = 0) -> np.ndarray:
    with np.errstate(over="ignore"):
        idx = np.arange(n, dtype=np.uint64) * np.uint64(2) + np.uint64(stream)
        base = splitmix64(np.full(1, seed, dtype=np.uint64))[0]
        bits = splitmix64(idx ^ base)
    return ((bits >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / (1 << 53))


def normal(seed: int, shape, std: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape))
    u1, u2 = uniform01(seed, n, 0), uniform01(seed, n, 1)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (z * std).reshape(shape)


def to_bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16)


def bf16_normal(seed: int, shape, std: float = 1.0) -> torch.Tensor:
    """bf16 tensor ~N(0, std)."""
    return to_bf16(normal(seed, shape, std))


def with_outliers(x: torch.Tensor, seed: int, every: int = 1000, factor: float = 50.0) -> torch.Tensor:
    """Multiplies about one element in `every` by `factor` (config 1's outliers)."""
    with np.errstate(over="ignore"):
        h = splitmix64(np.arange(x.numel(), dtype=np.uint64) ^ np.uint64(seed))
    mask = torch.from_numpy((h % np.uint64(every)) == 0).reshape(x.shape)
    return torch.where(mask, (x.float() * factor).to(x.dtype), x)


def rel_fro(a: np.ndarray, ref: np.ndarray) -> float:
    d = np.linalg.norm(a.astype(np.float64) - ref.astype(np.float64))
    n = np.linalg.norm(ref.astype(np.float64))
    return float(d / n) if n > 0 else float(d)


def set_e2m1_one(buf: np.ndarray, element: int) -> None:
    """crates/cuda-kernels/tests/common/nvfp4.rs:14-21."""
    b = int(buf[element // 2])
    buf[element // 2] = (b & 0xF0) | 0x2 if element % 2 == 0 else (b & 0x0F) | 0x20
