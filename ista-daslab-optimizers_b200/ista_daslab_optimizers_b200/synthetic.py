"""Seeded synthetic parameters and gradients for tests, golden vectors and the benchmark.

Everything here is a pure function of (seed, stream, element index) computed with 64-bit
integer arithmetic and correctly rounded float64 operations only (+, -, *, /, sqrt), so the
same call returns the same bits on every machine and any slice of a tensor can be produced
without producing the rest.  "Normal" samples are Irwin-Hall sums of twelve 16-bit uniforms
(variance 1, support +-6 sigma): close enough to N(0, sigma) for an optimizer input and free
of libm calls.
"""
from __future__ import annotations

import numpy as np
import torch

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over='ignore'):
        x = x + np.uint64(0x9E3779B97F4A7C15)
        z = x
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _stream_key(seed: int, stream: int) -> np.uint64:
    k = _splitmix64(np.array([seed & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64))
    k = _splitmix64(k ^ np.uint64(stream & 0xFFFFFFFFFFFFFFFF))
    return k[0]


def standard_normal(seed: int, stream: int, start: int, count: int) -> np.ndarray:
    """float64 approximately-N(0,1) samples for element indices [start, start + count)."""
    key = _stream_key(seed, stream)
    idx = np.arange(start, start + count, dtype=np.uint64)
    total = np.zeros(count, dtype=np.int64)
    with np.errstate(over='ignore'):
        for j in range(3):
            h = _splitmix64((idx * np.uint64(3) + np.uint64(j)) ^ key)
            for s in (0, 16, 32, 48):
                total += ((h >> np.uint64(s)) & np.uint64(0xFFFF)).astype(np.int64)
    # twelve uniforms on {0..65535}: mean 12*32767.5, variance 12*(65536^2-1)/12
    return (total.astype(np.float64) - 393210.0) / np.sqrt(65536.0 ** 2 - 1.0)


def normal_tensor(seed: int, stream: int, numel: int, sigma: float, dtype=torch.float32,
                  start: int = 0) -> torch.Tensor:
    z = standard_normal(seed, stream, start, numel) * sigma
    return torch.from_numpy(z.astype(np.float32)).to(dtype)


def student_t3_tensor(seed: int, stream: int, numel: int, scale: float, start: int = 0) -> torch.Tensor:
    """Student-t with 3 degrees of freedom, times `scale`, as float32 (heavy-tailed gradients)."""
    z = standard_normal(seed, stream * 4 + 0, start, numel)
    chi = np.zeros(numel, dtype=np.float64)
    for j in (1, 2, 3):
        w = standard_normal(seed, stream * 4 + j, start, numel)
        chi += w * w
    t = z / np.sqrt(np.maximum(chi, 1e-12) / 3.0)
    return torch.from_numpy((t * scale).astype(np.float32))


def round_to_8_mantissa_bits(x: torch.Tensor) -> torch.Tensor:
    """float32 -> bfloat16 -> float32 round trip: injects many exact ties."""
    return x.to(torch.bfloat16).to(torch.float32)


def llama3_8b_shapes():
    """The 290-tensor Llama-3-8B parameter list (shapes only): embed, 32 x [q, k, v, o, gate,
    up, down, norm, norm], lm_head."""
    shapes = [(128256, 4096)]
    for _ in range(32):
        shapes += [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096),
                   (14336, 4096), (14336, 4096), (4096, 14336), (4096,), (4096,)]
    shapes.append((128256, 4096))
    return shapes


def stress_shapes(seed: int, count: int = 300, lo: int = 64, hi: int = 8192):
    """Mixed 2-D shapes with every 10th a conv-like [256, 256, 3, 3]."""
    key = _stream_key(seed, 0x5EED)
    h = _splitmix64(np.arange(2 * count, dtype=np.uint64) ^ key)
    dims = (h % np.uint64(hi - lo + 1)).astype(np.int64) + lo
    shapes = []
    for i in range(count):
        shapes.append((256, 256, 3, 3) if i % 10 == 9 else (int(dims[2 * i]), int(dims[2 * i + 1])))
    return shapes
