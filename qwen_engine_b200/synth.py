"""Seeded synthetic tensors with the value distributions of the benchmark configurations:
activations fp16 ~ N(0,1); weight nibbles uniform 0..15 (zero-point 8) in the packed
.qwenbin word order; scales fp16 ~ U[0.002, 0.02], one per 128-wide K group.

All generators are counter-based (numpy Philox) and depend only on (seed, name), so the
CUDA kernels, the CPU oracle and the rebuilt reference kernels are fed the same bytes.
"""
from __future__ import annotations

import zlib

import numpy as np

GROUP = 128


def _rng(seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed & 0xFFFFFFFFFFFFFFFF, zlib.crc32(name.encode())]))


def packed_weights(seed: int, name: str, N: int, K: int) -> np.ndarray:
    """uint32 [N][K/8]; every nibble of a uniform 32-bit word is uniform in 0..15."""
    return _rng(seed, name + ".w").integers(0, 1 << 32, size=(N, K // 8), dtype=np.uint32)


def scales(seed: int, name: str, N: int, K: int) -> np.ndarray:
    return _rng(seed, name + ".s").uniform(0.002, 0.02, size=(N, K // GROUP)).astype(np.float16)


def activations(seed: int, name: str, *shape: int) -> np.ndarray:
    return _rng(seed, name + ".x").standard_normal(size=shape, dtype=np.float32).astype(np.float16)


# Qwen2.5-1.5B projection shapes (reference include/config.cuh:10-22): name -> (N, K)
HIDDEN, INTER, Q_DIM, KV_DIM, VOCAB, LAYERS = 1536, 8960, 1536, 256, 151936, 28
SHAPES = {
    "q": (Q_DIM, HIDDEN), "k": (KV_DIM, HIDDEN), "v": (KV_DIM, HIDDEN),
    "o": (HIDDEN, Q_DIM), "gate_up": (2 * INTER, HIDDEN), "down": (HIDDEN, INTER),
    "lm_head": (VOCAB, HIDDEN),
}


def weight_bytes(N: int, K: int) -> int:
    return N * K // 2 + N * (K // GROUP) * 2


def q8_1_bytes(K: int) -> int:
    """int8 q8[K] + fp32 scale[K/128] + int32 sum8[K/8]"""
    return K * 49 // 32


def gemv_algorithmic_bytes(N: int, K: int, n_out: int | None = None, residual: bool = False) -> int:
    """Packed weights + scales + Q8_1 activation + fp16 outputs (+ fp16 residual)."""
    n_out = N if n_out is None else n_out
    return weight_bytes(N, K) + q8_1_bytes(K) + 2 * n_out + (2 * n_out if residual else 0)


def layer_algorithmic_bytes() -> int:
    qkv = sum(weight_bytes(*SHAPES[t]) for t in "qkv") + q8_1_bytes(HIDDEN) + 2 * (Q_DIM + 2 * KV_DIM)
    o = gemv_algorithmic_bytes(*SHAPES["o"], residual=True)
    gu = gemv_algorithmic_bytes(*SHAPES["gate_up"], n_out=INTER)
    down = gemv_algorithmic_bytes(*SHAPES["down"], residual=True)
    return qkv + o + gu + down


def sweep_algorithmic_bytes(layers: int = LAYERS) -> int:
    return layers * layer_algorithmic_bytes()
