"""Seeded synthetic inputs shared by the tests (the mixture recipe of the benchmark configs) and small utilities."""

import numpy as np
import torch


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 values to the nearest bf16 and return them as fp32."""
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).bfloat16().float().numpy()


def mixture(count: int, dim: int, centres: int, sigma: float, seed: int) -> np.ndarray:
    """`count` vectors drawn around `centres` N(0,1) centres with spread `sigma`."""
    rng = np.random.default_rng(seed)
    mu = rng.standard_normal((centres, dim), dtype=np.float32)
    return mu[rng.integers(0, centres, count)] + sigma * rng.standard_normal((count, dim), dtype=np.float32)


def unit_rows(x: np.ndarray) -> np.ndarray:
    return (x / np.maximum(np.linalg.norm(x, axis=-1, keepdims=True), 1e-12)).astype(np.float32)


def layer_inputs(T: int, Hq: int, Hkv: int, dh: int, centres: int, seed: int):
    """q [T,Hq,dh], k, v [T,Hkv,dh] as bf16-valued fp32: clustered keys, queries = their key head plus noise."""
    rng = np.random.default_rng(seed)
    mu = rng.standard_normal((centres, Hkv, dh), dtype=np.float32)
    label = rng.integers(0, centres, T)
    k = mu[label] + 0.3 * rng.standard_normal((T, Hkv, dh), dtype=np.float32)
    q = np.repeat(k, Hq // Hkv, axis=1) + 0.5 * rng.standard_normal((T, Hq, dh), dtype=np.float32)
    v = rng.standard_normal((T, Hkv, dh), dtype=np.float32)
    return bf16_round(q), bf16_round(k), bf16_round(v)


def cuda(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dtype is None else t.to(dtype)


def sets(lists):
    return [sorted(row[row >= 0].tolist()) for row in np.asarray(lists)]
