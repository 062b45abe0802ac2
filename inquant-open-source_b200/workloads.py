"""Seeded synthetic KV tensors with the shapes and value distributions of the workloads
the packed-KV path is measured on (Qwen2.5-7B / Mistral-7B long-context decode).

No model weights or datasets are involved: keys are N(0,1) per channel with a few
outlier channels per head scaled by 10-20x (three of them adjacent, which forces the
donor search away from immediate neighbours); values are N(0,1).  The numpy generators
are bit-reproducible on any host and feed the parity tests and golden fixtures; the
torch generators build the full-size benchmark tensors directly on the device.
"""
from __future__ import annotations

import numpy as np


def bf16_exact(x: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest-even bf16 value, kept in fp32 storage."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    out = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return out.view(np.float32).reshape(x.shape)


def outlier_plan(rng: np.random.Generator, heads: int, dim: int, outliers: int, adjacent: int):
    """Per head: ``outliers`` distinct channels, the first ``adjacent`` of them contiguous."""
    plan = np.zeros((heads, outliers), np.int64)
    for h in range(heads):
        start = int(rng.integers(0, dim - adjacent))
        run = list(range(start, start + adjacent))
        rest = [c for c in rng.permutation(dim) if c not in run][: outliers - adjacent]
        plan[h] = run + [int(c) for c in rest]
    return plan


def make_kv(seed: int, heads: int, tokens: int, dim: int = 128, *, outliers: int = 6,
            adjacent: int = 3, scale_range=(10.0, 20.0), batch: int = 1):
    """K, V as fp32 arrays ``[batch, heads, tokens, dim]`` holding bf16-exact values."""
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((batch, heads, tokens, dim), dtype=np.float32)
    v = rng.standard_normal((batch, heads, tokens, dim), dtype=np.float32)
    plan = outlier_plan(rng, heads, dim, outliers, adjacent)
    lo, hi = scale_range
    for h in range(heads):
        factors = rng.uniform(lo, hi, size=outliers).astype(np.float32) if hi > lo else np.full(outliers, lo, np.float32)
        k[:, h, :, plan[h]] *= factors[:, None, None]
    return bf16_exact(k), bf16_exact(v)


def make_query(seed: int, q_heads: int, dim: int = 128) -> np.ndarray:
    rng = np.random.default_rng(seed + 7919)
    return bf16_exact(rng.standard_normal((q_heads, dim), dtype=np.float32))


def make_kv_torch(seed: int, heads: int, tokens: int, device, dim: int = 128, *, outliers: int = 6,
                  adjacent: int = 3, scale_range=(10.0, 20.0)):
    """Device-side generator of the same distribution (bf16 tensors ``[1,H,T,D]``)."""
    import torch
    gen = torch.Generator(device=device).manual_seed(seed)
    k = torch.randn((1, heads, tokens, dim), generator=gen, device=device, dtype=torch.float32)
    v = torch.randn((1, heads, tokens, dim), generator=gen, device=device, dtype=torch.float32)
    plan = outlier_plan(np.random.default_rng(seed), heads, dim, outliers, adjacent)
    lo, hi = scale_range
    factors = torch.empty((heads, outliers), device=device).uniform_(lo, hi, generator=gen)
    for h in range(heads):
        k[0, h][:, torch.as_tensor(plan[h], device=device)] *= factors[h]
    return k.to(torch.bfloat16), v.to(torch.bfloat16)
