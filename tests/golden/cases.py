"""Definitions of the golden cases (inputs are regenerated from seeds, outputs are stored)."""
from __future__ import annotations

import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                                "inquant-open-source_b200"))
import workloads  # noqa: E402


def _k4(seed, shape, dtype="bfloat16", policy="min_error", fraction=0.125, stride=8, zero_row=False,
        boundaries=False):
    return dict(seed=seed, shape=shape, dtype=dtype, policy=policy, fraction=fraction, stride=stride,
                zero_row=zero_row, boundaries=boundaries)


K4_CASES = {
    "preset_256": _k4(29, (2, 2, 256, 128), zero_row=True),
    "preset_neighbors": _k4(119, (1, 2, 256, 128), policy="neighbors"),
    "page_128": _k4(112, (2, 2, 128, 128)),
    "page_64": _k4(513, (2, 4, 64, 128)),
    "page_16": _k4(921, (4, 2, 16, 128)),
    "ragged_41_fp16": _k4(125, (1, 3, 41, 128), dtype="float16", policy="neighbors"),
    "fraction0": _k4(831, (1, 2, 64, 128), fraction=0.0),
    "fraction_half": _k4(7, (1, 2, 32, 128), fraction=0.5),
    "fp32_min_error": _k4(71, (1, 2, 64, 128), dtype="float32"),
    "small_c16": _k4(915, (2, 3, 41, 16), policy="neighbors", fraction=0.25),
    "stride3_c16": _k4(811, (6, 3, 8, 16), fraction=0.25, stride=3),
    # channels that put the float64 mean / variance update and the float32 roundings after it on
    # their boundaries (constant, zero-mean, offset, all-zero)
    "boundaries_bf16": _k4(5, (2, 2, 256, 128), boundaries=True),
    "boundaries_fp16": _k4(6, (1, 2, 256, 128), dtype="float16", boundaries=True),
}

V_CASES = {
    "v2_g64": dict(seed=99, shape=(2, 2, 64, 128), dtype="bfloat16", bits=2, group=64, zero_row=True),
    "v4_g64": dict(seed=17, shape=(1, 2, 32, 128), dtype="bfloat16", bits=4, group=64, zero_row=False),
    "v2_g32": dict(seed=27, shape=(1, 2, 32, 128), dtype="float16", bits=2, group=32, zero_row=False),
    "v2_g128": dict(seed=31, shape=(1, 2, 16, 128), dtype="float32", bits=2, group=128, zero_row=False),
    # groups of range zero (constant rows), groups dominated by one large channel, exact zeros
    "v2_boundaries": dict(seed=41, shape=(2, 2, 64, 128), dtype="bfloat16", bits=2, group=64, zero_row=True,
                          boundaries=True),
    "v4_boundaries_fp16": dict(seed=43, shape=(1, 2, 32, 128), dtype="float16", bits=4, group=32, zero_row=False,
                               boundaries=True),
}

SELECT_CASES = {f"{policy}_{count}": dict(seed=112, count=count, policy=policy)
                for policy in ("neighbors", "min_error") for count in (0, 1, 8, 16, 32, 64)}

PAGE_CASES = {
    "b64_h2": dict(seed=37, block=64, heads=2, pages=3),
    "b256_h4": dict(seed=52, block=256, heads=4, pages=1),
}

DECODE_CASES = {
    # config 0 of the benchmark definition: one layer, 4 KV heads, 4096 tokens, 28 query heads
    "cfg0": dict(seed=0, kv_heads=4, q_heads=28, tokens=4096, block=256, residual=128, sink=4,
                 scale_range=(15.0, 15.0)),
    "short_blocks": dict(seed=21, kv_heads=2, q_heads=8, tokens=700, block=64, residual=32, sink=4,
                         scale_range=(10.0, 20.0)),
}


def k4_input(case) -> np.ndarray:
    """fp32 array of values exactly representable in the case's dtype."""
    b, h, t, c = case["shape"]
    rng = np.random.default_rng(case["seed"])
    x = rng.standard_normal((b, h, t, c), dtype=np.float32) * (rng.random((1, h, 1, c), dtype=np.float32) * 3 + 0.1)
    hot = rng.permutation(c)[: max(1, c // 20)]
    x[..., hot] *= rng.uniform(10, 20, size=len(hot)).astype(np.float32)
    if c >= 64:
        x[..., 32:35] *= 15
    if case.get("zero_row"):
        x[0, 0] = 0
    if case.get("boundaries"):
        sign = np.where(np.arange(t) % 2 == 0, 1.0, -1.0).astype(np.float32)[:, None]
        x[..., 0::8] = 0.5                                   # constant: variance exactly zero
        x[..., 1::8] = 0.5 + sign * 2.0 ** -7                # constant plus a one-step ripple
        x[..., 2::8] = sign * 1.25                           # mean exactly zero
        x[..., 3::8] = 100.0 + 0.01 * x[..., 3::8]           # mean far above the spread
        x[..., 4::8] = 0.0                                   # all zero
        x[..., 5::8] = sign * 3.0 + 2.0 ** -8                # tiny mean, large swings
        if t > 7:
            x[0, -1, 5] = 0.75                               # a token row that is constant: every value group has range zero
            x[-1, 0, 7, : c // 2] = -2.5                     # one constant value group beside an ordinary one
    if case["dtype"] == "bfloat16":
        return workloads.bf16_exact(x)
    if case["dtype"] == "float16":
        return x.astype(np.float16).astype(np.float32)
    return x


def select_input(case):
    """Saliency rows with an all-zero row, a 40-wide tie plateau and an outlier at channel 127."""
    rng = np.random.default_rng(case["seed"])
    score = rng.random((3, 4, 128), dtype=np.float32)
    score[0] = 0
    score[1, :, 30:70] = 5
    score[2, :, 127] = 9
    error = rng.integers(0, 4, size=score.shape).astype(np.float32) if case["policy"] == "min_error" else None
    return score, error
