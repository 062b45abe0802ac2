"""Shared helpers of the GPU parity tests: numpy <-> torch conversion and byte comparison."""
import numpy as np
import torch

TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def to_device(x32: np.ndarray, dtype: str = "bfloat16") -> torch.Tensor:
    """fp32 numpy array of dtype-exact values -> CUDA tensor of that dtype."""
    return torch.from_numpy(np.ascontiguousarray(x32)).to(TORCH_DTYPE[dtype]).cuda()


def to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        return t.float().numpy()
    return t.numpy()


def assert_same_bytes(actual: torch.Tensor, expected: np.ndarray, what: str = "") -> None:
    a = np.ascontiguousarray(to_numpy(actual))
    e = np.ascontiguousarray(expected)
    assert a.shape == e.shape, (what, a.shape, e.shape)
    assert a.dtype == e.dtype, (what, a.dtype, e.dtype)
    if a.tobytes() != e.tobytes():
        bad = np.flatnonzero(a.reshape(-1).view(np.uint8) != e.reshape(-1).view(np.uint8))
        raise AssertionError(f"{what}: {bad.size} differing bytes, first at {bad[:5]}")


def attention_close(actual: np.ndarray, expected: np.ndarray, max_abs: float = 2e-2, cosine: float = 0.9999):
    """Attention tolerance: max-abs 2e-2 and per-head cosine >= 0.9999 (bf16 outputs)."""
    actual = actual.astype(np.float64)
    expected = expected.astype(np.float64)
    assert np.isfinite(actual).all()
    err = np.abs(actual - expected).max()
    assert err < max_abs, f"max abs error {err}"
    cos = (actual * expected).sum(-1) / np.sqrt((actual * actual).sum(-1) * (expected * expected).sum(-1) + 1e-300)
    assert cos.min() >= cosine, f"cosine {cos.min()}"
