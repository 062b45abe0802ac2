"""Configuration and argument checks that answer before any device call, with the reference's
messages (reference ``codec.py:38-55``, ``cache.py:24-54``, ``value_codec.py:51-60``,
``tests/test_codec.py:126-146``).  CPU tensors must be refused loudly: the packed-KV path has no
CPU implementation to fall back to."""
import pytest
import torch

from inquant.cache import CacheConfig, InQuantCache
from inquant.codec import CodecConfig, quantize
from inquant.value_codec import quantize_values


def test_codec_config_mirrors_the_reference_checks():
    assert CodecConfig() == CodecConfig(8, 0.125, "neighbors", "torch")
    for bad in (-0.1, 0.51, float("nan"), float("inf")):
        with pytest.raises(ValueError, match="salient_fraction"):
            CodecConfig(salient_fraction=bad)
    for bad in (0, -1, 1.5, True):
        with pytest.raises(ValueError, match="sample_stride"):
            CodecConfig(sample_stride=bad)
    with pytest.raises(ValueError, match="donor_policy"):
        CodecConfig(donor_policy="nearest")
    with pytest.raises(ValueError, match="donor_backend"):
        CodecConfig(donor_backend="cuda")
    for backend in ("torch", "triton", "auto"):
        assert CodecConfig(donor_backend=backend).donor_backend == backend


def test_cache_config_mirrors_the_reference_checks():
    default = CacheConfig()
    assert (default.block_size, default.residual_length, default.sink_tokens) == (256, 128, 4)
    assert default.value_bits is None and default.value_group_size == 64 and default.validate_positions
    for name in ("block_size", "residual_length", "sink_tokens"):
        for bad in (1.0, True, "4"):
            with pytest.raises(ValueError, match=f"{name} must be an integer"):
                CacheConfig(**{name: bad})
    for kwargs in ({"block_size": 0}, {"residual_length": -1}, {"sink_tokens": -1}):
        with pytest.raises(ValueError, match="block_size must be positive"):
            CacheConfig(**kwargs)
    for name in ("validate_positions", "shared_workspace", "track_peak_bytes"):
        with pytest.raises(ValueError, match=f"{name} must be a boolean"):
            CacheConfig(**{name: 1})
    for bad in (3, 8, True, 2.0):
        with pytest.raises(ValueError, match="value_bits"):
            CacheConfig(value_bits=bad)
    for bad in (16, 256, 64.0):
        with pytest.raises(ValueError, match="value_group_size"):
            CacheConfig(value_group_size=bad)


def test_shape_and_dtype_checks_come_before_the_device_check():
    with pytest.raises(ValueError, match="even"):
        quantize(torch.zeros(1, 1, 8, 7))
    with pytest.raises(ValueError, match="nonempty"):
        quantize(torch.zeros(1, 1, 0, 8))
    with pytest.raises(ValueError, match="floating"):
        quantize(torch.zeros(1, 1, 8, 8, dtype=torch.int32))
    with pytest.raises(ValueError, match="bits"):
        quantize_values(torch.zeros(1, 1, 8, 128), bits=3)
    with pytest.raises(ValueError, match="group size"):
        quantize_values(torch.zeros(1, 1, 8, 128), group_size=48)
    with pytest.raises(ValueError, match="divisible"):
        quantize_values(torch.zeros(1, 1, 8, 96), group_size=64)


def test_cpu_tensors_are_refused_not_served():
    x = torch.zeros(1, 2, 16, 128, dtype=torch.bfloat16)
    for call in (lambda: quantize(x), lambda: quantize_values(x), lambda: InQuantCache().update(x, x, 0)):
        with pytest.raises((ValueError, RuntimeError, NotImplementedError), match="CUDA"):
            call()
    cache = InQuantCache()
    with pytest.raises(ValueError, match="layer_idx"):
        cache.update(x, x, -1)
    with pytest.raises(NotImplementedError, match="batch size 1"):
        cache.update(torch.zeros(2, 2, 4, 128), torch.zeros(2, 2, 4, 128), 0)
    with pytest.raises(ValueError, match="matching"):
        cache.update(x, x[:, :1], 0)
    assert len(cache) == 0 and cache.get_seq_length() == 0
