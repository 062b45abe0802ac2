"""Parity at the sizes the benchmark times (config 1 and config 2 of the workload list): the
28-layer x 127-block decode launch (443 CTAs whose ranges cross pair boundaries) against the
oracle, and a 32768-token prompt sealed as 16 chunks of 2048 against the one-shot seal and the
oracle's encoders, bit for bit."""
import numpy as np
import pytest
import torch

import inquant_oracle as oracle
import workloads
from helpers import to_numpy

pytestmark = pytest.mark.gpu

HEADS, CONTEXT, BLOCK, RESIDUAL, SINK = 4, 32768, 256, 128, 4


def _config():
    from inquant.cache import CacheConfig
    from inquant.codec import CodecConfig
    return CacheConfig(CodecConfig(donor_policy="min_error", donor_backend="triton"), block_size=BLOCK,
                       residual_length=RESIDUAL, sink_tokens=SINK, value_bits=2, value_group_size=64,
                       validate_positions=False)


def _fields(blocks):
    names = ("payload", "scales", "salient_channels", "donor_channels", "padding") if hasattr(blocks[0], "padding") \
        else ("payload", "scales", "offsets")
    return {name: to_numpy(torch.cat([getattr(b, name) for b in blocks], 0)) for name in names}


def test_chunked_seal_of_32768_tokens_equals_one_shot_seal_and_oracle():
    """Reference semantics `cache.py:179-200`: chunks of a prompt seal the same 256-token windows
    as one prefill does, so every packed field and descriptor must come out identical."""
    from inquant.cache import InQuantCache
    device = torch.device("cuda", 0)
    k, v = workloads.make_kv_torch(321, HEADS, CONTEXT, device)
    whole = InQuantCache(_config())
    whole.update(k, v, 0)
    chunked = InQuantCache(_config())
    chunk = 2048
    for c0 in range(0, CONTEXT, chunk):
        ks, vs = k[:, :, c0:c0 + chunk], v[:, :, c0:c0 + chunk]
        if c0 < 2 * chunk:
            full_k, _ = chunked.update(ks, vs, 0)      # the materialising path of the reference
            assert full_k.shape[2] == c0 + chunk
        else:
            chunked.extend(ks, vs, 0)
    a, b = whole._layers[0], chunked._layers[0]
    assert len(a.key_blocks) == len(b.key_blocks) == 127 and a.tail_count == b.tail_count == 252
    assert torch.equal(a.residual_key, b.residual_key) and torch.equal(a.sink_value, b.sink_value)
    one_k, one_v, many_k, many_v = _fields(a.key_blocks), _fields(a.value_blocks), _fields(b.key_blocks), _fields(b.value_blocks)
    body = slice(SINK, SINK + 127 * BLOCK)
    shape = (HEADS, 127, BLOCK, 128)
    kb = np.ascontiguousarray(to_numpy(k)[0][:, body].reshape(shape).transpose(1, 0, 2, 3))
    vb = np.ascontiguousarray(to_numpy(v)[0][:, body].reshape(shape).transpose(1, 0, 2, 3))
    want_k = oracle.quantize_k4(kb, "bfloat16", 8, 0.125, "min_error").fields()
    want_v = oracle.quantize_values(vb, "bfloat16", 2, 64).fields()
    for got_one, got_many, want in ((one_k, many_k, want_k), (one_v, many_v, want_v)):
        for name, array in want.items():
            assert got_one[name].dtype == array.dtype and got_one[name].shape == array.shape, name
            assert got_one[name].tobytes() == array.tobytes(), f"one-shot {name} differs from the oracle"
            assert got_many[name].tobytes() == array.tobytes(), f"chunked {name} differs from the oracle"


def test_28_layer_launch_at_32768_tokens_matches_oracle_on_three_layers():
    """The launch the benchmark times: 28 sequences x 4 KV heads x 127 blocks in one grid.  Uses
    the benchmark's own checker, so that checker is covered too."""
    import bench
    from inquant import _native as N
    from inquant.batched import DecodeBatch, SequenceState
    from inquant.cache import InQuantCache
    device = torch.device("cuda", 0)
    layers = 28
    cache = InQuantCache(_config())
    for layer in range(layers):
        k, v = workloads.make_kv_torch(7000 + layer, HEADS, CONTEXT, device)
        cache.update(k, v, layer)
        del k, v
    batch = DecodeBatch([SequenceState.from_cache_layer(cache, i) for i in range(layers)], 28, torch.bfloat16)
    gen = torch.Generator(device=device).manual_seed(5)
    for step in range(3):   # tails of 253, 254, 255 tokens
        batch.inputs.copy_(torch.randn(batch.inputs.shape, device=device, generator=gen).bfloat16())
        batch.step()
    report = bench.check_decode_parity(torch, batch, cache, [0, 13, 27], seed_base=7000, encode_layer=27)
    assert report["max_abs"] < 2e-2 and report["min_cos"] >= 0.9999 and report["encode_mismatched_bytes"] == 0
    assert N.take_status(device) == 0
