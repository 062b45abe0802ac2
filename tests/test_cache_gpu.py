"""Cache state machine on the GPU vs the oracle's restatement of the sealing rules.
Mirrors the reference's tests/test_cache.py and the append tests of tests/test_qwen_fused.py."""
import numpy as np
import pytest
import torch

import inquant_oracle as oracle
from helpers import assert_same_bytes, to_device, to_numpy

pytestmark = pytest.mark.gpu


def _mods():
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig, quantize
    return CacheConfig, InQuantCache, CodecConfig, quantize


def _randn(seed, shape):
    return oracle.round_to_bf16(np.random.default_rng(seed).standard_normal(shape, dtype=np.float32))


def _oracle_materialize(x, sink, block, residual, fraction, policy, stride=8, values=None):
    """What the cache must hold after seeing all of x in any chunking: sink | blocks | tail."""
    total = x.shape[2]
    take, blocks, tail = oracle.seal_plan(0, 0, total, sink_tokens=sink, residual_length=residual, block_size=block)
    pieces = [x[:, :, :take]]
    for i in range(blocks):
        part = x[:, :, take + i * block: take + (i + 1) * block]
        if values is None:
            pieces.append(oracle.dequantize_k4(oracle.quantize_k4(part, "bfloat16", stride, fraction, policy)))
        else:
            pieces.append(oracle.dequantize_values(oracle.quantize_values(part, "bfloat16", *values)))
    pieces.append(x[:, :, take + blocks * block:])
    return np.concatenate(pieces, axis=2), blocks


def test_prefill_returns_inputs_and_accounts_bytes():
    CacheConfig, InQuantCache, CodecConfig, _ = _mods()
    cfg = CacheConfig(CodecConfig(salient_fraction=0), block_size=8, residual_length=3, sink_tokens=2)
    cache = InQuantCache(cfg)
    key, value = to_device(_randn(17, (1, 2, 37, 8))), to_device(_randn(18, (1, 2, 37, 8)))
    rk, rv = cache.update(key, value, 0)
    assert rk is key and rv is value
    layer = cache._layers[0]
    assert len(layer.key_blocks) == 4 and layer.residual_key.shape[2] == 3 and layer.sink_key.shape[2] == 2
    packed = sum(b.nbytes for b in layer.key_blocks + layer.value_blocks)
    assert cache.nbytes == packed + cache.sink_nbytes + cache.residual_nbytes
    assert cache.bf16_nbytes == 2 * key.numel() * 2
    assert cache.memory_stats()["quantized_layer_tokens"] == 32
    assert cache.get_seq_length() == 37 and cache.get_usable_length(2) == 37 and cache.get_max_cache_shape() is None


@pytest.mark.parametrize("value_bits", [None, 2])
def test_chunked_appends_match_oracle_and_old_blocks_immutable(value_bits):
    CacheConfig, InQuantCache, CodecConfig, _ = _mods()
    cfg = CacheConfig(CodecConfig(salient_fraction=0.125, donor_policy="min_error"), block_size=8, residual_length=3,
                      sink_tokens=2, value_bits=value_bits)
    k32, v32 = _randn(1, (1, 3, 61, 128)), _randn(2, (1, 3, 61, 128))
    key, value = to_device(k32), to_device(v32)
    cache = InQuantCache(cfg)
    cache.update(key[:, :, :21], value[:, :, :21], 0)
    old_block = cache._layers[0].key_blocks[0]
    old_decoded = old_block.dequantize().clone()
    seen = 21
    for count in (1, 7, 12, 20):
        prior_key, prior_value = cache.materialize()
        out_key, out_value = cache.update(key[:, :, seen:seen + count], value[:, :, seen:seen + count], 0)
        assert torch.equal(out_key, torch.cat((prior_key, key[:, :, seen:seen + count]), dim=2))
        assert torch.equal(out_value, torch.cat((prior_value, value[:, :, seen:seen + count]), dim=2))
        seen += count
    assert cache._layers[0].key_blocks[0] is old_block
    assert torch.equal(old_block.dequantize(), old_decoded)
    mk, mv = cache.materialize()
    want_k, blocks = _oracle_materialize(k32, 2, 8, 3, 0.125, "min_error")
    want_v, _ = _oracle_materialize(v32, 2, 8, 3, 0.125, "min_error", values=None if value_bits is None else (2, 64))
    assert_same_bytes(mk.float(), want_k, "keys")
    assert_same_bytes(mv.float(), want_v, "values")
    assert len(cache._layers[0].key_blocks) == blocks
    assert cache._layers[0].residual_key.shape[2] < cfg.residual_length + cfg.block_size


def test_sink_accumulates_across_single_token_prefills():
    CacheConfig, InQuantCache, CodecConfig, _ = _mods()
    cache = InQuantCache(CacheConfig(CodecConfig(salient_fraction=0), block_size=8, residual_length=3, sink_tokens=2))
    x = to_device(_randn(3, (1, 2, 7, 8)))
    for pos in range(7):
        result, _ = cache.update(x[:, :, pos:pos + 1], x[:, :, pos:pos + 1], 0)
        assert torch.equal(result, x[:, :, :pos + 1])
    assert torch.equal(cache.materialize()[0], x)


def test_append_snapshot_matches_update_across_block_boundary():
    CacheConfig, InQuantCache, CodecConfig, _ = _mods()
    for cfg in (CacheConfig(CodecConfig(salient_fraction=.125), block_size=8, residual_length=2, sink_tokens=2),
                CacheConfig(CodecConfig(donor_policy="min_error"), block_size=8, residual_length=3, sink_tokens=2,
                            value_bits=2, track_peak_bytes=True)):
        reference, packed = InQuantCache(cfg), InQuantCache(cfg)
        key, value = to_device(_randn(27, (1, 2, 51, 128))), to_device(_randn(28, (1, 2, 51, 128)))
        reference.update(key[:, :, :19], value[:, :, :19], 0)
        packed.update(key[:, :, :19], value[:, :, :19], 0)
        for token in range(19, 51):
            expected = reference.update(key[:, :, token:token + 1], value[:, :, token:token + 1], 0)
            view = packed.append_for_attention(key[:, :, token:token + 1], value[:, :, token:token + 1], 0)
            for wanted, sink, blocks, tail in zip(expected, (view.sink_key, view.sink_value),
                                                 (view.key_blocks, view.value_blocks),
                                                 (view.residual_key, view.residual_value)):
                actual = torch.cat([sink] + [b.dequantize() for b in blocks] + [tail], dim=2)
                assert torch.equal(actual, wanted)
            for a, b in zip(packed.materialize(), reference.materialize()):
                assert torch.equal(a, b)
            assert packed.nbytes == reference.nbytes and view.seq_length == token + 1
            if cfg.track_peak_bytes:
                assert packed.peak_nbytes == reference.peak_nbytes >= packed.nbytes
        stats = packed.memory_stats()
        assert stats['nbytes'] == sum(stats[k] for k in
                                      ['payload_nbytes', 'metadata_nbytes', 'sink_nbytes', 'residual_nbytes', 'auxiliary_nbytes'])


def test_tail_views_survive_later_seals():
    """A sealing decode step completes the tail buffer in place and takes over the buffer retired by
    the seal before it, but only when no view handed out earlier still refers to that buffer."""
    CacheConfig, InQuantCache, CodecConfig, _ = _mods()
    cfg = CacheConfig(CodecConfig(salient_fraction=.125), block_size=8, residual_length=4, sink_tokens=2, value_bits=2)
    key, value = to_device(_randn(31, (1, 2, 70, 128))), to_device(_randn(32, (1, 2, 70, 128)))
    for hold in (True, False):
        cache = InQuantCache(cfg)
        cache.update(key[:, :, :9], value[:, :, :9], 0)
        kept, buffers = [], set()
        for token in range(9, 70):
            view = cache.append_for_attention(key[:, :, token:token + 1], value[:, :, token:token + 1], 0)
            # sink | dequantised blocks | tail of every view is the history up to and including the token
            tail_start = token + 1 - view.residual_key.shape[2]
            assert torch.equal(view.residual_key, key[:, :, tail_start:token + 1])
            assert torch.equal(view.residual_value, value[:, :, tail_start:token + 1])
            buffers.add(cache._layers[0].tail_key_buffer.data_ptr())
            if hold:
                kept.append((tail_start, token + 1, view.residual_key, view.residual_value))
        for start, stop, k, v in kept:
            assert torch.equal(k, key[:, :, start:stop]) and torch.equal(v, value[:, :, start:stop])
        seals = len(cache._layers[0].key_blocks)
        assert seals >= 6
        # held views pin every retired buffer; without them two buffers alternate
        assert len(buffers) == (seals + 1 if hold else 2) or not hold and len(buffers) <= 3
        expected, _ = _oracle_materialize(to_numpy(key), 2, 8, 4, .125, "neighbors")
        assert np.array_equal(to_numpy(cache.materialize(0)[0]), expected)


def test_append_while_sink_is_still_filling():
    CacheConfig, InQuantCache, CodecConfig, _ = _mods()
    cfg = CacheConfig(sink_tokens=4, block_size=8, residual_length=2)
    reference, packed = InQuantCache(cfg), InQuantCache(cfg)
    x = to_device(_randn(5, (1, 2, 9, 8)))
    for cache in (reference, packed):
        cache.update(x[:, :, :1], x[:, :, :1], 0)
    for index in range(1, 9):
        expected = reference.update(x[:, :, index:index + 1], x[:, :, index:index + 1], 0)
        view = packed.append_for_attention(x[:, :, index:index + 1], x[:, :, index:index + 1], 0)
        for wanted, sink, blocks, tail in zip(expected, (view.sink_key, view.sink_value),
                                             (view.key_blocks, view.value_blocks), (view.residual_key, view.residual_value)):
            actual = torch.cat(([] if sink is None else [sink]) + [b.dequantize() for b in blocks] + [tail], dim=2)
            assert torch.equal(actual, wanted)


def test_batched_prefill_matches_serial_blocks():
    CacheConfig, InQuantCache, CodecConfig, quantize = _mods()
    from unittest.mock import patch
    config = CacheConfig(CodecConfig(sample_stride=3, salient_fraction=.25), block_size=8, residual_length=3, sink_tokens=2)
    key = to_device(_randn(6, (1, 3, 16, 55))).transpose(2, 3)
    value = to_device(_randn(7, (1, 3, 16, 55))).transpose(2, 3)
    assert not key.is_contiguous()
    cache = InQuantCache(config)
    with patch("inquant.cache.quantize", wraps=quantize) as observed:
        cache.update(key, value, 0)
    assert observed.call_count == 2
    assert tuple(observed.call_args_list[0].args[0].shape) == (6, 3, 8, 16)
    layer = cache._layers[0]
    expected_bytes = 0
    for original, blocks in ((key, layer.key_blocks), (value, layer.value_blocks)):
        assert len(blocks) == 6
        for index, actual in enumerate(blocks):
            start = 2 + index * 8
            serial = quantize(original[:, :, start:start + 8], config.codec)
            assert actual.shape == serial.shape and actual.nbytes == serial.nbytes
            expected_bytes += serial.nbytes
            for name, tensor in actual.tensors.items():
                assert torch.equal(tensor, serial.tensors[name]), name
            assert torch.equal(actual.dequantize(), serial.dequantize())
    assert cache.nbytes == expected_bytes + cache.sink_nbytes + cache.residual_nbytes


@pytest.mark.parametrize("value_bits", [None, 2, 4])
def test_direct_sealing_equals_the_call_by_call_path(value_bits, monkeypatch):
    """Sealing with computed descriptors (key encoder first, then ``inq_seal_blocks``: value
    encoder and the sink / tail copies from one host call)
    leaves byte for byte what the general path leaves: every packed field, the sink and the tail,
    over a prefill of several blocks, chunks that cross block boundaries, sink tokens arriving in
    the same call as sealed blocks, and decode steps that seal."""
    CacheConfig, InQuantCache, CodecConfig, _ = _mods()
    cfg = CacheConfig(CodecConfig(donor_policy="min_error"), block_size=32, residual_length=16, sink_tokens=4,
                      value_bits=value_bits, value_group_size=64, validate_positions=False)
    key, value = to_device(_randn(61, (1, 2, 400, 128))), to_device(_randn(62, (1, 2, 400, 128)))
    # heads-major memory as a model hands it over: [1, tokens, heads, 128] transposed
    strided_key = key.transpose(1, 2).contiguous().transpose(1, 2)
    chunks = [(0, 3), (3, 150), (150, 151), (151, 290), (290, 291)] + [(t, t + 1) for t in range(291, 400)]

    def run(one_call, k):
        calls = []
        if one_call:
            original = InQuantCache._seal_direct

            def counted(self, *args):
                result = original(self, *args)
                calls.append(result is not None)
                return result
            monkeypatch.setattr(InQuantCache, "_seal_direct", counted)
        else:
            monkeypatch.setattr(InQuantCache, "_seal_direct", lambda self, *args: None)
        cache = InQuantCache(cfg)
        for start, stop in chunks:
            if stop - start == 1 and start > 150:
                cache.append_for_attention(k[:, :, start:stop], value[:, :, start:stop], 0)
            else:
                cache.extend(k[:, :, start:stop], value[:, :, start:stop], 0)
        monkeypatch.undo()
        return cache._layers[0], calls

    general, _ = run(False, key)
    for k in (key, strided_key):
        fast, calls = run(True, k)
        assert calls and all(calls)
        assert len(fast.key_blocks) == len(general.key_blocks) == (400 - 4 - 16) // 32
        assert fast.sink_count == general.sink_count == 4 and fast.tail_count == general.tail_count
        for mine, theirs in zip(fast.key_blocks + fast.value_blocks, general.key_blocks + general.value_blocks):
            assert type(mine).__mro__[-2] is type(theirs).__mro__[-2] and mine.shape == theirs.shape
            for name, tensor in theirs.tensors.items():
                assert torch.equal(mine.tensors[name], tensor), name
        for a, b in ((fast.sink_key, general.sink_key), (fast.sink_value, general.sink_value),
                     (fast.residual_key, general.residual_key), (fast.residual_value, general.residual_value)):
            assert torch.equal(a, b)


def test_positions_layers_reset_and_unsupported_operations():
    CacheConfig, InQuantCache, CodecConfig, _ = _mods()
    from unittest.mock import patch
    cache = InQuantCache(CacheConfig(CodecConfig(salient_fraction=0), block_size=8, residual_length=3, sink_tokens=2))
    x = to_device(_randn(8, (1, 2, 7, 8)))
    pos = torch.arange(7, device="cuda")
    cache.update(x, x, 0, {"cache_position": pos})
    cache.update(x, x, 1, {"cache_position": pos})
    assert len(cache) == 2 and cache.seen_tokens == 7 and cache.get_seq_length(5) == 0
    assert cache.get_mask_sizes(torch.arange(7, 9), 1) == (9, 0)
    with pytest.raises(ValueError):
        cache.update(x, x, 0, {"cache_position": pos})
    assert cache.get_seq_length() == 7
    with pytest.raises(NotImplementedError):
        cache.update(x.expand(2, -1, -1, -1), x.expand(2, -1, -1, -1), 0)
    with pytest.raises(NotImplementedError):
        cache.reorder_cache(torch.tensor([0]))
    with pytest.raises(NotImplementedError):
        cache.crop(3)
    with pytest.raises(ValueError):
        cache.update(x[:, :, :, :7], x[:, :, :, :7], 2)
    with pytest.raises(RuntimeError, match="CUDA"):
        InQuantCache().update(x.cpu(), x.cpu(), 0)
    cache.release()
    assert cache.nbytes == 0 and cache.get_seq_length() == 0 and len(cache) == 0
    quiet = InQuantCache(CacheConfig(validate_positions=False))
    with patch("inquant.cache.torch.equal", side_effect=AssertionError("Unexpected value synchronization")):
        quiet.update(x[:, :, :3], x[:, :, :3], 0, {"cache_position": torch.arange(3)})
        quiet.append_for_attention(x[:, :, :1], x[:, :, :1], 0, {"cache_position": torch.tensor([3])})
    assert quiet.get_seq_length() == 4
    for bad in (torch.tensor([[4]]), torch.tensor([4, 5]), torch.tensor([4.0]), [4]):
        with pytest.raises(ValueError):
            quiet.append_for_attention(x[:, :, :1], x[:, :, :1], 0, {"cache_position": bad})
        assert quiet.get_seq_length() == 4
    with pytest.raises(ValueError):
        CacheConfig(validate_positions="false")


def test_32k_shape_and_persistent_bytes():
    CacheConfig, InQuantCache, CodecConfig, _ = _mods()
    cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), value_bits=2))
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(1, 4, 32768, 128, device="cuda", generator=gen).bfloat16()
    cache.update(x, x, 0)
    layer = cache._layers[0]
    assert len(layer.key_blocks) == 127 and layer.residual_key.shape[2] == 252 and layer.sink_key.shape[2] == 4
    # 13.83 MB of packed blocks per layer at 32K (storage figure of the reference's README)
    assert cache.payload_nbytes + cache.metadata_nbytes == 127 * 4 * (256 * 104 + 512 + 16 + 16 + 64)
    tail = torch.randn(1, 4, 3, 128, device="cuda", generator=gen).bfloat16()
    out, _ = cache.update(tail, tail, 0)
    assert tuple(out.shape) == (1, 4, 32771, 128) and cache.get_seq_length() == 32771
    assert cache.nbytes < cache.bf16_nbytes * 0.3
