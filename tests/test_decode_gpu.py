"""Packed decode attention (table layout) vs the CPU oracle: dequantise everything with the
oracle, run float64 attention, compare within max-abs 2e-2 and cosine >= 0.9999 (the bound
stated for bf16 attention outputs); most cases also hold the reference tests' atol 1e-3 /
rtol 2e-2.  Mirrors the reference's tests/test_triton_attention.py and
tests/test_incremental_state.py."""
import numpy as np
import pytest
import torch

import inquant_oracle as oracle
import workloads
from cases import DECODE_CASES, k4_input
from helpers import TORCH_DTYPE, attention_close, to_device, to_numpy

pytestmark = pytest.mark.gpu


def _mods():
    from inquant.codec import CodecConfig, quantize
    from inquant.value_codec import quantize_values
    from inquant.triton_attention import PackedDecodeState, SharedDecodeWorkspace, packed_decode
    return CodecConfig, quantize, quantize_values, PackedDecodeState, SharedDecodeWorkspace, packed_decode


def _random(seed, shape, dtype):
    x = np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)
    return oracle.round_to_dtype(x, dtype)


def _expected(q, pieces_k, pieces_v, scale=128 ** -0.5):
    keys = np.concatenate(pieces_k, axis=1)
    vals = np.concatenate(pieces_v, axis=1)
    return oracle.attention_decode(q, keys, vals, scale)


def _check(actual, expected, atol=1e-3, rtol=0.02):
    actual = to_numpy(actual.float()).reshape(expected.shape)
    attention_close(actual, expected)
    assert np.all(np.abs(actual - expected) <= atol + rtol * np.abs(expected) + 4e-3 * np.abs(expected).max()), \
        np.abs(actual - expected).max()


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("fraction", [0.0, 0.125, 0.5])
@pytest.mark.parametrize("policy", ["neighbors", "min_error"])
def test_packed_gqa_with_sink_and_unsealed_tail(dtype, fraction, policy):
    CodecConfig, quantize, quantize_values, PackedDecodeState, _, _ = _mods()
    cfg = CodecConfig(salient_fraction=fraction, donor_policy=policy)
    ks = [_random(921 + i, (1, 4, 256, 128), dtype) for i in range(3)]
    vs = [_random(1921 + i, (1, 4, 256, 128), dtype) for i in range(3)]
    ks = [oracle.round_to_dtype(k * np.where((np.arange(128) >= 5) & (np.arange(128) < 8), 12, 1).astype(np.float32), dtype)
          for k in ks]
    keys = [quantize(to_device(k, dtype), cfg) for k in ks]
    values = [quantize_values(to_device(v, dtype)) for v in vs]
    sink_k, sink_v = _random(1, (1, 4, 4, 128), dtype), _random(2, (1, 4, 4, 128), dtype)
    tail_k, tail_v = _random(3, (1, 4, 281, 128), dtype), _random(4, (1, 4, 281, 128), dtype)
    q = _random(5, (28, 128), dtype)
    state = PackedDecodeState(keys, values)
    descriptor_bytes = state.nbytes
    args = dict(sink_key=to_device(sink_k, dtype), sink_value=to_device(sink_v, dtype),
                residual_key=to_device(tail_k, dtype), residual_value=to_device(tail_v, dtype))
    query = to_device(q, dtype).view(1, 28, 1, 128)
    actual = state.decode(query, **args)
    ok = [oracle.quantize_k4(k, dtype, 8, fraction, policy) for k in ks]
    ov = [oracle.quantize_values(v, dtype) for v in vs]
    expected = _expected(q, [sink_k[0]] + [oracle.dequantize_k4(b)[0] for b in ok] + [tail_k[0]],
                         [sink_v[0]] + [oracle.dequantize_values(b)[0] for b in ov] + [tail_v[0]])
    _check(actual, expected)
    assert actual.shape == query.shape and actual.dtype == TORCH_DTYPE[dtype]
    assert state.nbytes == descriptor_bytes + state._workspace.numel() * 4
    pointer = state._workspace.data_ptr()
    again = state.decode(query, **args)
    assert state._workspace.data_ptr() == pointer
    assert torch.equal(actual, again)


@pytest.mark.parametrize("tokens", [1, 4, 15, 16, 17, 257])
def test_dense_only_before_any_block_is_sealed(tokens):
    *_, packed_decode = _mods()
    q = _random(7, (14, 128), "bfloat16")
    key, value = _random(8, (1, 2, tokens, 128), "bfloat16"), _random(9, (1, 2, tokens, 128), "bfloat16")
    actual = packed_decode(to_device(q).view(1, 14, 1, 128), [], [], residual_key=to_device(key), residual_value=to_device(value))
    _check(actual, _expected(q, [key[0]], [value[0]]), atol=5e-3)


@pytest.mark.parametrize("tokens,heads,q_heads", [(41, 1, 3), (16, 2, 16), (200, 1, 1), (64, 2, 32)])
def test_no_dense_tensors_and_nondefault_packed_block_length(tokens, heads, q_heads):
    CodecConfig, quantize, quantize_values, _, _, packed_decode = _mods()
    k, v = _random(10, (1, heads, tokens, 128), "float16"), _random(11, (1, heads, tokens, 128), "float16")
    k[..., 100] *= 8   # power of two: stays exactly representable
    q = _random(12, (q_heads, 128), "float16")
    actual = packed_decode(to_device(q, "float16").view(1, q_heads, 1, 128),
                           [quantize(to_device(k, "float16"), CodecConfig(salient_fraction=0.125))],
                           [quantize_values(to_device(v, "float16"))])
    expected = _expected(q, [oracle.dequantize_k4(oracle.quantize_k4(k, "float16"))[0]],
                         [oracle.dequantize_values(oracle.quantize_values(v, "float16"))[0]])
    _check(actual, expected)


def test_extreme_softmax_and_zero_blocks_remain_finite():
    CodecConfig, quantize, quantize_values, _, _, packed_decode = _mods()
    key = np.zeros((1, 1, 256, 128), np.float32)
    key[..., 0, :] = 30
    value = _random(13, key.shape, "bfloat16")
    q = np.full((7, 128), 20, np.float32)
    actual = packed_decode(to_device(q).view(1, 7, 1, 128), [quantize(to_device(key))], [quantize_values(to_device(value))])
    expected = _expected(q, [oracle.dequantize_k4(oracle.quantize_k4(key))[0]],
                         [oracle.dequantize_values(oracle.quantize_values(value))[0]])
    assert torch.isfinite(actual).all()
    _check(actual, expected)


def test_growing_state_matches_fresh_state_and_rejects_replacement():
    CodecConfig, quantize, quantize_values, PackedDecodeState, _, _ = _mods()
    keys, values, raw = [], [], []
    state = PackedDecodeState([], [])
    q = _random(831, (8, 128), "bfloat16")
    query = to_device(q).view(1, 8, 1, 128)
    for i in range(11):
        k = _random(100 + i, (1, 2, 32, 128), "bfloat16")
        k[..., 127] *= 16   # source / donor indices at the signed-byte boundary
        v = _random(200 + i, (1, 2, 32, 128), "bfloat16")
        raw.append((k, v))
        keys.append(quantize(to_device(k), CodecConfig(donor_policy="min_error")))
        values.append(quantize_values(to_device(v)))
        state.extend(keys, values)
        fresh = PackedDecodeState(keys, values)
        assert torch.equal(state.decode(query), fresh.decode(query))
        assert state._key_map.dtype == torch.int8
        assert torch.equal(state._key_map[:i + 1], fresh._key_map[:i + 1])
        ok = oracle.quantize_k4(k, "bfloat16", 8, 0.125, "min_error")
        assert np.array_equal(to_numpy(state._key_map[i]),
                              oracle.role_map(ok.salient_channels, ok.donor_channels, 128)[0])
    expected = _expected(q, [oracle.dequantize_k4(oracle.quantize_k4(k, "bfloat16", 8, 0.125, "min_error"))[0] for k, _ in raw],
                         [oracle.dequantize_values(oracle.quantize_values(v))[0] for _, v in raw])
    _check(state.decode(query), expected)
    with pytest.raises(ValueError, match="append-only"):
        state.extend(keys[:-1], values[:-1])
    with pytest.raises(ValueError, match="append-only"):
        state.extend(list(reversed(keys)), values)
    state.extend(keys, values)
    assert torch.equal(state.decode(query), fresh.decode(query))


def test_growing_tail_lengths_and_strided_tail_views():
    CodecConfig, quantize, quantize_values, PackedDecodeState, _, _ = _mods()
    k, v = _random(20, (1, 4, 256, 128), "bfloat16"), _random(21, (1, 4, 256, 128), "bfloat16")
    state = PackedDecodeState([quantize(to_device(k))], [quantize_values(to_device(v))])
    tail_k, tail_v = _random(22, (1, 4, 192, 128), "bfloat16"), _random(23, (1, 4, 192, 128), "bfloat16")
    tk, tv = to_device(tail_k), to_device(tail_v)
    q = _random(24, (28, 128), "bfloat16")
    query = to_device(q).view(1, 28, 1, 128)
    dk = oracle.dequantize_k4(oracle.quantize_k4(k))[0]
    dv = oracle.dequantize_values(oracle.quantize_values(v))[0]
    for length in (129, 130, 143, 144, 145, 192):
        compact = state.decode(query, residual_key=tk[:, :, :length].contiguous(), residual_value=tv[:, :, :length].contiguous())
        strided = state.decode(query, residual_key=tk[:, :, :length], residual_value=tv[:, :, :length])
        assert torch.equal(compact, strided)
        _check(compact, _expected(q, [dk, tail_k[0, :, :length]], [dv, tail_v[0, :, :length]]))


def test_workspace_pool_is_shared_and_rejects_other_stream():
    CodecConfig, quantize, quantize_values, PackedDecodeState, SharedDecodeWorkspace, _ = _mods()
    pool = SharedDecodeWorkspace()
    q = _random(30, (28, 128), "bfloat16")
    k, v = _random(31, (1, 4, 19, 128), "bfloat16"), _random(32, (1, 4, 19, 128), "bfloat16")
    query = to_device(q).view(1, 28, 1, 128)
    states = [PackedDecodeState([], [], workspace_pool=pool) for _ in range(3)]
    for i, state in enumerate(states):
        actual = state.decode(query, residual_key=to_device(k), residual_value=to_device(v + i))
        _check(actual, _expected(q, [k[0]], [v[0] + i]), atol=8e-3)
        assert state._workspace is None and state.nbytes == 0
    first_pointer = pool.tensor.data_ptr()
    states[0].decode(query, residual_key=to_device(k), residual_value=to_device(v))
    assert first_pointer == pool.tensor.data_ptr()
    torch.cuda.synchronize()
    with torch.cuda.stream(torch.cuda.Stream()):
        with pytest.raises(RuntimeError, match="one CUDA stream"):
            states[0].decode(query, residual_key=to_device(k), residual_value=to_device(v))


def test_argument_validation():
    CodecConfig, quantize, quantize_values, PackedDecodeState, _, packed_decode = _mods()
    q = torch.zeros(1, 4, 1, 128, device="cuda", dtype=torch.bfloat16)
    kv = torch.zeros(1, 2, 8, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="nonempty KV head count"):
        packed_decode(q, [], [])
    with pytest.raises(ValueError, match="both"):
        packed_decode(q, [], [], residual_key=kv)
    with pytest.raises(ValueError, match="divisible"):
        packed_decode(torch.zeros(1, 3, 1, 128, device="cuda", dtype=torch.bfloat16), [], [], residual_key=kv, residual_value=kv)
    with pytest.raises(ValueError, match="dtype"):
        packed_decode(q.half(), [], [], residual_key=kv, residual_value=kv)
    with pytest.raises(ValueError, match="scale"):
        packed_decode(q, [], [], residual_key=kv, residual_value=kv, scale=0.0)
    assert packed_decode(q.float(), [], [], residual_key=kv.float(), residual_value=kv.float()).dtype == torch.float32
    with pytest.raises(ValueError, match="counts"):
        PackedDecodeState([quantize(kv)], [])
    with pytest.raises(ValueError, match="same quantizer"):
        PackedDecodeState([quantize(kv), quantize(kv)], [quantize(kv), quantize_values(kv)])


def test_extend_judges_the_blocks_of_an_encoder_launch_by_their_arena():
    """Blocks sealed by one launch are checked and addressed through their arena: none of their
    field views is created, a plain block sealed later joins them, and blocks of another geometry
    or codec are refused with the reference's messages."""
    from inquant.cache import CacheConfig, InQuantCache
    CodecConfig, quantize, quantize_values, PackedDecodeState, _, _ = _mods()

    def cache_with(block, tokens, value_bits=2, seed=5):
        cache = InQuantCache(CacheConfig(CodecConfig(), block_size=block, residual_length=8, sink_tokens=4,
                                         value_bits=value_bits, validate_positions=False))
        x = to_device(_random(seed, (1, 2, tokens, 128), "bfloat16"))
        cache.extend(x, x, 0)
        return cache, x

    cache, x = cache_with(32, 4 + 5 * 32 + 8 + 31)
    layer = cache._layers[0]
    assert len(layer.key_blocks) == 5 and all(hasattr(b, "_arena") for b in layer.key_blocks)
    state = PackedDecodeState(layer.key_blocks, layer.value_blocks)
    assert all(not vars(b) for b in layer.key_blocks + layer.value_blocks)      # nothing was materialised
    q = to_device(_random(6, (1, 4, 1, 128), "bfloat16"))
    before = state.decode(q, sink_key=layer.sink_key, sink_value=layer.sink_value,
                          residual_key=layer.residual_key, residual_value=layer.residual_value)
    cache.extend(x[:, :, :1], x[:, :, :1], 0)                                  # completes a block: a plain one
    assert len(layer.key_blocks) == 6 and not hasattr(layer.key_blocks[5], "_arena")
    state.extend(layer.key_blocks, layer.value_blocks)
    after = state.decode(q, sink_key=layer.sink_key, sink_value=layer.sink_value,
                         residual_key=layer.residual_key, residual_value=layer.residual_value)
    dense_k, dense_v = cache.materialize(0)
    want = oracle.attention_decode(to_numpy(q.float())[0, :, 0], to_numpy(dense_k.float())[0], to_numpy(dense_v.float())[0],
                                   128 ** -0.5)
    attention_close(to_numpy(after.float()).reshape(want.shape), want)
    assert before.shape == after.shape

    other, _ = cache_with(64, 4 + 3 * 64 + 8)
    with pytest.raises(ValueError, match="share shape"):
        PackedDecodeState(layer.key_blocks + other._layers[0].key_blocks, layer.value_blocks + other._layers[0].value_blocks)
    four_bit, _ = cache_with(32, 4 + 2 * 32 + 8, value_bits=4)
    with pytest.raises(ValueError, match="same quantizer"):
        PackedDecodeState(layer.key_blocks + four_bit._layers[0].key_blocks,
                          layer.value_blocks + four_bit._layers[0].value_blocks)


@pytest.mark.parametrize("name", sorted(DECODE_CASES))
def test_single_layer_roundtrip_matches_reference_output(golden, name):
    """Config 0 of the benchmark definition (and a short-block variant): encode on the GPU,
    decode on the GPU, compare with the reference's own attention output."""
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.triton_attention import PackedDecodeState
    case = DECODE_CASES[name]
    k, v = workloads.make_kv(case["seed"], case["kv_heads"], case["tokens"], outliers=6, adjacent=3,
                             scale_range=case["scale_range"])
    q = workloads.make_query(case["seed"], case["q_heads"])
    cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), block_size=case["block"],
                                     residual_length=case["residual"], sink_tokens=case["sink"], value_bits=2,
                                     value_group_size=64, validate_positions=False))
    kt, vt = to_device(k), to_device(v)
    n = case["tokens"] - 1
    cache.update(kt[:, :, :n], vt[:, :, :n], 0)
    view = cache.append_for_attention(kt[:, :, n:], vt[:, :, n:], 0)
    assert [len(view.key_blocks), view.sink_key.shape[2], view.residual_key.shape[2]] == list(golden[f"decode/{name}/layout"])
    state = PackedDecodeState(view.key_blocks, view.value_blocks)
    out = state.decode(to_device(q).view(1, case["q_heads"], 1, 128), sink_key=view.sink_key, sink_value=view.sink_value,
                       residual_key=view.residual_key, residual_value=view.residual_value, scale=128 ** -0.5)
    attention_close(to_numpy(out.float()).reshape(case["q_heads"], 128), golden[f"decode/{name}/output"])


# ---------------------------------------------------------------------------------------------
# Codec variants outside the K4/V2 preset and fp32 queries run the general kernel
# (the reference's tests/test_triton_attention.py cover the same combinations).
@pytest.mark.parametrize("value_codec,dtype,q_heads", [
    ("inquant", "bfloat16", 8), ("inquant", "float16", 14), ((4, 64), "bfloat16", 8), ((2, 32), "bfloat16", 4),
    ((2, 128), "float16", 8), ((4, 32), "bfloat16", 34), ((2, 64), "float32", 8), ("inquant", "float32", 4)])
def test_general_kernel_covers_non_preset_value_codecs_and_fp32(value_codec, dtype, q_heads):
    CodecConfig, quantize, quantize_values, PackedDecodeState, _, _ = _mods()
    heads, blocks, block, tail, sink, fraction = 2, 3, 64, 37, 4, 0.125
    cfg = CodecConfig(salient_fraction=fraction, donor_policy="min_error")
    boost = np.where((np.arange(128) >= 5) & (np.arange(128) < 8), 12, 1).astype(np.float32)
    ks = [oracle.round_to_dtype(_random(400 + i, (1, heads, block, 128), dtype) * boost, dtype) for i in range(blocks)]
    vs = [_random(500 + i, (1, heads, block, 128), dtype) for i in range(blocks)]
    keys = [quantize(to_device(k, dtype), cfg) for k in ks]
    dense_k = [oracle.dequantize_k4(oracle.quantize_k4(k, dtype, 8, fraction, "min_error"))[0] for k in ks]
    if value_codec == "inquant":
        values = [quantize(to_device(v, dtype), cfg) for v in vs]
        dense_v = [oracle.dequantize_k4(oracle.quantize_k4(v, dtype, 8, fraction, "min_error"))[0] for v in vs]
    else:
        bits, group = value_codec
        values = [quantize_values(to_device(v, dtype), bits, group) for v in vs]
        dense_v = [oracle.dequantize_values(oracle.quantize_values(v, dtype, bits, group))[0] for v in vs]
    sink_k, sink_v = _random(1, (1, heads, sink, 128), dtype), _random(2, (1, heads, sink, 128), dtype)
    tail_k, tail_v = _random(3, (1, heads, tail, 128), dtype), _random(4, (1, heads, tail, 128), dtype)
    q = _random(5, (q_heads, 128), dtype)
    state = PackedDecodeState(keys, values)
    assert state._preset == (value_codec == (2, 64))
    actual = state.decode(to_device(q, dtype).view(1, q_heads, 1, 128),
                          sink_key=to_device(sink_k, dtype), sink_value=to_device(sink_v, dtype),
                          residual_key=to_device(tail_k, dtype), residual_value=to_device(tail_v, dtype))
    expected = _expected(q, [sink_k[0]] + dense_k + [tail_k[0]], [sink_v[0]] + dense_v + [tail_v[0]])
    _check(actual, expected)
    assert actual.dtype == TORCH_DTYPE[dtype]
    # a growing state keeps working on the general path
    grown = PackedDecodeState(keys[:1], values[:1])
    grown.extend(keys, values)
    again = grown.decode(to_device(q, dtype).view(1, q_heads, 1, 128),
                         sink_key=to_device(sink_k, dtype), sink_value=to_device(sink_v, dtype),
                         residual_key=to_device(tail_k, dtype), residual_value=to_device(tail_v, dtype))
    assert torch.equal(actual, again)


@pytest.mark.parametrize("dtype,q_heads,heads,block,blocks,tail", [
    ("bfloat16", 28, 4, 256, 3, 281), ("float16", 14, 2, 256, 5, 17), ("bfloat16", 8, 2, 128, 7, 0),
    ("bfloat16", 12, 1, 256, 40, 300)])
def test_values_stored_as_inquant_tensors_run_the_streaming_kernel(dtype, q_heads, heads, block, blocks, tail):
    """The reference's CacheConfig default (value_bits=None): V blocks are InQuant packed tensors.
    With 16 salient channels on both sides and whole-slice blocks the one-launch kernel serves
    them (value nibbles as MMA operands, block sums folded with the per-channel scales); checked
    against the oracle's dequantised values, outlier channels in V included, and against the
    general kernel's output for the same state."""
    CodecConfig, quantize, _, PackedDecodeState, _, _ = _mods()
    cfg = CodecConfig(salient_fraction=0.125, donor_policy="min_error")
    boost_k = np.where((np.arange(128) >= 5) & (np.arange(128) < 8), 12, 1).astype(np.float32)
    boost_v = np.where((np.arange(128) % 29) == 3, 4, 1).astype(np.float32)
    ks = [oracle.round_to_dtype(_random(700 + i, (1, heads, block, 128), dtype) * boost_k, dtype) for i in range(blocks)]
    vs = [oracle.round_to_dtype(_random(800 + i, (1, heads, block, 128), dtype) * boost_v, dtype) for i in range(blocks)]
    keys = [quantize(to_device(k, dtype), cfg) for k in ks]
    values = [quantize(to_device(v, dtype), cfg) for v in vs]
    dense_k = [oracle.dequantize_k4(oracle.quantize_k4(k, dtype, 8, 0.125, "min_error"))[0] for k in ks]
    dense_v = [oracle.dequantize_k4(oracle.quantize_k4(v, dtype, 8, 0.125, "min_error"))[0] for v in vs]
    sink_k, sink_v = _random(1, (1, heads, 4, 128), dtype), _random(2, (1, heads, 4, 128), dtype)
    q = _random(5, (q_heads, 128), dtype)
    args = dict(sink_key=to_device(sink_k, dtype), sink_value=to_device(sink_v, dtype))
    pieces_k, pieces_v = [sink_k[0]] + dense_k, [sink_v[0]] + dense_v
    if tail:
        tail_k, tail_v = _random(3, (1, heads, tail, 128), dtype), _random(4, (1, heads, tail, 128), dtype)
        args.update(residual_key=to_device(tail_k, dtype), residual_value=to_device(tail_v, dtype))
        pieces_k.append(tail_k[0])
        pieces_v.append(tail_v[0])
    state = PackedDecodeState(keys, values)
    assert state._inquant_values and not state._preset
    query = to_device(q, dtype).view(1, q_heads, 1, 128)
    actual = state.decode(query, **args)
    assert state._workspace.ndim == 2            # the streaming kernel took the call (its scratch is [records, floats])
    _check(actual, _expected(q, pieces_k, pieces_v))
    general = state._decode_general(query, heads, q_heads // heads, blocks, args["sink_key"], args["sink_value"], 4,
                                    args.get("residual_key"), args.get("residual_value"), tail, 128 ** -0.5)
    attention_close(to_numpy(actual.float()).reshape(q_heads, 128), to_numpy(general.float()).reshape(q_heads, 128))
    from inquant import _native as N
    assert N.take_status(torch.device("cuda", 0)) == 0


@pytest.mark.parametrize("bits,group,dtype,q_heads,heads,block,blocks,tail", [
    (4, 64, "bfloat16", 28, 4, 256, 3, 281), (4, 32, "float16", 14, 2, 256, 5, 17), (4, 128, "bfloat16", 8, 2, 128, 7, 0),
    (4, 32, "bfloat16", 12, 1, 256, 40, 300), (2, 128, "bfloat16", 28, 4, 256, 3, 281), (2, 128, "float16", 8, 2, 128, 9, 5),
    (2, 32, "bfloat16", 28, 4, 256, 3, 281), (2, 32, "float16", 14, 2, 128, 11, 40)])
def test_four_bit_values_run_the_streaming_kernel(bits, group, dtype, q_heads, heads, block, blocks, tail):
    """4-bit values in groups of 32, 64 or 128 channels and 2-bit values in one group of 128
    (value_codec.py) on the one-launch kernel: checked against the oracle's dequantised values and
    the general kernel's output."""
    CodecConfig, quantize, quantize_values, PackedDecodeState, _, _ = _mods()
    cfg = CodecConfig(salient_fraction=0.125, donor_policy="min_error")
    boost_k = np.where((np.arange(128) >= 5) & (np.arange(128) < 8), 12, 1).astype(np.float32)
    ks = [oracle.round_to_dtype(_random(700 + i, (1, heads, block, 128), dtype) * boost_k, dtype) for i in range(blocks)]
    vs = [oracle.round_to_dtype(_random(800 + i, (1, heads, block, 128), dtype) + 0.5, dtype) for i in range(blocks)]
    keys = [quantize(to_device(k, dtype), cfg) for k in ks]
    values = [quantize_values(to_device(v, dtype), bits, group) for v in vs]
    dense_k = [oracle.dequantize_k4(oracle.quantize_k4(k, dtype, 8, 0.125, "min_error"))[0] for k in ks]
    dense_v = [oracle.dequantize_values(oracle.quantize_values(v, dtype, bits, group))[0] for v in vs]
    sink_k, sink_v = _random(1, (1, heads, 4, 128), dtype), _random(2, (1, heads, 4, 128), dtype)
    q = _random(5, (q_heads, 128), dtype)
    args = dict(sink_key=to_device(sink_k, dtype), sink_value=to_device(sink_v, dtype))
    pieces_k, pieces_v = [sink_k[0]] + dense_k, [sink_v[0]] + dense_v
    if tail:
        tail_k, tail_v = _random(3, (1, heads, tail, 128), dtype), _random(4, (1, heads, tail, 128), dtype)
        args.update(residual_key=to_device(tail_k, dtype), residual_value=to_device(tail_v, dtype))
        pieces_k.append(tail_k[0])
        pieces_v.append(tail_v[0])
    state = PackedDecodeState(keys, values)
    assert not state._preset and not state._inquant_values
    query = to_device(q, dtype).view(1, q_heads, 1, 128)
    actual = state.decode(query, **args)
    assert state._workspace.ndim == 2            # the streaming kernel took the call
    _check(actual, _expected(q, pieces_k, pieces_v))
    general = state._decode_general(query, heads, q_heads // heads, blocks, args["sink_key"], args["sink_value"], 4,
                                    args.get("residual_key"), args.get("residual_value"), tail, 128 ** -0.5)
    attention_close(to_numpy(actual.float()).reshape(q_heads, 128), to_numpy(general.float()).reshape(q_heads, 128))
    from inquant import _native as N
    assert N.take_status(torch.device("cuda", 0)) == 0


def test_streaming_and_general_kernel_agree_on_random_shapes_and_value_codecs():
    """Forty seeded random configurations (value codec, block length 64/128/256, KV heads, query heads per KV
    head up to 16, 1..40 blocks, sink and tail lengths, dtype, donor policy): the one-launch kernel and the
    general kernel are two independent implementations of the same contract and must agree."""
    CodecConfig, quantize, quantize_values, PackedDecodeState, _, _ = _mods()
    from inquant import _native as N
    rng = np.random.default_rng(20240)
    dev = torch.device("cuda", 0)
    codecs = {"preset": (2, 64), "v4g32": (4, 32), "v4g64": (4, 64), "v4g128": (4, 128), "v2g128": (2, 128), "v2g32": (2, 32)}
    for case in range(40):
        kind = str(rng.choice(["coded", *codecs]))
        block, heads = int(rng.choice([64, 128, 256])), int(rng.choice([1, 2, 4, 8]))
        group = int(rng.choice([1, 2, 4, 7, 8, 9, 16]))
        blocks = int(rng.integers(1, 40 if heads <= 2 else 16))
        tail, sink = int(rng.choice([0, 1, 15, 16, 17, 100, 300])), int(rng.choice([0, 2, 4]))
        dtype = torch.bfloat16 if rng.random() < 0.6 else torch.float16
        cfg = CodecConfig(salient_fraction=0.125, donor_policy="min_error" if rng.random() < 0.5 else "neighbors")
        gen = torch.Generator(device=dev).manual_seed(5000 + case)
        boost = torch.ones(128, device=dev)
        boost[torch.from_numpy(rng.integers(0, 128, size=3)).to(dev)] = 8.0

        def randn(*shape):
            return torch.randn(shape, device=dev, generator=gen)

        keys = [quantize((randn(1, heads, block, 128) * boost).to(dtype), cfg) for _ in range(blocks)]
        if kind == "coded":
            values = [quantize((randn(1, heads, block, 128) * boost + 0.3).to(dtype), cfg) for _ in range(blocks)]
        else:
            values = [quantize_values((randn(1, heads, block, 128) + 0.3).to(dtype), *codecs[kind]) for _ in range(blocks)]
        query = randn(1, heads * group, 1, 128).to(dtype)
        dense = {}
        if sink:
            dense.update(sink_key=randn(1, heads, sink, 128).to(dtype), sink_value=randn(1, heads, sink, 128).to(dtype))
        if tail:
            dense.update(residual_key=randn(1, heads, tail, 128).to(dtype), residual_value=randn(1, heads, tail, 128).to(dtype))
        state = PackedDecodeState(keys, values)
        assert state.streaming_value_kind() is not None
        fast = state.decode(query, **dense).float().reshape(heads * group, 128)
        general = state._decode_general(query, heads, group, blocks, dense.get("sink_key"), dense.get("sink_value"), sink,
                                        dense.get("residual_key"), dense.get("residual_value"), tail, 128 ** -0.5)
        general = general.float().reshape(heads * group, 128)
        label = (case, kind, block, heads, group, blocks, tail, sink, dtype)
        assert torch.isfinite(fast).all(), label
        assert (fast - general).abs().max().item() < 2e-2 + 8e-3 * general.abs().max().item(), label
        assert torch.nn.functional.cosine_similarity(fast, general, dim=1).min().item() > 0.9999, label
        assert N.take_status(dev) == 0, label


def test_general_kernel_dense_only_fp32():
    _, _, _, _, _, packed_decode = _mods()
    k, v, q = _random(7, (1, 2, 150, 128), "float32"), _random(8, (1, 2, 150, 128), "float32"), _random(9, (6, 128), "float32")
    out = packed_decode(to_device(q, "float32").view(1, 6, 1, 128), [], [],
                        residual_key=to_device(k, "float32"), residual_value=to_device(v, "float32"))
    attention_close(to_numpy(out).reshape(6, 128), oracle.attention_decode(q, k[0], v[0], 128 ** -0.5),
                    max_abs=1e-4, cosine=0.999999)
