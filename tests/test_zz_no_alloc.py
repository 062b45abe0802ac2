"""The allocation-free decode entry point (`inq_decode_attention_noalloc`).

Some callers of this library cannot allocate device memory when they decode: a serving engine
that gave the whole device to its page pool at start-up, or a host runtime that owns all device
memory itself.  For them the library keeps the
split-KV scratch in a fixed device array.  This test drives that entry point directly through
the C ABI and checks it against the ordinary entry point (which uses caller-provided scratch)
on two consecutive calls, because the fixed array keeps the previous call's contents.

The file name sorts last on purpose: a failure here must not hide the other tests' results.
"""
import ctypes

import numpy as np
import pytest
import torch

import inquant_oracle as oracle
import workloads
from helpers import attention_close, to_device, to_numpy

pytestmark = pytest.mark.gpu


def _noalloc_decode(N, state, query, sink_k, sink_v, tail_k, tail_v, scale):
    """Fill inq_decode_seq_t / inq_decode_args_t by hand and call the entry point."""
    output = torch.empty_like(query)
    seq = N.DecodeSeq()
    seq.query, seq.output, seq.query_head_stride = query.data_ptr(), output.data_ptr(), query.stride(1)
    seq.table, seq.roles = state._tables.data_ptr(), state._key_map.data_ptr()
    seq.n_blocks = len(state.key_blocks)
    seq.sink_key, seq.sink_value = sink_k.data_ptr(), sink_v.data_ptr()
    seq.sink_key_stride_h, seq.sink_key_stride_t = sink_k.stride(1), sink_k.stride(2)
    seq.sink_value_stride_h, seq.sink_value_stride_t = sink_v.stride(1), sink_v.stride(2)
    seq.tail_key, seq.tail_value = tail_k.data_ptr(), tail_v.data_ptr()
    seq.tail_key_stride_h, seq.tail_key_stride_t = tail_k.stride(1), tail_k.stride(2)
    seq.tail_value_stride_h, seq.tail_value_stride_t = tail_v.stride(1), tail_v.stride(2)
    seq.sink_tokens, seq.tail_tokens = sink_k.shape[2], tail_k.shape[2]
    args = N.DecodeArgs()
    args.n_seq, args.seq_host = 1, ctypes.pointer(seq)
    args.kv_heads, args.q_per_kv = state._kv_heads, query.shape[1] // state._kv_heads
    args.block_tokens, args.n_pad = state._packed_tokens, state._salient
    args.layout, args.dtype, args.scale = 0, N.DTYPE_CODE[query.dtype], scale
    args.status = N.status_word(query.device).data_ptr()
    # partials / partials_floats / counters stay NULL: the entry point must not need them
    rc = N.library().inq_decode_attention_noalloc(ctypes.byref(args), N.stream_pointer(query.device))
    assert rc == N.OK, rc
    return output


def _oracle_view_output(view, q32):
    """The oracle's attention over the blocks of a cache view (their device bytes), the exact sink
    and the exact tail."""
    def host(t):
        return to_numpy(t.float() if t.dtype == torch.bfloat16 else t)
    keys, values = [host(view.sink_key)[0]], [host(view.sink_value)[0]]
    for kb, vb in zip(view.key_blocks, view.value_blocks):
        pk = oracle.PackedK(host(kb.payload), host(kb.scales), host(kb.salient_channels), host(kb.donor_channels),
                            host(kb.padding), tuple(kb.shape), "bfloat16")
        pv = oracle.PackedV(host(vb.payload), scales=host(vb.scales), offsets=host(vb.offsets), shape=tuple(vb.shape),
                            dtype="bfloat16", bits=2, group_size=64)
        keys.append(oracle.dequantize_k4(pk)[0])
        values.append(oracle.dequantize_values(pv)[0])
    keys.append(host(view.residual_key)[0])
    values.append(host(view.residual_value)[0])
    return oracle.attention_decode(q32, np.concatenate(keys, 1), np.concatenate(values, 1), 128 ** -0.5)


def test_noalloc_entry_point_matches_regular_entry_point_and_oracle_twice():
    from inquant import _native as N
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.triton_attention import PackedDecodeState
    heads, q_heads, tokens = 4, 28, 1500
    k, v = workloads.make_kv(77, heads, tokens)
    cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), block_size=256, residual_length=128,
                                     sink_tokens=4, value_bits=2, validate_positions=False))
    kt, vt = to_device(k), to_device(v)
    cache.update(kt[:, :, :tokens - 1], vt[:, :, :tokens - 1], 0)
    view = cache.append_for_attention(kt[:, :, tokens - 1:], vt[:, :, tokens - 1:], 0)
    state = PackedDecodeState(view.key_blocks, view.value_blocks)
    scale = 128 ** -0.5
    for call in range(2):   # two calls in a row share the fixed scratch
        q32 = workloads.make_query(500 + call, q_heads)
        q = to_device(q32).view(1, q_heads, 1, 128)
        expected = state.decode(q, sink_key=view.sink_key, sink_value=view.sink_value,
                                residual_key=view.residual_key, residual_value=view.residual_value, scale=scale)
        actual = _noalloc_decode(N, state, q, view.sink_key, view.sink_value, view.residual_key, view.residual_value, scale)
        torch.cuda.synchronize()
        attention_close(to_numpy(actual.float()).reshape(q_heads, 128), to_numpy(expected.float()).reshape(q_heads, 128))
        assert torch.equal(actual, expected)   # same kernel, same work split: identical bits
        attention_close(to_numpy(actual.float()).reshape(q_heads, 128), _oracle_view_output(view, q32))
    assert N.take_status(q.device) == 0


def test_noalloc_entry_point_serves_a_batch_close_to_its_pair_limit():
    """63 sequences x 4 KV heads = 252 of the 256 pairs the fixed scratch holds, described by a
    device array of sequence records, twice in a row; every output equals the ordinary entry
    point's bit for bit and three of them are compared with the oracle."""
    from inquant import _native as N
    from inquant.batched import DecodeBatch, SequenceState
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    heads, q_heads, n_seq = 4, 28, 63
    config = CacheConfig(CodecConfig(donor_policy="min_error"), block_size=64, residual_length=32, sink_tokens=4,
                         value_bits=2, validate_positions=False)
    caches, raw = [], []
    for index in range(n_seq):
        tokens = 140 + 37 * (index % 5)          # 1 to 3 sealed blocks
        k, v = workloads.make_kv(900 + index, heads, tokens)
        cache = InQuantCache(config)
        cache.update(to_device(k), to_device(v), 0)
        caches.append(cache)
        raw.append((k, v))
    batch = DecodeBatch([SequenceState.from_cache_layer(c, 0) for c in caches], q_heads, torch.bfloat16)
    for call in range(2):
        q32 = workloads.bf16_exact(np.random.default_rng(60 + call).standard_normal((n_seq, q_heads, 128), dtype=np.float32))
        batch.queries.copy_(to_device(q32))
        expected = batch.attend().clone()
        args = N.DecodeArgs.from_buffer_copy(batch._decode_args)
        args.partials, args.partials_floats, args.counters = None, 0, None   # the entry point must not need them
        batch.outputs.zero_()
        rc = N.library().inq_decode_attention_noalloc(ctypes.byref(args), N.stream_pointer(batch.device))
        assert rc == N.OK, rc
        torch.cuda.synchronize()
        assert torch.equal(batch.outputs, expected)
        for index in (0, 31, 62):
            k, v = raw[index]
            take, blocks, tail = oracle.seal_plan(0, 0, k.shape[2], sink_tokens=4, residual_length=32, block_size=64)
            pieces_k, pieces_v = [k[0, :, :take]], [v[0, :, :take]]
            for b in range(blocks):
                sl = slice(take + b * 64, take + (b + 1) * 64)
                pieces_k.append(oracle.dequantize_k4(oracle.quantize_k4(k[:, :, sl], donor_policy="min_error"))[0])
                pieces_v.append(oracle.dequantize_values(oracle.quantize_values(v[:, :, sl]))[0])
            pieces_k.append(k[0, :, take + blocks * 64:])
            pieces_v.append(v[0, :, take + blocks * 64:])
            want = oracle.attention_decode(q32[index], np.concatenate(pieces_k, 1), np.concatenate(pieces_v, 1), 128 ** -0.5)
            attention_close(to_numpy(batch.outputs[index].float()), want)
    assert N.take_status(batch.device) == 0


def test_noalloc_entry_point_rejects_sizes_beyond_its_fixed_scratch():
    from inquant import _native as N
    args = N.DecodeArgs()
    args.n_seq, args.kv_heads, args.q_per_kv = 65, 4, 7    # 260 pairs > 256
    rc = N.library().inq_decode_attention_noalloc(ctypes.byref(args), N.stream_pointer(torch.device("cuda", 0)))
    assert rc == N.ERR_CAPACITY
