"""The allocation-free decode entry point (`inq_decode_attention_noalloc`).

Some callers of this library cannot allocate device memory when they decode: a serving engine
that gave the whole device to its page pool at start-up, a host runtime that owns all device
memory itself, or code that runs inside a CUDA-graph capture.  For them the library keeps the
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


def test_noalloc_entry_point_matches_regular_entry_point_twice():
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
        q = to_device(workloads.make_query(500 + call, q_heads)).view(1, q_heads, 1, 128)
        expected = state.decode(q, sink_key=view.sink_key, sink_value=view.sink_value,
                                residual_key=view.residual_key, residual_value=view.residual_value, scale=scale)
        actual = _noalloc_decode(N, state, q, view.sink_key, view.sink_value, view.residual_key, view.residual_value, scale)
        torch.cuda.synchronize()
        attention_close(to_numpy(actual.float()).reshape(q_heads, 128), to_numpy(expected.float()).reshape(q_heads, 128))
        assert torch.equal(actual, expected)   # same kernel, same work split: identical bits
    assert N.take_status(q.device) == 0


def test_noalloc_entry_point_rejects_sizes_beyond_its_fixed_scratch():
    from inquant import _native as N
    args = N.DecodeArgs()
    args.n_seq, args.kv_heads, args.q_per_kv = 65, 4, 7    # 260 pairs > 256
    rc = N.library().inq_decode_attention_noalloc(ctypes.byref(args), N.stream_pointer(torch.device("cuda", 0)))
    assert rc == N.ERR_CAPACITY
