"""Paged K4/V2 decode: no dense history, no host page lookup (reference
``inquant_vllm/kernels.py``).  One sm_100a launch (C ABI ``inq_decode_attention``, page layout)
covers the packed pages, the exact sink and the exact tail, and merges the partials."""
import ctypes

import torch

from inquant import _native as N
from inquant.triton_attention import pair_units, workspace_floats


def fill_paged_sequence(seq, query, output, cache, blocks, dense, num_pages, tail_tokens, sink_tokens, layout):
    """Fill one ``inq_decode_seq_t`` for the page layout; ``dense`` is ``[2,H,B+4,128]`` with the
    sink in tokens 0..3 and the unsealed tail from token 4 (reference ``backend.py:130-163``)."""
    es = dense.element_size()
    plane = dense.stride(0)
    seq.query, seq.output, seq.query_head_stride = query.data_ptr(), output.data_ptr(), 128
    seq.pool, seq.page_table, seq.n_blocks = cache.data_ptr(), blocks.data_ptr(), num_pages
    seq.pool_pages = cache.shape[0]   # page ids are checked on the device against the pool size
    seq.sink_key, seq.sink_value = dense.data_ptr(), dense.data_ptr() + plane * es
    seq.tail_key = dense.data_ptr() + 4 * dense.stride(2) * es
    seq.tail_value = seq.tail_key + plane * es
    for name in ("sink_key", "sink_value", "tail_key", "tail_value"):
        setattr(seq, name + "_stride_h", dense.stride(1))
        setattr(seq, name + "_stride_t", dense.stride(2))
    seq.sink_tokens, seq.tail_tokens = sink_tokens, tail_tokens
    # packed tokens covered by the exact sink are masked; so are tail tokens that the sink holds
    seq.first_visible = sink_tokens
    seq.tail_skip = max(0, sink_tokens - num_pages * layout.block_size)


def page_offsets_array(layout):
    o = layout.offsets
    return (ctypes.c_int64 * 6)(o['key_scales'], o['key_map'], o['key_padding'], o['value_payload'],
                                o['value_scales'], o['value_offsets'])


def paged_decode(query, cache, blocks, dense, num_pages, tail_tokens, sink_tokens, layout, workspace, scale, output=None):
    if query.shape[0] != 1 or query.shape[-1] != 128 or query.dtype != torch.bfloat16:
        raise ValueError("Paged decode expects one BF16 query [1, heads, 128]")
    hq, hkv = query.shape[1], layout.heads
    if hq % hkv or hq // hkv > 16:
        raise ValueError("Expected 1..16 query heads per KV head")
    N.require_cuda(query, "paged_decode")
    if not query.is_contiguous():
        query = query.contiguous()
    if blocks.dtype != torch.int32:
        blocks = blocks.to(torch.int32)
    if dense.dtype != query.dtype or tuple(dense.shape) != (2, hkv, layout.block_size + 4, 128) or not dense.is_contiguous():
        raise ValueError("dense must be a contiguous [2, KV_heads, block_size + 4, 128] tensor of the query dtype")
    if not (num_pages * layout.block_size + tail_tokens) and not sink_tokens:
        raise ValueError("Attention requires at least one key/value token")
    q_per_kv = hq // hkv
    pairs = hkv * ((q_per_kv + 7) // 8)
    floats = workspace_floats(pairs, pairs * pair_units(num_pages, layout.block_size))
    scratch = workspace.acquire((floats,), query.device)
    if output is None:
        output = torch.empty_like(query)
    elif not output.is_contiguous():
        raise ValueError("output must be contiguous")
    seq = N.DecodeSeq()
    fill_paged_sequence(seq, query, output, cache, blocks, dense, num_pages, tail_tokens, sink_tokens, layout)
    args = N.DecodeArgs()
    args.n_seq, args.seq_host = 1, ctypes.pointer(seq)
    args.kv_heads, args.q_per_kv, args.block_tokens, args.n_pad = hkv, q_per_kv, layout.block_size, 16
    args.layout, args.dtype, args.scale = 1, N.DTYPE_CODE[query.dtype], scale
    args.page_bytes, args.page_offsets = layout.page_bytes, page_offsets_array(layout)
    args.partials, args.partials_floats = scratch.data_ptr(), scratch.numel()
    args.counters = N.decode_counters(query.device, pairs).data_ptr()
    args.status = N.status_word(query.device).data_ptr()
    N.check(N.library().inq_decode_attention(ctypes.byref(args), N.stream_pointer(query.device)), "inq_decode_attention")
    return output
