"""One-launch batched decode (many (request, layer) sequences) vs per-sequence decode and the
CPU oracle: table layout with appends through device counters and CUDA-graph replay, and the
paged layout with requests of different lengths (the batched-serving configuration)."""
import numpy as np
import pytest
import torch

import inquant_oracle as oracle
import workloads
from helpers import attention_close, to_device, to_numpy

pytestmark = pytest.mark.gpu


def _cache(tokens, seed, heads=4, block=64, residual=32):
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    k, v = workloads.make_kv(seed, heads, tokens)
    cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), block_size=block, residual_length=residual,
                                     sink_tokens=4, value_bits=2, validate_positions=False))
    cache.update(to_device(k), to_device(v), 0)
    return cache, k, v


def _oracle_output(k, v, q, block, residual, extra_k=None, extra_v=None):
    total = k.shape[2]
    take, blocks, tail = oracle.seal_plan(0, 0, total, sink_tokens=4, residual_length=residual, block_size=block)
    pk, pv = [k[0, :, :take]], [v[0, :, :take]]
    for i in range(blocks):
        sl = slice(take + i * block, take + (i + 1) * block)
        pk.append(oracle.dequantize_k4(oracle.quantize_k4(k[:, :, sl], donor_policy="min_error"))[0])
        pv.append(oracle.dequantize_values(oracle.quantize_values(v[:, :, sl]))[0])
    pk.append(k[0, :, take + blocks * block:])
    pv.append(v[0, :, take + blocks * block:])
    if extra_k is not None:
        pk.append(extra_k)
        pv.append(extra_v)
    return oracle.attention_decode(q, np.concatenate(pk, 1), np.concatenate(pv, 1), 128 ** -0.5)


def test_table_batch_matches_per_sequence_decode_oracle_and_graph_replay():
    from inquant.batched import DecodeBatch, SequenceState
    lengths = (700, 333, 1290, 40)   # different block counts, one sequence without any sealed block
    caches = [_cache(n, 10 + i) for i, n in enumerate(lengths)]
    seqs = [SequenceState.from_cache_layer(c, 0) for c, _, _ in caches]
    batch = DecodeBatch(seqs, 28, torch.bfloat16)
    rng = np.random.default_rng(3)
    steps = 5
    new_q = [workloads.bf16_exact(rng.standard_normal((len(lengths), 28, 128), dtype=np.float32)) for _ in range(steps)]
    new_k = [workloads.bf16_exact(rng.standard_normal((len(lengths), 4, 128), dtype=np.float32)) for _ in range(steps)]
    new_v = [workloads.bf16_exact(rng.standard_normal((len(lengths), 4, 128), dtype=np.float32)) for _ in range(steps)]
    appended_k = [[] for _ in lengths]
    appended_v = [[] for _ in lengths]
    for step in range(steps):
        batch.queries.copy_(to_device(new_q[step]))
        batch.new_keys.copy_(to_device(new_k[step]))
        batch.new_values.copy_(to_device(new_v[step]))
        if step == 2:
            batch.capture()
        out = batch.replay() if step >= 2 else batch.step()
        torch.cuda.synchronize()
        for i, (cache, k, v) in enumerate(caches):
            appended_k[i].append(new_k[step][i][:, None, :])
            appended_v[i].append(new_v[step][i][:, None, :])
            want = _oracle_output(k, v, new_q[step][i], 64, 32, np.concatenate(appended_k[i], 1), np.concatenate(appended_v[i], 1))
            attention_close(to_numpy(out[i].float()), want)
    assert batch.tail_tokens == [s.tail_count + steps for s in seqs]
    assert to_numpy(batch.tail_counters).tolist() == batch.tail_tokens
    # the batch wrote into the caches' own tail buffers: a per-sequence decode sees the same tokens
    from inquant.triton_attention import PackedDecodeState
    for i, (cache, k, v) in enumerate(caches):
        layer = cache._layers[0]
        n = batch.tail_tokens[i]
        single = PackedDecodeState(layer.key_blocks, layer.value_blocks).decode(
            batch.queries[i].unsqueeze(0).unsqueeze(2).contiguous(), sink_key=layer.sink_key, sink_value=layer.sink_value,
            residual_key=layer.tail_key_buffer[:, :, :n], residual_value=layer.tail_value_buffer[:, :, :n])
        attention_close(to_numpy(single.float()).reshape(28, 128), to_numpy(batch.outputs[i].float()))
    from inquant import _native as N
    assert N.take_status(batch.device) == 0
    with pytest.raises(RuntimeError, match="full"):
        for _ in range(200):
            batch.step()


@pytest.mark.parametrize("value_bits,group", [(None, 64), (4, 32), (4, 128), (2, 128), (2, 32)])
def test_table_batch_of_other_value_codecs_matches_per_sequence_decode(value_bits, group):
    """Values stored as InQuant packed tensors (the reference's default), 4-bit values and 2-bit values in one
    group: the batched one-launch step (new token appended by the launch, CUDA-graph replay) equals the
    per-sequence decode over the same caches, which the decode tests check against the oracle."""
    from inquant.batched import DecodeBatch, SequenceState
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.triton_attention import PackedDecodeState
    from inquant import _native as N
    lengths = (900, 1300, 2100)
    caches = []
    for i, tokens in enumerate(lengths):
        k, v = workloads.make_kv(30 + i, 4, tokens)
        cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), block_size=128, residual_length=64,
                                         sink_tokens=4, value_bits=value_bits, value_group_size=group, validate_positions=False))
        cache.update(to_device(k), to_device(v), 0)
        caches.append(cache)
    seqs = [SequenceState.from_cache_layer(c, 0) for c in caches]
    batch = DecodeBatch(seqs, 28, torch.bfloat16)
    assert (batch.value_kind, batch.value_groups) == {None: (1, 0), 4: (2, 128 // group), 2: (0, 128 // group)}[value_bits]
    gen = torch.Generator(device="cuda").manual_seed(11)
    steps = torch.randn((4, len(lengths), 28 + 8, 128), device="cuda", generator=gen).bfloat16()
    for step in range(4):
        batch.inputs.copy_(steps[step])
        if step == 2:
            batch.capture()
        out = batch.replay() if step >= 2 else batch.step()
        torch.cuda.synchronize()
        for i, cache in enumerate(caches):
            layer = cache._layers[0]
            n = batch.tail_tokens[i]
            single = PackedDecodeState(layer.key_blocks, layer.value_blocks).decode(
                batch.queries[i].unsqueeze(0).unsqueeze(2).contiguous(), sink_key=layer.sink_key, sink_value=layer.sink_value,
                residual_key=layer.tail_key_buffer[:, :, :n], residual_value=layer.tail_value_buffer[:, :, :n])
            attention_close(to_numpy(single.float()).reshape(28, 128), to_numpy(out[i].float()), max_abs=8e-3, cosine=0.99999)
    assert N.take_status(batch.device) == 0


@pytest.mark.parametrize("block,heads,q_heads", [(16, 8, 32), (64, 4, 28)])
def test_paged_batch_of_requests_with_different_lengths(block, heads, q_heads):
    """Batched paged decode: requests of seeded lengths, shuffled physical pages, one launch."""
    from inquant.batched import DecodeBatch, PagedSequenceState
    from inquant_vllm.layout import PageLayout, pack_pages_into
    layout = PageLayout(block, heads)
    rng = np.random.default_rng(11)
    lengths = [int(x) for x in rng.integers(3, 40 * block, size=6)] + [2, block, 4 * block + 1]
    total_pages = sum(n // block for n in lengths)
    pool = torch.zeros((total_pages + 5, layout.page_bytes), dtype=torch.uint8, device="cuda")
    free = torch.randperm(total_pages + 5, generator=torch.Generator().manual_seed(1)).tolist()
    seqs, expected, queries = [], [], []
    for i, n in enumerate(lengths):
        k, v = workloads.make_kv(100 + i, heads, n)
        pages, tail, sink = n // block, n % block, min(4, n)
        ids = torch.tensor([free.pop() for _ in range(pages)], dtype=torch.int32, device="cuda")
        dense = torch.full((2, heads, block + 4, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        kd, vd = to_device(k[0]), to_device(v[0])
        dense[0, :, :sink], dense[1, :, :sink] = kd[:, :sink], vd[:, :sink]
        if tail:
            dense[0, :, 4:4 + tail], dense[1, :, 4:4 + tail] = kd[:, n - tail:], vd[:, n - tail:]
        kr, vr = k[0].copy(), v[0].copy()
        if pages:
            kt = np.ascontiguousarray(k[0][:, :pages * block].reshape(heads, pages, block, 128).transpose(1, 0, 2, 3))
            vt = np.ascontiguousarray(v[0][:, :pages * block].reshape(heads, pages, block, 128).transpose(1, 0, 2, 3))
            pack_pages_into(to_device(kt), to_device(vt), layout, pool, ids)
            dk, dv = oracle.unpack_pages(oracle.pack_pages(kt, vt, block, heads), block, heads)
            kr[:, :pages * block] = dk.transpose(1, 0, 2, 3).reshape(heads, -1, 128)
            vr[:, :pages * block] = dv.transpose(1, 0, 2, 3).reshape(heads, -1, 128)
            kr[:, :sink], vr[:, :sink] = k[0][:, :sink], v[0][:, :sink]
        q = workloads.make_query(200 + i, q_heads)
        queries.append(q)
        expected.append(oracle.attention_decode(q, kr, vr, 128 ** -0.5))
        seqs.append(PagedSequenceState(pool, ids, pages, dense, tail, sink, layout))
    batch = DecodeBatch(seqs, q_heads, torch.bfloat16)
    batch.queries.copy_(to_device(np.stack(queries)))
    out = batch.attend()
    torch.cuda.synchronize()
    for i in range(len(lengths)):
        attention_close(to_numpy(out[i].float()), expected[i])
    from inquant import _native as N
    assert N.take_status(batch.device) == 0
