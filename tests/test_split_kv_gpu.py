"""Split-KV kernels on one GPU: the ranks of a split are emulated one after another (each
builds its own batch over its share of the blocks), their partial records are stacked as an
all-gather would deliver them, and the merge kernel must reproduce the unsplit decode."""
import numpy as np
import pytest
import torch

import workloads
from helpers import attention_close, to_device, to_numpy

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_emulated_ranks_merge_to_the_unsplit_result(world):
    from inquant.batched import DecodeBatch, SequenceState
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.split_kv import merge_records, shard_layer
    heads, q_heads, layers = 4, 28, 3
    cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), block_size=64, residual_length=32,
                                     sink_tokens=4, value_bits=2, validate_positions=False))
    for layer, tokens in enumerate((1000, 1000, 1000)):
        k, v = workloads.make_kv(40 + layer, heads, tokens)
        cache.update(to_device(k), to_device(v), layer)
    full = DecodeBatch([SequenceState.from_cache_layer(cache, i) for i in range(layers)], q_heads, torch.bfloat16)
    q = to_device(np.stack([workloads.make_query(60 + i, q_heads) for i in range(layers)]))
    full.queries.copy_(q)
    expected = full.attend().clone()
    records = []
    for rank in range(world):
        part = DecodeBatch([shard_layer(cache, i, world, rank) for i in range(layers)], q_heads, torch.bfloat16,
                           partials_only=True)
        part.queries.copy_(q)
        part.attend()
        records.append(part.partial_records.view(-1, 130).clone())
    merged = torch.empty((layers * q_heads, 128), dtype=torch.bfloat16, device="cuda")
    merge_records(torch.stack(records).contiguous(), merged)
    torch.cuda.synchronize()
    attention_close(to_numpy(merged.float()), to_numpy(expected.float()).reshape(-1, 128), max_abs=8e-3, cosine=0.99999)
    from inquant import _native as N
    assert N.take_status(torch.device("cuda", 0)) == 0


def test_single_rank_driver_graph_replay_matches_eager_steps():
    """SplitKVDecode on one rank (no process group): a captured step replays to the same outputs
    as eager steps that see the same appended tokens."""
    from inquant.batched import SequenceState
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.split_kv import SplitKVDecode
    heads, q_heads, layers = 2, 14, 2
    config = CacheConfig(CodecConfig(donor_policy="min_error"), block_size=64, residual_length=32, sink_tokens=4,
                         value_bits=2, validate_positions=False)

    def build():
        cache = InQuantCache(config)
        for layer in range(layers):
            k, v = workloads.make_kv(70 + layer, heads, 500)
            cache.update(to_device(k), to_device(v), layer)
        return SplitKVDecode([SequenceState.from_cache_layer(cache, i) for i in range(layers)], q_heads, owns_tail=True)

    gen = torch.Generator(device="cuda").manual_seed(3)
    steps = torch.randn((4, layers, q_heads + 2 * heads, 128), device="cuda", generator=gen).bfloat16()
    eager, graphed = build(), build()
    expected = []
    for i in range(4):
        eager.inputs.copy_(steps[i])
        expected.append(eager.step().clone())
    graphed.inputs.copy_(steps[0])
    assert torch.equal(graphed.step(), expected[0])
    graphed.capture()
    for i in range(1, 4):
        graphed.inputs.copy_(steps[i])
        assert torch.equal(graphed.replay(), expected[i])
    with pytest.raises(RuntimeError, match="capture"):
        build().replay()
