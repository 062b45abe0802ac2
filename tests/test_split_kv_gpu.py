"""Split-KV kernels on one GPU: the ranks of a split are emulated one after another (each
builds its own batch over its share of the blocks), their partial records are stacked as an
all-gather would deliver them, and the merge kernel must reproduce the unsplit decode."""
import numpy as np
import pytest
import torch

import workloads
from helpers import attention_close, to_device, to_numpy

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,value_bits,block", [(1, 2, 64), (2, 2, 64), (3, 2, 64), (8, 2, 64), (3, None, 128), (2, 4, 128)])
def test_emulated_ranks_merge_to_the_unsplit_result(world, value_bits, block):
    from inquant.batched import DecodeBatch, SequenceState
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.split_kv import merge_records, shard_layer
    heads, q_heads, layers = 4, 28, 3
    cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), block_size=block, residual_length=32,
                                     sink_tokens=4, value_bits=value_bits, validate_positions=False))
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


def _emulated_exchange(records, steps=1, spin_limit=0, only_rank=None):
    """All ranks of an exchange inside one cooperative launch on this GPU (or, with ``only_rank``,
    that rank alone next to inboxes nobody writes).  ``records`` [world, rows, 130]."""
    import ctypes
    from inquant import _native as N
    lib = N.library()
    world, rows = records.shape[0], records.shape[1]
    device = records.device
    inboxes = [torch.zeros(lib.inq_exchange_inbox_bytes(world, rows), dtype=torch.uint8, device=device) for _ in range(world)]
    table = (ctypes.c_void_p * world)(*[b.data_ptr() for b in inboxes])
    epochs = torch.zeros((world, 2), dtype=torch.int32, device=device)
    outs = torch.full((world, rows, 128), 7.0, dtype=torch.bfloat16, device=device)
    ranks = range(world) if only_rank is None else [only_rank]
    entries = (N.ExchangeRank * len(ranks))(*[
        N.ExchangeRank(records[r].data_ptr(), table, outs[r].data_ptr(), epochs[r].data_ptr(),
                       N.status_word(device).data_ptr(), r) for r in ranks])
    args = N.ExchangeArgs(entries, len(ranks), world, rows, N.DTYPE_CODE[torch.bfloat16], spin_limit)
    for _ in range(steps):
        N.check(lib.inq_exchange_merge(ctypes.byref(args), N.stream_pointer(device)), "inq_exchange_merge")
    torch.cuda.synchronize()
    return outs, epochs


@pytest.mark.parametrize("world,rows", [(2, 84), (3, 61), (8, 84), (2, 4500)])
def test_peer_exchange_protocol_with_all_ranks_in_one_cooperative_launch(world, rows):
    """Push, per-chunk flags, wait and merge of inq_exchange_merge: every emulated rank must end
    with exactly what the all-gather + inq_merge_partials path computes, on odd and even steps."""
    from inquant import _native as N
    from inquant.split_kv import merge_records
    gen = torch.Generator(device="cuda").manual_seed(world * 1000 + rows)
    records = torch.randn((world, rows, 130), device="cuda", generator=gen)
    records[:, :, 128] *= 8.0                       # running maxima, base-2 units
    records[:, :, 129] = records[:, :, 129].abs() + 0.5
    expected = merge_records(records.contiguous(), torch.empty((rows, 128), dtype=torch.bfloat16, device="cuda"))
    for steps in (1, 2, 3):
        outs, epochs = _emulated_exchange(records, steps=steps)
        assert N.take_status(torch.device("cuda", 0)) == 0
        assert epochs[:, 0].tolist() == [steps] * world and epochs[:, 1].tolist() == [0] * world
        for r in range(world):
            assert torch.equal(outs[r], expected)


def test_peer_exchange_wait_gives_up_and_reports_when_a_peer_never_signals():
    """Rank 0 of a two-rank exchange alone: the flag of rank 1 is never set, so the bounded wait
    runs out, the status word carries the timeout bit and the rows are zeroed."""
    from inquant import _native as N
    records = torch.ones((2, 20, 130), device="cuda")
    outs, epochs = _emulated_exchange(records, spin_limit=200, only_rank=0)
    assert N.take_status(torch.device("cuda", 0)) == N.STATUS_WAIT_TIMEOUT
    assert int(epochs[0, 0]) == 1
    assert torch.count_nonzero(outs[0]) == 0


def _fused_rank(cache, layers, q_heads, world, rank, q, peer_records=None, spin_limit=0, steps=1):
    """One rank of a split whose decode launch exchanges its records itself.  The peers do not
    run: their inboxes are buffers of this process that soak up the pushes, and ``peer_records``
    ([world, rows, 130]) stand in this rank's inbox as the peers would have stored them for the steps
    run here (every word tagged with its step number: step 1 in the odd half, step 2 in the even one)."""
    import ctypes
    from inquant import _native as N
    from inquant.batched import DecodeBatch
    from inquant.split_kv import shard_layer
    lib = N.library()
    device = torch.device("cuda", 0)
    rows = layers * q_heads
    size = lib.inq_decode_exchange_inbox_bytes(world, rows)
    flag_bytes = 2 * 8 * 512 * 4
    inboxes = [torch.zeros(size, dtype=torch.uint8, device=device) for _ in range(world)]
    if peer_records is not None:
        words = inboxes[rank][flag_bytes:].view(torch.int32).view(2, world, rows, 130, 2)
        for src in range(world):
            if src != rank:
                words[:, src, :, :, 0] = peer_records[src].view(torch.int32)
                words[1, src, :, :, 1] = 1     # step 1 uses the odd half of the double buffer
                words[0, src, :, :, 1] = 2     # step 2 the even one
    epoch = torch.zeros(2, dtype=torch.int32, device=device)
    view = N.DecodeExchange()
    for peer in range(world):
        view.inboxes[peer] = inboxes[peer].data_ptr()
    view.epoch, view.n_rows, view.world, view.rank, view.spin_limit = epoch.data_ptr(), rows, world, rank, spin_limit
    view_device = torch.frombuffer(bytearray(bytes(view)), dtype=torch.uint8).to(device)
    batch = DecodeBatch([shard_layer(cache, i, world, rank) for i in range(layers)], q_heads, torch.bfloat16)
    batch.use_exchange(view_device)
    batch.queries.copy_(q)
    outs = []
    for _ in range(steps):
        outs.append(batch.attend().clone())
    torch.cuda.synchronize()
    return outs, epoch, inboxes


def _split_fixture(layers=3, heads=4, tokens=1000):
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), block_size=64, residual_length=32,
                                     sink_tokens=4, value_bits=2, validate_positions=False))
    for layer in range(layers):
        k, v = workloads.make_kv(140 + layer, heads, tokens)
        cache.update(to_device(k), to_device(v), layer)
    return cache


@pytest.mark.parametrize("world", [1, 2, 4])
def test_decode_launch_that_exchanges_its_records_matches_the_gathered_merge(world):
    """The exchange inside the decode launch (inq_decode_exchange_t): every rank, run alone with the
    peers' records already in its inbox, must write exactly the rows that all-gather +
    inq_merge_partials give, must leave its own records (every word tagged with the step) in the
    peers' inboxes, and must advance the step number; two steps use both halves of the double-buffered
    inbox."""
    from inquant import _native as N
    from inquant.batched import DecodeBatch
    from inquant.split_kv import merge_records, shard_layer
    layers, q_heads = 3, 28
    cache = _split_fixture(layers)
    q = to_device(np.stack([workloads.make_query(160 + i, q_heads) for i in range(layers)]))
    records = []
    for rank in range(world):
        part = DecodeBatch([shard_layer(cache, i, world, rank) for i in range(layers)], q_heads, torch.bfloat16,
                           partials_only=True)
        part.queries.copy_(q)
        part.attend()
        records.append(part.partial_records.view(-1, 130).clone())
    records = torch.stack(records).contiguous()
    expected = merge_records(records, torch.empty((layers * q_heads, 128), dtype=torch.bfloat16, device="cuda"))
    flag_bytes = 2 * 8 * 512 * 4
    for rank in range(world):
        outs, epoch, inboxes = _fused_rank(cache, layers, q_heads, world, rank, q, peer_records=records, steps=2)
        assert N.take_status(torch.device("cuda", 0)) == 0
        assert int(epoch[0]) == 2
        for out in outs:
            assert torch.equal(out.view(-1, 128), expected)
        for peer in range(world):
            if peer == rank:
                continue
            pushed = inboxes[peer][flag_bytes:].view(torch.int32).view(2, world, layers * q_heads, 130, 2)
            want = records[rank].view(torch.int32)
            assert torch.equal(pushed[0, rank, :, :, 0], want) and torch.equal(pushed[1, rank, :, :, 0], want)
            assert bool((pushed[1, rank, :, :, 1] == 1).all()) and bool((pushed[0, rank, :, :, 1] == 2).all())
            others = [src for src in range(world) if src != rank]
            assert int(pushed[:, others].abs().sum()) == 0 and int(inboxes[peer][:flag_bytes].sum()) == 0


def test_decode_launch_exchange_gives_up_when_a_peer_never_publishes():
    """Rank 0 of two, alone: rank 1's words never arrive, the bounded wait of every pair runs out,
    the status word carries the timeout bit, the rows are zero and the context stays usable."""
    from inquant import _native as N
    layers, q_heads = 2, 28
    cache = _split_fixture(layers)
    q = to_device(np.stack([workloads.make_query(170 + i, q_heads) for i in range(layers)]))
    outs, epoch, _ = _fused_rank(cache, layers, q_heads, 2, 0, q, peer_records=None, spin_limit=100)
    assert N.take_status(torch.device("cuda", 0)) == N.STATUS_WAIT_TIMEOUT
    assert int(epoch[0]) == 1 and torch.count_nonzero(outs[0]) == 0
    again, _, _ = _fused_rank(cache, layers, q_heads, 1, 0, q)
    assert N.take_status(torch.device("cuda", 0)) == 0 and torch.count_nonzero(again[0]) > 0
