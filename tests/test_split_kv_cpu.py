"""Host-side logic of the split-KV path on CPU ranks (gloo, world size 2): block sharding,
the layout of the gathered partial records and the log-sum-exp merge (oracle arithmetic)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import inquant_oracle as oracle
import workloads


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (os.path.join(root, "inquant-open-source_b200"), os.path.join(root, "oracle")):
        sys.path.insert(0, p)
    from inquant.split_kv import shard_blocks
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    heads, q_heads, block, n_blocks, sink, tail = 2, 6, 16, 5, 4, 9
    tokens = sink + n_blocks * block + tail
    k, v = workloads.make_kv(5, heads, tokens)
    q = workloads.make_query(5, q_heads)
    start, end = shard_blocks(n_blocks, world, rank)
    pieces_k, pieces_v = [], []
    if rank == 0:
        pieces_k.append(k[0, :, :sink]); pieces_v.append(v[0, :, :sink])
    lo, hi = sink + start * block, sink + end * block
    pieces_k.append(k[0, :, lo:hi]); pieces_v.append(v[0, :, lo:hi])
    if rank == world - 1:
        pieces_k.append(k[0, :, sink + n_blocks * block:]); pieces_v.append(v[0, :, sink + n_blocks * block:])
    acc, m, l = oracle.attention_partial(q, np.concatenate(pieces_k, 1), np.concatenate(pieces_v, 1), 0.1)
    record = torch.from_numpy(np.concatenate([acc, m[:, None], l[:, None]], 1))   # [q_heads, 130]
    gathered = [torch.empty_like(record) for _ in range(world)]
    dist.all_gather(gathered, record)
    g = torch.stack(gathered).numpy()
    merged = oracle.merge_partials(g[:, :, :128], g[:, :, 128], g[:, :, 129])
    full = oracle.attention_decode(q, k[0], v[0], 0.1)
    np.save(os.path.join(out_dir, f"ok_{rank}.npy"), np.array([np.abs(merged - full).max()]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_cpu_ranks_gather_and_merge_partials(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        assert np.load(tmp_path / f"ok_{rank}.npy")[0] < 1e-12


def test_block_sharding_is_a_contiguous_partition():
    from inquant.split_kv import shard_blocks
    for n in (0, 1, 7, 127, 511):
        for world in (1, 2, 4, 8):
            ranges = [shard_blocks(n, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [b - a for a, b in ranges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_blocks(4, 2, 2)


def test_requests_are_dealt_by_length_to_the_least_loaded_rank():
    """Batched serving shards whole requests: every request lands on exactly one rank, the
    assignment is the same wherever it is computed, and the longest rank stays within one request
    of the mean for the bench's seeded lengths."""
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "inquant-open-source_b200"))
    from inquant.batched import shard_requests
    lengths = [int(x) for x in np.random.default_rng(2024).integers(4096, 32769, size=16)]
    for world in (1, 2, 4, 8):
        shards = shard_requests(lengths, world)
        assert sorted(i for shard in shards for i in shard) == list(range(16))
        assert shards == shard_requests(list(lengths), world)
        loads = [sum(lengths[i] for i in shard) for shard in shards]
        assert max(loads) - sum(loads) / world <= max(lengths)
        if world == 8:
            assert max(loads) <= 1.25 * sum(loads) / world
    assert shard_requests([5, 5, 5], 2) == [[0, 2], [1]]
    assert shard_requests([], 3) == [[], [], []]
    with pytest.raises(ValueError):
        shard_requests([1], 0)
