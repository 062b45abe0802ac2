"""Worker of tests/test_split_kv_multigpu.py: run under torch.distributed.run with one process
per GPU.  One request is sharded by sequence over the ranks; the split decode must reproduce the
unsplit decode with every exchange (all-gather, peer memory, peer memory inside the decode launch),
eagerly and from a CUDA graph."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(os.path.dirname(HERE), "inquant-open-source_b200"))


def main() -> None:
    import workloads
    from inquant import _native as N
    from inquant.batched import DecodeBatch, SequenceState
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.split_kv import SplitKVDecode, shard_layer
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    device = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    heads, q_heads, layers = 4, 28, 3

    def on_device(x32):
        return torch.from_numpy(np.ascontiguousarray(x32)).to(torch.bfloat16).to(device)

    cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), block_size=64, residual_length=32,
                                     sink_tokens=4, value_bits=2, validate_positions=False))
    for layer in range(layers):                      # the same cache on every rank
        k, v = workloads.make_kv(40 + layer, heads, 1500)
        cache.update(on_device(k), on_device(v), layer)
    queries = [on_device(np.stack([workloads.make_query(60 + 10 * s + i, q_heads) for i in range(layers)])) for s in range(6)]
    full = DecodeBatch([SequenceState.from_cache_layer(cache, i) for i in range(layers)], q_heads, torch.bfloat16)
    expected = []
    for q in queries:
        full.queries.copy_(q)
        expected.append(full.attend().clone())
    results = {}
    for exchange in ("nccl", "p2p", "fused"):
        split = SplitKVDecode([shard_layer(cache, i, world, rank) for i in range(layers)], q_heads,
                              owns_tail=False, exchange=exchange)
        assert split.exchange == exchange
        outs = []
        for q in queries[:3]:
            split.batch.queries.copy_(q)
            outs.append(split.step(append=False).clone())
        split.capture()
        for q in queries[3:]:
            split.batch.queries.copy_(q)
            outs.append(split.replay().clone())
        torch.cuda.synchronize()
        assert N.take_status(device) == 0
        results[exchange] = outs
        for got, want in zip(outs, expected):
            # the merge order differs from the unsplit kernel's: one bf16 ulp (2^-7 relative) of slack
            assert torch.allclose(got.float(), want.float(), atol=4e-3, rtol=2.0 ** -7), exchange
    for a, b, c in zip(results["nccl"], results["p2p"], results["fused"]):
        assert torch.equal(a, b) and torch.equal(a, c)
    dist.barrier()
    split.peers.close()
    dist.destroy_process_group()
    print(f"split-kv rank {rank} of {world}: ok", flush=True)


if __name__ == "__main__":
    main()
