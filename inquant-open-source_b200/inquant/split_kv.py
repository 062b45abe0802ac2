"""Split-KV decode of one long request across the GPUs of a node.

The sealed blocks of every layer are partitioned by sequence: rank r owns a contiguous range
of blocks (all layers, all KV heads), rank 0 also owns the exact sink and the last rank the
exact tail.  Each rank runs the ordinary one-launch decode over its share but keeps the
un-normalised ``(acc[128], m, l)`` record per (layer, query head) -- the reference's partial
format (``triton_attention.py:162-165``).  ONE ``all_gather`` per decode step moves the records
of all layers (``layers * q_heads * 130`` floats per rank, 408 KB for 28 x 28) over NVLink into
local memory, and a small kernel applies the log-sum-exp merge (``inq_merge_partials``, the
cross-rank form of ``triton_attention.py:168-181``).  Nothing else is exchanged: encode and
append are block-local.  The reference has no multi-GPU path; this module is new.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _native as N
from .batched import DecodeBatch, SequenceState
from .triton_attention import PackedDecodeState


def shard_blocks(n_blocks: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous block range [start, end) of ``rank``; earlier ranks take the remainder."""
    if world < 1 or not 0 <= rank < world or n_blocks < 0:
        raise ValueError("invalid shard request")
    base, extra = divmod(n_blocks, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_layer(cache, layer_idx: int, world: int, rank: int) -> SequenceState:
    """This rank's share of one cached layer as a decode sequence."""
    layer = cache._layers[layer_idx]
    start, end = shard_blocks(len(layer.key_blocks), world, rank)
    state = PackedDecodeState(layer.key_blocks[start:end], layer.value_blocks[start:end])
    if layer.tail_key_buffer is None:
        raise ValueError("the layer has no tail buffer yet")
    owns_sink, owns_tail = rank == 0, rank == world - 1
    return SequenceState(state, layer.sink_key if owns_sink else None, layer.sink_value if owns_sink else None,
                         layer.tail_key_buffer, layer.tail_value_buffer, layer.tail_count if owns_tail else 0)


def merge_records(records: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``records`` [parts, rows, 130] fp32 -> ``out`` [rows, 128] (fp16/bf16), on the current stream."""
    if records.dtype != torch.float32 or records.ndim != 3 or records.shape[2] != 130 or not records.is_contiguous():
        raise ValueError("records must be a contiguous [parts, rows, 130] float32 tensor")
    if out.shape != (records.shape[1], 128) or not out.is_contiguous() or out.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("out must be a contiguous [rows, 128] fp16/bf16 tensor")
    N.require_cuda(records, "merge_records")
    rc = N.library().inq_merge_partials(records.data_ptr(), records.shape[0], records.shape[1], out.data_ptr(),
                                        N.DTYPE_CODE[out.dtype], N.stream_pointer(records.device))
    N.check(rc, "inq_merge_partials")
    return out


class SplitKVDecode:
    """Per-rank driver: local decode over this rank's blocks, one all-gather, local merge."""

    def __init__(self, sequences: list[SequenceState], q_heads: int, group=None, dtype=torch.bfloat16,
                 owns_tail: bool | None = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.owns_tail = (self.rank == self.world - 1) if owns_tail is None else owns_tail
        self.batch = DecodeBatch(sequences, q_heads, dtype, partials_only=True)
        n = len(sequences)
        self.gathered = torch.empty((self.world, n * q_heads, 130), dtype=torch.float32, device=self.batch.device)
        self.outputs = torch.empty((n, q_heads, 128), dtype=dtype, device=self.batch.device)

    @property
    def inputs(self) -> torch.Tensor:
        return self.batch.inputs

    def step(self, append: bool = True) -> torch.Tensor:
        """One decode step; ``inputs`` must hold the same queries on every rank (and the new
        token's K/V on the rank that owns the tail)."""
        if append and self.owns_tail:
            self.batch.append()
        self.batch.attend()
        local = self.batch.partial_records.view(-1, 130)
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered.view(-1, 130), local, group=self.group)
        else:
            self.gathered[0].copy_(local)
        merge_records(self.gathered, self.outputs.view(-1, 128))
        return self.outputs

    def capture(self) -> None:
        """Record one step (append on the tail owner, local decode, all-gather, merge) into a CUDA
        graph; ``replay`` then costs one graph launch per step.  Run eager steps first: the first
        launches set kernel attributes and NCCL builds its communicator outside a capture."""
        graph = torch.cuda.CUDAGraph()
        counters = self.batch.tail_counters.clone()
        with torch.cuda.graph(graph):
            if self.owns_tail:
                self.batch._launch_append()
            self.batch._launch_attend()
            local = self.batch.partial_records.view(-1, 130)
            if self.world > 1:
                dist.all_gather_into_tensor(self.gathered.view(-1, 130), local, group=self.group)
            else:
                self.gathered[0].copy_(local)
            merge_records(self.gathered, self.outputs.view(-1, 128))
        self.batch.tail_counters.copy_(counters)
        self._graph = graph

    def replay(self) -> torch.Tensor:
        if getattr(self, "_graph", None) is None:
            raise RuntimeError("call capture() first")
        if self.owns_tail and self.batch.capacity_left < 1:
            raise RuntimeError("a tail buffer is full: seal a block before appending")
        self._graph.replay()
        if self.owns_tail:
            self.batch._appended += 1
        return self.outputs
