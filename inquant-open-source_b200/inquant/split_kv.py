"""Split-KV decode of one long request across the GPUs of a node.

The sealed blocks of every layer are partitioned by sequence: rank r owns a contiguous range
of blocks (all layers, all KV heads), rank 0 also owns the exact sink and the last rank the
exact tail.  Each rank runs the ordinary one-launch decode over its share but keeps the
un-normalised ``(acc[128], m, l)`` record per (layer, query head) -- the reference's partial
format (``triton_attention.py:162-165``).  The records of all layers (``layers * q_heads * 130``
floats per rank, 408 KB for 28 x 28) are exchanged once per decode step and merged by the
log-sum-exp rule (the cross-rank form of ``triton_attention.py:168-181``).  Two exchanges exist:

``"p2p"``   ``PeerExchange``: ONE kernel of this library per rank stores the records straight into
            every peer's inbox over NVLink peer memory (CUDA IPC mappings), signals per chunk,
            waits (bounded) for the peers' chunks and merges them (``inq_exchange_merge``);
``"nccl"``  one ``all_gather`` followed by the merge kernel ``inq_merge_partials``.

``"fused"`` no launch of its own: the decode kernel's merging CTA of every (layer, KV head, head tile)
            stores that pair's record into the peers' inboxes (every word with its step number: no
            fence, no flags), awaits theirs (bounded) and merges them (``inq_decode_exchange_t``), so a step
            is ONE launch per rank;

``"auto"`` takes peer memory inside the decode launch when every rank sits on the same host and the
mappings can be made (the fastest of the three as measured on 2, 4 and 8 GPUs), else the all-gather.  Nothing else is exchanged: encode and append are block-local.  The reference
has no multi-GPU path; this module is new.
"""
from __future__ import annotations

import ctypes
import socket

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


class PeerExchange:
    """This rank's inbox, mapped into every peer of the node, and the mappings of theirs.

    Collective over ``group``: every rank constructs it with the same ``n_rows`` and calls ``run``
    the same number of times.  ``run`` launches ONE kernel on the current stream (push to the
    peers, signal, bounded wait, merge); a wait that runs out sets the wait-timeout bit of the
    device status word (``_native.take_status``) instead of hanging.  Raises ``RuntimeError`` on
    every rank when the ranks span hosts or a mapping cannot be made.
    """

    def __init__(self, n_rows: int, device: torch.device, group=None, spin_limit: int = 0):
        if not dist.is_initialized():
            raise RuntimeError("PeerExchange needs an initialised process group")
        self.group, self.device, self.n_rows, self.spin_limit = group, device, int(n_rows), int(spin_limit)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        lib = N.library()
        if not 1 <= self.world <= 8:
            raise RuntimeError("PeerExchange serves at most 8 ranks")
        self._own = ctypes.c_void_p()
        self._opened: list[ctypes.c_void_p] = []
        handle = (ctypes.c_ubyte * 64)()
        error = None
        with torch.cuda.device(device):
            try:
                # sized for either form of the exchange (the decode launch's own tags every word: twice the bytes)
                N.check(lib.inq_peer_buffer_create(max(lib.inq_exchange_inbox_bytes(self.world, self.n_rows),
                                                       lib.inq_decode_exchange_inbox_bytes(self.world, self.n_rows)),
                                                   ctypes.byref(self._own), handle), "inq_peer_buffer_create")
            except (RuntimeError, ValueError) as exc:
                error = str(exc)
            offers = [None] * self.world
            dist.all_gather_object(offers, (socket.gethostname(), bytes(handle), error), group=group)
            pointers = [None] * self.world
            if error is None and any(o[2] for o in offers):
                error = "a peer could not create its inbox"
            if error is None and len({o[0] for o in offers}) != 1:
                error = "the ranks are not on one host"
            if error is None:
                for peer, (_, peer_handle, _) in enumerate(offers):
                    if peer == self.rank:
                        pointers[peer] = self._own.value
                        continue
                    mapped = ctypes.c_void_p()
                    rc = lib.inq_peer_buffer_open((ctypes.c_ubyte * 64).from_buffer_copy(peer_handle), ctypes.byref(mapped))
                    if rc != N.OK:
                        error = f"mapping the inbox of rank {peer} failed: {lib.inq_last_error().decode()}"
                        break
                    self._opened.append(mapped)
                    pointers[peer] = mapped.value
            verdicts = [None] * self.world
            dist.all_gather_object(verdicts, error, group=group)
        if any(verdicts):
            self.close()
            raise RuntimeError("peer exchange unavailable: " + next(v for v in verdicts if v))
        self._inboxes = (ctypes.c_void_p * self.world)(*pointers)
        self._epoch = torch.zeros(2, dtype=torch.int32, device=device)

    def decode_view(self) -> torch.Tensor:
        """This exchange as the decode kernel reads it (``inq_decode_exchange_t`` in device memory): the
        kernel then pushes, awaits and merges the records pair by pair itself.  An exchange serves
        either ``run`` or the decode kernel, not both: they lay the records out differently."""
        view = N.DecodeExchange()
        for peer in range(self.world):
            view.inboxes[peer] = self._inboxes[peer]
        view.epoch, view.n_rows = self._epoch.data_ptr(), self.n_rows
        view.world, view.rank, view.spin_limit = self.world, self.rank, self.spin_limit
        self._view = torch.frombuffer(bytearray(bytes(view)), dtype=torch.uint8).to(self.device)
        return self._view

    def run(self, local: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``local`` [n_rows, 130] fp32 (this rank's records) -> ``out`` [n_rows, 128] fp16/bf16, merged
        over all ranks."""
        if local.dtype != torch.float32 or local.shape != (self.n_rows, 130) or not local.is_contiguous():
            raise ValueError("local must be a contiguous [n_rows, 130] float32 tensor")
        if out.shape != (self.n_rows, 128) or not out.is_contiguous() or out.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("out must be a contiguous [n_rows, 128] fp16/bf16 tensor")
        N.require_cuda(local, "PeerExchange.run")
        entry = N.ExchangeRank(local.data_ptr(), self._inboxes, out.data_ptr(), self._epoch.data_ptr(),
                               N.status_word(self.device).data_ptr(), self.rank)
        args = N.ExchangeArgs(ctypes.pointer(entry), 1, self.world, self.n_rows, N.DTYPE_CODE[out.dtype], self.spin_limit)
        N.check(N.library().inq_exchange_merge(ctypes.byref(args), N.stream_pointer(self.device)), "inq_exchange_merge")
        return out

    def close(self) -> None:
        """Unmap the peers' inboxes and free this rank's.  Call it on every rank once no launch
        that uses the exchange is still in flight anywhere (e.g. after a barrier)."""
        lib = N.library()
        with torch.cuda.device(self.device):
            for mapped in self._opened:
                lib.inq_peer_buffer_close(mapped)
            self._opened = []
            if self._own:
                lib.inq_peer_buffer_destroy(self._own)
                self._own = ctypes.c_void_p()


class SplitKVDecode:
    """Per-rank driver: local decode over this rank's blocks, then the exchange and merge of the
    partial records (``exchange``: "p2p", "nccl" or "auto", see the module text)."""

    def __init__(self, sequences: list[SequenceState], q_heads: int, group=None, dtype=torch.bfloat16,
                 owns_tail: bool | None = None, exchange: str = "auto"):
        if exchange not in ("auto", "p2p", "nccl", "fused"):
            raise ValueError("exchange must be 'auto', 'p2p', 'nccl' or 'fused'")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.owns_tail = (self.rank == self.world - 1) if owns_tail is None else owns_tail
        # measured on 2, 4 and 8 B200s: the exchange inside the decode launch is the fastest of the three
        self.fused = self.world > 1 and exchange in ("fused", "auto")
        self.batch = DecodeBatch(sequences, q_heads, dtype, partials_only=not self.fused)
        n = len(sequences)
        self.peers = None
        if self.world > 1 and exchange != "nccl":
            try:
                self.peers = PeerExchange(n * q_heads, self.batch.device, group)
            except RuntimeError:
                if exchange in ("p2p", "fused"):
                    raise
                self.fused = False
                self.batch = DecodeBatch(sequences, q_heads, dtype, partials_only=True)
        if self.fused:
            # ONE launch per step: the decode kernel stores every pair's record into the peers'
            # inboxes, awaits theirs (bounded) and merges them itself
            self.batch.use_exchange(self.peers.decode_view())
            self.outputs = self.batch.outputs
            self.exchange = "fused"
            return
        self.gathered = torch.empty((self.world, n * q_heads, 130), dtype=torch.float32, device=self.batch.device)
        self.outputs = torch.empty((n, q_heads, 128), dtype=dtype, device=self.batch.device)
        self.exchange = "p2p" if self.peers is not None else "nccl"

    def _exchange_and_merge(self) -> None:
        if self.fused:
            return
        local = self.batch.partial_records.view(-1, 130)
        if self.peers is not None:
            self.peers.run(local, self.outputs.view(-1, 128))
            return
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered.view(-1, 130), local, group=self.group)
        else:
            self.gathered[0].copy_(local)
        merge_records(self.gathered, self.outputs.view(-1, 128))

    @property
    def inputs(self) -> torch.Tensor:
        return self.batch.inputs

    def step(self, append: bool = True) -> torch.Tensor:
        """One decode step; ``inputs`` must hold the same queries on every rank (and the new
        token's K/V on the rank that owns the tail)."""
        if append and self.owns_tail:
            self.batch.step()        # one launch: attends to the new token and appends it
        else:
            self.batch.attend()
        self._exchange_and_merge()
        return self.outputs

    def capture(self) -> None:
        """Record one step (local decode, with the fused append on the tail owner, exchange, merge) into a CUDA
        graph; ``replay`` then costs one graph launch per step.  Run eager steps first: the first
        launches set kernel attributes and NCCL builds its communicator outside a capture."""
        graph = torch.cuda.CUDAGraph()
        counters = self.batch.tail_counters.clone()
        with torch.cuda.graph(graph):
            if self.owns_tail:
                self.batch._launch_step()
            else:
                self.batch._launch_attend()
            self._exchange_and_merge()
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
