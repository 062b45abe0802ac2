"""One-launch decode step for many (request, layer) sequences.

The reference decodes layer by layer (``qwen_fused.py:138-158``), two Triton launches per
layer.  A layer of a 32K-token request is only ~14 MB of packed cache, i.e. ~2 microseconds
of HBM time on a B200, so per-layer launches are latency-bound.  ``DecodeBatch`` keeps a
device-resident array of sequence descriptors (C ABI ``inq_decode_seq_t``) and runs

    step():  1 launch  inq_decode_attention with `fused_append`: the new K/V token of every sequence
             is attended to from the staging rows, stored behind its tail, and the device-side tail
             lengths advance when the launch ends (all sequences, fused split-KV merge)

(`append()` and `attend()` remain as two separate launches, inq_append_token_batch and
inq_decode_attention.)

with tail lengths held in device counters, so a decode loop makes no host round trip and
can be captured in a CUDA graph.  Sequences are independent: this is also the collective-
free batched-serving path (requests sharded across GPUs simply build one batch per rank).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _native as N
from .triton_attention import PackedDecodeState, workspace_floats


@dataclass
class SequenceState:
    """One (request, layer): packed blocks plus exact sink and tail buffers."""

    decode_state: PackedDecodeState          # pointer table + role maps of the sealed blocks
    sink_key: torch.Tensor | None            # [1, H, sink, 128] (views allowed)
    sink_value: torch.Tensor | None
    tail_key_buffer: torch.Tensor            # [1, H, capacity, 128]
    tail_value_buffer: torch.Tensor
    tail_count: int

    @classmethod
    def from_cache_layer(cls, cache, layer_idx: int) -> "SequenceState":
        layer = cache._layers[layer_idx]
        state = PackedDecodeState(layer.key_blocks, layer.value_blocks)
        if layer.tail_key_buffer is None:
            raise ValueError("the layer has no tail buffer yet")
        return cls(state, layer.sink_key, layer.sink_value, layer.tail_key_buffer, layer.tail_value_buffer,
                   layer.tail_count)


@dataclass
class PagedSequenceState:
    """One (request, layer) in the paged layout: physical pages of a pool reached through a
    page table, plus the ``[2,H,B+4,128]`` dense tensor holding the exact sink (tokens 0..3) and
    the unsealed tail (from token 4), as the reference's serving backend keeps them."""

    pool: torch.Tensor               # [num_pages, page_bytes] uint8
    page_table: torch.Tensor         # int32 physical page of logical page i
    num_pages: int
    dense: torch.Tensor              # [2, H, B + 4, 128]
    tail_count: int
    sink_count: int
    layout: object                   # inquant_vllm.layout.PageLayout


def shard_requests(lengths, world: int) -> list[list[int]]:
    """Deal independent requests to ``world`` ranks so that the longest rank is as short as a
    greedy pass gets it: requests in order of decreasing context length, each to the rank with
    the fewest tokens so far (ties: fewer requests, then lower rank).  Every rank computes the same
    assignment from the same lengths, so no collective is involved.  Returns the request indices
    of every rank in increasing order."""
    if world < 1:
        raise ValueError("world must be positive")
    load, shards = [0] * world, [[] for _ in range(world)]
    for index in sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i)):
        rank = min(range(world), key=lambda r: (load[r], len(shards[r]), r))
        load[rank] += int(lengths[index])
        shards[rank].append(index)
    return [sorted(shard) for shard in shards]


def _struct_array_to_device(array, device) -> torch.Tensor:
    raw = bytes(array)
    return torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)


class DecodeBatch:
    """Device-resident descriptors, queries, outputs and scratch for a fixed set of sequences."""

    def __init__(self, sequences: list[SequenceState], q_heads: int, dtype: torch.dtype = torch.bfloat16,
                 scale: float | None = None, partials_only: bool = False):
        if not sequences:
            raise ValueError("at least one sequence is required")
        self.paged = isinstance(sequences[0], PagedSequenceState)
        if any(isinstance(s, PagedSequenceState) != self.paged for s in sequences):
            raise ValueError("a batch holds either table-layout or paged sequences")
        self.sequences = sequences
        if self.paged:
            self.layout = sequences[0].layout
            self.device = sequences[0].pool.device
            self.kv_heads = self.layout.heads
            self.value_kind, self.value_groups = 0, 0
        else:
            with_blocks = [s.decode_state for s in sequences if s.decode_state.key_blocks]
            kinds = {state.streaming_value_kind() for state in with_blocks}
            if None in kinds or len(kinds) > 1:
                raise NotImplementedError("batched decode needs one value codec that the streaming kernel serves "
                                          "(PackedDecodeState.streaming_value_kind)")
            self.value_kind, self.value_groups = kinds.pop() if kinds else (0, 0)
            first = with_blocks[0] if with_blocks else sequences[0].decode_state
            self.device = sequences[0].tail_key_buffer.device
            self.kv_heads = sequences[0].tail_key_buffer.shape[1]
        if q_heads % self.kv_heads:
            raise ValueError("query_heads must be divisible by the KV head count")
        if dtype not in (torch.float16, torch.bfloat16):
            raise NotImplementedError("batched decode supports fp16 and bf16")
        self.q_heads, self.dtype = q_heads, dtype
        self.q_per_kv = q_heads // self.kv_heads
        self.scale = 128 ** -0.5 if scale is None else float(scale)
        self.block_tokens = self.layout.block_size if self.paged else first._packed_tokens
        self.n_pad = 16 if self.paged else first._salient
        n = len(sequences)
        # one staging tensor per step: [query heads | new key heads | new value heads] x 128
        self.inputs = torch.zeros((n, q_heads + 2 * self.kv_heads, 128), dtype=dtype, device=self.device)
        self.queries = self.inputs[:, :q_heads]
        self.new_keys = self.inputs[:, q_heads:q_heads + self.kv_heads]
        self.new_values = self.inputs[:, q_heads + self.kv_heads:]
        self.outputs = torch.empty((n, q_heads, 128), dtype=dtype, device=self.device)
        # split-KV across GPUs: keep un-normalised (acc[128], m, l) records instead of outputs
        self.partial_records = (torch.zeros((n, q_heads, 130), dtype=torch.float32, device=self.device)
                                if partials_only else None)
        self.tail_counters = torch.tensor([s.tail_count for s in sequences], dtype=torch.int32).to(self.device)
        self._build_descriptors()
        tiles = (self.q_per_kv + 7) // 8
        n_pairs = n * self.kv_heads * tiles
        # prefix sums of the work units of every (sequence, KV head, head tile) pair
        units = [int(N.library().inq_decode_units(self._blocks_of(s), self.block_tokens))
                 for s in sequences for _ in range(self.kv_heads * tiles)]
        starts = torch.tensor([0] + units, dtype=torch.int64).cumsum(0)
        self.total_units = int(starts[-1])
        self.pair_starts = starts.to(self.device)
        self.partials = torch.empty(workspace_floats(n_pairs, self.total_units), dtype=torch.float32, device=self.device)
        self.counters = torch.zeros(n_pairs + 1, dtype=torch.int32, device=self.device)   # + the launch-wide arrival counter
        self.launches = 0
        self._initial_counters = self.tail_counters.clone()
        self._prepare_launch_arguments()

    def _blocks_of(self, s) -> int:
        return s.num_pages if self.paged else len(s.decode_state.key_blocks)

    def _tail_capacity_of(self, s) -> int:
        return self.layout.block_size if self.paged else s.tail_key_buffer.shape[2]

    def _build_paged_descriptors(self) -> None:
        from inquant_vllm.kernels import fill_paged_sequence
        n = len(self.sequences)
        es = self.queries.element_size()
        seqs = (N.DecodeSeq * n)()
        apps = (N.AppendArgs * n)()
        for i, s in enumerate(self.sequences):
            if s.layout != self.layout or s.dense.dtype != self.dtype or not s.dense.is_contiguous():
                raise ValueError("all paged sequences must share the layout and hold contiguous dense tensors of the batch dtype")
            table = s.page_table if s.page_table.dtype == torch.int32 else s.page_table.to(torch.int32)
            s.page_table = table
            fill_paged_sequence(seqs[i], self.queries[i], self.outputs[i], s.pool, table, s.dense, s.num_pages,
                                s.tail_count, s.sink_count, self.layout)
            seqs[i].tail_tokens_device = self.tail_counters[i:].data_ptr()
            a = apps[i]
            a.key, a.value, a.src_stride_h = self.new_keys[i].data_ptr(), self.new_values[i].data_ptr(), 128 * es
            a.tail_key, a.tail_value = seqs[i].tail_key, seqs[i].tail_value
            a.tail_stride_h, a.tail_stride_t = s.dense.stride(1) * es, s.dense.stride(2) * es
            a.tail_position, a.tail_capacity = s.tail_count, self.layout.block_size
            a.tail_counter = self.tail_counters[i:].data_ptr()
            a.sink_position = -1
            a.heads, a.row_bytes = self.kv_heads, 128 * es
        self._finish_descriptors(seqs, apps)

    def _finish_descriptors(self, seqs, apps) -> None:
        es = self.queries.element_size()
        for i, s in enumerate(self.sequences):
            # the step's new token, read by launches with fused_append
            seqs[i].new_key, seqs[i].new_value = self.new_keys[i].data_ptr(), self.new_values[i].data_ptr()
            seqs[i].new_stride_h = self.new_keys.stride(1)
            seqs[i].tail_capacity = self._tail_capacity_of(s)
        if self.partial_records is not None:
            for i in range(len(self.sequences)):
                seqs[i].partial_output = self.partial_records[i].data_ptr()
        self._seq_records = _struct_array_to_device(seqs, self.device)
        self._append_records = _struct_array_to_device(apps, self.device)

    def _build_descriptors(self) -> None:
        if self.paged:
            return self._build_paged_descriptors()
        n = len(self.sequences)
        es = self.queries.element_size()
        seqs = (N.DecodeSeq * n)()
        apps = (N.AppendArgs * n)()
        for i, s in enumerate(self.sequences):
            st = s.decode_state
            if st.key_blocks and (st._packed_tokens != self.block_tokens or st._salient != self.n_pad):
                raise ValueError("all sequences must share block length and salient-channel count")
            d = seqs[i]
            d.query = self.queries[i].data_ptr()
            d.output = self.outputs[i].data_ptr()
            d.query_head_stride = 128
            n_blocks = len(st.key_blocks)
            d.table = st._tables.data_ptr() if n_blocks else None
            d.roles = st._key_map.data_ptr() if n_blocks else None
            d.value_roles = st._value_map.data_ptr() if n_blocks and self.value_kind == 1 else None
            d.n_blocks = n_blocks
            if s.sink_key is not None and s.sink_key.shape[2]:
                for t in (s.sink_key, s.sink_value):
                    if not N.dense_rows_aligned(t):
                        raise ValueError("sink rows must be 16-byte aligned")
                d.sink_key, d.sink_value = s.sink_key.data_ptr(), s.sink_value.data_ptr()
                d.sink_key_stride_h, d.sink_key_stride_t = s.sink_key.stride(1), s.sink_key.stride(2)
                d.sink_value_stride_h, d.sink_value_stride_t = s.sink_value.stride(1), s.sink_value.stride(2)
                d.sink_tokens = s.sink_key.shape[2]
            tk, tv = s.tail_key_buffer, s.tail_value_buffer
            for t in (tk, tv):
                if not N.dense_rows_aligned(t) or t.dtype != self.dtype:
                    raise ValueError("tail buffers must match the batch dtype with 16-byte aligned rows")
            d.tail_key, d.tail_value = tk.data_ptr(), tv.data_ptr()
            d.tail_key_stride_h, d.tail_key_stride_t = tk.stride(1), tk.stride(2)
            d.tail_value_stride_h, d.tail_value_stride_t = tv.stride(1), tv.stride(2)
            d.tail_tokens = s.tail_count
            d.tail_tokens_device = self.tail_counters[i:].data_ptr()
            a = apps[i]
            a.key, a.value, a.src_stride_h = self.new_keys[i].data_ptr(), self.new_values[i].data_ptr(), 128 * es
            a.tail_key, a.tail_value = tk.data_ptr(), tv.data_ptr()
            a.tail_stride_h, a.tail_stride_t = tk.stride(1) * es, tk.stride(2) * es
            a.tail_position, a.tail_capacity = s.tail_count, tk.shape[2]
            a.tail_counter = self.tail_counters[i:].data_ptr()
            a.sink_position = -1
            a.heads, a.row_bytes = self.kv_heads, 128 * es
        self._finish_descriptors(seqs, apps)

    @property
    def capacity_left(self) -> int:
        """Appends that still fit every tail buffer (host-side bookkeeping)."""
        return self._capacity - self._appended

    def _prepare_launch_arguments(self) -> None:
        n = len(self.sequences)
        self._capacity = min(self._tail_capacity_of(s) - s.tail_count for s in self.sequences)
        self._appended = 0
        args = N.DecodeArgs()
        args.n_seq, args.seqs_device = n, self._seq_records.data_ptr()
        args.kv_heads, args.q_per_kv = self.kv_heads, self.q_per_kv
        args.block_tokens, args.n_pad = self.block_tokens, self.n_pad
        args.layout, args.dtype, args.scale = int(self.paged), N.DTYPE_CODE[self.dtype], self.scale
        args.value_kind, args.value_groups = self.value_kind, self.value_groups
        if self.paged:
            from inquant_vllm.kernels import page_offsets_array
            args.page_bytes, args.page_offsets = self.layout.page_bytes, page_offsets_array(self.layout)
        args.pair_starts, args.total_units = self.pair_starts.data_ptr(), self.total_units
        args.partials, args.partials_floats = self.partials.data_ptr(), self.partials.numel()
        args.counters = self.counters.data_ptr()
        args.status = N.status_word(self.device).data_ptr()
        self._decode_args = args
        self._decode_args_ref = ctypes.byref(args)
        self._step_args = N.DecodeArgs.from_buffer_copy(args)
        self._step_args.fused_append = 1
        self._step_args_ref = ctypes.byref(self._step_args)
        self._status_pointer = N.status_word(self.device).data_ptr()
        self._graph = None

    def use_exchange(self, view: torch.Tensor | None) -> None:
        """Exchange and merge every pair's record with the peer GPUs inside the decode launch
        (``inq_decode_exchange_t`` in device memory, e.g. ``PeerExchange.decode_view()``); ``None``
        switches it off.  ``outputs`` then holds the rows merged over all ranks."""
        self._exchange_view = view
        pointer = None if view is None else view.data_ptr()
        self._decode_args.exchange_device = pointer
        self._step_args.exchange_device = pointer

    def _launch_append(self) -> None:
        rc = N.library().inq_append_token_batch(self._append_records.data_ptr(), len(self.sequences),
                                                self._status_pointer, N.stream_pointer(self.device))
        if rc:
            N.check(rc, "inq_append_token_batch")

    def _launch_attend(self) -> None:
        rc = N.library().inq_decode_attention(self._decode_args_ref, N.stream_pointer(self.device))
        if rc:
            N.check(rc, "inq_decode_attention")

    def _launch_step(self) -> None:
        rc = N.library().inq_decode_attention(self._step_args_ref, N.stream_pointer(self.device))
        if rc:
            N.check(rc, "inq_decode_attention")

    def append(self) -> None:
        """Write ``new_keys`` / ``new_values`` at the end of every tail and advance the device counters."""
        if self.capacity_left < 1:
            raise RuntimeError("a tail buffer is full: seal a block before appending")
        self._launch_append()
        self._appended += 1
        self.launches += 1

    def attend(self) -> torch.Tensor:
        """Attention of ``queries`` over every sequence; returns ``outputs`` ([n, q_heads, 128])."""
        self._launch_attend()
        self.launches += 1
        return self.outputs

    def step(self) -> torch.Tensor:
        """One decode step in one launch: attend to history plus the new token of every sequence
        and append that token to its tail."""
        if self.capacity_left < 1:
            raise RuntimeError("a tail buffer is full: seal a block before appending")
        self._launch_step()
        self._appended += 1
        self.launches += 1
        return self.outputs

    def capture(self) -> None:
        """Record the fused step into a CUDA graph; ``replay`` then costs one graph launch.
        Run at least one eager ``step`` first (the first launch sets kernel attributes)."""
        graph = torch.cuda.CUDAGraph()
        counters = self.tail_counters.clone()
        with torch.cuda.graph(graph):
            self._launch_step()
        self.tail_counters.copy_(counters)  # capture does not execute, but keep the state explicit
        self._graph = graph

    def replay(self) -> torch.Tensor:
        if self._graph is None:
            raise RuntimeError("call capture() first")
        if self.capacity_left < 1:
            raise RuntimeError("a tail buffer is full: seal a block before appending")
        self._graph.replay()
        self._appended += 1
        self.launches += 1
        return self.outputs

    def rewind(self, appended: int = 0) -> None:
        """Reset every tail to its length at construction plus ``appended`` tokens (benchmarks
        re-use the same tail slots instead of sealing)."""
        self.tail_counters.copy_(self._initial_counters + appended)
        self._appended = appended

    @property
    def tail_tokens(self) -> list[int]:
        return [s.tail_count + self._appended for s in self.sequences]

    def algorithmic_bytes(self) -> dict[str, int]:
        """Bytes one ``attend`` must read/write: packed blocks, their metadata, exact sink and
        tail, queries and outputs (the model used for the roofline figures)."""
        h, t = self.kv_heads, self.block_tokens
        es = self.queries.element_size()
        packed = meta = dense = 0
        for s in self.sequences:
            nb = self._blocks_of(s)
            if self.value_kind == 1:       # values coded like the keys
                value_row, value_meta = 64, 512 + 16 * 2 + 16 * 4
            elif self.value_kind == 2:     # 4-bit codes, fp16 scale and offset per token and group
                value_row, value_meta = 64 + 4 * self.value_groups, 0
            else:                          # 2-bit codes in two groups (or one)
                value_row, value_meta = 32 + 4 * (self.value_groups or 2), 0
            packed += h * nb * t * (64 + value_row)
            meta += h * nb * ((832 if self.paged else 512 + self.n_pad * 2 + self.n_pad * 4) + value_meta)
            sink = s.sink_count if self.paged else (0 if s.sink_key is None else s.sink_key.shape[2])
            dense += (sink + s.tail_count + self._appended) * h * 128 * es * 2
        qo = len(self.sequences) * self.q_heads * 128 * es * 2
        return {"packed": packed, "metadata": meta, "dense": dense, "query_output": qo,
                "total": packed + meta + dense + qo}
