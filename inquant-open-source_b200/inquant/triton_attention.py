"""Single-query GQA attention directly over the packed layout, with the reference's
``inquant.triton_attention`` interface (the module name is kept for drop-in use; nothing
here uses Triton).

``PackedDecodeState`` owns the per-block pointer table and the int8 channel-role maps and
launches ONE sm_100a kernel per decode (C ABI ``inq_decode_attention``): partial softmax
over the packed K4/V2 blocks, the exact sink and the exact tail, and the log-sum-exp merge
by the last CTA of each KV head (reference: two Triton kernels,
``triton_attention.py:67-181``).

Limitations of this build: CUDA, batch 1, head_dim 128, one query token, fp16/bf16 query,
uniform packed block length, values stored as 2-bit ``PackedValues`` with group 64.  Other
variants raise ``NotImplementedError``; there is no fallback.
"""
from __future__ import annotations

import math

import torch

from . import _native as N
from .codec import PackedTensor
from .value_codec import PackedValues


class SharedDecodeWorkspace:
    """One scratch allocation per request, usable only on one CUDA stream
    (reference ``triton_attention.py:184-208``)."""

    def __init__(self):
        self.tensor = None
        self._stream_identity = None

    @property
    def nbytes(self):
        return 0 if self.tensor is None else self.tensor.numel() * self.tensor.element_size()

    def acquire(self, shape, device):
        identity = N.stream_identity(device)
        if self._stream_identity is not None and identity != self._stream_identity:
            raise RuntimeError("Shared decode workspace requires one CUDA stream per cache")
        self._stream_identity = identity
        required = math.prod(shape)
        if self.tensor is None or self.tensor.numel() < required:
            self.tensor = torch.empty(required, dtype=torch.float32, device=device)
        return self.tensor[:required].view(shape)

    def acquire_address(self, floats: int, device, identity=None) -> int:
        """``acquire`` for a caller that only needs the device address of ``floats`` scratch floats
        (no view tensors are built); ``identity`` is the caller's current-stream identity when it
        already has it."""
        if identity is None:
            identity = N.stream_identity(device)
        if self._stream_identity is not None and identity != self._stream_identity:
            raise RuntimeError("Shared decode workspace requires one CUDA stream per cache")
        self._stream_identity = identity
        if self.tensor is None or self.tensor.numel() < floats:
            self.tensor = torch.empty(floats, dtype=torch.float32, device=device)
        return self.tensor.data_ptr()


def workspace_floats(n_pairs: int, total_units: int) -> int:
    """Scratch floats for the split-KV partial records of ``n_pairs`` (sequence, KV head,
    8-query-head tile) pairs holding ``total_units`` 32-token slices on the current device."""
    return int(N.library().inq_decode_workspace_floats(n_pairs, total_units))


def pair_units(n_blocks: int, block_tokens: int) -> int:
    return int(N.library().inq_decode_units(n_blocks, block_tokens))


def _stacked_field(blocks, name: str) -> torch.Tensor:
    """``torch.cat`` of one field over ``blocks`` along the block axis, contiguous.  Consecutive
    blocks of one encoder arena are taken as ONE slice of the arena's tensor, so that a layer sealed
    by a single launch needs neither a view per block nor a copy."""
    pieces, run = [], None      # run: [arena, first index, one past the last index]
    for block in blocks:
        arena = getattr(block, "_arena", None)
        if arena is not None and run is not None and run[0] is arena[0] and run[2] == arena[1]:
            run[2] += 1
            continue
        if run is not None:
            pieces.append(getattr(run[0], name)[run[1]:run[2]])
            run = None
        if arena is not None:
            run = [arena[0], arena[1], arena[1] + 1]
        else:
            pieces.append(getattr(block, name))
    if run is not None:
        pieces.append(getattr(run[0], name)[run[1]:run[2]])
    return (pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=0)).contiguous()


class PackedDecodeState:
    """Reusable descriptors for immutable blocks; exact tails are per-call inputs
    (reference ``triton_attention.py:211-388``)."""

    def __init__(self, key_blocks, value_blocks, *, workspace_pool=None):
        if len(key_blocks) != len(value_blocks):
            raise ValueError("Key and value block counts must match")
        self.key_blocks = ()
        self.value_blocks = ()
        self._workspace = None
        self._workspace_pool = workspace_pool
        self._tables = None
        self._host_tables = None     # pinned mirror of the table: new rows reach the device without a synchronisation
        self._key_map = None
        self._value_map = None
        self._device = None
        self._kv_heads = None
        self._packed_tokens = 256
        self._salient = 0
        self._value_bits = 0
        self._value_group = 64
        self._value_salient = 0
        self._inquant_values = False
        self._preset = True
        self._capacity = 0
        self._stream_identity = None
        self._record_counts = {}
        self._checked_sink = None    # sink tensors that passed decode()'s checks, with the dtype and device they passed against
        self._seq_struct = N.DecodeSeq()
        self._args_struct = N.DecodeArgs()
        self._args_struct.seq_host = N.ctypes.pointer(self._seq_struct)
        self.extend(key_blocks, value_blocks)

    def extend(self, key_blocks, value_blocks):
        """Append immutable blocks, building descriptors only for the new suffix."""
        if len(key_blocks) != len(value_blocks):
            raise ValueError("Key and value block counts must match")
        old_count = len(self.key_blocks)
        if len(key_blocks) < old_count or any(a is not b for a, b in zip(self.key_blocks, key_blocks)) or any(
                a is not b for a, b in zip(self.value_blocks, value_blocks)):
            raise ValueError("PackedDecodeState.extend requires an immutable append-only prefix")
        if len(key_blocks) == old_count:
            return
        # Blocks of an encoder arena are judged by the arena's tensors, each arena once: none of
        # their field views (nor their instance dictionaries) has to be created here -- a 32K-token
        # layer holds over a thousand fields in 254 blocks.
        def owners(blocks):
            """(tensors' owner, shape of one block) per plain block and per run of one arena's blocks."""
            last = None
            for block in blocks:
                arena = getattr(block, "_arena", None)
                if arena is None:
                    last = None
                    yield block, block.shape
                elif arena[0] is not last:
                    last = arena[0]
                    yield last, (1, *last.shape[1:])

        first, first_shape = next(owners(key_blocks[:1]))
        first_device = first.payload.device
        if first_shape[0] != 1 or first_shape[-1] != 128 or first_device.type != "cuda":
            raise ValueError("Packed decode requires CUDA blocks with batch=1 and head_dim=128")
        identity = N.stream_identity(first_device)
        if self._stream_identity is not None and self._stream_identity != identity:
            raise RuntimeError("Descriptor updates require one CUDA stream per state")
        self._stream_identity = identity
        self._device = first_device
        self._kv_heads = first_shape[1]
        self._packed_tokens = first_shape[2]
        self._salient = first.salient_channels.shape[-1]
        # Only the new suffix is checked: the prefix was checked when it was added and is immutable.
        new_keys, new_values = key_blocks[old_count:], value_blocks[old_count:]
        key_owners, value_owners = list(owners(new_keys)), list(owners(new_values))
        for owner, shape in key_owners:
            if not isinstance(owner, PackedTensor) or shape != first_shape \
                    or owner.salient_channels.shape[-1] != self._salient:
                raise ValueError("All packed K/V blocks must share shape and salient-channel count")
        # the preset (2-bit values in groups of 64) runs the streaming kernel; every other value
        # codec the reference accepts runs the general kernel
        first_value = next(owners(value_blocks[:1]))[0]
        self._inquant_values = isinstance(first_value, PackedTensor)
        if self._inquant_values:
            self._value_bits, self._value_group = 0, 64
            self._value_salient = first_value.salient_channels.shape[-1]
        elif isinstance(first_value, PackedValues):
            self._value_bits = first_value.bits
            self._value_group = first_value.group_size
            self._value_salient = 0
        else:
            raise ValueError("Value blocks must be PackedValues or PackedTensor")
        self._preset = not self._inquant_values and (self._value_bits, self._value_group) == (2, 64)
        for owner, shape in value_owners:
            if shape != first_shape:
                raise ValueError("All packed blocks must share shape")
            if self._inquant_values:
                if not isinstance(owner, PackedTensor) or owner.salient_channels.shape[-1] != self._value_salient:
                    raise ValueError("All V blocks must share the same quantizer")
            elif not isinstance(owner, PackedValues) or (owner.bits, owner.group_size) != (self._value_bits, self._value_group):
                raise ValueError("All V blocks must share the same quantizer")
        checked = set()
        for owner, _ in (*key_owners, *value_owners):
            if id(owner) in checked:
                continue
            checked.add(id(owner))
            if any(t.device != self._device for t in owner.tensors.values()):
                raise ValueError("All packed tensors must share the same CUDA device")
        last_field = "padding" if self._inquant_values else "offsets"
        pointers = []
        bases = {}     # per encoder arena: (address, bytes per block) of the three fields the kernel reads

        def located(block, names):
            arena = getattr(block, "_arena", None)
            if arena is None:
                return None
            owner, index = arena
            entry = bases.get(id(owner))
            if entry is None:
                entry = bases[id(owner)] = [(t.data_ptr(), t.stride(0) * t.element_size())
                                            for t in (getattr(owner, name) for name in names)]
            return [base + index * step for base, step in entry]

        key_fields, value_fields = ("payload", "scales", "padding"), ("payload", "scales", last_field)
        for k, v in zip(new_keys, new_values):
            # blocks of one encoder launch: contiguous slices of its arena, addressed directly
            at_k, at_v = located(k, key_fields), located(v, value_fields)
            if at_k is not None and at_v is not None:
                pointers.append(at_k + at_v)
                continue
            for t in (*k.tensors.values(), *v.tensors.values()):
                if not t.is_contiguous():
                    raise ValueError("Packed block tensors must be contiguous")
            pointers.append([k.payload.data_ptr(), k.scales.data_ptr(), k.padding.data_ptr(),
                             v.payload.data_ptr(), v.scales.data_ptr(), getattr(v, last_field).data_ptr()])
        count = len(key_blocks)
        if count > self._capacity:
            # a few rows to spare from the first allocation on: the seal that follows a prefill (and
            # seven more) then extends the tables in place instead of reallocating them and their
            # pinned mirror in the middle of a decode step
            capacity = count + 8 if not self._capacity else max(count + 8, min(self._capacity * 2, count + 64))
            tables = torch.empty((capacity, 6), dtype=torch.int64, device=self._device)
            key_map = torch.empty((capacity, self._kv_heads, 128), dtype=torch.int8, device=self._device)
            value_map = torch.empty((capacity, self._kv_heads, 128) if self._inquant_values else (0,),
                                    dtype=torch.int8, device=self._device)
            host_tables = torch.empty((capacity, 6), dtype=torch.int64, pin_memory=True)
            if old_count:
                host_tables[:old_count].copy_(self._host_tables[:old_count])
            self._host_tables = host_tables
            if old_count:
                tables[:old_count].copy_(self._tables[:old_count])
                key_map[:old_count].copy_(self._key_map[:old_count])
                if self._inquant_values:
                    value_map[:old_count].copy_(self._value_map[:old_count])
            self._tables, self._key_map, self._value_map = tables, key_map, value_map
            self._capacity = capacity
        # rows of the pinned mirror are written once and never again, so the asynchronous copy needs no fence
        self._host_tables[old_count:count].copy_(torch.tensor(pointers, dtype=torch.int64))
        self._tables[old_count:count].copy_(self._host_tables[old_count:count], non_blocking=True)
        self._write_maps(self._key_map[old_count:count], new_keys, self._salient)
        if self._inquant_values:
            self._write_maps(self._value_map[old_count:count], new_values, self._value_salient)
        self.key_blocks, self.value_blocks = tuple(key_blocks), tuple(value_blocks)

    def _write_maps(self, result, blocks, count):
        """Roles: donor channel 0..127 for a salient channel, -1 normal, -2-i for the i-th donor
        (C ABI ``inq_build_roles``; reference ``triton_attention.py:301-309``)."""
        sources = _stacked_field(blocks, "salient_channels")
        donors = _stacked_field(blocks, "donor_channels")
        rows = len(blocks) * self._kv_heads
        rc = N.library().inq_build_roles(N.pointer(sources), N.pointer(donors), 0, rows, 128, count,
                                         N.pointer(result), 1, N.stream_pointer(self._device))
        N.check(rc, "inq_build_roles")
        return result

    @property
    def nbytes(self) -> int:
        """Auxiliary live GPU allocations; input packed blocks are counted elsewhere."""
        return sum(t.numel() * t.element_size() for t in
                   (self._tables, self._key_map, self._value_map, self._workspace) if t is not None)

    def streaming_value_kind(self):
        """``(value_kind, value_groups)`` of ``inq_decode_attention`` for this state's value codec, or
        ``None`` when only the general kernel serves it.  The preset (2-bit values in groups of 64) runs
        every geometry; values stored as InQuant packed tensors (the reference's default), 4-bit values in
        groups of 32 / 64 / 128 and 2-bit values in groups of 32 or 128 run it when both sides have 16
        salient channels and the blocks are whole 32-token slices (at least two)."""
        if self._preset:
            return 0, 0
        if not (self._salient == 16 and self._packed_tokens % 32 == 0 and self._packed_tokens >= 64):
            return None
        if self._inquant_values:
            return (1, 0) if self._value_salient == 16 else None
        if self._value_bits == 4:
            return 2, 128 // self._value_group
        if self._value_bits == 2:
            return 0, 128 // self._value_group
        return None

    @torch.no_grad()
    def decode(self, query, *, sink_key=None, sink_value=None, residual_key=None, residual_value=None, scale=None):
        if query.ndim != 4 or query.shape[0] != 1 or query.shape[1] < 1 or query.shape[-2:] != (1, 128):
            raise ValueError("query must have shape [1, query_heads, 1, 128]")
        if query.device.type != "cuda" or query.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            raise ValueError("query must be a CUDA FP16, BF16 or FP32 tensor")
        if query.stride(-1) != 1:
            raise ValueError("query head dimension must be contiguous")
        if self._device is not None and query.device != self._device:
            raise ValueError("query and packed blocks must share a device")
        kv_heads = self._kv_heads
        dense = []
        checked = self._checked_sink
        for name, key, value in (("sink", sink_key, sink_value), ("residual", residual_key, residual_value)):
            if (key is None) != (value is None):
                raise ValueError(f"{name} key/value must both be provided")
            if key is None:
                dense.append((None, None, 0))
                continue
            if name == "sink" and checked is not None and key is checked[0] and value is checked[1] \
                    and query.dtype == checked[2] and query.device == checked[3]:
                # the very tensors (a cache hands out the same sink views step after step) that passed
                # the checks below on an earlier call, against a query of the same dtype and device
                dense.append((checked[4], checked[5], checked[4].shape[2]))
                continue
            if key.ndim != 4 or key.shape != value.shape or key.shape[0] != 1 or key.shape[-1] != 128:
                raise ValueError(f"{name} K/V must have matching [1, KV_heads, tokens, 128] shapes")
            if key.dtype != query.dtype or value.dtype != query.dtype or key.device != query.device or value.device != query.device:
                raise ValueError(f"{name} K/V must match query dtype and device")
            if key.stride(-1) != 1 or value.stride(-1) != 1:
                raise ValueError(f"{name} head dimension must be contiguous")
            kv_heads = key.shape[1] if kv_heads is None else kv_heads
            if key.shape[1] != kv_heads:
                raise ValueError("All inputs must share their KV head count")
            given = (key, value)
            if not N.dense_rows_aligned(key):
                key = key.contiguous()
            if not N.dense_rows_aligned(value):
                value = value.contiguous()
            if name == "sink" and self._kv_heads is not None:
                self._checked_sink = (*given, query.dtype, query.device, key, value)
            dense.append((key, value, key.shape[2]))
        if kv_heads is None or query.shape[1] % kv_heads:
            raise ValueError("query_heads must be divisible by the nonempty KV head count")
        (sink_key, sink_value, sink_t), (residual_key, residual_value, residual_t) = dense
        n_blocks = len(self.key_blocks)
        if not (n_blocks + sink_t + residual_t):
            raise ValueError("Attention requires at least one key/value token")
        if scale is None:
            scale = 128 ** -0.5
        if not math.isfinite(scale) or scale <= 0:
            raise ValueError("attention scale must be positive and finite")
        identity = N.stream_identity(query.device)
        if self._stream_identity is not None and self._stream_identity != identity:
            raise RuntimeError("Packed decode state requires one CUDA stream per state")
        q_per_kv = query.shape[1] // kv_heads
        kind = self.streaming_value_kind() if n_blocks else (0, 0)
        if query.dtype == torch.float32 or kind is None:
            return self._decode_general(query, kv_heads, q_per_kv, n_blocks, sink_key, sink_value, sink_t,
                                        residual_key, residual_value, residual_t, scale)
        tiles = (q_per_kv + 7) // 8
        pairs = kv_heads * tiles
        records = self._record_counts.get((pairs, n_blocks))
        if records is None:
            records = workspace_floats(pairs, pairs * pair_units(n_blocks, self._packed_tokens)) // N.RECORD_FLOATS
            self._record_counts = {(pairs, n_blocks): records}     # one entry: the count changes when a block is sealed
        workspace_shape = (records, N.RECORD_FLOATS)
        workspace_floats_needed = records * N.RECORD_FLOATS
        if self._workspace_pool is not None:
            workspace_address = self._workspace_pool.acquire_address(workspace_floats_needed, query.device, identity)
        else:
            if self._workspace is None or self._workspace.shape != workspace_shape or self._workspace.device != query.device:
                self._workspace = torch.empty(workspace_shape, dtype=torch.float32, device=query.device)
            workspace_address = self._workspace.data_ptr()
        if query.data_ptr() % 16 or query.stride(1) % 8:     # rows of a head: 16-byte aligned (unit channel stride was checked)
            query = query.contiguous()
        output = torch.empty(query.shape, dtype=query.dtype, device=query.device)
        if self._tables is None:
            self._tables = torch.empty((0, 6), dtype=torch.int64, device=query.device)
            self._key_map = torch.empty((0, kv_heads, 128), dtype=torch.int8, device=query.device)
            self._value_map = torch.empty((0,), dtype=torch.int8, device=query.device)
            self._device = query.device
        seq = self._seq_struct        # reused from call to call: every field a call may leave unset is reset below
        seq.query, seq.output, seq.query_head_stride = query.data_ptr(), output.data_ptr(), query.stride(1)
        seq.table = self._tables.data_ptr() if n_blocks else None
        seq.roles = self._key_map.data_ptr() if n_blocks else None
        seq.value_roles = self._value_map.data_ptr() if kind[0] == 1 else None
        if sink_t:
            seq.sink_key, seq.sink_value = sink_key.data_ptr(), sink_value.data_ptr()
            seq.sink_key_stride_h, seq.sink_key_stride_t = sink_key.stride(1), sink_key.stride(2)
            seq.sink_value_stride_h, seq.sink_value_stride_t = sink_value.stride(1), sink_value.stride(2)
        else:
            seq.sink_key = seq.sink_value = None
        if residual_t:
            seq.tail_key, seq.tail_value = residual_key.data_ptr(), residual_value.data_ptr()
            seq.tail_key_stride_h, seq.tail_key_stride_t = residual_key.stride(1), residual_key.stride(2)
            seq.tail_value_stride_h, seq.tail_value_stride_t = residual_value.stride(1), residual_value.stride(2)
        else:
            seq.tail_key = seq.tail_value = None
        seq.n_blocks, seq.sink_tokens, seq.tail_tokens = n_blocks, sink_t, residual_t
        args = self._args_struct
        args.n_seq = 1
        args.kv_heads, args.q_per_kv = kv_heads, q_per_kv
        args.block_tokens, args.n_pad = self._packed_tokens, self._salient
        args.layout, args.dtype, args.scale = 0, N.DTYPE_CODE[query.dtype], scale
        args.value_kind, args.value_groups = kind
        args.partials, args.partials_floats = workspace_address, workspace_floats_needed
        args.counters = N.decode_counters(query.device, kv_heads * tiles).data_ptr()
        args.status = N.status_word(query.device).data_ptr()
        rc = N.library().inq_decode_attention(N.ctypes.byref(args), N.stream_pointer(query.device))
        N.check(rc, "inq_decode_attention")
        return output


    def _decode_general(self, query, kv_heads, q_per_kv, n_blocks, sink_key, sink_value, sink_t,
                        residual_key, residual_value, residual_t, scale):
        """Codec variants outside the K4/V2 preset and fp32 queries (C ABI ``inq_decode_generic``)."""
        lib = N.library()
        floats = lib.inq_decode_generic_workspace_floats(query.shape[1], n_blocks, sink_t, residual_t, 128)
        shape = (floats,)
        if self._workspace_pool is not None:
            workspace = self._workspace_pool.acquire(shape, query.device)
        else:
            if self._workspace is None or self._workspace.numel() < floats or self._workspace.device != query.device:
                self._workspace = torch.empty(shape, dtype=torch.float32, device=query.device)
            workspace = self._workspace
        rows = query.reshape(query.shape[1], 128) if query.is_contiguous() else query.contiguous().reshape(query.shape[1], 128)
        output = torch.empty(query.shape, dtype=query.dtype, device=query.device)
        a = N.GenericDecodeArgs()
        a.q, a.out, a.q_stride_h = rows.data_ptr(), output.data_ptr(), rows.stride(0)
        if n_blocks:
            a.table, a.key_roles = self._tables.data_ptr(), self._key_map.data_ptr()
            a.value_roles = self._value_map.data_ptr() if self._inquant_values else None
            a.value_kind = 1 if self._inquant_values else 0
            a.value_bits, a.value_group = self._value_bits, self._value_group
            a.key_pad, a.value_pad = self._salient, self._value_salient
        if sink_t:
            a.sink_key, a.sink_value = sink_key.data_ptr(), sink_value.data_ptr()
            a.sink_key_stride_h, a.sink_key_stride_t = sink_key.stride(1), sink_key.stride(2)
            a.sink_value_stride_h, a.sink_value_stride_t = sink_value.stride(1), sink_value.stride(2)
        if residual_t:
            a.tail_key, a.tail_value = residual_key.data_ptr(), residual_value.data_ptr()
            a.tail_key_stride_h, a.tail_key_stride_t = residual_key.stride(1), residual_key.stride(2)
            a.tail_value_stride_h, a.tail_value_stride_t = residual_value.stride(1), residual_value.stride(2)
        a.n_blocks, a.sink_tokens, a.tail_tokens = n_blocks, sink_t, residual_t
        a.kv_heads, a.q_per_kv, a.block_tokens, a.head_dim = kv_heads, q_per_kv, self._packed_tokens, 128
        a.dtype, a.scale = N.DTYPE_CODE[query.dtype], scale
        a.partials, a.partials_floats = workspace.data_ptr(), workspace.numel()
        N.check(lib.inq_decode_generic(N.ctypes.byref(a), N.stream_pointer(query.device)), "inq_decode_generic")
        return output


def packed_decode(query, key_blocks, value_blocks, sink_key=None, sink_value=None,
                  residual_key=None, residual_value=None, *, scale=None):
    """One-shot convenience wrapper; reuse PackedDecodeState for repeated decoding."""
    return PackedDecodeState(key_blocks, value_blocks).decode(
        query, sink_key=sink_key, sink_value=sink_value,
        residual_key=residual_key, residual_value=residual_value, scale=scale,
    )
