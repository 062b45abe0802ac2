"""Append-only packed KV cache with the reference's ``inquant.cache`` interface.

State per layer: an exact attention sink, immutable sealed blocks (K4 keys, V2/V4 or K4
values) and an exact recent tail.  Differences from the reference implementation
(``cache.py:122-419``), none of which change what a caller observes through the API:

* the tail and the sink live in preallocated device buffers; one decoded token is written
  by a single small kernel (C ABI ``inq_append_token``) instead of ``torch.cat`` + ``clone``
  of the whole tail, and ``residual_key`` / ``sink_key`` are views of those buffers;
* all blocks sealed by one call come out of ONE fused encoder launch per tensor and are
  exposed as views of its output arena (no per-block clones); the launches take their
  descriptors from the strides of the pending tensors, the key encoder goes first and the value
  encoder and the sink / tail row copies follow in one host call (C ABI ``inq_seal_blocks``);
* byte accounting is logical (``numel * itemsize``), which equals the storage sizes the
  reference reports for its compact clones.

Only batch-one, append-only inference on CUDA tensors is supported.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Iterator

import torch

try:
    from transformers.cache_utils import Cache as _HFCache
except ImportError:
    class _HFCache:  # the codec and cache work without transformers installed
        pass

from . import _native as N
from .codec import ArenaPackedTensor, CodecConfig, PackedTensor, quantize


@dataclass(frozen=True)
class CacheConfig:
    """Reference ``cache.py:24-54``."""

    codec: CodecConfig = field(default_factory=CodecConfig)
    block_size: int = 256
    residual_length: int = 128
    sink_tokens: int = 4
    validate_positions: bool = True
    shared_workspace: bool = False
    value_bits: int | None = None
    value_group_size: int = 64
    track_peak_bytes: bool = False

    def __post_init__(self) -> None:
        for name in ("block_size", "residual_length", "sink_tokens"):
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool):
                raise ValueError(f"{name} must be an integer")
        if self.block_size < 1 or self.residual_length < 0 or self.sink_tokens < 0:
            raise ValueError("block_size must be positive; residual_length and sink_tokens nonnegative")
        if not isinstance(self.validate_positions, bool):
            raise ValueError("validate_positions must be a boolean")
        if not isinstance(self.shared_workspace, bool):
            raise ValueError("shared_workspace must be a boolean")
        if not isinstance(self.track_peak_bytes, bool):
            raise ValueError("track_peak_bytes must be a boolean")
        if self.value_bits is not None and (type(self.value_bits) is not int or self.value_bits not in (2, 4)):
            raise ValueError("value_bits must be None, 2 or 4")
        if type(self.value_group_size) is not int or self.value_group_size not in (32, 64, 128):
            raise ValueError("value_group_size must be 32, 64 or 128")


@dataclass
class _Layer:
    shape: tuple[int, int, int, int]
    dtype: torch.dtype
    device: torch.device
    seq_length: int = 0
    sink_key_buffer: torch.Tensor | None = None     # [1, H, sink_tokens, C]
    sink_value_buffer: torch.Tensor | None = None
    sink_count: int = 0
    tail_key_buffer: torch.Tensor | None = None     # [1, H, capacity, C]
    tail_value_buffer: torch.Tensor | None = None
    tail_count: int = 0
    key_blocks: list = field(default_factory=list)
    value_blocks: list = field(default_factory=list)
    packed_nbytes: int = 0
    retired_tail: tuple | None = None               # the tail buffers replaced by the last seal
    append_args: tuple | None = None                # launch structure of the one-token append, per tail buffer pair

    sink_views: tuple | None = None                 # (count, key view, value view) handed out last

    def _sink_pair(self):
        """The sink views for the current count: the same two tensor objects until the count changes
        (a full sink never changes again, so every decode step of a layer gets the pair it got
        before and whoever checked it once need not check it again)."""
        cached = self.sink_views
        if cached is None or cached[0] != self.sink_count:
            cached = self.sink_views = (self.sink_count, self.sink_key_buffer[:, :, :self.sink_count],
                                        self.sink_value_buffer[:, :, :self.sink_count])
        return cached

    @property
    def sink_key(self):
        return None if not self.sink_count else self._sink_pair()[1]

    @property
    def sink_value(self):
        return None if not self.sink_count else self._sink_pair()[2]

    @property
    def residual_key(self):
        return None if self.tail_key_buffer is None else self.tail_key_buffer[:, :, :self.tail_count]

    @property
    def residual_value(self):
        return None if self.tail_value_buffer is None else self.tail_value_buffer[:, :, :self.tail_count]


@dataclass(frozen=True)
class PackedAttentionView:
    """Read-only old packed blocks plus exact sink/recent/new tokens for attention
    (reference ``cache.py:72-82``)."""

    key_blocks: tuple
    value_blocks: tuple
    sink_key: torch.Tensor | None
    sink_value: torch.Tensor | None
    residual_key: torch.Tensor
    residual_value: torch.Tensor
    seq_length: int


_storage_use_count = getattr(torch._C, "_storage_Use_Count", None)


def _use_count(tensor: torch.Tensor) -> int:
    return _storage_use_count(tensor.untyped_storage()._cdata)


_SOLE_USE_COUNT = _use_count(torch.empty(1)) if _storage_use_count is not None else -1


def _sole_owner(tensor: torch.Tensor) -> bool:
    """True when no other tensor (a view handed out earlier, a decode state) shares the storage."""
    return _storage_use_count is not None and tensor._base is None and _use_count(tensor) <= _SOLE_USE_COUNT


def _tensor_bytes(tensor: torch.Tensor | None) -> int:
    return 0 if tensor is None else tensor.numel() * tensor.element_size()


def _quantize_temporal_blocks(tensor, block_count, block_size, config):
    """Seal ``block_count`` independent temporal blocks with one encoder launch: the block axis
    becomes the batch axis through strides alone (reference ``cache.py:89-119``)."""
    if block_count == 0:
        return []
    if block_count == 1:
        return [quantize(tensor[:, :, :block_size], config)]
    _, heads, _, channels = tensor.shape
    blocked = tensor[0, :, :block_count * block_size].reshape(
        heads, block_count, block_size, channels
    ).permute(1, 0, 2, 3)
    packed = quantize(blocked, config)
    shape = (1, heads, block_size, channels)
    return ArenaPackedTensor.split(packed, block_count, shape, tensor.dtype)


def _dequantize_arena_into(arena, out: torch.Tensor, position: int) -> bool:
    """Dequantise the blocks of one encoder arena ([blocks, heads, T, C] fields) straight into ``out``
    [1, heads, tokens, C] from token ``position`` on (C ABI ``inq_k4_dequantize_strided`` /
    ``inq_v_dequantize_strided``); False when the layouts do not allow it."""
    from .value_codec import PackedValues
    run, heads, tokens, channels = arena.shape
    if out.stride(3) != 1 or out.stride(2) != channels or out.dtype not in N.DTYPE_CODE or not arena.payload.is_contiguous():
        return False
    base = out.data_ptr() + position * out.stride(2) * out.element_size()
    lib, stream = N.library(), N.stream_pointer(out.device)
    if isinstance(arena, PackedValues):
        if not (arena.scales.is_contiguous() and arena.offsets.is_contiguous()):
            return False
        rc = lib.inq_v_dequantize_strided(N.pointer(arena.payload), N.pointer(arena.scales), N.pointer(arena.offsets), run, heads,
                                          tokens, channels, arena.bits, arena.group_size, base, tokens * out.stride(2),
                                          out.stride(1), N.DTYPE_CODE[out.dtype], stream)
        N.check(rc, "inq_v_dequantize_strided")
        return True
    fields = (arena.scales, arena.salient_channels, arena.donor_channels, arena.padding)
    if not all(t.is_contiguous() for t in fields):
        return False
    count = arena.salient_channels.shape[-1]
    rc = lib.inq_k4_dequantize_strided(N.pointer(arena.payload), N.pointer(arena.scales), N.pointer(arena.salient_channels),
                                       N.pointer(arena.donor_channels), int(arena.salient_channels.dtype == torch.int32),
                                       N.pointer(arena.padding), run, heads, tokens, channels, count, base,
                                       tokens * out.stride(2), out.stride(1), N.DTYPE_CODE[out.dtype], stream)
    N.check(rc, "inq_k4_dequantize_strided")
    return True


def restore_blocks(blocks, out: torch.Tensor, position: int) -> int:
    """Dequantise ``blocks`` into ``out`` [1, H, tokens, C] from token ``position`` on; returns the
    position after the last block.  Blocks sealed by one call share an encoder arena: each arena is
    dequantised by one launch instead of block by block."""
    heads, channels = out.shape[1], out.shape[3]
    index = 0
    while index < len(blocks):
        arena = getattr(blocks[index], "_arena", None)
        run = 1
        if arena is not None and arena[1] == 0:
            while index + run < len(blocks):
                other = getattr(blocks[index + run], "_arena", None)
                if other is None or other[0] is not arena[0] or other[1] != run:
                    break
                run += 1
        tokens = blocks[index].shape[2]
        if run > 1 and run == arena[0].shape[0] and _dequantize_arena_into(arena[0], out, position):
            pass   # one launch wrote every block of the arena at its token position
        elif run > 1 and run == arena[0].shape[0]:
            dense = arena[0].dequantize(dtype=out.dtype)            # [run, heads, tokens, channels]
            out[0, :, position:position + run * tokens].view(heads, run, tokens, channels).copy_(
                dense.permute(1, 0, 2, 3))
        else:
            run = 1
            out[:, :, position:position + tokens].copy_(blocks[index].dequantize(dtype=out.dtype))
        position += run * tokens
        index += run
    return position


class InQuantCache(_HFCache):
    """Immutable quantized history plus exact sink and a bounded recent tail
    (reference ``cache.py:122-419``)."""

    is_compileable = False

    def __init__(self, config: CacheConfig | None = None) -> None:
        try:
            super().__init__()
        except (TypeError, ValueError):  # newer transformers want a layer list
            super().__init__(layers=[])
        self.config = config or CacheConfig()
        self._layers: dict[int, _Layer] = {}
        self._attention_states: dict[int, Any] = {}
        self._shared_decode_workspace = None
        self._tracked_storage = {}
        self._tracked_auxiliary = {}
        self._tracked_live_bytes = 0
        self._tracked_aux_bytes = 0
        self.peak_nbytes = 0
        self._seen_tokens = 0
        self._pending_commit = None

    def _flush_pending(self) -> None:
        """A graphed decode step (``inquant.graph_decode``) advances the tails on the device and books
        the tokens into the host-side counters later; it registers that booking here so that every
        entry point of the cache sees current lengths."""
        hook = self._pending_commit
        if hook is not None:
            hook()

    def __len__(self) -> int:
        return max(self._layers, default=-1) + 1

    def __getitem__(self, layer_idx: int):
        return self.materialize(layer_idx)

    def __iter__(self) -> Iterator[tuple[torch.Tensor, torch.Tensor]]:
        for idx in range(len(self)):
            yield self.materialize(idx)

    def get_seq_length(self, layer_idx: int | None = 0) -> int:
        self._flush_pending()
        layer = self._layers.get(0 if layer_idx is None else layer_idx)
        return 0 if layer is None else layer.seq_length

    def get_usable_length(self, new_seq_length: int, layer_idx: int | None = 0) -> int:
        return self.get_seq_length(layer_idx)

    def get_max_cache_shape(self) -> None:
        return None

    def get_max_length(self) -> None:
        return None

    def get_mask_sizes(self, cache_position, layer_idx: int) -> tuple[int, int]:
        count = int(cache_position.numel()) if isinstance(cache_position, torch.Tensor) else int(cache_position)
        return self.get_seq_length(layer_idx) + count, 0

    @property
    def seen_tokens(self) -> int:
        return self._seen_tokens

    # ------------------------------------------------------------------ updates
    @torch.no_grad()
    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        """Reference ``cache.py:179-200``: a fresh prefill returns its inputs unchanged; later
        calls return dequantised history followed by the new states, then seal."""
        layer = self._validate_update(key_states, value_states, layer_idx, cache_kwargs)
        if layer is None:
            layer = _Layer(tuple(key_states.shape), key_states.dtype, key_states.device)
            full_key, full_value = key_states, value_states
        else:
            old_key, old_value = self.materialize(layer_idx)
            full_key = torch.cat((old_key, key_states), dim=2)
            full_value = torch.cat((old_value, value_states), dim=2)
        self._append(layer, key_states, value_states)
        self._layers[layer_idx] = layer
        self.record_peak(layer_idx)
        if layer_idx == 0:
            self._seen_tokens = layer.seq_length
        return full_key, full_value

    @torch.no_grad()
    def extend(self, key_states, value_states, layer_idx, cache_kwargs=None) -> None:
        """``update`` without its return value: the new states are appended and full blocks sealed
        exactly as ``update`` does (reference ``cache.py:179-200``), but the dense history is
        neither built nor returned.  Not in the reference; used by ``inquant.prefill``, which keeps
        its own dense history across the chunks of a prompt."""
        layer = self._validate_update(key_states, value_states, layer_idx, cache_kwargs)
        if layer is None:
            layer = _Layer(tuple(key_states.shape), key_states.dtype, key_states.device)
        self._append(layer, key_states, value_states)
        self._layers[layer_idx] = layer
        self.record_peak(layer_idx)
        if layer_idx == 0:
            self._seen_tokens = layer.seq_length

    def _validate_update(self, key_states, value_states, layer_idx, cache_kwargs):
        self._flush_pending()
        if not isinstance(layer_idx, int) or layer_idx < 0:
            raise ValueError("layer_idx must be a nonnegative integer")
        if key_states.ndim != 4 or value_states.shape != key_states.shape:
            raise ValueError("K/V must have matching [batch, KV_heads, tokens, head_dim] shapes")
        if key_states.shape[0] != 1:
            raise NotImplementedError("InQuantCache currently supports batch size 1 only")
        if not key_states.is_floating_point() or not value_states.is_floating_point():
            raise ValueError("K/V must be floating-point tensors")
        if key_states.dtype != value_states.dtype or key_states.device != value_states.device:
            raise ValueError("K/V must share dtype and device")
        if any(size < 1 for size in key_states.shape):
            raise ValueError("K/V dimensions must be nonempty")
        if key_states.shape[3] % 2:
            raise ValueError("Packed cache requires an even head dimension")
        N.require_cuda(key_states, "InQuantCache")
        layer = self._layers.get(layer_idx)
        old_length = 0 if layer is None else layer.seq_length
        if layer is not None:
            if (key_states.shape[0], key_states.shape[1], key_states.shape[3]) != (
                layer.shape[0], layer.shape[1], layer.shape[3]
            ) or key_states.dtype != layer.dtype or key_states.device != layer.device:
                raise ValueError("Layer shape, dtype and device must remain unchanged")
        position = (cache_kwargs or {}).get("cache_position")
        if position is not None:
            if not isinstance(position, torch.Tensor) or position.ndim != 1 or (
                position.numel() != key_states.shape[2] or position.dtype not in (torch.int32, torch.int64)
            ):
                raise ValueError("cache_position must be a 1D integer tensor with one position per new token")
            if self.config.validate_positions:
                expected = torch.arange(
                    old_length, old_length + key_states.shape[2], device=position.device, dtype=position.dtype
                )
                if not torch.equal(position, expected):
                    raise ValueError("Only contiguous append positions are supported; reset before a new request")
        return layer

    @torch.no_grad()
    def append_for_attention(self, key_states, value_states, layer_idx, cache_kwargs=None) -> PackedAttentionView:
        """Append one token without materialising history (reference ``cache.py:242-269``).
        The snapshot holds the blocks sealed BEFORE this append and a tail that ends with the
        new token; blocks sealed by this append are used from the next step on."""
        layer = self._validate_update(key_states, value_states, layer_idx, cache_kwargs)
        if key_states.shape[2] != 1 or layer is None:
            raise ValueError("append_for_attention requires one new token after an existing prefill")
        old_blocks = (tuple(layer.key_blocks), tuple(layer.value_blocks))
        old_sink = (layer.sink_key, layer.sink_value)
        tail_key, tail_value = self._append(layer, key_states, value_states, want_tail=True)
        view = PackedAttentionView(*old_blocks, *old_sink, tail_key, tail_value, layer.seq_length)
        self.record_peak(layer_idx)
        if layer_idx == 0:
            self._seen_tokens = layer.seq_length
        return view

    def _tail_capacity(self) -> int:
        return self.config.residual_length + self.config.block_size

    def _new_buffers(self, layer: _Layer, tokens: int):
        shape = (1, layer.shape[1], tokens, layer.shape[3])
        return (torch.empty(shape, dtype=layer.dtype, device=layer.device),
                torch.empty(shape, dtype=layer.dtype, device=layer.device))

    def _tail_buffers_for(self, layer: _Layer, tokens: int):
        """Tail buffers for the tokens left over by a seal: the pair retired by the previous seal when
        it has the size and no tensor but the layer's own refers to its storage, else a new pair."""
        retired, layer.retired_tail = layer.retired_tail, None
        if retired is not None and retired[0] is not None and retired[0].shape[2] == tokens and all(
                _sole_owner(t) for t in retired):
            return retired
        return self._new_buffers(layer, tokens)

    def _seal_direct(self, layer: _Layer, pending_key, pending_value, blocks: int, copy_sources, copies):
        """Seal ``blocks`` temporal blocks of 16-bit 128-channel keys and values with descriptors
        computed from the strides of the pending tensors (the block axis becomes the batch axis of
        a launch through strides alone, reference ``cache.py:89-119``) and nothing read back.  The
        key encoder -- the longest kernel of a seal -- is launched first (``inq_k4_encode``), so
        that it runs while the host allocates the rest; the value encoder and the row ranges
        ``copies()`` names (source tensor, first source token, destination tensor, first
        destination token, tokens; destinations are the layer's own contiguous buffers) follow in
        ONE host call (``inq_seal_blocks``).  Returns the new key and value blocks, or None -- before
        anything is launched -- when the layout is outside what this path covers (the general path
        then does the same work call by call)."""
        cfg = self.config
        codec = cfg.codec
        batch, heads, _, channels = pending_key.shape
        dtype = pending_key.dtype
        if (batch != 1 or channels != 128 or dtype not in (torch.float16, torch.bfloat16) or pending_value.dtype != dtype
                or pending_value.shape != pending_key.shape or not pending_key.is_cuda):
            return None
        if cfg.value_bits is not None and channels % cfg.value_group_size:
            return None
        for tensor in (pending_key, pending_value, *copy_sources):
            strides = tensor.stride()
            if strides[3] != 1 or tensor.data_ptr() % 16 or strides[1] % 8 or strides[2] % 8:
                return None
        tokens = cfg.block_size
        device = pending_key.device
        code = N.DTYPE_CODE[dtype]
        status = N.status_word(device).data_ptr()
        lib = N.library()
        none = N.Field(None, 0, 0)

        def rows(tensor):
            _, stride_h, stride_t, _ = tensor.stride()
            return N.Input(tensor.data_ptr(), code, blocks, heads, tokens * stride_t, stride_h, stride_t, tokens, channels,
                           None, 0, 0)

        def field(tensor, row_bytes):
            return N.Field(tensor.data_ptr(), row_bytes * heads, row_bytes)

        def k4_arguments(tensor):
            count = math.floor(channels * codec.salient_fraction)
            payload = torch.empty((blocks, heads, tokens, channels // 2), dtype=torch.uint8, device=device)
            scales = torch.empty((blocks, heads, channels), dtype=torch.float32, device=device)
            salient = torch.empty((blocks, heads, count), dtype=torch.uint8, device=device)
            donors = torch.empty((blocks, heads, count), dtype=torch.uint8, device=device)
            padding = torch.empty((blocks, heads, count), dtype=torch.float32, device=device)
            args = N.K4EncodeArgs()
            args.input = rows(tensor)
            args.sample_stride, args.count = codec.sample_stride, count
            args.min_error = int(codec.donor_policy == "min_error")
            args.payload, args.scales = field(payload, tokens * channels // 2), field(scales, channels * 4)
            args.padding = field(padding, count * 4) if count else none
            args.salient = field(salient, count) if count else none
            args.donors = field(donors, count) if count else none
            return args, (payload, scales, salient, donors, padding)

        shape = (blocks, heads, tokens, channels)
        key_args, key_fields = k4_arguments(pending_key)
        N.check(lib.inq_k4_encode(N.ctypes.byref(key_args), status, N.stream_pointer(device)), "inq_k4_encode")
        packed_keys = PackedTensor(*key_fields, shape, dtype)

        seal = N.SealArgs()
        seal.heads, seal.row_bytes = heads, channels * 2
        n = 0
        for source, first, target, start, count in copies():
            if not count:
                continue
            entry = seal.copies[n]
            _, source_h, source_t, _ = source.stride()
            _, target_h, target_t, _ = target.stride()
            entry.src = source.data_ptr() + first * source_t * 2
            entry.dst = target.data_ptr() + start * target_t * 2
            entry.src_stride_h, entry.src_stride_t = source_h * 2, source_t * 2
            entry.dst_stride_h, entry.dst_stride_t = target_h * 2, target_t * 2
            entry.tokens = count
            n += 1
        seal.n_copies = n
        if cfg.value_bits is None:
            value_args, value_fields = k4_arguments(pending_value)
            seal.value_k4 = N.ctypes.pointer(value_args)
            packed_values = PackedTensor(*value_fields, shape, dtype)
        else:
            from .value_codec import ArenaPackedValues, PackedValues
            bits, group = cfg.value_bits, cfg.value_group_size
            payload = torch.empty((blocks, heads, tokens, channels * bits // 8), dtype=torch.uint8, device=device)
            scales = torch.empty((blocks, heads, tokens, channels // group), dtype=torch.float16, device=device)
            offsets = torch.empty((blocks, heads, tokens, channels // group), dtype=torch.float16, device=device)
            value_args = N.VEncodeArgs()
            value_args.input = rows(pending_value)
            value_args.bits, value_args.group = bits, group
            value_args.payload = field(payload, tokens * channels * bits // 8)
            value_args.scales = field(scales, tokens * (channels // group) * 2)
            value_args.offsets = field(offsets, tokens * (channels // group) * 2)
            seal.value = N.ctypes.pointer(value_args)
            packed_values = PackedValues(payload, scales, offsets, shape, dtype, bits, group)
        N.check(lib.inq_seal_blocks(N.ctypes.byref(seal), status, N.stream_pointer(device)), "inq_seal_blocks")
        if blocks == 1:
            return [packed_keys], [packed_values]
        new_keys = ArenaPackedTensor.split(packed_keys, blocks)
        if cfg.value_bits is None:
            return new_keys, ArenaPackedTensor.split(packed_values, blocks)
        return new_keys, ArenaPackedValues.split(packed_values, blocks)

    def _write_token(self, layer: _Layer, keys, values, sink_position: int) -> bool:
        """One-kernel write of a single token into the tail (and the sink); False when the
        layout does not meet the kernel's 16-byte alignment rules."""
        es = keys.element_size()
        row_bytes = layer.shape[3] * es
        if row_bytes % 16 or keys.data_ptr() % 16 or values.data_ptr() % 16 or keys.stride(-1) != 1 or values.stride(-1) != 1:
            return False
        if (keys.stride(1) * es) % 16 or keys.stride(1) != values.stride(1):
            return False
        tk, tv = layer.tail_key_buffer, layer.tail_value_buffer
        cached = layer.append_args
        if cached is None or cached[0] != tk.data_ptr() or cached[1] != tv.data_ptr():
            # what only changes when the tail buffers are replaced (a seal) is filled once
            if tk.data_ptr() % 16 or tv.data_ptr() % 16 or tk.stride(-1) != 1 or tv.stride(-1) != 1:
                return False
            args = N.AppendArgs()
            args.tail_key, args.tail_value = tk.data_ptr(), tv.data_ptr()
            args.tail_stride_h, args.tail_stride_t = tk.stride(1) * es, tk.stride(2) * es
            args.tail_capacity = tk.shape[2]
            args.heads, args.row_bytes = layer.shape[1], row_bytes
            args.status = N.status_word(layer.device).data_ptr()
            cached = layer.append_args = (tk.data_ptr(), tv.data_ptr(), args, N.ctypes.byref(args))
        args = cached[2]
        args.key, args.value, args.src_stride_h = keys.data_ptr(), values.data_ptr(), keys.stride(1) * es
        args.tail_position = layer.tail_count
        args.sink_position = sink_position
        if sink_position >= 0:
            sk, sv = layer.sink_key_buffer, layer.sink_value_buffer
            args.sink_key, args.sink_value = sk.data_ptr(), sv.data_ptr()
            args.sink_stride_h, args.sink_stride_t = sk.stride(1) * es, sk.stride(2) * es
        N.check(N.library().inq_append_token(cached[3], N.stream_pointer(layer.device)), "inq_append_token")
        return True

    def _append(self, layer: _Layer, keys, values, want_tail: bool = False):
        """Reference ``cache.py:271-306``.  Returns the (old tail + new tokens) pair when
        ``want_tail`` is set."""
        cfg = self.config
        new_tokens = keys.shape[2]
        take_sink = min(cfg.sink_tokens - layer.sink_count, new_tokens)
        pending_count = layer.tail_count + new_tokens - take_sink
        blocks = max(0, (pending_count - cfg.residual_length) // cfg.block_size)
        if cfg.sink_tokens and layer.sink_key_buffer is None:
            layer.sink_key_buffer, layer.sink_value_buffer = self._new_buffers(layer, cfg.sink_tokens)
        capacity = self._tail_capacity()

        if new_tokens == 1 and blocks == 0 and layer.tail_count < capacity:
            # decode fast path: one token, nothing to seal
            if layer.tail_key_buffer is None:
                layer.tail_key_buffer, layer.tail_value_buffer = self._new_buffers(layer, capacity)
            sink_position = layer.sink_count if take_sink else -1
            if not self._write_token(layer, keys, values, sink_position):
                layer.tail_key_buffer[:, :, layer.tail_count].copy_(keys[:, :, 0])
                layer.tail_value_buffer[:, :, layer.tail_count].copy_(values[:, :, 0])
                if take_sink:
                    layer.sink_key_buffer[:, :, layer.sink_count].copy_(keys[:, :, 0])
                    layer.sink_value_buffer[:, :, layer.sink_count].copy_(values[:, :, 0])
            tail = None
            if want_tail:
                tail = (layer.tail_key_buffer[:, :, :layer.tail_count + 1],
                        layer.tail_value_buffer[:, :, :layer.tail_count + 1])
            layer.sink_count += take_sink
            layer.tail_count += 1 - take_sink
            layer.seq_length += 1
            return tail

        tail = None
        pending_key = pending_value = None
        if (new_tokens == 1 and blocks == 1 and not take_sink and layer.tail_key_buffer is not None
                and layer.tail_count == layer.tail_key_buffer.shape[2] - 1 and self._write_token(layer, keys, values, -1)):
            # decode step that seals a block: the token completes the tail buffer in place (views
            # handed out earlier end before it), so old tail + new token is the buffer itself
            pending_key, pending_value = layer.tail_key_buffer, layer.tail_value_buffer
            if want_tail:
                tail = (pending_key, pending_value)
        # general path: build new storage first so that a failing codec call leaves the layer intact
        elif want_tail:
            tail = ((keys, values) if not layer.tail_count else
                    (torch.cat((layer.residual_key, keys), dim=2), torch.cat((layer.residual_value, values), dim=2)))
        if pending_key is None:
            pending_key, pending_value = keys[:, :, take_sink:], values[:, :, take_sink:]
            if layer.tail_count:
                if want_tail and not take_sink:
                    pending_key, pending_value = tail
                else:
                    pending_key = torch.cat((layer.residual_key, pending_key), dim=2)
                    pending_value = torch.cat((layer.residual_value, pending_value), dim=2)
        offset = blocks * cfg.block_size
        remainder = pending_key.shape[2] - offset
        tail_buffers = []

        def new_tail():
            # a new tail buffer: views handed out earlier keep the old one alive and unchanged.  The
            # buffer retired by the previous seal is taken again when nothing else refers to it any more.
            if not tail_buffers:
                tail_buffers.extend(self._tail_buffers_for(layer, max(capacity, remainder)))
            return tail_buffers

        def row_copies():
            tail_key_buffer, tail_value_buffer = new_tail()
            return ((pending_key, offset, tail_key_buffer, 0, remainder),
                    (pending_value, offset, tail_value_buffer, 0, remainder),
                    (keys, 0, layer.sink_key_buffer, layer.sink_count, take_sink),
                    (values, 0, layer.sink_value_buffer, layer.sink_count, take_sink))

        # Both encoders are launched before either finite check is read: the key and value kernels
        # run back to back while the host builds the block views, and one read of the status word
        # (one synchronisation instead of two) decides before any state changes.  Where the layout
        # allows, the key encoder starts before the new tail is even allocated, and the value encoder
        # and the copies into the new tail and the sink are one host call; rows that the copies write
        # lie beyond what the layer's counters expose until the check passed.
        sealed = None
        if blocks:
            sealed = self._seal_direct(layer, pending_key, pending_value, blocks,
                                       (keys, values) if take_sink else (), row_copies)
        tail_key_buffer, tail_value_buffer = new_tail()
        if sealed is not None:
            new_keys, new_values = sealed
        else:
            with N.deferred_status():
                new_keys = _quantize_temporal_blocks(pending_key, blocks, cfg.block_size, cfg.codec)
                if cfg.value_bits is None:
                    new_values = _quantize_temporal_blocks(pending_value, blocks, cfg.block_size, cfg.codec)
                else:
                    from .value_codec import quantize_value_blocks
                    new_values = quantize_value_blocks(pending_value, blocks, cfg.block_size, cfg.value_bits,
                                                       cfg.value_group_size)
            if remainder:
                tail_key_buffer[:, :, :remainder].copy_(pending_key[:, :, offset:])
                tail_value_buffer[:, :, :remainder].copy_(pending_value[:, :, offset:])
        if blocks and N.nonfinite_reported(layer.device):
            # the failure path alone works out which tensor it was (same messages as the codecs)
            if not bool(torch.isfinite(pending_key[:, :, :offset]).all()):
                raise ValueError("x must contain finite values representable in float32")
            if cfg.value_bits is None:
                raise ValueError("x must contain finite values representable in float32")
            raise ValueError("Values and stored FP16 quantization parameters must be finite")
        if take_sink and sealed is None:
            layer.sink_key_buffer[:, :, layer.sink_count:layer.sink_count + take_sink].copy_(keys[:, :, :take_sink])
            layer.sink_value_buffer[:, :, layer.sink_count:layer.sink_count + take_sink].copy_(values[:, :, :take_sink])
        layer.sink_count += take_sink
        # the next seal takes the retired pair; a first call (prefill) provides one, so that no decode
        # step has to wait for the allocator
        layer.retired_tail = ((layer.tail_key_buffer, layer.tail_value_buffer) if layer.tail_key_buffer is not None
                              else self._new_buffers(layer, capacity))
        layer.tail_key_buffer, layer.tail_value_buffer, layer.tail_count = tail_key_buffer, tail_value_buffer, remainder
        layer.key_blocks.extend(new_keys)
        layer.value_blocks.extend(new_values)
        if cfg.track_peak_bytes:
            layer.packed_nbytes += sum(block.nbytes for block in new_keys + new_values)
        layer.seq_length += new_tokens
        return tail

    def record_peak(self, layer_idx):
        """Live persistent bytes in O(1) per layer update (reference ``cache.py:308-326``)."""
        if not self.config.track_peak_bytes:
            return
        layer = self._layers[layer_idx]
        owned = layer.packed_nbytes + sum(_tensor_bytes(t) for t in (
            layer.sink_key, layer.sink_value, layer.residual_key, layer.residual_value))
        self._tracked_live_bytes += owned - self._tracked_storage.get(layer_idx, 0)
        self._tracked_storage[layer_idx] = owned
        state = self._attention_states.get(layer_idx)
        aux = 0 if state is None else state.nbytes
        self._tracked_aux_bytes += aux - self._tracked_auxiliary.get(layer_idx, 0)
        self._tracked_auxiliary[layer_idx] = aux
        shared = 0 if self._shared_decode_workspace is None else self._shared_decode_workspace.nbytes
        self.peak_nbytes = max(self.peak_nbytes, self._tracked_live_bytes + self._tracked_aux_bytes + shared)

    @torch.no_grad()
    def materialize(self, layer_idx: int = 0):
        """Reconstruct this layer; returned tensors are not retained (reference ``cache.py:328-345``)."""
        self._flush_pending()
        if layer_idx not in self._layers:
            raise KeyError(f"No cached layer {layer_idx}")
        layer = self._layers[layer_idx]

        def restore(sink, blocks, tail):
            _, heads, _, channels = layer.shape
            sink_tokens = 0 if sink is None else sink.shape[2]
            tail_tokens = 0 if tail is None else tail.shape[2]
            packed_tokens = sum(block.shape[2] for block in blocks)
            out = torch.empty((1, heads, sink_tokens + packed_tokens + tail_tokens, channels),
                              dtype=layer.dtype, device=layer.device)
            if sink_tokens:
                out[:, :, :sink_tokens].copy_(sink)
            position = restore_blocks(blocks, out, sink_tokens)
            if tail_tokens:
                out[:, :, position:].copy_(tail)
            return out

        return (
            restore(layer.sink_key, layer.key_blocks, layer.residual_key),
            restore(layer.sink_value, layer.value_blocks, layer.residual_value),
        )

    # ------------------------------------------------------------------ accounting
    @property
    def payload_nbytes(self) -> int:
        return sum(b.payload_nbytes for layer in self._layers.values() for b in layer.key_blocks + layer.value_blocks)

    @property
    def metadata_nbytes(self) -> int:
        return sum(b.metadata_nbytes for layer in self._layers.values() for b in layer.key_blocks + layer.value_blocks)

    @property
    def residual_nbytes(self) -> int:
        self._flush_pending()
        return sum(_tensor_bytes(layer.residual_key) + _tensor_bytes(layer.residual_value) for layer in self._layers.values())

    @property
    def sink_nbytes(self) -> int:
        return sum(_tensor_bytes(layer.sink_key) + _tensor_bytes(layer.sink_value) for layer in self._layers.values())

    @property
    def auxiliary_nbytes(self) -> int:
        shared = 0 if self._shared_decode_workspace is None else self._shared_decode_workspace.nbytes
        return shared + sum(state.nbytes for state in self._attention_states.values())

    @property
    def nbytes(self) -> int:
        """Live persistent tensor bytes, including codec metadata and exact tails."""
        return self.payload_nbytes + self.metadata_nbytes + self.residual_nbytes + self.sink_nbytes + self.auxiliary_nbytes

    @property
    def bf16_nbytes(self) -> int:
        self._flush_pending()
        return sum(2 * 2 * layer.shape[0] * layer.shape[1] * layer.seq_length * layer.shape[3] for layer in self._layers.values())

    def memory_stats(self) -> dict[str, int | float]:
        self._flush_pending()
        total, baseline = self.nbytes, self.bf16_nbytes
        return {
            "nbytes": total,
            "peak_nbytes": self.peak_nbytes if self.config.track_peak_bytes else None,
            "payload_nbytes": self.payload_nbytes,
            "metadata_nbytes": self.metadata_nbytes,
            "residual_nbytes": self.residual_nbytes,
            "sink_nbytes": self.sink_nbytes,
            "auxiliary_nbytes": self.auxiliary_nbytes,
            "bf16_nbytes": baseline,
            "quantized_layer_tokens": sum(block.shape[2] for layer in self._layers.values() for block in layer.key_blocks),
            "kv_reduction_vs_bf16": 1 - total / baseline if baseline else 0.0,
        }

    def reset(self) -> None:
        self._pending_commit = None
        self._layers.clear()
        self._attention_states.clear()
        self._shared_decode_workspace = None
        self._tracked_storage.clear()
        self._tracked_auxiliary.clear()
        self._tracked_live_bytes = self._tracked_aux_bytes = self.peak_nbytes = 0
        self._seen_tokens = 0

    def release(self) -> None:
        self.reset()

    def reorder_cache(self, beam_idx) -> None:
        raise NotImplementedError("Beam search/reordering is unsupported; use num_beams=1")

    def crop(self, max_length: int) -> None:
        raise NotImplementedError("Cache rollback/speculative decoding is unsupported; use append-only generation")

    def batch_repeat_interleave(self, repeats: int) -> None:
        raise NotImplementedError("Batch expansion is unsupported; use batch size 1")

    def batch_select_indices(self, indices) -> None:
        raise NotImplementedError("Batch selection is unsupported; use batch size 1")
