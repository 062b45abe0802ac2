"""Mixed 4/8-bit key codec: same interface as the reference ``inquant/codec.py``.

``quantize`` runs ONE fused sm_100a kernel per call (sampled statistics, donor selection,
scales, nibble packing, padding statistics; C ABI ``inq_k4_encode``) instead of the
reference's chain of eager torch ops (``codec.py:181-243``).  Packed bytes, scales,
descriptors and padding are bit-identical to the reference's CPU result for 128-channel
inputs.  Tensors must live on a CUDA device.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass
from itertools import repeat

import torch

from . import _native as N


@dataclass(frozen=True)
class CodecConfig:
    """Reference ``codec.py:38-55``; ``donor_backend`` keeps its accepted strings, all of
    which select the one CUDA implementation."""

    sample_stride: int = 8
    salient_fraction: float = 0.125
    donor_policy: str = "neighbors"
    donor_backend: str = "torch"

    def __post_init__(self) -> None:
        if self.donor_backend not in ("torch", "triton", "auto"):
            raise ValueError("donor_backend must be torch, triton or auto")
        if isinstance(self.sample_stride, bool) or not isinstance(self.sample_stride, int):
            raise ValueError("sample_stride must be a positive integer")
        if self.sample_stride < 1:
            raise ValueError("sample_stride must be a positive integer")
        if not math.isfinite(self.salient_fraction) or not 0 <= self.salient_fraction <= 0.5:
            raise ValueError("salient_fraction must be finite and in [0, 0.5]")
        if self.donor_policy not in ("neighbors", "min_error"):
            raise ValueError("donor_policy must be neighbors or min_error")


def _logical_bytes(tensor: torch.Tensor) -> int:
    return tensor.numel() * tensor.element_size()


@dataclass(frozen=True)
class PackedTensor:
    """Packed keys plus the descriptor shared by every token of a block
    (reference ``codec.py:58-134``).

    Byte counts are logical (``numel * itemsize``): blocks sealed together share one device
    arena and are exposed as views, so the per-tensor storage size the reference reports for
    its cloned blocks is reproduced from shapes instead of from ``untyped_storage()``.
    """

    payload: torch.Tensor
    scales: torch.Tensor
    salient_channels: torch.Tensor
    donor_channels: torch.Tensor
    padding: torch.Tensor
    shape: tuple[int, int, int, int]
    original_dtype: torch.dtype

    @property
    def tensors(self) -> dict[str, torch.Tensor]:
        return {
            "payload": self.payload,
            "scales": self.scales,
            "salient_channels": self.salient_channels,
            "donor_channels": self.donor_channels,
            "padding": self.padding,
        }

    @property
    def payload_nbytes(self) -> int:
        return _logical_bytes(self.payload)

    @property
    def nbytes(self) -> int:
        return sum(_logical_bytes(t) for t in self.tensors.values())

    @property
    def metadata_nbytes(self) -> int:
        return self.nbytes - self.payload_nbytes

    def storage_stats(self) -> dict[str, int | float]:
        source_nbytes = math.prod(self.shape) * self.original_dtype.itemsize
        return {
            "payload_nbytes": self.payload_nbytes,
            "scale_nbytes": _logical_bytes(self.scales),
            "descriptor_nbytes": _logical_bytes(self.salient_channels) + _logical_bytes(self.donor_channels),
            "padding_nbytes": _logical_bytes(self.padding),
            "metadata_nbytes": self.metadata_nbytes,
            "nbytes": self.nbytes,
            "source_nbytes": source_nbytes,
            "compression_ratio": source_nbytes / self.nbytes,
        }

    @torch.no_grad()
    def dequantize(self, dtype: torch.dtype | None = None) -> torch.Tensor:
        """Dense tensor including the sampled-mean donor approximation (C ABI
        ``inq_k4_dequantize``; reference ``codec.py:112-134``)."""
        dtype = self.original_dtype if dtype is None else dtype
        if not dtype.is_floating_point:
            raise ValueError("dequantize dtype must be floating point")
        if dtype not in N.DTYPE_CODE:
            raise NotImplementedError("dequantize supports float32, float16 and bfloat16")
        N.require_cuda(self.payload, "PackedTensor.dequantize")
        batch, heads, tokens, channels = self.shape
        count = self.salient_channels.shape[-1]
        out = torch.empty(self.shape, dtype=dtype, device=self.payload.device)
        payload, scales = self.payload.contiguous(), self.scales.contiguous()
        salient, donors = self.salient_channels.contiguous(), self.donor_channels.contiguous()
        padding = self.padding.contiguous()
        rc = N.library().inq_k4_dequantize(
            N.pointer(payload), N.pointer(scales), N.pointer(salient), N.pointer(donors),
            int(salient.dtype == torch.int32), N.pointer(padding), batch * heads, tokens, channels,
            count, N.pointer(out), N.DTYPE_CODE[dtype], N.stream_pointer(out.device))
        N.check(rc, "inq_k4_dequantize")
        return out


class ArenaPackedTensor(PackedTensor):
    """One block of a batch that a single encoder launch sealed.  An instance holds nothing but
    ``(arena, index)`` in a slot: its field tensors are views of that launch's output arena, created
    on first access, and its shape and dtype are read off the arena -- a 32K-token prefill seals 127
    blocks per layer, and building views (or even instance dictionaries) for each costs more host
    time than the launch."""

    __slots__ = ("_arena",)
    _FIELDS = ("payload", "scales", "salient_channels", "donor_channels", "padding")

    def __init__(self, arena: PackedTensor, index: int, shape=None, original_dtype=None) -> None:
        object.__setattr__(self, "_arena", (arena, index))

    @classmethod
    def split(cls, arena: PackedTensor, count: int, shape=None, original_dtype=None) -> list:
        """The ``count`` blocks of ``arena`` as a list, built without running Python code per block
        (the slot's descriptor is applied by ``map``)."""
        blocks = list(map(object.__new__, repeat(cls, count)))
        deque(map(cls.__dict__["_arena"].__set__, blocks, zip(repeat(arena), range(count))), maxlen=0)
        return blocks

    def __getattr__(self, name):   # reached only while an attribute has not been materialised yet
        if name == "_arena":
            raise AttributeError(name)
        arena, index = self._arena
        if name in ArenaPackedTensor._FIELDS:
            value = getattr(arena, name)[index:index + 1]
        elif name == "shape":
            value = (1, *arena.shape[1:])
        elif name == "original_dtype":
            value = arena.original_dtype
        else:
            raise AttributeError(name)
        object.__setattr__(self, name, value)
        return value

    def field_pointer(self, name: str) -> int:
        """Device address of a field without creating its view."""
        arena, index = self._arena
        tensor = getattr(arena, name)
        return tensor.data_ptr() + index * tensor.stride(0) * tensor.element_size()

    @property
    def payload_nbytes(self) -> int:
        arena, _ = self._arena
        return _logical_bytes(arena.payload) // arena.payload.shape[0]

    @property
    def nbytes(self) -> int:
        arena, _ = self._arena
        return sum(_logical_bytes(t) // t.shape[0] for t in arena.tensors.values())


def _reuse_map(saliency: torch.Tensor, count: int, donor_error: torch.Tensor | None = None):
    """Disjoint sources/donors (C ABI ``inq_select_donors``; reference ``codec.py:137-178``).

    ``saliency`` (and ``donor_error``) are float32 ``[..., channels]`` CUDA tensors.
    """
    N.require_cuda(saliency, "_reuse_map")
    if saliency.dtype != torch.float32:
        raise ValueError("saliency must be float32")
    *prefix, channels = saliency.shape
    if not 0 <= count <= channels // 2:
        raise ValueError("count must be in [0, channels // 2]")
    if donor_error is not None and (donor_error.shape != saliency.shape or donor_error.dtype != saliency.dtype
                                   or donor_error.device != saliency.device):
        raise ValueError("Donor error must match saliency shape, dtype and device")
    sources = torch.empty((*prefix, count), dtype=torch.int64, device=saliency.device)
    donors = torch.empty_like(sources)
    rows = saliency.numel() // channels if channels else 0
    if count and rows:
        sal = saliency.contiguous()
        err = None if donor_error is None else donor_error.contiguous()
        rc = N.library().inq_select_donors(N.pointer(sal), N.pointer(err), rows, channels, count,
                                           N.pointer(sources), N.pointer(donors), N.stream_pointer(sal.device))
        N.check(rc, "inq_select_donors")
    return sources, donors


def _validate_input(x: torch.Tensor) -> None:
    if x.ndim != 4 or any(size < 1 for size in x.shape):
        raise ValueError("x must have nonempty [batch, heads, tokens, channels] dimensions")
    if not x.is_floating_point():
        raise ValueError("x must have a floating-point dtype")
    if x.shape[-1] % 2:
        raise ValueError("head dimension must be even for two nibbles per byte")
    if x.dtype not in N.DTYPE_CODE:
        raise NotImplementedError("quantize supports float32, float16 and bfloat16 inputs")
    N.require_cuda(x, "quantize")


def encode_into(x: torch.Tensor, config: CodecConfig, payload, scales, salient, donors, padding,
                roles=None, page_ids=None, num_slots: int = 0) -> None:
    """Launch the fused encoder on ``x`` = [outer, inner, tokens, channels] (unit channel
    stride); outputs are ``_native.Field`` descriptors.  No synchronisation."""
    channels = x.shape[-1]
    count = math.floor(channels * config.salient_fraction)
    args = N.K4EncodeArgs()
    args.input = N.make_input(x, page_ids, num_slots)
    args.sample_stride = config.sample_stride
    args.count = count
    args.min_error = int(config.donor_policy == "min_error")
    args.payload, args.scales, args.padding = payload, scales, padding
    args.salient = salient if salient is not None else N.Field(None, 0, 0)
    args.donors = donors if donors is not None else N.Field(None, 0, 0)
    args.roles = roles[0] if roles is not None else N.Field(None, 0, 0)
    args.role_bytes = roles[1] if roles is not None else 0
    args.descriptor_i32 = int(channels > 256)
    rc = N.library().inq_k4_encode(N.ctypes.byref(args), N.pointer(N.status_word(x.device)),
                                   N.stream_pointer(x.device))
    N.check(rc, "inq_k4_encode")


@torch.no_grad()
def quantize(x: torch.Tensor, config: CodecConfig = CodecConfig()) -> PackedTensor:
    """Pack one ``[batch, heads, tokens, even_head_dim]`` temporal KV block
    (reference ``codec.py:181-243``).  The finite check reads a device status word after the
    launch, i.e. it synchronises exactly where the reference does."""
    _validate_input(x)
    if x.stride(-1) != 1:
        x = x.contiguous()
    batch, heads, tokens, channels = x.shape
    count = math.floor(channels * config.salient_fraction)
    device = x.device
    descriptor_dtype = torch.uint8 if channels <= 256 else torch.int32
    payload = torch.empty((batch, heads, tokens, channels // 2), dtype=torch.uint8, device=device)
    scales = torch.empty((batch, heads, channels), dtype=torch.float32, device=device)
    salient = torch.empty((batch, heads, count), dtype=descriptor_dtype, device=device)
    donors = torch.empty_like(salient)
    padding = torch.empty((batch, heads, count), dtype=torch.float32, device=device)
    encode_into(x.detach(), config, N.compact_field(payload, heads), N.compact_field(scales, heads),
                N.compact_field(salient, heads), N.compact_field(donors, heads), N.compact_field(padding, heads))
    if N.nonfinite_reported(device):
        raise ValueError("x must contain finite values representable in float32")
    return PackedTensor(payload, scales, salient, donors, padding, tuple(x.shape), x.dtype)
