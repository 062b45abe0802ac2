"""Per-token affine INT2/INT4 value codec: same interface as the reference
``inquant/value_codec.py``, computed by the sm_100a kernel behind ``inq_v_encode``."""
from collections import deque
from dataclasses import dataclass
from itertools import repeat

import torch

from . import _native as N


def _logical_bytes(tensor):
    return tensor.numel() * tensor.element_size()


@dataclass(frozen=True)
class PackedValues:
    """Reference ``value_codec.py:12-48``; byte counts are logical (see ``PackedTensor``)."""

    payload: torch.Tensor
    scales: torch.Tensor
    offsets: torch.Tensor
    shape: tuple[int, int, int, int]
    original_dtype: torch.dtype
    bits: int
    group_size: int

    @property
    def tensors(self):
        return {"payload": self.payload, "scales": self.scales, "offsets": self.offsets}

    @property
    def payload_nbytes(self):
        return _logical_bytes(self.payload)

    @property
    def nbytes(self):
        return sum(_logical_bytes(t) for t in self.tensors.values())

    @property
    def metadata_nbytes(self):
        return self.nbytes - self.payload_nbytes

    @torch.no_grad()
    def dequantize(self, dtype=None):
        dtype = self.original_dtype if dtype is None else dtype
        if not dtype.is_floating_point:
            raise ValueError("dequantize dtype must be floating point")
        if dtype not in N.DTYPE_CODE:
            raise NotImplementedError("dequantize supports float32, float16 and bfloat16")
        N.require_cuda(self.payload, "PackedValues.dequantize")
        batch, heads, tokens, channels = self.shape
        out = torch.empty(self.shape, dtype=dtype, device=self.payload.device)
        payload, scales, offsets = self.payload.contiguous(), self.scales.contiguous(), self.offsets.contiguous()
        rc = N.library().inq_v_dequantize(N.pointer(payload), N.pointer(scales), N.pointer(offsets),
                                          batch * heads, tokens, channels, self.bits, self.group_size,
                                          N.pointer(out), N.DTYPE_CODE[dtype], N.stream_pointer(out.device))
        N.check(rc, "inq_v_dequantize")
        return out


class ArenaPackedValues(PackedValues):
    """One block of a batch sealed by a single value-encoder launch: ``(arena, index)`` in a slot,
    everything else read off the arena on first access (see ``codec.ArenaPackedTensor``)."""

    __slots__ = ("_arena",)
    _FIELDS = ("payload", "scales", "offsets")

    def __init__(self, arena: PackedValues, index: int, shape=None, original_dtype=None) -> None:
        object.__setattr__(self, "_arena", (arena, index))

    @classmethod
    def split(cls, arena: PackedValues, count: int, shape=None, original_dtype=None) -> list:
        """The ``count`` blocks of ``arena`` as a list (see ``codec.ArenaPackedTensor.split``)."""
        blocks = list(map(object.__new__, repeat(cls, count)))
        deque(map(cls.__dict__["_arena"].__set__, blocks, zip(repeat(arena), range(count))), maxlen=0)
        return blocks

    def __getattr__(self, name):
        if name == "_arena":
            raise AttributeError(name)
        arena, index = self._arena
        if name in ArenaPackedValues._FIELDS:
            value = getattr(arena, name)[index:index + 1]
        elif name == "shape":
            value = (1, *arena.shape[1:])
        elif name in ("original_dtype", "bits", "group_size"):
            value = getattr(arena, name)
        else:
            raise AttributeError(name)
        object.__setattr__(self, name, value)
        return value

    def field_pointer(self, name: str) -> int:
        arena, index = self._arena
        tensor = getattr(arena, name)
        return tensor.data_ptr() + index * tensor.stride(0) * tensor.element_size()

    @property
    def payload_nbytes(self):
        arena, _ = self._arena
        return _logical_bytes(arena.payload) // arena.payload.shape[0]

    @property
    def nbytes(self):
        arena, _ = self._arena
        return sum(_logical_bytes(t) // t.shape[0] for t in arena.tensors.values())


def encode_values_into(x, bits, group_size, payload, scales, offsets, page_ids=None, num_slots: int = 0):
    """Launch the value encoder on ``x`` = [outer, inner, tokens, channels]; no synchronisation."""
    args = N.VEncodeArgs()
    args.input = N.make_input(x, page_ids, num_slots)
    args.bits, args.group = bits, group_size
    args.payload, args.scales, args.offsets = payload, scales, offsets
    rc = N.library().inq_v_encode(N.ctypes.byref(args), N.pointer(N.status_word(x.device)),
                                  N.stream_pointer(x.device))
    N.check(rc, "inq_v_encode")


@torch.no_grad()
def quantize_values(x, bits=2, group_size=64):
    """Reference ``value_codec.py:51-72``."""
    if type(bits) is not int or bits not in (2, 4):
        raise ValueError("Value bits must be 2 or 4")
    if type(group_size) is not int or group_size not in (32, 64, 128):
        raise ValueError("Value group size must be 32, 64 or 128")
    if x.ndim != 4 or min(x.shape) < 1 or not x.is_floating_point() or x.shape[-1] % group_size:
        raise ValueError("Expected nonempty floating [batch, heads, tokens, channels] divisible by group_size")
    if x.dtype not in N.DTYPE_CODE:
        raise NotImplementedError("quantize_values supports float32, float16 and bfloat16 inputs")
    N.require_cuda(x, "quantize_values")
    if x.stride(-1) != 1:
        x = x.contiguous()
    batch, heads, tokens, channels = x.shape
    device = x.device
    payload = torch.empty((batch, heads, tokens, channels * bits // 8), dtype=torch.uint8, device=device)
    scales = torch.empty((batch, heads, tokens, channels // group_size), dtype=torch.float16, device=device)
    offsets = torch.empty_like(scales)
    encode_values_into(x.detach(), bits, group_size, N.compact_field(payload, heads),
                       N.compact_field(scales, heads), N.compact_field(offsets, heads))
    if N.nonfinite_reported(device):
        raise ValueError("Values and stored FP16 quantization parameters must be finite")
    return PackedValues(payload, scales, offsets, tuple(x.shape), x.dtype, bits, group_size)


def quantize_value_blocks(tensor, block_count, block_size, bits, group_size):
    """Reference ``value_codec.py:75-88``: the temporal block axis becomes the batch axis of
    ONE kernel launch; the per-block results are views of that launch's output arena."""
    if not block_count:
        return []
    if block_count == 1:
        return [quantize_values(tensor[:, :, :block_size], bits, group_size)]
    _, heads, _, channels = tensor.shape
    blocked = tensor[0, :, :block_count * block_size].reshape(
        heads, block_count, block_size, channels).permute(1, 0, 2, 3)
    packed = quantize_values(blocked, bits, group_size)
    shape = (1, heads, block_size, channels)
    return ArenaPackedValues.split(packed, block_count, shape, tensor.dtype)
