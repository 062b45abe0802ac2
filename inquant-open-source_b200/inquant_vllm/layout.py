"""Versioned byte layout: every packed page owns all its decoding metadata
(reference ``inquant_vllm/layout.py``).  Sealing runs the fused sm_100a encoders with the
physical pages as their destination; nothing is staged."""
from dataclasses import dataclass
import math

import torch

from inquant import _native as N
from inquant.codec import CodecConfig, encode_into
from inquant.value_codec import encode_values_into


@dataclass(frozen=True)
class PageLayout:
    """Reference ``layout.py:8-53``.  Block sizes 16 and 32 are accepted in addition to the
    reference's 64/128/256 (the byte formula is the same; the reference's engine plugin
    rejects them)."""

    block_size: int
    heads: int
    dim: int = 128

    def __post_init__(self):
        if self.block_size not in (16, 32, 64, 128, 256) or self.dim != 128 or self.heads < 1:
            raise ValueError("Expected block_size 64/128/256, head_dim 128, positive KV heads")

    @property
    def fields(self):
        b, h, d = self.block_size, self.heads, self.dim
        return (
            ("key_payload", torch.uint8, (h, b, d // 2)),
            ("key_scales", torch.float32, (h, d)),
            ("key_map", torch.int16, (h, d)),
            ("key_padding", torch.float32, (h, d // 8)),
            ("value_payload", torch.uint8, (h, b, d // 4)),
            ("value_scales", torch.float16, (h, b, d // 64)),
            ("value_offsets", torch.float16, (h, b, d // 64)),
        )

    @property
    def offsets(self):
        offset, result = 0, {}
        for name, dtype, shape in self.fields:
            result[name] = offset
            offset += math.prod(shape) * dtype.itemsize
        return result

    @property
    def page_bytes(self):
        return self.heads * (104 * self.block_size + 832)

    def views(self, pages):
        if pages.dtype != torch.uint8 or pages.ndim != 2 or pages.shape[1] != self.page_bytes:
            raise ValueError("Expected [pages, page_bytes] uint8 storage")
        out = {}
        for name, dtype, shape in self.fields:
            offset = self.offsets[name]
            size = math.prod(shape) * dtype.itemsize
            out[name] = pages[:, offset:offset + size].view(dtype).view(-1, *shape)
        return out

    def field(self, pool: torch.Tensor, name: str) -> N.Field:
        """Destination descriptor of one field inside a page pool (C ABI ``inq_field_t``)."""
        for fname, dtype, shape in self.fields:
            if fname == name:
                inner = math.prod(shape[1:]) * dtype.itemsize
                return N.Field(pool.data_ptr() + self.offsets[name], self.page_bytes, inner)
        raise KeyError(name)


def _check_pages(keys, values, layout):
    if keys.shape != values.shape or tuple(keys.shape[1:]) != (layout.heads, layout.block_size, 128):
        raise ValueError("Invalid full-page K/V shape")
    N.require_cuda(keys, "page sealing")
    if keys.dtype not in N.DTYPE_CODE or values.dtype != keys.dtype:
        raise ValueError("K/V pages must share a float32, float16 or bfloat16 dtype")


def _seal(keys, values, layout, pool, page_ids):
    if keys.stride(-1) != 1:
        keys = keys.contiguous()
    if values.stride(-1) != 1:
        values = values.contiguous()
    config = CodecConfig(donor_policy="min_error")
    slots = 0 if page_ids is None else pool.shape[0]   # ids are checked on the device against the pool size
    encode_into(keys, config, layout.field(pool, "key_payload"), layout.field(pool, "key_scales"), None, None,
                layout.field(pool, "key_padding"), roles=(layout.field(pool, "key_map"), 2), page_ids=page_ids,
                num_slots=slots)
    encode_values_into(values, 2, 64, layout.field(pool, "value_payload"), layout.field(pool, "value_scales"),
                       layout.field(pool, "value_offsets"), page_ids=page_ids, num_slots=slots)
    status = N.take_status(keys.device, N.STATUS_NONFINITE | N.STATUS_BAD_INDEX)
    if status & N.STATUS_BAD_INDEX:
        raise IndexError("a physical page id lies outside the page pool; that page was not written")
    if status & N.STATUS_NONFINITE:
        raise ValueError("K/V pages must contain finite values with finite FP16 value parameters")


@torch.no_grad()
def pack_pages(keys, values, layout):
    """Seal full temporal pages ``[P,H,B,128]`` into fresh page storage (reference ``layout.py:56-81``)."""
    _check_pages(keys, values, layout)
    result = torch.empty((keys.shape[0], layout.page_bytes), dtype=torch.uint8, device=keys.device)
    _seal(keys, values, layout, result, None)
    return result


@torch.no_grad()
def pack_pages_into(keys, values, layout, destination, page_ids, *, donor_backend="torch"):
    """Seal fresh pages directly into their assigned physical slots (reference ``layout.py:103-115``).
    The caller owns unique in-range page ids; only those pages are written."""
    _check_pages(keys, values, layout)
    if donor_backend not in ("torch", "triton", "auto"):
        raise ValueError("donor_backend must be torch, triton or auto")
    if destination.dtype != torch.uint8 or destination.ndim != 2 or destination.shape[1] != layout.page_bytes \
            or not destination.is_contiguous():
        raise ValueError('Expected contiguous uint8 destination page pool')
    if page_ids.ndim != 1 or page_ids.numel() != keys.shape[0] or page_ids.dtype not in (torch.int32, torch.int64):
        raise ValueError('One integer physical page ID is required per input page')
    if page_ids.device != destination.device or keys.device != destination.device:
        raise ValueError('K/V, page IDs and pool must share a CUDA device')
    _seal(keys, values, layout, destination, page_ids.contiguous())


def unpack_pages_reference(pages, layout, dtype=torch.bfloat16):
    """Testing/inspection only: dense K and V of every page (reference ``layout.py:84-100``)."""
    f = layout.views(pages)
    role = f["key_map"].long()
    payload = f["key_payload"]
    slots = torch.stack((payload & 15, payload >> 4), -1).flatten(-2).int()
    partner = slots.gather(-1, role.clamp_min(0).unsqueeze(-2).expand_as(slots))
    wide = (slots << 4 | partner) - 128
    code = torch.where(role.unsqueeze(-2) >= 0, wide, slots - 8)
    keys = code.float() * f["key_scales"].unsqueeze(-2)
    padding = f["key_padding"].gather(-1, (-role - 2).clamp_min(0))
    keys = torch.where(role.unsqueeze(-2) <= -2, padding.unsqueeze(-2), keys)
    vp = f["value_payload"]
    codes = torch.stack([(vp >> shift) & 3 for shift in (0, 2, 4, 6)], -1).flatten(-2)
    values = codes.float().reshape(*codes.shape[:-1], 2, 64)
    values = values * f["value_scales"].float().unsqueeze(-1)
    values = values + f["value_offsets"].float().unsqueeze(-1)
    return keys.to(dtype), values.flatten(-2).to(dtype)
