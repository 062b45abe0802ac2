"""CPU oracle for the InQuant packed-KV hot path (TEST INFRASTRUCTURE ONLY).

A numpy restatement of the reference algorithm, written from its behaviour and
checked against the reference itself (run on CPU) by ``tests/golden/make_golden.py``;
the resulting vectors are committed under ``tests/golden`` and re-checked by the CPU
test-suite.  Nothing in the shipped package imports this module: only ``tests/``,
``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference`` legs of
``bench.py`` may use it, and only as the checker or the timed CPU baseline.

Reduction orders matter for bit-exactness and are stated explicitly:

* sampled statistics (``codec.py:202-206``): fp32 outer-dimension sum in the
  cascade order torch's CPU kernel uses whenever the channel count is a multiple
  of 64 (all decode-capable layouts have 128 channels): rows are added
  sequentially into a level-0 accumulator which is folded into the next level
  every ``2**max(4, ceil_log2(n)//4)`` rows; the mean is ``sum / n`` (IEEE).
  For other channel counts torch's order depends on the host's vector width, so
  last-ulp differences in ``padding`` are possible there (never for bf16 inputs
  whose sums are exact).
* full-block variance / mean (``codec.py:208-210``): Welford's update in float64,
  sequentially over tokens, then rounded to fp32 -- torch's CPU ``var_mean``.

All arrays are numpy; bf16 tensors are carried as float32 holding bf16-exact values.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

F32_TINY = np.float32(np.finfo(np.float32).tiny)
F16_TINY = np.float32(np.finfo(np.float16).tiny)


# --------------------------------------------------------------------------- dtype helpers
def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16, returned as fp32 (finite inputs)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return rounded.view(np.float32).reshape(x.shape)


def round_to_dtype(x: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "bfloat16":
        return round_to_bf16(x)
    if dtype == "float16":
        return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)
    if dtype == "float32":
        return np.asarray(x, np.float32)
    raise ValueError(dtype)


# --------------------------------------------------------------------------- statistics
def cascade_sum(rows: np.ndarray) -> np.ndarray:
    """fp32 sum over axis -2 of ``rows[..., n, C]`` in torch's CPU cascade order."""
    rows = np.asarray(rows, np.float32)
    n = rows.shape[-2]
    ceil_log2 = 0 if n <= 1 else (n - 1).bit_length()
    level_power = max(4, ceil_log2 // 4)
    step = 1 << level_power
    mask = step - 1
    zero = np.zeros(rows.shape[:-2] + rows.shape[-1:], np.float32)
    acc = [zero.copy() for _ in range(4)]
    i = 0
    while i + step <= n:
        for _ in range(step):
            acc[0] = acc[0] + rows[..., i, :]
            i += 1
        for level in range(1, 4):
            acc[level] = acc[level] + acc[level - 1]
            acc[level - 1] = zero.copy()
            if i & (mask << (level * level_power)):
                break
    while i < n:
        acc[0] = acc[0] + rows[..., i, :]
        i += 1
    for level in range(1, 4):
        acc[0] = acc[0] + acc[level]
    return acc[0]


def sampled_stats(x32: np.ndarray, stride: int) -> tuple[np.ndarray, np.ndarray]:
    """``saliency = mean|x|`` and ``sampled_mean`` over every ``stride``-th token
    (reference ``codec.py:202-206``)."""
    samples = x32[..., ::stride, :]
    n = np.float32(samples.shape[-2])
    return cascade_sum(np.abs(samples)) / n, cascade_sum(samples) / n


def welford_var_mean(x32: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Population variance and mean over tokens, float64 Welford, rounded to fp32
    (torch CPU ``var_mean(correction=0)`` as called at ``codec.py:209``)."""
    x = np.asarray(x32, np.float64)
    mean = np.zeros(x.shape[:-2] + x.shape[-1:], np.float64)
    m2 = np.zeros_like(mean)
    for i in range(x.shape[-2]):
        row = x[..., i, :]
        delta = row - mean
        mean = mean + delta / float(i + 1)
        m2 = m2 + delta * (row - mean)
    return (m2 / float(x.shape[-2])).astype(np.float32), mean.astype(np.float32)


# --------------------------------------------------------------------------- donor selection
def reuse_map(saliency: np.ndarray, count: int, donor_error: np.ndarray | None = None):
    """Sources (salient channels, ascending) and their one-to-one donors.

    Restates ``codec.py:137-178`` / ``triton_selection.py:11-43``: stable top-``count``
    by saliency (ties: lower channel), optional pool of the ``count`` non-salient
    channels of least error (ties: lower channel); each source in ascending order takes
    a free immediate neighbour if there is one, else the free channel(s) nearest to
    either end of its contiguous salient run; among candidates the least saliency wins,
    then the lower channel.
    """
    saliency = np.asarray(saliency, np.float32)
    prefix, channels = saliency.shape[:-1], saliency.shape[-1]
    flat = saliency.reshape(-1, channels)
    rows = flat.shape[0]
    sources = np.zeros((rows, count), np.int64)
    donors = np.zeros((rows, count), np.int64)
    err = None if donor_error is None else np.asarray(donor_error, np.float32).reshape(-1, channels)
    for r in range(rows):
        s = flat[r]
        order = np.argsort(-s.astype(np.float64), kind="stable")  # descending, ties -> lower channel
        src = np.sort(order[:count])
        selected = np.zeros(channels, bool)
        selected[src] = True
        available = ~selected
        if err is not None:
            e = np.where(selected, np.inf, err[r].astype(np.float64))
            pool = np.argsort(e, kind="stable")[:count]
            available = np.zeros(channels, bool)
            available[pool] = True
        for i, source in enumerate(src):
            cands = [c for c in (source - 1, source + 1) if 0 <= c < channels and available[c]]
            if not cands:
                left = source
                while left - 1 >= 0 and selected[left - 1]:
                    left -= 1
                right = source
                while right + 1 < channels and selected[right + 1]:
                    right += 1
                best = None
                for c in np.flatnonzero(available):
                    d = min(abs(int(c) - left), abs(int(c) - right))
                    if best is None or d < best:
                        best, cands = d, [int(c)]
                    elif d == best:
                        cands.append(int(c))
            donor = min(cands, key=lambda c: (float(s[c]), c))
            sources[r, i], donors[r, i] = source, donor
            available[donor] = False
    return sources.reshape(*prefix, count), donors.reshape(*prefix, count)


# --------------------------------------------------------------------------- K4 codec
@dataclass
class PackedK:
    payload: np.ndarray          # uint8 [..., T, C/2]
    scales: np.ndarray           # float32 [..., C]
    salient_channels: np.ndarray  # uint8 (int32 when C > 256) [..., count]
    donor_channels: np.ndarray
    padding: np.ndarray          # float32 [..., count]
    shape: tuple
    dtype: str

    def fields(self):
        return {"payload": self.payload, "scales": self.scales,
                "salient_channels": self.salient_channels,
                "donor_channels": self.donor_channels, "padding": self.padding}


def quantize_k4(x: np.ndarray, dtype: str = "bfloat16", sample_stride: int = 8,
                salient_fraction: float = 0.125, donor_policy: str = "neighbors") -> PackedK:
    """The mixed 4/8-bit key encoder (reference ``codec.py:181-243``).

    ``x`` is fp32 holding values exactly representable in ``dtype``; shape [B,H,T,C].
    """
    x32 = np.asarray(x, np.float32)
    if x32.ndim != 4 or min(x32.shape) < 1:
        raise ValueError("x must have nonempty [batch, heads, tokens, channels] dimensions")
    if x32.shape[-1] % 2:
        raise ValueError("head dimension must be even for two nibbles per byte")
    if not np.isfinite(x32).all():
        raise ValueError("x must contain finite values representable in float32")
    channels = x32.shape[-1]
    count = math.floor(channels * salient_fraction)
    saliency, sampled_mean = sampled_stats(x32, sample_stride)
    donor_error = None
    if donor_policy == "min_error":
        variance, full_mean = welford_var_mean(x32)
        diff = full_mean - sampled_mean
        donor_error = variance + diff * diff
    sources, donors = reuse_map(saliency, count, donor_error)
    selected = np.zeros(saliency.shape, bool)
    np.put_along_axis(selected, sources, True, -1)
    denominator = np.where(selected, np.float32(127.0), np.float32(7.0)).astype(np.float32)
    scales = np.maximum(np.abs(x32).max(-2) / denominator, F32_TINY).astype(np.float32)
    slots = (np.clip(np.rint(x32 / scales[..., None, :]), -7, 7) + 8).astype(np.uint8)
    if count:
        src_t = np.broadcast_to(sources[..., None, :], x32.shape[:-1] + (count,))
        don_t = np.broadcast_to(donors[..., None, :], src_t.shape)
        values = np.take_along_axis(x32, src_t, -1)
        src_scales = np.take_along_axis(scales, sources, -1)[..., None, :]
        codes = (np.clip(np.rint(values / src_scales), -127, 127) + 128).astype(np.uint8)
        np.put_along_axis(slots, src_t, codes >> 4, -1)
        np.put_along_axis(slots, don_t, codes & 15, -1)
    payload = np.ascontiguousarray(slots[..., 0::2] | (slots[..., 1::2] << 4))
    padding = np.take_along_axis(sampled_mean, donors, -1).astype(np.float32)
    ddt = np.uint8 if channels <= 256 else np.int32
    return PackedK(payload, scales, sources.astype(ddt), donors.astype(ddt), padding,
                   tuple(x32.shape), dtype)


def dequantize_k4(p: PackedK, dtype: str | None = None) -> np.ndarray:
    """Exact inverse view of the packed keys (reference ``codec.py:112-134``)."""
    dtype = p.dtype if dtype is None else dtype
    slots = np.stack((p.payload & 15, p.payload >> 4), -1).reshape(*p.payload.shape[:-1], -1)
    decoded = (slots.astype(np.float32) - np.float32(8)) * p.scales[..., None, :]
    count = p.salient_channels.shape[-1]
    if count:
        sources = p.salient_channels.astype(np.int64)
        donors = p.donor_channels.astype(np.int64)
        src_t = np.broadcast_to(sources[..., None, :], slots.shape[:-1] + (count,))
        don_t = np.broadcast_to(donors[..., None, :], src_t.shape)
        high = np.take_along_axis(slots, src_t, -1).astype(np.int32)
        low = np.take_along_axis(slots, don_t, -1).astype(np.int32)
        codes = ((high << 4) | low).astype(np.float32) - np.float32(128)
        src_scales = np.take_along_axis(p.scales, sources, -1)[..., None, :]
        np.put_along_axis(decoded, src_t, (codes * src_scales).astype(np.float32), -1)
        np.put_along_axis(decoded, don_t, np.broadcast_to(p.padding[..., None, :], codes.shape), -1)
    return round_to_dtype(decoded, dtype)


# --------------------------------------------------------------------------- V codec
@dataclass
class PackedV:
    payload: np.ndarray   # uint8 [..., T, C*bits/8]
    scales: np.ndarray    # float16 [..., T, C/group]
    offsets: np.ndarray   # float16
    shape: tuple
    dtype: str
    bits: int
    group_size: int

    def fields(self):
        return {"payload": self.payload, "scales": self.scales, "offsets": self.offsets}


def quantize_values(x: np.ndarray, dtype: str = "bfloat16", bits: int = 2, group_size: int = 64) -> PackedV:
    """Per-token per-group affine INT2/INT4 (reference ``value_codec.py:51-72``)."""
    if bits not in (2, 4):
        raise ValueError("Value bits must be 2 or 4")
    if group_size not in (32, 64, 128):
        raise ValueError("Value group size must be 32, 64 or 128")
    x32 = np.asarray(x, np.float32)
    if x32.ndim != 4 or min(x32.shape) < 1 or x32.shape[-1] % group_size:
        raise ValueError("Expected nonempty floating [batch, heads, tokens, channels] divisible by group_size")
    grouped = x32.reshape(*x32.shape[:-1], -1, group_size)
    lower, upper = grouped.min(-1), grouped.max(-1)
    levels = np.float32((1 << bits) - 1)
    with np.errstate(over="ignore", invalid="ignore"):
        offsets = lower.astype(np.float16)
        scales = np.maximum((upper - lower) / levels, F16_TINY).astype(np.float16)
    if not (np.isfinite(grouped).all() and np.isfinite(offsets).all() and np.isfinite(scales).all()):
        raise ValueError("Values and stored FP16 quantization parameters must be finite")
    codes = (grouped - offsets.astype(np.float32)[..., None]) / scales.astype(np.float32)[..., None]
    codes = np.clip(np.rint(codes), 0, levels).astype(np.uint8).reshape(x32.shape)
    per_byte = 8 // bits
    packed = codes[..., 0::per_byte].copy()
    for index in range(1, per_byte):
        packed |= codes[..., index::per_byte] << np.uint8(index * bits)
    return PackedV(np.ascontiguousarray(packed), offsets=offsets, scales=scales,
                   shape=tuple(x32.shape), dtype=dtype, bits=bits, group_size=group_size)


def dequantize_values(p: PackedV, dtype: str | None = None) -> np.ndarray:
    """``code * scale + offset`` with a separate fp32 multiply and add
    (reference ``value_codec.py:38-48``)."""
    dtype = p.dtype if dtype is None else dtype
    mask = (1 << p.bits) - 1
    slots = np.stack([(p.payload >> np.uint8(s)) & mask for s in range(0, 8, p.bits)], -1)
    slots = slots.reshape(*p.payload.shape[:-1], -1)
    grouped = slots.astype(np.float32).reshape(*p.shape[:-1], -1, p.group_size)
    dense = (grouped * p.scales.astype(np.float32)[..., None]).astype(np.float32)
    dense = dense + p.offsets.astype(np.float32)[..., None]
    return round_to_dtype(dense.reshape(p.shape), dtype)


# --------------------------------------------------------------------------- role maps / pages
def role_map(sources: np.ndarray, donors: np.ndarray, channels: int, dtype=np.int8) -> np.ndarray:
    """Per-channel role: donor index (>=0) for a salient channel, -1 for a normal one,
    ``-2-i`` for the i-th donor (reference ``triton_attention.py:301-309``,
    ``layout.py:73-77``)."""
    sources = np.asarray(sources, np.int64)
    donors = np.asarray(donors, np.int64)
    result = np.full(sources.shape[:-1] + (channels,), -1, dtype)
    np.put_along_axis(result, sources, donors.astype(dtype), -1)
    pad_index = (-2 - np.arange(sources.shape[-1])).astype(dtype)
    np.put_along_axis(result, donors, np.broadcast_to(pad_index, donors.shape), -1)
    return result


def page_fields(block_size: int, heads: int, dim: int = 128):
    """(name, numpy dtype, shape) of one page, in byte order (reference ``layout.py:18-29``)."""
    b, h, d = block_size, heads, dim
    return (
        ("key_payload", np.uint8, (h, b, d // 2)),
        ("key_scales", np.float32, (h, d)),
        ("key_map", np.int16, (h, d)),
        ("key_padding", np.float32, (h, d // 8)),
        ("value_payload", np.uint8, (h, b, d // 4)),
        ("value_scales", np.float16, (h, b, d // 64)),
        ("value_offsets", np.float16, (h, b, d // 64)),
    )


def page_offsets(block_size: int, heads: int, dim: int = 128) -> dict:
    offset, result = 0, {}
    for name, dtype, shape in page_fields(block_size, heads, dim):
        result[name] = offset
        offset += math.prod(shape) * np.dtype(dtype).itemsize
    result["page_bytes"] = offset
    return result


def pack_pages(keys: np.ndarray, values: np.ndarray, block_size: int, heads: int,
               dtype: str = "bfloat16") -> np.ndarray:
    """Seal full pages ``[P,H,B,128]`` into the byte layout (reference ``layout.py:56-81``)."""
    k = quantize_k4(keys, dtype, donor_policy="min_error")
    v = quantize_values(values, dtype, 2, 64)
    offs = page_offsets(block_size, heads)
    pages = np.zeros((keys.shape[0], offs["page_bytes"]), np.uint8)
    parts = {
        "key_payload": k.payload, "key_scales": k.scales,
        "key_map": role_map(k.salient_channels, k.donor_channels, 128, np.int16),
        "key_padding": k.padding, "value_payload": v.payload,
        "value_scales": v.scales, "value_offsets": v.offsets,
    }
    for name, ndt, shape in page_fields(block_size, heads):
        raw = np.ascontiguousarray(parts[name].astype(ndt)).reshape(keys.shape[0], -1).view(np.uint8)
        pages[:, offs[name]:offs[name] + raw.shape[1]] = raw
    return pages


def unpack_pages(pages: np.ndarray, block_size: int, heads: int, dtype: str = "bfloat16"):
    """Dense K and V ``[P,H,B,128]`` from page bytes (reference ``layout.py:84-100``)."""
    offs = page_offsets(block_size, heads)
    f = {}
    for name, ndt, shape in page_fields(block_size, heads):
        size = math.prod(shape) * np.dtype(ndt).itemsize
        f[name] = np.ascontiguousarray(pages[:, offs[name]:offs[name] + size]).view(ndt).reshape(-1, *shape)
    role = f["key_map"].astype(np.int64)
    slots = np.stack((f["key_payload"] & 15, f["key_payload"] >> 4), -1).reshape(*f["key_payload"].shape[:-1], -1)
    partner = np.take_along_axis(slots, np.broadcast_to(np.maximum(role, 0)[..., None, :], slots.shape), -1)
    code = np.where(role[..., None, :] >= 0,
                    ((slots.astype(np.int32) << 4) | partner.astype(np.int32)) - 128,
                    slots.astype(np.int32) - 8)
    keys = code.astype(np.float32) * f["key_scales"][..., None, :]
    padding = np.take_along_axis(f["key_padding"], np.maximum(-role - 2, 0), -1)
    keys = np.where(role[..., None, :] <= -2, padding[..., None, :], keys)
    vp = f["value_payload"]
    codes = np.stack([(vp >> np.uint8(s)) & 3 for s in (0, 2, 4, 6)], -1).reshape(*vp.shape[:-1], -1)
    vals = codes.astype(np.float32).reshape(*codes.shape[:-1], 2, 64)
    vals = (vals * f["value_scales"].astype(np.float32)[..., None]).astype(np.float32)
    vals = vals + f["value_offsets"].astype(np.float32)[..., None]
    return round_to_dtype(keys, dtype), round_to_dtype(vals.reshape(*vals.shape[:-2], 128), dtype)


# --------------------------------------------------------------------------- cache state machine
def seal_plan(sink_have: int, pending_have: int, new_tokens: int, *, sink_tokens: int,
              residual_length: int, block_size: int) -> tuple[int, int, int]:
    """How one append of ``new_tokens`` splits (reference ``cache.py:271-306``):
    returns (tokens taken by the sink, blocks sealed, tokens left in the tail)."""
    take = min(sink_tokens - sink_have, new_tokens)
    pending = pending_have + new_tokens - take
    blocks = max(0, (pending - residual_length) // block_size)
    return take, blocks, pending - blocks * block_size


# --------------------------------------------------------------------------- attention
def attention_decode(query: np.ndarray, keys: np.ndarray, values: np.ndarray, scale: float) -> np.ndarray:
    """Single-query grouped-query attention in float64 over dense K/V.

    ``query`` [Hq,128]; ``keys``/``values`` [Hkv,T,128], already rounded to the model
    dtype as the reference's oracle does (``qwen_fused.py:21-30``).  Returns [Hq,128] fp64.
    """
    hq, hkv = query.shape[0], keys.shape[0]
    group = hq // hkv
    out = np.zeros((hq, keys.shape[-1]), np.float64)
    for h in range(hq):
        k = keys[h // group].astype(np.float64)
        v = values[h // group].astype(np.float64)
        s = (k @ query[h].astype(np.float64)) * scale
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ v
    return out


def attention_partial(query, keys, values, scale):
    """Un-normalised partial ``(acc[Hq,128], m[Hq], l[Hq])`` over one partition, the record
    the reference's split-KV kernel stores (``triton_attention.py:162-165``)."""
    hq, hkv = query.shape[0], keys.shape[0]
    group = hq // hkv
    acc = np.zeros((hq, keys.shape[-1]), np.float64)
    m = np.full(hq, -np.inf)
    l = np.zeros(hq)
    for h in range(hq):
        k = keys[h // group].astype(np.float64)
        v = values[h // group].astype(np.float64)
        s = (k @ query[h].astype(np.float64)) * scale
        m[h] = s.max()
        p = np.exp(s - m[h])
        l[h] = p.sum()
        acc[h] = p @ v
    return acc, m, l


def merge_partials(acc, m, l):
    """Log-sum-exp merge over the leading partition axis (reference
    ``triton_attention.py:168-181``)."""
    top = m.max(0)
    w = np.exp(m - top)
    return (acc * w[..., None]).sum(0) / (l * w).sum(0)[..., None]
