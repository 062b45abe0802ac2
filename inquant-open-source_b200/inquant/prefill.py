"""Chunked-prefill attention over the packed cache on the tcgen05 tensor cores.

The reference serves a query chunk that follows earlier chunks through its stock forward:
``InQuantCache.update`` returns the dequantised history followed by the new states
(``cache.py:179-200``) and the model calls SDPA with a causal mask.  Here the same result comes
from ``inq_prefill_attention``: the history of one layer is dequantised by this library's
kernels into dense tensors, the chunk's keys and values are appended, and one kernel computes
causal attention for every query head (GQA) with both contractions on tcgen05 and the
accumulators in tensor memory.
"""
from __future__ import annotations

import ctypes

import torch

from . import _native as N


# per-device scratch for the kernel's partial results (one stream at a time, like the decode workspace)
_SCRATCH: dict = {}


def prefill_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, scale: float | None = None,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of ``query`` [1, Hq, Tq, 128] over ``key``/``value`` [1, H, L, 128] whose
    last Tq rows belong to the query tokens themselves (query i sees rows 0 .. L - Tq + i)."""
    if query.ndim != 4 or key.ndim != 4 or value.shape != key.shape or query.shape[0] != 1 or key.shape[0] != 1:
        raise ValueError("Expected query [1, Hq, Tq, D] and key/value [1, H, L, D]")
    N.require_cuda(query, "prefill_attention")
    if query.dtype not in (torch.float16, torch.bfloat16) or key.dtype != query.dtype or value.dtype != query.dtype:
        raise NotImplementedError("prefill_attention takes fp16 or bf16 tensors of one dtype")
    if query.shape[3] != 128 or key.shape[3] != 128:
        raise NotImplementedError("prefill_attention requires head_dim=128")
    q_heads, q_tokens = query.shape[1], query.shape[2]
    kv_heads, kv_tokens = key.shape[1], key.shape[2]
    if q_heads % kv_heads or kv_tokens < q_tokens or q_tokens < 1:
        raise ValueError("Query heads must be a multiple of KV heads and the chunk must be part of key/value")
    if key.device != query.device or value.device != query.device:
        raise ValueError("query, key and value must share a device")

    def rows(t):   # 16-byte aligned rows with unit channel stride
        ok = t.stride(3) == 1 and t.stride(1) % 8 == 0 and t.stride(2) % 8 == 0 and t.data_ptr() % 16 == 0
        return t if ok else t.contiguous()
    query, key, value = rows(query), rows(key), rows(value)
    if out is None:
        out = torch.empty((1, q_heads, q_tokens, 128), dtype=query.dtype, device=query.device)
    elif out.shape != (1, q_heads, q_tokens, 128) or out.dtype != query.dtype or rows(out) is not out:
        raise ValueError("out must be a [1, Hq, Tq, 128] tensor of the query dtype with aligned rows")
    need = N.library().inq_prefill_workspace_bytes(q_heads, q_tokens)
    scratch = _SCRATCH.get(query.device)
    if scratch is None or scratch.numel() < need:
        scratch = _SCRATCH[query.device] = torch.empty(max(need, 16), dtype=torch.uint8, device=query.device)
    args = N.PrefillArgs(
        query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(),
        query.stride(1), query.stride(2), key.stride(1), key.stride(2), value.stride(1), value.stride(2),
        out.stride(1), out.stride(2), q_heads, kv_heads, q_tokens, kv_tokens, N.DTYPE_CODE[query.dtype],
        float(scale if scale is not None else 128 ** -0.5), N.status_word(query.device).data_ptr(),
        scratch.data_ptr(), scratch.numel())
    N.check(N.library().inq_prefill_attention(ctypes.byref(args), N.stream_pointer(query.device)), "inq_prefill_attention")
    return out


@torch.no_grad()
def prefill_chunk(cache, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, layer_idx: int,
                  scale: float | None = None, cache_kwargs=None) -> torch.Tensor:
    """One chunk of a chunked prefill for one layer: attention of the chunk's queries over the
    cache's history plus the chunk itself, then the chunk is appended (and sealed) exactly as
    ``InQuantCache.update`` does.  Returns the attention output [1, Hq, Tq, 128]."""
    full_key, full_value = cache.update(key, value, layer_idx, cache_kwargs)
    return prefill_attention(query, full_key, full_value, scale)
