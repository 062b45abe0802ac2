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


class PrefillHistory:
    """Dense copy of what the next chunk of a prompt attends to, kept across chunks.

    ``InQuantCache.update`` rebuilds the whole dequantised history for every chunk and
    concatenates the new states behind it (reference ``cache.py:179-200, 328-345``): over a
    prompt that is quadratic in copies and dequantisation.  This object holds, per layer, one
    ``[1, H, capacity, C]`` key and value tensor indexed by absolute token position with the same
    contents -- the exact sink, the DEQUANTISED sealed blocks, the exact tail -- and keeps it
    current: a chunk's exact keys and values are written behind the history, the attention kernel
    reads the tensors in place, and after the cache has sealed blocks only those new blocks are
    dequantised over the exact rows they replace.  Every block is restored once.

    With ``defer_checks`` (the default) the encoders' finite check does not synchronise after every
    seal: a non-finite input sets a bit in the device status word instead of raising at once, and
    ``check`` -- to be called when the prompt is done -- raises the ``ValueError`` then (the cache
    contents are undefined after that; reset it).  ``defer_checks=False`` keeps the reference's
    behaviour of raising inside the call, at one stream synchronisation per sealed tensor.

    The price of keeping it is memory: 2 * layers * H * tokens * C elements of the model dtype while
    the prompt is being prefilled (1.9 GB for 32768 tokens of a 28-layer, 4-KV-head model) -- the
    dense cache the packed one exists to avoid.  ``persistent=False`` (the default) therefore keeps
    NO per-layer copy: one scratch pair serves every layer, and a layer's history is rebuilt into it
    from the packed cache for each of its chunks (sink and tail copied, every sealed block
    dequantised by ONE launch addressed through the layer's decode descriptors,
    ``inq_restore_blocks_table``: a few per cent of the chunk's attention time).  That is
    the reference's own semantics (``update`` materialises per call) at 2 * H * tokens * C elements
    in total (71 MB for the same prompt).  ``persistent=True`` keeps the per-layer copies and
    dequantises every block once.  ``release`` frees either.  Tensors grow geometrically unless
    ``capacity_tokens`` covers the prompt.
    """

    def __init__(self, cache, capacity_tokens: int = 4096, defer_checks: bool = True, persistent: bool = False):
        if capacity_tokens < 1:
            raise ValueError("capacity_tokens must be positive")
        self.cache, self.capacity_tokens, self.defer_checks = cache, int(capacity_tokens), bool(defer_checks)
        self.persistent = bool(persistent)
        self._layers: dict[int, list] = {}    # layer -> [key, value, tokens, restored blocks]
        self._scratch: list = [None, None, 0, 0]   # the shared pair of the non-persistent mode
        self._descriptors: dict[int, object] = {}  # layer -> decode descriptors of its sealed blocks (block table, role map)

    def release(self) -> None:
        self._layers.clear()
        self._descriptors.clear()
        self._scratch = [None, None, 0, 0]

    def _restore_all(self, layer_idx: int, layer, out_key: torch.Tensor, out_value: torch.Tensor, position: int) -> int | None:
        """Every sealed block of the layer into the two histories by ONE launch, addressed through the
        layer's decode descriptors (kept here and extended by the blocks each chunk seals); None when the
        layout is not the one that launch serves (then the blocks are restored arena by arena)."""
        from .triton_attention import PackedDecodeState
        blocks = len(layer.key_blocks)
        if not blocks:
            return position
        state = self._descriptors.get(layer_idx)
        try:
            if state is None or len(state.key_blocks) > blocks:
                state = self._descriptors[layer_idx] = PackedDecodeState(layer.key_blocks, layer.value_blocks)
            elif len(state.key_blocks) < blocks:
                state.extend(layer.key_blocks, layer.value_blocks)
        except (ValueError, RuntimeError):
            self._descriptors.pop(layer_idx, None)
            return None
        channels = out_key.shape[3]
        if not state._preset or channels != 128 or out_key.dtype not in (torch.float16, torch.bfloat16) \
                or out_key.stride(3) != 1 or out_key.stride(2) != channels or out_value.stride() != out_key.stride():
            return None
        tokens = state._packed_tokens
        rc = N.library().inq_restore_blocks_table(state._tables.data_ptr(), state._key_map.data_ptr(), blocks, out_key.shape[1],
                                                  tokens, state._salient, out_key.data_ptr(), out_value.data_ptr(),
                                                  out_key.stride(1), position, N.DTYPE_CODE[out_key.dtype],
                                                  N.stream_pointer(out_key.device))
        N.check(rc, "inq_restore_blocks_table")
        return position + blocks * tokens

    def check(self) -> None:
        """Raise for failures recorded while checks were deferred (synchronises the stream)."""
        devices = {state[0].device for state in list(self._layers.values()) + [self._scratch] if state[0] is not None}
        for device in devices:
            status = N.take_status(device)
            if status & N.STATUS_NONFINITE:
                raise ValueError("K/V must contain finite values representable in float32 (reported by a deferred check)")
            if status:
                raise RuntimeError(f"a kernel reported status {status} during the prefill")

    @property
    def nbytes(self) -> int:
        return sum(s[0].numel() * s[0].element_size() * 2 for s in list(self._layers.values()) + [self._scratch] if s[0] is not None)

    def _room(self, state: list, tokens: int, like: torch.Tensor) -> None:
        key = state[0]
        if key is not None and key.shape[2] >= tokens:
            return
        capacity = max(tokens, self.capacity_tokens if key is None else 2 * key.shape[2])
        shape = (1, like.shape[1], capacity, like.shape[3])
        grown = [torch.empty(shape, dtype=like.dtype, device=like.device) for _ in range(2)]
        if key is not None and state[2]:
            grown[0][:, :, :state[2]].copy_(state[0][:, :, :state[2]])
            grown[1][:, :, :state[2]].copy_(state[1][:, :, :state[2]])
        state[0], state[1] = grown

    @torch.no_grad()
    def chunk(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, layer_idx: int,
              scale: float | None = None, cache_kwargs=None) -> torch.Tensor:
        """Attention of the chunk over history + chunk, then append and seal; see ``prefill_chunk``."""
        from .cache import restore_blocks
        cache = self.cache
        if not self.persistent:
            return self._chunk_from_packed(query, key, value, layer_idx, scale, cache_kwargs)
        state = self._layers.setdefault(layer_idx, [None, None, 0, 0])
        seen = cache.get_seq_length(layer_idx) if layer_idx in cache._layers else 0
        if state[2] != seen and state[2] != 0:
            raise RuntimeError("state mismatch: the cache was updated outside this prefill history")
        cache._validate_update(key, value, layer_idx, cache_kwargs)
        tokens = key.shape[2]
        self._room(state, seen + tokens, key)
        if state[2] != seen:
            # first use on a layer that already holds tokens (e.g. a first chunk that went through
            # the model's stock forward): take the history over from the cache once
            old_key, old_value = cache.materialize(layer_idx)
            state[0][:, :, :seen].copy_(old_key)
            state[1][:, :, :seen].copy_(old_value)
            state[2], state[3] = seen, len(cache._layers[layer_idx].key_blocks)
        state[0][:, :, seen:seen + tokens].copy_(key)
        state[1][:, :, seen:seen + tokens].copy_(value)
        out = prefill_attention(query, state[0][:, :, :seen + tokens], state[1][:, :, :seen + tokens], scale)
        if self.defer_checks:
            with N.deferred_status():
                cache.extend(key, value, layer_idx, cache_kwargs)
        else:
            cache.extend(key, value, layer_idx, cache_kwargs)
        layer = cache._layers[layer_idx]
        if len(layer.key_blocks) > state[3]:
            # blocks follow the sink; the block length is fixed per cache
            position = layer.sink_count + state[3] * cache.config.block_size
            restore_blocks(layer.key_blocks[state[3]:], state[0], position)
            restore_blocks(layer.value_blocks[state[3]:], state[1], position)
            state[3] = len(layer.key_blocks)
        state[2] = seen + tokens
        return out


    def _chunk_from_packed(self, query, key, value, layer_idx, scale, cache_kwargs) -> torch.Tensor:
        """One chunk with the layer's history rebuilt from the packed cache into the shared scratch."""
        from .cache import restore_blocks
        cache, scratch = self.cache, self._scratch
        seen = cache.get_seq_length(layer_idx) if layer_idx in cache._layers else 0
        cache._validate_update(key, value, layer_idx, cache_kwargs)
        tokens = key.shape[2]
        scratch[2] = 0          # nothing of another layer's contents is kept
        if scratch[0] is not None and (scratch[0].dtype != key.dtype or scratch[0].device != key.device
                                       or scratch[0].shape[1] != key.shape[1] or scratch[0].shape[3] != key.shape[3]):
            scratch[0] = scratch[1] = None
        self._room(scratch, seen + tokens, key)
        if seen:
            layer = cache._layers[layer_idx]
            sink_tokens = 0 if layer.sink_key is None else layer.sink_key.shape[2]
            after_blocks = self._restore_all(layer_idx, layer, scratch[0], scratch[1], sink_tokens)
            for out, sink, blocks, tail in ((scratch[0], layer.sink_key, layer.key_blocks, layer.residual_key),
                                            (scratch[1], layer.sink_value, layer.value_blocks, layer.residual_value)):
                position = sink_tokens
                if position:
                    out[:, :, :position].copy_(sink)
                position = restore_blocks(blocks, out, position) if after_blocks is None else after_blocks
                if tail is not None and tail.shape[2]:
                    out[:, :, position:position + tail.shape[2]].copy_(tail)
        scratch[0][:, :, seen:seen + tokens].copy_(key)
        scratch[1][:, :, seen:seen + tokens].copy_(value)
        out = prefill_attention(query, scratch[0][:, :, :seen + tokens], scratch[1][:, :, :seen + tokens], scale)
        if self.defer_checks:
            with N.deferred_status():
                cache.extend(key, value, layer_idx, cache_kwargs)
        else:
            cache.extend(key, value, layer_idx, cache_kwargs)
        return out


@torch.no_grad()
def prefill_chunk(cache, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, layer_idx: int,
                  scale: float | None = None, cache_kwargs=None, history: PrefillHistory | None = None) -> torch.Tensor:
    """One chunk of a chunked prefill for one layer: attention of the chunk's queries over the
    cache's history plus the chunk itself, then the chunk is appended (and sealed) exactly as
    ``InQuantCache.update`` does.  Returns the attention output [1, Hq, Tq, 128].

    Without ``history`` the dense history comes from ``InQuantCache.update`` (rebuilt per chunk, as
    in the reference); with a ``PrefillHistory`` that was used for every earlier chunk of this
    layer it is kept across chunks and only new blocks are dequantised."""
    if history is not None:
        if history.cache is not cache:
            raise ValueError("the prefill history belongs to another cache")
        return history.chunk(query, key, value, layer_idx, scale, cache_kwargs)
    full_key, full_value = cache.update(key, value, layer_idx, cache_kwargs)
    return prefill_attention(query, full_key, full_value, scale)
