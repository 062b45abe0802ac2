"""Request state machine of the paged serving backend (mirror of the reference's
``extensions/vllm/src/inquant_vllm/backend.py:82-177``) on this library's sm_100a kernels.

``InQuantImpl.forward(layer, query, key, value, kv_cache, attn_metadata, output)`` keeps the
reference's call signature, state transitions and error messages:

* prefill (``context_len == 0``): the first four tokens go to the exact sink, attention runs over
  the fresh uncompressed K/V (here: this library's tcgen05 causal kernel, where the reference calls
  flash-attn), the ``n // block`` full pages are sealed into their physical pages in one encoder
  launch (``pack_pages_into``), the remainder stays exact in ``dense[:, :, 4:4 + rem]``;
* decode: the token is written at ``dense[..., 4 + tail]`` (and into the sink while it fills) by one
  append kernel, ``paged_decode`` attends over pages + sink + tail, and the page that the token
  fills is sealed AFTER attention, so only later queries see its quantised form;
* a decode call whose request id or context length does not continue the stored state is refused
  ("state mismatch"), never served from a stale tail.

What differs from the reference: nothing here imports vLLM (the engine glue -- platform plugin,
worker, metadata builder -- is version-pinned to vLLM 0.9.1 and stays outside this library), so the
class is a plain object with the attributes vLLM's ``FlashAttentionImpl.__init__`` would set; and
the state is kept PER REQUEST ID, so several requests can be active at once
(``max_requests``; the reference serves one).  ``forward`` accepts one request's metadata or an
``InQuantBatchMetadata`` that lists several decode requests, which are then served one after
another on the current stream.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field

import torch

from inquant import _native as N
from inquant.triton_attention import SharedDecodeWorkspace

from .kernels import paged_decode
from .layout import PageLayout, pack_pages, pack_pages_into

# One scratch allocation per process, consumed in stream order (reference ``backend.py:13-15``).
WORKSPACE = SharedDecodeWorkspace()


def get_current_vllm_config():
    """vLLM's current configuration (only ``cache_config.block_size`` and
    ``model_config.max_model_len`` are read).  Resolved lazily so that this module imports
    without vLLM; tests replace it, as the reference's tests do."""
    from vllm.config import get_current_vllm_config as current
    return current()


@dataclass
class InQuantMetadata:
    """Reference ``backend.py:18-25``."""
    num_actual_tokens: int
    seq_len: int
    context_len: int
    query_start_loc: torch.Tensor
    block_table: torch.Tensor
    request_id: str


@dataclass
class InQuantBatchMetadata:
    """Several single-token decode requests of one step: ``requests[i]`` describes request i, whose
    query / key / value / output rows are row i of the tensors passed to ``forward``."""
    requests: list = field(default_factory=list)


@dataclass
class _Request:
    dense: torch.Tensor        # [2, H, block + 4, 128]: exact sink in tokens 0..3, unsealed tail from token 4
    tokens: int = 0
    sealed_pages: int = 0


class InQuantImpl:
    def __init__(self, num_heads, head_size, scale, num_kv_heads=None, alibi_slopes=None, sliding_window=None,
                 kv_cache_dtype="auto", blocksparse_params=None, logits_soft_cap=None, attn_type="decoder",
                 kv_sharing_target_layer_name=None, use_irope=False, *, max_requests: int = 1):
        self.num_heads, self.head_size, self.scale = int(num_heads), int(head_size), float(scale)
        self.num_kv_heads = int(num_heads if num_kv_heads is None else num_kv_heads)
        if alibi_slopes is not None or sliding_window not in (None, (-1, -1)) or logits_soft_cap:
            raise ValueError("InQuant supports full causal attention without ALiBi/softcap")
        if kv_sharing_target_layer_name is not None or use_irope:
            raise ValueError("KV sharing and iRoPE are not implemented")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("Query heads must be a multiple of KV heads")
        self.num_queries_per_kv = self.num_heads // self.num_kv_heads
        if self.num_queries_per_kv > 16:
            raise ValueError("At most 16 query heads per KV head")
        if self.head_size != 128:
            raise ValueError("InQuant pages hold heads of 128 channels")
        if max_requests < 1:
            raise ValueError("max_requests must be positive")
        config = get_current_vllm_config()
        self.layout = PageLayout(config.cache_config.block_size, self.num_kv_heads, self.head_size)
        self.max_pages = math.ceil(config.model_config.max_model_len / self.layout.block_size)
        self.max_requests = int(max_requests)
        self.requests: dict[str, _Request] = {}
        self._free: list[torch.Tensor] = []
        self.max_tokens_seen = 0
        self.prefill_calls = self.decode_calls = self.seal_calls = 0

    # ------------------------------------------------------------------ the reference's single-request view
    @property
    def request_id(self):
        return next(reversed(self.requests), None)

    @property
    def tokens(self) -> int:
        return self.requests[self.request_id].tokens if self.requests else 0

    @property
    def sealed_pages(self) -> int:
        return self.requests[self.request_id].sealed_pages if self.requests else 0

    @property
    def dense(self):
        return self.requests[self.request_id].dense if self.requests else (self._free[-1] if self._free else None)

    # ------------------------------------------------------------------ storage
    def _new_dense(self, query) -> torch.Tensor:
        if self._free:
            return self._free.pop()
        return torch.empty((2, self.num_kv_heads, self.layout.block_size + 4, 128), dtype=query.dtype, device=query.device)

    def _allocate_aux(self, query) -> None:
        """Auxiliary storage exists before the engine budgets its page pool (reference ``backend.py:99-104``)."""
        if not self.requests and not self._free:
            self._free.append(self._new_dense(query))
        WORKSPACE.acquire((self.num_heads, self.max_pages + 1, 130), query.device)

    def finish_request(self, request_id: str) -> None:
        """Forget a request; its exact-tail buffer is reused by the next prefill."""
        state = self.requests.pop(request_id, None)
        if state is not None:
            self._free.append(state.dense)

    def _seal(self, keys, values, cache, block_table, start_page) -> None:
        """All new full pages in one encoder launch, scattered by the engine's physical block table
        (any page order, reused page ids; reference ``backend.py:106-116``)."""
        ids = block_table[start_page:start_page + keys.shape[0]]
        if os.environ.get("INQUANT_DIRECT_WRITE", "1") == "1":
            pack_pages_into(keys, values, self.layout, cache, ids,
                            donor_backend=os.environ.get("INQUANT_DONOR_BACKEND", "torch"))
        else:
            cache.index_copy_(0, ids.long(), pack_pages(keys, values, self.layout))
        self.seal_calls += 1

    # ------------------------------------------------------------------ steps
    def _prefill(self, m, query, key, value, kv_cache, output) -> None:
        from inquant.prefill import prefill_attention
        n, b = m.num_actual_tokens, self.layout.block_size
        self.finish_request(m.request_id)
        while len(self.requests) >= self.max_requests:      # the oldest request makes room
            self.finish_request(next(iter(self.requests)))
        state = _Request(self._new_dense(query), tokens=n, sealed_pages=n // b)
        sink = min(4, n)
        state.dense[0, :, :sink].copy_(key[:sink].transpose(0, 1))
        state.dense[1, :, :sink].copy_(value[:sink].transpose(0, 1))
        # the whole prompt attends to its fresh, uncompressed K/V; no dense history is kept afterwards
        result = prefill_attention(query[:n].transpose(0, 1).unsqueeze(0), key[:n].transpose(0, 1).unsqueeze(0),
                                   value[:n].transpose(0, 1).unsqueeze(0), self.scale)
        output[:n].copy_(result[0].transpose(0, 1))
        if state.sealed_pages:
            full = state.sealed_pages * b
            keys = key[:full].view(state.sealed_pages, b, self.num_kv_heads, 128).transpose(1, 2)
            values = value[:full].view(state.sealed_pages, b, self.num_kv_heads, 128).transpose(1, 2)
            self._seal(keys, values, kv_cache, m.block_table, 0)
        rem = n % b
        if rem:
            state.dense[0, :, 4:4 + rem].copy_(key[n - rem:n].transpose(0, 1))
            state.dense[1, :, 4:4 + rem].copy_(value[n - rem:n].transpose(0, 1))
        self.requests[m.request_id] = state
        self.prefill_calls += 1
        self.max_tokens_seen = max(self.max_tokens_seen, state.tokens)

    def _write_token(self, state: _Request, key_row, value_row, tail: int) -> None:
        """The new token's rows into the exact tail (and the sink while it fills): one launch of the
        append kernel when the rows meet its 16-byte rules, else the reference's copies."""
        dense, es = state.dense, state.dense.element_size()
        row_bytes = 128 * es
        aligned = (key_row.stride(-1) == 1 and value_row.stride(-1) == 1 and key_row.data_ptr() % 16 == 0
                   and value_row.data_ptr() % 16 == 0 and (key_row.stride(0) * es) % 16 == 0
                   and key_row.stride(0) == value_row.stride(0))
        if not aligned:
            dense[0, :, 4 + tail].copy_(key_row)
            dense[1, :, 4 + tail].copy_(value_row)
            if state.tokens < 4:
                dense[0, :, state.tokens].copy_(key_row)
                dense[1, :, state.tokens].copy_(value_row)
            return
        args = N.AppendArgs()
        args.key, args.value, args.src_stride_h = key_row.data_ptr(), value_row.data_ptr(), key_row.stride(0) * es
        args.tail_key = dense.data_ptr() + 4 * dense.stride(2) * es
        args.tail_value = args.tail_key + dense.stride(0) * es
        args.tail_stride_h, args.tail_stride_t = dense.stride(1) * es, dense.stride(2) * es
        args.tail_position, args.tail_capacity = tail, self.layout.block_size
        args.sink_position = state.tokens if state.tokens < 4 else -1
        if state.tokens < 4:
            args.sink_key, args.sink_value = dense.data_ptr(), dense.data_ptr() + dense.stride(0) * es
            args.sink_stride_h, args.sink_stride_t = dense.stride(1) * es, dense.stride(2) * es
        args.heads, args.row_bytes = self.num_kv_heads, row_bytes
        args.status = N.status_word(dense.device).data_ptr()
        N.check(N.library().inq_append_token(N.ctypes.byref(args), N.stream_pointer(dense.device)), "inq_append_token")

    def _decode(self, m, query, key, value, kv_cache, output) -> None:
        b = self.layout.block_size
        state = self.requests.get(m.request_id)
        if state is None or m.context_len != state.tokens or m.num_actual_tokens != 1:
            raise RuntimeError("InQuant request state mismatch; refusing stale tail reuse")
        tail = state.tokens % b
        self._write_token(state, key[0], value[0], tail)
        state.tokens += 1
        paged_decode(query[:1], kv_cache, m.block_table, state.dense, state.sealed_pages, tail + 1, min(4, state.tokens),
                     self.layout, WORKSPACE, self.scale, output[:1])
        # the query that fills a page still used its exact values; the page is sealed afterwards
        if tail + 1 == b:
            self._seal(state.dense[0, :, 4:].unsqueeze(0), state.dense[1, :, 4:].unsqueeze(0), kv_cache, m.block_table,
                       state.sealed_pages)
            state.sealed_pages += 1
        self.requests[m.request_id] = self.requests.pop(m.request_id)     # most recently used last
        self.decode_calls += 1
        self.max_tokens_seen = max(self.max_tokens_seen, state.tokens)

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None):
        if output is None:
            raise ValueError("vLLM must supply an output buffer")
        self._allocate_aux(query)
        if attn_metadata is None:
            # a memory-profiling call: auxiliary storage exists now, request state is untouched
            return output
        if kv_cache.dtype != torch.uint8 or kv_cache.ndim != 2 or kv_cache.shape[1] != self.layout.page_bytes:
            raise RuntimeError("InQuant cache spec was not installed; refusing dense fallback")
        if isinstance(attn_metadata, InQuantBatchMetadata):
            for row, m in enumerate(attn_metadata.requests):
                if m.context_len == 0 or m.num_actual_tokens != 1:
                    raise RuntimeError("a batch lists single-token decode requests only")
                self._decode(m, query[row:row + 1], key[row:row + 1], value[row:row + 1], kv_cache, output[row:row + 1])
            return output
        if attn_metadata.context_len == 0:
            self._prefill(attn_metadata, query, key, value, kv_cache, output)
        else:
            self._decode(attn_metadata, query, key, value, kv_cache, output)
        return output
