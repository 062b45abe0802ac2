"""Whole-model single-token decode step captured in one CUDA graph.

The reference decodes with one Python call per layer and two Triton launches inside it
(``qwen_fused.py:138-158``); at ~14 MB of packed cache per layer the step is bound by Python and
launch latency, not by the GPU.  ``GraphedDecodeStep`` records the complete forward of a model
patched by ``enable_fused_attention`` -- embedding, every layer's projections, RoPE, the append
and packed-decode kernels of this library, MLPs, the LM head and the greedy arg-max -- into ONE
CUDA graph and replays it per token.  What makes the step replayable:

* every layer appends into the cache's own tail buffer at a position held in a DEVICE counter
  (``DecodeBatch`` of one sequence), so the graph does not depend on the tail length;
* token id and position are static device tensors updated in place;
* the cache's host-side bookkeeping (tail length, sequence length) is applied afterwards by
  ``commit``.  While a graph is attached the stepper registers ``commit`` with the cache
  (``InQuantCache._pending_commit``), and every entry point of the cache that reads or changes its
  lengths (``update``, ``extend``, ``append_for_attention``, ``materialize``, ``get_seq_length``,
  ``memory_stats``) runs it first, so direct use of the cache between steps sees current state.
  A forward of the patched model that does not come from this stepper (a plain ``model(...)`` or
  ``generate`` call) commits, detaches the graph and takes the ordinary path.

When a tail is about to reach the length at which the cache seals a block, the step is run
eagerly once through the ordinary patched forward (which seals exactly as
``InQuantCache.append_for_attention`` does) and the graph is recorded again over the new block
list.  Caches whose value codec the one-launch kernel serves (``PackedDecodeState.streaming_value_kind``),
batch 1, fp16/bf16 models.
"""
from __future__ import annotations

import inspect
from typing import Any

import torch

from .batched import DecodeBatch, SequenceState
from .cache import InQuantCache


class GraphedDecodeStep:
    def __init__(self, model: Any, cache: InQuantCache):
        self.model, self.cache = model, cache
        self.modules = [layer.self_attn for layer in model.model.layers]
        if any(not hasattr(m, "_inquant_original_forward") for m in self.modules):
            raise ValueError("call enable_fused_attention(model) first")
        if model.training or torch.is_grad_enabled():
            raise RuntimeError("Packed decode is inference-only; use model.eval() and torch.no_grad()")
        if cache.get_seq_length() < max(1, cache.config.sink_tokens):
            raise ValueError("prefill the cache (at least the sink) before graphed decode")
        self.device = next(model.parameters()).device
        if self.device.type != "cuda":
            raise RuntimeError("Graphed decode requires CUDA; this library has no CPU path")
        self.token = torch.zeros((1, 1), dtype=torch.long, device=self.device)
        self.position = torch.zeros((1,), dtype=torch.long, device=self.device)
        self.next_token = torch.zeros((1, 1), dtype=torch.long, device=self.device)
        self.logits: torch.Tensor | None = None
        self._takes_cache_position = "cache_position" in inspect.signature(model.forward).parameters
        self._graph: torch.cuda.CUDAGraph | None = None
        self._pending = 0          # replayed steps not yet booked into the cache
        self._driving = False      # True while this stepper itself runs the model's forward
        self._room = 0             # replays left before a tail reaches its sealing length
        self.replays = self.eager_steps = self.captures = 0

    # ------------------------------------------------------------------ graph life cycle
    def _forward(self):
        extra = {"cache_position": self.position} if self._takes_cache_position else {}
        previous, self._driving = self._driving, True
        try:
            out = self.model(input_ids=self.token, position_ids=self.position.view(1, 1), past_key_values=self.cache,
                             use_cache=True, **extra)
        finally:
            self._driving = previous
        return out.logits

    def _detach(self) -> None:
        for module in self.modules:
            module._inquant_graph_batch = None
            module._inquant_graph_owner = None
        if self.cache._pending_commit == self.commit:
            self.cache._pending_commit = None
        self._graph = None

    def _capture(self) -> None:
        cache = self.cache
        capacity = cache._tail_capacity()
        rooms = []
        for index, module in enumerate(self.modules):
            layer = cache._layers[index]
            if layer.sink_count < cache.config.sink_tokens or layer.tail_key_buffer is None:
                raise ValueError("the sink must be full and a tail buffer present before graphed decode")
            heads = module.config.num_attention_heads
            module._inquant_graph_batch = DecodeBatch([SequenceState.from_cache_layer(cache, index)], heads,
                                                      layer.dtype, scale=module.scaling)
            module._inquant_graph_owner = self
            # the cache appends in place while tail + 1 stays below its capacity, then seals
            rooms.append(min(capacity, layer.tail_key_buffer.shape[2]) - 1 - layer.tail_count)
        self._room = min(rooms)
        if self._room < 1:
            self._detach()
            return
        calls = sum(m._inquant_fused_decode_calls for m in self.modules)
        position = self.position.clone()
        # warm-up on a side stream (library handles, kernel attributes), then undo its append
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._forward()
        torch.cuda.current_stream(self.device).wait_stream(side)
        if sum(m._inquant_fused_decode_calls for m in self.modules) - calls != len(self.modules):
            self._detach()
            raise RuntimeError("the model's forward did not reach the packed decode path in every layer")
        for module in self.modules:
            module._inquant_graph_batch.rewind(0)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits = self._forward()
            self.next_token.copy_(logits[:, -1].argmax(-1, keepdim=True))
            self.position.add_(1)
        self.position.copy_(position)
        reached = sum(m._inquant_fused_decode_calls for m in self.modules) - calls
        for module in self.modules:
            module._inquant_graph_batch.rewind(0)
            module._inquant_fused_decode_calls -= 2   # warm-up and capture were not decode steps
        if reached != 2 * len(self.modules):
            self._detach()
            raise RuntimeError("the captured forward did not reach the packed decode path in every layer")
        self.logits, self._graph = logits, graph
        cache._pending_commit = self.commit
        self.captures += 1

    def commit(self) -> None:
        """Book the replayed steps into the cache (tail and sequence lengths)."""
        pending, self._pending = self._pending, 0   # cleared first: the cache calls back into commit
        if not pending:
            return
        for index in range(len(self.modules)):
            layer = self.cache._layers[index]
            layer.tail_count += pending
            layer.seq_length += pending
        for index in range(len(self.modules)):
            self.cache.record_peak(index)
        self.cache._seen_tokens = self.cache._layers[0].seq_length

    def close(self) -> None:
        """Commit and hand the model back to the ordinary patched forward."""
        self.commit()
        self._detach()

    # ------------------------------------------------------------------ stepping
    def step(self, token: torch.Tensor | int | None = None) -> torch.Tensor:
        """Decode one token (``None``: the arg-max of the previous step) and return the logits
        ``[1, 1, vocab]`` -- a static tensor that the next step overwrites."""
        if token is None:
            self.token.copy_(self.next_token)
        elif isinstance(token, torch.Tensor):
            self.token.copy_(token.reshape(1, 1))
        else:
            self.token.fill_(int(token))
        if self._graph is None:
            self.position.fill_(self.cache.get_seq_length())
            self._capture()
        if self._graph is not None and self._room > 0:
            self._graph.replay()
            self._pending += 1
            self._room -= 1
            self.replays += 1
            for module in self.modules:
                module._inquant_fused_decode_calls += 1
            return self.logits
        # a tail is at its sealing length: one ordinary step, then a new graph over the new blocks
        self.commit()
        self._detach()
        logits = self._forward()
        self.next_token.copy_(logits[:, -1].argmax(-1, keepdim=True))
        self.eager_steps += 1
        if self.logits is None or self.logits.shape != logits.shape:
            self.logits = logits.clone()
        else:
            self.logits.copy_(logits)
        return self.logits

    def greedy(self, first_token: torch.Tensor | int, steps: int) -> torch.Tensor:
        """``steps`` greedy tokens after ``first_token`` with no host round trip per token;
        returns them as a ``[steps]`` tensor."""
        out = torch.empty(steps, dtype=torch.long, device=self.device)
        for index in range(steps):
            self.step(first_token if index == 0 else None)
            out[index] = self.next_token[0, 0]
        return out
