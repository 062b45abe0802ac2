"""Instance-local Qwen2.5 / Mistral single-token decode over the packed KV cache
(mirror of the reference's ``src/inquant/qwen_fused.py:1-188``).

``enable_fused_attention(model)`` replaces the ``forward`` of every attention module of ONE
instantiated model.  A decode step (batch 1, one new token, no explicit mask, an
``InQuantCache`` that already holds a prefill) projects q/k/v, applies RoPE, appends the new
token with ``InQuantCache.append_for_attention`` and runs the packed decode kernel of this
library through ``PackedDecodeState.decode``; every other call (prefill, masks,
``output_attentions``, other cache types) goes to the module's original forward.

Differences from the reference, none visible through the call signatures:

* the attention interface of both Transformers 4.53 (``past_key_value=``) and 5.x
  (``past_key_values=``) is accepted;
* ``fused_prefill=True`` (not in the reference) also routes query chunks that FOLLOW earlier
  tokens of an ``InQuantCache`` through this library's tcgen05 prefill kernel
  (``inquant.prefill.prefill_chunk``) instead of the stock forward; the chunk is attended
  causally and any mask the model built is ignored, so enable it only for unpadded batch-one
  prompts.  A ``PrefillHistory`` of the cache stored by the caller as ``cache._prefill_history``
  is used (the dense history is then kept across chunks instead of being rebuilt per chunk);
* there is no CPU path in this library: ``allow_cpu_reference`` is accepted for signature
  compatibility, but a non-CUDA decode step always raises (the reference would run its
  materialising oracle there), and ``cpu_reference_calls`` therefore stays 0.
"""
from __future__ import annotations

from dataclasses import dataclass
import inspect
from types import MethodType
from typing import Any

import torch

from .cache import InQuantCache


@dataclass
class _KernelState:
    kernel: Any

    @property
    def nbytes(self) -> int:
        return self.kernel.nbytes


@dataclass
class FusedQwen2Handle:
    """Owns only this model's forward overrides; restore removes them."""
    originals: list[tuple[Any, Any]]
    restored: bool = False

    @property
    def fused_decode_calls(self) -> int:
        return sum(getattr(module, "_inquant_fused_decode_calls", 0) for module, _ in self.originals)

    @property
    def fused_prefill_calls(self) -> int:
        return sum(getattr(module, "_inquant_fused_prefill_calls", 0) for module, _ in self.originals)

    @property
    def cpu_reference_calls(self) -> int:
        return sum(getattr(module, "_inquant_cpu_reference_calls", 0) for module, _ in self.originals)

    def restore(self) -> None:
        if self.restored:
            return
        for module, original in self.originals:
            module.forward = original
            delattr(module, "_inquant_original_forward")
        self.restored = True

    def __enter__(self) -> "FusedQwen2Handle":
        return self

    def __exit__(self, *_args) -> None:
        self.restore()


def _attention_class(model: Any):
    model_type = getattr(model.config, "model_type", None)
    if model_type == "qwen2":
        from transformers.models.qwen2.modeling_qwen2 import Qwen2Attention as Attention, apply_rotary_pos_emb
    elif model_type == "mistral":
        from transformers.models.mistral.modeling_mistral import MistralAttention as Attention, apply_rotary_pos_emb
        if getattr(model.config, "sliding_window", None) is not None:
            raise ValueError("Mistral sliding-window attention requires a window-aware cache and is not supported")
    else:
        raise ValueError("Expected a dense Qwen2 or Mistral model")
    return Attention, apply_rotary_pos_emb


def enable_fused_attention(model: Any, *, allow_cpu_reference: bool = False,
                           fused_prefill: bool = False) -> FusedQwen2Handle:
    """Patch this instantiated model only; retain its weights and prefill forward
    (reference ``qwen_fused.py:71-174``).

    The packed path requires CUDA, head_dim=128, batch=1, q_len=1, full attention, no padding
    mask and an InQuantCache.  Other query lengths and cache types retain the original forward.
    Arbitrary masks/output_attentions also retain the original forward and therefore may
    materialize KV.
    """
    Attention, apply_rotary_pos_emb = _attention_class(model)
    if model.training:
        raise ValueError("Call model.eval() before enabling inference-only packed decode")
    modules = [layer.self_attn for layer in model.model.layers]
    cache_names = []
    for module in modules:
        if not isinstance(module, Attention):
            raise TypeError("Expected an unmodified attention instance for this model family")
        parameters = inspect.signature(module.forward).parameters
        if "position_embeddings" not in parameters:
            raise RuntimeError("Unsupported Transformers attention interface; validated versions are 4.53.x and 5.x")
        cache_names.append("past_key_values" if "past_key_values" in parameters else "past_key_value")
        if getattr(module, "sliding_window", None) is not None:
            raise ValueError("Sliding-window attention is unsupported by packed decode")
        if hasattr(module, "_inquant_original_forward"):
            raise ValueError("This model already has fused InQuant decode enabled")
        if module.head_dim != 128:
            raise ValueError("The CUDA packed decode kernel currently requires head_dim=128")

    def forward(
        attention,
        hidden_states: torch.Tensor,
        position_embeddings: tuple[torch.Tensor, torch.Tensor],
        attention_mask: torch.Tensor | None = None,
        past_key_values=None,
        past_key_value=None,
        cache_position=None,
        **kwargs,
    ):
        cache = past_key_values if past_key_values is not None else past_key_value
        use_packed = (
            isinstance(cache, InQuantCache)
            and hidden_states.shape[1] == 1
            and cache.get_seq_length(attention.layer_idx) > 0
            # inside a graphed step (inquant.graph_decode) the model may hand over the all-true
            # causal mask of a single query token, which Transformers materialises while a
            # stream is capturing; batch one has no padding, so it carries no information
            and (attention_mask is None or attention._inquant_graph_batch is not None)
            and not kwargs.get("output_attentions", False)
        )
        use_prefill = (
            fused_prefill and not use_packed
            and isinstance(cache, InQuantCache)
            and hidden_states.shape[0] == 1 and hidden_states.shape[1] > 1
            and hidden_states.device.type == "cuda"
            and hidden_states.dtype in (torch.float16, torch.bfloat16)
            and cache.get_seq_length(attention.layer_idx) > 0
            and not kwargs.get("output_attentions", False)
            and not torch.is_grad_enabled()
        )
        if use_prefill:
            from .prefill import prefill_chunk
            input_shape = hidden_states.shape[:-1]
            hidden_shape = (*input_shape, -1, attention.head_dim)
            query = attention.q_proj(hidden_states).view(hidden_shape).transpose(1, 2)
            key = attention.k_proj(hidden_states).view(hidden_shape).transpose(1, 2)
            value = attention.v_proj(hidden_states).view(hidden_shape).transpose(1, 2)
            cos, sin = position_embeddings
            query, key = apply_rotary_pos_emb(query, key, cos, sin)
            history = getattr(cache, "_prefill_history", None)
            if history is not None and history.cache is not cache:
                history = None
            result = prefill_chunk(cache, query, key, value, attention.layer_idx, attention.scaling, history=history)
            attention._inquant_fused_prefill_calls += 1
            output = result.transpose(1, 2).reshape(*input_shape, -1).contiguous()
            return attention.o_proj(output), None
        if not use_packed:
            extra = dict(kwargs)
            extra[attention._inquant_cache_name] = cache
            if cache_position is not None or "cache_position" in inspect.signature(
                    attention._inquant_original_forward).parameters:
                extra["cache_position"] = cache_position
            return attention._inquant_original_forward(
                hidden_states=hidden_states, position_embeddings=position_embeddings,
                attention_mask=attention_mask, **extra,
            )
        if attention.training or torch.is_grad_enabled():
            raise RuntimeError("Packed decode is inference-only; use model.eval() and torch.no_grad()")
        if hidden_states.shape[0] != 1:
            raise ValueError("Packed decode supports batch size 1 only")
        if hidden_states.device.type != "cuda":
            raise RuntimeError("Packed decode requires CUDA; this library has no CPU reference path")
        input_shape = hidden_states.shape[:-1]
        hidden_shape = (*input_shape, -1, attention.head_dim)
        query = attention.q_proj(hidden_states).view(hidden_shape).transpose(1, 2)
        key = attention.k_proj(hidden_states).view(hidden_shape).transpose(1, 2)
        value = attention.v_proj(hidden_states).view(hidden_shape).transpose(1, 2)
        cos, sin = position_embeddings
        query, key = apply_rotary_pos_emb(query, key, cos, sin)
        graph_batch = attention._inquant_graph_batch
        owner = getattr(attention, "_inquant_graph_owner", None)
        if graph_batch is not None and not (owner is not None and owner._driving):
            # a forward that does not come from the graphed stepper: book its replayed tokens into
            # the cache, drop the graph and decode through the ordinary path
            if owner is not None:
                owner.close()
            else:
                attention._inquant_graph_batch = None
            graph_batch = None
        if graph_batch is not None:
            # graph-safe step (inquant.graph_decode): the tail length lives in a device counter and
            # the cache's host bookkeeping is applied afterwards, so nothing here depends on the step
            graph_batch.queries[0].copy_(query[0, :, 0])
            graph_batch.new_keys[0].copy_(key[0, :, 0])
            graph_batch.new_values[0].copy_(value[0, :, 0])
            graph_batch._launch_step()   # attention over history + the new token, which is appended by the same launch
            attention._inquant_fused_decode_calls += 1
            return attention.o_proj(graph_batch.outputs.reshape(*input_shape, -1)), None
        view = cache.append_for_attention(
            key, value, attention.layer_idx,
            {"sin": sin, "cos": cos, "cache_position": cache_position},
        )
        from .triton_attention import PackedDecodeState, SharedDecodeWorkspace
        if cache.config.shared_workspace and cache._shared_decode_workspace is None:
            cache._shared_decode_workspace = SharedDecodeWorkspace()
        state = cache._attention_states.get(attention.layer_idx)
        if state is None:
            state = _KernelState(PackedDecodeState(
                view.key_blocks, view.value_blocks,
                workspace_pool=cache._shared_decode_workspace))
            cache._attention_states[attention.layer_idx] = state
        elif len(state.kernel.key_blocks) != len(view.key_blocks):
            state.kernel.extend(view.key_blocks, view.value_blocks)
        result = state.kernel.decode(
            query, sink_key=view.sink_key, sink_value=view.sink_value,
            residual_key=view.residual_key, residual_value=view.residual_value,
            scale=attention.scaling,
        )
        cache.record_peak(attention.layer_idx)
        attention._inquant_fused_decode_calls += 1
        output = result.transpose(1, 2).reshape(*input_shape, -1).contiguous()
        return attention.o_proj(output), None

    originals = []
    for module, cache_name in zip(modules, cache_names):
        originals.append((module, module.forward))
        module._inquant_original_forward = module.forward
        module._inquant_cache_name = cache_name
        module._inquant_fused_decode_calls = 0
        module._inquant_cpu_reference_calls = 0
        module._inquant_fused_prefill_calls = 0
        module._inquant_graph_batch = None
        module._inquant_graph_owner = None
        module.forward = MethodType(forward, module)
    return FusedQwen2Handle(originals)


def enable_fused_qwen2(model: Any, *, allow_cpu_reference: bool = False) -> FusedQwen2Handle:
    """Backward-compatible Qwen-only entry point (reference ``qwen_fused.py:177-181``)."""
    if getattr(model.config, "model_type", None) != "qwen2":
        raise ValueError("Expected a dense Qwen2/Qwen2.5 model")
    return enable_fused_attention(model, allow_cpu_reference=allow_cpu_reference)


def enable_fused_mistral(model: Any, *, allow_cpu_reference: bool = False) -> FusedQwen2Handle:
    """Mistral full-attention entry point; preserves native projections and RoPE
    (reference ``qwen_fused.py:184-188``)."""
    if getattr(model.config, "model_type", None) != "mistral":
        raise ValueError("Expected a dense Mistral model")
    return enable_fused_attention(model, allow_cpu_reference=allow_cpu_reference)
