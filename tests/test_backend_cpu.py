"""Host-side checks of the paged backend's state machine that need no GPU: configuration
gatekeeping of the constructor and the metadata containers (the reference pins the same messages,
extensions/vllm/src/inquant_vllm/backend.py:82-97)."""
from types import SimpleNamespace as NS

import pytest


def _patch(monkeypatch, block=64):
    import inquant_vllm.backend as backend
    monkeypatch.setattr(backend, "get_current_vllm_config", lambda: NS(
        cache_config=NS(block_size=block), model_config=NS(max_model_len=1000)))
    return backend


def test_constructor_mirrors_the_reference_gatekeeping(monkeypatch):
    backend = _patch(monkeypatch)
    impl = backend.InQuantImpl(28, 128, 128 ** -0.5, 4, None, None, "auto")
    assert impl.layout.block_size == 64 and impl.layout.heads == 4 and impl.max_pages == 16
    assert impl.num_queries_per_kv == 7 and impl.request_id is None and impl.tokens == 0 and impl.sealed_pages == 0
    with pytest.raises(ValueError, match="ALiBi/softcap"):
        backend.InQuantImpl(28, 128, 0.1, 4, [1.0], None, "auto")
    with pytest.raises(ValueError, match="ALiBi/softcap"):
        backend.InQuantImpl(28, 128, 0.1, 4, None, (128, 0), "auto")
    with pytest.raises(ValueError, match="ALiBi/softcap"):
        backend.InQuantImpl(28, 128, 0.1, 4, None, None, "auto", logits_soft_cap=30.0)
    with pytest.raises(ValueError, match="KV sharing"):
        backend.InQuantImpl(28, 128, 0.1, 4, None, None, "auto", kv_sharing_target_layer_name="layer.0")
    with pytest.raises(ValueError, match="16 query heads"):
        backend.InQuantImpl(68, 128, 0.1, 4, None, None, "auto")
    with pytest.raises(ValueError):
        backend.InQuantImpl(28, 128, 0.1, 4, None, None, "auto", max_requests=0)


def test_unsupported_page_size_is_rejected_by_the_layout(monkeypatch):
    backend = _patch(monkeypatch, block=48)
    with pytest.raises(ValueError):
        backend.InQuantImpl(28, 128, 0.1, 4, None, None, "auto")


def test_forward_without_an_output_buffer_is_refused(monkeypatch):
    backend = _patch(monkeypatch)
    impl = backend.InQuantImpl(28, 128, 0.1, 4, None, None, "auto")
    with pytest.raises(ValueError, match="output buffer"):
        impl.forward(None, None, None, None, None, None, None)
    meta = backend.InQuantMetadata(1, 2, 1, None, None, "r")
    assert meta.context_len == 1 and backend.InQuantBatchMetadata([meta]).requests[0] is meta
