"""Patch/restore semantics of the fused-attention adapter that need no GPU
(mirrors the CPU part of the reference's tests/test_qwen_fused.py)."""
import copy

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _model(head_dim=128, layers=1, model_type="qwen2"):
    if model_type == "qwen2":
        from transformers import Qwen2Config as Config, Qwen2ForCausalLM as Model
    else:
        from transformers import MistralConfig as Config, MistralForCausalLM as Model
    config = Config(
        vocab_size=97, hidden_size=4 * head_dim, intermediate_size=8 * head_dim,
        num_hidden_layers=layers, num_attention_heads=4, num_key_value_heads=2,
        max_position_embeddings=65536, bos_token_id=1, eos_token_id=96, pad_token_id=0,
        attn_implementation="sdpa", **({"sliding_window": None} if model_type == "mistral" else {}))
    return Model(config).eval()


def test_patch_is_instance_local_and_restore_is_idempotent():
    from inquant.qwen_fused import enable_fused_qwen2
    torch.manual_seed(31)
    model = _model()
    twin = copy.deepcopy(model)
    original = model.model.layers[0].self_attn.forward
    handle = enable_fused_qwen2(model)
    assert not hasattr(twin.model.layers[0].self_attn, "_inquant_original_forward")
    with pytest.raises(ValueError):
        enable_fused_qwen2(model)
    # anything that is not a packed decode step goes to the original forward
    tokens = torch.randint(2, 90, (1, 9))
    with torch.no_grad():
        torch.testing.assert_close(model(tokens).logits, twin(tokens).logits, rtol=0, atol=0)
    assert handle.fused_decode_calls == 0 and handle.cpu_reference_calls == 0
    handle.restore()
    handle.restore()
    assert model.model.layers[0].self_attn.forward == original


def test_context_manager_restores():
    from inquant.qwen_fused import enable_fused_attention
    model = _model()
    original = model.model.layers[0].self_attn.forward
    with enable_fused_attention(model) as handle:
        assert model.model.layers[0].self_attn.forward != original
        assert not handle.restored
    assert handle.restored and model.model.layers[0].self_attn.forward == original


def test_rejections():
    from inquant.qwen_fused import enable_fused_attention, enable_fused_mistral, enable_fused_qwen2
    with pytest.raises(ValueError, match="head_dim=128"):
        enable_fused_qwen2(_model(head_dim=8))
    with pytest.raises(ValueError, match="Mistral"):
        enable_fused_mistral(_model())
    with pytest.raises(ValueError, match="Qwen2"):
        enable_fused_qwen2(_model(model_type="mistral"))
    training = _model()
    training.train()
    with pytest.raises(ValueError, match="eval"):
        enable_fused_attention(training)
    with enable_fused_mistral(_model(model_type="mistral")) as handle:
        assert len(handle.originals) == 1
