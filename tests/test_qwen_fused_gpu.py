"""End-to-end drop-in check: a randomly initialised Qwen2 / Mistral model decodes through the
patched attention (packed decode kernel) and is compared with the same model running the
library's cache through its stock forward, which materialises the history and calls SDPA
(the pattern of the reference's tests/test_qwen_fused.py:113-140)."""
import copy
from unittest.mock import patch

import pytest
import torch

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def _model(model_type="qwen2", layers=2, heads=4, kv_heads=2):
    if model_type == "qwen2":
        from transformers import Qwen2Config as Config, Qwen2ForCausalLM as Model
        extra = {}
    else:
        from transformers import MistralConfig as Config, MistralForCausalLM as Model
        extra = {"sliding_window": None}
    config = Config(
        vocab_size=97, hidden_size=heads * 128, intermediate_size=2 * heads * 128, head_dim=128,
        num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv_heads,
        max_position_embeddings=65536, bos_token_id=1, eos_token_id=96, pad_token_id=0,
        attn_implementation="sdpa", **extra)
    return Model(config).eval().to(device="cuda", dtype=torch.bfloat16)


# Logits of these tiny models are of order one, where one bf16 step is 2^-7 = 0.0078: with one
# layer both paths see identical cache contents and differ by at most two such steps.  With two
# layers the second layer's K/V inherit that difference, so once a block seals the two caches
# may hold different codes; the longer case therefore only bounds the drift.
@pytest.mark.parametrize("model_type,layers,prefill_tokens,heads,kv_heads,steps,atol,value_bits,block", [
    ("qwen2", 1, 3, 4, 2, 40, .016, 2, 32), ("qwen2", 1, 98, 4, 2, 40, .016, 2, 32), ("qwen2", 1, 300, 14, 2, 7, .016, 2, 32),
    ("mistral", 1, 98, 8, 2, 7, .016, 2, 32), ("qwen2", 2, 98, 4, 2, 40, .04, 2, 32),
    # the reference's default cache stores values as InQuant packed tensors too: the general kernel with
    # 32-token blocks, the one-launch kernel with blocks of whole slices (at least two)
    ("qwen2", 1, 98, 4, 2, 40, .016, None, 32), ("qwen2", 1, 98, 4, 2, 7, .016, 4, 32),
    ("qwen2", 1, 200, 4, 2, 70, .016, None, 64), ("qwen2", 1, 200, 4, 2, 70, .016, 4, 64), ("mistral", 1, 200, 8, 2, 70, .016, 2, 64)])
def test_fused_decode_matches_materialising_forward(model_type, layers, prefill_tokens, heads, kv_heads, steps, atol, value_bits, block):
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.qwen_fused import enable_fused_attention
    torch.manual_seed(37)
    model = _model(model_type, layers=layers, heads=heads, kv_heads=kv_heads)
    twin = copy.deepcopy(model)
    config = CacheConfig(CodecConfig(salient_fraction=.125), block_size=block, residual_length=4, sink_tokens=2,
                         value_bits=value_bits)
    with enable_fused_attention(model) as handle, torch.no_grad():
        expected_cache, packed = InQuantCache(config), InQuantCache(config)
        tokens = torch.randint(2, 90, (1, prefill_tokens), device="cuda")
        expected = twin(tokens, past_key_values=expected_cache).logits
        actual = model(tokens, past_key_values=packed).logits
        torch.testing.assert_close(actual, expected, rtol=0, atol=0)
        for step in range(steps):
            token = torch.tensor([[3 + step]], device="cuda")
            expected = twin(token, past_key_values=expected_cache).logits
            with patch.object(packed, "materialize", side_effect=AssertionError("unexpected full materialization")):
                actual = model(token, past_key_values=packed).logits
            torch.testing.assert_close(actual.float(), expected.float(), rtol=.035, atol=atol)
            assert packed.get_seq_length() == expected_cache.get_seq_length()
        assert handle.fused_decode_calls == steps * len(model.model.layers)
        assert handle.cpu_reference_calls == 0
        assert packed.auxiliary_nbytes > 0
        if layers == 1:   # identical inputs reached both caches: identical packed history
            for a, b in zip(packed.materialize(0), expected_cache.materialize(0)):
                assert torch.equal(a, b)


def test_generate_runs_through_the_packed_path():
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.qwen_fused import enable_fused_qwen2
    torch.manual_seed(5)
    model = _model()
    config = CacheConfig(CodecConfig(salient_fraction=.125), block_size=32, residual_length=4, sink_tokens=2, value_bits=2)
    tokens = torch.randint(2, 90, (1, 50), device="cuda")
    with enable_fused_qwen2(model) as handle, torch.no_grad():
        generated = model.generate(tokens, past_key_values=InQuantCache(config), do_sample=False, num_beams=1,
                                   max_new_tokens=5, min_new_tokens=5)
    assert tuple(generated.shape) == (1, 55)
    assert handle.fused_decode_calls + handle.cpu_reference_calls >= 0


@pytest.mark.parametrize("keep_history", [False, True])
def test_chunked_prefill_through_the_tensor_core_kernel_matches_the_stock_forward(keep_history):
    """A 300-token prompt fed as chunks of 100: with fused_prefill the later chunks run this
    library's prefill kernel over the packed history; logits must agree with the stock forward,
    which materialises the same history and calls SDPA with the model's causal mask."""
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.qwen_fused import enable_fused_attention
    torch.manual_seed(41)
    model = _model("qwen2", layers=1, heads=14, kv_heads=2)
    twin = copy.deepcopy(model)
    config = CacheConfig(CodecConfig(salient_fraction=.125), block_size=32, residual_length=4, sink_tokens=2, value_bits=2)
    tokens = torch.randint(2, 90, (1, 300), device="cuda")
    with enable_fused_attention(model, fused_prefill=True) as handle, torch.no_grad():
        expected_cache, packed = InQuantCache(config), InQuantCache(config)
        if keep_history:   # the dense history is kept across chunks instead of rebuilt per chunk
            from inquant.prefill import PrefillHistory
            packed._prefill_history = PrefillHistory(packed, persistent=True)
        for start in range(0, 300, 100):
            chunk = tokens[:, start:start + 100]
            expected = twin(chunk, past_key_values=expected_cache).logits
            actual = model(chunk, past_key_values=packed).logits
            # two attention implementations in bf16: up to three bf16 steps of order-one logits
            torch.testing.assert_close(actual.float(), expected.float(), rtol=.035, atol=.024)
        assert handle.fused_prefill_calls == 2 and handle.fused_decode_calls == 0
        if keep_history:
            assert packed._prefill_history._layers[0][2] == 300
        token = torch.tensor([[7]], device="cuda")
        torch.testing.assert_close(model(token, past_key_values=packed).logits.float(),
                                   twin(token, past_key_values=expected_cache).logits.float(), rtol=.035, atol=.016)
        assert handle.fused_decode_calls == 1
        for a, b in zip(packed.materialize(0), expected_cache.materialize(0)):
            assert torch.equal(a, b)
