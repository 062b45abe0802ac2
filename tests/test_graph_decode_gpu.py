"""The whole-model decode step replayed from one CUDA graph must track the ordinary patched
forward token by token, across block seals, and leave the cache in the same state."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")

from test_qwen_fused_gpu import _model  # noqa: E402


def _config():
    from inquant.cache import CacheConfig
    from inquant.codec import CodecConfig
    return CacheConfig(CodecConfig(salient_fraction=.125), block_size=32, residual_length=4, sink_tokens=2, value_bits=2)


@pytest.mark.parametrize("model_type,layers,atol", [("qwen2", 1, .016), ("qwen2", 2, .04), ("mistral", 1, .016)])
def test_graphed_steps_match_eager_steps_across_seals(model_type, layers, atol):
    from inquant import _native as N
    from inquant.cache import InQuantCache
    from inquant.graph_decode import GraphedDecodeStep
    from inquant.qwen_fused import enable_fused_attention
    torch.manual_seed(11)
    model = _model(model_type, layers=layers)
    twin = copy.deepcopy(model)
    prompt = torch.randint(2, 90, (1, 70), device="cuda")
    steps = 90                                   # capacity 36: the tails seal at least twice
    with enable_fused_attention(model) as handle, enable_fused_attention(twin), torch.no_grad():
        eager_cache, graph_cache = InQuantCache(_config()), InQuantCache(_config())
        twin(prompt, past_key_values=eager_cache)
        model(prompt, past_key_values=graph_cache)
        stepper = GraphedDecodeStep(model, graph_cache)
        for step in range(steps):
            token = 3 + step % 80
            expected = twin(torch.tensor([[token]], device="cuda"), past_key_values=eager_cache).logits
            actual = stepper.step(token)
            torch.testing.assert_close(actual.float(), expected.float(), rtol=.035, atol=atol, msg=lambda m: f"step {step}: {m}")
        stepper.close()
        assert stepper.replays + stepper.eager_steps == steps
        assert stepper.eager_steps >= 2 and stepper.captures >= 2 and stepper.replays > stepper.eager_steps
        assert handle.fused_decode_calls == steps * layers
        assert graph_cache.get_seq_length() == eager_cache.get_seq_length() == 70 + steps
        for index in range(layers):
            a, b = graph_cache._layers[index], eager_cache._layers[index]
            assert (a.tail_count, a.seq_length, len(a.key_blocks)) == (b.tail_count, b.seq_length, len(b.key_blocks))
        if layers == 1:   # identical inputs reached both caches: identical contents
            for a, b in zip(graph_cache.materialize(0), eager_cache.materialize(0)):
                assert torch.equal(a, b)
        # the ordinary forward continues on the committed cache
        expected = twin(torch.tensor([[5]], device="cuda"), past_key_values=eager_cache).logits
        actual = model(torch.tensor([[5]], device="cuda"), past_key_values=graph_cache).logits
        torch.testing.assert_close(actual.float(), expected.float(), rtol=.035, atol=atol)
    assert N.take_status(torch.device("cuda", 0)) == 0


def test_device_side_greedy_loop_equals_host_fed_argmax():
    from inquant.cache import InQuantCache
    from inquant.graph_decode import GraphedDecodeStep
    from inquant.qwen_fused import enable_fused_attention
    torch.manual_seed(13)
    model = _model("qwen2", layers=2)
    prompt = torch.randint(2, 90, (1, 50), device="cuda")
    with enable_fused_attention(model), torch.no_grad():
        first, second = InQuantCache(_config()), InQuantCache(_config())
        model(prompt, past_key_values=first)
        model(prompt, past_key_values=second)
        device_loop = GraphedDecodeStep(model, first)
        on_device = device_loop.greedy(7, 45)
        device_loop.close()
        stepper = GraphedDecodeStep(model, second)
        token, fed = 7, []
        for _ in range(45):
            token = int(stepper.step(token)[0, -1].argmax())
            fed.append(token)
        stepper.close()
    assert on_device.tolist() == fed


def test_graphed_decode_rejects_an_unpatched_model_and_an_empty_cache():
    from inquant.cache import InQuantCache
    from inquant.graph_decode import GraphedDecodeStep
    from inquant.qwen_fused import enable_fused_attention
    model = _model("qwen2", layers=1)
    with torch.no_grad():
        with pytest.raises(ValueError, match="enable_fused_attention"):
            GraphedDecodeStep(model, InQuantCache(_config()))
        with enable_fused_attention(model):
            with pytest.raises(ValueError, match="prefill"):
                GraphedDecodeStep(model, InQuantCache(_config()))
