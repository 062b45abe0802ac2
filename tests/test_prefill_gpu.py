"""Chunked-prefill attention (tcgen05 kernel) against float32 causal attention computed by torch
from the same bf16/fp16 tensors, and against the cache's materialising semantics."""
import numpy as np
import pytest
import torch

from helpers import attention_close, to_numpy

pytestmark = pytest.mark.gpu


def _reference(q, k, v, scale):
    """fp32 causal attention; query i sees keys 0 .. L - Tq + i."""
    q32, k32, v32 = q.float(), k.float(), v.float()
    groups = q.shape[1] // k.shape[1]
    k32 = k32.repeat_interleave(groups, dim=1)
    v32 = v32.repeat_interleave(groups, dim=1)
    tq, tk = q.shape[2], k.shape[2]
    s = torch.einsum("bhqd,bhkd->bhqk", q32, k32) * scale
    pos = torch.arange(tq, device=q.device)[:, None] + (tk - tq)
    s = s.masked_fill(torch.arange(tk, device=q.device)[None, :] > pos, float("-inf"))
    return torch.einsum("bhqk,bhkd->bhqd", torch.softmax(s, dim=-1), v32)


@pytest.mark.parametrize("q_heads,kv_heads,q_tokens,history,dtype", [
    (2, 1, 128, 0, torch.bfloat16),        # one tile, pure causal
    (4, 2, 256, 128, torch.bfloat16),      # full tiles with history
    (7, 1, 200, 77, torch.bfloat16),       # ragged query and history lengths, GQA 7
    (4, 4, 1, 300, torch.bfloat16),        # a single query token
    (8, 2, 384, 1000, torch.float16),      # fp16, several KV tiles
    (28, 4, 512, 2048, torch.bfloat16),    # Qwen2.5-7B head counts; items cut into 2 KV segments
    (28, 4, 2048, 6144, torch.bfloat16),   # config 2's chunk shape: 224 items cut into 3 KV segments each
    (3, 1, 300, 5000, torch.float16),      # few items over a long history: cut into 8 segments
    (28, 4, 4224, 0, torch.bfloat16),      # a long unchunked prompt: many items, no cut, ragged last pair
])
def test_prefill_attention_matches_fp32_causal_attention(q_heads, kv_heads, q_tokens, history, dtype):
    from inquant.prefill import prefill_attention
    gen = torch.Generator(device="cuda").manual_seed(11 + q_tokens + history)
    q = torch.randn((1, q_heads, q_tokens, 128), device="cuda", generator=gen).to(dtype)
    k = torch.randn((1, kv_heads, history + q_tokens, 128), device="cuda", generator=gen).to(dtype)
    v = torch.randn((1, kv_heads, history + q_tokens, 128), device="cuda", generator=gen).to(dtype)
    k[:, :, :, 5] *= 6.0   # an outlier channel sharpens the softmax
    scale = 128 ** -0.5
    out = prefill_attention(q, k, v, scale)
    from inquant import _native
    assert _native.take_status(q.device) == 0
    expected = _reference(q, k, v, scale)
    attention_close(to_numpy(out.float())[0], to_numpy(expected)[0])


def test_prefill_attention_accepts_strided_views_and_rejects_bad_arguments():
    from inquant.prefill import prefill_attention
    gen = torch.Generator(device="cuda").manual_seed(3)
    # [1, T, H, D] projections viewed as [1, H, T, D], as a model produces them
    q = torch.randn((1, 160, 4, 128), device="cuda", generator=gen).bfloat16().transpose(1, 2)
    k = torch.randn((1, 400, 2, 128), device="cuda", generator=gen).bfloat16().transpose(1, 2)
    v = torch.randn((1, 400, 2, 128), device="cuda", generator=gen).bfloat16().transpose(1, 2)
    out = prefill_attention(q, k, v, 0.1)
    attention_close(to_numpy(out.float())[0], to_numpy(_reference(q, k, v, 0.1))[0])
    with pytest.raises(ValueError):
        prefill_attention(q, k[:, :, :100], v[:, :, :100])          # fewer keys than queries
    with pytest.raises(NotImplementedError):
        prefill_attention(q.float(), k.float(), v.float())
    with pytest.raises(ValueError):
        prefill_attention(q[:, :3], k, v)                            # 3 query heads over 2 KV heads


def test_prefill_chunks_through_the_cache_match_one_shot_attention_over_materialised_history():
    """16 chunks... here 3 chunks of 256: every chunk attends to the cache's dequantised history
    plus itself, exactly what `InQuantCache.update` hands to the model's attention."""
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.prefill import prefill_chunk
    gen = torch.Generator(device="cuda").manual_seed(19)
    heads, q_heads, chunk, chunks = 2, 14, 256, 3
    cfg = CacheConfig(CodecConfig(donor_policy="min_error"), block_size=64, residual_length=16, sink_tokens=4,
                      value_bits=2, value_group_size=64)
    cache, shadow = InQuantCache(cfg), InQuantCache(cfg)
    scale = 128 ** -0.5
    for c in range(chunks):
        q = torch.randn((1, q_heads, chunk, 128), device="cuda", generator=gen).bfloat16()
        k = torch.randn((1, heads, chunk, 128), device="cuda", generator=gen).bfloat16()
        v = torch.randn((1, heads, chunk, 128), device="cuda", generator=gen).bfloat16()
        out = prefill_chunk(cache, q, k, v, 0, scale)
        full_k, full_v = shadow.update(k, v, 0)
        assert full_k.shape[2] == (c + 1) * chunk
        attention_close(to_numpy(out.float())[0], to_numpy(_reference(q, full_k, full_v, scale))[0])
    for a, b in zip(cache.materialize(0), shadow.materialize(0)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("value_bits,chunk_sizes", [(2, (256, 256, 256, 100, 37)), (None, (300, 212)), (4, (64, 1, 500))])
def test_prefill_history_holds_exactly_what_update_would_return(value_bits, chunk_sizes):
    """The dense history kept across chunks is bit-identical to the tensors `InQuantCache.update`
    rebuilds per chunk, so the two forms of `prefill_chunk` give the same attention, and both caches
    end up with the same contents."""
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.prefill import PrefillHistory, prefill_chunk
    gen = torch.Generator(device="cuda").manual_seed(23)
    heads, q_heads = 2, 14
    cfg = CacheConfig(CodecConfig(donor_policy="min_error"), block_size=64, residual_length=16, sink_tokens=4,
                      value_bits=value_bits, value_group_size=64)
    cache, shadow, plain = InQuantCache(cfg), InQuantCache(cfg), InQuantCache(cfg)
    history = PrefillHistory(cache, capacity_tokens=128, persistent=True)      # forces the tensors to grow
    scale, seen = 128 ** -0.5, 0
    for tokens in chunk_sizes:
        q = torch.randn((1, q_heads, tokens, 128), device="cuda", generator=gen).bfloat16()
        k = torch.randn((1, heads, tokens, 128), device="cuda", generator=gen).bfloat16()
        v = torch.randn((1, heads, tokens, 128), device="cuda", generator=gen).bfloat16()
        out = prefill_chunk(cache, q, k, v, 0, scale, history=history)
        full_k, full_v = shadow.update(k, v, 0)
        seen += tokens
        key, value = history._layers[0][0], history._layers[0][1]
        assert history._layers[0][2] == seen == cache.get_seq_length(0)
        assert torch.equal(out, prefill_chunk(plain, q, k, v, 0, scale))
        attention_close(to_numpy(out.float())[0], to_numpy(_reference(q, full_k, full_v, scale))[0])
        # after sealing, the history equals what the NEXT update would put before its new states
        next_k, next_v = shadow.materialize(0)
        assert torch.equal(key[:, :, :seen], next_k) and torch.equal(value[:, :, :seen], next_v)
    for a, b in zip(cache.materialize(0), shadow.materialize(0)):
        assert torch.equal(a, b)
    assert history.nbytes > 0
    # a history first used on a filled layer takes the dense state over from the cache
    late = PrefillHistory(plain, persistent=True)
    q = torch.randn((1, q_heads, 50, 128), device="cuda", generator=gen).bfloat16()
    k = torch.randn((1, heads, 50, 128), device="cuda", generator=gen).bfloat16()
    assert torch.equal(prefill_chunk(plain, q, k, k, 0, scale, history=late), prefill_chunk(cache, q, k, k, 0, scale, history=history))
    seen += 50
    # an update behind the history's back is detected
    k = torch.randn((1, heads, 8, 128), device="cuda", generator=gen).bfloat16()
    cache.update(k, k, 0)
    with pytest.raises(RuntimeError, match="state mismatch"):
        prefill_chunk(cache, torch.zeros((1, q_heads, 8, 128), device="cuda", dtype=torch.bfloat16), k, k, 0, scale, history=history)
    with pytest.raises(ValueError, match="another cache"):
        prefill_chunk(plain, torch.zeros((1, q_heads, 8, 128), device="cuda", dtype=torch.bfloat16), k, k, 0, scale, history=history)
    history.release()
    assert history.nbytes == 0


def test_prefill_history_reports_non_finite_input_at_check_or_at_once():
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.prefill import PrefillHistory, prefill_chunk
    cfg = CacheConfig(CodecConfig(donor_policy="min_error"), block_size=64, residual_length=16, sink_tokens=4, value_bits=2)
    q = torch.zeros((1, 4, 200, 128), device="cuda", dtype=torch.bfloat16)
    k = torch.randn((1, 2, 200, 128), device="cuda").bfloat16()
    bad = k.clone()
    bad[0, 1, 30, 7] = float("inf")
    cache = InQuantCache(cfg)
    history = PrefillHistory(cache)
    prefill_chunk(cache, q, k, k, 0, history=history)
    history.check()                                  # nothing to report
    prefill_chunk(cache, q, bad, k, 0, history=history)   # deferred: no exception here
    with pytest.raises(ValueError, match="finite"):
        history.check()
    history.check()                                  # the report clears the word
    strict = InQuantCache(cfg)
    with pytest.raises(ValueError, match="finite"):
        prefill_chunk(strict, q, bad, k, 0, history=PrefillHistory(strict, defer_checks=False))


def test_prefill_history_without_a_dense_copy_rebuilds_from_the_packed_cache():
    """The default history keeps no per-layer dense tensors: every chunk's history comes out of the
    packed cache into one scratch pair shared by the layers.  Outputs and cache contents equal the
    materialising form chunk by chunk, for two layers that alternate."""
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.prefill import PrefillHistory, prefill_chunk
    gen = torch.Generator(device="cuda").manual_seed(29)
    heads, q_heads = 2, 14
    cfg = CacheConfig(CodecConfig(donor_policy="min_error"), block_size=64, residual_length=16, sink_tokens=4, value_bits=2)
    cache, plain = InQuantCache(cfg), InQuantCache(cfg)
    history = PrefillHistory(cache, capacity_tokens=64)
    assert not history.persistent
    scale = 128 ** -0.5
    for tokens in (3, 200, 130, 70):
        for layer in (0, 1):
            q = torch.randn((1, q_heads, tokens, 128), device="cuda", generator=gen).bfloat16()
            k = torch.randn((1, heads, tokens, 128), device="cuda", generator=gen).bfloat16()
            v = torch.randn((1, heads, tokens, 128), device="cuda", generator=gen).bfloat16()
            out = prefill_chunk(cache, q, k, v, layer, scale, history=history)
            assert torch.equal(out, prefill_chunk(plain, q, k, v, layer, scale))
    history.check()
    for layer in (0, 1):
        for a, b in zip(cache.materialize(layer), plain.materialize(layer)):
            assert torch.equal(a, b)
    assert not history._layers
    assert 0 < history.nbytes <= 2 * heads * 1024 * 128 * 2     # one pair for both layers, grown geometrically
    history.release()
    assert history.nbytes == 0
