"""Request state machine of the paged serving backend, driven the way the reference's own test
drives it (extensions/vllm/tests/test_backend.py:48-95): vLLM is faked with SimpleNamespace, a
prompt is prefilled, tokens are decoded across a page boundary, requests are reset on reused
pages, and a stale tail is refused.  Expected values come from SDPA over the pages as the
reference's unpack_pages_reference reads them."""
from types import SimpleNamespace as NS

import pytest
import torch

pytestmark = pytest.mark.gpu


def _impl(monkeypatch, direct_write, **kwargs):
    monkeypatch.setenv("INQUANT_DIRECT_WRITE", direct_write)
    monkeypatch.setenv("INQUANT_DONOR_BACKEND", "triton")
    import inquant_vllm.backend as backend
    from inquant.triton_attention import SharedDecodeWorkspace
    monkeypatch.setattr(backend, "WORKSPACE", SharedDecodeWorkspace())
    monkeypatch.setattr(backend, "get_current_vllm_config", lambda: NS(
        cache_config=NS(block_size=64), model_config=NS(max_model_len=512)))
    return backend, backend.InQuantImpl(28, 128, 128 ** -0.5, 4, None, None, "auto", **kwargs)


def _expected_decode(k, v, q, index, layout):
    from inquant_vllm.layout import pack_pages, unpack_pages_reference
    old_pages = index // 64
    kr, vr = k[:index + 1].transpose(0, 1).clone(), v[:index + 1].transpose(0, 1).clone()
    if old_pages:
        kp = kr[:, :old_pages * 64].reshape(4, old_pages, 64, 128).transpose(0, 1)
        vp = vr[:, :old_pages * 64].reshape(4, old_pages, 64, 128).transpose(0, 1)
        kd, vd = unpack_pages_reference(pack_pages(kp, vp, layout), layout)
        kr[:, :old_pages * 64] = kd.transpose(0, 1).reshape(4, -1, 128)
        vr[:, :old_pages * 64] = vd.transpose(0, 1).reshape(4, -1, 128)
        kr[:, :4], vr[:, :4] = k[:4].transpose(0, 1), v[:4].transpose(0, 1)
    return torch.nn.functional.scaled_dot_product_attention(
        q[index:index + 1].transpose(0, 1).unsqueeze(0).float(), kr.unsqueeze(0).float(), vr.unsqueeze(0).float(),
        enable_gqa=True)[0].transpose(0, 1)


@pytest.mark.parametrize("direct_write", ["0", "1"])
def test_prefill_decode_page_boundary_request_reset_and_stale_tail(monkeypatch, direct_write):
    backend, impl = _impl(monkeypatch, direct_write)
    pool = torch.full((12, impl.layout.page_bytes), 255, dtype=torch.uint8, device="cuda")
    blocks = torch.tensor([7, 2, 9, 3, 5, 8, 6, 1], dtype=torch.int32, device="cuda")
    torch.manual_seed(99)
    assert impl.forward(None, torch.zeros(1, 28, 128, device="cuda", dtype=torch.bfloat16), None, None, pool, None,
                        torch.zeros(1, 28, 128, device="cuda", dtype=torch.bfloat16)) is not None   # profiling call
    for request, initial in [("one-token", 1), ("boundary", 63), ("reused-pages", 257)]:
        k, v = torch.randn(2, initial + 3, 4, 128, dtype=torch.bfloat16, device="cuda")
        q = torch.randn(initial + 3, 28, 128, dtype=torch.bfloat16, device="cuda")
        starts = torch.tensor([0, initial], dtype=torch.int32, device="cuda")
        meta = backend.InQuantMetadata(initial, initial, 0, starts, blocks, request)
        actual = impl.forward(None, q[:initial], k[:initial], v[:initial], pool, meta, torch.empty_like(q[:initial]))
        expected = torch.nn.functional.scaled_dot_product_attention(
            q[:initial].transpose(0, 1).unsqueeze(0).float(), k[:initial].transpose(0, 1).unsqueeze(0).float(),
            v[:initial].transpose(0, 1).unsqueeze(0).float(), is_causal=True, enable_gqa=True)[0].transpose(0, 1)
        torch.testing.assert_close(actual.float(), expected, atol=0.02, rtol=0.02)
        assert impl.request_id == request and impl.tokens == initial and impl.sealed_pages == initial // 64
        for step in range(3):
            index = initial + step
            starts = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
            meta = backend.InQuantMetadata(1, index + 1, index, starts, blocks, request)
            actual = impl.forward(None, q[index:index + 1], k[index:index + 1], v[index:index + 1], pool, meta,
                                  torch.empty_like(q[:1]))
            torch.testing.assert_close(actual.float(), _expected_decode(k, v, q, index, impl.layout), atol=0.02, rtol=0.02)
        assert impl.tokens == initial + 3 and impl.sealed_pages == (initial + 3) // 64
    assert impl.prefill_calls == 3 and impl.decode_calls == 9 and len(impl.requests) == 1
    # untouched physical pages keep their fill byte
    assert (pool[torch.tensor([0, 4, 10, 11], device="cuda")] == 255).all()
    meta.request_id = "wrong-request"
    with pytest.raises(RuntimeError, match="state mismatch"):
        impl.forward(None, q[:1], k[:1], v[:1], pool, meta, torch.empty_like(q[:1]))
    meta.request_id, meta.context_len = "reused-pages", 5          # a context that does not continue the state
    with pytest.raises(RuntimeError, match="state mismatch"):
        impl.forward(None, q[:1], k[:1], v[:1], pool, meta, torch.empty_like(q[:1]))
    with pytest.raises(RuntimeError, match="cache spec"):
        impl.forward(None, q[:1], k[:1], v[:1], pool.view(-1, impl.layout.page_bytes // 2), meta, torch.empty_like(q[:1]))
    with pytest.raises(ValueError, match="output buffer"):
        impl.forward(None, q[:1], k[:1], v[:1], pool, meta, None)
    from inquant import _native as N
    assert N.take_status(torch.device("cuda", 0)) == 0


def test_several_active_requests_decode_from_one_batch_metadata(monkeypatch):
    """Three requests with their own block tables stay active together; a decode step lists all of
    them in one InQuantBatchMetadata and each is served from its own exact tail and pages."""
    backend, impl = _impl(monkeypatch, "1", max_requests=3)
    pool = torch.full((24, impl.layout.page_bytes), 255, dtype=torch.uint8, device="cuda")
    tables = {name: torch.tensor(ids, dtype=torch.int32, device="cuda")
              for name, ids in (("a", [3, 17, 8, 1]), ("b", [20, 5, 11, 2]), ("c", [9, 14, 0, 6]))}
    lengths = {"a": 62, "b": 130, "c": 5}
    torch.manual_seed(5)
    data = {}
    for name, n in lengths.items():
        k, v = torch.randn(2, n + 4, 4, 128, dtype=torch.bfloat16, device="cuda")
        q = torch.randn(n + 4, 28, 128, dtype=torch.bfloat16, device="cuda")
        data[name] = (k, v, q)
        starts = torch.tensor([0, n], dtype=torch.int32, device="cuda")
        impl.forward(None, q[:n], k[:n], v[:n], pool, backend.InQuantMetadata(n, n, 0, starts, tables[name], name),
                     torch.empty_like(q[:n]))
    assert set(impl.requests) == {"a", "b", "c"}
    for step in range(4):      # request a crosses its page boundary at step 1
        names = ["c", "a", "b"]
        metas = [backend.InQuantMetadata(1, lengths[n] + step + 1, lengths[n] + step, None, tables[n], n) for n in names]
        rows = lambda i: torch.cat([data[n][i][lengths[n] + step:lengths[n] + step + 1] for n in names], 0)
        out = torch.empty((3, 28, 128), dtype=torch.bfloat16, device="cuda")
        impl.forward(None, rows(2), rows(0), rows(1), pool, backend.InQuantBatchMetadata(metas), out)
        for row, n in enumerate(names):
            k, v, q = data[n]
            torch.testing.assert_close(out[row:row + 1].float(), _expected_decode(k, v, q, lengths[n] + step, impl.layout),
                                       atol=0.02, rtol=0.02)
    assert impl.requests["a"].sealed_pages == 1 and impl.requests["b"].sealed_pages == 2 and impl.requests["c"].sealed_pages == 0
    impl.finish_request("b")
    with pytest.raises(RuntimeError, match="state mismatch"):
        impl.forward(None, data["b"][2][:1], data["b"][0][:1], data["b"][1][:1], pool,
                     backend.InQuantMetadata(1, 135, 134, None, tables["b"], "b"), torch.empty((1, 28, 128), dtype=torch.bfloat16, device="cuda"))
    # a fourth prefill evicts the least recently used request
    k, v, q = data["c"]
    impl.forward(None, q[:5], k[:5], v[:5], pool, backend.InQuantMetadata(5, 5, 0, None, tables["b"], "d"), torch.empty_like(q[:5]))
    impl.forward(None, q[:5], k[:5], v[:5], pool, backend.InQuantMetadata(5, 5, 0, None, tables["b"], "e"), torch.empty_like(q[:5]))
    assert len(impl.requests) == 3 and "d" in impl.requests and "e" in impl.requests
