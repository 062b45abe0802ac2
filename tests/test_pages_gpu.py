"""Paged (vLLM-extension) layout: page bytes vs the reference's golden pages and the oracle,
direct sealing into scattered physical pages, paged decode with random page order and reuse.
Mirrors the reference's extensions/vllm/tests/test_pages.py and test_direct_packing.py."""
import numpy as np
import pytest
import torch

import inquant_oracle as oracle
import workloads
from cases import PAGE_CASES
from helpers import assert_same_bytes, attention_close, to_device, to_numpy

pytestmark = pytest.mark.gpu


def _pages_input(seed, heads, pages, block):
    k, v = workloads.make_kv(seed, heads, pages * block)
    shape = (heads, pages, block, 128)
    kt = np.ascontiguousarray(k[0].reshape(shape).transpose(1, 0, 2, 3))
    vt = np.ascontiguousarray(v[0].reshape(shape).transpose(1, 0, 2, 3))
    return kt, vt


@pytest.mark.parametrize("name", sorted(PAGE_CASES))
def test_page_bytes_match_reference_golden(golden, name):
    from inquant_vllm.layout import PageLayout, pack_pages, unpack_pages_reference
    case = PAGE_CASES[name]
    kt, vt = _pages_input(case["seed"], case["heads"], case["pages"], case["block"])
    layout = PageLayout(case["block"], case["heads"])
    pages = pack_pages(to_device(kt), to_device(vt), layout)
    assert pages.numel() == case["pages"] * layout.page_bytes
    assert_same_bytes(pages, golden[f"pages/{name}/bytes"], "page bytes")
    rk, rv = unpack_pages_reference(pages, layout)
    ok, ov = oracle.unpack_pages(golden[f"pages/{name}/bytes"], case["block"], case["heads"])
    assert_same_bytes(rk.float(), ok, "unpacked keys")
    assert_same_bytes(rv.float(), ov, "unpacked values")


@pytest.mark.parametrize("block", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("heads", [2, 8])
def test_page_layout_matches_codecs_and_oracle(block, heads):
    from inquant.codec import CodecConfig, quantize
    from inquant.value_codec import quantize_values
    from inquant_vllm.layout import PageLayout, pack_pages, unpack_pages_reference
    kt, vt = _pages_input(7 + block, heads, 3, block)
    layout = PageLayout(block, heads)
    assert layout.page_bytes == heads * (104 * block + 832)
    k, v = to_device(kt), to_device(vt)
    pages = pack_pages(k, v, layout)
    assert_same_bytes(pages, oracle.pack_pages(kt, vt, block, heads), "pages")
    rk, rv = unpack_pages_reference(pages, layout)
    assert torch.equal(rk, quantize(k, CodecConfig(donor_policy="min_error")).dequantize())
    assert torch.equal(rv, quantize_values(v).dequantize())
    if block >= 64:
        assert layout.page_bytes < block * 2 * 128 * heads * 2 * 0.8


@pytest.mark.parametrize("block", [64, 128, 256])
@pytest.mark.parametrize("heads", [4, 8])
@pytest.mark.parametrize("id_dtype", [torch.int32, torch.int64])
def test_direct_scattered_pages_match_staged_and_leave_other_pages_intact(block, heads, id_dtype):
    from inquant.codec import CodecConfig, quantize
    from inquant.value_codec import quantize_values
    from inquant_vllm.layout import PageLayout, pack_pages, pack_pages_into
    from inquant_vllm.packing import write_codec_pages
    layout = PageLayout(block, heads)
    pool = torch.full((7, layout.page_bytes), 173, device='cuda', dtype=torch.uint8)
    ids = torch.tensor([5, 0, 3], device='cuda', dtype=id_dtype)
    for round_ in range(2):
        kt, vt = _pages_input(915 + round_, heads, 3, block)
        k, v = to_device(kt), to_device(vt)
        reference = pack_pages(k, v, layout)
        pack_pages_into(k, v, layout, pool, ids, donor_backend="triton")
        assert torch.equal(pool[ids.long()], reference)
        assert (pool[torch.tensor([1, 2, 4, 6], device='cuda')] == 173).all()
        staged = torch.full_like(pool, 173)
        write_codec_pages(quantize(k, CodecConfig(donor_policy="min_error")), quantize_values(v), layout, staged, ids)
        assert torch.equal(staged, pool)
    # token-major source [tokens, heads, 128] viewed as pages, as the serving backend passes it
    kt, vt = _pages_input(3, heads, 3, block)
    k_tm = to_device(kt).permute(0, 2, 1, 3).contiguous().view(3 * block, heads, 128)
    keys = k_tm.view(3, block, heads, 128).transpose(1, 2)
    assert not keys.is_contiguous()
    a = torch.zeros_like(pool)
    b = torch.zeros_like(pool)
    pack_pages_into(keys, to_device(vt), layout, a, ids)
    pack_pages_into(keys.contiguous(), to_device(vt), layout, b, ids)
    assert torch.equal(a, b)


@pytest.mark.parametrize("block,pages,tail", [(64, 0, 1), (64, 0, 63), (64, 1, 0), (64, 1, 64), (128, 3, 17),
                                               (256, 128, 128), (16, 5, 7), (32, 9, 31)])
def test_paged_decode_random_page_order_and_reuse(block, pages, tail):
    from inquant.triton_attention import SharedDecodeWorkspace
    from inquant_vllm.kernels import paged_decode
    from inquant_vllm.layout import PageLayout, pack_pages
    h, hq = 4, 28
    layout = PageLayout(block, h)
    gen = torch.Generator().manual_seed(71)
    pool = torch.full((pages + 7, layout.page_bytes), 255, dtype=torch.uint8, device='cuda')
    ids = torch.randperm(pages + 7, generator=gen)[:pages].to(torch.int32).cuda()
    dense = torch.full((2, h, block + 4, 128), float('nan'), dtype=torch.bfloat16, device='cuda')
    workspace = SharedDecodeWorkspace()
    for reuse in range(2):
        total = pages * block + tail
        k32, v32 = workloads.make_kv(71 + reuse, h, total)
        k32, v32 = k32[0], v32[0]
        sink = min(4, total)
        k, v = to_device(k32), to_device(v32)
        dense[0, :, :sink], dense[1, :, :sink] = k[:, :sink], v[:, :sink]
        if tail:
            dense[0, :, 4:4 + tail], dense[1, :, 4:4 + tail] = k[:, total - tail:], v[:, total - tail:]
        if pages:
            kt = np.ascontiguousarray(k32[:, :pages * block].reshape(h, pages, block, 128).transpose(1, 0, 2, 3))
            vt = np.ascontiguousarray(v32[:, :pages * block].reshape(h, pages, block, 128).transpose(1, 0, 2, 3))
            pool.index_copy_(0, ids.long(), pack_pages(to_device(kt), to_device(vt), layout))
            kr, vr = oracle.unpack_pages(oracle.pack_pages(kt, vt, block, h), block, h)
            kr = kr.transpose(1, 0, 2, 3).reshape(h, -1, 128).copy()
            vr = vr.transpose(1, 0, 2, 3).reshape(h, -1, 128).copy()
            kr[:, :sink], vr[:, :sink] = k32[:, :sink], v32[:, :sink]   # the exact sink replaces the packed copy
            kr = np.concatenate((kr, k32[:, pages * block:]), 1)
            vr = np.concatenate((vr, v32[:, pages * block:]), 1)
        else:
            kr, vr = k32, v32
        q32 = workloads.make_query(5 + reuse, hq)
        actual = paged_decode(to_device(q32).view(1, hq, 128), pool, ids, dense, pages, tail, sink, layout, workspace, 128 ** -0.5)
        expected = oracle.attention_decode(q32, kr, vr, 128 ** -0.5)
        attention_close(to_numpy(actual.float()).reshape(hq, 128), expected)


def test_paged_decode_argument_validation():
    from inquant.triton_attention import SharedDecodeWorkspace
    from inquant_vllm.kernels import paged_decode
    from inquant_vllm.layout import PageLayout
    layout = PageLayout(64, 4)
    pool = torch.zeros((2, layout.page_bytes), dtype=torch.uint8, device="cuda")
    dense = torch.zeros((2, 4, 68, 128), dtype=torch.bfloat16, device="cuda")
    ids = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="BF16"):
        paged_decode(torch.zeros(1, 28, 128, device="cuda"), pool, ids, dense, 0, 1, 1, layout, SharedDecodeWorkspace(), 0.1)
    with pytest.raises(ValueError, match="query heads per KV head"):
        paged_decode(torch.zeros(1, 30, 128, device="cuda", dtype=torch.bfloat16), pool, ids, dense, 0, 1, 1, layout,
                     SharedDecodeWorkspace(), 0.1)
    with pytest.raises(ValueError):
        PageLayout(48, 4)


def test_out_of_range_page_ids_are_skipped_and_reported():
    """A physical page id beyond the pool is never used as an address: the encoders leave that
    page unwritten (every other page is sealed, the pool's remaining pages keep their fill byte)
    and the call reports it; the decode kernel reads its first page instead and sets the status bit."""
    from inquant import _native as N
    from inquant.triton_attention import SharedDecodeWorkspace
    from inquant_vllm.kernels import paged_decode
    from inquant_vllm.layout import PageLayout, pack_pages, pack_pages_into
    block, heads = 64, 4
    layout = PageLayout(block, heads)
    kt, vt = _pages_input(41, heads, 3, block)
    k, v = to_device(kt), to_device(vt)
    reference = pack_pages(k, v, layout)
    for bad in (7, -1, 1 << 20):
        pool = torch.full((7, layout.page_bytes), 173, device="cuda", dtype=torch.uint8)
        ids = torch.tensor([5, bad, 3], device="cuda", dtype=torch.int64)
        with pytest.raises(IndexError, match="outside the page pool"):
            pack_pages_into(k, v, layout, pool, ids)
        assert torch.equal(pool[5], reference[0]) and torch.equal(pool[3], reference[2])
        assert (pool[torch.tensor([0, 1, 2, 4, 6], device="cuda")] == 173).all()
    assert N.take_status(torch.device("cuda", 0)) == 0
    # decode: a table entry beyond the pool
    pool = torch.zeros((4, layout.page_bytes), device="cuda", dtype=torch.uint8)
    pool[:3] = reference
    dense = torch.zeros((2, heads, block + 4, 128), dtype=torch.bfloat16, device="cuda")
    q = to_device(workloads.make_query(3, 28)).view(1, 28, 128)
    table = torch.tensor([0, 9, 2], device="cuda", dtype=torch.int32)
    out = paged_decode(q, pool, table, dense, 3, 1, 4, layout, SharedDecodeWorkspace(), 128 ** -0.5)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert N.take_status(torch.device("cuda", 0), N.STATUS_BAD_INDEX) == N.STATUS_BAD_INDEX
    assert N.take_status(torch.device("cuda", 0)) == 0
