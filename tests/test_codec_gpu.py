"""CUDA key/value codec vs the CPU oracle and the reference's golden vectors, bit for bit.
Mirrors the reference's tests/test_codec.py, test_value_codec.py and test_triton_selection.py."""
import math

import numpy as np
import pytest
import torch

import inquant_oracle as oracle
from cases import K4_CASES, SELECT_CASES, V_CASES, k4_input, select_input
from helpers import TORCH_DTYPE, assert_same_bytes, to_device, to_numpy

pytestmark = pytest.mark.gpu


def _codec():
    from inquant.codec import CodecConfig, quantize, _reuse_map
    return CodecConfig, quantize, _reuse_map


@pytest.mark.parametrize("name", sorted(K4_CASES))
def test_k4_matches_reference_golden(golden, name):
    CodecConfig, quantize, _ = _codec()
    case = K4_CASES[name]
    x = to_device(k4_input(case), case["dtype"])
    packed = quantize(x, CodecConfig(sample_stride=case["stride"], salient_fraction=case["fraction"],
                                     donor_policy=case["policy"]))
    for field, tensor in packed.tensors.items():
        assert_same_bytes(tensor, golden[f"k4/{name}/{field}"], f"{name}/{field}")
    ref = oracle.quantize_k4(k4_input(case), case["dtype"], case["stride"], case["fraction"], case["policy"])
    assert_same_bytes(packed.dequantize().float(), oracle.dequantize_k4(ref), f"{name}/dequantize")
    assert packed.dequantize(torch.float32).dtype == torch.float32


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("shape", [(5, 4, 256, 128), (3, 2, 128, 128), (2, 4, 64, 128), (7, 2, 16, 128),
                                   (2, 1, 41, 128), (2, 2, 300, 128), (1, 2, 33, 64), (2, 3, 24, 16)])
@pytest.mark.parametrize("policy", ["neighbors", "min_error"])
def test_k4_matches_oracle_on_seeded_inputs(dtype, shape, policy):
    CodecConfig, quantize, _ = _codec()
    for fraction in (0.0, 0.125, 0.5):
        case = dict(seed=hash((shape, fraction)) % 1000, shape=shape, dtype=dtype, zero_row=True)
        x32 = k4_input(case)
        packed = quantize(to_device(x32, dtype), CodecConfig(salient_fraction=fraction, donor_policy=policy))
        ref = oracle.quantize_k4(x32, dtype, 8, fraction, policy)
        for field, tensor in packed.tensors.items():
            assert_same_bytes(tensor, ref.fields()[field], f"{field} f={fraction}")
        assert_same_bytes(packed.dequantize().float(), oracle.dequantize_k4(ref), "dequantize")


@pytest.mark.parametrize("tokens", [32, 64, 96, 256, 512])
@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_k4_ring_staged_rows_match_strided_rows_and_oracle(tokens, dtype):
    """Contiguous 16-bit rows in groups of 32 tokens take the shared-memory ring kernel, a
    token-major view of the same values (token stride = heads x channels) the direct-load one:
    both must give the oracle's bytes (1, 2, 3, 8 and 16 groups: shorter than, equal to and longer
    than the ring)."""
    CodecConfig, quantize, _ = _codec()
    cfg = CodecConfig(donor_policy="min_error")
    x32 = k4_input(dict(seed=40 + tokens, shape=(3, 4, tokens, 128), dtype=dtype))
    x = to_device(x32, dtype)
    token_major = x.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    assert x.is_contiguous() and not token_major.is_contiguous() and token_major.stride(2) == 4 * 128
    staged, direct = quantize(x, cfg), quantize(token_major, cfg)
    ref = oracle.quantize_k4(x32, dtype, 8, 0.125, "min_error")
    for name in staged.tensors:
        assert torch.equal(staged.tensors[name], direct.tensors[name]), name
        assert_same_bytes(staged.tensors[name], ref.fields()[name], name)


def test_block_axis_in_batch_and_token_major_strides_match_contiguous():
    CodecConfig, quantize, _ = _codec()
    cfg = CodecConfig(donor_policy="min_error")
    x32 = k4_input(dict(seed=3, shape=(1, 4, 3 * 64 + 5, 128), dtype="bfloat16"))
    x = to_device(x32)
    blocked = x[0, :, 2:2 + 3 * 64].reshape(4, 3, 64, 128).permute(1, 0, 2, 3)
    assert not blocked.is_contiguous()
    a, b = quantize(blocked, cfg), quantize(blocked.contiguous(), cfg)
    for name in a.tensors:
        assert torch.equal(a.tensors[name], b.tensors[name]), name
    ref = oracle.quantize_k4(np.ascontiguousarray(x32[0, :, 2:2 + 192].reshape(4, 3, 64, 128).transpose(1, 0, 2, 3)),
                             donor_policy="min_error")
    for field, tensor in a.tensors.items():
        assert_same_bytes(tensor, ref.fields()[field], field)
    token_major = x[0].transpose(0, 1).contiguous().transpose(0, 1).unsqueeze(0)  # [1,H,T,C], token stride H*C
    assert token_major.stride(2) == 4 * 128
    c = quantize(token_major[:, :, 2:66], cfg)
    d = quantize(x[:, :, 2:66].contiguous(), cfg)
    for name in c.tensors:
        assert torch.equal(c.tensors[name], d.tensors[name]), name
    # channel-strided input is made contiguous first
    e = quantize(x[:, :, :64].transpose(2, 3).contiguous().transpose(2, 3), cfg)
    f = quantize(x[:, :, :64], cfg)
    assert torch.equal(e.payload, f.payload)


def test_payload_shapes_and_byte_accounting():
    CodecConfig, quantize, _ = _codec()
    rng = np.random.default_rng(29)
    x32 = rng.standard_normal((2, 3, 41, 16), dtype=np.float32) * 0.1
    x32[..., 6:10] *= 100
    x = to_device(x32.astype(np.float16).astype(np.float32), "float16")
    packed = quantize(x, CodecConfig(salient_fraction=0.25))
    assert packed.payload.shape == (2, 3, 41, 8) and packed.payload.dtype == torch.uint8
    assert packed.payload_nbytes == math.prod(x.shape) // 2
    assert set(packed.tensors) == {"payload", "scales", "salient_channels", "donor_channels", "padding"}
    assert all(t.device == x.device and t.is_contiguous() for t in packed.tensors.values())
    expected_metadata = 2 * 3 * (16 * 4 + 4 * (1 + 1 + 4))
    assert packed.metadata_nbytes == expected_metadata
    assert packed.nbytes == packed.payload_nbytes + expected_metadata
    assert packed.storage_stats()["source_nbytes"] == x.numel() * x.element_size()
    assert packed.storage_stats()["compression_ratio"] < 4
    sources, donors = packed.salient_channels.long(), packed.donor_channels.long()
    assert torch.equal(sources, torch.tensor([6, 7, 8, 9], device="cuda").expand_as(sources))
    assert torch.all(torch.sort(donors, dim=-1).values.diff(dim=-1) > 0)
    assert torch.all(donors[..., 0] == 5)


@pytest.mark.parametrize("fraction", [0.0, 0.125, 0.5])
def test_all_zero_is_finite_and_exact(fraction):
    CodecConfig, quantize, _ = _codec()
    x = torch.zeros(1, 2, 17, 16, dtype=torch.bfloat16, device="cuda")
    restored = quantize(x, CodecConfig(salient_fraction=fraction)).dequantize()
    assert restored.dtype == x.dtype and torch.count_nonzero(restored) == 0


def test_every_int4_code_roundtrips_and_sampling_positions():
    CodecConfig, quantize, _ = _codec()
    x = torch.arange(-7, 8, dtype=torch.float32, device="cuda").view(1, 1, 15, 1).expand(1, 1, 15, 16)
    packed = quantize(x, CodecConfig(salient_fraction=0))
    assert torch.equal(packed.dequantize(), x)
    assert packed.salient_channels.numel() == packed.donor_channels.numel() == packed.padding.numel() == 0
    y = torch.ones(1, 1, 16, 8, device="cuda")
    y[..., 1::2, 0] = 1000
    y[..., ::8, 6] = 10
    assert quantize(y, CodecConfig(sample_stride=8, salient_fraction=0.125)).salient_channels.tolist() == [[[6]]]


@pytest.mark.parametrize("channels", [2, 128, 258])
def test_half_salient_fraction_always_has_enough_donors(channels):
    CodecConfig, quantize, _ = _codec()
    x32 = np.random.default_rng(channels).standard_normal((1, 1, 3, channels), dtype=np.float32)
    packed = quantize(to_device(x32, "float32"), CodecConfig(salient_fraction=0.5))
    assert packed.donor_channels.unique().numel() == channels // 2
    assert torch.isfinite(packed.dequantize()).all()
    ref = oracle.quantize_k4(x32, "float32", 8, 0.5)
    assert_same_bytes(packed.salient_channels, ref.salient_channels, "sources")
    assert_same_bytes(packed.donor_channels, ref.donor_channels, "donors")
    assert_same_bytes(packed.payload, ref.payload, "payload")
    if channels > 256:
        assert packed.donor_channels.dtype == torch.int32


def test_argument_validation_matches_reference_messages():
    CodecConfig, quantize, _ = _codec()
    for bad in (-0.1, 0.51, float("nan")):
        with pytest.raises(ValueError, match="salient_fraction"):
            CodecConfig(salient_fraction=bad)
    for bad in (0, -1, 1.5, True):
        with pytest.raises(ValueError, match="sample_stride"):
            CodecConfig(sample_stride=bad)
    with pytest.raises(ValueError, match="even"):
        quantize(torch.ones(1, 1, 8, 7, device="cuda"))
    with pytest.raises(ValueError, match="nonempty"):
        quantize(torch.ones(1, 1, 0, 8, device="cuda"))
    with pytest.raises(ValueError, match="floating"):
        quantize(torch.ones(1, 1, 8, 8, dtype=torch.int32, device="cuda"))
    for bad in (float("nan"), float("inf")):
        with pytest.raises(ValueError, match="finite"):
            quantize(torch.full((1, 1, 8, 8), bad, device="cuda"))
    # the status word is cleared after a failure: the next call succeeds
    quantize(torch.ones(1, 1, 8, 8, device="cuda"))
    with pytest.raises(RuntimeError, match="CUDA"):
        quantize(torch.ones(1, 1, 8, 8))


def test_min_error_donor_avoids_destroying_a_varying_neighbor():
    CodecConfig, quantize, _ = _codec()
    w = np.random.default_rng(119).standard_normal((1, 2, 128, 8), dtype=np.float32)
    w[..., 0] = 100
    w[..., 1] *= 10
    w[..., 7] = 2
    x = to_device(w, "float32")
    local = quantize(x, CodecConfig(salient_fraction=0.125))
    selected = quantize(x, CodecConfig(salient_fraction=0.125, donor_policy="min_error"))
    assert torch.all(local.donor_channels == 1) and torch.all(selected.donor_channels == 7)
    assert torch.equal(selected.salient_channels, local.salient_channels)
    assert ((selected.dequantize() - x) ** 2).mean() < ((local.dequantize() - x) ** 2).mean()


@pytest.mark.parametrize("name", sorted(SELECT_CASES))
def test_selector_matches_reference_with_ties_and_adjacent_outliers(golden, name):
    from inquant.triton_selection import reuse_map
    _, _, _reuse_map = _codec()
    case = SELECT_CASES[name]
    score, error = select_input(case)
    s = torch.from_numpy(score).cuda()
    e = None if error is None else torch.from_numpy(error).cuda()
    for fn in (reuse_map, _reuse_map):
        sources, donors = fn(s, case["count"], e)
        assert sources.dtype == torch.int64
        assert_same_bytes(sources, golden[f"select/{name}/sources"], "sources")
        assert_same_bytes(donors, golden[f"select/{name}/donors"], "donors")


def test_selector_fuzz_against_oracle():
    _, _, _reuse_map = _codec()
    rng = np.random.default_rng(5)
    for channels, count in ((128, 16), (128, 64), (64, 8), (258, 129), (16, 4), (8, 1), (1024, 100)):
        score = rng.random((6, channels), dtype=np.float32)
        score[0] = 0
        score[1, channels // 4: channels // 2] = 3
        score[2, -1] = 9
        quant = np.floor(score * 8) / 8  # many ties
        for sal in (score, quant.astype(np.float32)):
            for error in (None, rng.integers(0, 5, size=sal.shape).astype(np.float32)):
                want = oracle.reuse_map(sal, count, error)
                got = _reuse_map(torch.from_numpy(sal).cuda(), count, None if error is None else torch.from_numpy(error).cuda())
                assert_same_bytes(got[0], want[0], f"sources C={channels}")
                assert_same_bytes(got[1], want[1], f"donors C={channels}")


@pytest.mark.parametrize("name", sorted(V_CASES))
def test_values_match_reference_golden(golden, name):
    from inquant.value_codec import quantize_values
    case = V_CASES[name]
    x32 = k4_input(case)
    packed = quantize_values(to_device(x32, case["dtype"]), case["bits"], case["group"])
    for field, tensor in packed.tensors.items():
        assert_same_bytes(tensor, golden[f"v/{name}/{field}"], f"{name}/{field}")
    ref = oracle.quantize_values(x32, case["dtype"], case["bits"], case["group"])
    assert_same_bytes(packed.dequantize().float(), oracle.dequantize_values(ref), "dequantize")


@pytest.mark.parametrize("bits,group", [(2, 32), (2, 64), (2, 128), (4, 32), (4, 64), (4, 128)])
@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
def test_values_match_oracle(bits, group, dtype):
    from inquant.value_codec import quantize_values
    for shape in ((3, 4, 256, 128), (1, 2, 41, 128), (2, 2, 9, 256), (1, 1, 5, 32 if group == 32 else group)):
        if shape[-1] % group:
            continue
        x32 = k4_input(dict(seed=bits * 100 + group, shape=shape, dtype=dtype, zero_row=True))
        packed = quantize_values(to_device(x32, dtype), bits, group)
        ref = oracle.quantize_values(x32, dtype, bits, group)
        for field, tensor in packed.tensors.items():
            assert_same_bytes(tensor, ref.fields()[field], f"{field} {shape}")
        assert_same_bytes(packed.dequantize().float(), oracle.dequantize_values(ref), "dequantize")


@pytest.mark.parametrize("bits", [2, 4])
def test_known_affine_codes_physical_packing_and_zero_range(bits):
    from inquant.value_codec import quantize_values
    codes = torch.arange(1 << bits).repeat(128 // (1 << bits))
    x = (codes.float() * 2 - 3).view(1, 1, 1, 128).expand(2, 3, 7, 128).clone().cuda()
    q = quantize_values(x, bits, 64)
    assert q.payload[0, 0, 0, 0].item() == sum(i << (bits * i) for i in range(8 // bits))
    assert q.payload_nbytes == x.numel() * bits // 8 and q.metadata_nbytes == x.numel() // 64 * 4
    assert torch.equal(q.dequantize(), x)
    for constant in (0., 3., -7.):
        y = torch.full((1, 2, 17, 128), constant, dtype=torch.bfloat16, device="cuda")
        assert torch.equal(quantize_values(y, bits).dequantize(), y)


def test_value_codec_rejects_unrepresentable_parameters_and_blocks_match():
    from inquant.value_codec import quantize_values, quantize_value_blocks
    for value in (float('nan'), float('inf'), 1e6):
        with pytest.raises(ValueError, match="finite"):
            quantize_values(torch.full((1, 1, 2, 128), value, device="cuda"))
    with pytest.raises(ValueError):
        quantize_values(torch.zeros(1, 1, 2, 48, device="cuda"))
    x = to_device(k4_input(dict(seed=52, shape=(1, 3, 103, 128), dtype="bfloat16")))
    blocks = quantize_value_blocks(x, 3, 32, 2, 64)
    for i, block in enumerate(blocks):
        expected = quantize_values(x[:, :, i * 32:(i + 1) * 32], 2, 64)
        for name, tensor in block.tensors.items():
            assert torch.equal(tensor, expected.tensors[name])
        assert block.nbytes == expected.nbytes and block.shape == (1, 3, 32, 128)
