"""Host-side containers of sealed blocks that need no GPU: the per-block objects of an encoder
arena (``ArenaPackedTensor`` / ``ArenaPackedValues``: reference ``codec.py:58-110`` and
``value_codec.py:12-36`` give the fields and byte counts they must report) and the helper that
gathers one field over the blocks of a decode state."""
import pytest
import torch

from inquant.codec import ArenaPackedTensor, PackedTensor
from inquant.value_codec import ArenaPackedValues, PackedValues

B, H, T, C, PAD = 5, 4, 32, 128, 16


def _key_arena():
    g = torch.Generator().manual_seed(3)
    return PackedTensor(torch.randint(0, 255, (B, H, T, C // 2), dtype=torch.uint8, generator=g),
                        torch.rand((B, H, C), generator=g),
                        torch.randint(0, 127, (B, H, PAD), dtype=torch.uint8, generator=g),
                        torch.randint(0, 127, (B, H, PAD), dtype=torch.uint8, generator=g),
                        torch.rand((B, H, PAD), generator=g), (B, H, T, C), torch.bfloat16)


def _value_arena():
    g = torch.Generator().manual_seed(4)
    return PackedValues(torch.randint(0, 255, (B, H, T, C // 4), dtype=torch.uint8, generator=g),
                        torch.rand((B, H, T, 2), generator=g).half(), torch.rand((B, H, T, 2), generator=g).half(),
                        (B, H, T, C), torch.bfloat16, 2, 64)


def test_arena_blocks_report_what_a_block_of_their_own_would():
    arena = _key_arena()
    blocks = ArenaPackedTensor.split(arena, B)
    assert len(blocks) == B and all(isinstance(b, PackedTensor) for b in blocks)
    for index, block in enumerate(blocks):
        assert block._arena[0] is arena and block._arena[1] == index
        assert block.shape == (1, H, T, C) and block.original_dtype == torch.bfloat16
        for name, whole in arena.tensors.items():
            part = getattr(block, name)
            assert part.shape == (1, *whole.shape[1:]) and torch.equal(part[0], whole[index])
            assert part.data_ptr() == block.field_pointer(name)       # a view, not a copy
            assert getattr(block, name) is part                       # materialised once
        own = PackedTensor(*(t[index:index + 1].clone() for t in arena.tensors.values()), (1, H, T, C), torch.bfloat16)
        assert block.nbytes == own.nbytes and block.payload_nbytes == own.payload_nbytes
        assert block.metadata_nbytes == own.metadata_nbytes
        assert block.storage_stats() == own.storage_stats()
    with pytest.raises(AttributeError):
        blocks[0].no_such_field
    single = ArenaPackedTensor(arena, 2)
    assert torch.equal(single.scales[0], arena.scales[2])


def test_arena_value_blocks_carry_the_codec_parameters_of_their_arena():
    arena = _value_arena()
    blocks = ArenaPackedValues.split(arena, B)
    for index, block in enumerate(blocks):
        assert isinstance(block, PackedValues) and (block.bits, block.group_size) == (2, 64)
        assert block.shape == (1, H, T, C) and block.original_dtype == torch.bfloat16
        assert set(block.tensors) == {"payload", "scales", "offsets"}
        for name, whole in arena.tensors.items():
            assert torch.equal(getattr(block, name)[0], whole[index])
        own = PackedValues(*(t[index:index + 1].clone() for t in arena.tensors.values()), (1, H, T, C), torch.bfloat16, 2, 64)
        assert block.nbytes == own.nbytes and block.payload_nbytes == own.payload_nbytes


def test_a_block_that_was_never_bound_to_an_arena_raises_instead_of_recursing():
    orphan = object.__new__(ArenaPackedTensor)
    with pytest.raises(AttributeError):
        orphan.payload
    assert getattr(orphan, "_arena", None) is None


def test_stacked_field_takes_runs_of_one_arena_as_one_slice():
    from inquant.triton_attention import _stacked_field
    arena, other = _key_arena(), _key_arena()
    blocks = ArenaPackedTensor.split(arena, B)
    whole = _stacked_field(blocks, "salient_channels")
    assert whole.data_ptr() == arena.salient_channels.data_ptr() and whole.shape == (B, H, PAD)   # no copy at all
    tail = _stacked_field(blocks[2:], "donor_channels")
    assert tail.data_ptr() == blocks[2].field_pointer("donor_channels") and torch.equal(tail, arena.donor_channels[2:])
    plain = PackedTensor(*(t[1:2].clone() for t in other.tensors.values()), (1, H, T, C), torch.bfloat16)
    mixed = [plain, blocks[1], blocks[2], plain, blocks[4], blocks[0]] + ArenaPackedTensor.split(other, B)[3:]
    got = _stacked_field(mixed, "salient_channels")
    want = torch.cat([m.salient_channels for m in mixed], dim=0)
    assert got.is_contiguous() and torch.equal(got, want)
