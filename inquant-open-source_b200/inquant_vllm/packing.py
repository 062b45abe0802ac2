"""Write already-encoded codec output into physical pages (reference ``inquant_vllm/packing.py``).
The fused path (``pack_pages_into``) never materialises codec tensors; this function exists
for callers that hold ``PackedTensor`` / ``PackedValues`` objects."""
import torch

from inquant import _native as N


def write_codec_pages(keys, values, layout, pool, page_ids):
    """Caller owns allocation and supplies unique, in-range GPU page IDs."""
    if pool.dtype != torch.uint8 or pool.ndim != 2 or pool.shape[1] != layout.page_bytes or not pool.is_contiguous():
        raise ValueError('Expected contiguous uint8 destination page pool')
    if page_ids.ndim != 1 or page_ids.numel() != keys.shape[0] or page_ids.dtype not in (torch.int32, torch.int64):
        raise ValueError('One integer physical page ID is required per input page')
    if page_ids.device != pool.device or keys.payload.device != pool.device or values.payload.device != pool.device:
        raise ValueError('Codec tensors, page IDs and pool must share a CUDA device')
    pages, heads = keys.shape[0], layout.heads
    roles = torch.empty((pages, heads, 128), dtype=torch.int16, device=pool.device)
    rc = N.library().inq_build_roles(N.pointer(keys.salient_channels.contiguous()), N.pointer(keys.donor_channels.contiguous()),
                                     0, pages * heads, 128, keys.salient_channels.shape[-1], N.pointer(roles), 2,
                                     N.stream_pointer(pool.device))
    N.check(rc, "inq_build_roles")
    fields = layout.views(pool)
    index = page_ids.long()
    for name, tensor in (("key_payload", keys.payload), ("key_scales", keys.scales), ("key_map", roles),
                         ("key_padding", keys.padding), ("value_payload", values.payload),
                         ("value_scales", values.scales), ("value_offsets", values.offsets)):
        fields[name][index] = tensor.reshape(fields[name][index].shape)
