"""Write already-encoded codec output into physical pages (reference ``inquant_vllm/packing.py``):
one launch of ``inq_write_codec_pages`` scatters every field and builds the pages' role maps.
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
    if keys.salient_channels.shape[-1] != 16 or keys.salient_channels.dtype != torch.uint8:
        raise ValueError('The page layout holds 16 salient channels per head')
    from .kernels import page_offsets_array
    tensors = [t.contiguous() for t in (keys.payload, keys.scales, keys.salient_channels, keys.donor_channels, keys.padding,
                                        values.payload, values.scales, values.offsets)]
    ids = page_ids.contiguous()
    args = N.WritePagesArgs(*(t.data_ptr() for t in tensors), keys.shape[0], layout.heads, layout.block_size, 16,
                            pool.data_ptr(), layout.page_bytes, page_offsets_array(layout), ids.data_ptr(),
                            int(ids.dtype == torch.int64), pool.shape[0], N.status_word(pool.device).data_ptr())
    N.check(N.library().inq_write_codec_pages(N.ctypes.byref(args), N.stream_pointer(pool.device)), "inq_write_codec_pages")
