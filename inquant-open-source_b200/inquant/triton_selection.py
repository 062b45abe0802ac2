"""GPU donor selection with the reference's ``triton_selection.reuse_map`` signature.

The name is kept for drop-in compatibility; there is no Triton here.  One CTA per row ranks
the channels by counting, builds the selected / available bit masks and assigns donors with
bit scans (C ABI ``inq_select_donors``; reference ``triton_selection.py:11-60``).
"""
import torch

from .codec import _reuse_map


def reuse_map(saliency, count, donor_error=None):
    if saliency.device.type != 'cuda' or saliency.dtype != torch.float32 or saliency.shape[-1] != 128:
        raise ValueError('Fused selector requires CUDA float32 saliency with 128 channels')
    if not 0 <= count <= 64:
        raise ValueError('Expected 0..64 selected channels')
    return _reuse_map(saliency, count, donor_error)
