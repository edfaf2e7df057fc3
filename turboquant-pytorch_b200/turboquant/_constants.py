"""Device-resident constants shared by the compressor classes."""

from __future__ import annotations

import torch

from . import _native


class RotationSet:
    """Pi and Pi^T as contiguous fp32 tensors on one device."""

    def __init__(self, pi: torch.Tensor):
        self.pi = pi.contiguous()
        self.pi_t = pi.T.contiguous()


def device_codebook(centroids: torch.Tensor, bits: int, device) -> torch.Tensor:
    return _native.codebook_block(centroids, bits).to(device)
