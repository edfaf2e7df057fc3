"""Whole-cache entry points: every layer's K and V in one library call.

A KV cache is many small independent problems (one rotation and codebook per
layer and per K/V).  Submitting them together lets the library schedule all
tiles of all layers as a single persistent launch instead of two launches per
layer.  Results are identical to calling each TurboQuantV3 on its own.
"""

from __future__ import annotations

from typing import Sequence

import torch

from . import _ops
from .compressors_v3 import TurboQuantV3


@torch.no_grad()
def compress_kv_layers(codecs: Sequence[TurboQuantV3], keys: Sequence[torch.Tensor], values: Sequence[torch.Tensor]):
    """[(compressed_k, compressed_v)] for layers 0..L-1, one tq_quantize call for all of them."""
    jobs, results, keep = [], [], []
    for codec, k, v in zip(codecs, keys, values):
        j, res, ka = codec.compress_jobs(k, v)
        jobs.extend(j)
        results.append(res)
        keep.append(ka)
    if jobs:
        _ops.run_quantize(jobs, keys[0].device)
    return results


@torch.no_grad()
def decompress_kv_layers(codecs: Sequence[TurboQuantV3], compressed: Sequence[tuple]):
    """[(keys, values)] in the cache dtype, one tq_dequantize call for all layers."""
    jobs, results, keep = [], [], []
    device = None
    for codec, (ck, cv) in zip(codecs, compressed):
        if ck["compressed"] is None:
            results.append((ck["fp16"], cv["fp16"]))
            continue
        j, outs, ka = codec.decompress_jobs(ck, cv)
        jobs.extend(j)
        results.append(outs)
        keep.append(ka)
        device = outs[0].device
    if jobs:
        _ops.run_dequantize(jobs, device)
    return results


def shard_units(n_layers: int, n_kv_heads: int, rank: int, world: int):
    """(layer, kv_head) units owned by `rank`: contiguous blocks of the layer-major unit list.

    Units are independent (no collective on the data path); a contiguous block
    keeps each rank's layers adjacent, so it needs the constants of as few layers
    as possible.
    """
    total = n_layers * n_kv_heads
    lo = total * rank // world
    hi = total * (rank + 1) // world
    return [(u // n_kv_heads, u % n_kv_heads) for u in range(lo, hi)]
