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


class CachePlan:
    """Static-buffer plan for one whole KV cache (all layers, K and V).

    Built once for fixed input tensors: packed outputs, reconstruction outputs and the job
    arrays handed to the C ABI are allocated here, so compress() and decompress() are one
    library call each with no per-call allocation or Python work per layer -- the form a
    serving engine with preallocated cache buffers uses.  Results equal those of the
    per-layer TurboQuantV3 calls on the same tensors.
    """

    def __init__(self, codecs: Sequence[TurboQuantV3], keys: Sequence[torch.Tensor], values: Sequence[torch.Tensor]):
        from . import _native as N
        self.device = keys[0].device
        self._keep = []
        qjobs, self.compressed = [], []
        for codec, k, v in zip(codecs, keys, values):
            j, res, ka = codec.compress_jobs(k, v)
            qjobs.extend(j)
            self.compressed.append(res)
            self._keep.append(ka)
        djobs, self.reconstructed = [], []
        for codec, (ck, cv) in zip(codecs, self.compressed):
            if ck["compressed"] is None:
                self.reconstructed.append((ck["fp16"], cv["fp16"]))
                continue
            j, outs, ka = codec.decompress_jobs(ck, cv)
            djobs.extend(j)
            self.reconstructed.append(outs)
            self._keep.append(ka)
        self._n_q, self._n_d = len(qjobs), len(djobs)
        self._qarr = (N.QuantizeJob * max(self._n_q, 1))(*qjobs)
        self._darr = (N.DequantizeJob * max(self._n_d, 1))(*djobs)
        self._lib = N.lib()
        self._check = N.check
        self._stream = N.stream_ptr

    @torch.no_grad()
    def compress(self):
        """Quantise + pack every layer into the plan's packed buffers (self.compressed)."""
        if self._n_q:
            with torch.cuda.device(self.device):
                self._check(self._lib.tq_quantize(self._qarr, self._n_q, self._stream(self.device)), "tq_quantize")
        return self.compressed

    @torch.no_grad()
    def decompress(self):
        """Unpack + dequantise every layer into the plan's output buffers (self.reconstructed).

        The residual-window tokens were copied into the outputs when the plan was built; call
        refresh_window() if the input tensors changed since."""
        if self._n_d:
            with torch.cuda.device(self.device):
                self._check(self._lib.tq_dequantize(self._darr, self._n_d, self._stream(self.device)), "tq_dequantize")
        return self.reconstructed

    @torch.no_grad()
    def refresh_window(self):
        for (ck, cv), outs in zip(self.compressed, self.reconstructed):
            if ck["compressed"] is None:
                continue
            for comp, full in ((ck, outs[0]), (cv, outs[1])):
                cut = comp["split_at"]
                if full.shape[2] > cut:
                    full[:, :, cut:, :].copy_(comp["fp16"])


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
