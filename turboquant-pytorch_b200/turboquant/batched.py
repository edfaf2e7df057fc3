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
    def capture(self, decompress: bool = True) -> "torch.cuda.CUDAGraph":
        """compress() (and decompress()) recorded into a CUDA graph for replay with `graph.replay()`.

        The plan's buffers and job arrays are static, and from its second call on the library only issues the
        kernel launch for an unchanged job array, so the calls can be stream-captured; one eager pass runs first.
        A plan with a residual window copies the window tokens inside the graph as well."""
        has_window = any(ck["compressed"] is not None and ck["fp16"].shape[2] > 0 for ck, _ in self.compressed)
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):             # eager pass: the library builds and keeps its launch descriptions
            self.compress()
            if decompress:
                self.decompress()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.compress()
            if decompress:
                if has_window:
                    self.refresh_window()
                self.decompress()
        return graph

    @torch.no_grad()
    def refresh_window(self):
        for (ck, cv), outs in zip(self.compressed, self.reconstructed):
            if ck["compressed"] is None:
                continue
            for comp, full in ((ck, outs[0]), (cv, outs[1])):
                cut = comp["split_at"]
                if full.shape[2] > cut:
                    full[:, :, cut:, :].copy_(comp["fp16"])


class HostStreamedCache:
    """Round trip of a KV cache that lives in pinned host memory, pipelined over PCIe.

    The layers are split into groups.  Each group has its own device staging tensors and
    CachePlan; three streams carry host->device copies, the two kernels and device->host
    copies, so that group g is being quantised and dequantised while group g+1 arrives
    and group g-1 leaves (the link is full duplex).  Results are those of CachePlan on
    the same tensors.  run() returns once everything is enqueued; the calling stream waits
    for the last copy, so ordinary stream semantics hold for the caller.
    """

    def __init__(self, codecs: Sequence[TurboQuantV3], host_keys: Sequence[torch.Tensor],
                 host_values: Sequence[torch.Tensor], device, groups: int = 6):
        if not all(t.is_pinned() for t in list(host_keys) + list(host_values)):
            raise ValueError("HostStreamedCache needs pinned host tensors")
        self.device = torch.device(device)
        n = len(codecs)
        groups = max(1, min(groups, n))
        self.host_keys, self.host_values = list(host_keys), list(host_values)
        self.host_out_keys = [torch.empty_like(t).pin_memory() for t in host_keys]
        self.host_out_values = [torch.empty_like(t).pin_memory() for t in host_values]
        self.dev_keys = [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in host_keys]
        self.dev_values = [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in host_values]
        self.bounds = [(n * g // groups, n * (g + 1) // groups) for g in range(groups)]
        self.plans = [CachePlan(codecs[a:b], self.dev_keys[a:b], self.dev_values[a:b]) for a, b in self.bounds]
        self._windows = any(c.residual_window > 0 for c in codecs)
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        mk = lambda: [torch.cuda.Event() for _ in self.bounds]
        self.ev_in, self.ev_packed, self.ev_run, self.ev_out = mk(), mk(), mk(), mk()
        self._ran = False
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in self.host_keys + self.host_values)
        self.d2h_bytes = self.h2d_bytes

    @torch.no_grad()
    def run(self):
        """Copy in, compress, decompress, copy out; returns the pinned output tensors."""
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for st in (self.s_in, self.s_run, self.s_out):
            st.wait_event(start)
        for g, (a, b) in enumerate(self.bounds):
            plan = self.plans[g]
            with torch.cuda.stream(self.s_in):
                if self._ran:
                    self.s_in.wait_event(self.ev_packed[g])      # last run's quantize has read the staging tensors
                for l in range(a, b):
                    self.dev_keys[l].copy_(self.host_keys[l], non_blocking=True)
                    self.dev_values[l].copy_(self.host_values[l], non_blocking=True)
                self.ev_in[g].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[g])
                if self._ran:
                    self.s_run.wait_event(self.ev_out[g])        # last run's outputs have left the device
                plan.compress()
                self.ev_packed[g].record(self.s_run)
                if self._windows:
                    plan.refresh_window()
                plan.decompress()
                self.ev_run[g].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[g])
                for i, l in enumerate(range(a, b)):
                    rk, rv = plan.reconstructed[i]
                    self.host_out_keys[l].copy_(rk, non_blocking=True)
                    self.host_out_values[l].copy_(rv, non_blocking=True)
                self.ev_out[g].record(self.s_out)
        self._ran = True
        for st in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(st)
        return self.host_out_keys, self.host_out_values


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
