"""Whole-cache entry points: every layer's K and V in one library call.

A KV cache is many small independent problems (one rotation and codebook per
layer and per K/V).  Submitting them together lets the library schedule all
tiles of all layers as a single persistent launch instead of two launches per
layer.  Results are identical to calling each TurboQuantV3 on its own.
"""

from __future__ import annotations

import ctypes as C
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
    per-layer TurboQuantV3 calls on the same tensors.  Both calls take an optional layer
    range [lo, hi) so that a caller can pipeline groups of layers over the same buffers.
    """

    def __init__(self, codecs: Sequence[TurboQuantV3], keys: Sequence[torch.Tensor], values: Sequence[torch.Tensor]):
        from . import _native as N
        self.device = keys[0].device
        self.n_layers = len(codecs)
        self._keep = []
        qjobs, self.compressed = [], []
        self._q_range, self._d_range, self._c_range = [], [], []      # per layer: job index ranges
        for codec, k, v in zip(codecs, keys, values):
            j, res, ka = codec.compress_jobs(k, v)
            self._q_range.append((len(qjobs), len(qjobs) + len(j)))
            qjobs.extend(j)
            self.compressed.append(res)
            self._keep.append(ka)
        djobs, cjobs, self.reconstructed = [], [], []
        self._torch_windows = []          # (dst view, src) pairs the copy kernel cannot take (odd alignment)
        for codec, (ck, cv) in zip(codecs, self.compressed):
            d0, c0 = len(djobs), len(cjobs)
            if ck["compressed"] is None:
                self.reconstructed.append((ck["fp16"], cv["fp16"]))
            else:
                j, outs, ka = codec.decompress_jobs(ck, cv)
                djobs.extend(j)
                self.reconstructed.append(outs)
                self._keep.append(ka)
                for comp, full in ((ck, outs[0]), (cv, outs[1])):
                    cut, win = comp["split_at"], comp["fp16"]
                    if full.shape[2] > cut:
                        job = self._copy_job(N, win, full[:, :, cut:, :])
                        if job is None:
                            self._torch_windows.append((len(self.reconstructed) - 1, full[:, :, cut:, :], win))
                        else:
                            cjobs.append(job)
            self._d_range.append((d0, len(djobs)))
            self._c_range.append((c0, len(cjobs)))
        self._n_q, self._n_d, self._n_c = len(qjobs), len(djobs), len(cjobs)
        self._qarr = (N.QuantizeJob * max(self._n_q, 1))(*qjobs)
        self._darr = (N.DequantizeJob * max(self._n_d, 1))(*djobs)
        self._carr = (N.CopyJob * max(self._n_c, 1))(*cjobs)
        self._qsize, self._dsize, self._csize = (C.sizeof(N.QuantizeJob), C.sizeof(N.DequantizeJob),
                                                 C.sizeof(N.CopyJob))
        self._lib = N.lib()
        self._check = N.check
        self._stream = N.stream_ptr

    @staticmethod
    def _copy_job(N, src: torch.Tensor, dst: torch.Tensor):
        """A TqCopyJob for src -> dst ((B,H,S,D) views with unit last stride), or None when the kernel's
        16-byte alignment rules do not hold."""
        B, H, S, D = src.shape
        eb = src.element_size()
        if src.dtype != dst.dtype or eb not in (2, 4) or (D * eb) % 16 or src.stride(3) != 1 or dst.stride(3) != 1:
            return None
        if src.data_ptr() % 16 or dst.data_ptr() % 16:
            return None
        for t in (src, dst):
            for dim in range(3):
                if t.shape[dim] > 1 and (t.stride(dim) * eb) % 16:
                    return None
        return N.CopyJob(src=src.data_ptr(), dst=dst.data_ptr(), elem_bytes=eb, D=D, B=B, H=H, S=S,
                         sstride_b=src.stride(0), sstride_h=src.stride(1), sstride_s=src.stride(2),
                         dstride_b=dst.stride(0), dstride_h=dst.stride(1), dstride_s=dst.stride(2))

    def _span(self, ranges, lo, hi):
        lo = 0 if lo is None else lo
        hi = self.n_layers if hi is None else hi
        if hi <= lo:
            return 0, 0
        return ranges[lo][0], ranges[hi - 1][1]

    @staticmethod
    def _sub(arr, first, size):
        """Pointer to element `first` of a ctypes job array (the C ABI takes pointer + count)."""
        return C.cast(C.addressof(arr) + first * size, C.POINTER(arr._type_))

    @torch.no_grad()
    def compress(self, lo: int = None, hi: int = None):
        """Quantise + pack layers [lo, hi) (default: all) into the plan's packed buffers (self.compressed)."""
        a, b = self._span(self._q_range, lo, hi)
        if b > a:
            with torch.cuda.device(self.device):
                self._check(self._lib.tq_quantize(self._sub(self._qarr, a, self._qsize), b - a,
                                                  self._stream(self.device)), "tq_quantize")
        return self.compressed

    @torch.no_grad()
    def decompress(self, lo: int = None, hi: int = None, window: bool = True):
        """Unpack + dequantise layers [lo, hi) into the plan's output buffers (self.reconstructed).

        With `window` (default) the kept residual-window tokens are copied into the outputs first, so the
        outputs are what TurboQuantV3.decompress_kv returns for the inputs' current contents."""
        if window:
            self.refresh_window(lo, hi)
        a, b = self._span(self._d_range, lo, hi)
        if b > a:
            with torch.cuda.device(self.device):
                self._check(self._lib.tq_dequantize(self._sub(self._darr, a, self._dsize), b - a,
                                                    self._stream(self.device)), "tq_dequantize")
        return self.reconstructed

    @torch.no_grad()
    def refresh_window(self, lo: int = None, hi: int = None):
        """Copy the kept 16-bit window tokens of layers [lo, hi) into the outputs: one tq_copy_rows call."""
        a, b = self._span(self._c_range, lo, hi)
        if b > a:
            with torch.cuda.device(self.device):
                self._check(self._lib.tq_copy_rows(self._sub(self._carr, a, self._csize), b - a,
                                                   self._stream(self.device)), "tq_copy_rows")
        l0 = 0 if lo is None else lo
        l1 = self.n_layers if hi is None else hi
        for layer, dst, src in self._torch_windows:
            if l0 <= layer < l1:
                dst.copy_(src)

    @torch.no_grad()
    def capture(self, decompress: bool = True) -> "torch.cuda.CUDAGraph":
        """compress() (and decompress()) recorded into a CUDA graph for replay with `graph.replay()`.

        The plan's buffers and job arrays are static.  When the whole plan goes out as ONE tensor-core launch
        per call (every job eligible, one input dtype, at most 96 jobs) the library keeps the prepared launch
        descriptions of the last four distinct job arrays of the calling thread and the captured call only issues
        the kernel; a plan that splits into
        several launches re-encodes its tensor maps on every call, which stream capture tolerates but which
        costs host time.  One eager pass runs first."""
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
                self.decompress()
        return graph


class HostStreamedCache:
    """Round trip of a KV cache that lives in pinned host memory, pipelined over PCIe.

    The layers are split into groups.  Three streams carry host->device copies, the kernels
    and device->host copies, so that group g is being quantised and dequantised while group
    g+1 arrives and group g-1 leaves (the link is full duplex).  All groups share ONE
    CachePlan (one set of device buffers); a group is a layer range of it.  Results are those
    of CachePlan on the same tensors.  run() returns once everything is enqueued; the
    calling stream waits for the last copy, so ordinary stream semantics hold for the caller.
    `plan`, `dev_keys`, `dev_values` may be given to reuse device buffers that already exist.
    """

    def __init__(self, codecs: Sequence[TurboQuantV3], host_keys: Sequence[torch.Tensor],
                 host_values: Sequence[torch.Tensor], device, groups: int = 6, plan: "CachePlan" = None,
                 dev_keys=None, dev_values=None, host_out_keys=None, host_out_values=None):
        if not all(t.is_pinned() for t in list(host_keys) + list(host_values)):
            raise ValueError("HostStreamedCache needs pinned host tensors")
        self.device = torch.device(device)
        n = len(codecs)
        groups = max(1, min(groups, n))
        self.host_keys, self.host_values = list(host_keys), list(host_values)
        self.host_out_keys = host_out_keys or [torch.empty_like(t).pin_memory() for t in host_keys]
        self.host_out_values = host_out_values or [torch.empty_like(t).pin_memory() for t in host_values]
        self.dev_keys = dev_keys or [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in host_keys]
        self.dev_values = dev_values or [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in host_values]
        self.bounds = [(n * g // groups, n * (g + 1) // groups) for g in range(groups)]
        self.plan = plan or CachePlan(codecs, self.dev_keys, self.dev_values)
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        mk = lambda: [torch.cuda.Event() for _ in self.bounds]
        self.ev_in, self.ev_packed, self.ev_run, self.ev_out = mk(), mk(), mk(), mk()
        self._ran = False
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in self.host_keys + self.host_values)
        self.d2h_bytes = self.h2d_bytes

    @torch.no_grad()
    def run(self, kernels: bool = True):
        """Copy in, compress, decompress, copy out; returns the pinned output tensors.

        kernels=False moves the same bytes without launching the codec kernels (the copy-only floor of
        this round trip; the outputs then hold whatever the buffers held)."""
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for st in (self.s_in, self.s_run, self.s_out):
            st.wait_event(start)
        plan = self.plan
        for g, (a, b) in enumerate(self.bounds):
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
                if kernels:
                    plan.compress(a, b)
                self.ev_packed[g].record(self.s_run)
                if kernels:
                    plan.decompress(a, b)
                self.ev_run[g].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[g])
                for l in range(a, b):
                    rk, rv = plan.reconstructed[l]
                    self.host_out_keys[l].copy_(rk, non_blocking=True)
                    self.host_out_values[l].copy_(rv, non_blocking=True)
                self.ev_out[g].record(self.s_out)
        self._ran = True
        for st in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(st)
        return self.host_out_keys, self.host_out_values


def shard_units(n_layers: int, n_kv_heads: int, rank: int, world: int, layer_costs=None):
    """(layer, kv_head) units owned by `rank`: contiguous blocks of the layer-major unit list.

    Units are independent (no collective on the data path); a contiguous block
    keeps each rank's layers adjacent, so it needs the constants of as few layers
    as possible.  With layer_costs (one relative cost per layer, e.g. from tile_cost()) the blocks have equal
    cost instead of equal length: the 8-bit protected layers at both ends of a cache cost ~1.25 x an ordinary
    K6/V4 layer, and with equal lengths the first and the last rank finish last.
    """
    total = n_layers * n_kv_heads
    if layer_costs is None:
        lo = total * rank // world
        hi = total * (rank + 1) // world
    else:
        if len(layer_costs) != n_layers or min(layer_costs) <= 0:
            raise ValueError("layer_costs: one positive number per layer")
        cum = [0.0]
        for u in range(total):
            cum.append(cum[-1] + float(layer_costs[u // n_kv_heads]))
        bounds = [0]
        for r in range(1, world):
            target = cum[-1] * r / world
            b = bounds[-1]
            while b < total and abs(cum[b + 1] - target) <= abs(cum[b] - target):
                b += 1
            bounds.append(b)
        bounds.append(total)
        lo, hi = bounds[rank], bounds[rank + 1]
    return [(u // n_kv_heads, u % n_kv_heads) for u in range(lo, hi)]


def tile_cost(key_bits: int, value_bits: int) -> float:
    """Relative cost of quantising and dequantising one K and one V vector at these widths on the tensor-core path
    (bf16 tile weights of the library, measured on B200): for cost-balanced shards."""
    q = {1: 133, 2: 133, 3: 144, 4: 144, 5: 144, 6: 170, 7: 219, 8: 219}
    d = {1: 127, 2: 127, 3: 130, 4: 130, 5: 152, 6: 152, 7: 152, 8: 157}
    return float(q[key_bits] + q[value_bits] + d[key_bits] + d[value_bits])
