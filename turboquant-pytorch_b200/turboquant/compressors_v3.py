"""V3 API: MSECompressor (bit-packed MSE-only codec) and TurboQuantV3 (asymmetric K/V
widths, 16-bit residual window, protected layers).

Drop-in for the reference classes of the same names (turboquant/compressors_v3.py):
same constructor arguments, dict keys, dtypes and shapes.  The per-vector work
(norm, rotation, nearest centroid, bit packing and the inverse) runs in fused
sm_100a kernels; strided views such as keys[:, :, :split] are read in place and
decompress_kv writes straight into the final cache-dtype buffer.
"""

from __future__ import annotations

import math

import torch

from . import _native as N
from . import _ops
from .lloyd_max import LloydMaxCodebook
from .turboquant import generate_rotation_matrix


class MSECompressor:
    """L2-normalise, rotate, Lloyd-Max quantise, bit-pack; keeps fp16 norms."""

    def __init__(self, head_dim: int, bits: int, seed: int, device: str = "cpu"):
        N.warn_if_not_cuda(device, "MSECompressor")
        self.head_dim = head_dim
        self.bits = bits
        self.device = device
        self.Pi = generate_rotation_matrix(head_dim, seed=seed, device=device)
        self.centroids = LloydMaxCodebook(head_dim, bits).centroids.to(device)
        self._pi_t = self.Pi.T.contiguous()
        self._cb = N.codebook_block(self.centroids, bits).to(device) if 1 <= bits <= 8 else None
        self._img_q = N.rotation_image(self.Pi)          # tensor-core operands (None off-GPU or for other head_dims)
        self._img_d = N.rotation_image(self._pi_t)

    def _need_bits(self):
        if self._cb is None:
            raise N.BitsError(f"bits must be in 1..8 for bit packing, got {self.bits}")

    # -- jobs, so that callers can batch many compressors into one launch ------
    def compress_job(self, states: torch.Tensor):
        self._need_bits()
        B, H, S, D = states.shape
        if D != self.head_dim:
            raise ValueError(f"last dimension {D} != head_dim {self.head_dim}")
        job, idx, norms, keep = _ops.quantize_job(states, self._pi_t, self._cb, self.bits, True, N.IDX_PACKED,
                                                  image=self._img_q)
        ipb = 8 // self.bits
        result = {"idx_bytes": idx, "vec_norms": norms, "shape": (B, H, S, D), "idx_pad": (ipb - D % ipb) % ipb}
        return job, result, keep

    def decompress_job(self, compressed: dict, out: torch.Tensor):
        self._need_bits()
        return _ops.dequantize_job(compressed["idx_bytes"], compressed["vec_norms"], compressed["shape"], self.Pi,
                                   self._cb, self.bits, N.IDX_PACKED, out, image=self._img_d)

    @torch.no_grad()
    def compress(self, states: torch.Tensor) -> dict:
        """(B, H, S, D) -> {"idx_bytes" uint8 (B,H,S,G), "vec_norms" fp16 (B,H,S), "shape", "idx_pad"}."""
        job, result, _keep = self.compress_job(states)
        _ops.run_quantize([job], states.device)
        return result

    @torch.no_grad()
    def decompress(self, compressed: dict) -> torch.Tensor:
        """Back to an fp32 (B, H, S, D) tensor."""
        B, H, S, D = compressed["shape"]
        out = torch.empty((B, H, S, D), dtype=torch.float32, device=compressed["idx_bytes"].device)
        job, _keep = self.decompress_job(compressed, out)
        _ops.run_dequantize([job], out.device)
        return out

    @torch.no_grad()
    def attention_scores(self, queries: torch.Tensor, compressed: dict, scale: float = 1.0, softmax: bool = False):
        """q . k_hat for every compressed key without reconstructing keys.

        queries (B, Hq, Sq, D) with Hq a multiple of the compressed head count;
        returns fp32 logits (B, Hq, Sq, S) and, with softmax=True, the
        probabilities too.  Equals matmul(q, decompress(compressed)^T) * scale.
        """
        self._need_bits()
        return _ops.score_packed(queries, compressed["idx_bytes"], compressed["vec_norms"], self._pi_t, self._cb,
                                 self.bits, scale=scale, softmax=softmax)

    def memory_bytes(self, B: int, H: int, S: int) -> dict:
        n = B * H * S
        packed = n * math.ceil(self.head_dim / (8 // self.bits)) + n * 2
        dense = n * self.head_dim * 2
        return {"compressed_bytes": packed, "fp16_bytes": dense,
                "compression_ratio": dense / packed if packed > 0 else 0}


class TurboQuantV3:
    """KV-cache compressor: MSE-only, separate key/value widths, recent tokens kept as they are."""

    def __init__(self, head_dim: int, key_bits: int = 4, value_bits: int = 2, residual_window: int = 128,
                 layer_idx: int = 0, n_layers: int = 36, protected_layers: int = 4, protected_bits: int = 8,
                 seed: int = 42, device: str = "cpu"):
        self.head_dim = head_dim
        self.residual_window = residual_window
        self.device = device
        guarded = layer_idx < protected_layers or layer_idx >= (n_layers - protected_layers)
        self.key_bits = min(protected_bits if guarded else key_bits, 8)
        self.value_bits = min(protected_bits if guarded else value_bits, 8)
        base = seed + layer_idx * 1000
        self.key_compressor = MSECompressor(head_dim, self.key_bits, seed=base, device=device)
        self.val_compressor = MSECompressor(head_dim, self.value_bits, seed=base + 500, device=device)

    def _passthrough(self, keys, values):
        B, H, S, D = keys.shape
        return ({"fp16": keys, "compressed": None, "shape": (B, H, S, D), "split_at": S},
                {"fp16": values, "compressed": None, "shape": (B, H, S, D), "split_at": S})

    def compress_jobs(self, keys: torch.Tensor, values: torch.Tensor):
        """(jobs, (compressed_k, compressed_v), keepalive); jobs is empty for the passthrough case."""
        B, H, S, D = keys.shape
        if S <= self.residual_window:
            return [], self._passthrough(keys, values), ()
        cut = S - self.residual_window
        jk, rk, keep_k = self.key_compressor.compress_job(keys[:, :, :cut, :])
        jv, rv, keep_v = self.val_compressor.compress_job(values[:, :, :cut, :])
        ck = {"compressed": rk, "fp16": keys[:, :, cut:, :], "shape": (B, H, S, D), "split_at": cut}
        cv = {"compressed": rv, "fp16": values[:, :, cut:, :], "shape": (B, H, S, D), "split_at": cut}
        return [jk, jv], (ck, cv), (keep_k, keep_v)

    @torch.no_grad()
    def compress_kv(self, keys: torch.Tensor, values: torch.Tensor):
        jobs, result, _keep = self.compress_jobs(keys, values)
        if jobs:
            _ops.run_quantize(jobs, keys.device)
        return result

    def decompress_jobs(self, compressed_k: dict, compressed_v: dict):
        """(jobs, (keys, values), keepalive): outputs are allocated in the cache dtype, the window copied in."""
        outs, jobs, keep = [], [], []
        for comp, codec in ((compressed_k, self.key_compressor), (compressed_v, self.val_compressor)):
            B, H, S, D = comp["shape"]
            window = comp["fp16"]
            cut = comp["split_at"]
            full = torch.empty((B, H, S, D), dtype=window.dtype, device=window.device)
            if S > cut:
                full[:, :, cut:, :].copy_(window)
            job, k = codec.decompress_job(comp["compressed"], full[:, :, :cut, :])
            jobs.append(job)
            keep.append(k)
            outs.append(full)
        return jobs, tuple(outs), keep

    @torch.no_grad()
    def decompress_kv(self, compressed_k: dict, compressed_v: dict):
        if compressed_k["compressed"] is None:
            return compressed_k["fp16"], compressed_v["fp16"]
        jobs, outs, _keep = self.decompress_jobs(compressed_k, compressed_v)
        _ops.run_dequantize(jobs, outs[0].device)
        return outs

    @torch.no_grad()
    def decode_attention(self, queries: torch.Tensor, compressed_k: dict, compressed_v: dict, scale: float = None):
        """Attention output straight from what compress_kv returned, without decompress_kv.

        queries (B, Hq, Sq, head_dim) with Hq a multiple of the cache's KV heads; returns fp32 (B, Hq, Sq, head_dim)
        equal to  softmax(scale * q K^T) V  over the tokens decompress_kv would return (reconstructed packed
        tokens followed by the kept window tokens).  scale defaults to head_dim ** -0.5.  Not part of the
        reference API: the reference decompresses every chunk and attends on the result
        (turboquant/generation_test_v2.py:131-147); this is that composition in one pass over the packed bytes.
        """
        if scale is None:
            scale = self.head_dim ** -0.5
        self.key_compressor._need_bits()
        self.val_compressor._need_bits()
        return _ops.decode_attention(queries, compressed_k["compressed"], compressed_v["compressed"], self.key_compressor,
                                     self.val_compressor, compressed_k["fp16"], compressed_v["fp16"], scale)

    def memory_bytes(self, B: int, H: int, S: int) -> dict:
        window = min(self.residual_window, S)
        packed_tokens = max(S - window, 0)
        packed = 0
        if packed_tokens > 0:
            packed = (self.key_compressor.memory_bytes(B, H, packed_tokens)["compressed_bytes"]
                      + self.val_compressor.memory_bytes(B, H, packed_tokens)["compressed_bytes"])
        kept = B * H * window * self.head_dim * 2 * 2
        total = packed + kept
        dense = B * H * S * self.head_dim * 2 * 2
        return {"compressed_bytes": total, "fp16_bytes": dense,
                "compression_ratio": dense / total if total > 0 else 0,
                "compressed_tokens": packed_tokens, "fp16_tokens": window,
                "key_bits": self.key_bits, "value_bits": self.value_bits}
