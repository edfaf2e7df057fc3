"""V1 API: TurboQuantMSE, TurboQuantProd, TurboQuantKVCache and the matrix generators.

Same names, signatures and return structures as the reference module of the
same name (tonbistudio/turboquant-pytorch, turboquant/turboquant.py); the
arithmetic on vectors runs in the sm_100a kernels of libturboquant_b200.so.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import _native as N
from . import _ops
from .lloyd_max import LloydMaxCodebook


def _seeded_gaussian(rows: int, cols: int, seed: Optional[int]) -> torch.Tensor:
    # The CPU generator stream is part of the format: the same seed must give the
    # same matrix on every machine, so the draw never happens on the GPU.
    gen = torch.Generator(device="cpu")
    if seed is not None:
        gen.manual_seed(seed)
    return torch.randn(rows, cols, generator=gen)


def generate_rotation_matrix(d: int, seed: Optional[int] = None, device: str = "cpu") -> torch.Tensor:
    """Haar-random orthogonal d x d matrix: Q of a Gaussian's QR with R's diagonal made positive."""
    q, r = torch.linalg.qr(_seeded_gaussian(d, d, seed))
    flip = torch.sign(torch.diag(r))
    flip[flip == 0] = 1.0
    # LAPACK hands Q back column-major; the kernels take raw pointers, so fix the layout here
    return (q * flip.unsqueeze(0)).contiguous().to(device)


def generate_qjl_matrix(d: int, m: Optional[int] = None, seed: Optional[int] = None, device: str = "cpu") -> torch.Tensor:
    """i.i.d. N(0,1) projection matrix of shape (m, d); m defaults to d."""
    return _seeded_gaussian(d if m is None else m, d, seed).to(device)


class TurboQuantMSE(nn.Module):
    """Stage 1: rotate by Pi, then per-coordinate Lloyd-Max quantisation (expects unit vectors)."""

    def __init__(self, d: int, bits: int, seed: int = 42, device: str = "cpu"):
        super().__init__()
        self.d = d
        self.bits = bits
        self.device = device
        N.warn_if_not_cuda(device, "TurboQuantMSE")
        self.codebook = LloydMaxCodebook(d, bits)
        pi = generate_rotation_matrix(d, seed=seed, device=device)
        self.register_buffer("Pi", pi)
        self.register_buffer("centroids", self.codebook.centroids.to(device))
        self.register_buffer("boundaries", self.codebook.boundaries.to(device))
        # kernel-side constants; not part of the state dict
        self.register_buffer("_pi_t", pi.T.contiguous(), persistent=False)
        self.register_buffer("_cb", N.codebook_block(self.codebook.centroids, bits).to(device), persistent=False)
        self.register_load_state_dict_post_hook(TurboQuantMSE._after_load)

    @staticmethod
    def _after_load(module, _incompatible_keys):
        module._refresh_kernel_constants()          # a post hook must return None

    def _refresh_kernel_constants(self):
        """Re-derive the kernel-side constants from Pi and centroids (after load_state_dict changed them)."""
        with torch.no_grad():
            self._pi_t.copy_(self.Pi.T)
            self._cb.copy_(N.codebook_block(self.centroids, self.bits))
            self.codebook.centroids = self.centroids.detach().cpu().clone()
            self.codebook.boundaries = self.boundaries.detach().cpu().clone()

    def rotate(self, x: torch.Tensor) -> torch.Tensor:
        return _ops.project(x, self._pi_t)

    def unrotate(self, y: torch.Tensor) -> torch.Tensor:
        return _ops.project(y, self.Pi)

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        flat = x.reshape(1, 1, -1, self.d)
        job, idx, _norms, keep = _ops.quantize_job(flat, self._pi_t, self._cb, self.bits, False, N.IDX_I64)
        _ops.run_quantize([job], x.device)
        return idx.reshape(x.shape)

    def dequantize(self, indices: torch.Tensor) -> torch.Tensor:
        n = indices.numel() // self.d
        out = torch.empty((1, 1, n, self.d), dtype=torch.float32, device=indices.device)
        job, keep = _ops.dequantize_job(indices.reshape(n, self.d), None, (1, 1, n, self.d), self.Pi, self._cb,
                                        self.bits, N.IDX_I64, out)
        _ops.run_dequantize([job], indices.device)
        return out.reshape(indices.shape)

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        indices = self.quantize(x)
        return self.dequantize(indices), indices


class TurboQuantProd(nn.Module):
    """Stage 1 at bits-1 plus a 1-bit QJL sketch of the residual: unbiased inner products."""

    def __init__(self, d: int, bits: int, qjl_dim: Optional[int] = None, seed: int = 42, device: str = "cpu"):
        super().__init__()
        self.d = d
        self.bits = bits
        self.mse_bits = max(bits - 1, 1)
        self.qjl_dim = qjl_dim or d
        self.device = device
        N.warn_if_not_cuda(device, "TurboQuantProd")
        self.mse = TurboQuantMSE(d, self.mse_bits, seed=seed, device=device)
        s = generate_qjl_matrix(d, m=self.qjl_dim, seed=seed + 1, device=device)
        self.register_buffer("S", s)
        self.register_buffer("_s_t", s.T.contiguous(), persistent=False)
        self.register_load_state_dict_post_hook(TurboQuantProd._after_load)

    @staticmethod
    def _after_load(module, _incompatible_keys):
        with torch.no_grad():
            module._s_t.copy_(module.S.T)

    def quantize(self, x: torch.Tensor) -> dict:
        flat = x.reshape(1, 1, -1, self.d)
        _k, idx, signs, rnorm = _ops.qjl_compress(flat, self.mse.Pi, self.mse._pi_t, self.mse._cb, self._s_t,
                                                  self.mse_bits, normalize=False, want_k_mse=False,
                                                  idx_mode=N.IDX_I64, signs_fp32=True, rnorm_fp32=True)
        lead = x.shape[:-1]
        return {"mse_indices": idx.reshape(*lead, self.d), "qjl_signs": signs.reshape(*lead, self.qjl_dim),
                "residual_norm": rnorm.reshape(lead)}

    def dequantize(self, compressed: dict) -> torch.Tensor:
        return self.mse.dequantize(compressed["mse_indices"])

    def inner_product(self, y: torch.Tensor, compressed: dict) -> torch.Tensor:
        idx = compressed["mse_indices"]
        lead = idx.shape[:-1]
        idx2 = idx.reshape(-1, self.d)
        n = idx2.shape[0]
        y2 = y.reshape(-1, self.d)
        if y2.shape[0] != n:
            if y2.shape[0] == 1 or all(st == 0 for st in y.stride()[:-1]):
                y2 = y2[:1]
            else:
                raise ValueError(f"cannot pair {y2.shape[0]} query rows with {n} compressed vectors")
        elif y.dim() > 1 and n > 1 and all(st == 0 for st in y.stride()[:-1]):
            y2 = y2[:1]          # an expanded single query
        out = _ops.prod_inner_product(y2, idx2, compressed["qjl_signs"].reshape(n, self.qjl_dim),
                                      compressed["residual_norm"].reshape(n), self.mse.Pi, self.mse._cb, self._s_t)
        return out.reshape(lead if len(lead) else (1,)) if y.dim() > 1 or len(lead) else out.reshape(())

    def forward(self, x: torch.Tensor) -> dict:
        return self.quantize(x)


class TurboQuantKVCache:
    """Chunk-list KV cache: TurboQuantProd keys (inner products), TurboQuantMSE values."""

    def __init__(self, d_key: int, d_value: int, bits: int = 3, seed: int = 42, device: str = "cpu"):
        self.d_key = d_key
        self.d_value = d_value
        self.bits = bits
        self.device = device
        N.warn_if_not_cuda(device, "TurboQuantKVCache")
        self.key_quantizer = TurboQuantProd(d_key, bits, seed=seed, device=device)
        self.value_quantizer = TurboQuantMSE(d_value, bits, seed=seed + 100, device=device)
        self.key_cache = []
        self.value_cache = []

    def append(self, keys: torch.Tensor, values: torch.Tensor):
        packed = self.key_quantizer.quantize(keys.reshape(-1, self.d_key))
        packed["shape"] = keys.shape
        self.key_cache.append(packed)
        self.value_cache.append({"indices": self.value_quantizer.quantize(values.reshape(-1, self.d_value)),
                                 "shape": values.shape})

    def attention_scores(self, queries: torch.Tensor) -> torch.Tensor:
        parts = [self.key_quantizer.inner_product(queries, chunk) for chunk in self.key_cache]
        return torch.cat(parts, dim=-1) if parts else torch.tensor([])

    def get_values(self) -> torch.Tensor:
        parts = [self.value_quantizer.dequantize(chunk["indices"]) for chunk in self.value_cache]
        return torch.cat(parts, dim=0) if parts else torch.tensor([])

    def memory_usage_bits(self) -> dict:
        n_idx = sum(c["mse_indices"].numel() for c in self.key_cache)
        n_sign = sum(c["qjl_signs"].numel() for c in self.key_cache)
        n_norm = sum(c["residual_norm"].numel() for c in self.key_cache)
        n_val = sum(c["indices"].numel() for c in self.value_cache)
        key_bits = n_idx * self.key_quantizer.mse_bits + n_sign * 1 + n_norm * 16
        value_bits = n_val * self.bits
        total = key_bits + value_bits
        fp16 = (n_idx + n_val) * 16
        return {"key_bits": key_bits, "value_bits": value_bits, "total_bits": total, "fp16_bits": fp16,
                "compression_ratio": fp16 / total if total > 0 else 0}

    def __len__(self):
        return sum(c["mse_indices"].shape[0] for c in self.key_cache)
