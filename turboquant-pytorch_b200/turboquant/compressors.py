"""V2 API: TurboQuantCompressorV2 (MSE + QJL keys, asymmetric scores) and
TurboQuantCompressorMSE (values).  Drop-in for turboquant/compressors.py of the
reference; compress and the score estimator each run as one fused kernel chain.
"""

from __future__ import annotations

import torch

from . import _native as N
from . import _ops
from .lloyd_max import solve_codebook_v2
from .turboquant import generate_qjl_matrix, generate_rotation_matrix


class TurboQuantCompressorV2:
    """Stores k_mse (fp16), QJL signs (int8) and residual norms (fp16); scores without decompression."""

    def __init__(self, head_dim: int, bits: int, seed: int, device: str = "cpu"):
        self.head_dim = head_dim
        self.bits = bits
        self.mse_bits = max(bits - 1, 1)
        self.device = device
        N.warn_if_not_cuda(device, "TurboQuantCompressorV2")
        self.Pi = generate_rotation_matrix(head_dim, seed=seed, device=device)
        self.centroids = solve_codebook_v2(head_dim, self.mse_bits).to(device)
        self.S = generate_qjl_matrix(head_dim, m=head_dim, seed=seed + 10000, device=device)
        self.PiT = self.Pi.T.contiguous()
        self._s_t = self.S.T.contiguous()
        self._cb = N.codebook_block(self.centroids, self.mse_bits).to(device)

    @torch.no_grad()
    def compress(self, states: torch.Tensor) -> dict:
        B, H, S, D = states.shape
        k_mse, _idx, signs, rnorm = _ops.qjl_compress(states, self.Pi, self.PiT, self._cb, self._s_t, self.mse_bits,
                                                      normalize=True, want_k_mse=True, idx_mode=None,
                                                      signs_fp32=False, rnorm_fp32=False)
        return {"k_mse": k_mse.reshape(B, H, S, D), "qjl_signs": signs.reshape(B, H, S, D),
                "residual_norm": rnorm.reshape(B, H, S), "shape": (B, H, S, D)}

    @torch.no_grad()
    def asymmetric_attention_scores(self, queries: torch.Tensor, compressed: dict) -> torch.Tensor:
        return _ops.qjl_scores(queries, compressed["k_mse"], compressed["qjl_signs"], compressed["residual_norm"],
                               self._s_t)


class TurboQuantCompressorMSE:
    """MSE-only codec with one uint8 per index (no packing), for values."""

    def __init__(self, head_dim: int, bits: int, seed: int, device: str = "cpu"):
        self.head_dim = head_dim
        self.bits = bits
        self.device = device
        N.warn_if_not_cuda(device, "TurboQuantCompressorMSE")
        self.Pi = generate_rotation_matrix(head_dim, seed=seed, device=device)
        self.centroids = solve_codebook_v2(head_dim, bits).to(device)
        self._pi_t = self.Pi.T.contiguous()
        self._cb = N.codebook_block(self.centroids, bits).to(device)

    @torch.no_grad()
    def compress(self, states: torch.Tensor) -> dict:
        B, H, S, D = states.shape
        job, idx, norms, _keep = _ops.quantize_job(states, self._pi_t, self._cb, self.bits, True, N.IDX_U8)
        _ops.run_quantize([job], states.device)
        return {"indices": idx, "vec_norms": norms.reshape(-1), "shape": (B, H, S, D)}

    @torch.no_grad()
    def decompress(self, compressed: dict) -> torch.Tensor:
        B, H, S, D = compressed["shape"]
        out = torch.empty((B, H, S, D), dtype=torch.float32, device=compressed["indices"].device)
        job, _keep = _ops.dequantize_job(compressed["indices"], compressed["vec_norms"], (B, H, S, D), self.Pi,
                                         self._cb, self.bits, N.IDX_U8, out)
        _ops.run_dequantize([job], out.device)
        return out
