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
    def compress(self, states: torch.Tensor, packed: bool = False) -> dict:
        """The reference's dict ("k_mse" fp16, "qjl_signs" int8, "residual_norm" fp16, "shape"), or with packed=True
        the packed form of the same information (not in the reference, whose stored form is larger than the 16-bit
        keys; its own size accounting, turboquant/validate.py:120-134, assumes this layout):
          "mse_idx_bytes" (B,H,S,G) uint8   MSE indices, bit-packed as in compressors_v3.py:64-74
          "sign_bits"     (B,H,S,D/8) uint8 QJL signs, coordinate j in bit 7 - j % 8 of byte j / 8, set for +1
          "vec_norms"     (B,H,S) fp32      ||x||: k_mse = (centroids[idx] @ Pi) * vec_norms
          "residual_norm" (B,H,S) fp16, "shape", "packed": True
        asymmetric_attention_scores takes either form; unpack() turns the packed one into the reference's."""
        B, H, S, D = states.shape
        if not packed:
            k_mse, _idx, signs, rnorm = _ops.qjl_compress(states, self.Pi, self.PiT, self._cb, self._s_t, self.mse_bits,
                                                          normalize=True, want_k_mse=True, idx_mode=None,
                                                          signs_fp32=False, rnorm_fp32=False)
            return {"k_mse": k_mse.reshape(B, H, S, D), "qjl_signs": signs.reshape(B, H, S, D),
                    "residual_norm": rnorm.reshape(B, H, S), "shape": (B, H, S, D)}
        if D % 8:
            raise ValueError("packed=True needs head_dim to be a multiple of 8")
        rows, bits, rnorm, vnorm = _ops.qjl_compress_packed(states, self.Pi, self.PiT, self._cb, self._s_t, self.mse_bits)
        return {"mse_idx_bytes": rows.reshape(B, H, S, -1), "sign_bits": bits.reshape(B, H, S, D // 8),
                "vec_norms": vnorm.reshape(B, H, S), "residual_norm": rnorm.reshape(B, H, S), "shape": (B, H, S, D),
                "packed": True}

    @torch.no_grad()
    def unpack(self, packed: dict) -> dict:
        """The reference's dict from the packed form: signs and residual norms exactly, k_mse as
        fp16((centroids[idx] @ Pi) * vec_norms), which equals compress()'s k_mse up to the rounding of the product."""
        B, H, S, D = packed["shape"]
        ipb = 8 // self.mse_bits
        rows = packed["mse_idx_bytes"].reshape(B * H * S, -1).to(torch.int32)
        shifts = torch.tensor([self.mse_bits * (ipb - 1 - f) for f in range(ipb)], dtype=torch.int32, device=rows.device)
        idx = ((rows.unsqueeze(-1) >> shifts) & ((1 << self.mse_bits) - 1)).reshape(B * H * S, -1)[:, :D].to(torch.uint8)
        sb = packed["sign_bits"].reshape(B * H * S, D // 8).to(torch.int32)
        bit = (sb.unsqueeze(-1) >> torch.arange(7, -1, -1, dtype=torch.int32, device=sb.device)) & 1
        signs = (bit.reshape(B * H * S, D) * 2 - 1).to(torch.int8)
        k32 = torch.empty((1, 1, B * H * S, D), dtype=torch.float32, device=rows.device)
        job, _keep = _ops.dequantize_job(idx, None, (1, 1, B * H * S, D), self.Pi, self._cb, self.mse_bits, N.IDX_U8, k32)
        _ops.run_dequantize([job], rows.device)
        k_mse = (k32.reshape(B * H * S, D) * packed["vec_norms"].reshape(-1, 1)).to(torch.float16)
        return {"k_mse": k_mse.reshape(B, H, S, D), "qjl_signs": signs.reshape(B, H, S, D),
                "residual_norm": packed["residual_norm"], "shape": (B, H, S, D)}

    @staticmethod
    def stored_bytes(compressed: dict) -> int:
        """Bytes of the tensors of a compressed dict (either form)."""
        return sum(v.numel() * v.element_size() for v in compressed.values() if torch.is_tensor(v))

    @torch.no_grad()
    def asymmetric_attention_scores(self, queries: torch.Tensor, compressed: dict) -> torch.Tensor:
        if compressed.get("packed"):
            return _ops.qjl_scores_packed(queries, compressed["mse_idx_bytes"], compressed["sign_bits"],
                                          compressed["vec_norms"], compressed["residual_norm"], self.PiT, self._s_t,
                                          self._cb, self.mse_bits)
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
