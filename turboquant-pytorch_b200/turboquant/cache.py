"""Incremental packed KV cache: the caller of the compression path during generation.

Mirror of the reference's V3Cache (turboquant/generation_test_v2.py:48-166) without
its transformers base class: update(key_states, value_states, layer_idx) appends
the new tokens, compresses whatever has left the 16-bit residual window and returns
the layer's full keys and values in the cache dtype -- compressed tokens as their
reconstructions, recent tokens as they came.

The reference keeps a list of compressed chunks per layer and decompresses every
chunk again on every step.  Here each layer owns one preallocated (B, H, capacity, D)
buffer in the cache dtype that always holds what that concatenation would produce:
a token is quantised once, when it leaves the window, and its reconstruction is
written over its own slot by the dequantise kernel (strided output).  A decode step
therefore costs one quantise and one dequantise launch for the tokens that left
the window, independent of the context length.  The packed chunks are kept (they
are the compressed store, and MSECompressor.attention_scores reads them directly).
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from . import _ops
from .compressors_v3 import TurboQuantV3


class _Layer:
    __slots__ = ("codec", "k", "v", "total", "compressed", "chunks_k", "chunks_v")

    def __init__(self, codec):
        self.codec = codec
        self.k: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None
        self.total = 0
        self.compressed = 0
        self.chunks_k: List[dict] = []
        self.chunks_v: List[dict] = []


class V3Cache:
    """Compressed KV cache for autoregressive generation (reference: generation_test_v2.py:48-166).

    Same constructor arguments and the same update / get_seq_length / get_compression_info
    behaviour as the reference class.  The tensors returned by update() are views of the
    layer's persistent buffer: valid until the next update() of that layer, which is how
    attention layers use them.
    """

    def __init__(self, key_bits: int = 4, value_bits: int = 2, residual_window: int = 128,
                 protected_layers: int = 0, n_layers: int = 36, initial_capacity: int = 1024):
        self.key_bits = key_bits
        self.value_bits = value_bits
        self.residual_window = residual_window
        self.protected_layers = protected_layers
        self.n_layers = n_layers
        self.initial_capacity = initial_capacity
        self._layers: Dict[int, _Layer] = {}

    def _layer(self, layer_idx: int, head_dim: int, device) -> _Layer:
        st = self._layers.get(layer_idx)
        if st is None:
            codec = TurboQuantV3(head_dim=head_dim, key_bits=self.key_bits, value_bits=self.value_bits,
                                 residual_window=0, layer_idx=layer_idx, n_layers=self.n_layers,
                                 protected_layers=self.protected_layers, seed=42, device=device)
            st = self._layers[layer_idx] = _Layer(codec)
        return st

    @staticmethod
    def _grow(buf: Optional[torch.Tensor], like: torch.Tensor, used: int, need: int, initial: int) -> torch.Tensor:
        B, H, _, D = like.shape
        cap = 0 if buf is None else buf.shape[2]
        if need <= cap:
            return buf
        new_cap = max(initial, cap)
        while new_cap < need:
            new_cap *= 2
        new = torch.empty((B, H, new_cap, D), dtype=like.dtype, device=like.device)
        if buf is not None and used:
            new[:, :, :used].copy_(buf[:, :, :used])
        return new

    @torch.no_grad()
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs=None) -> Tuple[torch.Tensor, torch.Tensor]:
        B, H, S_new, D = key_states.shape
        st = self._layer(layer_idx, D, key_states.device)
        need = st.total + S_new
        st.k = self._grow(st.k, key_states, st.total, need, self.initial_capacity)
        st.v = self._grow(st.v, value_states, st.total, need, self.initial_capacity)
        st.k[:, :, st.total:need].copy_(key_states)
        st.v[:, :, st.total:need].copy_(value_states)
        st.total = need
        recent = st.total - st.compressed
        rw = self.residual_window
        n_c = recent if rw == 0 else max(0, recent - rw)       # tokens leaving the window now
        if n_c > 0:
            lo, hi = st.compressed, st.compressed + n_c
            view_k, view_v = st.k[:, :, lo:hi], st.v[:, :, lo:hi]
            kc, vc = st.codec.key_compressor, st.codec.val_compressor
            jk, rk, keep_k = kc.compress_job(view_k)
            jv, rv, keep_v = vc.compress_job(view_v)
            _ops.run_quantize([jk, jv], key_states.device)
            dk, keep_dk = kc.decompress_job(rk, view_k)         # reconstruction over the token's own slot
            dv, keep_dv = vc.decompress_job(rv, view_v)
            _ops.run_dequantize([dk, dv], key_states.device)
            st.chunks_k.append(rk)
            st.chunks_v.append(rv)
            st.compressed = hi
        return st.k[:, :, :st.total], st.v[:, :, :st.total]

    def get_seq_length(self, layer_idx: int = 0) -> int:
        st = self._layers.get(layer_idx)
        return st.total if st is not None else 0

    def get_compression_info(self) -> str:
        if not self._layers:
            return "no compression"
        st = self._layers.get(0)
        comp = st.compressed if st is not None else 0
        total = st.total if st is not None else 0
        return f"{comp} compressed, {total - comp} fp16, {total} total"

    # -- beyond the reference ---------------------------------------------------
    def packed_chunks(self, layer_idx: int):
        """The compressed store of a layer: lists of MSECompressor dicts for keys and values."""
        st = self._layers[layer_idx]
        return st.chunks_k, st.chunks_v

    def memory_bytes(self, layer_idx: int = 0) -> dict:
        """Bytes of the compressed representation (packed rows + norms + 16-bit window) vs a plain 16-bit cache."""
        st = self._layers[layer_idx]
        B, H, _, D = st.k.shape
        packed = sum(c["idx_bytes"].numel() + 2 * c["vec_norms"].numel() for c in st.chunks_k + st.chunks_v)
        window = 2 * B * H * (st.total - st.compressed) * D * st.k.element_size()
        dense = 2 * B * H * st.total * D * st.k.element_size()
        return {"compressed_bytes": packed + window, "fp16_bytes": dense,
                "compression_ratio": dense / (packed + window) if packed + window else 0}
