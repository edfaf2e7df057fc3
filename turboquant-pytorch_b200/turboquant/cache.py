"""Incremental packed KV cache: the caller of the compression path during generation.

Mirror of the reference's V3Cache (turboquant/generation_test_v2.py:48-166): a
transformers DynamicCache subclass (when transformers is importable; a plain object
otherwise) whose update(key_states, value_states, layer_idx) appends the new tokens,
compresses whatever has left the 16-bit residual window and returns the layer's full keys
and values in the cache dtype -- compressed tokens as their reconstructions, recent tokens
as they came.

The reference keeps a list of compressed chunks per layer and decompresses every chunk
again on every step.  Here each layer owns one preallocated (B, H, capacity, D) buffer in
the cache dtype that always holds what that concatenation would produce: a token is
quantised once, when it leaves the window, and its reconstruction is written over its own
slot by the dequantise kernel (strided output).  A decode step therefore costs work for the
tokens that left the window only, independent of the context length.  The packed rows are
kept (they are the compressed store; MSECompressor.attention_scores and
TurboQuantV3.decode_attention read them directly).

step(keys_by_layer, values_by_layer) does one token step for ALL layers with three library
calls (copy the new tokens in, quantise, dequantise) whatever the number of layers; update()
is the per-layer form the transformers attention modules call.
"""

from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _native as N
from .compressors_v3 import TurboQuantV3

try:                                                   # the reference class is a DynamicCache (generation_test_v2.py:48)
    from transformers.cache_utils import DynamicCache as _Base
    try:
        from transformers.cache_utils import DynamicLayer as _DynamicLayer
    except Exception:                                  # older transformers: no per-layer objects
        _DynamicLayer = None
except Exception:                                      # transformers absent: same behaviour, plain object
    _Base = object
    _DynamicLayer = None


class _Layer:
    __slots__ = ("codec", "k", "v", "total", "compressed", "packed")

    def __init__(self, codec):
        self.codec = codec
        self.k: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None
        self.total = 0
        self.compressed = 0
        # compressed store: [(first token, n tokens, k idx, k norms, v idx, v norms)], tensors laid out (B, H, n, ...)
        self.packed: List[tuple] = []


class V3Cache(_Base):
    """Compressed KV cache for autoregressive generation (reference: generation_test_v2.py:48-166).

    Same constructor arguments and the same update / get_seq_length / get_compression_info
    behaviour as the reference class.  The tensors returned by update() are views of the
    layer's persistent buffer: valid until the next update() of that layer, which is how
    attention layers use them.
    """

    def __init__(self, key_bits: int = 4, value_bits: int = 2, residual_window: int = 128,
                 protected_layers: int = 0, n_layers: int = 36, initial_capacity: int = 1024):
        if _Base is not object:
            super().__init__()
        self.key_bits = key_bits
        self.value_bits = value_bits
        self.residual_window = residual_window
        self.protected_layers = protected_layers
        self.n_layers = n_layers
        self.initial_capacity = initial_capacity
        self._layers: Dict[int, _Layer] = {}
        self._step_plan = None

    # ------------------------------------------------------------------ layers and buffers
    def _layer(self, layer_idx: int, head_dim: int, device) -> _Layer:
        st = self._layers.get(layer_idx)
        if st is None:
            codec = TurboQuantV3(head_dim=head_dim, key_bits=self.key_bits, value_bits=self.value_bits,
                                 residual_window=0, layer_idx=layer_idx, n_layers=self.n_layers,
                                 protected_layers=self.protected_layers, seed=42, device=device)
            st = self._layers[layer_idx] = _Layer(codec)
            self._step_plan = None
        if _DynamicLayer is not None and hasattr(self, "layers"):
            while len(self.layers) <= layer_idx:       # keeps the base class's per-layer bookkeeping in step
                self.layers.append(_DynamicLayer())
        return st

    def _grow(self, buf: Optional[torch.Tensor], like: torch.Tensor, used: int, need: int) -> torch.Tensor:
        B, H, _, D = like.shape
        cap = 0 if buf is None else buf.shape[2]
        if need <= cap:
            return buf
        new_cap = max(self.initial_capacity, cap)
        while new_cap < need:
            new_cap *= 2
        new = torch.empty((B, H, new_cap, D), dtype=like.dtype, device=like.device)
        if buf is not None and used:
            new[:, :, :used].copy_(buf[:, :, :used])
        self._step_plan = None
        return new

    def _leaving(self, st: _Layer, need: int) -> int:
        """Tokens that leave the 16-bit window when the layer holds `need` tokens."""
        recent = need - st.compressed
        rw = self.residual_window
        return recent if rw == 0 else max(0, recent - rw)

    # ------------------------------------------------------------------ per-layer update (reference API)
    @torch.no_grad()
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs=None) -> Tuple[torch.Tensor, torch.Tensor]:
        from . import _ops
        B, H, S_new, D = key_states.shape
        st = self._layer(layer_idx, D, key_states.device)
        need = st.total + S_new
        st.k = self._grow(st.k, key_states, st.total, need)
        st.v = self._grow(st.v, value_states, st.total, need)
        st.k[:, :, st.total:need].copy_(key_states)
        st.v[:, :, st.total:need].copy_(value_states)
        st.total = need
        n_c = self._leaving(st, need)
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
            st.packed.append((lo, n_c, rk["idx_bytes"], rk["vec_norms"], rv["idx_bytes"], rv["vec_norms"]))
            st.compressed = hi
        return st.k[:, :, :st.total], st.v[:, :, :st.total]

    # ------------------------------------------------------------------ one step for all layers
    def _build_step_plan(self, L: int, like: torch.Tensor):
        """Persistent job arrays for step(): everything that does not change from step to step is filled in once."""
        sts = [self._layers[l] for l in range(L)]
        B, H, _, D = like.shape
        eb = like.element_size()
        q = (N.QuantizeJob * (2 * L))()
        d = (N.DequantizeJob * (2 * L))()
        c = (N.CopyJob * (2 * L))()
        row_bytes = []
        for l, st in enumerate(sts):
            for j, (buf, comp, bits) in enumerate(((st.k, st.codec.key_compressor, st.codec.key_bits),
                                                   (st.v, st.codec.val_compressor, st.codec.value_bits))):
                i = 2 * l + j
                g = N.packed_row_bytes(D, bits)
                row_bytes.append(g)
                q[i] = N.QuantizeJob(x=0, x_dtype=N.dtype_code(buf), D=D, bits=bits, normalize=1, B=B, H=H, S=0,
                                     stride_b=buf.stride(0), stride_h=buf.stride(1), stride_s=buf.stride(2),
                                     rotation_t=comp._pi_t.data_ptr(), codebook=comp._cb.data_ptr(),
                                     idx_mode=N.IDX_PACKED, reserved=0, idx_out=0, norms_out=0,
                                     rotation_image=comp._img_q.data_ptr() if comp._img_q is not None else None)
                d[i] = N.DequantizeJob(idx=0, norms=0, idx_mode=N.IDX_PACKED, D=D, bits=bits, out_dtype=N.dtype_code(buf),
                                       B=B, H=H, S=0, out=0, ostride_b=buf.stride(0), ostride_h=buf.stride(1),
                                       ostride_s=buf.stride(2), rotation=comp.Pi.data_ptr(), codebook=comp._cb.data_ptr(),
                                       rotation_image=comp._img_d.data_ptr() if comp._img_d is not None else None)
                c[i] = N.CopyJob(src=0, dst=0, elem_bytes=eb, D=D, B=B, H=H, S=0, sstride_b=0, sstride_h=0, sstride_s=0,
                                 dstride_b=buf.stride(0), dstride_h=buf.stride(1), dstride_s=buf.stride(2))
        base = [(st.k.data_ptr(), st.v.data_ptr()) for st in sts]
        cap = min(min(st.k.shape[2], st.v.shape[2]) for st in sts)
        return {"L": L, "B": B, "H": H, "D": D, "eb": eb, "dtype": like.dtype, "device": like.device, "q": q, "d": d, "c": c,
                "row_bytes": row_bytes, "base": base, "cap": cap, "tok_bytes": D * eb}

    @torch.no_grad()
    def step(self, key_states: Sequence[torch.Tensor], value_states: Sequence[torch.Tensor], return_views: bool = True):
        """One step for layers 0..L-1 at once: append key_states[l] / value_states[l] ((B, H, S_new, D) each) to
        layer l, quantise what left the window and put its reconstruction in place.  Three library calls in all.

        Returns [(keys, values)] per layer as update() would (views of the persistent buffers), or None with
        return_views=False.  Falls back to per-layer update() calls while layers are being created or grown."""
        L = len(key_states)
        k0 = key_states[0]
        B, H, S_new, D = k0.shape
        dev = k0.device
        eb = k0.element_size()
        ready = all(l in self._layers and self._layers[l].k is not None for l in range(L))
        if ready:
            if self._step_plan is None or self._step_plan["L"] != L:
                self._step_plan = self._build_step_plan(L, self._layers[0].k)
            p = self._step_plan
            ready = (p["B"], p["H"], p["D"], p["dtype"], p["device"]) == (B, H, D, k0.dtype, dev) and \
                all(self._layers[l].total + S_new <= p["cap"] for l in range(L)) and (D * eb) % 16 == 0
        if not ready:
            outs = [self.update(key_states[l], value_states[l], l) for l in range(L)]
            return outs if return_views else None
        p = self._step_plan
        q, d, c, rowb, base, tokb = p["q"], p["d"], p["c"], p["row_bytes"], p["base"], p["tok_bytes"]
        # one allocation for this step's packed rows and norms of every layer
        n_cs = [self._leaving(self._layers[l], self._layers[l].total + S_new) for l in range(L)]
        slabs = B * H
        sizes = []
        for l in range(L):
            n = slabs * n_cs[l]
            for j in range(2):
                sizes.append(((n * rowb[2 * l + j] + 15) // 16 * 16, (2 * n + 15) // 16 * 16))
        total_bytes = sum(a + b for a, b in sizes)
        store = torch.empty(max(total_bytes, 16), dtype=torch.uint8, device=dev) if total_bytes else None
        sp = store.data_ptr() if store is not None else 0
        off = 0
        for l in range(L):
            st = self._layers[l]
            n_c = n_cs[l]
            offsets = []
            for j, x in enumerate((key_states[l], value_states[l])):
                i = 2 * l + j
                cj = c[i]
                cj.src = x.data_ptr()
                cj.S = S_new
                cj.sstride_b, cj.sstride_h, cj.sstride_s = x.stride(0), x.stride(1), x.stride(2)
                cj.dst = base[l][j] + st.total * tokb
                slot = base[l][j] + st.compressed * tokb
                qj, dj = q[i], d[i]
                qj.S = dj.S = n_c
                qj.x = dj.out = slot
                a, b = sizes[i]
                qj.idx_out = dj.idx = sp + off
                qj.norms_out = dj.norms = sp + off + a
                offsets += [off, off + a]
                off += a + b
            if n_c > 0:
                st.packed.append((st.compressed, n_c, store, tuple(offsets)))     # views are made on demand
            st.total += S_new
            st.compressed += n_c
        lib = N.lib()
        stream = N.stream_ptr(dev)
        with torch.cuda.device(dev):
            N.check(lib.tq_copy_rows(c, 2 * L, stream), "tq_copy_rows")
            if total_bytes:
                N.check(lib.tq_quantize(q, 2 * L, stream), "tq_quantize")
                N.check(lib.tq_dequantize(d, 2 * L, stream), "tq_dequantize")
        if not return_views:
            return None
        return [(self._layers[l].k[:, :, :self._layers[l].total], self._layers[l].v[:, :, :self._layers[l].total])
                for l in range(L)]

    # ------------------------------------------------------------------ reference accessors
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

    # ------------------------------------------------------------------ beyond the reference
    def _chunk_tensors(self, st: _Layer, entry):
        """(first token, n, k idx, k norms, v idx, v norms) of one compressed-store entry, as (B, H, n, ...) tensors."""
        if len(entry) == 6:
            return entry
        lo, n, store, (ok_idx, ok_nrm, ov_idx, ov_nrm) = entry            # a step's shared store and byte offsets
        B, H, _, D = st.k.shape
        gk = N.packed_row_bytes(D, st.codec.key_bits)
        gv = N.packed_row_bytes(D, st.codec.value_bits)
        rows = B * H * n
        k_idx = store[ok_idx:ok_idx + rows * gk].view(B, H, n, gk)
        k_nrm = store[ok_nrm:ok_nrm + 2 * rows].view(torch.float16).view(B, H, n)
        v_idx = store[ov_idx:ov_idx + rows * gv].view(B, H, n, gv)
        v_nrm = store[ov_nrm:ov_nrm + 2 * rows].view(torch.float16).view(B, H, n)
        return lo, n, k_idx, k_nrm, v_idx, v_nrm

    def packed_chunks(self, layer_idx: int):
        """The compressed store of a layer: lists of MSECompressor dicts for keys and values, in token order."""
        st = self._layers[layer_idx]
        B, H, _, D = st.k.shape
        cks, cvs = [], []
        for entry in st.packed:
            _lo, n, k_idx, k_nrm, v_idx, v_nrm = self._chunk_tensors(st, entry)
            cks.append({"idx_bytes": k_idx, "vec_norms": k_nrm, "shape": (B, H, n, D), "idx_pad": 0})
            cvs.append({"idx_bytes": v_idx, "vec_norms": v_nrm, "shape": (B, H, n, D), "idx_pad": 0})
        return cks, cvs

    def packed_layer(self, layer_idx: int):
        """(compressed_k, compressed_v) of a layer in the form TurboQuantV3.compress_kv returns: all packed tokens as
        one MSECompressor dict each, the window tokens as views of the persistent buffers.  What
        TurboQuantV3.decode_attention takes."""
        st = self._layers[layer_idx]
        B, H, _, D = st.k.shape
        cks, cvs = self.packed_chunks(layer_idx)
        out = []
        for chunks, buf in ((cks, st.k), (cvs, st.v)):
            comp = None
            if chunks:
                comp = {"idx_bytes": torch.cat([ch["idx_bytes"] for ch in chunks], dim=2),
                        "vec_norms": torch.cat([ch["vec_norms"] for ch in chunks], dim=2),
                        "shape": (B, H, st.compressed, D), "idx_pad": 0}
            out.append({"compressed": comp, "fp16": buf[:, :, st.compressed:st.total], "shape": (B, H, st.total, D),
                        "split_at": st.compressed})
        return tuple(out)

    def memory_bytes(self, layer_idx: int = 0) -> dict:
        """Bytes of the compressed representation (packed rows + norms + 16-bit window) vs a plain 16-bit cache."""
        st = self._layers[layer_idx]
        B, H, _, D = st.k.shape
        packed = B * H * st.compressed * (N.packed_row_bytes(D, st.codec.key_bits) + 2 +
                                          N.packed_row_bytes(D, st.codec.value_bits) + 2)
        window = 2 * B * H * (st.total - st.compressed) * D * st.k.element_size()
        dense = 2 * B * H * st.total * D * st.k.element_size()
        return {"compressed_bytes": packed + window, "fp16_bytes": dense,
                "compression_ratio": dense / (packed + window) if packed + window else 0}

    # ------------------------------------------------------------------ persistence
    def cache_state(self) -> dict:
        """Everything needed to continue generation later, as plain tensors and numbers (torch.save-able): per layer
        the tokens so far in the cache dtype (reconstructions + window), the counters and the packed store."""
        layers = {}
        for l, st in self._layers.items():
            ck, cv = self.packed_layer(l)
            layers[l] = {"k": st.k[:, :, :st.total].clone(), "v": st.v[:, :, :st.total].clone(), "total": st.total,
                         "compressed": st.compressed,
                         "packed_k": None if ck["compressed"] is None else {k: (v.clone() if torch.is_tensor(v) else v)
                                                                            for k, v in ck["compressed"].items()},
                         "packed_v": None if cv["compressed"] is None else {k: (v.clone() if torch.is_tensor(v) else v)
                                                                            for k, v in cv["compressed"].items()}}
        return {"config": {"key_bits": self.key_bits, "value_bits": self.value_bits, "residual_window": self.residual_window,
                           "protected_layers": self.protected_layers, "n_layers": self.n_layers,
                           "initial_capacity": self.initial_capacity}, "layers": layers}

    @classmethod
    def from_cache_state(cls, state: dict, device=None) -> "V3Cache":
        """Rebuild a cache from cache_state() (constants are re-derived from the constructor arguments)."""
        cache = cls(**state["config"])
        for l, s in sorted(state["layers"].items()):
            k = s["k"].to(device) if device is not None else s["k"]
            v = s["v"].to(device) if device is not None else s["v"]
            st = cache._layer(l, k.shape[-1], k.device)
            st.k = cache._grow(None, k, 0, s["total"])
            st.v = cache._grow(None, v, 0, s["total"])
            st.k[:, :, :s["total"]].copy_(k)
            st.v[:, :, :s["total"]].copy_(v)
            st.total, st.compressed = s["total"], s["compressed"]
            if s["packed_k"] is not None:
                pk, pv = s["packed_k"], s["packed_v"]
                mv = (lambda t: t.to(device)) if device is not None else (lambda t: t)
                st.packed.append((0, s["compressed"], mv(pk["idx_bytes"]), mv(pk["vec_norms"]), mv(pv["idx_bytes"]),
                                  mv(pv["vec_norms"])))
        return cache
