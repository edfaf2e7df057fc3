"""CPU oracle for the TurboQuant KV-cache compression hot path.

TEST INFRASTRUCTURE ONLY.  This module is a CPU restatement of the reference
algorithm (tonbistudio/turboquant-pytorch); it exists to check the CUDA path and
to be timed as the CPU baseline.  Nothing in the shipped package imports it.

Parity status: PINNED.  Every function below is checked against golden vectors
that were produced by importing the reference itself (tests/golden/make_golden.py
records how), see tests/test_oracle_golden.py.

The floating-point steps use the same torch CPU operators, in the same order, as
the reference (norm -> divide -> matmul -> |y-c| argmin), so that on one machine
the oracle and the reference agree bit for bit.  The byte/integer steps (bit
packing, unpacking) are restated in numpy.  The only structural difference is
that the (N, D, 2^bits) distance tensor is evaluated in row chunks, which does
not change any value.

Citations are file:line in the reference tree (turboquant/...).
"""

from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

# --------------------------------------------------------------------------- #
# Constants built at construction time
# --------------------------------------------------------------------------- #


def rotation_matrix(d: int, seed: Optional[int]) -> torch.Tensor:
    """Haar rotation Pi = Q * sign(diag R) from the QR of a seeded Gaussian.

    Follows turboquant/turboquant.py:18-33 (the same code is inlined in
    turboquant/compressors.py:37-43 and :167-173).
    """
    g = torch.Generator(device="cpu")
    if seed is not None:
        g.manual_seed(seed)
    gauss = torch.randn(d, d, generator=g)
    q, r = torch.linalg.qr(gauss)
    s = torch.sign(torch.diag(r))
    s[s == 0] = 1.0
    return q * s.unsqueeze(0)


def qjl_matrix(d: int, m: Optional[int], seed: Optional[int]) -> torch.Tensor:
    """Gaussian projection S (m, d).  turboquant/turboquant.py:36-48."""
    if m is None:
        m = d
    g = torch.Generator(device="cpu")
    if seed is not None:
        g.manual_seed(seed)
    return torch.randn(m, d, generator=g)


def _coordinate_pdf(d: int, exact: bool):
    """pdf of one coordinate of a rotated unit vector.

    Gaussian N(0, 1/d): turboquant/lloyd_max.py:26-29.  Exact Beta form:
    turboquant/lloyd_max.py:18-23.
    """
    if exact:
        coeff = math.gamma(d / 2) / (math.sqrt(math.pi) * math.gamma((d - 1) / 2))

        def pdf(x):
            if abs(x) >= 1.0:
                return 0.0
            return coeff * (1 - x * x) ** ((d - 3) / 2)

        return pdf
    sigma2 = 1.0 / d
    norm = 1.0 / math.sqrt(2 * math.pi * sigma2)

    def pdf(x):
        return norm * math.exp(-x * x / (2 * sigma2))

    return pdf


def lloyd_max(d: int, bits: int, use_exact: bool = False, max_iter: int = 200, tol: float = 1e-10):
    """Lloyd-Max fixed point; returns (centroids fp32 [L], boundaries fp32 [L-1]).

    turboquant/lloyd_max.py:32-86.  The last computed iterate is the one
    returned (the assignment precedes the convergence test, :72-78).
    """
    from scipy import integrate

    levels = 2 ** bits
    pdf = _coordinate_pdf(d, use_exact)
    sigma = 1.0 / math.sqrt(d)
    lo, hi = -3.5 * sigma, 3.5 * sigma
    cent = [lo + (hi - lo) * (i + 0.5) / levels for i in range(levels)]
    for _ in range(max_iter):
        mids = [(cent[i] + cent[i + 1]) / 2.0 for i in range(levels - 1)]
        edges = [lo * 3] + mids + [hi * 3]
        new = []
        for i in range(levels):
            a, b = edges[i], edges[i + 1]
            num, _e = integrate.quad(lambda x: x * pdf(x), a, b)
            den, _e = integrate.quad(pdf, a, b)
            new.append(num / den if den > 1e-15 else cent[i])
        shift = max(abs(new[i] - cent[i]) for i in range(levels))
        cent = new
        if shift < tol:
            break
    mids = [(cent[i] + cent[i + 1]) / 2.0 for i in range(levels - 1)]
    return torch.tensor(cent, dtype=torch.float32), torch.tensor(mids, dtype=torch.float32)


def lloyd_max_v2(d: int, bits: int) -> torch.Tensor:
    """The codebook solver inlined in the V2 compressors.

    turboquant/compressors.py:57-81 and :178-198.  It differs from lloyd_max in
    two ways: the pdf is written with sigma**2, and on convergence it breaks
    BEFORE adopting the newest iterate (:77-79).
    """
    from scipy import integrate

    levels = 2 ** bits
    sigma = 1.0 / math.sqrt(d)

    def pdf(x):
        return (1.0 / math.sqrt(2 * math.pi * sigma ** 2)) * math.exp(-x * x / (2 * sigma ** 2))

    lo, hi = -3.5 * sigma, 3.5 * sigma
    cent = [lo + (hi - lo) * (i + 0.5) / levels for i in range(levels)]
    for _ in range(200):
        mids = [(cent[i] + cent[i + 1]) / 2.0 for i in range(levels - 1)]
        edges = [lo * 3] + mids + [hi * 3]
        new = []
        for i in range(levels):
            a, b = edges[i], edges[i + 1]
            num, _e = integrate.quad(lambda x: x * pdf(x), a, b)
            den, _e = integrate.quad(pdf, a, b)
            new.append(num / den if den > 1e-15 else cent[i])
        if max(abs(new[i] - cent[i]) for i in range(levels)) < 1e-10:
            break
        cent = new
    return torch.tensor(cent, dtype=torch.float32)


def expected_distortion(d: int, bits: int, centroids: torch.Tensor, boundaries: torch.Tensor,
                        use_exact: bool = False) -> float:
    """Per-coordinate expected squared error.  turboquant/lloyd_max.py:89-104."""
    from scipy import integrate

    pdf = _coordinate_pdf(d, use_exact)
    sigma = 1.0 / math.sqrt(d)
    edges = [-3.5 * sigma * 3] + boundaries.tolist() + [3.5 * sigma * 3]
    total = 0.0
    for i in range(len(centroids)):
        c = centroids[i].item()
        part, _e = integrate.quad(lambda x: (x - c) ** 2 * pdf(x), edges[i], edges[i + 1])
        total += part
    return total


# --------------------------------------------------------------------------- #
# Integer / byte stages
# --------------------------------------------------------------------------- #


def nearest_centroid(y: torch.Tensor, centroids: torch.Tensor, rows_per_chunk: int = 2048) -> torch.Tensor:
    """argmin_k |y - c_k| in fp32, first minimum wins; returns int64 like torch.

    turboquant/compressors_v3.py:60-61, turboquant/turboquant.py:84-85,
    turboquant/lloyd_max.py:117-121.  Evaluated in row chunks.
    """
    flat = y.reshape(-1, y.shape[-1]) if y.dim() > 1 else y.reshape(1, -1)
    out = torch.empty(flat.shape, dtype=torch.int64)
    for s in range(0, flat.shape[0], rows_per_chunk):
        blk = flat[s:s + rows_per_chunk]
        out[s:s + rows_per_chunk] = (blk.unsqueeze(-1) - centroids).abs().argmin(dim=-1)
    return out.reshape(y.shape)


def indices_per_byte(bits: int) -> int:
    """8 // bits.  turboquant/compressors_v3.py:64."""
    return 8 // bits


def pack_indices(idx: np.ndarray, bits: int):
    """(N, D) small ints -> ((N, G) uint8, idx_pad).  MSB-first within a byte.

    turboquant/compressors_v3.py:64-74: right-pad each row with zero indices to
    a multiple of ipb, then byte = sum_i idx[g*ipb+i] << (bits*(ipb-1-i)).
    """
    idx = np.asarray(idx).astype(np.int64)
    n, d = idx.shape
    ipb = indices_per_byte(bits)
    pad = (ipb - d % ipb) % ipb
    if pad:
        idx = np.concatenate([idx, np.zeros((n, pad), dtype=np.int64)], axis=1)
    groups = idx.shape[1] // ipb
    acc = np.zeros((n, groups), dtype=np.int64)
    view = idx.reshape(n, groups, ipb)
    for i in range(ipb):
        acc += view[:, :, i] << (bits * (ipb - 1 - i))
    return (acc & 0xFF).astype(np.uint8), pad


def unpack_indices(packed: np.ndarray, bits: int, d: int) -> np.ndarray:
    """(N, G) uint8 -> (N, D) int64.  turboquant/compressors_v3.py:92-101."""
    packed = np.asarray(packed).astype(np.int64)
    n, groups = packed.shape
    ipb = indices_per_byte(bits)
    mask = (1 << bits) - 1
    out = np.empty((n, groups, ipb), dtype=np.int64)
    for i in range(ipb):
        out[:, :, i] = (packed >> (bits * (ipb - 1 - i))) & mask
    return out.reshape(n, groups * ipb)[:, :d]


# --------------------------------------------------------------------------- #
# V3: MSECompressor / TurboQuantV3
# --------------------------------------------------------------------------- #


def rotate_unit(states: torch.Tensor, pi: torch.Tensor):
    """(…, D) -> (flat fp32 (N,D), norms fp32 (N,), rotated unit vectors (N,D)).

    turboquant/compressors_v3.py:52-59.
    """
    d = states.shape[-1]
    flat = states.reshape(-1, d).float()
    norms = torch.norm(flat, dim=-1)
    unit = flat / (norms.unsqueeze(-1) + 1e-8)
    return flat, norms, unit @ pi.T


def mse_compress(states: torch.Tensor, pi: torch.Tensor, centroids: torch.Tensor, bits: int) -> dict:
    """MSECompressor.compress.  turboquant/compressors_v3.py:45-81."""
    b, h, s, d = states.shape
    _flat, norms, rot = rotate_unit(states, pi)
    idx = nearest_centroid(rot, centroids)
    packed, pad = pack_indices(idx.numpy(), bits)
    return {
        "idx_bytes": torch.from_numpy(packed).reshape(b, h, s, packed.shape[1]),
        "vec_norms": norms.to(torch.float16).reshape(b, h, s),
        "shape": (b, h, s, d),
        "idx_pad": pad,
    }


def mse_decompress(comp: dict, pi: torch.Tensor, centroids: torch.Tensor, bits: int) -> torch.Tensor:
    """MSECompressor.decompress -> fp32 (B,H,S,D).  turboquant/compressors_v3.py:83-105."""
    b, h, s, d = comp["shape"]
    n = b * h * s
    packed = comp["idx_bytes"].reshape(n, -1).numpy()
    norms = comp["vec_norms"].reshape(n, 1).float()
    idx = torch.from_numpy(unpack_indices(packed, bits, d))
    return ((centroids[idx] @ pi) * norms).reshape(b, h, s, d)


def mse_memory_bytes(head_dim: int, bits: int, b: int, h: int, s: int) -> dict:
    """turboquant/compressors_v3.py:107-120."""
    n = b * h * s
    comp = n * math.ceil(head_dim / indices_per_byte(bits)) + n * 2
    fp16 = n * head_dim * 2
    return {"compressed_bytes": comp, "fp16_bytes": fp16,
            "compression_ratio": fp16 / comp if comp > 0 else 0}


def v3_effective_bits(key_bits, value_bits, layer_idx, n_layers, protected_layers, protected_bits):
    """Layer-adaptive widths, capped at 8.  turboquant/compressors_v3.py:157-164."""
    prot = layer_idx < protected_layers or layer_idx >= (n_layers - protected_layers)
    kb = protected_bits if prot else key_bits
    vb = protected_bits if prot else value_bits
    return min(kb, 8), min(vb, 8)


def v3_seeds(seed: int, layer_idx: int):
    """(key seed, value seed).  turboquant/compressors_v3.py:166-168."""
    base = seed + layer_idx * 1000
    return base, base + 500


class V3Oracle:
    """Function bundle standing in for TurboQuantV3 (turboquant/compressors_v3.py:123-265)."""

    def __init__(self, head_dim, key_bits=4, value_bits=2, residual_window=128, layer_idx=0,
                 n_layers=36, protected_layers=4, protected_bits=8, seed=42, codebook_cache=None):
        self.head_dim = head_dim
        self.residual_window = residual_window
        self.key_bits, self.value_bits = v3_effective_bits(
            key_bits, value_bits, layer_idx, n_layers, protected_layers, protected_bits)
        ks, vs = v3_seeds(seed, layer_idx)
        self.k_pi, self.v_pi = rotation_matrix(head_dim, ks), rotation_matrix(head_dim, vs)
        cache = codebook_cache if codebook_cache is not None else {}
        for bits in (self.key_bits, self.value_bits):
            if (head_dim, bits) not in cache:
                cache[(head_dim, bits)] = lloyd_max(head_dim, bits)[0]
        self.k_cent = cache[(head_dim, self.key_bits)]
        self.v_cent = cache[(head_dim, self.value_bits)]

    def compress_kv(self, keys, values):
        """turboquant/compressors_v3.py:170-212."""
        b, h, s, d = keys.shape
        rw = self.residual_window
        if s <= rw:
            return ({"fp16": keys, "compressed": None, "shape": (b, h, s, d), "split_at": s},
                    {"fp16": values, "compressed": None, "shape": (b, h, s, d), "split_at": s})
        cut = s - rw
        ck = {"compressed": mse_compress(keys[:, :, :cut, :], self.k_pi, self.k_cent, self.key_bits),
              "fp16": keys[:, :, cut:, :], "shape": (b, h, s, d), "split_at": cut}
        cv = {"compressed": mse_compress(values[:, :, :cut, :], self.v_pi, self.v_cent, self.value_bits),
              "fp16": values[:, :, cut:, :], "shape": (b, h, s, d), "split_at": cut}
        return ck, cv

    def decompress_kv(self, ck, cv):
        """turboquant/compressors_v3.py:214-233."""
        if ck["compressed"] is None:
            return ck["fp16"], cv["fp16"]
        old_k = mse_decompress(ck["compressed"], self.k_pi, self.k_cent, self.key_bits)
        old_v = mse_decompress(cv["compressed"], self.v_pi, self.v_cent, self.value_bits)
        dt = ck["fp16"].dtype
        return (torch.cat([old_k.to(dt), ck["fp16"]], dim=2),
                torch.cat([old_v.to(dt), cv["fp16"]], dim=2))

    def memory_bytes(self, b, h, s):
        """turboquant/compressors_v3.py:235-265."""
        rw = min(self.residual_window, s)
        cs = max(s - rw, 0)
        comp = 0
        if cs > 0:
            comp = (mse_memory_bytes(self.head_dim, self.key_bits, b, h, cs)["compressed_bytes"]
                    + mse_memory_bytes(self.head_dim, self.value_bits, b, h, cs)["compressed_bytes"])
        window = b * h * rw * self.head_dim * 2 * 2
        total = comp + window
        full = b * h * s * self.head_dim * 2 * 2
        return {"compressed_bytes": total, "fp16_bytes": full,
                "compression_ratio": full / total if total > 0 else 0,
                "compressed_tokens": cs, "fp16_tokens": rw,
                "key_bits": self.key_bits, "value_bits": self.value_bits}


class V3CacheOracle:
    """The incremental cache the reference's generation harness wraps around TurboQuantV3
    (turboquant/generation_test_v2.py:48-166), without the transformers base class: a list of
    compressed chunks plus a list of recent 16-bit tokens per layer; every update decompresses
    all chunks and concatenates."""

    def __init__(self, key_bits=4, value_bits=2, residual_window=128, protected_layers=0, n_layers=36):
        self.key_bits, self.value_bits = key_bits, value_bits
        self.residual_window = residual_window
        self.protected_layers, self.n_layers = protected_layers, n_layers
        self._codec, self._chunks, self._recent = {}, {}, {}
        self._total, self._compressed = {}, {}
        self._codebooks = {}

    def update(self, key_states, value_states, layer_idx):
        """generation_test_v2.py:80-152."""
        d = key_states.shape[-1]
        if layer_idx not in self._codec:                      # :64-78, residual_window=0 inside the codec
            self._codec[layer_idx] = V3Oracle(d, self.key_bits, self.value_bits, residual_window=0,
                                              layer_idx=layer_idx, n_layers=self.n_layers,
                                              protected_layers=self.protected_layers, seed=42,
                                              codebook_cache=self._codebooks)
            self._chunks[layer_idx], self._recent[layer_idx] = [], []
            self._total[layer_idx] = self._compressed[layer_idx] = 0
        codec = self._codec[layer_idx]
        self._total[layer_idx] += key_states.shape[2]
        self._recent[layer_idx].append((key_states, value_states))
        rk = torch.cat([k for k, _ in self._recent[layer_idx]], dim=2)
        rv = torch.cat([v for _, v in self._recent[layer_idx]], dim=2)
        rw = self.residual_window
        if rw == 0:                                           # :104-112
            if rk.shape[2] > 0:
                self._chunks[layer_idx].append(codec.compress_kv(rk, rv))
                self._compressed[layer_idx] += rk.shape[2]
                self._recent[layer_idx] = []
        elif rk.shape[2] > rw:                                # :113-127
            over = rk.shape[2] - rw
            self._chunks[layer_idx].append(codec.compress_kv(rk[:, :, :over, :], rv[:, :, :over, :]))
            self._compressed[layer_idx] += over
            self._recent[layer_idx] = [(rk[:, :, over:, :], rv[:, :, over:, :])]
        parts_k, parts_v = [], []                             # :129-146
        for ck, cv in self._chunks[layer_idx]:
            dk, dv = codec.decompress_kv(ck, cv)
            parts_k.append(dk.to(key_states.dtype))
            parts_v.append(dv.to(value_states.dtype))
        if self._recent[layer_idx]:
            parts_k.append(torch.cat([k for k, _ in self._recent[layer_idx]], dim=2))
            parts_v.append(torch.cat([v for _, v in self._recent[layer_idx]], dim=2))
        return torch.cat(parts_k, dim=2), torch.cat(parts_v, dim=2)

    def get_seq_length(self, layer_idx=0):
        return self._total.get(layer_idx, 0)

    def get_compression_info(self):
        """generation_test_v2.py:157-165."""
        if not self._compressed:
            return "no compression"
        comp, total = self._compressed.get(0, 0), self._total.get(0, 0)
        return f"{comp} compressed, {total - comp} fp16, {total} total"


def v3_scores(queries: torch.Tensor, keys_recon: torch.Tensor) -> torch.Tensor:
    """Attention logits on reconstructed keys.  turboquant/validate_v3.py:86-87.

    queries (B, Hq, Sq, D); keys_recon (B, Hkv, Sk, D) with Hq a multiple of Hkv
    (query head g reads KV head g // (Hq // Hkv), the usual grouped-query
    layout; the reference script expands KV heads the same way before :87).
    """
    b, hq, sq, d = queries.shape
    hkv = keys_recon.shape[1]
    rep = hq // hkv
    k = keys_recon.float().repeat_interleave(rep, dim=1) if rep > 1 else keys_recon.float()
    return torch.matmul(queries.float(), k.transpose(-2, -1))


def v3_decode_attention(queries: torch.Tensor, keys_full: torch.Tensor, values_full: torch.Tensor,
                        scale: float) -> torch.Tensor:
    """Attention on what TurboQuantV3.decompress_kv returns: softmax(scale * q K^T) V, fp32.

    The composition the generation harness performs after decompressing every chunk
    (turboquant/generation_test_v2.py:131-147 feeding the model's attention): scores as in
    turboquant/validate_v3.py:86-87, values from turboquant/compressors_v3.py:83-105.
    queries (B, Hq, Sq, D); keys_full / values_full (B, Hkv, S, D); grouped-query layout as v3_scores.
    """
    logits = v3_scores(queries, keys_full).double() * scale
    probs = torch.softmax(logits, dim=-1)
    rep = queries.shape[1] // values_full.shape[1]
    v = values_full.double().repeat_interleave(rep, dim=1) if rep > 1 else values_full.double()
    return torch.matmul(probs, v).float()


# --------------------------------------------------------------------------- #
# V2: MSE + QJL
# --------------------------------------------------------------------------- #


def v2_compress(states: torch.Tensor, pi: torch.Tensor, centroids: torch.Tensor, s_mat: torch.Tensor) -> dict:
    """TurboQuantCompressorV2.compress.  turboquant/compressors.py:83-120."""
    b, h, s, d = states.shape
    flat = states.reshape(-1, d).float()
    norms = torch.norm(flat, dim=-1, keepdim=True)
    unit = flat / (norms + 1e-8)
    rot = unit @ pi.T
    idx = nearest_centroid(rot, centroids)
    k_mse = (centroids[idx] @ pi) * norms
    resid = flat - k_mse
    r_norm = torch.norm(resid, dim=-1)
    proj = resid @ s_mat.T
    signs = (proj >= 0).to(torch.int8) * 2 - 1
    return {"k_mse": k_mse.to(torch.float16).reshape(b, h, s, d),
            "qjl_signs": signs.reshape(b, h, s, d),
            "residual_norm": r_norm.to(torch.float16).reshape(b, h, s),
            "shape": (b, h, s, d)}


def v2_scores(queries: torch.Tensor, comp: dict, s_mat: torch.Tensor) -> torch.Tensor:
    """asymmetric_attention_scores.  turboquant/compressors.py:122-158."""
    k_mse = comp["k_mse"].float()
    signs = comp["qjl_signs"].float()
    r_norm = comp["residual_norm"].float()
    term1 = torch.matmul(queries.float(), k_mse.transpose(-2, -1))
    q_proj = torch.matmul(queries.float(), s_mat.T)
    ip = torch.matmul(q_proj, signs.transpose(-2, -1))
    scale = math.sqrt(math.pi / 2) / s_mat.shape[0]
    return term1 + scale * ip * r_norm.unsqueeze(-2)


def v2_pack(idx: torch.Tensor, signs: torch.Tensor, bits: int):
    """Packed form of the V2 representation, which the reference does not store but whose size its accounting assumes
    (turboquant/validate.py:120-134): indices bit-packed as in turboquant/compressors_v3.py:64-74; signs one bit per
    coordinate, coordinate j in bit 7 - j % 8 of byte j / 8, set for +1.  (n, D) int -> ((n, G) uint8, (n, D/8) uint8)."""
    rows, _ = pack_indices(idx.cpu().numpy(), bits)
    sbits = np.packbits((signs.cpu().numpy() > 0).astype(np.uint8), axis=-1, bitorder="big")
    return torch.from_numpy(rows), torch.from_numpy(sbits)


def v2_scores_packed(queries: torch.Tensor, rows: torch.Tensor, sbits: torch.Tensor, vec_norms: torch.Tensor,
                     r_norm: torch.Tensor, pi: torch.Tensor, centroids: torch.Tensor, s_mat: torch.Tensor,
                     bits: int) -> torch.Tensor:
    """asymmetric_attention_scores (turboquant/compressors.py:122-158) evaluated from the packed form, in float64:
    k_mse = (centroids[idx] @ Pi) * vec_norms is rebuilt without the fp16 rounding of the stored k_mse.
    queries (B,H,Sq,D); rows (B,H,Sk,G); sbits (B,H,Sk,D/8); vec_norms, r_norm (B,H,Sk)."""
    b, h, sk, _ = rows.shape
    d = queries.shape[-1]
    idx = torch.from_numpy(unpack_indices(rows.reshape(b * h * sk, -1).cpu().numpy(), bits, d))
    k_mse = (centroids.double()[idx] @ pi.double()) * vec_norms.double().reshape(-1, 1)
    signs = np.unpackbits(sbits.reshape(b * h * sk, -1).cpu().numpy(), axis=-1, bitorder="big")[:, :d]
    signs = torch.from_numpy(signs.astype(np.float64)) * 2 - 1
    q = queries.double().cpu()
    term1 = torch.matmul(q, k_mse.reshape(b, h, sk, d).transpose(-2, -1))
    ip = torch.matmul(torch.matmul(q, s_mat.double().T), signs.reshape(b, h, sk, d).transpose(-2, -1))
    scale = math.sqrt(math.pi / 2) / s_mat.shape[0]
    return term1 + scale * ip * r_norm.double().cpu().unsqueeze(-2)


def v2mse_compress(states: torch.Tensor, pi: torch.Tensor, centroids: torch.Tensor) -> dict:
    """TurboQuantCompressorMSE.compress (unpacked uint8).  turboquant/compressors.py:200-213."""
    b, h, s, d = states.shape
    flat = states.reshape(-1, d).float()
    norms = torch.norm(flat, dim=-1, keepdim=True)
    unit = flat / (norms + 1e-8)
    idx = nearest_centroid(unit @ pi.T, centroids).to(torch.uint8)
    return {"indices": idx, "vec_norms": norms.squeeze(-1).to(torch.float16), "shape": (b, h, s, d)}


def v2mse_decompress(comp: dict, pi: torch.Tensor, centroids: torch.Tensor) -> torch.Tensor:
    """TurboQuantCompressorMSE.decompress.  turboquant/compressors.py:215-221."""
    b, h, s, d = comp["shape"]
    rec = centroids[comp["indices"].long()] @ pi
    return (rec * comp["vec_norms"].float().unsqueeze(-1)).reshape(b, h, s, d)


# --------------------------------------------------------------------------- #
# V1: TurboQuantMSE / TurboQuantProd
# --------------------------------------------------------------------------- #


def v1_mse_quantize(x: torch.Tensor, pi: torch.Tensor, centroids: torch.Tensor) -> torch.Tensor:
    """TurboQuantMSE.quantize (no normalisation) -> int64.  turboquant/turboquant.py:80-86."""
    return nearest_centroid(x @ pi.T, centroids)


def v1_mse_dequantize(idx: torch.Tensor, pi: torch.Tensor, centroids: torch.Tensor) -> torch.Tensor:
    """TurboQuantMSE.dequantize.  turboquant/turboquant.py:88-91."""
    return centroids[idx] @ pi


def v1_prod_quantize(x: torch.Tensor, pi: torch.Tensor, centroids: torch.Tensor, s_mat: torch.Tensor) -> dict:
    """TurboQuantProd.quantize.  turboquant/turboquant.py:134-159."""
    idx = v1_mse_quantize(x, pi, centroids)
    x_hat = v1_mse_dequantize(idx, pi, centroids)
    resid = x - x_hat
    r_norm = torch.norm(resid, dim=-1, keepdim=True)
    signs = torch.sign(resid @ s_mat.T)
    signs[signs == 0] = 1.0
    return {"mse_indices": idx, "qjl_signs": signs, "residual_norm": r_norm.squeeze(-1)}


def v1_prod_inner_product(y: torch.Tensor, comp: dict, pi: torch.Tensor, centroids: torch.Tensor,
                          s_mat: torch.Tensor) -> torch.Tensor:
    """TurboQuantProd.inner_product.  turboquant/turboquant.py:165-192."""
    x_mse = v1_mse_dequantize(comp["mse_indices"], pi, centroids)
    term1 = (y * x_mse).sum(dim=-1)
    ip = ((y @ s_mat.T) * comp["qjl_signs"]).sum(dim=-1)
    scale = math.sqrt(math.pi / 2) / s_mat.shape[0]
    return term1 + comp["residual_norm"] * scale * ip


# --------------------------------------------------------------------------- #
# Seeded synthetic KV tensors (stand in for model-derived caches)
# --------------------------------------------------------------------------- #


def synthetic_kv(shape, dtype, seed: int, outlier_channels: int = 4, outlier_scale: float = 10.0):
    """N(0,1) tensor (B,H,S,D) with `outlier_channels` channels per head scaled.

    Generated on the CPU generator so the oracle and the GPU see identical bits.
    """
    b, h, s, d = shape
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(b, h, s, d, generator=g, dtype=torch.float32)
    if outlier_channels:
        for head in range(h):
            ch = torch.randperm(d, generator=g)[:outlier_channels]
            x[:, head, :, ch] *= outlier_scale
    return x.to(dtype)
