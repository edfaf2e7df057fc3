"""Lloyd-Max codebooks for the coordinates of a randomly rotated unit vector.

Host-side, float64, scipy QUADPACK -- the same numerical recipe as the reference
(tonbistudio/turboquant-pytorch, turboquant/lloyd_max.py:32-86), because the fp32
centroids it returns are constants of the compressed format: indices are only
comparable between implementations that share them bit for bit.  Solved
codebooks are memoised per (d, bits, use_exact, max_iter, tol), since a KV cache
builds the same few codebooks once per layer, and kept on disk between processes
(an 8-bit codebook costs ~0.8 s of quadrature): float64 iterates in
$TURBOQUANT_B200_CACHE_DIR (default ~/.cache/turboquant_b200), one small file per
(solver variant, d, bits, use_exact, max_iter, tol, scipy version); set the variable to an
empty string to switch the disk cache off.  A stored codebook is used only if it has the
expected length; anything else is recomputed and rewritten.
"""

from __future__ import annotations

import functools
import math
import os

import numpy as np
import scipy
import torch
from scipy import integrate, special  # noqa: F401  (special kept for API parity of the module namespace)

__all__ = ["beta_pdf", "gaussian_approx_pdf", "solve_lloyd_max", "compute_expected_distortion", "LloydMaxCodebook"]


def beta_pdf(x: float, d: int) -> float:
    """Exact density of one coordinate of a uniformly random point on S^(d-1)."""
    if abs(x) >= 1.0:
        return 0.0
    lead = math.gamma(d / 2) / (math.sqrt(math.pi) * math.gamma((d - 1) / 2))
    return lead * (1 - x * x) ** ((d - 3) / 2)


def gaussian_approx_pdf(x: float, d: int) -> float:
    """N(0, 1/d), the large-d limit of beta_pdf."""
    var = 1.0 / d
    return (1.0 / math.sqrt(2 * math.pi * var)) * math.exp(-x * x / (2 * var))


def _density(d: int, use_exact: bool):
    return (lambda x: beta_pdf(x, d)) if use_exact else (lambda x: gaussian_approx_pdf(x, d))


def _conditional_means(pdf, cells, previous):
    """E[X | X in cell] for consecutive cells; keeps the previous value for empty cells."""
    means = []
    for i, (a, b) in enumerate(cells):
        mass_x, _ = integrate.quad(lambda x: x * pdf(x), a, b)
        mass, _ = integrate.quad(pdf, a, b)
        means.append(mass_x / mass if mass > 1e-15 else previous[i])
    return means


def _cache_dir():
    d = os.environ.get("TURBOQUANT_B200_CACHE_DIR")
    if d is None:
        d = os.path.join(os.path.expanduser("~"), ".cache", "turboquant_b200")
    return d or None


def _disk_cached(name: str, n_values: int, compute):
    """float64 vector `name` from the disk cache, or compute() stored there (best effort, atomic rename)."""
    folder = _cache_dir()
    path = os.path.join(folder, f"{name}_scipy{scipy.__version__}.npy") if folder else None
    if path is not None:
        try:
            got = np.load(path)
            if got.dtype == np.float64 and got.shape == (n_values,) and np.all(np.isfinite(got)):
                return tuple(float(v) for v in got)
        except Exception:
            pass
    values = compute()
    if path is not None:
        try:
            os.makedirs(folder, exist_ok=True)
            tmp = f"{path}.{os.getpid()}.tmp"
            with open(tmp, "wb") as f:
                np.save(f, np.asarray(values, dtype=np.float64))
            os.replace(tmp, path)
        except Exception:
            pass
    return tuple(values)


@functools.lru_cache(maxsize=None)
def _solve(d: int, bits: int, use_exact: bool, max_iter: int, tol: float):
    levels = 2 ** bits
    points = _disk_cached(f"lloydmax_d{d}_b{bits}_x{int(use_exact)}_i{max_iter}_t{tol!r}", levels,
                          lambda: _solve_points(d, bits, use_exact, max_iter, tol))
    mids = tuple((points[i] + points[i + 1]) / 2.0 for i in range(levels - 1))
    return points, mids


def _solve_points(d: int, bits: int, use_exact: bool, max_iter: int, tol: float):
    levels = 2 ** bits
    pdf = _density(d, use_exact)
    sigma = 1.0 / math.sqrt(d)
    lo, hi = -3.5 * sigma, 3.5 * sigma
    points = [lo + (hi - lo) * (i + 0.5) / levels for i in range(levels)]
    for _ in range(max_iter):
        mids = [(points[i] + points[i + 1]) / 2.0 for i in range(levels - 1)]
        edges = [lo * 3] + mids + [hi * 3]
        updated = _conditional_means(pdf, list(zip(edges[:-1], edges[1:])), points)
        moved = max(abs(u - p) for u, p in zip(updated, points))
        points = updated
        if moved < tol:
            break
    return tuple(points)


def solve_lloyd_max(d: int, bits: int, use_exact: bool = False, max_iter: int = 200, tol: float = 1e-10):
    """Optimal 2^bits-level scalar quantiser: (centroids [L], boundaries [L-1]) as fp32 tensors."""
    points, mids = _solve(int(d), int(bits), bool(use_exact), int(max_iter), float(tol))
    return torch.tensor(points, dtype=torch.float32), torch.tensor(mids, dtype=torch.float32)


@functools.lru_cache(maxsize=None)
def _solve_inlined_v2(d: int, bits: int):
    return _disk_cached(f"lloydmax_v2_d{d}_b{bits}", 2 ** bits, lambda: _solve_inlined_v2_points(d, bits))


def _solve_inlined_v2_points(d: int, bits: int):
    """Codebook as the V2 compressors of the reference compute it.

    Their private solver (turboquant/compressors.py:57-81) writes the density with
    sigma**2 and, once converged, returns the iterate BEFORE the last update.
    """
    levels = 2 ** bits
    sigma = 1.0 / math.sqrt(d)

    def pdf(x):
        return (1.0 / math.sqrt(2 * math.pi * sigma ** 2)) * math.exp(-x * x / (2 * sigma ** 2))

    lo, hi = -3.5 * sigma, 3.5 * sigma
    points = [lo + (hi - lo) * (i + 0.5) / levels for i in range(levels)]
    for _ in range(200):
        mids = [(points[i] + points[i + 1]) / 2.0 for i in range(levels - 1)]
        edges = [lo * 3] + mids + [hi * 3]
        updated = _conditional_means(pdf, list(zip(edges[:-1], edges[1:])), points)
        if max(abs(u - p) for u, p in zip(updated, points)) < 1e-10:
            break
        points = updated
    return tuple(points)


def solve_codebook_v2(d: int, bits: int) -> torch.Tensor:
    return torch.tensor(_solve_inlined_v2(int(d), int(bits)), dtype=torch.float32)


def compute_expected_distortion(d: int, bits: int, centroids: torch.Tensor, boundaries: torch.Tensor,
                                use_exact: bool = False) -> float:
    """Expected squared error per coordinate of the given quantiser."""
    pdf = _density(d, use_exact)
    sigma = 1.0 / math.sqrt(d)
    edges = [-3.5 * sigma * 3] + boundaries.tolist() + [3.5 * sigma * 3]
    total = 0.0
    for i in range(len(centroids)):
        c = centroids[i].item()
        part, _ = integrate.quad(lambda x: (x - c) ** 2 * pdf(x), edges[i], edges[i + 1])
        total += part
    return total


class LloydMaxCodebook:
    """Codebook for (d, bits): centroids, boundaries and expected distortion.

    quantize()/dequantize() work on tensors of any shape.  On CUDA tensors they
    run the library's threshold kernel (bit-identical to the |x-c| argmin); on
    CPU tensors they evaluate the argmin directly, as this is a host-side
    utility class in the reference as well (turboquant/lloyd_max.py:107-131).
    """

    def __init__(self, d: int, bits: int, use_exact: bool = False):
        self.d = d
        self.bits = bits
        self.n_levels = 2 ** bits
        self.centroids, self.boundaries = solve_lloyd_max(d, bits, use_exact)
        self.distortion = compute_expected_distortion(d, bits, self.centroids, self.boundaries, use_exact)
        self._blocks = {}

    def _block(self, device):
        from . import _native
        key = str(device)
        if key not in self._blocks:
            self._blocks[key] = _native.codebook_block(self.centroids, self.bits).to(device)
        return self._blocks[key]

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda and 1 <= self.bits <= 8 and x.dtype == torch.float32 and x.numel() > 0:
            from . import _native
            flat = x.contiguous().reshape(1, -1)
            cols = 1
            for c in (256, 128, 64, 32, 16, 8, 4, 2):
                if flat.shape[1] % c == 0:
                    cols = c
                    break
            flat = flat.reshape(-1, cols)
            out = torch.empty(flat.shape, dtype=torch.int64, device=x.device)
            with torch.cuda.device(x.device):
                _native.check(_native.lib().tq_quantize_rotated(
                    flat.data_ptr(), flat.shape[0], cols, self.bits, self._block(x.device).data_ptr(),
                    _native.IDX_I64, out.data_ptr(), _native.stream_ptr(x.device)), "tq_quantize_rotated")
            return out.reshape(x.shape)
        gaps = x.unsqueeze(-1) - self.centroids.to(x.device)
        return gaps.abs().argmin(dim=-1)

    def dequantize(self, indices: torch.Tensor) -> torch.Tensor:
        return self.centroids.to(indices.device)[indices]

    def __repr__(self):
        return (f"LloydMaxCodebook(d={self.d}, bits={self.bits}, "
                f"levels={self.n_levels}, distortion_per_coord={self.distortion:.6f})")
