"""Comparison helpers shared by the GPU parity tests.

The bar (stated once here, applied everywhere):
  * rotated fp32 values in -> packed bytes: bit exact;
  * end to end: EVERY index mismatch is attributed -- a neighbouring index whose oracle-rotated value
    lies within 1e-6 of the decision boundary between the two -- and their number is bounded by a
    count (1e-4 of the coordinates, at least 2 on small inputs);
  * fp16 norms within 1 ulp;
  * reconstructions and scores: <= 1e-5 relative (fp32 I/O), <= 2e-3 of the vector's largest value
    (16-bit I/O), checked per vector.
"""

import math

import numpy as np
import torch

import tq_oracle as O
from conftest import bits16


def rel_err(got, want):
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def mismatch_budget(n_coords: int) -> int:
    return max(2, int(math.ceil(1e-4 * n_coords)))


def check_indices(got_packed, x_cpu, pi, cent, bnd, bits, d, max_mismatch=None):
    """Packed indices against the oracle; returns (oracle norms, agreement).  See the module docstring."""
    _flat, norms, rot = O.rotate_unit(x_cpu, pi)
    want = O.nearest_centroid(rot, cent).numpy()
    n = want.shape[0]
    got = O.unpack_indices(got_packed.cpu().numpy().reshape(n, -1), bits, d)
    bad = np.argwhere(got != want)
    b = bnd.numpy()
    for r, c in bad:
        y = rot[r, c].item()
        lo = min(int(got[r, c]), int(want[r, c]))
        assert abs(int(got[r, c]) - int(want[r, c])) == 1, (r, c, got[r, c], want[r, c])
        assert abs(float(b[lo]) - y) < 1e-6, (r, c, y, float(b[lo]))
    if max_mismatch is None:
        max_mismatch = mismatch_budget(want.size)
    assert len(bad) <= max_mismatch, (len(bad), max_mismatch, want.size)
    return norms, 1.0 - len(bad) / want.size


def check_norms(got_fp16, want_fp32):
    g = bits16(got_fp16).astype(np.int32).reshape(-1)
    w = bits16(want_fp32.to(torch.float16)).astype(np.int32).reshape(-1)
    assert np.all(np.abs(g - w) <= 1)


def check_recon_16bit(got, want, tol=2e-3):
    """A 16-bit reconstruction against the oracle's, per vector: every element within
    tol * (the vector's largest magnitude) plus the final rounding of the 16-bit format at that element --
    half a unit in the last place when `want` is fp32, a whole one when `want` has been rounded to the
    format as well (the reference's own .to(dtype))."""
    g = got.detach().float().cpu()
    w = want.detach().float().cpu()
    scale = w.abs().amax(dim=-1, keepdim=True)
    eps = 2.0 ** -8 if got.dtype == torch.bfloat16 else 2.0 ** -11      # half an ulp, relative (upper bound)
    if want.dtype == got.dtype:
        eps *= 2
    bound = tol * scale + eps * w.abs() + 1e-30
    worst = float(((g - w).abs() / bound).max())
    assert worst <= 1.0, worst
    return worst


def ulp_stats_16bit(got, want_fp32):
    """(fraction of elements within 1 unit in the last place, largest distance in units) between a 16-bit
    tensor and the oracle's fp32 result rounded to the same format."""
    w = want_fp32.detach().cpu().to(got.dtype)
    d = (got.detach().cpu().view(torch.int16).int() - w.view(torch.int16).int()).abs()
    return float((d <= 1).float().mean()), int(d.max())


def check_v2_compress(c, x_cpu, pi, cent, s_mat, max_differing=None):
    """TurboQuantCompressorV2.compress output against the oracle with every difference attributed.

    A vector is *marked* when one of its oracle-rotated coordinates lies within 1e-6 of a decision boundary:
    there the neighbouring index is an equally valid answer, and it changes that vector's k_mse, residual norm
    and signs.  A vector *agrees* when its k_mse is within 2e-3 of its largest value (fp16 output), its residual
    norm within 1 fp16 ulp, and its signs are exactly the oracle's except where the projected residual is
    numerically zero (|r . S_j| <= 1e-5 |r| |S_j|).  Every vector that does not agree must be marked, their
    number is bounded by a count, and their k_mse by one quantisation step per near-boundary coordinate.
    Returns the number of vectors that differ."""
    b, h, s, d = x_cpu.shape
    flat = x_cpu.reshape(-1, d).float()
    norms = torch.norm(flat, dim=-1, keepdim=True)
    unit = flat / (norms + 1e-8)
    rot = unit @ pi.T
    idx = O.nearest_centroid(rot, cent)
    bnd = (cent[:-1] + cent[1:]) / 2
    near = torch.zeros_like(rot, dtype=torch.bool)
    for bv in bnd.tolist():                                        # (N, D) at a time: no (N, D, L) tensor
        near |= (rot - bv).abs() < 1e-6
    marked = near.any(-1)
    k_mse = (cent[idx] @ pi) * norms
    resid = flat - k_mse
    r_norm = torch.norm(resid, dim=-1)
    proj = resid @ s_mat.T
    want_signs = (proj >= 0).to(torch.int8) * 2 - 1
    n = flat.shape[0]
    got_k = c["k_mse"].detach().float().cpu().reshape(n, d)
    got_s = c["qjl_signs"].detach().cpu().reshape(n, -1)
    got_r = c["residual_norm"].detach().cpu().reshape(n)
    scale = k_mse.abs().amax(-1, keepdim=True)
    bound = 2e-3 * scale + 2.0 ** -11 * k_mse.abs() + 1e-30
    k_ok = ((got_k - k_mse).abs() <= bound).all(-1)
    g16 = torch.from_numpy(bits16(got_r).astype(np.int32))
    w16 = torch.from_numpy(bits16(r_norm.to(torch.float16)).astype(np.int32))
    r_ok = (g16 - w16).abs() <= 1
    s_norm = torch.norm(s_mat, dim=-1)
    tiny = proj.abs() <= 1e-5 * r_norm.unsqueeze(-1) * s_norm.unsqueeze(0) + 1e-30
    s_ok = ~((got_s != want_signs) & ~tiny).any(-1)
    agrees = k_ok & r_ok & s_ok
    differing = ~agrees
    assert not bool((differing & ~marked).any()), \
        (int((differing & ~marked).sum()), int((~k_ok & ~marked).sum()), int((~r_ok & ~marked).sum()), int((~s_ok & ~marked).sum()))
    if max_differing is None:
        max_differing = mismatch_budget(n * d)
    assert int(differing.sum()) <= max_differing, (int(differing.sum()), max_differing)
    if bool(differing.any()):
        step = float((cent[1:] - cent[:-1]).max())
        lim = (near.sum(-1, keepdim=True).float().sqrt() * step * norms + bound)[differing]
        assert bool(((got_k - k_mse).abs()[differing] <= lim).all())
    assert set(torch.unique(got_s).tolist()) <= {-1, 1}
    return int(differing.sum())
