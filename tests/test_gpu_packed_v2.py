"""The packed form of the MSE+QJL (V2) representation on the GPU: packing is bit-exact against the oracle, the packed
compress carries the same indices, signs and norms as the reference-form compress, and scores computed straight from
the packed rows match the oracle's float64 evaluation of turboquant/compressors.py:122-158 within 1e-5."""

import numpy as np
import pytest
import torch

import tq_oracle as O
from parity_helpers import rel_err

import turboquant as tq
from turboquant import _native as N
from turboquant import _ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _cpu(d):
    return {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in d.items()}


@pytest.mark.parametrize("d,bits", [(128, 1), (128, 2), (128, 3), (256, 4), (256, 5), (64, 6), (128, 8), (72, 3)])
def test_pack_is_bit_exact(d, bits):
    g = torch.Generator().manual_seed(100 * d + bits)
    n = 333
    idx = torch.randint(0, 1 << bits, (n, d), generator=g, dtype=torch.int64).to(torch.uint8)
    signs = (torch.randint(0, 2, (n, d), generator=g, dtype=torch.int64) * 2 - 1).to(torch.int8)
    rows, sbits = _ops.pack_mse_qjl(idx.to(DEV), signs.to(DEV), d, bits)
    want_rows, want_bits = O.v2_pack(idx, signs, bits)
    assert rows.shape == want_rows.shape and torch.equal(rows.cpu(), want_rows)
    assert sbits.shape == want_bits.shape and torch.equal(sbits.cpu(), want_bits)
    only_rows, none = _ops.pack_mse_qjl(idx.to(DEV), None, d, bits)
    assert none is None and torch.equal(only_rows, rows)


@pytest.mark.parametrize("d,bits,shape", [(128, 3, (1, 2, 300, 128)), (256, 3, (2, 3, 77, 256)), (256, 5, (1, 1, 513, 256)),
                                          (128, 2, (1, 4, 128, 128)), (128, 4, (1, 2, 1000, 128))])
def test_packed_compress_carries_the_reference_form(d, bits, shape):
    x = O.synthetic_kv(shape, torch.float16, seed=61000 + d + bits, outlier_channels=0)
    comp = tq.TurboQuantCompressorV2(d, bits, seed=13, device=DEV)
    ref = comp.compress(x.to(DEV))
    pk = comp.compress(x.to(DEV), packed=True)
    b, h, s, _ = shape
    assert pk["packed"] is True and pk["shape"] == tuple(shape)
    assert tuple(pk["mse_idx_bytes"].shape) == (b, h, s, N.packed_row_bytes(d, comp.mse_bits))
    assert tuple(pk["sign_bits"].shape) == (b, h, s, d // 8) and pk["vec_norms"].dtype == torch.float32
    # same kernels, same inputs: signs and residual norms are the reference form's, bit for bit
    _rows, want_bits = O.v2_pack(torch.zeros(b * h * s, d, dtype=torch.uint8), ref["qjl_signs"].reshape(-1, d).cpu(),
                                 comp.mse_bits)
    assert torch.equal(pk["sign_bits"].reshape(-1, d // 8).cpu(), want_bits)
    assert torch.equal(pk["residual_norm"], ref["residual_norm"])
    norms = x.float().norm(dim=-1)
    assert torch.allclose(pk["vec_norms"].cpu(), norms, rtol=2e-6, atol=0)
    # indices: every coordinate is the nearest centroid of the rotated unit vector, or within rounding of a boundary
    idx = O.unpack_indices(pk["mse_idx_bytes"].reshape(b * h * s, -1).cpu().numpy(), comp.mse_bits, d)
    rot = (x.reshape(-1, d).double() / (x.reshape(-1, d).double().norm(dim=-1, keepdim=True) + 1e-8)) @ comp.Pi.cpu().double().T
    cents = comp.centroids.cpu().double()
    dist = (rot.unsqueeze(-1) - cents).abs()
    chosen = torch.gather(dist, -1, torch.from_numpy(idx).unsqueeze(-1)).squeeze(-1)
    assert float((chosen - dist.amin(-1)).max()) <= 2e-6
    # unpack() gives back the reference form: k_mse within 1e-3 of each vector's largest component of the directly stored one
    back = comp.unpack(pk)
    assert torch.equal(back["qjl_signs"], ref["qjl_signs"]) and back["k_mse"].dtype == torch.float16
    gap = (back["k_mse"].float() - ref["k_mse"].float()).abs().amax(-1)
    assert bool((gap <= 1e-3 * ref["k_mse"].float().abs().amax(-1) + 1e-30).all())
    # size: G + D/8 + 4 + 2 bytes a vector against 3 D + 2 in the reference form
    per_vec = N.packed_row_bytes(d, comp.mse_bits) + d // 8 + 6
    assert comp.stored_bytes(pk) == b * h * s * per_vec and comp.stored_bytes(ref) == b * h * s * (3 * d + 2)
    assert N.lib().tq_last_device_status() == 0


@pytest.mark.parametrize("d,bits,bh,sq,sk,qdt", [(128, 3, (1, 2), 1, 300, torch.float32), (128, 2, (2, 2), 7, 77, torch.float16),
                                                 (128, 4, (1, 3), 64, 1000, torch.bfloat16), (128, 5, (1, 1), 100, 513, torch.float32),
                                                 (256, 3, (1, 2), 64, 300, torch.float32), (256, 2, (2, 1), 5, 1, torch.float16),
                                                 (256, 5, (1, 2), 130, 4100, torch.float32), (128, 9, (1, 1), 3, 50, torch.float32)])
def test_scores_from_packed_rows_match_the_oracle(d, bits, bh, sq, sk, qdt):
    x = O.synthetic_kv((*bh, sk, d), torch.float16, seed=62000 + d + bits + sk, outlier_channels=0)
    q = torch.randn(*bh, sq, d, generator=torch.Generator().manual_seed(sq + sk)).to(qdt)
    comp = tq.TurboQuantCompressorV2(d, bits, seed=29, device=DEV)
    pk = comp.compress(x.to(DEV), packed=True)
    sc = comp.asymmetric_attention_scores(q.to(DEV), pk)
    c = _cpu(pk)
    want = O.v2_scores_packed(q, c["mse_idx_bytes"], c["sign_bits"], c["vec_norms"], c["residual_norm"], comp.Pi.cpu(),
                              comp.centroids.cpu(), comp.S.cpu(), comp.mse_bits)
    assert sc.dtype == torch.float32 and tuple(sc.shape) == (*bh, sq, sk)
    assert rel_err(sc, want.float()) <= 1e-5
    # and agree with the reference-form scores up to the fp16 rounding of its stored k_mse
    ref = comp.asymmetric_attention_scores(q.to(DEV), comp.unpack(pk))
    assert rel_err(sc, ref) <= 2e-3
    assert N.lib().tq_last_device_status() == 0


def test_packed_edges_zero_vector_and_other_input_layouts():
    comp = tq.TurboQuantCompressorV2(128, 3, seed=3, device=DEV)
    x = O.synthetic_kv((1, 1, 3, 128), torch.float16, seed=63000, outlier_channels=0)
    x[0, 0, 1] = 0
    pk = comp.compress(x.to(DEV), packed=True)
    assert float(pk["vec_norms"][0, 0, 1]) == 0.0 and bool((pk["sign_bits"][0, 0, 1] == 255).all())
    q = torch.randn(1, 1, 2, 128, generator=torch.Generator().manual_seed(1))
    sc = comp.asymmetric_attention_scores(q.to(DEV), pk)
    assert float(sc[0, 0, :, 1].abs().max()) == 0.0
    # bf16 and fp32 vectors and strided views go through the FP32 kernels and give the same packed form
    base = O.synthetic_kv((1, 2, 96, 128), torch.float16, seed=63001, outlier_channels=0)
    want = comp.compress(base.to(DEV), packed=True)
    got = comp.compress(base.float().to(DEV), packed=True)
    differ = (got["mse_idx_bytes"] != want["mse_idx_bytes"]).any(-1)
    assert int(differ.sum()) <= 2                       # a coordinate on a boundary may fall either way
    same = ~differ
    assert torch.equal(got["sign_bits"][same], want["sign_bits"][same])
    assert torch.allclose(got["vec_norms"], want["vec_norms"], rtol=2e-6, atol=0)
    view = base.to(DEV)[:, :, ::2]
    got = comp.compress(view, packed=True)
    assert tuple(got["mse_idx_bytes"].shape) == (1, 2, 48, 32)
    sc = comp.asymmetric_attention_scores(q.expand(1, 2, 2, 128).contiguous().to(DEV), got)
    c = _cpu(got)
    ref = O.v2_scores_packed(q.expand(1, 2, 2, 128), c["mse_idx_bytes"], c["sign_bits"], c["vec_norms"], c["residual_norm"],
                             comp.Pi.cpu(), comp.centroids.cpu(), comp.S.cpu(), comp.mse_bits)
    assert rel_err(sc, ref.float()) <= 1e-5
    with pytest.raises(ValueError):
        comp.asymmetric_attention_scores(q.to(DEV), {**pk, "vec_norms": pk["vec_norms"].half()})
