"""The tcgen05 quantise kernel against the FP32 kernel and the oracle.

Jobs with head_dim 128, 16-bit input and packed output run on the tensor cores;
setting TQ_FORCE_SIMT=1 sends the same call down the FP32 path, which gives an
in-library second opinion on top of the CPU oracle.
"""

import os

import numpy as np
import pytest
import torch

import tq_oracle as O
from conftest import bits16
from parity_helpers import check_indices, check_norms, check_recon_16bit, mismatch_budget

import turboquant as tq
from turboquant import _native as N
from turboquant import batched

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _simt(fn):
    os.environ["TQ_FORCE_SIMT"] = "1"
    try:
        return fn()
    finally:
        os.environ.pop("TQ_FORCE_SIMT", None)


def _compare(c_tc, c_ref, bits, d=128):
    """Tensor-core result against the FP32 kernels: neighbouring indices only, bounded by count."""
    a = O.unpack_indices(c_tc["idx_bytes"].cpu().numpy().reshape(-1, c_tc["idx_bytes"].shape[-1]), bits, d)
    b = O.unpack_indices(c_ref["idx_bytes"].cpu().numpy().reshape(-1, c_ref["idx_bytes"].shape[-1]), bits, d)
    diff = np.abs(a.astype(np.int64) - b)
    assert diff.max() <= 1
    assert int((diff != 0).sum()) <= mismatch_budget(a.size), (int((diff != 0).sum()), a.size)
    g = bits16(c_tc["vec_norms"]).astype(np.int32)
    w = bits16(c_ref["vec_norms"]).astype(np.int32)
    assert np.abs(g - w).max() <= 1


def _oracle_check(c, x_cpu, comp, bits):
    """Against the oracle: every mismatch attributed to a decision boundary, bounded by count; norms 1 ulp."""
    cent, bnd = O.lloyd_max(128, bits)
    norms, _ = check_indices(c["idx_bytes"], x_cpu, comp.Pi.cpu(), cent, bnd, bits, 128)
    check_norms(c["vec_norms"], norms)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_tensor_core_quantize_matches_fp32_path_and_oracle(dtype, bits):
    x = O.synthetic_kv((2, 3, 333, 128), dtype, seed=900 + bits)         # ragged: 333 = 2 tiles + 77 rows per slab
    comp = tq.MSECompressor(128, bits, seed=70 + bits, device=DEV)
    assert comp._img_q is not None
    xg = x.to(DEV)
    c_tc = comp.compress(xg)
    c_ref = _simt(lambda: comp.compress(xg))
    torch.cuda.synchronize()
    assert N.lib().tq_last_device_status() == 0
    _compare(c_tc, c_ref, bits)
    _oracle_check(c_tc, x, comp, bits)


def test_tensor_core_path_reads_strided_views():
    base = O.synthetic_kv((2, 4, 300, 128), torch.float16, seed=31)
    g = base.to(DEV)
    comp = tq.MSECompressor(128, 4, seed=3, device=DEV)
    views = [(g[:, :, :172, :], base[:, :, :172, :]), (g[:, 1:3, 40:, :], base[:, 1:3, 40:, :]),
             (g[1:, :, :, :], base[1:, :, :, :]),
             (g.transpose(1, 2).contiguous().transpose(1, 2), base)]
    for gv, cv in views:
        c = comp.compress(gv)
        _oracle_check(c, cv.contiguous(), comp, 4)
        assert c["shape"] == tuple(cv.shape)
    assert N.lib().tq_last_device_status() == 0


def test_tensor_core_tiny_and_single_row_inputs():
    comp = tq.MSECompressor(128, 4, seed=11, device=DEV)
    for shape in ((1, 1, 1, 128), (1, 1, 127, 128), (1, 1, 128, 128), (1, 1, 129, 128), (3, 1, 5, 128), (1, 5, 2, 128)):
        x = O.synthetic_kv(shape, torch.float16, seed=sum(shape))
        c = comp.compress(x.to(DEV))
        _oracle_check(c, x, comp, 4)


def test_many_layers_in_one_launch_match_per_layer_fp32_results():
    L = 12
    codecs = [tq.TurboQuantV3(128, key_bits=4, value_bits=2, residual_window=0, layer_idx=l, n_layers=L, protected_layers=2,
                              device=DEV) for l in range(L)]
    keys = [O.synthetic_kv((1, 2, 1000 + 64 * l, 128), torch.float16, 300 + l).to(DEV) for l in range(L)]
    vals = [O.synthetic_kv((1, 2, 1000 + 64 * l, 128), torch.float16, 400 + l).to(DEV) for l in range(L)]
    many = batched.compress_kv_layers(codecs, keys, vals)
    ref = _simt(lambda: batched.compress_kv_layers(codecs, keys, vals))
    torch.cuda.synchronize()
    assert N.lib().tq_last_device_status() == 0
    for l in range(L):
        _compare(many[l][0]["compressed"], ref[l][0]["compressed"], codecs[l].key_bits)
        _compare(many[l][1]["compressed"], ref[l][1]["compressed"], codecs[l].value_bits)


def test_nan_and_zero_rows_on_the_tensor_core_path():
    x = O.synthetic_kv((1, 1, 256, 128), torch.float16, seed=77)
    x[0, 0, 3] = 0
    x[0, 0, 9, 5] = float("nan")
    x[0, 0, 200, 17] = float("inf")
    comp = tq.MSECompressor(128, 4, seed=42, device=DEV)
    c = comp.compress(x.to(DEV))
    idx = c["idx_bytes"].cpu().numpy()[0, 0]
    assert np.all(idx[3] == 0x77)
    assert np.all(idx[9] == 0) and np.all(idx[200] == 0)
    n = c["vec_norms"].cpu()[0, 0]
    # an Inf coordinate meets both signs of the split rotation, so its norm comes out NaN here
    # (the FP32 path and the reference give Inf); the indices are 0 either way
    assert n[3].item() == 0 and torch.isnan(n[9]) and (torch.isinf(n[200]) or torch.isnan(n[200]))


# ------------------------------------------------------------------ dequantize
def _close_16bit(got, ref_fp32, dtype):
    """A 16-bit reconstruction against an fp32 one: per vector, every element within 2e-3 of the vector's
    largest value plus the final rounding of the format (half a unit in the last place of the element)."""
    assert got.dtype == dtype
    check_recon_16bit(got, ref_fp32)
    return True


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_tensor_core_dequantize_fp32_matches_fp32_path_and_oracle(bits):
    x = O.synthetic_kv((2, 3, 333, 128), torch.float16, seed=500 + bits)
    comp = tq.MSECompressor(128, bits, seed=20 + bits, device=DEV)
    assert comp._img_d is not None
    c = comp.compress(x.to(DEV))
    rec = comp.decompress(c)
    ref = _simt(lambda: comp.decompress(c))
    torch.cuda.synchronize()
    assert N.lib().tq_last_device_status() == 0
    assert rec.dtype == torch.float32 and rec.shape == (2, 3, 333, 128)
    scale = float(ref.abs().max())
    assert float((rec - ref).abs().max()) <= 1e-5 * scale
    cent = O.lloyd_max(128, bits)[0]
    want = O.mse_decompress({k: (v.cpu() if torch.is_tensor(v) else v) for k, v in c.items()}, comp.Pi.cpu(), cent, bits)
    assert float((rec.cpu() - want).abs().max()) <= 1e-5 * float(want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits,window", [(2, 0), (4, 0), (4, 37), (6, 16), (8, 128)])
def test_tensor_core_decompress_kv_into_cache_dtype(dtype, bits, window):
    keys = O.synthetic_kv((2, 2, 400, 128), dtype, seed=60 + bits)
    vals = O.synthetic_kv((2, 2, 400, 128), dtype, seed=61 + bits)
    codec = tq.TurboQuantV3(128, key_bits=bits, value_bits=max(bits - 2, 1), residual_window=window, layer_idx=7, n_layers=36,
                            protected_layers=0, device=DEV)
    ck, cv = codec.compress_kv(keys.to(DEV), vals.to(DEV))
    rk, rv = codec.decompress_kv(ck, cv)
    fk, fv = _simt(lambda: codec.decompress_kv(ck, cv))
    torch.cuda.synchronize()
    assert N.lib().tq_last_device_status() == 0
    for got, ref, src in ((rk, fk, keys), (rv, fv, vals)):
        assert got.dtype == dtype and got.shape == src.shape
        assert _close_16bit(got, ref, dtype)
        cut = 400 - window
        assert torch.equal(got[:, :, cut:].cpu(), src[:, :, cut:])
    # against the oracle end to end
    ref = O.V3Oracle(128, key_bits=bits, value_bits=max(bits - 2, 1), residual_window=window, layer_idx=7, n_layers=36,
                     protected_layers=0)
    cpu = lambda d: {k: (({kk: (vv.cpu() if torch.is_tensor(vv) else vv) for kk, vv in v.items()} if isinstance(v, dict)
                          else (v.cpu() if torch.is_tensor(v) else v))) for k, v in d.items()}
    ok_, ov_ = ref.decompress_kv(cpu(ck), cpu(cv))
    assert _close_16bit(rk, ok_, dtype) and _close_16bit(rv, ov_, dtype)


def test_tensor_core_dequantize_many_layers_one_launch():
    L = 10
    codecs = [tq.TurboQuantV3(128, key_bits=4, value_bits=2, residual_window=0, layer_idx=l, n_layers=L, protected_layers=1,
                              device=DEV) for l in range(L)]
    keys = [O.synthetic_kv((1, 2, 700 + 128 * l, 128), torch.float16, 800 + l).to(DEV) for l in range(L)]
    vals = [O.synthetic_kv((1, 2, 700 + 128 * l, 128), torch.float16, 900 + l).to(DEV) for l in range(L)]
    packed = batched.compress_kv_layers(codecs, keys, vals)
    outs = batched.decompress_kv_layers(codecs, packed)
    refs = _simt(lambda: batched.decompress_kv_layers(codecs, packed))
    torch.cuda.synchronize()
    assert N.lib().tq_last_device_status() == 0
    for l in range(L):
        for got, ref in zip(outs[l], refs[l]):
            assert float((got.float() - ref.float()).abs().max()) <= 2e-3 * float(ref.float().abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [2, 4, 6, 8])
def test_index_rows_at_a_16_byte_offset_equal_the_aligned_ones(bits):
    """The tensor-core quantiser writes 32 bytes per store when a row allows it; a destination that is only 16-byte
    aligned takes the narrower stores and must give the same bytes (and nothing outside its rows)."""
    import turboquant as tq
    from turboquant import _native as N, _ops
    x = O.synthetic_kv((1, 2, 300, 128), torch.bfloat16, seed=81000 + bits).to("cuda:0")
    comp = tq.MSECompressor(128, bits, seed=5, device="cuda:0")
    job, res, _keep = comp.compress_job(x)
    _ops.run_quantize([job], x.device)
    want = res["idx_bytes"].clone()
    g = want.shape[-1]
    raw = torch.full((want.numel() + 64,), 0xA5, dtype=torch.uint8, device=x.device)
    assert raw.data_ptr() % 32 == 0
    job.idx_out = raw.data_ptr() + 16
    _ops.run_quantize([job], x.device)
    torch.cuda.synchronize()
    got = raw[16:16 + want.numel()].reshape(want.shape)
    assert torch.equal(got, want)
    assert bool((raw[:16] == 0xA5).all()) and bool((raw[16 + want.numel():] == 0xA5).all())
    assert g == N.packed_row_bytes(128, bits) and N.lib().tq_last_device_status() == 0
