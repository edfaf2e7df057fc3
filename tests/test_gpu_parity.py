"""GPU parity: the CUDA path (through the Python mirror, i.e. through the C ABI)
against the CPU oracle on the same seeded inputs and against the golden fixtures.

Tolerances: see tests/parity_helpers.py (bit exact from rotated values; every end-to-end
index mismatch attributed to a decision boundary and bounded by count; fp16 norms within
1 ulp; <= 1e-5 relative for fp32 I/O, <= 2e-3 of the vector's largest value for 16-bit I/O).
"""

import numpy as np
import pytest
import torch

import tq_oracle as O
from conftest import bits16, from_bits16, load_golden
from parity_helpers import check_indices, check_norms, check_recon_16bit, check_v2_compress, rel_err

import turboquant as tq
from turboquant import _native as N
from turboquant import _ops, batched

pytestmark = pytest.mark.gpu
DEV = "cuda"



def few_neighbour_mismatches(mine, gold, k=2):
    """Indices against bytes the reference stored (its rotation matrix comes out of LAPACK QR and may differ in
    the last bits from the one rebuilt here): neighbouring indices only, at most k of them."""
    d = np.abs(np.asarray(mine).astype(np.int64) - np.asarray(gold).astype(np.int64))
    assert d.max() <= 1 and int((d != 0).sum()) <= k, (int(d.max()), int((d != 0).sum()))
    return (d != 0).reshape(d.shape[0], -1).any(-1)          # rows that hold a mismatch


def signs_equal_outside(mine, gold, rows_excluded, k=2):
    """QJL signs equal the stored ones on every row without an index mismatch, except for at most k coordinates
    (projections that are numerically zero)."""
    diff = (np.asarray(mine) != np.asarray(gold)).reshape(len(rows_excluded), -1)
    assert int(diff[~rows_excluded].sum()) <= k, int(diff[~rows_excluded].sum())


# --------------------------------------------------------------------------- K0
def test_k0_rotated_to_packed_is_bit_exact_on_fixtures():
    z = load_golden("mse_small.npz")
    for d, bits, n in z["cases"].tolist():
        k = f"{d}_{bits}"
        cb = N.codebook_block(O.lloyd_max(d, bits)[0], bits).to(DEV)
        got = _ops.quantize_rotated(torch.from_numpy(z[f"rot_{k}"]).to(DEV), cb, bits)
        assert np.array_equal(got.cpu().numpy(), z[f"idx_{k}"].reshape(n, -1)), k


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_k0_bit_exact_random_and_boundary_values(bits):
    d = 128
    cent, bnd = O.lloyd_max(d, bits)
    cb = N.codebook_block(cent, bits).to(DEV)
    g = torch.Generator().manual_seed(bits)
    y = torch.randn(4096, d, generator=g) / np.sqrt(d)
    # plant every boundary and its fp32 neighbours
    edge = []
    for b in bnd.tolist():
        v = np.float32(b)
        for _ in range(4):
            v = np.nextafter(v, np.float32(-np.inf))
        for _ in range(9):
            edge.append(float(v))
            v = np.nextafter(v, np.float32(np.inf))
    e = torch.tensor(edge, dtype=torch.float32)
    y.view(-1)[: e.numel()] = e
    y[100, :4] = torch.tensor([0.0, -0.0, 1.0, -1.0])
    want = O.nearest_centroid(y, cent)
    for mode, dt in ((N.IDX_PACKED, None), (N.IDX_U8, torch.uint8), (N.IDX_I64, torch.int64)):
        got = _ops.quantize_rotated(y.to(DEV), cb, bits, mode).cpu()
        if mode == N.IDX_PACKED:
            assert np.array_equal(got.numpy(), O.pack_indices(want.numpy(), bits)[0])
        else:
            assert got.dtype == dt and torch.equal(got.long(), want)


def test_codebook_quantize_on_gpu_matches_argmin():
    cbk = tq.LloydMaxCodebook(128, 3)
    x = torch.randn(7, 33, generator=torch.Generator().manual_seed(1)) * 0.1
    assert torch.equal(cbk.quantize(x.to(DEV)).cpu(), O.nearest_centroid(x, cbk.centroids))


# --------------------------------------------------------------------------- K1 / K2
def test_cfg1_roundtrip_against_oracle_and_golden():
    z = load_golden("cfg1.npz")
    x = torch.randn(1, 1, 4096, 128, generator=torch.Generator(device="cpu").manual_seed(0))
    for tag, bits, seed in (("k", 4, 42), ("v", 2, 542)):
        comp = tq.MSECompressor(128, bits, seed=seed, device=DEV)
        cent, bnd = O.lloyd_max(128, bits)
        c = comp.compress(x.to(DEV))
        assert c["idx_bytes"].dtype == torch.uint8 and c["idx_bytes"].shape == (1, 1, 4096, 128 * bits // 8)
        assert c["vec_norms"].dtype == torch.float16 and c["vec_norms"].shape == (1, 1, 4096)
        assert c["shape"] == (1, 1, 4096, 128) and c["idx_pad"] == 0
        norms, agree = check_indices(c["idx_bytes"], x, comp.Pi.cpu(), cent, bnd, bits, 128)
        check_norms(c["vec_norms"], norms)
        # against the bytes the reference itself stored (its rotation matrix comes out of LAPACK QR and may
        # differ in the last bits from the one rebuilt here): at most 1e-4 of the coordinates, neighbours only
        mine = O.unpack_indices(c["idx_bytes"].cpu().numpy().reshape(4096, -1), bits, 128).astype(np.int32)
        gold = O.unpack_indices(z[f"{tag}_idx"].reshape(4096, -1), bits, 128).astype(np.int32)
        assert np.abs(mine - gold).max() <= 1 and (mine != gold).sum() <= int(np.ceil(1e-4 * gold.size))
        rec = comp.decompress(c)
        assert rec.dtype == torch.float32 and rec.shape == (1, 1, 4096, 128)
        want = O.mse_decompress({k: (v.cpu() if torch.is_tensor(v) else v) for k, v in c.items()}, comp.Pi.cpu(), cent, bits)
        assert rel_err(rec, want) <= 1e-5
        mse = float(((rec.cpu() - x) ** 2).sum(-1).mean())
        assert mse == pytest.approx(float(z[f"{tag}_mse"]), rel=1e-3)
        packed_bytes = c["idx_bytes"].numel() + 2 * c["vec_norms"].numel()
        assert packed_bytes == int(z[f"{tag}_mem"][0]) == comp.memory_bytes(1, 1, 4096)["compressed_bytes"]


def test_small_cases_every_bits_and_head_dim_including_padding():
    z = load_golden("mse_small.npz")
    for d, bits, n in z["cases"].tolist():
        k = f"{d}_{bits}"
        x = torch.from_numpy(z[f"x_{k}"])
        comp = tq.MSECompressor(d, bits, seed=17 + bits, device=DEV)
        cent, bnd = O.lloyd_max(d, bits)
        c = comp.compress(x.to(DEV))
        assert c["idx_pad"] == int(z[f"pad_{k}"]) and tuple(c["idx_bytes"].shape) == z[f"idx_{k}"].shape
        norms, _ = check_indices(c["idx_bytes"], x, comp.Pi.cpu(), cent, bnd, bits, d)
        check_norms(c["vec_norms"], norms)
        gold = {"idx_bytes": torch.from_numpy(z[f"idx_{k}"]).to(DEV), "vec_norms": from_bits16(z[f"norms_{k}"], torch.float16).to(DEV),
                "shape": tuple(x.shape), "idx_pad": int(z[f"pad_{k}"])}
        rec = comp.decompress(gold)
        assert rel_err(rec, torch.from_numpy(z[f"rec_{k}"])) <= 1e-5, k


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_16bit_inputs_with_outlier_channels(dtype):
    x = O.synthetic_kv((1, 2, 1024, 128), dtype, seed=20000)
    for bits in (2, 4, 6, 8):
        comp = tq.MSECompressor(128, bits, seed=42 + bits, device=DEV)
        cent, bnd = O.lloyd_max(128, bits)
        c = comp.compress(x.to(DEV))
        norms, _ = check_indices(c["idx_bytes"], x, comp.Pi.cpu(), cent, bnd, bits, 128)
        check_norms(c["vec_norms"], norms)


def test_strided_views_are_read_in_place():
    base = O.synthetic_kv((2, 3, 80, 128), torch.float16, seed=7)
    comp = tq.MSECompressor(128, 4, seed=5, device=DEV)
    cent, bnd = O.lloyd_max(128, 4)
    g = base.to(DEV)
    views = [(g[:, :, :50, :], base[:, :, :50, :]),
             (g[:, 1:, 7:, :], base[:, 1:, 7:, :]),
             (g.transpose(1, 2).contiguous().transpose(1, 2), base)]       # (B,S,H,D) memory order
    for gv, cv in views:
        c = comp.compress(gv)
        norms, _ = check_indices(c["idx_bytes"], cv.contiguous(), comp.Pi.cpu(), cent, bnd, 4, 128)
        check_norms(c["vec_norms"], norms)
        assert c["shape"] == tuple(cv.shape)


def test_edge_vectors_match_reference():
    z = load_golden("edge.npz")
    x = torch.from_numpy(z["x"])
    comp = tq.MSECompressor(128, 4, seed=42, device=DEV)
    c = comp.compress(x.to(DEV))
    got = c["idx_bytes"].cpu().numpy()
    want = z["idx"]
    for row in (0, 1, 2, 5):      # zero vector, NaN, Inf, coordinate axis
        assert np.array_equal(got[0, 0, row], want[0, 0, row]), row
    assert (got == want).mean() > 0.99
    gn, wn = bits16(c["vec_norms"]).reshape(-1), z["norms"].reshape(-1)
    assert np.isnan(c["vec_norms"][0, 0, 1].item()) and np.isinf(c["vec_norms"][0, 0, 2].item())
    assert np.isinf(c["vec_norms"][0, 0, 3].item())                     # norm beyond the fp16 range
    fin = [0, 4, 5, 6, 7]
    assert np.all(np.abs(gn[fin].astype(np.int32) - wn[fin].astype(np.int32)) <= 1)
    gold = {"idx_bytes": torch.from_numpy(want).to(DEV), "vec_norms": from_bits16(z["norms"], torch.float16).to(DEV),
            "shape": (1, 1, 8, 128), "idx_pad": 0}
    rec = comp.decompress(gold).cpu().numpy()
    ok = np.isfinite(z["rec"])
    assert np.array_equal(np.isfinite(rec), ok)
    assert np.allclose(rec[ok], z["rec"][ok], rtol=0, atol=1e-5 * np.abs(z["rec"][ok]).max())


def test_empty_and_tiny_inputs():
    comp = tq.MSECompressor(128, 4, seed=1, device=DEV)
    c = comp.compress(torch.empty(1, 2, 0, 128, device=DEV, dtype=torch.float16))
    assert c["idx_bytes"].shape == (1, 2, 0, 64) and c["vec_norms"].shape == (1, 2, 0)
    assert comp.decompress(c).shape == (1, 2, 0, 128)
    for n in (1, 2, 63, 64, 65, 127, 129):
        x = torch.randn(1, 1, n, 128, generator=torch.Generator().manual_seed(n))
        c = comp.compress(x.to(DEV))
        cent, bnd = O.lloyd_max(128, 4)
        check_indices(c["idx_bytes"], x, comp.Pi.cpu(), cent, bnd, 4, 128)


def test_scale_invariance_and_idempotence_at_full_layer_size():
    # one layer of the Qwen2.5-3B-shaped cache: (1, 2, 8192, 128) fp16
    x = O.synthetic_kv((1, 2, 8192, 128), torch.float16, seed=20005).to(DEV)
    comp = tq.MSECompressor(128, 4, seed=5042, device=DEV)
    c1 = comp.compress(x)
    c2 = comp.compress(x * 2)                               # exact power-of-two scaling
    same = (c1["idx_bytes"] == c2["idx_bytes"]).float().mean().item()
    assert same >= 0.9999
    assert torch.equal(c2["vec_norms"].float(), (c1["vec_norms"].float() * 2).clamp(max=65504.0).half().float()) or \
        (c2["vec_norms"].float() - 2 * c1["vec_norms"].float()).abs().max() <= 2 * 2 ** -10 * c2["vec_norms"].float().max()
    rec = comp.decompress(c1)
    c3 = comp.compress(rec)                                 # re-quantising a reconstruction returns the same codes
    assert (c3["idx_bytes"] == c1["idx_bytes"]).float().mean().item() >= 0.9999
    relmse = float((((rec - x.float()) ** 2).sum(-1) / (x.float() ** 2).sum(-1)).mean())
    assert 0.005 < relmse < 0.015                          # 4-bit: ~0.0094 on Gaussian data
    assert c1["idx_bytes"].numel() + 2 * c1["vec_norms"].numel() == comp.memory_bytes(1, 2, 8192)["compressed_bytes"]


# --------------------------------------------------------------------------- V3
V3_CASES = {
    "a": (torch.float16, dict(key_bits=4, value_bits=2, residual_window=0, layer_idx=3, n_layers=36, protected_layers=0)),
    "b": (torch.bfloat16, dict(key_bits=6, value_bits=4, residual_window=16, layer_idx=0, n_layers=32, protected_layers=4)),
    "c": (torch.bfloat16, dict(key_bits=6, value_bits=4, residual_window=16, layer_idx=10, n_layers=32, protected_layers=4)),
    "d": (torch.float16, dict(key_bits=4, value_bits=2, residual_window=128, layer_idx=5, n_layers=36, protected_layers=4)),
}


@pytest.mark.parametrize("tag", list(V3_CASES))
def test_v3_compress_decompress_kv_against_golden(tag):
    z = load_golden("v3_kv.npz")
    dt, kw = V3_CASES[tag]
    keys = from_bits16(z[f"{tag}_keys"], dt).to(DEV)
    vals = from_bits16(z[f"{tag}_vals"], dt).to(DEV)
    codec = tq.TurboQuantV3(128, device=DEV, **kw)
    ck, cv = codec.compress_kv(keys, vals)
    assert ck["split_at"] == int(z[f"{tag}_split"]) and ck["shape"] == tuple(keys.shape)
    if tag == "d":
        assert ck["compressed"] is None and ck["fp16"] is keys
    else:
        cut = ck["split_at"]
        assert ck["fp16"].shape[2] == keys.shape[2] - cut and ck["fp16"].dtype == dt
        assert ck["fp16"].data_ptr() == keys[:, :, cut:, :].data_ptr() or ck["fp16"].numel() == 0   # a view, not a copy
        for c, nm, bits, comp in ((ck, "k", codec.key_bits, codec.key_compressor), (cv, "v", codec.value_bits, codec.val_compressor)):
            src = (keys if nm == "k" else vals)[:, :, :cut, :].cpu().contiguous()
            cent, bnd = O.lloyd_max(128, bits)
            norms, _ = check_indices(c["compressed"]["idx_bytes"], src, comp.Pi.cpu(), cent, bnd, bits, 128)
            check_norms(c["compressed"]["vec_norms"], norms)
            gold = O.unpack_indices(z[f"{tag}_{nm}_idx"].reshape(-1, z[f"{tag}_{nm}_idx"].shape[-1]), bits, 128)
            mine = O.unpack_indices(c["compressed"]["idx_bytes"].cpu().numpy().reshape(gold.shape[0], -1), bits, 128)
            diff = np.abs(gold.astype(np.int32) - mine.astype(np.int32))
            assert diff.max() <= 1 and (diff != 0).sum() <= max(2, int(np.ceil(1e-4 * gold.size)))
    rk, rv = codec.decompress_kv(ck, cv)
    assert rk.dtype == dt and rk.shape == keys.shape and rv.shape == vals.shape
    for got, want in ((rk, from_bits16(z[f"{tag}_rk"], dt)), (rv, from_bits16(z[f"{tag}_rv"], dt))):
        # the fixture holds the reference's own 16-bit output: per vector within 2e-3 of the largest value
        # plus the final rounding of the format (one unit in the last place between two roundings)
        g, w = got.float().cpu(), want.float()
        eps = 2.0 ** -7 if dt == torch.bfloat16 else 2.0 ** -10
        bound = 2e-3 * w.abs().amax(-1, keepdim=True) + eps * w.abs() + 1e-30
        assert bool(((g - w).abs() <= bound).all()), float(((g - w).abs() / bound).max())
    if tag != "d":
        cut = ck["split_at"]
        assert torch.equal(rk[:, :, cut:], keys[:, :, cut:]) and torch.equal(rv[:, :, cut:], vals[:, :, cut:])


def test_batched_layers_equal_per_layer_calls():
    L = 5
    codecs = [tq.TurboQuantV3(128, key_bits=4, value_bits=2, residual_window=8, layer_idx=l, n_layers=L, protected_layers=1,
                              device=DEV) for l in range(L)]
    keys = [O.synthetic_kv((1, 2, 200, 128), torch.float16, 100 + l).to(DEV) for l in range(L)]
    vals = [O.synthetic_kv((1, 2, 200, 128), torch.float16, 200 + l).to(DEV) for l in range(L)]
    many = batched.compress_kv_layers(codecs, keys, vals)
    for l in range(L):
        ck, cv = codecs[l].compress_kv(keys[l], vals[l])
        assert torch.equal(many[l][0]["compressed"]["idx_bytes"], ck["compressed"]["idx_bytes"])
        assert torch.equal(many[l][1]["compressed"]["vec_norms"], cv["compressed"]["vec_norms"])
    outs = batched.decompress_kv_layers(codecs, many)
    for l in range(L):
        rk, rv = codecs[l].decompress_kv(*many[l])
        assert torch.equal(outs[l][0], rk) and torch.equal(outs[l][1], rv)


# --------------------------------------------------------------------------- K3
def test_packed_key_scores_against_golden_and_oracle():
    z = load_golden("scores.npz")
    comp = tq.MSECompressor(128, 4, seed=42, device=DEV)
    gold = {"idx_bytes": torch.from_numpy(z["idx"]).to(DEV), "vec_norms": from_bits16(z["norms"], torch.float16).to(DEV),
            "shape": (1, 2, 256, 128), "idx_pad": 0}
    q = torch.from_numpy(z["q"]).to(DEV)
    logits, probs = comp.attention_scores(q, gold, softmax=True)
    assert logits.shape == (1, 8, 1, 256) and logits.dtype == torch.float32
    assert rel_err(logits, torch.from_numpy(z["logits"])) <= 1e-5
    assert np.allclose(probs.cpu().numpy(), z["probs"], rtol=2e-4, atol=1e-7)
    only = comp.attention_scores(q, gold, scale=0.5)
    assert torch.allclose(only, logits * 0.5, rtol=1e-6, atol=0)


@pytest.mark.parametrize("bits,d,hq,hkv,sq,sk", [(4, 128, 8, 2, 3, 3000), (2, 128, 4, 4, 1, 1500), (8, 64, 6, 2, 5, 700),
                                                 (3, 128, 2, 1, 1, 1025), (6, 256, 4, 2, 2, 520)])
def test_packed_key_scores_general_shapes(bits, d, hq, hkv, sq, sk):
    keys = O.synthetic_kv((2, hkv, sk, d), torch.float16, seed=bits * 100 + d)
    q = torch.randn(2, hq, sq, d, generator=torch.Generator().manual_seed(3))
    comp = tq.MSECompressor(d, bits, seed=9, device=DEV)
    c = comp.compress(keys.to(DEV))
    logits, probs = comp.attention_scores(q.to(DEV), c, softmax=True)
    rec = comp.decompress(c).cpu()
    want = O.v3_scores(q, rec)
    assert rel_err(logits, want) <= 1e-5
    assert torch.allclose(probs.cpu(), torch.softmax(want, -1), rtol=2e-4, atol=1e-7)
    assert torch.allclose(probs.sum(-1).cpu(), torch.ones(2, hq, sq), atol=1e-4)


# --------------------------------------------------------------------------- V2
def test_v2_compress_and_scores_against_golden():
    z = load_golden("v2.npz")
    for tag in "abc":
        d, bits, seed, sq = z[f"{tag}_meta"].tolist()
        x = from_bits16(z[f"{tag}_x"], torch.float16)
        q = torch.from_numpy(z[f"{tag}_q"])
        comp = tq.TurboQuantCompressorV2(d, bits, seed=seed, device=DEV)
        assert comp.mse_bits == max(bits - 1, 1) and comp.S.shape == (d, d) and comp.PiT.shape == (d, d)
        c = comp.compress(x.to(DEV))
        assert c["k_mse"].dtype == torch.float16 and c["qjl_signs"].dtype == torch.int8
        assert c["residual_norm"].dtype == torch.float16 and c["shape"] == tuple(x.shape)
        check_v2_compress(c, x, comp.Pi.cpu(), comp.centroids.cpu(), comp.S.cpu())
        gold = {"k_mse": from_bits16(z[f"{tag}_kmse"], torch.float16).to(DEV), "qjl_signs": torch.from_numpy(z[f"{tag}_signs"]).to(DEV),
                "residual_norm": from_bits16(z[f"{tag}_rnorm"], torch.float16).to(DEV), "shape": tuple(x.shape)}
        sc = comp.asymmetric_attention_scores(q.to(DEV), gold)
        assert sc.shape == z[f"{tag}_scores"].shape and rel_err(sc, torch.from_numpy(z[f"{tag}_scores"])) <= 1e-5
    x = from_bits16(z["m_x"], torch.float16)
    comp = tq.TurboQuantCompressorMSE(128, 2, seed=9, device=DEV)
    c = comp.compress(x.to(DEV))
    assert c["indices"].dtype == torch.uint8 and tuple(c["indices"].shape) == (64, 128) and c["vec_norms"].shape == (64,)
    few_neighbour_mismatches(c["indices"].cpu().numpy(), z["m_idx"])
    gold = {"indices": torch.from_numpy(z["m_idx"]).to(DEV), "vec_norms": from_bits16(z["m_norms"], torch.float16).to(DEV),
            "shape": (1, 2, 32, 128)}
    assert rel_err(comp.decompress(gold), torch.from_numpy(z["m_rec"])) <= 1e-5


def test_v2_scores_head_dim_256_many_queries():
    x = O.synthetic_kv((1, 2, 300, 256), torch.float16, seed=50001, outlier_channels=0)
    q = torch.randn(1, 2, 64, 256, generator=torch.Generator().manual_seed(8))
    comp = tq.TurboQuantCompressorV2(256, 3, seed=21, device=DEV)
    c = comp.compress(x.to(DEV))
    sc = comp.asymmetric_attention_scores(q.to(DEV), c)
    want = O.v2_scores(q, {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in c.items()}, comp.S.cpu())
    assert rel_err(sc, want) <= 1e-5
    true = torch.matmul(q, x.float().transpose(-2, -1))
    err = sc.cpu() - true
    assert abs(float(err.mean())) < 0.15 * float(true.std())          # unbiased estimator
    q16 = q.half()
    sc16 = comp.asymmetric_attention_scores(q16.to(DEV), c)
    assert rel_err(sc16, O.v2_scores(q16, {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in c.items()}, comp.S.cpu())) <= 1e-5


# --------------------------------------------------------------------------- V1
def test_v1_classes_against_golden():
    z = load_golden("v1.npz")
    x, y = torch.from_numpy(z["x"]), torch.from_numpy(z["y"])
    mse = tq.TurboQuantMSE(128, 3, seed=42, device=DEV)
    assert rel_err(mse.rotate(x.to(DEV)), torch.from_numpy(z["mse_rot"])) <= 1e-5
    xh, idx = mse(x.to(DEV))
    assert idx.dtype == torch.int64 and idx.shape == (32, 128)
    few_neighbour_mismatches(idx.cpu().numpy(), z["mse_idx"])
    assert rel_err(mse.dequantize(torch.from_numpy(z["mse_idx"]).to(DEV)), torch.from_numpy(z["mse_xhat"])) <= 1e-5
    assert rel_err(mse.unrotate(mse.rotate(x.to(DEV))), x) <= 1e-5
    one = mse.quantize(x[0].to(DEV))
    assert one.shape == (128,) and torch.equal(one, idx[0])

    prod = tq.TurboQuantProd(128, 3, seed=42, device=DEV)
    c = prod.quantize(x.to(DEV))
    assert c["mse_indices"].dtype == torch.int64 and c["qjl_signs"].dtype == torch.float32
    assert c["qjl_signs"].shape == (32, 128) and c["residual_norm"].shape == (32,)
    rows = few_neighbour_mismatches(c["mse_indices"].cpu().numpy(), z["prod_idx"])
    signs_equal_outside(c["qjl_signs"].cpu().numpy(), z["prod_signs"], rows)
    assert np.allclose(c["residual_norm"].cpu().numpy()[~rows], z["prod_rnorm"][~rows], rtol=1e-4)
    gold = {"mse_indices": torch.from_numpy(z["prod_idx"]).to(DEV), "qjl_signs": torch.from_numpy(z["prod_signs"]).to(DEV),
            "residual_norm": torch.from_numpy(z["prod_rnorm"]).to(DEV)}
    ip = prod.inner_product(y.to(DEV), gold)
    assert ip.shape == (32,) and rel_err(ip, torch.from_numpy(z["prod_ip"])) <= 1e-5
    single = prod.inner_product(y[:1].to(DEV).expand(32, -1), gold)
    want1 = O.v1_prod_inner_product(y[:1].expand(32, -1), {k: v.cpu() for k, v in gold.items()}, prod.mse.Pi.cpu(),
                                    prod.mse.centroids.cpu(), prod.S.cpu())
    assert rel_err(single, want1) <= 1e-5

    prod64 = tq.TurboQuantProd(128, 4, qjl_dim=64, seed=3, device=DEV)
    c64 = prod64.quantize(x.to(DEV))
    assert c64["qjl_signs"].shape == (32, 64)
    signs_equal_outside(c64["qjl_signs"].cpu().numpy(), z["prod64_signs"], np.zeros(32, dtype=bool))
    gold64 = {"mse_indices": c64["mse_indices"], "qjl_signs": torch.from_numpy(z["prod64_signs"]).to(DEV),
              "residual_norm": c64["residual_norm"]}
    assert rel_err(prod64.inner_product(y.to(DEV), gold64), torch.from_numpy(z["prod64_ip"])) <= 1e-3

    cache = tq.TurboQuantKVCache(128, 128, bits=3, seed=42, device=DEV)
    kv = torch.from_numpy(z["cache_kv"]).to(DEV)
    cache.append(kv[:, :24], kv[:, :24] * 0.5)
    cache.append(kv[0, 24:], kv[0, 24:] * 2.0)
    assert len(cache) == int(z["cache_len"])
    mu = cache.memory_usage_bits()
    assert [mu["key_bits"], mu["value_bits"], mu["total_bits"], mu["fp16_bits"]] == z["cache_mem"].tolist()
    sc = cache.attention_scores(torch.from_numpy(z["cache_q"]).to(DEV))
    assert sc.shape == z["cache_scores"].shape
    assert rel_err(sc, torch.from_numpy(z["cache_scores"])) <= 2e-2      # a few indices/signs may flip
    vals = cache.get_values()
    assert vals.shape == z["cache_values"].shape
    assert float(((vals.cpu() - torch.from_numpy(z["cache_values"])) ** 2).mean()) < 1e-3


def test_cache_plan_equals_per_layer_calls_and_can_rerun():
    L = 4
    codecs = [tq.TurboQuantV3(128, key_bits=4, value_bits=2, residual_window=16, layer_idx=l, n_layers=L, protected_layers=1,
                              device=DEV) for l in range(L)]
    keys = [O.synthetic_kv((1, 2, 300, 128), torch.float16, 700 + l).to(DEV) for l in range(L)]
    vals = [O.synthetic_kv((1, 2, 300, 128), torch.float16, 750 + l).to(DEV) for l in range(L)]
    plan = batched.CachePlan(codecs, keys, vals)
    for _ in range(2):                      # the second pass overwrites the same buffers
        packed = plan.compress()
        outs = plan.decompress()
    for l in range(L):
        ck, cv = codecs[l].compress_kv(keys[l], vals[l])
        assert torch.equal(packed[l][0]["compressed"]["idx_bytes"], ck["compressed"]["idx_bytes"])
        assert torch.equal(packed[l][1]["compressed"]["vec_norms"], cv["compressed"]["vec_norms"])
        rk, rv = codecs[l].decompress_kv(ck, cv)
        assert torch.equal(outs[l][0], rk) and torch.equal(outs[l][1], rv)
    keys[0].mul_(0.5)                        # inputs changed in place: window must be refreshed by the caller
    plan.compress(); plan.refresh_window(); plan.decompress()
    rk, _ = codecs[0].decompress_kv(*codecs[0].compress_kv(keys[0], vals[0]))
    assert torch.equal(plan.reconstructed[0][0], rk)


@pytest.mark.gpu
def test_host_streamed_cache_equals_per_layer_calls():
    """Pinned-host round trip pipelined over layer groups: same bytes as per-layer calls, also on reuse."""
    from turboquant import batched
    L = 5
    codecs = [tq.TurboQuantV3(128, key_bits=4, value_bits=2, residual_window=16, layer_idx=l, n_layers=L, protected_layers=1,
                              device=DEV) for l in range(L)]
    hk = [O.synthetic_kv((1, 2, 300, 128), torch.float16, 800 + l).pin_memory() for l in range(L)]
    hv = [O.synthetic_kv((1, 2, 300, 128), torch.float16, 850 + l).pin_memory() for l in range(L)]
    with pytest.raises(ValueError):
        batched.HostStreamedCache(codecs, [t.clone() for t in hk], hv, DEV)       # not pinned
    cache = batched.HostStreamedCache(codecs, hk, hv, DEV, groups=3)
    for rep in range(2):
        if rep == 1:                          # new contents in the same pinned tensors: buffers are reused
            for t in hk + hv:
                t.mul_(0.75)
        ok, ov = cache.run()
        torch.cuda.synchronize()
        for l in range(L):
            k, v = hk[l].to(DEV), hv[l].to(DEV)
            rk, rv = codecs[l].decompress_kv(*codecs[l].compress_kv(k, v))
            assert torch.equal(ok[l].to(DEV), rk) and torch.equal(ov[l].to(DEV), rv)


@pytest.mark.gpu
def test_incremental_cache_matches_reference_harness():
    """turboquant.cache.V3Cache against outputs of the reference's V3Cache (prefill, then one token per step)."""
    from turboquant.cache import V3Cache
    z = load_golden("v3_cache.npz")

    def frac_off(got, want, tol=2e-3):
        g, w = got.float().cpu(), want.float()
        return float(((g - w).abs() > tol * float(w.abs().max())).float().mean())

    for tag, rw, prefill in (("w", 16, 150), ("z", 0, 40)):
        cache = V3Cache(key_bits=4, value_bits=2, residual_window=rw, protected_layers=1, n_layers=4, initial_capacity=64)
        for layer in (0, 1):
            k = from_bits16(z[f"{tag}{layer}_k"], torch.float16).to(DEV)
            v = from_bits16(z[f"{tag}{layer}_v"], torch.float16).to(DEV)
            total = k.shape[2]
            fk, fv = cache.update(k[:, :, :prefill], v[:, :, :prefill], layer)
            assert frac_off(fk, from_bits16(z[f"{tag}{layer}_prefill_k"], torch.float16)) <= 1e-4
            assert frac_off(fv, from_bits16(z[f"{tag}{layer}_prefill_v"], torch.float16)) <= 1e-4
            for t in range(prefill, total):       # the buffer grows past its initial capacity on the way
                fk, fv = cache.update(k[:, :, t:t + 1], v[:, :, t:t + 1], layer)
            assert fk.shape == (1, 2, total, 128) and fk.dtype == torch.float16
            assert frac_off(fk, from_bits16(z[f"{tag}{layer}_full_k"], torch.float16)) <= 1e-4
            assert frac_off(fv, from_bits16(z[f"{tag}{layer}_full_v"], torch.float16)) <= 1e-4
            if rw:
                assert torch.equal(fk[:, :, -rw:], k[:, :, -rw:])
            assert cache.get_seq_length(layer) == int(z[f"{tag}{layer}_len"])
            ck, cv = cache.packed_chunks(layer)
            assert sum(c["shape"][2] for c in ck) == total - (rw if rw else 0)
            mem = cache.memory_bytes(layer)
            assert mem["fp16_bytes"] == 2 * 2 * total * 128 * 2 and mem["compression_ratio"] > 1.5
        assert cache.get_compression_info() == str(z[f"{tag}_info"])


@pytest.mark.gpu
@pytest.mark.parametrize("d,sq,sk,bh", [(128, 70, 1000, 6), (256, 5, 129, 3), (128, 1, 128, 2)])
def test_v2_scores_tensor_core_shapes(d, sq, sk, bh):
    """Asymmetric scores on the tensor-core path: several query blocks, ragged key tiles, both head_dims;
    checked against the oracle and against the FP32 kernels (TQ_FORCE_SIMT=1)."""
    import os
    x = O.synthetic_kv((1, bh, sk, d), torch.float16, seed=52000 + d + sq, outlier_channels=0)
    q = torch.randn(1, bh, sq, d, generator=torch.Generator().manual_seed(sq))
    comp = tq.TurboQuantCompressorV2(d, 3, seed=5, device=DEV)
    c = comp.compress(x.to(DEV))
    sc = comp.asymmetric_attention_scores(q.to(DEV), c)
    want = O.v2_scores(q, {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in c.items()}, comp.S.cpu())
    assert sc.shape == (1, bh, sq, sk) and rel_err(sc, want) <= 1e-5
    os.environ["TQ_FORCE_SIMT"] = "1"
    try:
        sc_simt = comp.asymmetric_attention_scores(q.to(DEV), c)
    finally:
        del os.environ["TQ_FORCE_SIMT"]
    assert rel_err(sc, sc_simt) <= 1e-5
    from turboquant import _native
    assert _native.lib().tq_last_device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("bits,hq,hkv,sq,sk", [(4, 8, 2, 1, 1000), (2, 4, 4, 3, 129), (8, 16, 1, 1, 300), (3, 2, 2, 8, 77),
                                                (6, 32, 8, 1, 2048), (4, 8, 2, 5, 500)])
def test_packed_scores_shapes_and_widths(bits, hq, hkv, sq, sk):
    """Logits and softmax from packed keys for several code widths, GQA group sizes, query counts and ragged key
    counts, against the oracle composition (decompress + matmul)."""
    keys = O.synthetic_kv((2, hkv, sk, 128), torch.float16, seed=53000 + bits + sk)
    q = torch.randn(2, hq, sq, 128, generator=torch.Generator().manual_seed(bits * 10 + sq))
    comp = tq.MSECompressor(128, bits, seed=77, device=DEV)
    c = comp.compress(keys.to(DEV))
    logits, probs = comp.attention_scores(q.to(DEV), c, scale=0.25, softmax=True)
    rec = comp.decompress(c).cpu()
    want = O.v3_scores(q, rec) * 0.25
    assert logits.shape == (2, hq, sq, sk) and rel_err(logits, want) <= 1e-5
    assert torch.allclose(probs.cpu(), torch.softmax(want, -1), rtol=2e-4, atol=1e-7)


@pytest.mark.gpu
@pytest.mark.parametrize("d,bits,shape", [(128, 3, (1, 2, 300, 128)), (256, 3, (2, 3, 77, 256)), (256, 5, (1, 1, 513, 256)),
                                          (128, 2, (1, 4, 128, 128))])
def test_v2_compress_tensor_core_against_fp32_kernels(d, bits, shape):
    """MSE+QJL compress on the tensor-core path (fp16, head_dim 128/256) against the oracle and the FP32 kernels:
    ragged tile counts, several widths of the MSE stage."""
    import os
    x = O.synthetic_kv(shape, torch.float16, seed=54000 + d + bits, outlier_channels=0)
    comp = tq.TurboQuantCompressorV2(d, bits, seed=13, device=DEV)
    c = comp.compress(x.to(DEV))
    want = O.v2_compress(x, comp.Pi.cpu(), comp.centroids.cpu(), comp.S.cpu())
    assert c["k_mse"].shape == x.shape and c["qjl_signs"].shape == x.shape and c["residual_norm"].shape == x.shape[:3]
    marked = check_v2_compress(c, x, comp.Pi.cpu(), comp.centroids.cpu(), comp.S.cpu())

    def vectors_close(a, b):
        a, b = a.float().cpu(), b.float().cpu()
        return (a - b).abs().amax(-1) <= 2e-3 * b.abs().amax(-1) + 1e-30

    os.environ["TQ_FORCE_SIMT"] = "1"
    try:
        c2 = comp.compress(x.to(DEV))
    finally:
        del os.environ["TQ_FORCE_SIMT"]
    # the FP32 kernels as a second opinion: they may differ only on vectors with a coordinate on a boundary
    marked2 = check_v2_compress(c2, x, comp.Pi.cpu(), comp.centroids.cpu(), comp.S.cpu())
    differ = ~vectors_close(c["k_mse"], c2["k_mse"])
    assert int(differ.sum()) <= marked + marked2
    from turboquant import _native
    assert _native.lib().tq_last_device_status() == 0


@pytest.mark.gpu
def test_cache_plan_replays_as_a_cuda_graph():
    """compress + decompress of a whole cache captured once and replayed on new contents of the same buffers."""
    from turboquant import batched
    L = 3
    codecs = [tq.TurboQuantV3(128, key_bits=4, value_bits=2, residual_window=0, layer_idx=l, n_layers=L, protected_layers=0,
                              device=DEV) for l in range(L)]
    keys = [O.synthetic_kv((1, 2, 384, 128), torch.float16, 900 + l).to(DEV) for l in range(L)]
    vals = [O.synthetic_kv((1, 2, 384, 128), torch.float16, 950 + l).to(DEV) for l in range(L)]
    plan = batched.CachePlan(codecs, keys, vals)
    graph = plan.capture()
    for t in keys + vals:                      # new contents, same storage
        t.mul_(-0.5)
    for ck, cv in plan.compressed:             # poison the outputs: the replay must rewrite them
        ck["compressed"]["idx_bytes"].fill_(255)
        cv["compressed"]["vec_norms"].zero_()
    for rk, rv in plan.reconstructed:
        rk.zero_(); rv.zero_()
    graph.replay()
    torch.cuda.synchronize()
    for l in range(L):
        ck, cv = codecs[l].compress_kv(keys[l], vals[l])
        assert torch.equal(plan.compressed[l][0]["compressed"]["idx_bytes"], ck["compressed"]["idx_bytes"])
        assert torch.equal(plan.compressed[l][1]["compressed"]["vec_norms"], cv["compressed"]["vec_norms"])
        rk, rv = codecs[l].decompress_kv(ck, cv)
        assert torch.equal(plan.reconstructed[l][0], rk) and torch.equal(plan.reconstructed[l][1], rv)


@pytest.mark.gpu
def test_v2_tensor_core_edge_shapes():
    """One vector, one key, a zero vector: the tensor-core V2 kernels against the oracle."""
    for d in (128, 256):
        comp = tq.TurboQuantCompressorV2(d, 3, seed=3, device=DEV)
        x = O.synthetic_kv((1, 1, 3, d), torch.float16, seed=55000 + d, outlier_channels=0)
        x[0, 0, 1] = 0                                  # zero vector: norm 0, every sign +1
        for s in (1, 3):
            xs = x[:, :, :s].contiguous()
            c = comp.compress(xs.to(DEV))
            want = O.v2_compress(xs, comp.Pi.cpu(), comp.centroids.cpu(), comp.S.cpu())
            check_v2_compress(c, xs, comp.Pi.cpu(), comp.centroids.cpu(), comp.S.cpu(), max_differing=0)
            if s == 3:
                assert bool((c["qjl_signs"][0, 0, 1] == 1).all()) and float(c["k_mse"][0, 0, 1].abs().max()) == 0.0
            q = torch.randn(1, 1, 2, d, generator=torch.Generator().manual_seed(s))
            sc = comp.asymmetric_attention_scores(q.to(DEV), c)
            ref = O.v2_scores(q, {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in c.items()}, comp.S.cpu())
            assert sc.shape == (1, 1, 2, s) and rel_err(sc, ref) <= 1e-5
    from turboquant import _native
    assert _native.lib().tq_last_device_status() == 0


@pytest.mark.gpu
def test_v2_compress_other_layouts_use_the_fp32_kernels():
    """Inputs the tensor-core path does not take (a strided view, bf16 and fp32 vectors) give the same results
    through the FP32 kernels."""
    comp = tq.TurboQuantCompressorV2(128, 3, seed=17, device=DEV)
    base = O.synthetic_kv((1, 2, 96, 128), torch.float16, seed=56000, outlier_channels=0)
    for x in (base[:, :, ::2], base.to(torch.bfloat16), base.float()):
        c = comp.compress(x.to(DEV) if x.is_contiguous() else base.to(DEV)[:, :, ::2])
        want = O.v2_compress(x, comp.Pi.cpu(), comp.centroids.cpu(), comp.S.cpu())
        assert c["k_mse"].shape == x.shape
        check_v2_compress(c, x.contiguous(), comp.Pi.cpu(), comp.centroids.cpu(), comp.S.cpu())
