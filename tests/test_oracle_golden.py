"""Pin the CPU oracle against golden vectors produced by the reference itself.

Floating-point stages that go through a BLAS call may differ in the last bit
between CPU models, so those comparisons allow index flips only where the stored
rotated value sits within 1e-6 of a decision boundary; integer stages and stages
fed from stored intermediates must match bit for bit.
"""

import hashlib

import numpy as np
import pytest
import torch

import tq_oracle as O
from conftest import load_golden, from_bits16, bits16


def _sha(t):
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def _ulp16_close(a_bits, b_bits, ulps=1):
    a = a_bits.astype(np.int32)
    b = b_bits.astype(np.int32)
    return np.all(np.abs(a - b) <= ulps)


def _idx_agreement(got_packed, want_packed, bits, d):
    g = O.unpack_indices(got_packed.reshape(-1, got_packed.shape[-1]), bits, d)
    w = O.unpack_indices(want_packed.reshape(-1, want_packed.shape[-1]), bits, d)
    return (g == w).mean(), g, w


@pytest.mark.parametrize("d", [64, 128, 256])
@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6])
def test_codebooks_bit_exact(d, bits):
    z = load_golden("codebooks.npz")
    c, b = O.lloyd_max(d, bits)
    assert np.array_equal(c.numpy().view(np.uint32), z[f"c_{d}_{bits}"].view(np.uint32))
    assert np.array_equal(b.numpy().view(np.uint32), z[f"b_{d}_{bits}"].view(np.uint32))
    dist = O.expected_distortion(d, bits, c, b)
    assert dist == pytest.approx(float(z[f"dist_{d}_{bits}"]), rel=1e-12)


def test_codebook_8bit_and_exact_and_v2_variant():
    z = load_golden("codebooks.npz")
    c, b = O.lloyd_max(128, 8)
    assert np.array_equal(c.numpy().view(np.uint32), z["c_128_8"].view(np.uint32))
    for d, bits in ((128, 2), (64, 3)):
        c, b = O.lloyd_max(d, bits, use_exact=True)
        assert np.array_equal(c.numpy(), z[f"cx_{d}_{bits}"])
        assert np.array_equal(b.numpy(), z[f"bx_{d}_{bits}"])
    for d, bits in ((128, 1), (128, 2), (128, 3), (128, 4), (256, 2), (64, 2)):
        assert np.array_equal(O.lloyd_max_v2(d, bits).numpy(), z[f"v2c_{d}_{bits}"])


def test_codebook_symmetry_anchor():
    # the reference's only assert: sum(centroids) ~ 0 (test_turboquant.py:32-35)
    z = load_golden("codebooks.npz")
    for d in (64, 128, 256):
        for bits in range(1, 5):
            assert abs(float(z[f"c_{d}_{bits}"].sum())) < 0.01


def test_matrices():
    z = load_golden("matrices.npz")
    for d, seed in ((128, 0), (128, 42), (128, 542), (64, 7), (256, 42), (128, 3042)):
        pi = O.rotation_matrix(d, seed)
        assert np.allclose(pi[:2].numpy(), z[f"pi_rows_{d}_{seed}"], atol=2e-6)
        assert np.allclose(torch.diag(pi).numpy(), z[f"pi_diag_{d}_{seed}"], atol=2e-6)
        eye = pi.double() @ pi.double().T
        assert torch.allclose(eye, torch.eye(d, dtype=torch.float64), atol=1e-5)
    for d, m, seed in ((128, None, 43), (256, None, 10042), (128, 64, 5)):
        s = O.qjl_matrix(d, m, seed)
        assert _sha(s) == str(z[f"s_sha_{d}_{m}_{seed}"])   # pure RNG stream: bit exact


def test_cfg1_roundtrip():
    z = load_golden("cfg1.npz")
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(1, 1, 4096, 128, generator=g)
    assert _sha(x) == str(z["x_sha"])
    for tag, bits, seed in (("k", 4, 42), ("v", 2, 542)):
        pi = O.rotation_matrix(128, seed)
        cent = O.lloyd_max(128, bits)[0]
        c = O.mse_compress(x, pi, cent, bits)
        agree, _, _ = _idx_agreement(c["idx_bytes"].numpy(), z[f"{tag}_idx"], bits, 128)
        assert agree >= 0.9999
        assert c["idx_pad"] == int(z[f"{tag}_pad"])
        assert _ulp16_close(bits16(c["vec_norms"]), z[f"{tag}_norms"])
        gold = {"idx_bytes": torch.from_numpy(z[f"{tag}_idx"]), "vec_norms": from_bits16(z[f"{tag}_norms"], torch.float16),
                "shape": (1, 1, 4096, 128), "idx_pad": 0}
        rec = O.mse_decompress(gold, pi, cent, bits)
        want = torch.from_numpy(z[f"{tag}_rec_head"])
        assert torch.allclose(rec[0, 0, :64], want, rtol=0, atol=1e-5 * float(want.abs().max()))
        assert float(((rec - x) ** 2).sum(-1).mean()) == pytest.approx(float(z[f"{tag}_mse"]), rel=1e-5)
        mem = O.mse_memory_bytes(128, bits, 1, 1, 4096)
        assert [mem["compressed_bytes"], mem["fp16_bytes"]] == z[f"{tag}_mem"].tolist()
    assert O.mse_memory_bytes(128, 4, 1, 1, 4096)["compressed_bytes"] == 270336
    assert O.mse_memory_bytes(128, 2, 1, 1, 4096)["compressed_bytes"] == 139264


def test_small_cases_all_bits():
    z = load_golden("mse_small.npz")
    for d, bits, n in z["cases"].tolist():
        k = f"{d}_{bits}"
        x = torch.from_numpy(z[f"x_{k}"])
        rot = torch.from_numpy(z[f"rot_{k}"])
        pi = O.rotation_matrix(d, 17 + bits)
        cent, bnd = O.lloyd_max(d, bits)
        # integer stage from the stored rotated values: bit exact
        idx = O.nearest_centroid(rot, cent)
        packed, pad = O.pack_indices(idx.numpy(), bits)
        assert pad == int(z[f"pad_{k}"])
        assert np.array_equal(packed, z[f"idx_{k}"].reshape(n, -1)), k
        assert np.array_equal(O.unpack_indices(packed, bits, d), idx.numpy())
        # whole path
        c = O.mse_compress(x, pi, cent, bits)
        got = O.unpack_indices(c["idx_bytes"].reshape(n, -1).numpy(), bits, d)
        bad = np.argwhere(got != idx.numpy())
        for r, col in bad:
            assert np.min(np.abs(bnd.numpy() - rot[r, col].item())) < 1e-6
        assert len(bad) <= max(1, int(1e-4 * n * d))
        assert _ulp16_close(bits16(c["vec_norms"]).reshape(-1), z[f"norms_{k}"].reshape(-1))
        gold = {"idx_bytes": torch.from_numpy(z[f"idx_{k}"]), "vec_norms": from_bits16(z[f"norms_{k}"], torch.float16),
                "shape": tuple(x.shape), "idx_pad": pad}
        rec = O.mse_decompress(gold, pi, cent, bits)
        want = torch.from_numpy(z[f"rec_{k}"])
        assert torch.allclose(rec, want, rtol=0, atol=1e-5 * float(want.abs().max())), k


def test_v3_kv_cases():
    z = load_golden("v3_kv.npz")
    cases = {
        "a": (torch.float16, dict(key_bits=4, value_bits=2, residual_window=0, layer_idx=3, n_layers=36, protected_layers=0)),
        "b": (torch.bfloat16, dict(key_bits=6, value_bits=4, residual_window=16, layer_idx=0, n_layers=32, protected_layers=4)),
        "c": (torch.bfloat16, dict(key_bits=6, value_bits=4, residual_window=16, layer_idx=10, n_layers=32, protected_layers=4)),
        "d": (torch.float16, dict(key_bits=4, value_bits=2, residual_window=128, layer_idx=5, n_layers=36, protected_layers=4)),
    }
    cache = {}
    for tag, (dt, kw) in cases.items():
        keys = from_bits16(z[f"{tag}_keys"], dt)
        vals = from_bits16(z[f"{tag}_vals"], dt)
        tq = O.V3Oracle(128, codebook_cache=cache, **kw)
        assert [tq.key_bits, tq.value_bits] == z[f"{tag}_bits"].tolist()
        ck, cv = tq.compress_kv(keys, vals)
        assert ck["split_at"] == int(z[f"{tag}_split"])
        if tag == "d":
            assert ck["compressed"] is None and ck["fp16"] is keys
        else:
            for c, nm, bits in ((ck, "k", tq.key_bits), (cv, "v", tq.value_bits)):
                agree, _, _ = _idx_agreement(c["compressed"]["idx_bytes"].numpy(), z[f"{tag}_{nm}_idx"], bits, 128)
                assert agree >= 0.9999, (tag, nm)
                assert _ulp16_close(bits16(c["compressed"]["vec_norms"]), z[f"{tag}_{nm}_norms"])
        rk, rv = tq.decompress_kv(ck, cv)
        assert rk.dtype == dt and rk.shape == keys.shape
        for got, want in ((rk, from_bits16(z[f"{tag}_rk"], dt)), (rv, from_bits16(z[f"{tag}_rv"], dt))):
            err = (got.float() - want.float()).abs().max() / want.float().abs().max()
            assert float(err) <= 2e-3
        mem = tq.memory_bytes(*keys.shape[:3])
        assert [mem["compressed_bytes"], mem["fp16_bytes"], mem["compressed_tokens"], mem["fp16_tokens"]] \
            == z[f"{tag}_mem"].tolist()
    assert int(z["cfg2_packed_total"]) == 58982400


def test_edge_vectors():
    z = load_golden("edge.npz")
    x = torch.from_numpy(z["x"])
    pi, cent = O.rotation_matrix(128, 42), O.lloyd_max(128, 4)[0]
    c = O.mse_compress(x, pi, cent, 4)
    got, want = c["idx_bytes"].numpy(), z["idx"]
    # zero vector -> byte 0x77 everywhere; NaN / Inf rows -> index 0
    assert np.all(want[0, 0, 0] == 0x77) and np.all(want[0, 0, 1] == 0) and np.all(want[0, 0, 2] == 0)
    for row in (0, 1, 2, 5):
        assert np.array_equal(got[0, 0, row], want[0, 0, row])
    assert (got == want).mean() > 0.99
    assert np.array_equal(bits16(c["vec_norms"]), z["norms"])
    assert np.isinf(c["vec_norms"][0, 0, 3].item()) and np.isnan(c["vec_norms"][0, 0, 1].item())
    gold = {"idx_bytes": torch.from_numpy(want), "vec_norms": from_bits16(z["norms"], torch.float16),
            "shape": (1, 1, 8, 128), "idx_pad": 0}
    rec = O.mse_decompress(gold, pi, cent, 4).numpy()
    fin = np.isfinite(z["rec"])
    assert np.array_equal(np.isfinite(rec), fin)
    # the rotation comes out of a LAPACK QR whose last bits depend on the BLAS threading
    assert np.allclose(rec[fin], z["rec"][fin], rtol=0, atol=1e-5 * np.abs(z["rec"][fin]).max())


def test_v2_cases():
    z = load_golden("v2.npz")
    for tag in "abc":
        d, bits, seed, sq = z[f"{tag}_meta"].tolist()
        x = from_bits16(z[f"{tag}_x"], torch.float16)
        q = torch.from_numpy(z[f"{tag}_q"])
        pi = O.rotation_matrix(d, seed)
        cent = O.lloyd_max_v2(d, max(bits - 1, 1))
        s_mat = O.qjl_matrix(d, d, seed + 10000)
        c = O.v2_compress(x, pi, cent, s_mat)
        want_k = from_bits16(z[f"{tag}_kmse"], torch.float16).float()
        assert float((c["k_mse"].float() - want_k).abs().max()) <= 2e-3 * float(want_k.abs().max())
        assert (c["qjl_signs"].numpy() == z[f"{tag}_signs"]).mean() > 0.999
        assert c["qjl_signs"].dtype == torch.int8
        assert _ulp16_close(bits16(c["residual_norm"]), z[f"{tag}_rnorm"])
        gold = {"k_mse": from_bits16(z[f"{tag}_kmse"], torch.float16), "qjl_signs": torch.from_numpy(z[f"{tag}_signs"]),
                "residual_norm": from_bits16(z[f"{tag}_rnorm"], torch.float16), "shape": tuple(x.shape)}
        sc = O.v2_scores(q, gold, s_mat)
        want = torch.from_numpy(z[f"{tag}_scores"])
        assert torch.allclose(sc, want, rtol=0, atol=1e-5 * float(want.abs().max()))
    x = from_bits16(z["m_x"], torch.float16)
    pi, cent = O.rotation_matrix(128, 9), O.lloyd_max_v2(128, 2)
    c = O.v2mse_compress(x, pi, cent)
    assert c["indices"].dtype == torch.uint8 and tuple(c["indices"].shape) == (64, 128)
    assert (c["indices"].numpy() == z["m_idx"]).mean() >= 0.9999
    gold = {"indices": torch.from_numpy(z["m_idx"]), "vec_norms": from_bits16(z["m_norms"], torch.float16),
            "shape": (1, 2, 32, 128)}
    assert np.allclose(O.v2mse_decompress(gold, pi, cent).numpy(), z["m_rec"], rtol=0, atol=1e-5 * np.abs(z["m_rec"]).max())


def test_v1_cases():
    z = load_golden("v1.npz")
    x, y = torch.from_numpy(z["x"]), torch.from_numpy(z["y"])
    pi = O.rotation_matrix(128, 42)
    cent2, cent3 = O.lloyd_max(128, 2)[0], O.lloyd_max(128, 3)[0]
    idx = O.v1_mse_quantize(x, pi, cent3)
    assert idx.dtype == torch.int64
    assert (idx.numpy() == z["mse_idx"]).mean() >= 0.9999
    xh = O.v1_mse_dequantize(torch.from_numpy(z["mse_idx"]), pi, cent3)
    assert np.allclose(xh.numpy(), z["mse_xhat"], atol=1e-6)
    s_mat = O.qjl_matrix(128, 128, 43)
    c = O.v1_prod_quantize(x, pi, cent2, s_mat)
    assert (c["mse_indices"].numpy() == z["prod_idx"]).mean() >= 0.9999
    assert (c["qjl_signs"].numpy() == z["prod_signs"]).mean() > 0.999
    assert c["qjl_signs"].dtype == torch.float32
    assert np.allclose(c["residual_norm"].numpy(), z["prod_rnorm"], rtol=1e-5)
    gold = {"mse_indices": torch.from_numpy(z["prod_idx"]), "qjl_signs": torch.from_numpy(z["prod_signs"]),
            "residual_norm": torch.from_numpy(z["prod_rnorm"])}
    ip = O.v1_prod_inner_product(y, gold, pi, cent2, s_mat)
    assert np.allclose(ip.numpy(), z["prod_ip"], rtol=0, atol=1e-5 * np.abs(z["prod_ip"]).max())


def test_packed_scores():
    z = load_golden("scores.npz")
    keys = from_bits16(z["keys"], torch.float16)
    q = torch.from_numpy(z["q"])
    pi, cent = O.rotation_matrix(128, 42), O.lloyd_max(128, 4)[0]
    gold = {"idx_bytes": torch.from_numpy(z["idx"]), "vec_norms": from_bits16(z["norms"], torch.float16),
            "shape": tuple(keys.shape), "idx_pad": 0}
    rec = O.mse_decompress(gold, pi, cent, 4)
    logits = O.v3_scores(q, rec)
    want = torch.from_numpy(z["logits"])
    assert torch.allclose(logits, want, rtol=0, atol=1e-5 * float(want.abs().max()))
    assert np.allclose(torch.softmax(logits, -1).numpy(), z["probs"], rtol=1e-4, atol=1e-7)


def test_pack_layout_msb_first():
    idx = np.array([[1, 2, 3, 0, 3, 3, 0, 1]])
    p, pad = O.pack_indices(idx, 2)
    assert pad == 0 and p.tolist() == [[0b01101100, 0b11110001]]
    p, pad = O.pack_indices(np.array([[5, 6, 7]]), 3)   # two 3-bit fields per byte, one zero pad
    assert pad == 1 and p.tolist() == [[(5 << 3) | 6, 7 << 3]]
    p, pad = O.pack_indices(np.array([[200, 3]]), 8)
    assert pad == 0 and p.tolist() == [[200, 3]]
    p, pad = O.pack_indices(np.array([[1, 0, 1]]), 1)
    assert pad == 5 and p.tolist() == [[0b10100000]]


def _frac_off(got, want, tol=2e-3):
    """Fraction of elements further than tol * max|want| from the fixture (an index that flips moves one element)."""
    g, w = got.float(), want.float()
    return float(((g - w).abs() > tol * float(w.abs().max())).float().mean())


def test_v3_cache_prefill_and_decode_steps():
    """The incremental cache of the generation harness: same tokens in, same full K/V out after every phase."""
    z = load_golden("v3_cache.npz")
    for tag, rw, prefill in (("w", 16, 150), ("z", 0, 40)):
        cache = O.V3CacheOracle(key_bits=4, value_bits=2, residual_window=rw, protected_layers=1, n_layers=4)
        for layer in (0, 1):
            k = from_bits16(z[f"{tag}{layer}_k"], torch.float16)
            v = from_bits16(z[f"{tag}{layer}_v"], torch.float16)
            total = k.shape[2]
            fk, fv = cache.update(k[:, :, :prefill], v[:, :, :prefill], layer)
            assert _frac_off(fk, from_bits16(z[f"{tag}{layer}_prefill_k"], torch.float16)) <= 1e-4
            assert _frac_off(fv, from_bits16(z[f"{tag}{layer}_prefill_v"], torch.float16)) <= 1e-4
            for t in range(prefill, total):
                fk, fv = cache.update(k[:, :, t:t + 1], v[:, :, t:t + 1], layer)
            assert fk.shape == (1, 2, total, 128) and fk.dtype == torch.float16
            assert _frac_off(fk, from_bits16(z[f"{tag}{layer}_full_k"], torch.float16)) <= 1e-4
            assert _frac_off(fv, from_bits16(z[f"{tag}{layer}_full_v"], torch.float16)) <= 1e-4
            if rw:                                  # the window tokens pass through untouched
                assert torch.equal(fk[:, :, -rw:], k[:, :, -rw:])
            assert cache.get_seq_length(layer) == int(z[f"{tag}{layer}_len"])
        assert cache.get_compression_info() == str(z[f"{tag}_info"])
