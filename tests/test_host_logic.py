"""Host-side logic that needs no GPU: the C ABI surface, exact decision thresholds,
accounting, layer-adaptive widths, error behaviour, sharding."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

import tq_oracle as O
from conftest import ROOT, load_golden

import turboquant as tq
from turboquant import _native as N
from turboquant import batched, lloyd_max


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "turboquant_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = N.lib()
    names = _declared_functions()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), name
    assert lib.tq_version() >= 100
    assert lib.tq_strerror(0) == b"ok"
    assert b"bits" in lib.tq_strerror(-2)


def test_argument_checks_do_not_touch_the_gpu():
    lib = N.lib()
    assert lib.tq_packed_row_bytes(128, 4) == 64
    assert lib.tq_packed_row_bytes(128, 3) == 64      # two 3-bit fields per byte
    assert lib.tq_packed_row_bytes(128, 5) == 128
    assert lib.tq_packed_row_bytes(100, 1) == 13
    assert lib.tq_packed_row_bytes(128, 9) == -2
    assert lib.tq_packed_row_bytes(0, 4) == -3
    assert lib.tq_quantize(None, 1, None) == -4
    assert lib.tq_quantize(None, 0, None) == 0
    assert lib.tq_quantize(None, -1, None) == -1
    job = N.QuantizeJob(D=128, bits=11, B=1, H=1, S=1)
    assert lib.tq_quantize(ctypes.byref(job), 1, None) == -2
    job = N.QuantizeJob(D=512, bits=4, B=1, H=1, S=1)
    assert lib.tq_quantize(ctypes.byref(job), 1, None) == -3
    job = N.QuantizeJob(D=128, bits=4, B=1, H=1, S=1, x_dtype=7)
    assert lib.tq_quantize(ctypes.byref(job), 1, None) == -6
    job = N.QuantizeJob(D=128, bits=4, B=1, H=1, S=1)          # null pointers
    assert lib.tq_quantize(ctypes.byref(job), 1, None) == -4
    job = N.QuantizeJob(D=128, bits=4, B=1, H=1, S=0)          # empty job is fine
    assert lib.tq_quantize(ctypes.byref(job), 1, None) == 0
    assert lib.tq_dequantize(None, 2, None) == -4
    assert lib.tq_project(None, 0, 0, 128, None, 128, None, None) == 0
    assert lib.tq_project(None, 0, 4, 300, None, 128, None, None) == -3
    sj = N.ScoreJob(D=128, bits=4, B=1, Hq=6, Sq=1, Hkv=4, Sk=8)
    assert lib.tq_score_packed(ctypes.byref(sj), None) == -1   # Hq not a multiple of Hkv
    with pytest.raises(ValueError):
        N.check(-3, "x")
    with pytest.raises(ZeroDivisionError):
        N.check(-2, "x")
    with pytest.raises(RuntimeError):
        N.check(-7, "x")


def _argmin_f32(y, c):
    y = np.asarray(y, dtype=np.float32)
    return np.abs(y[:, None] - c[None, :].astype(np.float32)).argmin(axis=1)


@pytest.mark.parametrize("d", [64, 128, 256])
def test_thresholds_reproduce_fp32_argmin(d):
    z = load_golden("codebooks.npz")
    rng = np.random.default_rng(d)
    for bits in range(1, 9):
        c = z[f"c_{d}_{bits}"]
        block = N.codebook_block(torch.from_numpy(c), bits).numpy()
        L = 2 ** bits
        thr = block[256:256 + L - 1]
        assert np.array_equal(block[:L], c) and np.all(np.isinf(block[L:256])) and np.all(np.isinf(block[256 + L - 1:512]))
        assert np.all(np.diff(thr) > 0)
        assert np.allclose(thr, z[f"b_{d}_{bits}"], atol=1e-7)
        # every float within +-16 ulp of each threshold, plus random draws and specials
        probes = [rng.normal(0, 1 / np.sqrt(d), 20000).astype(np.float32),
                  np.array([0.0, -0.0, 1.0, -1.0, 1e-30, -1e-30, 8.0, -8.0, 100.0, -100.0], dtype=np.float32), c]
        for t in thr:
            v = np.float32(t)
            lo = v
            for _ in range(16):
                lo = np.nextafter(lo, np.float32(-np.inf))
            run = [lo]
            for _ in range(32):
                run.append(np.nextafter(run[-1], np.float32(np.inf)))
            probes.append(np.array(run, dtype=np.float32))
        y = np.concatenate(probes)
        want = _argmin_f32(y, c)
        got = (y[:, None] > thr[None, :]).sum(axis=1)
        assert np.array_equal(got, want), (d, bits)
    assert (np.float32(np.nan) > thr).sum() == 0     # NaN lands on index 0, like argmin over NaNs


def test_codebook_block_rejects_unsorted():
    with pytest.raises(ValueError):
        N.codebook_block(torch.tensor([0.1, 0.1, 0.2, 0.3]), 2)
    with pytest.raises(ValueError):
        N.codebook_block(torch.tensor([0.1, 0.2, 0.3]), 2)


def test_lloyd_max_mirror_is_bit_identical_to_reference_fixtures():
    z = load_golden("codebooks.npz")
    for d, bits in ((64, 1), (64, 4), (128, 2), (128, 4), (128, 6), (256, 3)):
        cb = tq.LloydMaxCodebook(d, bits)
        assert np.array_equal(cb.centroids.numpy(), z[f"c_{d}_{bits}"])
        assert np.array_equal(cb.boundaries.numpy(), z[f"b_{d}_{bits}"])
        assert cb.distortion == pytest.approx(float(z[f"dist_{d}_{bits}"]), rel=1e-12)
        assert cb.n_levels == 2 ** bits and "LloydMaxCodebook(d=" in repr(cb)
    c, b = tq.solve_lloyd_max(128, 2, use_exact=True)
    assert np.array_equal(c.numpy(), z["cx_128_2"]) and np.array_equal(b.numpy(), z["bx_128_2"])
    for d, bits in ((128, 1), (128, 2), (128, 3), (256, 2)):
        assert np.array_equal(lloyd_max.solve_codebook_v2(d, bits).numpy(), z[f"v2c_{d}_{bits}"])
    x = torch.randn(5, 7) * 0.1
    cb = tq.LloydMaxCodebook(128, 3)
    assert torch.equal(cb.quantize(x), O.nearest_centroid(x, cb.centroids))
    assert torch.equal(cb.dequantize(cb.quantize(x)), cb.centroids[cb.quantize(x)])


def test_generators_match_oracle():
    from turboquant.turboquant import generate_qjl_matrix, generate_rotation_matrix
    assert torch.equal(generate_rotation_matrix(128, seed=42), O.rotation_matrix(128, 42))
    assert torch.equal(generate_qjl_matrix(128, seed=43), O.qjl_matrix(128, None, 43))
    assert generate_qjl_matrix(128, m=64, seed=5).shape == (64, 128)


def test_v3_layer_adaptive_bits_seeds_and_accounting():
    z = load_golden("v3_kv.npz")
    t = tq.TurboQuantV3(128, key_bits=6, value_bits=4, residual_window=16, layer_idx=0, n_layers=32, protected_layers=4)
    assert (t.key_bits, t.value_bits) == (8, 8)
    t = tq.TurboQuantV3(128, key_bits=6, value_bits=4, residual_window=16, layer_idx=10, n_layers=32, protected_layers=4)
    assert (t.key_bits, t.value_bits) == (6, 4)
    mem = t.memory_bytes(2, 2, 72)
    assert [mem["compressed_bytes"], mem["fp16_bytes"], mem["compressed_tokens"], mem["fp16_tokens"]] == z["c_mem"].tolist()
    t = tq.TurboQuantV3(128, key_bits=4, value_bits=2, protected_bits=12, layer_idx=35, n_layers=36)
    assert (t.key_bits, t.value_bits) == (8, 8)       # capped at 8
    assert torch.equal(t.key_compressor.Pi, O.rotation_matrix(128, 42 + 35000))
    assert torch.equal(t.val_compressor.Pi, O.rotation_matrix(128, 42 + 35000 + 500))
    total = sum(tq.TurboQuantV3(128, 4, 2, residual_window=0, layer_idx=l, n_layers=36, protected_layers=0)
                .memory_bytes(1, 2, 8192)["compressed_bytes"] for l in (0, 17, 35)) * 12
    assert total == 58982400 == int(z["cfg2_packed_total"])
    assert tq.MSECompressor(128, 4, seed=1).memory_bytes(1, 1, 4096)["compressed_bytes"] == 270336


def test_passthrough_window_aliases_inputs_on_any_device():
    t = tq.TurboQuantV3(128, residual_window=128, layer_idx=5)
    k, v = torch.randn(1, 2, 24, 128), torch.randn(1, 2, 24, 128)
    ck, cv = t.compress_kv(k, v)
    assert ck["compressed"] is None and ck["fp16"] is k and cv["fp16"] is v and ck["split_at"] == 24
    rk, rv = t.decompress_kv(ck, cv)
    assert rk is k and rv is v


def test_no_cpu_fallback_and_error_types():
    c = tq.MSECompressor(128, 4, seed=42)
    with pytest.raises(RuntimeError, match="no CPU path"):
        c.compress(torch.randn(1, 1, 4, 128))
    with pytest.raises(ValueError):
        c.compress(torch.randn(4, 128))               # not 4-D, as in the reference
    t = tq.TurboQuantV3(128, residual_window=0, layer_idx=5)
    with pytest.raises(RuntimeError, match="no CPU path"):
        t.compress_kv(torch.randn(1, 1, 4, 128), torch.randn(1, 1, 4, 128))
    m = tq.TurboQuantMSE(128, 3)
    assert sorted(m.state_dict().keys()) == ["Pi", "boundaries", "centroids"]
    with pytest.raises(RuntimeError):
        m.quantize(torch.randn(2, 128))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(N, "_lib", None)
    monkeypatch.setattr(N, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="build it"):
        N.lib()


def test_shard_units_partition():
    for world in (1, 2, 4, 8):
        seen = []
        for r in range(world):
            seen += batched.shard_units(36, 2, r, world)
        assert sorted(seen) == [(l, h) for l in range(36) for h in range(2)]
        sizes = [len(batched.shard_units(36, 2, r, world)) for r in range(world)]
        assert max(sizes) - min(sizes) <= 1


def test_search_shortcut_parameters_bracket_the_exact_index():
    """index = e + (y > thr[e]) needs the exact index to be e or e+1 for every y."""
    z = load_golden("codebooks.npz")
    rng = np.random.default_rng(0)
    for d in (64, 128, 256):
        for bits in range(1, 9):
            block = N.codebook_block(torch.from_numpy(z[f"c_{d}_{bits}"]), bits).numpy().astype(np.float64)
            n = 2 ** bits - 1
            thr = block[256:256 + n]
            if bits > 6:                          # byte table over 1024 cells of t
                assert block[512] == 2.0 and block[517] == 1024.0, (d, bits)
                raw = N.codebook_block(torch.from_numpy(z[f"c_{d}_{bits}"]), bits).numpy()
                cells = raw[528:528 + 257].view(np.uint8)[:1025].astype(np.int64)
                s = block[513]
                y = np.concatenate([rng.normal(0, 1 / np.sqrt(d), 50000), np.linspace(-1, 1, 20001), thr,
                                    np.nextafter(thr.astype(np.float32), np.float32(np.inf)).astype(np.float64)])
                t = np.clip(y * s + 0.5, 0.0, 1.0)
                e = cells[np.rint(t * 1024).astype(np.int64)]
                exact = (y[:, None] > thr[None, :]).sum(axis=1)
                assert np.all((e == exact) | (e + 1 == exact)), (d, bits)
                continue
            assert block[512] == 1.0, (d, bits)
            s, c1, c2, c3 = block[513:517]
            if block[518] == 1.0:                 # a straight line passed the host check
                assert c2 == 0.0 and c3 == 0.0 and bits <= 3
            y = np.concatenate([rng.normal(0, 1 / np.sqrt(d), 50000), np.linspace(-1, 1, 20001), thr,
                                np.nextafter(thr.astype(np.float32), np.float32(np.inf)).astype(np.float64)])
            t = np.clip(y * s + 0.5, 0.0, 1.0)
            e = np.rint(t * (c1 + t * (c2 + t * c3)))
            exact = (y[:, None] > thr[None, :]).sum(axis=1)
            assert np.all((e == exact) | (e + 1 == exact)), (d, bits)
            # up to 31 thresholds kernels look the threshold up across the lanes of a warp; the 63 thresholds of
            # 6-bit codes still have a bracketing cubic and are looked up in shared memory
            assert e.min() >= 0 and e.max() <= (31 if bits <= 5 else 63)


def test_codebook_disk_cache_round_trip(tmp_path, monkeypatch):
    """Solved codebooks come back from the disk cache bit for bit, a damaged file is recomputed, and an empty
    TURBOQUANT_B200_CACHE_DIR switches the cache off."""
    z = load_golden("codebooks.npz")
    monkeypatch.setenv("TURBOQUANT_B200_CACHE_DIR", str(tmp_path))
    lloyd_max._solve.cache_clear()
    lloyd_max._solve_inlined_v2.cache_clear()
    c1, b1 = tq.solve_lloyd_max(64, 4)
    v1 = lloyd_max.solve_codebook_v2(128, 2)
    files = sorted(p.name for p in tmp_path.iterdir())
    assert len(files) == 2 and all(f.endswith(".npy") for f in files)
    lloyd_max._solve.cache_clear()
    lloyd_max._solve_inlined_v2.cache_clear()
    calls = []
    monkeypatch.setattr(lloyd_max, "_solve_points", lambda *a: calls.append(a) or (0.0,) * 16)
    c2, b2 = tq.solve_lloyd_max(64, 4)                 # served from disk: the solver is not called
    assert not calls and torch.equal(c1, c2) and torch.equal(b1, b2)
    assert np.array_equal(c2.numpy(), z["c_64_4"]) and np.array_equal(lloyd_max.solve_codebook_v2(128, 2).numpy(), v1.numpy())
    monkeypatch.undo()
    monkeypatch.setenv("TURBOQUANT_B200_CACHE_DIR", str(tmp_path))
    for p in tmp_path.iterdir():                       # damage every file: wrong length
        np.save(open(p, "wb"), np.zeros(3))
    lloyd_max._solve.cache_clear()
    c3, _ = tq.solve_lloyd_max(64, 4)
    assert np.array_equal(c3.numpy(), z["c_64_4"])
    monkeypatch.setenv("TURBOQUANT_B200_CACHE_DIR", "")
    lloyd_max._solve.cache_clear()
    assert lloyd_max._cache_dir() is None
    c4, _ = tq.solve_lloyd_max(64, 4)
    assert np.array_equal(c4.numpy(), z["c_64_4"])
    lloyd_max._solve.cache_clear()
    lloyd_max._solve_inlined_v2.cache_clear()


def test_v1_state_dict_reloads_into_a_fresh_module():
    """Buffers saved from one module and loaded into one built with another seed make it identical."""
    a = tq.TurboQuantProd(128, 3, seed=42)
    b = tq.TurboQuantProd(128, 3, seed=7)
    assert not torch.equal(a.S, b.S) and not torch.equal(a.mse.Pi, b.mse.Pi)
    b.load_state_dict(a.state_dict())
    for k, v in a.state_dict().items():
        assert torch.equal(v, b.state_dict()[k]), k
    assert torch.equal(a._s_t, b._s_t) and torch.equal(a.mse._pi_t, b.mse._pi_t) and torch.equal(a.mse._cb, b.mse._cb)
    m1, m2 = tq.TurboQuantMSE(64, 2, seed=1), tq.TurboQuantMSE(64, 2, seed=2)
    m2.load_state_dict(m1.state_dict())
    assert torch.equal(m1.Pi, m2.Pi) and torch.equal(m1.centroids, m2.centroids) and torch.equal(m1.boundaries, m2.boundaries)
    assert torch.equal(m1._pi_t, m2._pi_t)            # the kernel-side constants follow the loaded buffers
