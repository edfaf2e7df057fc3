"""Generate the golden fixtures in this directory from the reference itself.

Run once, in a container where the reference checkout is importable:

    python tests/golden/make_golden.py --reference <checkout of tonbistudio/turboquant-pytorch>

The script imports the reference package `turboquant` (CPU), feeds it seeded
inputs and stores inputs and outputs as .npz files next to this script.  The
fixtures travel with the repository; the reference does not.  16-bit float
tensors are stored as their uint16 bit patterns.
"""

from __future__ import annotations

import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


ONLY = None     # with --only: the fixture files to (re)write; the others are computed but left untouched


def save(name: str, **arrays):
    if ONLY is not None and name not in ONLY:
        print(f"{name}: kept")
        return
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **arrays)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (the directory holding turboquant/)")
    ap.add_argument("--only", nargs="*", default=None, help="rewrite only these fixture files")
    args = ap.parse_args()
    global ONLY
    ONLY = set(args.only) if args.only else None
    sys.path.insert(0, args.reference)
    import turboquant as ref  # the reference package
    from turboquant.lloyd_max import solve_lloyd_max, LloydMaxCodebook
    from turboquant.turboquant import generate_rotation_matrix, generate_qjl_matrix
    from tq_oracle import synthetic_kv  # input generator only

    # ---- 1. codebooks ------------------------------------------------------
    out = {}
    for d in (64, 128, 256):
        for bits in range(1, 9):
            cb = LloydMaxCodebook(d, bits)
            out[f"c_{d}_{bits}"] = cb.centroids.numpy()
            out[f"b_{d}_{bits}"] = cb.boundaries.numpy()
            out[f"dist_{d}_{bits}"] = np.float64(cb.distortion)
    for d, bits in ((128, 2), (64, 3)):
        c, b = solve_lloyd_max(d, bits, use_exact=True)
        out[f"cx_{d}_{bits}"] = c.numpy()
        out[f"bx_{d}_{bits}"] = b.numpy()
    v2 = ref.TurboQuantCompressorV2.__new__(ref.TurboQuantCompressorV2)
    for d, bits in ((128, 1), (128, 2), (128, 3), (128, 4), (256, 2), (64, 2)):
        out[f"v2c_{d}_{bits}"] = v2._solve_codebook(d, bits).numpy()
    save("codebooks.npz", **out)

    # ---- 2. rotation / projection matrices ----------------------------------
    out = {}
    for d, seed in ((128, 0), (128, 42), (128, 542), (64, 7), (256, 42), (128, 3042)):
        pi = generate_rotation_matrix(d, seed=seed)
        out[f"pi_sha_{d}_{seed}"] = np.array(sha(pi))
        out[f"pi_rows_{d}_{seed}"] = pi[:2].numpy()
        out[f"pi_diag_{d}_{seed}"] = torch.diag(pi).numpy()
    for d, m, seed in ((128, None, 43), (256, None, 10042), (128, 64, 5)):
        s = generate_qjl_matrix(d, m=m, seed=seed)
        out[f"s_sha_{d}_{m}_{seed}"] = np.array(sha(s))
        out[f"s_rows_{d}_{m}_{seed}"] = s[:2].numpy()
    save("matrices.npz", **out)

    # ---- 3. config 1: N=4096, d=128, fp32 N(0,1) seed 0, K4 / V2 ------------
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(1, 1, 4096, 128, generator=g)
    out = {"x_sha": np.array(sha(x))}
    for tag, bits, seed in (("k", 4, 42), ("v", 2, 542)):
        comp = ref.MSECompressor(128, bits, seed=seed)
        c = comp.compress(x)
        rec = comp.decompress(c)
        out[f"{tag}_idx"] = c["idx_bytes"].numpy()
        out[f"{tag}_norms"] = bits16(c["vec_norms"])
        out[f"{tag}_pad"] = np.int64(c["idx_pad"])
        out[f"{tag}_rec_head"] = rec[0, 0, :64].numpy()
        out[f"{tag}_mse"] = ((rec - x) ** 2).sum(-1).mean().numpy()
        mem = comp.memory_bytes(1, 1, 4096)
        out[f"{tag}_mem"] = np.array([mem["compressed_bytes"], mem["fp16_bytes"]], dtype=np.int64)
    save("cfg1.npz", **out)

    # ---- 4. small MSECompressor cases over bits / head_dim / padding --------
    out = {}
    cases = [(128, b, 32) for b in range(1, 9)] + [(64, b, 32) for b in (1, 3, 5, 8)] \
        + [(256, b, 16) for b in (2, 4)] + [(100, 1, 16), (100, 3, 16), (65, 2, 16), (65, 4, 16), (72, 6, 16)]
    for d, bits, n in cases:
        g = torch.Generator(device="cpu").manual_seed(1000 * d + bits)
        x = torch.randn(1, 2, n // 2, d, generator=g) * 3.0
        comp = ref.MSECompressor(d, bits, seed=17 + bits)
        flat = x.reshape(-1, d).float()
        norms = torch.norm(flat, dim=-1)
        rot = (flat / (norms.unsqueeze(-1) + 1e-8)) @ comp.Pi.T
        c = comp.compress(x)
        rec = comp.decompress(c)
        k = f"{d}_{bits}"
        out[f"x_{k}"] = x.numpy()
        out[f"rot_{k}"] = rot.numpy()
        out[f"idx_{k}"] = c["idx_bytes"].numpy()
        out[f"norms_{k}"] = bits16(c["vec_norms"])
        out[f"pad_{k}"] = np.int64(c["idx_pad"])
        out[f"rec_{k}"] = rec.numpy()
    out["cases"] = np.array(cases, dtype=np.int64)
    save("mse_small.npz", **out)

    # ---- 5. TurboQuantV3 on 16-bit caches with outlier channels -------------
    out = {}
    v3_cases = [
        ("a", dict(shape=(1, 2, 96, 128), dtype=torch.float16, seed=20003),
         dict(key_bits=4, value_bits=2, residual_window=0, layer_idx=3, n_layers=36, protected_layers=0)),
        ("b", dict(shape=(2, 2, 72, 128), dtype=torch.bfloat16, seed=30000),
         dict(key_bits=6, value_bits=4, residual_window=16, layer_idx=0, n_layers=32, protected_layers=4)),
        ("c", dict(shape=(2, 2, 72, 128), dtype=torch.bfloat16, seed=30010),
         dict(key_bits=6, value_bits=4, residual_window=16, layer_idx=10, n_layers=32, protected_layers=4)),
        ("d", dict(shape=(1, 2, 24, 128), dtype=torch.float16, seed=20099),
         dict(key_bits=4, value_bits=2, residual_window=128, layer_idx=5, n_layers=36, protected_layers=4)),
    ]
    for tag, inp, kw in v3_cases:
        keys = synthetic_kv(inp["shape"], inp["dtype"], inp["seed"])
        vals = synthetic_kv(inp["shape"], inp["dtype"], inp["seed"] + 5000)
        tq = ref.TurboQuantV3(128, **kw)
        ck, cv = tq.compress_kv(keys, vals)
        rk, rv = tq.decompress_kv(ck, cv)
        out[f"{tag}_keys"], out[f"{tag}_vals"] = bits16(keys), bits16(vals)
        out[f"{tag}_bits"] = np.array([tq.key_bits, tq.value_bits], dtype=np.int64)
        out[f"{tag}_split"] = np.int64(ck["split_at"])
        if ck["compressed"] is not None:
            out[f"{tag}_k_idx"] = ck["compressed"]["idx_bytes"].numpy()
            out[f"{tag}_k_norms"] = bits16(ck["compressed"]["vec_norms"])
            out[f"{tag}_v_idx"] = cv["compressed"]["idx_bytes"].numpy()
            out[f"{tag}_v_norms"] = bits16(cv["compressed"]["vec_norms"])
        out[f"{tag}_rk"], out[f"{tag}_rv"] = bits16(rk), bits16(rv)
        mem = tq.memory_bytes(*inp["shape"][:3])
        out[f"{tag}_mem"] = np.array([mem["compressed_bytes"], mem["fp16_bytes"], mem["compressed_tokens"],
                                      mem["fp16_tokens"]], dtype=np.int64)
    # accounting for the two headline configurations (pure arithmetic)
    tot2 = sum(ref.TurboQuantV3(128, 4, 2, residual_window=0, layer_idx=0, n_layers=36, protected_layers=0)
               .memory_bytes(1, 2, 8192)["compressed_bytes"] for _ in range(36))
    out["cfg2_packed_total"] = np.int64(tot2)
    save("v3_kv.npz", **out)

    # ---- 6. edge vectors ----------------------------------------------------
    x = torch.randn(1, 1, 8, 128, generator=torch.Generator().manual_seed(5))
    x[0, 0, 0] = 0.0
    x[0, 0, 1, 3] = float("nan")
    x[0, 0, 2, 7] = float("inf")
    x[0, 0, 3] *= 1e4          # norm above the fp16 range
    x[0, 0, 4] *= 1e-12        # norm comparable with the 1e-8 guard
    x[0, 0, 5] = 0.0
    x[0, 0, 5, 11] = 1.0       # a coordinate axis
    comp = ref.MSECompressor(128, 4, seed=42)
    c = comp.compress(x)
    rec = comp.decompress(c)
    save("edge.npz", x=x.numpy(), idx=c["idx_bytes"].numpy(), norms=bits16(c["vec_norms"]), rec=rec.numpy())

    # ---- 7. V2 compressors --------------------------------------------------
    out = {}
    for tag, d, bits, seed, shape, sq in (("a", 128, 3, 7, (1, 2, 48, 128), 8), ("b", 256, 3, 11, (1, 1, 16, 256), 4),
                                          ("c", 128, 4, 3, (2, 1, 24, 128), 3)):
        st = synthetic_kv(shape, torch.float16, 50000 + d + bits, outlier_channels=0)
        q = torch.randn(shape[0], shape[1], sq, d, generator=torch.Generator().manual_seed(60000 + d))
        comp = ref.TurboQuantCompressorV2(d, bits, seed=seed)
        c = comp.compress(st)
        sc = comp.asymmetric_attention_scores(q, c)
        out[f"{tag}_meta"] = np.array([d, bits, seed, sq], dtype=np.int64)
        out[f"{tag}_x"] = bits16(st)
        out[f"{tag}_q"] = q.numpy()
        out[f"{tag}_kmse"] = bits16(c["k_mse"])
        out[f"{tag}_signs"] = c["qjl_signs"].numpy()
        out[f"{tag}_rnorm"] = bits16(c["residual_norm"])
        out[f"{tag}_scores"] = sc.numpy()
    st = synthetic_kv((1, 2, 32, 128), torch.float16, 51000, outlier_channels=0)
    comp = ref.TurboQuantCompressorMSE(128, 2, seed=9)
    c = comp.compress(st)
    out["m_x"] = bits16(st)
    out["m_idx"] = c["indices"].numpy()
    out["m_norms"] = bits16(c["vec_norms"])
    out["m_rec"] = comp.decompress(c).numpy()
    save("v2.npz", **out)

    # ---- 8. V1 classes ------------------------------------------------------
    out = {}
    g = torch.Generator().manual_seed(77)
    x = torch.randn(32, 128, generator=g)
    x = x / torch.norm(x, dim=-1, keepdim=True)
    y = torch.randn(32, 128, generator=g)
    mse = ref.TurboQuantMSE(128, 3, seed=42)
    xh, idx = mse(x)
    out["x"], out["y"] = x.numpy(), y.numpy()
    out["mse_idx"], out["mse_xhat"] = idx.numpy(), xh.numpy()
    out["mse_rot"] = mse.rotate(x).numpy()
    prod = ref.TurboQuantProd(128, 3, seed=42)
    c = prod.quantize(x)
    out["prod_idx"], out["prod_signs"], out["prod_rnorm"] = (c["mse_indices"].numpy(), c["qjl_signs"].numpy(),
                                                             c["residual_norm"].numpy())
    out["prod_ip"] = prod.inner_product(y, c).numpy()
    prod64 = ref.TurboQuantProd(128, 4, qjl_dim=64, seed=3)
    c64 = prod64.quantize(x)
    out["prod64_signs"], out["prod64_ip"] = c64["qjl_signs"].numpy(), prod64.inner_product(y, c64).numpy()
    cache = ref.TurboQuantKVCache(128, 128, bits=3, seed=42)
    kv = torch.randn(2, 40, 128, generator=g)
    cache.append(kv[:, :24], kv[:, :24] * 0.5)
    cache.append(kv[0, 24:], kv[0, 24:] * 2.0)
    q1 = torch.randn(128, generator=g)
    out["cache_kv"], out["cache_q"] = kv.numpy(), q1.numpy()
    out["cache_scores"] = cache.attention_scores(q1).numpy()
    out["cache_values"] = cache.get_values().numpy()
    mu = cache.memory_usage_bits()
    out["cache_mem"] = np.array([mu["key_bits"], mu["value_bits"], mu["total_bits"], mu["fp16_bits"]], dtype=np.int64)
    out["cache_len"] = np.int64(len(cache))
    save("v1.npz", **out)

    # ---- 9. packed-key attention scores (decompress + matmul composition) ---
    keys = synthetic_kv((1, 2, 256, 128), torch.float16, 20000)
    q = torch.randn(1, 8, 1, 128, generator=torch.Generator().manual_seed(40000))
    comp = ref.MSECompressor(128, 4, seed=42)
    c = comp.compress(keys)
    rec = comp.decompress(c)
    rep = rec.float().repeat_interleave(4, dim=1)
    logits = torch.matmul(q.float(), rep.transpose(-2, -1))
    save("scores.npz", keys=bits16(keys), q=q.numpy(), idx=c["idx_bytes"].numpy(), norms=bits16(c["vec_norms"]),
         logits=logits.numpy(), probs=torch.softmax(logits, dim=-1).numpy())

    # ---- 10. incremental cache of the generation harness (prefill + decode steps) ----
    from turboquant.generation_test_v2 import V3Cache
    out = {}
    for tag, rw, prefill, steps in (("w", 16, 150, 10), ("z", 0, 40, 3)):
        cache = V3Cache(key_bits=4, value_bits=2, residual_window=rw, protected_layers=1, n_layers=4)
        for layer in (0, 1):                       # layer 0 is protected (8 bits), layer 1 is not
            total = prefill + steps
            k = synthetic_kv((1, 2, total, 128), torch.float16, 61000 + 10 * layer + rw)
            v = synthetic_kv((1, 2, total, 128), torch.float16, 62000 + 10 * layer + rw)
            fk, fv = cache.update(k[:, :, :prefill], v[:, :, :prefill], layer)
            out[f"{tag}{layer}_prefill_k"], out[f"{tag}{layer}_prefill_v"] = bits16(fk), bits16(fv)
            for t in range(prefill, total):
                fk, fv = cache.update(k[:, :, t:t + 1], v[:, :, t:t + 1], layer)
            out[f"{tag}{layer}_k"], out[f"{tag}{layer}_v"] = bits16(k), bits16(v)
            out[f"{tag}{layer}_full_k"], out[f"{tag}{layer}_full_v"] = bits16(fk), bits16(fv)
            out[f"{tag}{layer}_len"] = np.int64(cache.get_seq_length(layer))
        out[f"{tag}_info"] = np.array(cache.get_compression_info())
    save("v3_cache.npz", **out)


if __name__ == "__main__":
    main()
