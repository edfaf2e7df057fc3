"""GPU parity at the shapes and layouts the benchmark configurations name, against the CPU oracle.

  * the Llama-3-8B-shaped layer layout: batch 8, 8 KV heads, bf16, residual window 128, an 8-bit protected
    layer and an ordinary 6-bit-key / 4-bit-value layer (shorter sequence so that the oracle finishes);
  * decode scores straight from packed keys: one layer, 8 KV heads x 131072 4-bit keys, 32 query heads;
  * the MSE+QJL path at head_dim 256, 16 heads x 16384 keys, 64 queries per head, with the estimator's
    bias / RMSE / correlation against the true scores printed next to the oracle's own;
  * guard regions: ragged sequence lengths written into buffers with sentinel rows around every slab.
"""

import numpy as np
import pytest
import torch

import tq_oracle as O
from parity_helpers import check_indices, check_norms, check_recon_16bit, check_v2_compress, rel_err

import turboquant as tq
from turboquant import _native as N
from turboquant import _ops, batched

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cpu(d):
    return {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in d.items()}


@pytest.mark.parametrize("layer", [0, 10])
def test_llama_layer_layout_bf16_window_protected(layer):
    """(8, 8, 1152, 128) bf16, residual_window=128: layer 0 is protected (8-bit K and V), layer 10 is K6/V4."""
    B, H, S, D, W = 8, 8, 1152, 128, 128
    keys = O.synthetic_kv((B, H, S, D), torch.bfloat16, seed=30000 + layer)
    vals = O.synthetic_kv((B, H, S, D), torch.bfloat16, seed=35000 + layer)
    kw = dict(key_bits=6, value_bits=4, residual_window=W, layer_idx=layer, n_layers=32, protected_layers=4)
    codec = tq.TurboQuantV3(D, device=DEV, **kw)
    ref = O.V3Oracle(D, **kw)
    assert (codec.key_bits, codec.value_bits) == (ref.key_bits, ref.value_bits) == ((8, 8) if layer == 0 else (6, 4))
    gk, gv = keys.to(DEV), vals.to(DEV)
    ck, cv = codec.compress_kv(gk, gv)
    cut = S - W
    assert ck["split_at"] == cut and cv["split_at"] == cut and ck["shape"] == (B, H, S, D)
    # the "fp16" entries are views of the inputs (no copy), in the input dtype
    assert ck["fp16"].data_ptr() == gk[:, :, cut:, :].data_ptr() and ck["fp16"].dtype == torch.bfloat16
    assert cv["fp16"].data_ptr() == gv[:, :, cut:, :].data_ptr() and tuple(ck["fp16"].shape) == (B, H, W, D)
    for comp, src, pi, cent, bits in ((ck, keys, ref.k_pi, ref.k_cent, ref.key_bits),
                                      (cv, vals, ref.v_pi, ref.v_cent, ref.value_bits)):
        c = comp["compressed"]
        assert tuple(c["idx_bytes"].shape) == (B, H, cut, N.packed_row_bytes(D, bits)) and c["idx_pad"] == 0
        bnd = O.lloyd_max(D, bits)[1]
        norms, _ = check_indices(c["idx_bytes"], src[:, :, :cut].contiguous(), pi, cent, bnd, bits, D)
        check_norms(c["vec_norms"], norms)
    rk, rv = codec.decompress_kv(ck, cv)
    assert rk.dtype == torch.bfloat16 and rk.shape == (B, H, S, D) and rv.shape == (B, H, S, D)
    # window tokens bit-equal to the inputs
    assert torch.equal(rk[:, :, cut:].cpu(), keys[:, :, cut:]) and torch.equal(rv[:, :, cut:].cpu(), vals[:, :, cut:])
    # compressed tokens: the oracle decompresses the bytes the GPU packed (an attributed index mismatch, counted
    # above, is not counted twice) and rounds to bf16 like the reference
    for rec, comp, pi, cent, bits in ((rk, ck, ref.k_pi, ref.k_cent, ref.key_bits), (rv, cv, ref.v_pi, ref.v_cent, ref.value_bits)):
        want = O.mse_decompress(_cpu(comp["compressed"]), pi, cent, bits)
        check_recon_16bit(rec[:, :, :cut], want)
    # the whole-cache plan on the same tensors gives the same bytes
    plan = batched.CachePlan([codec], [gk], [gv])
    plan.compress()
    plan.decompress()
    torch.cuda.synchronize()
    assert torch.equal(plan.compressed[0][0]["compressed"]["idx_bytes"], ck["compressed"]["idx_bytes"])
    assert torch.equal(plan.reconstructed[0][0], rk) and torch.equal(plan.reconstructed[0][1], rv)
    assert N.lib().tq_last_device_status() == 0


def test_decode_scores_131072_packed_keys_gqa_32_on_8():
    """One layer of the decode-score configuration: logits and softmax for 32 query heads straight from
    8 KV heads x 131072 4-bit keys, against decompress + matmul on the CPU."""
    hkv, hq, sk, d = 8, 32, 131072, 128
    g = torch.Generator().manual_seed(40000)
    keys = torch.randn(1, hkv, sk, d, generator=g)
    keys[:, :, :, :4] *= 10.0
    keys = keys.half()
    q = torch.randn(1, hq, 1, d, generator=g)
    comp = tq.MSECompressor(d, 4, seed=42, device=DEV)
    c = comp.compress(keys.to(DEV))
    logits, probs = comp.attention_scores(q.to(DEV), c, softmax=True)
    assert logits.shape == (1, hq, 1, sk) and logits.dtype == torch.float32
    cent = O.lloyd_max(d, 4)[0]
    rec = O.mse_decompress(_cpu(c), comp.Pi.cpu(), cent, 4)
    want = O.v3_scores(q, rec)
    assert rel_err(logits, want) <= 1e-5
    wp = torch.softmax(want.double(), -1)
    assert float((probs.cpu().double() - wp).abs().max()) <= 2e-4 * float(wp.max()) + 1e-9
    assert torch.allclose(probs.sum(-1).cpu(), torch.ones(1, hq, 1), atol=1e-4)
    scaled = comp.attention_scores(q.to(DEV), c, scale=d ** -0.5)
    assert rel_err(scaled, want * d ** -0.5) <= 1e-5


def _estimator_stats(scores, true):
    err = (scores - true).double()
    t = true.double()
    corr = float(torch.corrcoef(torch.stack([scores.double().reshape(-1), t.reshape(-1)]))[0, 1])
    return float(err.mean()), float(err.pow(2).mean().sqrt()), corr


def test_v2_head_dim_256_16_heads_16384_keys_64_queries(capsys):
    """The MSE+QJL configuration at full size on the GPU; the oracle runs on a 4096-key slice per head.
    Prints bias / RMSE / correlation of the estimator against the true Q K^T next to the oracle's figures."""
    H, S, D, Sq, slice_n = 16, 16384, 256, 64, 4096
    g = torch.Generator().manual_seed(50000)
    x = torch.randn(1, H, S, D, generator=g).half()
    q = torch.randn(1, H, Sq, D, generator=g)
    comp = tq.TurboQuantCompressorV2(D, 3, seed=7, device=DEV)
    c = comp.compress(x.to(DEV))
    sc = comp.asymmetric_attention_scores(q.to(DEV), c)
    assert sc.shape == (1, H, Sq, S)
    xs = x[:, :, :slice_n].contiguous()
    cs = {"k_mse": c["k_mse"][:, :, :slice_n], "qjl_signs": c["qjl_signs"][:, :, :slice_n],
          "residual_norm": c["residual_norm"][:, :, :slice_n], "shape": (1, H, slice_n, D)}
    marked = check_v2_compress(cs, xs, comp.Pi.cpu(), comp.centroids.cpu(), comp.S.cpu())
    # scores: the oracle's formula on the GPU's own compressed tensors (full size), <= 1e-5
    want = O.v2_scores(q, _cpu(c), comp.S.cpu())
    assert rel_err(sc, want) <= 1e-5
    # estimator statistics on the slice, GPU next to the oracle end to end
    true = torch.matmul(q, xs.float().transpose(-2, -1))
    ref_c = O.v2_compress(xs, comp.Pi.cpu(), comp.centroids.cpu(), comp.S.cpu())
    ref_sc = O.v2_scores(q, ref_c, comp.S.cpu())
    mine = _estimator_stats(sc.cpu()[..., :slice_n], true)
    theirs = _estimator_stats(ref_sc, true)
    rms = float(true.double().pow(2).mean().sqrt())
    with capsys.disabled():
        print(f"\n[V2 estimator, head_dim 256, 3 bits, 16 x 4096 keys x 64 queries] true-score RMS {rms:.3f}; "
              f"GPU bias {mine[0]:+.4f} RMSE {mine[1]:.4f} corr {mine[2]:.5f} | "
              f"oracle bias {theirs[0]:+.4f} RMSE {theirs[1]:.4f} corr {theirs[2]:.5f} | marked vectors {marked}")
    assert abs(mine[0] - theirs[0]) <= 1e-3 * rms and abs(mine[1] - theirs[1]) <= 1e-3 * rms
    assert abs(mine[2] - theirs[2]) <= 1e-4
    assert abs(mine[0]) <= 0.01 * rms                       # unbiased
    assert N.lib().tq_last_device_status() == 0


SENTINEL_BYTE = 0xA5


@pytest.mark.parametrize("bits", [4, 6, 8])
def test_ragged_slabs_leave_guard_rows_untouched(bits):
    """Ragged sequence length (333 = 2 tiles + 77 rows) with sentinel rows before and after every (b, h) slab
    of every output: packed indices, norms, fp32 and 16-bit reconstructions (TMA-store path)."""
    B, H, S, D, G0 = 2, 3, 333, 128, 5                     # G0 guard rows on each side of a slab
    x = O.synthetic_kv((B, H, S, D), torch.float16, seed=61000 + bits)
    comp = tq.MSECompressor(D, bits, seed=31 + bits, device=DEV)
    row = N.packed_row_bytes(D, bits)
    SP = S + 2 * G0
    # outputs with guards: idx/norms are contiguous per job, so guard them at both ends of the whole buffer
    idx_buf = torch.full((B * H * S * row + 2 * 4096,), SENTINEL_BYTE, dtype=torch.uint8, device=DEV)
    nrm_buf = torch.full((B * H * S + 2 * 1024,), -7.0, dtype=torch.float16, device=DEV)
    idx = idx_buf[4096:4096 + B * H * S * row].view(B, H, S, row)
    nrm = nrm_buf[1024:1024 + B * H * S].view(B, H, S)
    gx = x.to(DEV)
    job, _idx, _n, keep = _ops.quantize_job(gx, comp._pi_t, comp._cb, bits, True, N.IDX_PACKED, image=comp._img_q)
    job.idx_out, job.norms_out = idx.data_ptr(), nrm.data_ptr()
    _ops.run_quantize([job], gx.device)
    ref = comp.compress(gx)
    torch.cuda.synchronize()
    assert torch.equal(idx, ref["idx_bytes"]) and torch.equal(nrm, ref["vec_norms"])
    assert bool((idx_buf[:4096] == SENTINEL_BYTE).all()) and bool((idx_buf[-4096:] == SENTINEL_BYTE).all())
    assert bool((nrm_buf[:1024] == -7.0).all()) and bool((nrm_buf[-1024:] == -7.0).all())
    want = comp.decompress(ref)
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        full = torch.full((B, H, SP, D), 123.0, dtype=dtype, device=DEV)
        out = full[:, :, G0:G0 + S, :]                     # strided view: every slab has guard rows on both sides
        job, keep = comp.decompress_job(ref, out)
        _ops.run_dequantize([job], out.device)
        torch.cuda.synchronize()
        assert bool((full[:, :, :G0] == 123.0).all()) and bool((full[:, :, G0 + S:] == 123.0).all()), dtype
        if dtype == torch.float32:
            assert rel_err(out, want) <= 1e-5
        else:
            check_recon_16bit(out, want)
    assert N.lib().tq_last_device_status() == 0


def test_v2_compress_ragged_leaves_guards_untouched():
    """V2 compress (tensor-core path, ragged 333 rows) writes exactly its own output range."""
    B, H, S, D = 1, 2, 333, 128
    x = O.synthetic_kv((B, H, S, D), torch.float16, seed=62000, outlier_channels=0)
    comp = tq.TurboQuantCompressorV2(D, 3, seed=5, device=DEV)
    c = comp.compress(x.to(DEV))
    # run the same job again into guarded buffers through the C ABI
    n = B * H * S
    k_buf = torch.full((n * D + 2 * 2048,), 9.0, dtype=torch.float16, device=DEV)
    s_buf = torch.full((n * D + 2 * 4096,), 77, dtype=torch.int8, device=DEV)
    r_buf = torch.full((n + 2 * 1024,), 9.0, dtype=torch.float16, device=DEV)
    import ctypes as C
    gx = x.to(DEV)
    L = N.lib()
    ws_bytes = L.tq_qjl_compress_workspace_bytes(n, D)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=DEV)
    job = N.QjlCompressJob(x=gx.data_ptr(), x_dtype=N.F16, D=D, bits=comp.mse_bits, normalize=1, B=B, H=H, S=S,
                           stride_b=gx.stride(0), stride_h=gx.stride(1), stride_s=gx.stride(2),
                           rotation_t=comp.PiT.data_ptr(), rotation=comp.Pi.data_ptr(), codebook=comp._cb.data_ptr(),
                           qjl_t=comp._s_t.data_ptr(), M=D, signs_dtype=0, rnorm_dtype=N.F16, idx_mode=N.IDX_U8,
                           k_mse_out=k_buf[2048:].data_ptr(), idx_out=None, signs_out=s_buf[4096:].data_ptr(),
                           rnorm_out=r_buf[1024:].data_ptr(), workspace=ws.data_ptr(), workspace_bytes=ws_bytes)
    with torch.cuda.device(gx.device):
        N.check(L.tq_qjl_compress(C.byref(job), N.stream_ptr(gx.device)), "tq_qjl_compress")
    torch.cuda.synchronize()
    assert torch.equal(k_buf[2048:2048 + n * D].view(B, H, S, D), c["k_mse"])
    assert torch.equal(s_buf[4096:4096 + n * D].view(B, H, S, D), c["qjl_signs"])
    assert torch.equal(r_buf[1024:1024 + n].view(B, H, S), c["residual_norm"])
    for buf, lo, hi, val in ((k_buf, 2048, 2048 + n * D, 9.0), (s_buf, 4096, 4096 + n * D, 77), (r_buf, 1024, 1024 + n, 9.0)):
        assert bool((buf[:lo] == val).all()) and bool((buf[hi:] == val).all())
    assert L.tq_last_device_status() == 0
