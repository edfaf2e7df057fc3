"""Fused decode attention on packed keys and packed values (TurboQuantV3.decode_attention) against the oracle
composition: decompress every packed token, append the kept window tokens, softmax(scale * q K^T) V on the CPU.

The oracle decompresses the bytes the GPU packed, so an index that differs from the oracle's own packing (checked
elsewhere, with attribution) is not counted a second time here.  Tolerance: 1e-5 of the output's largest value
(fp32 output)."""

import pytest
import torch

import tq_oracle as O

import turboquant as tq
from turboquant import _native as N

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cpu(d):
    return {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in d.items()}


def _oracle_kv(codec, ck, cv):
    """What decompress_kv returns, from the oracle's decompression of the GPU's packed bytes, in fp32."""
    parts_k, parts_v = [], []
    if ck["compressed"] is not None:
        ck_cent = O.lloyd_max(128, codec.key_bits)[0]
        cv_cent = O.lloyd_max(128, codec.value_bits)[0]
        parts_k.append(O.mse_decompress(_cpu(ck["compressed"]), codec.key_compressor.Pi.cpu(), ck_cent, codec.key_bits))
        parts_v.append(O.mse_decompress(_cpu(cv["compressed"]), codec.val_compressor.Pi.cpu(), cv_cent, codec.value_bits))
    if ck["fp16"].shape[2] > 0:
        parts_k.append(ck["fp16"].float().cpu())
        parts_v.append(cv["fp16"].float().cpu())
    return torch.cat(parts_k, dim=2), torch.cat(parts_v, dim=2)


def _check(codec, keys, vals, q, scale=None):
    ck, cv = codec.compress_kv(keys.to(DEV), vals.to(DEV))
    out = codec.decode_attention(q.to(DEV), ck, cv, scale=scale)
    torch.cuda.synchronize()
    assert out.dtype == torch.float32 and out.shape == q.shape
    kf, vf = _oracle_kv(codec, ck, cv)
    want = O.v3_decode_attention(q.float(), kf, vf, 128 ** -0.5 if scale is None else scale)
    err = float((out.cpu() - want).abs().max() / want.abs().max())
    assert err <= 1e-5, err
    assert N.lib().tq_last_device_status() == 0
    return err


@pytest.mark.parametrize("sk", [1, 129, 8192])
@pytest.mark.parametrize("kb,vb", [(4, 2), (6, 4)])
def test_decode_attention_gqa_32_on_8(sk, kb, vb):
    """32 query heads on 8 KV heads, one query token, residual window 128 (for sk = 1 and 129 the packed part is
    empty or a single token)."""
    codec = tq.TurboQuantV3(128, key_bits=kb, value_bits=vb, residual_window=128, layer_idx=9, n_layers=32,
                            protected_layers=0, device=DEV)
    keys = O.synthetic_kv((1, 8, sk, 128), torch.float16, seed=70000 + sk)
    vals = O.synthetic_kv((1, 8, sk, 128), torch.float16, seed=71000 + sk)
    q = torch.randn(1, 32, 1, 128, generator=torch.Generator().manual_seed(sk))
    _check(codec, keys, vals, q)


def test_decode_attention_131072_packed_tokens():
    """The decode-score configuration's key count with values attached: 8 KV heads x 131072 tokens, K4/V2."""
    sk = 131072
    codec = tq.TurboQuantV3(128, key_bits=4, value_bits=2, residual_window=0, layer_idx=3, n_layers=36,
                            protected_layers=0, device=DEV)
    g = torch.Generator().manual_seed(72000)
    keys = torch.randn(1, 8, sk, 128, generator=g)
    keys[:, :, :, :4] *= 10.0
    vals = torch.randn(1, 8, sk, 128, generator=g)
    q = torch.randn(1, 32, 1, 128, generator=g)
    _check(codec, keys.half(), vals.half(), q)


@pytest.mark.parametrize("kb,vb,hq,hkv,sq,sk,window,dtype", [
    (8, 8, 8, 2, 1, 700, 16, torch.bfloat16),      # protected-layer widths, bf16 cache
    (3, 5, 4, 4, 2, 333, 0, torch.float16),        # no grouping, two query tokens, no window
    (2, 1, 6, 2, 3, 2100, 37, torch.float16),      # 9 query rows per KV head: three passes; two key blocks
    (7, 3, 2, 1, 1, 50, 64, torch.float16),        # everything inside the window (passthrough)
])
def test_decode_attention_widths_shapes_and_windows(kb, vb, hq, hkv, sq, sk, window, dtype):
    codec = tq.TurboQuantV3(128, key_bits=kb, value_bits=vb, residual_window=window, layer_idx=5, n_layers=36,
                            protected_layers=0, device=DEV)
    keys = O.synthetic_kv((2, hkv, sk, 128), dtype, seed=73000 + kb)
    vals = O.synthetic_kv((2, hkv, sk, 128), dtype, seed=74000 + vb)
    q = torch.randn(2, hq, sq, 128, generator=torch.Generator().manual_seed(kb * 10 + vb))
    _check(codec, keys, vals, q, scale=0.07)
    _check(codec, keys, vals, q.half(), scale=0.07)


def test_decode_attention_argument_errors():
    codec = tq.TurboQuantV3(128, key_bits=4, value_bits=2, residual_window=0, layer_idx=0, n_layers=4, protected_layers=0,
                            device=DEV)
    keys = O.synthetic_kv((1, 2, 64, 128), torch.float16, seed=1).to(DEV)
    ck, cv = codec.compress_kv(keys, keys)
    with pytest.raises(ValueError):
        codec.decode_attention(torch.randn(1, 3, 1, 128, device=DEV), ck, cv)         # 3 query heads on 2 KV heads
    with pytest.raises(ValueError):
        codec.decode_attention(torch.randn(1, 4, 1, 64, device=DEV), ck, cv)          # head_dim
    with pytest.raises(RuntimeError, match="no CPU path"):
        codec.decode_attention(torch.randn(1, 4, 1, 128), ck, cv)
