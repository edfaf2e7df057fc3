"""The incremental cache beyond the reference harness: the all-layers step(), the transformers base class, saving
and restoring a cache, and decode attention straight from its packed store."""

import io

import pytest
import torch

import tq_oracle as O

import turboquant as tq
from turboquant.cache import V3Cache

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _tokens(L, total, seed):
    ks = [O.synthetic_kv((2, 2, total, 128), torch.float16, seed + l).to(DEV) for l in range(L)]
    vs = [O.synthetic_kv((2, 2, total, 128), torch.float16, seed + 100 + l).to(DEV) for l in range(L)]
    return ks, vs


@pytest.mark.parametrize("rw", [0, 16])
def test_step_for_all_layers_equals_per_layer_updates(rw):
    L, prefill, total = 3, 70, 110
    ks, vs = _tokens(L, total, 81000 + rw)
    kw = dict(key_bits=4, value_bits=2, residual_window=rw, protected_layers=1, n_layers=L, initial_capacity=256)
    a, b = V3Cache(**kw), V3Cache(**kw)
    for l in range(L):
        a.update(ks[l][:, :, :prefill], vs[l][:, :, :prefill], l)
    outs = b.step([k[:, :, :prefill] for k in ks], [v[:, :, :prefill] for v in vs])      # creates the layers: falls back
    assert len(outs) == L
    for t in range(prefill, total):
        for l in range(L):
            fa = a.update(ks[l][:, :, t:t + 1], vs[l][:, :, t:t + 1], l)
        outs = b.step([k[:, :, t:t + 1] for k in ks], [v[:, :, t:t + 1] for v in vs])
    torch.cuda.synchronize()
    for l in range(L):
        ka, va = a._layers[l].k[:, :, :total], a._layers[l].v[:, :, :total]
        assert torch.equal(outs[l][0], ka) and torch.equal(outs[l][1], va)
        assert b.get_seq_length(l) == a.get_seq_length(l) == total
        (cka, cva), (ckb, cvb) = a.packed_layer(l), b.packed_layer(l)
        assert torch.equal(cka["compressed"]["idx_bytes"], ckb["compressed"]["idx_bytes"])
        assert torch.equal(cva["compressed"]["vec_norms"], cvb["compressed"]["vec_norms"])
        assert cka["split_at"] == ckb["split_at"] == total - rw
        if rw:
            assert torch.equal(outs[l][0][:, :, -rw:], ks[l][:, :, -rw:])
    assert b.get_compression_info() == a.get_compression_info()
    assert b.step([k[:, :, :1] for k in ks], [v[:, :, :1] for v in vs], return_views=False) is None


def test_cache_is_a_transformers_dynamic_cache_when_available():
    try:
        from transformers.cache_utils import DynamicCache
    except Exception:
        pytest.skip("transformers is not installed")
    cache = V3Cache(n_layers=2)
    assert isinstance(cache, DynamicCache)
    k = O.synthetic_kv((1, 2, 5, 128), torch.float16, 5).to(DEV)
    fk, fv = cache.update(k, k, 1)                       # layer 1 first: the base class's layer list is padded
    assert fk.shape == (1, 2, 5, 128) and cache.get_seq_length(1) == 5 and cache.get_seq_length(0) == 0
    assert len(cache.layers) >= 2


def test_cache_state_round_trip_through_torch_save():
    L, total = 2, 90
    ks, vs = _tokens(L, total + 10, 82000)
    kw = dict(key_bits=6, value_bits=4, residual_window=8, protected_layers=1, n_layers=L, initial_capacity=128)
    cache = V3Cache(**kw)
    cache.step([k[:, :, :total] for k in ks], [v[:, :, :total] for v in vs])
    buf = io.BytesIO()
    torch.save(cache.cache_state(), buf)
    buf.seek(0)
    restored = V3Cache.from_cache_state(torch.load(buf, weights_only=False), device=DEV)
    for t in range(total, total + 10):                  # both continue identically
        o1 = cache.step([k[:, :, t:t + 1] for k in ks], [v[:, :, t:t + 1] for v in vs])
        o2 = restored.step([k[:, :, t:t + 1] for k in ks], [v[:, :, t:t + 1] for v in vs])
    for l in range(L):
        assert torch.equal(o1[l][0], o2[l][0]) and torch.equal(o1[l][1], o2[l][1])
        (c1, _), (c2, _) = cache.packed_layer(l), restored.packed_layer(l)
        assert torch.equal(c1["compressed"]["idx_bytes"], c2["compressed"]["idx_bytes"])
    assert restored.get_compression_info() == cache.get_compression_info()


def test_compressed_dicts_survive_torch_save():
    x = O.synthetic_kv((1, 2, 200, 128), torch.float16, 83000).to(DEV)
    codec = tq.TurboQuantV3(128, key_bits=4, value_bits=2, residual_window=16, layer_idx=1, n_layers=4, protected_layers=0,
                            device=DEV)
    ck, cv = codec.compress_kv(x, x * 0.5)
    buf = io.BytesIO()
    torch.save((ck, cv), buf)
    buf.seek(0)
    ck2, cv2 = torch.load(buf, weights_only=False)
    r1, r2 = codec.decompress_kv(ck, cv), codec.decompress_kv(ck2, cv2)
    assert torch.equal(r1[0], r2[0]) and torch.equal(r1[1], r2[1])
    v2 = tq.TurboQuantCompressorV2(128, 3, seed=3, device=DEV)
    c = v2.compress(x)
    buf = io.BytesIO()
    torch.save(c, buf)
    buf.seek(0)
    c2 = torch.load(buf, weights_only=False)
    q = torch.randn(1, 2, 3, 128, device=DEV)
    assert torch.equal(v2.asymmetric_attention_scores(q, c), v2.asymmetric_attention_scores(q, c2))


def test_decode_attention_from_the_cache_store():
    """Attention over a layer of the incremental cache straight from its packed store equals attention over the
    tensors update() returns (reconstructions + window), up to the 16-bit rounding of those tensors."""
    cache = V3Cache(key_bits=4, value_bits=2, residual_window=32, protected_layers=0, n_layers=2, initial_capacity=512)
    ks, vs = _tokens(1, 300, 84000)
    fk, fv = cache.update(ks[0][:, :, :200], vs[0][:, :, :200], 0)
    for t in range(200, 300):
        fk, fv = cache.update(ks[0][:, :, t:t + 1], vs[0][:, :, t:t + 1], 0)
    ck, cv = cache.packed_layer(0)
    q = torch.randn(2, 8, 1, 128, generator=torch.Generator().manual_seed(1))
    out = cache._layers[0].codec.decode_attention(q.to(DEV), ck, cv)
    want = O.v3_decode_attention(q, fk.float().cpu(), fv.float().cpu(), 128 ** -0.5)
    assert float((out.cpu() - want).abs().max() / want.abs().max()) <= 2e-3      # fk, fv are fp16 reconstructions
