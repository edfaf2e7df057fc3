"""The allocation-free packed-key score entry point (tq_score_packed_noalloc).

Who needs it: callers that cannot hand scratch memory to the library -- code living
inside another framework's fixed memory plan, serving loops that keep the allocator
off the request path, minimal FFI bindings.  The entry point must give the same
logits and probabilities as tq_score_packed while taking its scratch from the array
built into the library, on repeated calls that reuse that array.

This file sorts last on purpose: a run that stops at the first failure has then
already executed every other test.
"""

import ctypes

import pytest
import torch

import tq_oracle as O

import turboquant as tq
from turboquant import _native as N
from turboquant import _ops

DEV = "cuda"


def _case(seed, hkv, rep, sq, sk, bits):
    keys = O.synthetic_kv((2, hkv, sk, 128), torch.float16, seed=seed).to(DEV)
    q = torch.randn(2, hkv * rep, sq, 128, generator=torch.Generator().manual_seed(seed + 1)).to(DEV)
    comp = tq.MSECompressor(128, bits, seed=seed + 2, device=DEV)
    return comp, comp.compress(keys), q


@pytest.mark.gpu
def test_noalloc_scores_equal_the_workspace_entry_point_on_consecutive_calls():
    # two different problems back to back: the second call finds the first call's leftovers in the scratch
    for seed, hkv, rep, sq, sk, bits in ((11, 2, 4, 1, 5000, 4), (23, 1, 2, 3, 1300, 2)):
        comp, c, q = _case(seed, hkv, rep, sq, sk, bits)
        want_logits, want_probs = _ops.score_packed(q, c["idx_bytes"], c["vec_norms"], comp._pi_t, comp._cb, bits,
                                                    scale=0.25, softmax=True)
        logits = torch.full_like(want_logits, float("nan"))
        probs = torch.full_like(want_probs, float("nan"))
        _ops.score_packed_noalloc(q, c["idx_bytes"], c["vec_norms"], comp._pi_t, comp._cb, bits, logits, probs, scale=0.25)
        torch.cuda.synchronize()
        scale = float(want_logits.abs().max())
        assert float((logits - want_logits).abs().max()) <= 1e-5 * scale
        assert torch.allclose(probs, want_probs, rtol=2e-4, atol=1e-7)
        # and against the CPU oracle: decompress the same packed keys, then matmul and softmax
        cpu = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in c.items()}
        rec = O.mse_decompress(cpu, comp.Pi.cpu(), O.lloyd_max(128, bits)[0], bits)
        oracle_logits = O.v3_scores(q.cpu(), rec) * 0.25
        assert float((logits.cpu() - oracle_logits).abs().max()) <= 1e-5 * float(oracle_logits.abs().max())
        assert torch.allclose(probs.cpu(), torch.softmax(oracle_logits, -1), rtol=2e-4, atol=1e-7)
        # logits only (probs NULL)
        only = torch.empty_like(want_logits)
        _ops.score_packed_noalloc(q, c["idx_bytes"], c["vec_norms"], comp._pi_t, comp._cb, bits, only, None, scale=0.25)
        assert float((only - want_logits).abs().max()) <= 1e-5 * scale


@pytest.mark.gpu
def test_noalloc_rejects_problems_beyond_its_scratch():
    comp, c, q = _case(5, 1, 1, 1, 64, 4)
    lib = N.lib()
    rows_too_many = (N.SCORE_NOALLOC_SCRATCH_BYTES // (128 * 4)) + 8
    assert lib.tq_score_workspace_bytes(1, rows_too_many, 1, 64, 128) > N.SCORE_NOALLOC_SCRATCH_BYTES
    job = N.ScoreJob(q=q.data_ptr(), q_dtype=N.F32, D=128, bits=4, B=1, Hq=rows_too_many, Sq=1, Hkv=1, Sk=64,
                     idx_bytes=c["idx_bytes"].data_ptr(), norms=c["vec_norms"].data_ptr(), rotation_t=comp._pi_t.data_ptr(),
                     codebook=comp._cb.data_ptr(), scale=1.0, logits=q.data_ptr(), probs=None, workspace=None,
                     workspace_bytes=0)
    assert lib.tq_score_packed_noalloc(ctypes.byref(job), None) == -9          # TQ_ETOOBIG, nothing launched
    with pytest.raises(ValueError, match="capacity"):
        N.check(-9, "tq_score_packed_noalloc")


def test_noalloc_argument_checks_without_a_gpu():
    lib = N.lib()
    assert lib.tq_score_packed_noalloc(None, None) == -4
    job = N.ScoreJob(D=128, bits=9, B=1, Hq=1, Sq=1, Hkv=1, Sk=1)
    assert lib.tq_score_packed_noalloc(ctypes.byref(job), None) == -2
    job = N.ScoreJob(D=128, bits=4, B=1, Hq=3, Sq=1, Hkv=2, Sk=1)
    assert lib.tq_score_packed_noalloc(ctypes.byref(job), None) == -1
    job = N.ScoreJob(D=128, bits=4, B=0, Hq=4, Sq=1, Hkv=2, Sk=10)
    assert lib.tq_score_packed_noalloc(ctypes.byref(job), None) == 0              # empty problem
