"""Tensor-level wrappers over the C ABI: allocate outputs with torch, pass raw pointers.

Every function here runs on the tensors' CUDA device and on torch's current
stream; nothing synchronises.  Outputs are freshly allocated torch tensors.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _native as N


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def quantize_job(x: torch.Tensor, pi_t: torch.Tensor, codebook: torch.Tensor, bits: int, normalize: bool,
                 idx_mode: int, image: Optional[torch.Tensor] = None):
    """Prepare one quantise job for a (B,H,S,D) tensor; returns (job, idx_out, norms_out, keepalive)."""
    N.require_cuda(x, "quantize")
    B, H, S, D = x.shape
    x, sb, sh, ss = N.bhs_strides(x)
    n = B * H * S
    if idx_mode == N.IDX_PACKED:
        idx = torch.empty((B, H, S, N.packed_row_bytes(D, bits)), dtype=torch.uint8, device=x.device)
    elif idx_mode == N.IDX_U8:
        idx = torch.empty((n, D), dtype=torch.uint8, device=x.device)
    else:
        idx = torch.empty((n, D), dtype=torch.int64, device=x.device)
    norms = torch.empty((B, H, S), dtype=torch.float16, device=x.device) if normalize else None
    job = N.QuantizeJob(x=x.data_ptr(), x_dtype=N.dtype_code(x), D=D, bits=bits, normalize=int(normalize),
                        B=B, H=H, S=S, stride_b=sb, stride_h=sh, stride_s=ss, rotation_t=pi_t.data_ptr(),
                        codebook=codebook.data_ptr(), idx_mode=idx_mode, reserved=0, idx_out=idx.data_ptr(),
                        norms_out=_ptr(norms), rotation_image=_ptr(image))
    return job, idx, norms, x


def run_quantize(jobs: Sequence[N.QuantizeJob], device):
    arr = (N.QuantizeJob * len(jobs))(*jobs)
    with torch.cuda.device(device):
        N.check(N.lib().tq_quantize(arr, len(jobs), N.stream_ptr(device)), "tq_quantize")


def dequantize_job(idx: torch.Tensor, norms: Optional[torch.Tensor], shape, pi: torch.Tensor, codebook: torch.Tensor,
                   bits: int, idx_mode: int, out: torch.Tensor, image: Optional[torch.Tensor] = None):
    """One dequantise job writing into `out`, a (B,H,S,D) tensor or strided view with unit last stride."""
    N.require_cuda(idx, "dequantize")
    B, H, S, D = shape
    if not idx.is_contiguous():
        idx = idx.contiguous()
    if norms is not None and not norms.is_contiguous():
        norms = norms.contiguous()
    assert out.stride(-1) == 1 or D == 1
    job = N.DequantizeJob(idx=idx.data_ptr(), norms=_ptr(norms), idx_mode=idx_mode, D=D, bits=bits,
                          out_dtype=N.dtype_code(out), B=B, H=H, S=S, out=out.data_ptr(), ostride_b=out.stride(0),
                          ostride_h=out.stride(1), ostride_s=out.stride(2), rotation=pi.data_ptr(),
                          codebook=codebook.data_ptr(), rotation_image=_ptr(image))
    return job, (idx, norms)


def run_dequantize(jobs: Sequence[N.DequantizeJob], device):
    arr = (N.DequantizeJob * len(jobs))(*jobs)
    with torch.cuda.device(device):
        N.check(N.lib().tq_dequantize(arr, len(jobs), N.stream_ptr(device)), "tq_dequantize")


def project(x: torch.Tensor, m: torch.Tensor) -> torch.Tensor:
    """x (..., K) @ m (K, N) -> fp32 (..., N)."""
    N.require_cuda(x, "project")
    K, n_out = m.shape
    flat = x.reshape(-1, K)
    if not flat.is_contiguous():
        flat = flat.contiguous()
    out = torch.empty((flat.shape[0], n_out), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        N.check(N.lib().tq_project(flat.data_ptr(), N.dtype_code(flat), flat.shape[0], K, m.data_ptr(), n_out,
                                   out.data_ptr(), N.stream_ptr(x.device)), "tq_project")
    return out.reshape(*x.shape[:-1], n_out)


def quantize_rotated(y: torch.Tensor, codebook: torch.Tensor, bits: int, idx_mode: int = N.IDX_PACKED) -> torch.Tensor:
    """Rotated fp32 values (n, D) -> indices in the given layout."""
    N.require_cuda(y, "quantize_rotated")
    y = y.contiguous().float()
    n, D = y.shape
    if idx_mode == N.IDX_PACKED:
        out = torch.empty((n, N.packed_row_bytes(D, bits)), dtype=torch.uint8, device=y.device)
    elif idx_mode == N.IDX_U8:
        out = torch.empty((n, D), dtype=torch.uint8, device=y.device)
    else:
        out = torch.empty((n, D), dtype=torch.int64, device=y.device)
    with torch.cuda.device(y.device):
        N.check(N.lib().tq_quantize_rotated(y.data_ptr(), n, D, bits, codebook.data_ptr(), idx_mode, out.data_ptr(),
                                            N.stream_ptr(y.device)), "tq_quantize_rotated")
    return out


def _check_score_args(what, q, idx_bytes, norms, pi_t, codebook, bits, outs=()):
    """Shapes, dtypes, devices and contiguity of everything whose raw pointer goes to the score kernels: a
    wrong-size or wrong-dtype buffer would otherwise be read or written out of bounds.  Allocates nothing."""
    N.require_cuda(q, what)
    if q.dim() != 4 or idx_bytes.dim() != 4:
        raise ValueError(f"{what}: q must be (B,Hq,Sq,D) and idx_bytes (B,Hkv,Sk,G)")
    B, Hq, Sq, D = q.shape
    Bk, Hkv, Sk, G = idx_bytes.shape
    if Bk != B or Hkv < 1 or Hq % Hkv != 0:
        raise ValueError(f"{what}: batch {Bk} != {B} or query heads {Hq} not a multiple of KV heads {Hkv}")
    if idx_bytes.dtype != torch.uint8 or G != N.packed_row_bytes(D, bits):
        raise ValueError(f"{what}: idx_bytes must be uint8 with {N.packed_row_bytes(D, bits)} bytes per key")
    if norms.dtype != torch.float16 or tuple(norms.shape) != (B, Hkv, Sk):
        raise ValueError(f"{what}: norms must be float16 of shape {(B, Hkv, Sk)}")
    N.dtype_code(q)
    if pi_t.dtype != torch.float32 or tuple(pi_t.shape) != (D, D) or not pi_t.is_contiguous():
        raise ValueError(f"{what}: rotation must be a contiguous float32 ({D}, {D}) matrix")
    if codebook.dtype != torch.float32 or codebook.numel() != N.CODEBOOK_FLOATS or not codebook.is_contiguous():
        raise ValueError(f"{what}: codebook must be a contiguous float32 block of {N.CODEBOOK_FLOATS} values")
    for t in (idx_bytes, norms, pi_t, codebook) + tuple(outs):
        if t.device != q.device:
            raise ValueError(f"{what}: every tensor must be on {q.device}")
    for t in outs:
        if t.dtype != torch.float32 or tuple(t.shape) != (B, Hq, Sq, Sk) or not t.is_contiguous():
            raise ValueError(f"{what}: outputs must be contiguous float32 of shape {(B, Hq, Sq, Sk)}")
    return B, Hq, Sq, D, Hkv, Sk


def score_packed(q: torch.Tensor, idx_bytes: torch.Tensor, norms: torch.Tensor, pi_t: torch.Tensor,
                 codebook: torch.Tensor, bits: int, scale: float = 1.0, softmax: bool = False):
    """q (B,Hq,Sq,D); packed keys (B,Hkv,Sk,G) + norms (B,Hkv,Sk) -> logits (B,Hq,Sq,Sk) [, probs]."""
    q = q.contiguous()
    idx_bytes = idx_bytes.contiguous()
    norms = norms.contiguous()
    B, Hq, Sq, D, Hkv, Sk = _check_score_args("score_packed", q, idx_bytes, norms, pi_t, codebook, bits)
    logits = torch.empty((B, Hq, Sq, Sk), dtype=torch.float32, device=q.device)
    probs = torch.empty_like(logits) if softmax else None
    L = N.lib()
    ws_bytes = L.tq_score_workspace_bytes(B, Hq, Sq, Sk, D)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=q.device)
    job = N.ScoreJob(q=q.data_ptr(), q_dtype=N.dtype_code(q), D=D, bits=bits, reserved=0, B=B, Hq=Hq, Sq=Sq, Hkv=Hkv,
                     Sk=Sk, idx_bytes=idx_bytes.data_ptr(), norms=norms.data_ptr(), rotation_t=pi_t.data_ptr(),
                     codebook=codebook.data_ptr(), scale=float(scale), reserved2=0, logits=logits.data_ptr(),
                     probs=_ptr(probs), workspace=ws.data_ptr(), workspace_bytes=ws.numel())
    with torch.cuda.device(q.device):
        N.check(L.tq_score_packed(C.byref(job), N.stream_ptr(q.device)), "tq_score_packed")
    return (logits, probs) if softmax else logits


def score_packed_noalloc(q: torch.Tensor, idx_bytes: torch.Tensor, norms: torch.Tensor, pi_t: torch.Tensor,
                          codebook: torch.Tensor, bits: int, logits: torch.Tensor, probs: Optional[torch.Tensor] = None,
                          scale: float = 1.0):
    """score_packed for callers that bring every buffer themselves and may not allocate.

    `logits` (and `probs`, if wanted) are caller-owned (B,Hq,Sq,Sk) fp32 tensors; the
    scratch comes from the library's built-in 4 MiB array, so this wrapper creates no
    tensor.  Inputs must already be contiguous.  Raises ValueError when the problem
    needs more scratch than the built-in array holds.
    """
    for t in (q, idx_bytes, norms):
        if not t.is_contiguous():
            raise ValueError("score_packed_noalloc takes contiguous tensors (it will not make copies)")
    outs = (logits,) + ((probs,) if probs is not None else ())
    B, Hq, Sq, D, Hkv, Sk = _check_score_args("score_packed_noalloc", q, idx_bytes, norms, pi_t, codebook, bits, outs)
    job = N.ScoreJob(q=q.data_ptr(), q_dtype=N.dtype_code(q), D=D, bits=bits, reserved=0, B=B, Hq=Hq, Sq=Sq, Hkv=Hkv,
                     Sk=Sk, idx_bytes=idx_bytes.data_ptr(), norms=norms.data_ptr(), rotation_t=pi_t.data_ptr(),
                     codebook=codebook.data_ptr(), scale=float(scale), reserved2=0, logits=logits.data_ptr(),
                     probs=_ptr(probs), workspace=None, workspace_bytes=0)
    with torch.cuda.device(q.device):
        N.check(N.lib().tq_score_packed_noalloc(C.byref(job), N.stream_ptr(q.device)), "tq_score_packed_noalloc")
    return logits if probs is None else (logits, probs)


def decode_attention(q: torch.Tensor, k_comp: Optional[dict], v_comp: Optional[dict], key_codec, val_codec,
                     k_window: Optional[torch.Tensor], v_window: Optional[torch.Tensor], scale: float) -> torch.Tensor:
    """softmax(scale * q K_hat^T) V_hat over the packed tokens of (k_comp, v_comp) followed by the kept window tokens.

    q (B, Hq, Sq, 128); k_comp / v_comp are MSECompressor dicts ((B, Hkv, Sk, G) packed rows + norms) or None;
    the windows are (B, Hkv, W, 128) tensors (views are fine, unit last stride) or None.  Returns fp32 (B, Hq, Sq, 128).
    """
    N.require_cuda(q, "decode_attention")
    B, Hq, Sq, D = q.shape
    if D != 128:
        raise ValueError("decode_attention: head_dim must be 128")
    q = q.contiguous()
    dev = q.device
    Sk = 0
    k_idx = k_norms = v_idx = v_norms = None
    Hkv = None
    if k_comp is not None:
        k_idx, k_norms = k_comp["idx_bytes"].contiguous(), k_comp["vec_norms"].contiguous()
        v_idx, v_norms = v_comp["idx_bytes"].contiguous(), v_comp["vec_norms"].contiguous()
        _, Hkv, Sk, Gk = k_idx.shape
        if tuple(v_idx.shape[:3]) != (B, Hkv, Sk) or k_idx.shape[0] != B:
            raise ValueError("decode_attention: packed keys and values must cover the same (B, Hkv, Sk) tokens")
        if Gk != N.packed_row_bytes(D, key_codec.bits) or v_idx.shape[3] != N.packed_row_bytes(D, val_codec.bits):
            raise ValueError("decode_attention: packed row sizes do not match the code widths")
        if k_idx.dtype != torch.uint8 or v_idx.dtype != torch.uint8 or k_norms.dtype != torch.float16 or v_norms.dtype != torch.float16:
            raise ValueError("decode_attention: packed rows must be uint8 and norms float16")
    W = 0
    if k_window is not None and k_window.shape[2] > 0:
        if k_window.shape != v_window.shape or k_window.dtype != v_window.dtype or k_window.stride() != v_window.stride():
            raise ValueError("decode_attention: key and value windows must have the same shape, dtype and strides")
        if k_window.stride(3) != 1:
            k_window, v_window = k_window.contiguous(), v_window.contiguous()
        W = k_window.shape[2]
        Hkv = k_window.shape[1] if Hkv is None else Hkv
        if k_window.shape[0] != B or k_window.shape[1] != Hkv or k_window.shape[3] != D:
            raise ValueError("decode_attention: window shape does not match the queries / packed tokens")
    else:
        k_window = v_window = None
    if Hkv is None:
        raise ValueError("decode_attention: nothing to attend to")
    if Hq % Hkv:
        raise ValueError(f"decode_attention: {Hq} query heads over {Hkv} KV heads")
    for tt in (k_idx, k_norms, v_idx, v_norms, k_window, v_window):
        if tt is not None and tt.device != dev:
            raise ValueError(f"decode_attention: every tensor must be on {dev}")
    out = torch.empty((B, Hq, Sq, D), dtype=torch.float32, device=dev)
    L = N.lib()
    ws_bytes = L.tq_decode_attention_workspace_bytes(B, Hq, Sq, Sk)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
    job = N.DecodeAttnJob(q=q.data_ptr(), q_dtype=N.dtype_code(q), D=D, key_bits=key_codec.bits, value_bits=val_codec.bits,
                          B=B, Hq=Hq, Sq=Sq, Hkv=Hkv, Sk=Sk, k_idx=_ptr(k_idx), k_norms=_ptr(k_norms), v_idx=_ptr(v_idx),
                          v_norms=_ptr(v_norms), k_rotation_t=key_codec._pi_t.data_ptr(), v_rotation=val_codec.Pi.data_ptr(),
                          k_codebook=key_codec._cb.data_ptr(), v_codebook=val_codec._cb.data_ptr(), k_window=_ptr(k_window),
                          v_window=_ptr(v_window), window_dtype=N.dtype_code(k_window) if W else N.F16, reserved=0, W=W,
                          wstride_b=k_window.stride(0) if W else 0, wstride_h=k_window.stride(1) if W else 0,
                          wstride_s=k_window.stride(2) if W else 0, scale=float(scale), reserved2=0, out=out.data_ptr(),
                          workspace=ws.data_ptr(), workspace_bytes=ws.numel())
    with torch.cuda.device(dev):
        N.check(L.tq_decode_attention(C.byref(job), N.stream_ptr(dev)), "tq_decode_attention")
    return out


def qjl_compress(x: torch.Tensor, pi: torch.Tensor, pi_t: torch.Tensor, codebook: torch.Tensor, qjl_t: torch.Tensor,
                 bits: int, normalize: bool, want_k_mse: bool, idx_mode: Optional[int], signs_fp32: bool,
                 rnorm_fp32: bool, want_vec_norms: bool = False):
    """MSE stage + QJL signs for a (B,H,S,D) tensor.  Returns (k_mse|None, idx|None, signs (n,M), rnorm (n,)), and
    the fp32 vector norms (n,) as a fifth value with want_vec_norms."""
    N.require_cuda(x, "qjl_compress")
    B, H, S, D = x.shape
    x, sb, sh, ss = N.bhs_strides(x)
    n = B * H * S
    M = qjl_t.shape[1]
    dev = x.device
    k_mse = torch.empty((n, D), dtype=torch.float16, device=dev) if want_k_mse else None
    idx = None
    if idx_mode is not None:
        idx = torch.empty((n, D), dtype=torch.int64 if idx_mode == N.IDX_I64 else torch.uint8, device=dev)
    signs = torch.empty((n, M), dtype=torch.float32 if signs_fp32 else torch.int8, device=dev)
    rnorm = torch.empty((n,), dtype=torch.float32 if rnorm_fp32 else torch.float16, device=dev)
    # scratch for the tensor-core path (fp16 vectors, head_dim 128 / 256, the V2 output formats); without it
    # the library runs the FP32 kernels
    ws, ws_bytes = None, 0
    vnorm = torch.empty((n,), dtype=torch.float32, device=dev) if want_vec_norms else None
    if x.dtype == torch.float16 and normalize and idx_mode in (None, N.IDX_U8) and not signs_fp32 and not rnorm_fp32:
        ws_bytes = N.lib().tq_qjl_compress_workspace_bytes(n, D)
        if ws_bytes:
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    job = N.QjlCompressJob(x=x.data_ptr(), x_dtype=N.dtype_code(x), D=D, bits=bits, normalize=int(normalize), B=B, H=H,
                           S=S, stride_b=sb, stride_h=sh, stride_s=ss, rotation_t=pi_t.data_ptr(),
                           rotation=pi.data_ptr(), codebook=codebook.data_ptr(), qjl_t=qjl_t.data_ptr(), M=M,
                           signs_dtype=int(signs_fp32), rnorm_dtype=N.F32 if rnorm_fp32 else N.F16,
                           idx_mode=idx_mode if idx_mode is not None else N.IDX_U8, k_mse_out=_ptr(k_mse),
                           idx_out=_ptr(idx), signs_out=signs.data_ptr(), rnorm_out=rnorm.data_ptr(),
                           workspace=_ptr(ws), workspace_bytes=ws_bytes, vec_norms_out=_ptr(vnorm))
    with torch.cuda.device(dev):
        N.check(N.lib().tq_qjl_compress(C.byref(job), N.stream_ptr(dev)), "tq_qjl_compress")
    if want_vec_norms:
        return k_mse, idx, signs, rnorm, vnorm
    return k_mse, idx, signs, rnorm


def qjl_compress_packed(x: torch.Tensor, pi: torch.Tensor, pi_t: torch.Tensor, codebook: torch.Tensor,
                        qjl_t: torch.Tensor, bits: int):
    """MSE stage + QJL signs of a (B,H,S,D) tensor straight into the packed form: returns (index rows (n, G) uint8,
    sign bits (n, D/8) uint8, residual norms (n,) fp16, vector norms (n,) fp32).  The tensor-core path writes the packed
    rows from its epilogues; inputs it does not take go through the unpacked outputs and tq_pack_mse_qjl."""
    N.require_cuda(x, "qjl_compress")
    B, H, S, D = x.shape
    n = B * H * S
    dev = x.device
    L = N.lib()
    if x.dtype == torch.float16 and x.is_contiguous() and D in (128, 256) and qjl_t.shape[1] == D and n > 0:
        ws_bytes = L.tq_qjl_compress_workspace_bytes(n, D)
        if ws_bytes:
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            rows = torch.empty((n, N.packed_row_bytes(D, bits)), dtype=torch.uint8, device=dev)
            sbits = torch.empty((n, D // 8), dtype=torch.uint8, device=dev)
            rnorm = torch.empty((n,), dtype=torch.float16, device=dev)
            vnorm = torch.empty((n,), dtype=torch.float32, device=dev)
            job = N.QjlCompressJob(x=x.data_ptr(), x_dtype=N.dtype_code(x), D=D, bits=bits, normalize=1, B=B, H=H, S=S,
                                   stride_b=H * S * D, stride_h=S * D, stride_s=D, rotation_t=pi_t.data_ptr(),
                                   rotation=pi.data_ptr(), codebook=codebook.data_ptr(), qjl_t=qjl_t.data_ptr(), M=D,
                                   signs_dtype=2, rnorm_dtype=N.F16, idx_mode=N.IDX_PACKED, k_mse_out=None,
                                   idx_out=rows.data_ptr(), signs_out=sbits.data_ptr(), rnorm_out=rnorm.data_ptr(),
                                   workspace=ws.data_ptr(), workspace_bytes=ws_bytes, vec_norms_out=vnorm.data_ptr())
            with torch.cuda.device(dev):
                rc = L.tq_qjl_compress(C.byref(job), N.stream_ptr(dev))
            if rc == 0:
                return rows, sbits, rnorm, vnorm
            if rc != N.EINVAL:
                N.check(rc, "tq_qjl_compress")
    _k, idx, signs, rnorm, vnorm = qjl_compress(x, pi, pi_t, codebook, qjl_t, bits, normalize=True, want_k_mse=False,
                                                idx_mode=N.IDX_U8, signs_fp32=False, rnorm_fp32=False, want_vec_norms=True)
    rows, sbits = pack_mse_qjl(idx, signs, D, bits)
    return rows, sbits, rnorm, vnorm


def pack_mse_qjl(idx_u8: Optional[torch.Tensor], signs_i8: Optional[torch.Tensor], D: int, bits: int):
    """(n, D) uint8 indices and (n, D) int8 signs -> (packed index rows (n, G) | None, sign bits (n, D/8) | None)."""
    src = idx_u8 if idx_u8 is not None else signs_i8
    N.require_cuda(src, "pack_mse_qjl")
    n = src.shape[0]
    dev = src.device
    packed = torch.empty((n, N.packed_row_bytes(D, bits)), dtype=torch.uint8, device=dev) if idx_u8 is not None else None
    sbits = torch.empty((n, D // 8), dtype=torch.uint8, device=dev) if signs_i8 is not None else None
    if idx_u8 is not None:
        idx_u8 = idx_u8.contiguous()
    if signs_i8 is not None:
        signs_i8 = signs_i8.contiguous()
    with torch.cuda.device(dev):
        N.check(N.lib().tq_pack_mse_qjl(_ptr(idx_u8), _ptr(signs_i8), n, D, bits, _ptr(packed), _ptr(sbits),
                                        N.stream_ptr(dev)), "tq_pack_mse_qjl")
    return packed, sbits


def qjl_scores_packed(q: torch.Tensor, idx_packed: torch.Tensor, sign_bits: torch.Tensor, vec_norms: torch.Tensor,
                      rnorm: torch.Tensor, pi_t: torch.Tensor, qjl_t: torch.Tensor, codebook: torch.Tensor, bits: int):
    """q (B,H,Sq,D) against the packed MSE+QJL form ((B,H,Sk,G) index rows, (B,H,Sk,D/8) sign bits, fp32 vector norms,
    fp16 residual norms) -> (B,H,Sq,Sk) fp32."""
    N.require_cuda(q, "qjl_scores_packed")
    B, H, Sq, D = q.shape
    Sk = idx_packed.shape[2]
    if D not in (128, 256):
        raise ValueError("qjl_scores_packed: head_dim must be 128 or 256")
    if tuple(idx_packed.shape) != (B, H, Sk, N.packed_row_bytes(D, bits)) or tuple(sign_bits.shape) != (B, H, Sk, D // 8):
        raise ValueError("qjl_scores_packed: packed shapes do not match the queries")
    if idx_packed.dtype != torch.uint8 or sign_bits.dtype != torch.uint8 or vec_norms.dtype != torch.float32 or \
            rnorm.dtype != torch.float16 or tuple(vec_norms.shape) != (B, H, Sk) or tuple(rnorm.shape) != (B, H, Sk):
        raise ValueError("qjl_scores_packed: uint8 rows, fp32 vector norms and fp16 residual norms of shape (B, H, Sk)")
    q = q.contiguous()
    idx_packed, sign_bits, vec_norms, rnorm = (t.contiguous() for t in (idx_packed, sign_bits, vec_norms, rnorm))
    out = torch.empty((B, H, Sq, Sk), dtype=torch.float32, device=q.device)
    L = N.lib()
    ws_bytes = L.tq_qjl_scores_packed_workspace_bytes(B * H, Sq, D)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=q.device)
    job = N.QjlPackedScoreJob(q=q.data_ptr(), q_dtype=N.dtype_code(q), D=D, bits=bits, reserved=0, BH=B * H, Sq=Sq, Sk=Sk,
                              idx_packed=idx_packed.data_ptr(), sign_bits=sign_bits.data_ptr(),
                              vec_norms=vec_norms.data_ptr(), rnorm=rnorm.data_ptr(), rotation_t=pi_t.data_ptr(),
                              qjl_t=qjl_t.data_ptr(), codebook=codebook.data_ptr(), scores=out.data_ptr(),
                              workspace=ws.data_ptr(), workspace_bytes=ws.numel())
    with torch.cuda.device(q.device):
        N.check(L.tq_qjl_scores_packed(C.byref(job), N.stream_ptr(q.device)), "tq_qjl_scores_packed")
    return out


def qjl_scores(q: torch.Tensor, k_mse: torch.Tensor, signs: torch.Tensor, rnorm: torch.Tensor,
               qjl_t: torch.Tensor) -> torch.Tensor:
    """q (B,H,Sq,D) against the compressed dict tensors -> (B,H,Sq,Sk) fp32."""
    N.require_cuda(q, "qjl_scores")
    B, H, Sq, D = q.shape
    Sk = k_mse.shape[2]
    q = q.contiguous()
    k_mse, signs, rnorm = k_mse.contiguous(), signs.contiguous(), rnorm.contiguous()
    out = torch.empty((B, H, Sq, Sk), dtype=torch.float32, device=q.device)
    L = N.lib()
    ws_bytes = L.tq_qjl_scores_workspace_bytes(B * H, Sq, D)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=q.device)
    job = N.QjlScoreJob(q=q.data_ptr(), q_dtype=N.dtype_code(q), D=D, BH=B * H, Sq=Sq, Sk=Sk, k_mse=k_mse.data_ptr(),
                        signs=signs.data_ptr(), rnorm=rnorm.data_ptr(), qjl_t=qjl_t.data_ptr(), scores=out.data_ptr(),
                        workspace=ws.data_ptr(), workspace_bytes=ws.numel())
    with torch.cuda.device(q.device):
        N.check(L.tq_qjl_scores(C.byref(job), N.stream_ptr(q.device)), "tq_qjl_scores")
    return out


def prod_inner_product(y: torch.Tensor, idx: torch.Tensor, signs: torch.Tensor, rnorm: torch.Tensor, pi: torch.Tensor,
                       codebook: torch.Tensor, qjl_t: torch.Tensor) -> torch.Tensor:
    """Row-paired estimator; y is (n, D) or a single row (1, D)."""
    N.require_cuda(idx, "prod_inner_product")
    n, D = idx.shape
    M = signs.shape[1]
    y = y.float().contiguous()
    out = torch.empty((n,), dtype=torch.float32, device=idx.device)
    ws = torch.empty(max((n + y.shape[0]) * 256 * 4, 256), dtype=torch.uint8, device=idx.device)
    with torch.cuda.device(idx.device):
        N.check(N.lib().tq_prod_inner_product(
            y.data_ptr(), y.shape[0], idx.contiguous().data_ptr(), signs.contiguous().data_ptr(),
            rnorm.contiguous().data_ptr(), n, D, M, pi.data_ptr(), codebook.data_ptr(), qjl_t.data_ptr(),
            out.data_ptr(), ws.data_ptr(), ws.numel(), N.stream_ptr(idx.device)), "tq_prod_inner_product")
    return out
