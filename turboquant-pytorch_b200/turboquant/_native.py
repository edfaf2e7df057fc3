"""ctypes binding of libturboquant_b200.so (the C ABI in include/turboquant_b200.h).

There is no fallback: if the library is missing, importing the compressors
fails with instructions to build it, and every compute entry point refuses
tensors that are not on a CUDA device.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# TURBOQUANT_B200_LIB points at another build of the same library (a profiling build made with
# `build.py --ablate --out ...`); unset, the in-tree library next to this file is loaded.
LIB_PATH = os.environ.get("TURBOQUANT_B200_LIB") or os.path.join(_HERE, "libturboquant_b200.so")

F32, F16, BF16 = 0, 1, 2
IDX_PACKED, IDX_U8, IDX_I64 = 0, 1, 2
EINVAL = -1                      # TQ_EINVAL
CODEBOOK_FLOATS = 800
SCORE_NOALLOC_SCRATCH_BYTES = 4 << 20

_DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


class BitsError(ValueError, ZeroDivisionError):
    """bits outside 1..8 (the reference fails with ZeroDivisionError in 8 // bits)."""


class QuantizeJob(C.Structure):
    _fields_ = [("x", C.c_void_p), ("x_dtype", C.c_int32), ("D", C.c_int32), ("bits", C.c_int32),
                ("normalize", C.c_int32), ("B", C.c_int64), ("H", C.c_int64), ("S", C.c_int64),
                ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_s", C.c_int64),
                ("rotation_t", C.c_void_p), ("codebook", C.c_void_p), ("idx_mode", C.c_int32),
                ("reserved", C.c_int32), ("idx_out", C.c_void_p), ("norms_out", C.c_void_p),
                ("rotation_image", C.c_void_p)]


class DequantizeJob(C.Structure):
    _fields_ = [("idx", C.c_void_p), ("norms", C.c_void_p), ("idx_mode", C.c_int32), ("D", C.c_int32),
                ("bits", C.c_int32), ("out_dtype", C.c_int32), ("B", C.c_int64), ("H", C.c_int64), ("S", C.c_int64),
                ("out", C.c_void_p), ("ostride_b", C.c_int64), ("ostride_h", C.c_int64), ("ostride_s", C.c_int64),
                ("rotation", C.c_void_p), ("codebook", C.c_void_p), ("rotation_image", C.c_void_p)]


class CopyJob(C.Structure):
    _fields_ = [("src", C.c_void_p), ("dst", C.c_void_p), ("elem_bytes", C.c_int32), ("D", C.c_int32),
                ("B", C.c_int64), ("H", C.c_int64), ("S", C.c_int64),
                ("sstride_b", C.c_int64), ("sstride_h", C.c_int64), ("sstride_s", C.c_int64),
                ("dstride_b", C.c_int64), ("dstride_h", C.c_int64), ("dstride_s", C.c_int64)]


class ScoreJob(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_dtype", C.c_int32), ("D", C.c_int32), ("bits", C.c_int32),
                ("reserved", C.c_int32), ("B", C.c_int64), ("Hq", C.c_int64), ("Sq", C.c_int64), ("Hkv", C.c_int64),
                ("Sk", C.c_int64), ("idx_bytes", C.c_void_p), ("norms", C.c_void_p), ("rotation_t", C.c_void_p),
                ("codebook", C.c_void_p), ("scale", C.c_float), ("reserved2", C.c_int32), ("logits", C.c_void_p),
                ("probs", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class DecodeAttnJob(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_dtype", C.c_int32), ("D", C.c_int32), ("key_bits", C.c_int32),
                ("value_bits", C.c_int32), ("B", C.c_int64), ("Hq", C.c_int64), ("Sq", C.c_int64), ("Hkv", C.c_int64),
                ("Sk", C.c_int64), ("k_idx", C.c_void_p), ("k_norms", C.c_void_p), ("v_idx", C.c_void_p),
                ("v_norms", C.c_void_p), ("k_rotation_t", C.c_void_p), ("v_rotation", C.c_void_p),
                ("k_codebook", C.c_void_p), ("v_codebook", C.c_void_p), ("k_window", C.c_void_p),
                ("v_window", C.c_void_p), ("window_dtype", C.c_int32), ("reserved", C.c_int32), ("W", C.c_int64),
                ("wstride_b", C.c_int64), ("wstride_h", C.c_int64), ("wstride_s", C.c_int64), ("scale", C.c_float),
                ("reserved2", C.c_int32), ("out", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class QjlCompressJob(C.Structure):
    _fields_ = [("x", C.c_void_p), ("x_dtype", C.c_int32), ("D", C.c_int32), ("bits", C.c_int32),
                ("normalize", C.c_int32), ("B", C.c_int64), ("H", C.c_int64), ("S", C.c_int64),
                ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_s", C.c_int64),
                ("rotation_t", C.c_void_p), ("rotation", C.c_void_p), ("codebook", C.c_void_p), ("qjl_t", C.c_void_p),
                ("M", C.c_int32), ("signs_dtype", C.c_int32), ("rnorm_dtype", C.c_int32), ("idx_mode", C.c_int32),
                ("k_mse_out", C.c_void_p), ("idx_out", C.c_void_p), ("signs_out", C.c_void_p), ("rnorm_out", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("vec_norms_out", C.c_void_p)]


class QjlPackedScoreJob(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_dtype", C.c_int32), ("D", C.c_int32), ("bits", C.c_int32), ("reserved", C.c_int32),
                ("BH", C.c_int64), ("Sq", C.c_int64), ("Sk", C.c_int64), ("idx_packed", C.c_void_p),
                ("sign_bits", C.c_void_p), ("vec_norms", C.c_void_p), ("rnorm", C.c_void_p), ("rotation_t", C.c_void_p),
                ("qjl_t", C.c_void_p), ("codebook", C.c_void_p), ("scores", C.c_void_p), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_size_t)]


class QjlScoreJob(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_dtype", C.c_int32), ("D", C.c_int32), ("BH", C.c_int64), ("Sq", C.c_int64),
                ("Sk", C.c_int64), ("k_mse", C.c_void_p), ("signs", C.c_void_p), ("rnorm", C.c_void_p),
                ("qjl_t", C.c_void_p), ("scores", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python turboquant-pytorch_b200/build.py` "
            "(nvcc, sm_100a).  There is no CPU or PyTorch fallback for the compression kernels.")
    L = C.CDLL(LIB_PATH)
    vp, i32, i64, sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
    L.tq_version.restype = i32
    L.tq_strerror.restype = C.c_char_p
    L.tq_strerror.argtypes = [i32]
    L.tq_last_cuda_error.restype = i32
    L.tq_launch_count.restype = i64
    L.tq_packed_row_bytes.argtypes = [i32, i32]
    L.tq_build_codebook.argtypes = [vp, i32, vp]
    L.tq_rotation_image_bytes.restype = sz
    L.tq_rotation_image_bytes.argtypes = [i32]
    L.tq_prepare_rotation_image.argtypes = [vp, i32, vp, vp]
    L.tq_prepare_rotation_image.restype = i32
    L.tq_last_device_status.restype = i32
    L.tq_quantize_rotated.argtypes = [vp, i64, i32, i32, vp, i32, vp, vp]
    L.tq_quantize.argtypes = [C.POINTER(QuantizeJob), i32, vp]
    L.tq_dequantize.argtypes = [C.POINTER(DequantizeJob), i32, vp]
    L.tq_project.argtypes = [vp, i32, i64, i32, vp, i32, vp, vp]
    L.tq_copy_rows.argtypes = [C.POINTER(CopyJob), i32, vp]
    L.tq_ablation_build.restype = i32
    L.tq_score_workspace_bytes.restype = sz
    L.tq_score_workspace_bytes.argtypes = [i64, i64, i64, i64, i32]
    L.tq_score_packed.argtypes = [C.POINTER(ScoreJob), vp]
    L.tq_score_packed_noalloc.argtypes = [C.POINTER(ScoreJob), vp]
    L.tq_decode_attention_workspace_bytes.restype = sz
    L.tq_decode_attention_workspace_bytes.argtypes = [i64, i64, i64, i64]
    L.tq_decode_attention.argtypes = [C.POINTER(DecodeAttnJob), vp]
    L.tq_decode_attention.restype = i32
    L.tq_qjl_compress.argtypes = [C.POINTER(QjlCompressJob), vp]
    L.tq_qjl_compress_workspace_bytes.restype = sz
    L.tq_qjl_compress_workspace_bytes.argtypes = [i64, i32]
    L.tq_qjl_scores_workspace_bytes.restype = sz
    L.tq_qjl_scores_workspace_bytes.argtypes = [i64, i64, i32]
    L.tq_qjl_scores.argtypes = [C.POINTER(QjlScoreJob), vp]
    L.tq_pack_mse_qjl.argtypes = [vp, vp, i64, i32, i32, vp, vp, vp]
    L.tq_pack_mse_qjl.restype = i32
    L.tq_qjl_scores_packed_workspace_bytes.restype = sz
    L.tq_qjl_scores_packed_workspace_bytes.argtypes = [i64, i64, i32]
    L.tq_qjl_scores_packed.argtypes = [C.POINTER(QjlPackedScoreJob), vp]
    L.tq_qjl_scores_packed.restype = i32
    L.tq_prod_inner_product.argtypes = [vp, i64, vp, vp, vp, i64, i32, i32, vp, vp, vp, vp, vp, sz, vp]
    for name in ("tq_packed_row_bytes", "tq_build_codebook", "tq_quantize_rotated", "tq_quantize", "tq_dequantize",
                 "tq_project", "tq_copy_rows", "tq_score_packed", "tq_score_packed_noalloc", "tq_qjl_compress", "tq_qjl_scores", "tq_prod_inner_product"):
        getattr(L, name).restype = i32
    _lib = L
    return L


def check(rc: int, what: str):
    """Map a TQ_E* code to the Python exception a caller of the reference would expect."""
    if rc == 0:
        return
    msg = f"{what}: {lib().tq_strerror(rc).decode()} (code {rc})"
    if rc == -2:
        raise BitsError(msg)
    if rc in (-1, -3, -4, -5, -6, -8, -9):
        raise ValueError(msg)
    if rc == -7:
        msg += f"; cudaError {lib().tq_last_cuda_error()}"
    raise RuntimeError(msg)


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}; use float32, float16 or bfloat16") from None


def require_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise RuntimeError(f"{what}: tensor is on {t.device}; the compression kernels run on CUDA (sm_100a) only "
                           "and there is no CPU path")


def warn_if_not_cuda(device, what: str):
    """Constructors call this.  An object built for a CPU device keeps the reference's host-side behaviour
    (constants, bit widths, memory accounting, window passthrough) but every compute call on it raises: say so
    when it is built, not at the first call."""
    if torch.device(device).type != "cuda":
        import warnings
        warnings.warn(f"{what}(device={str(device)!r}): the compression kernels run on a CUDA device (sm_100a) only; "
                      "compress/decompress/score calls on this object will raise (there is no CPU path)",
                      RuntimeWarning, stacklevel=3)


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def packed_row_bytes(D: int, bits: int) -> int:
    if not 1 <= bits <= 8:
        raise BitsError(f"bits must be in 1..8, got {bits}")
    ipb = 8 // bits
    return (D + ipb - 1) // ipb


def codebook_block(centroids: torch.Tensor, bits: int) -> torch.Tensor:
    """Device-format codebook block (centroids, exact decision thresholds, search shortcut), on the CPU."""
    c = centroids.detach().to("cpu", torch.float32).contiguous()
    if c.numel() != 2 ** bits:
        raise ValueError(f"expected {2 ** bits} centroids, got {c.numel()}")
    block = torch.empty(CODEBOOK_FLOATS, dtype=torch.float32)
    check(lib().tq_build_codebook(c.data_ptr(), bits, block.data_ptr()), "tq_build_codebook")
    return block


def rotation_image(m: torch.Tensor):
    """Tensor-core operand image of a (D, D) fp32 CUDA matrix, or None when there is no such path for D."""
    if not m.is_cuda:
        return None
    D = m.shape[0]
    nbytes = lib().tq_rotation_image_bytes(D)
    if nbytes == 0:
        return None
    m = m.contiguous()
    # over-allocate so that the image can start on a 1024-byte boundary
    buf = torch.empty(nbytes + 1024, dtype=torch.uint8, device=m.device)
    off = (-buf.data_ptr()) % 1024
    img = buf[off:off + nbytes]
    with torch.cuda.device(m.device):
        check(lib().tq_prepare_rotation_image(m.data_ptr(), D, img.data_ptr(), stream_ptr(m.device)),
              "tq_prepare_rotation_image")
    return img


def bhs_strides(t: torch.Tensor):
    """(tensor with unit last stride, stride_b, stride_h, stride_s) of a (B,H,S,D) tensor."""
    if t.stride(-1) != 1 and t.shape[-1] > 1:
        t = t.contiguous()
    return t, t.stride(0), t.stride(1), t.stride(2)
