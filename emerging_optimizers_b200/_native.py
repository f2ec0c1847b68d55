"""ctypes binding of ``libeo_b200.so`` (C ABI declared in ``include/eo_b200.h``).

The library is built in-tree by ``emerging_optimizers_b200/build.py``.  There is no fallback: if the shared
object is missing or a call fails, the functions here raise.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_int64, c_size_t, c_uint32, c_void_p

import torch


_LIB_NAME = "libeo_b200.so"
_lib: ctypes.CDLL | None = None

EO_OK = 0
_STATUS_NAMES = {
    1: "EO_ERR_BAD_ARG",
    2: "EO_ERR_CUDA",
    3: "EO_ERR_UNSUPPORTED",
    4: "EO_ERR_WORKSPACE",
    5: "EO_ERR_DEVICE_WAIT",
}

# name -> (restype, argtypes); mirrors include/eo_b200.h one to one.
_PROTOTYPES: dict[str, tuple] = {
    "eo_version": (c_char_p, []),
    "eo_last_error": (c_char_p, []),
    "eo_read_device_status": (c_int, [POINTER(c_uint32), c_void_p]),
    "eo_gemm": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64]
        + [c_void_p, c_int, c_int64, c_int64]
        + [c_void_p, c_int64, c_int64]
        + [c_void_p, c_int64, c_int64]
        + [c_int, c_int, c_int, c_int]
        + [c_float, c_float, c_float]
        + [c_int, c_int, c_int, c_void_p],
    ),
    "eo_syrk": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64]
        + [c_void_p, c_int64, c_int64]
        + [c_void_p, c_int64, c_int64]
        + [c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_void_p],
    ),
    "eo_sumsq_scratch_bytes": (c_size_t, [c_int, c_int64, c_int64]),
    "eo_sumsq_f32": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_size_t, c_void_p],
    ),
    "eo_normalize_f32": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p, c_float, c_int]
        + [c_void_p, c_int64, c_int64, c_int, c_int, c_void_p],
    ),
}


class NativeLibraryError(RuntimeError):
    """Raised when ``libeo_b200.so`` is missing or one of its entry points reports a failure."""


def library_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), _LIB_NAME)


def exported_symbols() -> list[str]:
    """Names every build of the library must export (the functions declared in ``include/eo_b200.h``)."""
    return list(_PROTOTYPES)


def lib() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise NativeLibraryError(
                f"{path} not found: build it with `python -m emerging_optimizers_b200.build`. "
                "This package has no CPU or PyTorch fallback."
            )
        handle = ctypes.CDLL(path)
        for name, (restype, argtypes) in _PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def _check(rc: int, what: str) -> None:
    if rc != EO_OK:
        msg = lib().eo_last_error().decode()
        raise NativeLibraryError(f"{what} failed with {_STATUS_NAMES.get(rc, rc)}: {msg}")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(t: torch.Tensor, name: str = "tensor") -> None:
    if not t.is_cuda:
        raise NativeLibraryError(
            f"{name} is on {t.device}; emerging_optimizers_b200 runs on CUDA sm_100 devices only "
            "(there is no CPU path)."
        )


def read_device_status(device: torch.device | None = None) -> int:
    """Synchronise the current stream and return (and clear) the kernels' bounded-wait status word."""
    code = c_uint32(0)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(dev):
        _check(lib().eo_read_device_status(ctypes.byref(code), torch.cuda.current_stream(dev).cuda_stream), "status")
    return int(code.value)


def _mat_layout(t: torch.Tensor) -> tuple[int, int, int]:
    """(mn_major, ld, batch_stride) of a 2-D/3-D tensor whose last two dims are row- or column-major."""
    s1, s2 = t.stride(-2), t.stride(-1)
    bs = t.stride(0) if t.dim() == 3 else 0
    if s2 == 1 or t.size(-1) == 1:
        if t.size(-1) == 1 and s2 != 1:
            return 0, max(s1, 1), bs
        return 0, s1 if t.size(-2) > 1 else max(s1, t.size(-1)), bs
    if s1 == 1:
        return 1, s2 if t.size(-1) > 1 else max(s2, t.size(-2)), bs
    raise NativeLibraryError(f"unsupported strides {t.stride()} for shape {tuple(t.shape)}")


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    c: torch.Tensor | None,
    out: torch.Tensor,
    alpha: float = 1.0,
    beta: float = 0.0,
    post_scale: float = 1.0,
    round_bf16: bool = False,
) -> torch.Tensor:
    """``out = alpha * a @ b + beta * c`` with ``a`` (.., M, K), ``b`` (.., K, N); see ``eo_gemm``.

    ``a`` and ``b`` may be row- or column-major in their last two dims; ``c`` and ``out`` row-major.
    """
    require_cuda(a, "a")
    batch = a.size(0) if a.dim() == 3 else 1
    M, K = a.size(-2), a.size(-1)
    N = b.size(-1)
    assert b.size(-2) == K and out.size(-2) == M and out.size(-1) == N
    precision = 0 if a.dtype == torch.bfloat16 else 1
    # The kernel takes op(B) as N x K: b (K x N row-major) is "MN-major", b column-major is "K-major".
    a_mn, lda, sa = _mat_layout(a)
    bt_mn, ldb, sb = _mat_layout(b.mT)
    if c is not None:
        c_mn, ldc, sc = _mat_layout(c)
        assert c_mn == 0, "c must be row-major"
    else:
        ldc, sc = 0, 0
    d_mn, ldd, sd = _mat_layout(out)
    assert d_mn == 0, "out must be row-major"
    with torch.cuda.device(a.device):
        rc = lib().eo_gemm(
            a.data_ptr(), a_mn, lda, sa,
            b.data_ptr(), bt_mn, ldb, sb,
            c.data_ptr() if c is not None else None, ldc, sc,
            out.data_ptr(), ldd, sd,
            batch, M, N, K,
            alpha, beta, post_scale,
            precision, 1 if out.dtype == torch.float32 else 0, 1 if round_bf16 else 0, _stream(a),
        )  # fmt: skip
    _check(rc, "eo_gemm")
    return out


def syrk(
    a: torch.Tensor,
    c: torch.Tensor | None,
    out: torch.Tensor,
    alpha: float = 1.0,
    beta: float = 0.0,
    skip_upper: bool = False,
) -> torch.Tensor:
    """``out = alpha * a @ a.mT + beta * c`` (lower triangle computed, mirrored); see ``eo_syrk``."""
    require_cuda(a, "a")
    batch = a.size(0) if a.dim() == 3 else 1
    N, K = a.size(-2), a.size(-1)
    precision = 0 if a.dtype == torch.bfloat16 else 1
    a_mn, lda, sa = _mat_layout(a)
    if c is not None:
        # c is symmetric: a column-major c is read as its own transpose.
        _, ldc, sc = _mat_layout(c)
    else:
        ldc, sc = 0, 0
    d_mn, ldd, sd = _mat_layout(out)
    assert d_mn == 0, "out must be row-major"
    with torch.cuda.device(a.device):
        rc = lib().eo_syrk(
            a.data_ptr(), a_mn, lda, sa,
            c.data_ptr() if c is not None else None, ldc, sc,
            out.data_ptr(), ldd, sd,
            batch, N, K, alpha, beta, 1 if skip_upper else 0, precision, _stream(a),
        )  # fmt: skip
    _check(rc, "eo_syrk")
    return out


def sumsq(x: torch.Tensor) -> torch.Tensor:
    """Per-matrix sum of squares of an fp32 (B, M, N) / (M, N) tensor, float64, shape (B,) on the device."""
    require_cuda(x, "x")
    batch = x.size(0) if x.dim() == 3 else 1
    mn, ld, bs = _mat_layout(x)
    rows, cols = (x.size(-2), x.size(-1)) if mn == 0 else (x.size(-1), x.size(-2))
    out = torch.empty(batch, dtype=torch.float64, device=x.device)
    nbytes = lib().eo_sumsq_scratch_bytes(batch, rows, cols)
    scratch = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib().eo_sumsq_f32(
            x.data_ptr(), batch, rows, cols, ld, bs, out.data_ptr(), scratch.data_ptr(), nbytes, _stream(x)
        )
    _check(rc, "eo_sumsq_f32")
    return out


def normalize(
    x: torch.Tensor,
    sumsq_: torch.Tensor,
    eps: float,
    clamp_eps: bool,
    out_dtype: torch.dtype,
    round_bf16: bool = False,
) -> torch.Tensor:
    """``x / max(sqrt(sumsq), eps)`` per matrix, written in ``out_dtype`` with the same layout as ``x``."""
    require_cuda(x, "x")
    batch = x.size(0) if x.dim() == 3 else 1
    mn, ld, bs = _mat_layout(x)
    rows, cols = (x.size(-2), x.size(-1)) if mn == 0 else (x.size(-1), x.size(-2))
    # Output keeps the orientation of the input: dense row-major over the physical (rows, cols).
    shape = (batch, rows, cols) if x.dim() == 3 else (rows, cols)
    out = torch.empty(shape, dtype=out_dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib().eo_normalize_f32(
            x.data_ptr(), batch, rows, cols, ld, bs, sumsq_.data_ptr(), eps, 1 if clamp_eps else 0,
            out.data_ptr(), cols, rows * cols, 1 if out_dtype == torch.float32 else 0, 1 if round_bf16 else 0,
            _stream(x),
        )  # fmt: skip
    _check(rc, "eo_normalize_f32")
    return out.mT if mn == 1 else out
