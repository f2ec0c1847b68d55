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
    "eo_set_option": (c_int, [c_char_p, c_int]),
    "eo_read_device_status": (c_int, [POINTER(c_uint32), c_void_p]),
    "eo_gemm": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_int64]
        + [c_void_p, c_int, c_int64, c_int64, c_int64]
        + [c_void_p, c_int64, c_int64]
        + [c_void_p, c_int64, c_int64]
        + [c_int, c_int, c_int, c_int]
        + [c_float, c_float, c_float]
        + [c_int, c_int, c_int, c_void_p],
    ),
    "eo_syrk": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_int64]
        + [c_void_p, c_int64, c_int64]
        + [c_void_p, c_int64, c_int64]
        + [c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_void_p],
    ),
    "eo_split_f32": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p],
    ),
    "eo_sumsq_scratch_bytes": (c_size_t, [c_int, c_int64, c_int64]),
    "eo_sumsq_f32": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_size_t, c_void_p],
    ),
    "eo_sumsq_f32_noalloc": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p],
    ),
    "eo_sumsq_noalloc_max_partials": (c_size_t, []),
    "eo_muon_scratch_bytes": (c_size_t, [c_int64]),
    "eo_muon_momentum_f32": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int64, c_double, c_int, c_float, c_void_p, c_void_p, c_size_t, c_void_p],
    ),
    "eo_muon_normalize_bf16": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int64, c_double, c_int, c_float, c_void_p, c_float, c_void_p, c_void_p],
    ),
    "eo_muon_apply_f32": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_float, c_float, c_float, c_float, c_void_p]),
    "eo_muon_prepare_scratch_bytes": (c_size_t, [c_int, c_int64]),
    "eo_muon_prepare_batch": (
        c_int,
        [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_double, c_int, c_float, c_float, c_void_p, c_int64]
        + [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p],
    ),
    "eo_muon_apply_batch": (
        c_int,
        [c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_float, c_int, c_void_p],
    ),
    "eo_newton_schulz_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "eo_newton_schulz_bf16": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_void_p, c_int, c_int]
        + [c_void_p, c_int, c_int64, c_int64, c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    "eo_cast_sumsq_f32": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_float]
        + [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p],
    ),
    "eo_newton_schulz_f32_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "eo_newton_schulz_f32": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_void_p, c_int]
        + [c_void_p, c_int64, c_int64, c_void_p, c_size_t, c_void_p],
    ),
    "eo_tp_gram_inbox_bytes": (c_size_t, [c_int, c_int]),
    "eo_tp_gram_flag_count": (c_size_t, [c_int, c_int]),
    "eo_tp_gram_allreduce": (
        c_int,
        [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        + [c_int64, c_uint32, c_void_p],
    ),
    "eo_gemm_multicast": (
        c_int,
        [c_void_p, c_int, c_int64, c_void_p, c_int, c_int64, c_void_p, c_int64, c_void_p, c_int64]
        + [c_int, c_int, c_int, c_float, c_float, c_void_p],
    ),
    "eo_peek_device_status_async": (c_int, [c_void_p, c_void_p]),
    "eo_debug_pair_schedule": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int64, POINTER(c_int64)]),
    "eo_tp_gram_mirror": (c_int, [c_void_p, c_int, c_int64, c_void_p]),
    "eo_multicast_copy": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "eo_normalize_f32": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p, c_float, c_int]
        + [c_void_p, c_int64, c_int64, c_int, c_int, c_void_p],
    ),
}


# Kernel launches issued through this module since import (what a benchmark reports as its own launches), and an
# optional per-launch timing hook: when `launch_timer` is a list, every tensor-core launch appends
# (name, start_event, end_event, kernels) recorded on the launching stream around the `kernels` back-to-back launches
# of that call.
launch_count = 0
launch_timer: list | None = None


class _Timed:
    """Count the kernels one C call launches and, if asked, bracket it with CUDA events on its stream."""

    def __init__(self, name: str, kernels: int, device: torch.device, timed: bool = False):
        self.name, self.kernels, self.device, self.timed = name, kernels, device, timed

    def __enter__(self) -> None:
        global launch_count
        launch_count += self.kernels
        if self.timed and launch_timer is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record(torch.cuda.current_stream(self.device))

    def __exit__(self, *exc) -> None:
        if self.timed and launch_timer is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record(torch.cuda.current_stream(self.device))
            launch_timer.append((self.name, self.start, end, self.kernels))


class NativeLibraryError(RuntimeError):
    """Raised when ``libeo_b200.so`` is missing or one of its entry points reports a failure."""


def library_path() -> str:
    """Path of the shared library; ``EO_B200_LIB`` overrides the in-tree default (e.g. to compare two builds)."""
    return os.environ.get("EO_B200_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), _LIB_NAME)


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


def set_option(name: str, value: int) -> None:
    """Set a process-wide tuning knob of the library (see ``eo_set_option``), e.g. ``("gemm_tile_m", 256)``."""
    _check(lib().eo_set_option(name.encode(), int(value)), "eo_set_option")


def read_device_status(device: torch.device | None = None) -> int:
    """Synchronise the current stream and return (and clear) the kernels' bounded-wait status word."""
    code = c_uint32(0)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(dev):
        _check(lib().eo_read_device_status(ctypes.byref(code), torch.cuda.current_stream(dev).cuda_stream), "status")
    return int(code.value)


# Late but loud: every Newton-Schulz call leaves an asynchronous copy of the status word in pinned host memory and
# looks at the copy its predecessors left.  A kernel whose bounded wait ran out (its output is then incomplete) thus
# makes one of the next calls on that GPU raise, without any synchronisation on the way.
_STATUS_MIRRORS: dict[int, torch.Tensor] = {}


def raise_on_earlier_failure(device: torch.device) -> None:
    """Raise ``NativeLibraryError`` if a kernel of an earlier call on ``device`` gave up a bounded wait."""
    mirror = _STATUS_MIRRORS.get(device.index if device.index is not None else torch.cuda.current_device())
    if mirror is None:
        return
    code = int(mirror[0])
    if code != 0:
        mirror.zero_()
        read_device_status(device)  # synchronises and clears the device word
        raise NativeLibraryError(
            f"a kernel of an earlier call on {device} gave up a bounded wait (device status {code:#x}); "
            "results computed since then are incomplete"
        )


def note_status(device: torch.device) -> None:
    """Enqueue the asynchronous copy that a later :func:`raise_on_earlier_failure` looks at."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    mirror = _STATUS_MIRRORS.get(index)
    if mirror is None:
        mirror = _STATUS_MIRRORS[index] = torch.zeros(1, dtype=torch.int32).pin_memory()
    peek_device_status_async(mirror, device)


def pair_schedule(M: int, N: int, K: int, tri: bool, batch: int = 1, sm_count: int = 148):
    """Work items of the CTA-pair kernel for a product of ``batch`` matrices M x N x K as an int32 array of rows
    ``(matrix, tile row, tile column, first k-block, end k-block, split slot or -1)``; host only, no GPU needed (see
    ``eo_debug_pair_schedule``)."""
    import numpy as np

    n = c_int64(0)
    _check(lib().eo_debug_pair_schedule(M, N, K, int(tri), batch, sm_count, None, 0, ctypes.byref(n)), "schedule")
    out = np.zeros((n.value, 6), dtype=np.int32)
    _check(
        lib().eo_debug_pair_schedule(M, N, K, int(tri), batch, sm_count, out.ctypes.data, n.value, ctypes.byref(n)),
        "schedule",
    )
    return out


def _mat_layout(t: torch.Tensor) -> tuple[int, int, int]:
    """(mn_major, ld, batch_stride) of a 2-D/3-D tensor whose last two dims are row- or column-major.

    ``mn_major == 0``: the last dim is contiguous (row-major, ``ld`` = row stride);
    ``mn_major == 1``: the second-to-last dim is contiguous (a transposed view, ``ld`` = column stride).
    """
    rows, cols = t.size(-2), t.size(-1)
    s1, s2 = t.stride(-2), t.stride(-1)
    bs = t.stride(0) if t.dim() == 3 else 0
    if (s2 == 1 or cols == 1) and (s1 >= cols or rows == 1):
        return 0, (s1 if rows > 1 else cols), bs
    if (s1 == 1 or rows == 1) and (s2 >= rows or cols == 1):
        return 1, (s2 if cols > 1 else rows), bs
    raise NativeLibraryError(f"unsupported strides {t.stride()} for shape {tuple(t.shape)}")


def is_matrix_layout(t: torch.Tensor) -> bool:
    """True when the last two dims of ``t`` are row- or column-major (what the kernels can address)."""
    try:
        _mat_layout(t)
    except NativeLibraryError:
        return False
    return True


class Split3:
    """An fp32 matrix (batch) stored as three bf16 planes whose sum reproduces it to about 2^-24 relative.

    ``planes`` has shape (3, [B,] R, C) in the physical (row-major) orientation of the source; ``mn`` records
    whether the logical matrix is the transpose of that storage.  See ``eo_split_f32``.
    """

    def __init__(self, x: torch.Tensor):
        require_cuda(x, "x")
        assert x.dtype == torch.float32
        mn, ld, bs = _mat_layout(x)
        rows, cols = (x.size(-2), x.size(-1)) if mn == 0 else (x.size(-1), x.size(-2))
        batch = x.size(0) if x.dim() == 3 else 1
        ldo = (cols + 7) // 8 * 8
        mat = rows * ldo
        self.planes = torch.empty((3, batch, mat), dtype=torch.bfloat16, device=x.device)
        self.mn, self.ld, self.bstride, self.plane_stride = mn, ldo, mat, batch * mat
        self.shape, self.batch, self.device = tuple(x.shape), batch, x.device
        with torch.cuda.device(x.device), _Timed("split", 1, x.device):
            rc = lib().eo_split_f32(
                x.data_ptr(), batch, rows, cols, ld, bs, self.planes.data_ptr(), ldo, mat, self.plane_stride, _stream(x)
            )
        _check(rc, "eo_split_f32")

    @property
    def mT(self) -> "Split3":
        """The transposed matrix: same planes, opposite orientation flag."""
        t = object.__new__(Split3)
        t.__dict__.update(self.__dict__)
        t.mn = 1 - self.mn
        t.shape = (*self.shape[:-2], self.shape[-1], self.shape[-2])
        return t

    def data_ptr(self) -> int:
        return self.planes.data_ptr()

    def size(self, d: int) -> int:
        return self.shape[d]

    def dim(self) -> int:
        return len(self.shape)


def _operand(t: "torch.Tensor | Split3") -> tuple[int, int, int, int, int]:
    """(pointer, mn_major, ld, batch_stride, plane_stride) of a bf16 tensor or a split fp32 operand."""
    if isinstance(t, Split3):
        return t.data_ptr(), t.mn, t.ld, t.bstride, t.plane_stride
    mn, ld, bs = _mat_layout(t)
    return t.data_ptr(), mn, ld, bs, 0


def gemm(
    a: "torch.Tensor | Split3",
    b: "torch.Tensor | Split3",
    c: torch.Tensor | None,
    out: torch.Tensor,
    alpha: float = 1.0,
    beta: float = 0.0,
    post_scale: float = 1.0,
    round_bf16: bool = False,
) -> torch.Tensor:
    """``out = alpha * a @ b + beta * c`` with ``a`` (.., M, K), ``b`` (.., K, N); see ``eo_gemm``.

    bf16 tensors run the plain bf16 product; :class:`Split3` operands (both) run the fp32-accurate product with
    fp32 ``c`` / ``out``.  ``a`` and ``b`` may be row- or column-major; ``c`` and ``out`` row-major.
    """
    batch = a.size(0) if a.dim() == 3 else 1
    M, K = a.size(-2), a.size(-1)
    N = b.size(-1)
    assert b.size(-2) == K and out.size(-2) == M and out.size(-1) == N
    split = isinstance(a, Split3)
    assert split == isinstance(b, Split3), "both operands must be split, or neither"
    if not split:
        require_cuda(a, "a")
        assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    # The kernel takes op(B) as N x K: b (K x N row-major) is "MN-major", b column-major is "K-major".
    pa, a_mn, lda, sa, pla = _operand(a)
    pb, bt_mn, ldb, sb, plb = _operand(b.mT)
    if c is not None:
        c_mn, ldc, sc = _mat_layout(c)
        assert c_mn == 0, "c must be row-major"
        assert c.dtype == (torch.float32 if split else torch.bfloat16)
    else:
        ldc, sc = 0, 0
    d_mn, ldd, sd = _mat_layout(out)
    assert d_mn == 0, "out must be row-major"
    with torch.cuda.device(out.device), _Timed("gemm", 1, out.device, timed=True):
        rc = lib().eo_gemm(
            pa, a_mn, lda, sa, pla,
            pb, bt_mn, ldb, sb, plb,
            c.data_ptr() if c is not None else None, ldc, sc,
            out.data_ptr(), ldd, sd,
            batch, M, N, K,
            alpha, beta, post_scale,
            1 if split else 0, 1 if out.dtype == torch.float32 else 0, 1 if round_bf16 else 0, _stream(out),
        )  # fmt: skip
    _check(rc, "eo_gemm")
    return out


def syrk(
    a: "torch.Tensor | Split3",
    c: torch.Tensor | None,
    out: torch.Tensor,
    alpha: float = 1.0,
    beta: float = 0.0,
    skip_upper: bool = False,
) -> torch.Tensor:
    """``out = alpha * a @ a.mT + beta * c`` (lower triangle computed, mirrored); see ``eo_syrk``."""
    split = isinstance(a, Split3)
    if not split:
        require_cuda(a, "a")
    batch = a.size(0) if a.dim() == 3 else 1
    N, K = a.size(-2), a.size(-1)
    pa, a_mn, lda, sa, pla = _operand(a)
    if c is not None:
        # c is symmetric: a column-major c is read as its own transpose.
        _, ldc, sc = _mat_layout(c)
    else:
        ldc, sc = 0, 0
    d_mn, ldd, sd = _mat_layout(out)
    assert d_mn == 0, "out must be row-major"
    assert out.dtype == (torch.float32 if split else torch.bfloat16)
    with torch.cuda.device(out.device), _Timed("syrk", 1, out.device, timed=True):
        rc = lib().eo_syrk(
            pa, a_mn, lda, sa, pla,
            c.data_ptr() if c is not None else None, ldc, sc,
            out.data_ptr(), ldd, sd,
            batch, N, K, alpha, beta, 1 if skip_upper else 0, 1 if split else 0, _stream(out),
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
    with torch.cuda.device(x.device), _Timed("sumsq", 2, x.device):
        rc = lib().eo_sumsq_f32(
            x.data_ptr(), batch, rows, cols, ld, bs, out.data_ptr(), scratch.data_ptr(), nbytes, _stream(x)
        )
    _check(rc, "eo_sumsq_f32")
    return out


def sumsq_noalloc(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """:func:`sumsq` into a caller-provided float64 ``out`` through ``eo_sumsq_f32_noalloc``: the partial sums go
    to a fixed array inside the library, so nothing is allocated on the way (neither here nor in the library).

    Meant for callers that must not allocate device memory (allocator hooks, fixed-footprint loops, hosts that
    only hold raw device pointers).  Raises for requests beyond the built-in capacity.  Calls that may overlap on
    one GPU must be serialised by the caller: they share the array.
    """
    require_cuda(x, "x")
    batch = x.size(0) if x.dim() == 3 else 1
    assert out.dtype == torch.float64 and out.numel() == batch and out.is_contiguous() and out.device == x.device
    mn, ld, bs = _mat_layout(x)
    rows, cols = (x.size(-2), x.size(-1)) if mn == 0 else (x.size(-1), x.size(-2))
    with torch.cuda.device(x.device), _Timed("sumsq", 2, x.device):
        rc = lib().eo_sumsq_f32_noalloc(x.data_ptr(), batch, rows, cols, ld, bs, out.data_ptr(), _stream(x))
    _check(rc, "eo_sumsq_f32_noalloc")
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
    with torch.cuda.device(x.device), _Timed("normalize", 1, x.device):
        rc = lib().eo_normalize_f32(
            x.data_ptr(), batch, rows, cols, ld, bs, sumsq_.data_ptr(), eps, 1 if clamp_eps else 0,
            out.data_ptr(), cols, rows * cols, 1 if out_dtype == torch.float32 else 0, 1 if round_bf16 else 0,
            _stream(x),
        )  # fmt: skip
    _check(rc, "eo_normalize_f32")
    return out.mT if mn == 1 else out


def muon_momentum(
    g: torch.Tensor, m: torch.Tensor, p: torch.Tensor | None, momentum: float, nesterov: bool, l2: float
) -> torch.Tensor:
    """Update the momentum buffer ``m`` in place and return the float64 sum of squares (shape (1,)) of the tensor
    that will be orthogonalized; see ``eo_muon_momentum_f32``.  All tensors flat-contiguous fp32."""
    require_cuda(g, "g")
    numel = g.numel()
    out = torch.empty(1, dtype=torch.float64, device=g.device)
    nbytes = lib().eo_muon_scratch_bytes(numel)
    scratch = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=g.device)
    with torch.cuda.device(g.device), _Timed("muon_momentum", 2, g.device):
        rc = lib().eo_muon_momentum_f32(
            g.data_ptr(), m.data_ptr(), p.data_ptr() if (p is not None and l2 != 0.0) else None, numel,
            momentum, 1 if nesterov else 0, l2, out.data_ptr(), scratch.data_ptr(), nbytes, _stream(g),
        )  # fmt: skip
    _check(rc, "eo_muon_momentum_f32")
    return out


def muon_normalize(
    g: torch.Tensor, m: torch.Tensor, p: torch.Tensor | None, momentum: float, nesterov: bool, l2: float,
    sumsq_: torch.Tensor, eps: float, out: torch.Tensor,
) -> torch.Tensor:  # fmt: skip
    """Write the normalised, bf16-rounded tensor to orthogonalize into ``out`` (contiguous bf16, same numel)."""
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.numel() == g.numel()
    with torch.cuda.device(g.device), _Timed("muon_normalize", 1, g.device):
        rc = lib().eo_muon_normalize_bf16(
            g.data_ptr(), m.data_ptr(), p.data_ptr() if (p is not None and l2 != 0.0) else None, g.numel(),
            momentum, 1 if nesterov else 0, l2, sumsq_.data_ptr(), eps, out.data_ptr(), _stream(g),
        )  # fmt: skip
    _check(rc, "eo_muon_normalize_bf16")
    return out


def muon_apply(p: torch.Tensor, update: torch.Tensor, shrink: float, scale: float, extra: float, lr: float) -> None:
    """``p <- (p + shrink * p) - lr * ((update * scale) * extra)`` in place; ``update`` bf16 or fp32, contiguous."""
    require_cuda(p, "p")
    assert p.is_contiguous() and update.is_contiguous() and p.numel() == update.numel() and p.dtype == torch.float32
    assert update.dtype in (torch.bfloat16, torch.float32)
    with torch.cuda.device(p.device), _Timed("muon_apply", 1, p.device):
        rc = lib().eo_muon_apply_f32(
            p.data_ptr(), update.data_ptr(), 1 if update.dtype == torch.bfloat16 else 0, p.numel(),
            shrink, scale, extra, lr, _stream(p),
        )  # fmt: skip
    _check(rc, "eo_muon_apply_f32")


def _ptr_array(tensors) -> "ctypes.Array":
    arr = (c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr() if t is not None else None
    return arr


def muon_prepare_batch(
    grads, momenta, params, momentum: float, nesterov: bool, l2: float, eps: float, out_stack: torch.Tensor,
    scales: torch.Tensor | None = None,
) -> torch.Tensor:  # fmt: skip
    """Momentum update of ``n`` equally sized flat-contiguous fp32 tensors and their normalised bf16 images written
    to ``out_stack[i]``; returns the float64 sums of squares (n,).  With ``scales`` (fp32, shape (n, 2)) the division
    is deferred: ``out_stack[i]`` receives the un-normalised update and ``scales[i]`` the factors that
    :func:`newton_schulz_bf16` applies.  See ``eo_muon_prepare_batch``."""
    n = len(grads)
    dev = grads[0].device
    numel = grads[0].numel()
    assert out_stack.dtype == torch.bfloat16 and out_stack.is_contiguous() and out_stack.size(0) == n
    slot_stride = out_stack[0].numel()
    assert slot_stride >= numel and slot_stride % 8 == 0
    if scales is not None:
        assert scales.dtype == torch.float32 and scales.is_contiguous() and scales.numel() == 2 * n
    ss = torch.empty(n, dtype=torch.float64, device=dev)
    nbytes = lib().eo_muon_prepare_scratch_bytes(n, numel)
    scratch = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=dev)
    launches = (2 if scales is not None else 3) * ((n + 47) // 48)
    with torch.cuda.device(dev), _Timed("muon_prepare", launches, dev):
        rc = lib().eo_muon_prepare_batch(
            n, _ptr_array(grads), _ptr_array(momenta), _ptr_array(params) if l2 != 0.0 else None, numel,
            momentum, 1 if nesterov else 0, l2, eps, out_stack.data_ptr(), slot_stride,
            ss.data_ptr(), scales.data_ptr() if scales is not None else None, scratch.data_ptr(), nbytes,
            torch.cuda.current_stream(dev).cuda_stream,
        )  # fmt: skip
    _check(rc, "eo_muon_prepare_batch")
    return ss


def muon_apply_batch(
    params, updates, scales, shrink: float, extra: float, lr: float, max_blocks_per_tensor: int = 0
) -> None:
    """Fused weight update of a list of contiguous fp32 parameters; ``updates`` all bf16 or all fp32."""
    n = len(params)
    if n == 0:
        return
    dev = params[0].device
    is_bf16 = updates[0].dtype == torch.bfloat16
    numel = (c_int64 * n)(*[p.numel() for p in params])
    sc = (c_float * n)(*scales)
    with torch.cuda.device(dev), _Timed("muon_apply", (n + 47) // 48, dev):
        rc = lib().eo_muon_apply_batch(
            n, _ptr_array(params), _ptr_array(updates), 1 if is_bf16 else 0, numel, sc, shrink, extra, lr,
            max_blocks_per_tensor, torch.cuda.current_stream(dev).cuda_stream,
        )  # fmt: skip
    _check(rc, "eo_muon_apply_batch")


# Set to False to keep small matrices (rows <= 128) on the general kernels (comparison runs).
FUSED_SMALL_MATRICES = True


def cast_sumsq(x: torch.Tensor, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    """One pass over a row-major fp32 ``x`` ((B,) rows, cols): its bf16 image (un-normalised, dense) and the
    per-matrix factors ``[1 / norm^2, 1 / norm]`` (fp32, shape (B, 2)) that :func:`newton_schulz_bf16` applies in
    its first two epilogues instead of a normalisation pass.  See ``eo_cast_sumsq_f32``."""
    require_cuda(x, "x")
    assert x.dtype == torch.float32
    batch = x.size(0) if x.dim() == 3 else 1
    mn, ld, bs = _mat_layout(x)
    assert mn == 0, "x must be row-major"
    rows, cols = x.size(-2), x.size(-1)
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    scales = torch.empty((batch, 2), dtype=torch.float32, device=x.device)
    nbytes = lib().eo_sumsq_scratch_bytes(batch, rows, cols)
    scratch = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device), _Timed("cast_sumsq", 2, x.device):
        rc = lib().eo_cast_sumsq_f32(
            x.data_ptr(), batch, rows, cols, ld, bs if x.dim() == 3 else rows * ld, out.data_ptr(), cols, rows * cols,
            eps, None, scales.data_ptr(), scratch.data_ptr(), nbytes, _stream(x),
        )  # fmt: skip
    _check(rc, "eo_cast_sumsq_f32")
    return out, scales


def newton_schulz_bf16(
    x: torch.Tensor, schedule, use_syrk: bool, out_dtype: torch.dtype = torch.bfloat16,
    scales: torch.Tensor | None = None,
) -> torch.Tensor:  # fmt: skip
    """Run the whole iteration loop on a bf16 iterate ``x`` ((B,) rows, cols, row-major, 16-byte aligned rows) with
    one library call; ``x`` is clobbered.  ``x`` is the normalised input, or, with ``scales`` from
    :func:`cast_sumsq`, its un-normalised image.  Returns a new contiguous tensor of ``out_dtype``."""
    require_cuda(x, "x")
    assert x.dtype == torch.bfloat16 and len(schedule) >= 1
    batch = x.size(0) if x.dim() == 3 else 1
    rows, cols = x.size(-2), x.size(-1)
    mn, ld, bs = _mat_layout(x)
    assert mn == 0, "x must be row-major"
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    nbytes = lib().eo_newton_schulz_workspace_bytes(batch, rows, cols)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    abc = (c_float * (3 * len(schedule)))(*[v for t in schedule for v in t])
    # Launch count as the library decides it: one persistent kernel for stacks of small wide matrices, else two or
    # three tensor-core launches per iteration.
    if FUSED_SMALL_MATRICES and rows <= 128 and rows <= cols and cols >= 256 and len(schedule) <= 16:
        kernels = 1
    else:
        kernels = sum(3 if t[2] != 0.0 else 2 for t in schedule)
    raise_on_earlier_failure(x.device)
    with torch.cuda.device(x.device), _Timed("newton_schulz", kernels, x.device, timed=True):
        rc = lib().eo_newton_schulz_bf16(
            x.data_ptr(), batch, rows, cols, ld, bs if x.dim() == 3 else rows * ld, abc, len(schedule),
            (1 if use_syrk else 0) | (0 if FUSED_SMALL_MATRICES else 2),
            out.data_ptr(), 1 if out_dtype == torch.float32 else 0, cols, rows * cols,
            ws.data_ptr(), nbytes, scales.data_ptr() if scales is not None else None, _stream(x),
        )  # fmt: skip
    _check(rc, "eo_newton_schulz_bf16")
    note_status(x.device)
    return out


def newton_schulz_f32(x: torch.Tensor, schedule) -> torch.Tensor:
    """Run the whole iteration loop of the fp32 path on a normalised fp32 iterate ``x`` ((B,) rows, cols,
    row-major) with one library call (see ``eo_newton_schulz_f32``).  Returns a new contiguous fp32 tensor."""
    require_cuda(x, "x")
    assert x.dtype == torch.float32 and len(schedule) >= 1
    batch = x.size(0) if x.dim() == 3 else 1
    rows, cols = x.size(-2), x.size(-1)
    mn, ld, bs = _mat_layout(x)
    assert mn == 0, "x must be row-major"
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    nbytes = lib().eo_newton_schulz_f32_workspace_bytes(batch, rows, cols)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    abc = (c_float * (3 * len(schedule)))(*[v for t in schedule for v in t])
    kernels = sum(6 if t[2] != 0.0 else 4 for t in schedule)
    raise_on_earlier_failure(x.device)
    with torch.cuda.device(x.device), _Timed("newton_schulz", kernels, x.device, timed=True):
        rc = lib().eo_newton_schulz_f32(
            x.data_ptr(), batch, rows, cols, ld, bs if x.dim() == 3 else rows * ld, abc, len(schedule),
            out.data_ptr(), cols, rows * cols, ws.data_ptr(), nbytes, _stream(x),
        )  # fmt: skip
    _check(rc, "eo_newton_schulz_f32")
    note_status(x.device)
    return out


def tp_gram_allreduce(
    x: torch.Tensor, world: int, rank: int, partial_ptrs, flag_ptrs, gram_ptrs, partials_mc: int, gram_mc: int,
    ld_gram: int, seq: int,
) -> None:  # fmt: skip
    """Launch the fused tensor-parallel Gram exchange for this rank's bf16 shard ``x`` (see ``eo_tp_gram_allreduce``).

    ``partials_mc`` / ``gram_mc`` are the multicast addresses of the partial-tile buffers and Gram matrices, or 0.
    """
    require_cuda(x, "x")
    assert x.dtype == torch.bfloat16 and x.dim() == 2
    mn, ld, _ = _mat_layout(x)

    def arr(ptrs):
        a = (c_void_p * world)()
        for i, p in enumerate(ptrs):
            a[i] = p
        return a

    with torch.cuda.device(x.device), _Timed("tp_gram", 1, x.device, timed=True):
        rc = lib().eo_tp_gram_allreduce(
            x.data_ptr(), mn, ld, x.size(0), x.size(1), world, rank, arr(partial_ptrs), arr(flag_ptrs), arr(gram_ptrs),
            partials_mc or None, gram_mc or None, ld_gram, seq, _stream(x),
        )  # fmt: skip
    _check(rc, "eo_tp_gram_allreduce")


def gemm_multicast(
    a: torch.Tensor, b: torch.Tensor, c: torch.Tensor | None, out_local: torch.Tensor, out_mc_ptr: int,
    alpha: float = 1.0, beta: float = 0.0,
) -> None:  # fmt: skip
    """``alpha * a @ b + beta * c`` stored through the multicast address ``out_mc_ptr`` (see ``eo_gemm_multicast``).

    ``out_local`` is this rank's view of the destination (row-major, same shape as the product); it only supplies
    the layout, the stores go to ``out_mc_ptr`` and so to the same place in every rank's buffer.
    """
    require_cuda(a, "a")
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    M, K = a.shape
    N = b.size(1)
    assert b.size(0) == K and tuple(out_local.shape) == (M, N)
    pa, a_mn, lda, _, _ = _operand(a)
    pb, bt_mn, ldb, _, _ = _operand(b.mT)
    ldc = 0
    if c is not None:
        c_mn, ldc, _ = _mat_layout(c)
        assert c_mn == 0 and c.dtype == torch.bfloat16
    d_mn, ldd, _ = _mat_layout(out_local)
    assert d_mn == 0 and out_local.dtype == torch.bfloat16
    with torch.cuda.device(a.device), _Timed("gemm", 1, a.device, timed=True):
        rc = lib().eo_gemm_multicast(
            pa, a_mn, lda, pb, bt_mn, ldb, c.data_ptr() if c is not None else None, ldc, out_mc_ptr, ldd,
            M, N, K, alpha, beta, _stream(a),
        )  # fmt: skip
    _check(rc, "eo_gemm_multicast")


def tp_gram_mirror(gram: torch.Tensor, n: int, ld: int) -> None:
    """Copy the lower triangle of the local ``n x n`` bf16 Gram buffer onto its upper triangle."""
    with torch.cuda.device(gram.device), _Timed("tp_mirror", 1, gram.device):
        rc = lib().eo_tp_gram_mirror(gram.data_ptr(), n, ld, _stream(gram))
    _check(rc, "eo_tp_gram_mirror")


def multicast_copy(src: torch.Tensor, dst_mc_ptr: int) -> None:
    """Store the contiguous tensor ``src`` through the multicast address ``dst_mc_ptr`` (see ``eo_multicast_copy``)."""
    require_cuda(src, "src")
    assert src.is_contiguous()
    with torch.cuda.device(src.device), _Timed("multicast_copy", 1, src.device):
        rc = lib().eo_multicast_copy(src.data_ptr(), dst_mc_ptr, src.numel() * src.element_size(), _stream(src))
    _check(rc, "eo_multicast_copy")


def peek_device_status_async(pinned: torch.Tensor, device: torch.device) -> None:
    """Enqueue a copy of the kernels' status word into the pinned int32 tensor ``pinned`` (no synchronisation)."""
    assert pinned.is_pinned() and pinned.dtype == torch.int32 and pinned.numel() >= 1
    with torch.cuda.device(device):
        rc = lib().eo_peek_device_status_async(pinned.data_ptr(), torch.cuda.current_stream(device).cuda_stream)
    _check(rc, "eo_peek_device_status_async")
