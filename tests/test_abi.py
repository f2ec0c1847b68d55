"""The C ABI: every function declared in include/eo_b200.h is exported by the built library and bound in
``_native``.  No compute call is made, so this runs without a GPU."""

import ctypes
import os
import re

import pytest

from emerging_optimizers_b200 import _native
from emerging_optimizers_b200 import build as eo_build


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "eo_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(eo_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def library():
    eo_build.build()
    return ctypes.CDLL(_native.library_path())


def test_header_declares_functions():
    names = declared_functions()
    assert "eo_gemm" in names and "eo_syrk" in names and len(names) >= 8


def test_every_declared_function_is_exported(library):
    for name in declared_functions():
        assert hasattr(library, name), f"{name} declared in eo_b200.h but not exported"


def test_binding_covers_header():
    assert sorted(_native.exported_symbols()) == declared_functions()


def test_version_and_error_strings(library):
    library.eo_version.restype = ctypes.c_char_p
    library.eo_last_error.restype = ctypes.c_char_p
    assert library.eo_version().decode().startswith("eo_b200")
    # "" unless an earlier test of this process made a call fail on this thread
    assert isinstance(library.eo_last_error().decode(), str)


def test_scratch_size_query_needs_no_gpu():
    lib = _native.lib()
    assert lib.eo_sumsq_scratch_bytes(0, 10, 10) == 0
    one = lib.eo_sumsq_scratch_bytes(1, 8192, 28672)
    assert one % 8 == 0 and 8 <= one <= 8 * 1024
    assert lib.eo_sumsq_scratch_bytes(5, 8192, 28672) == 5 * one


def test_newton_schulz_workspace_queries_need_no_gpu():
    lib = _native.lib()
    for fn in (lib.eo_newton_schulz_workspace_bytes, lib.eo_newton_schulz_f32_workspace_bytes):
        assert fn(0, 128, 256) == 0 and fn(1, 0, 256) == 0
        assert fn(2, 1024, 4096) >= 2 * fn(1, 1024, 4096) - 4 * 32 * 1024 * 1024  # grows with the batch
        assert fn(1, 1024, 4096) == fn(1, 4096, 1024)  # a tall input is the same problem transposed
    # bf16: A and S (m x m) plus one temporary iterate
    assert lib.eo_newton_schulz_workspace_bytes(1, 1024, 4096) >= 2 * (2 * 1024 * 1024 + 1024 * 4096)
    # fp32: three planes of the iterate and of A / S, fp32 A, S and temporary iterate ...
    base = 3 * 2 * 1024 * 4096 + 2 * 4 * 1024 * 1024 + 3 * 2 * 1024 * 1024 + 4 * 1024 * 4096
    single = lib.eo_newton_schulz_f32_workspace_bytes(1, 1024, 4096)
    assert single % 256 == 0 and single >= base
    # ... and, for a single small matrix only, room for the partial Gram matrices of the K-split (2, 4 or 8)
    assert single - base >= 2 * 4 * 1024 * 1024
    batched = lib.eo_newton_schulz_f32_workspace_bytes(4, 1024, 4096)
    assert batched < 4 * base + 64 * 1024
    big = lib.eo_newton_schulz_f32_workspace_bytes(1, 8192, 28672)
    assert big < 3 * 2 * 8192 * 28672 + 2 * 4 * 8192 * 8192 + 3 * 2 * 8192 * 8192 + 4 * 8192 * 28672 + 64 * 1024


def test_cpu_tensors_are_rejected_loudly():
    import torch

    from emerging_optimizers_b200.orthogonalized_optimizers import muon_utils

    with pytest.raises(_native.NativeLibraryError, match="no CPU path"):
        muon_utils.newton_schulz(torch.randn(8, 16), steps=1)
