"""Host-side behaviour that needs no GPU: argument validation (same exception types and messages as the
reference), coefficient schedules, registry, optimizer plumbing around the orthogonalization call."""

import json
import os

import pytest
import torch

from emerging_optimizers_b200 import mixin, registry
from emerging_optimizers_b200 import triton_kernels as tk
from emerging_optimizers_b200.orthogonalized_optimizers import Muon, OrthogonalizedOptimizer, muon_utils
from emerging_optimizers_b200.orthogonalized_optimizers.muon import get_muon_scale_factor
from emerging_optimizers_b200.utils import fp32_matmul_precision, get_pg_rank, get_pg_size


def test_public_names_of_muon_utils():
    assert muon_utils.__all__ == ["newton_schulz", "newton_schulz_tp", "NSCoeffT", "get_coefficient_iterator", "CoeffIterMode"]
    for name in (
        "newton_schulz_step", "batched_newton_schulz_step", "newton_schulz_step_tsyrk",
        "batched_newton_schulz_step_tsyrk", "distributed_normalize_p2", "_COEFFICIENT_SETS",
    ):  # fmt: skip
        assert hasattr(muon_utils, name)


def test_coefficient_tables_match_reference(golden_dir):
    with open(os.path.join(golden_dir, "tables.json")) as f:
        tables = json.load(f)
    assert set(tables["schedules"]) == set(muon_utils._COEFFICIENT_SETS)
    for name, rec in tables["schedules"].items():
        got = list(muon_utils.get_coefficient_iterator(12, muon_utils._COEFFICIENT_SETS[name], rec["mode"]))
        assert [list(t) for t in got] == rec["steps12"]
    for key, val in tables["scale_factors"].items():
        mode, dims = key.split(":")
        m, n = (int(v) for v in dims.split("x"))
        assert get_muon_scale_factor(m, n, mode) == pytest.approx(val, rel=1e-15)
    with pytest.raises(ValueError, match="Invalid mode for Muon update scale factor"):
        get_muon_scale_factor(2, 2, "nope")


def test_coefficient_iterator_errors():
    with pytest.raises(ValueError, match="coefficient_sets must be non-empty"):
        muon_utils.get_coefficient_iterator(3, [])
    with pytest.raises(ValueError, match="Invalid mode"):
        muon_utils.get_coefficient_iterator(3, [(1.0, 2.0, 3.0)], mode="bounce")
    assert list(muon_utils.get_coefficient_iterator(0, [(1.0, 2.0, 3.0)])) == []


def test_newton_schulz_argument_errors():
    with pytest.raises(TypeError, match="must be 2d or 3d"):
        muon_utils.newton_schulz(torch.randn(8), steps=1)
    with pytest.raises(TypeError, match="must be 2d or 3d"):
        muon_utils.newton_schulz(torch.randn(2, 2, 2, 2), steps=1)
    with pytest.raises(TypeError, match="must be in float32, got torch.bfloat16"):
        muon_utils.newton_schulz(torch.randn(4, 4).bfloat16(), steps=1)
    with pytest.raises(ValueError, match="custom_coefficient_sets must be provided"):
        muon_utils.newton_schulz(torch.randn(4, 4), steps=1, coefficient_type="custom")
    with pytest.raises(ValueError, match="Invalid coefficient type: nope"):
        muon_utils.newton_schulz(torch.randn(4, 4), steps=1, coefficient_type="nope")
    with pytest.raises(ValueError, match="cubic5 is a fixed 5-step schedule; got steps=3"):
        muon_utils.newton_schulz(torch.randn(4, 4), steps=3, coefficient_type="cubic5")


def test_newton_schulz_tp_argument_errors(monkeypatch):
    seen = {}

    def fake_ns(x, *args, **kwargs):
        seen.update(kwargs)
        seen["args"] = args
        return x

    monkeypatch.setattr(muon_utils, "newton_schulz", fake_ns)
    x = torch.randn(4, 8)
    # no partition: plain call, use_syrk forwarded as a keyword
    assert muon_utils.newton_schulz_tp(x, 3, "simple", tp_group=None, use_syrk=True) is x
    assert seen["use_syrk"] is True and seen["args"] == (3, "simple")
    with pytest.raises(ValueError, match="Invalid partition_dim: 2"):
        muon_utils.newton_schulz_tp(x, 3, "simple", tp_group=None, partition_dim=2, tp_mode="distributed")
    with pytest.raises(ValueError, match="Invalid tp_mode: ring"):
        muon_utils.newton_schulz_tp(x, 3, "simple", tp_group=None, partition_dim=1, tp_mode="ring")
    muon_utils.newton_schulz_tp(x, 3, "simple", tp_group="G", partition_dim=0, tp_mode="distributed", use_syrk=True)
    assert seen["transpose"] is True and seen["tp_group"] == "G" and seen["use_syrk"] is True
    muon_utils.newton_schulz_tp(x, 3, "simple", tp_group="G", partition_dim=1, tp_mode="distributed")
    assert seen["transpose"] is False and seen["use_syrk"] is False


def test_syrk_argument_errors():
    bf = torch.bfloat16
    with pytest.raises(TypeError, match="must be bfloat16"):
        tk.tsyrk_ex(torch.zeros(8, 8))
    with pytest.raises(TypeError, match="must be 2D"):
        tk.tsyrk_ex(torch.zeros(2, 8, 8, dtype=bf))
    with pytest.raises(TypeError, match="must be contiguous"):
        tk.tsyrk_ex(torch.zeros(8, 16, dtype=bf)[:, ::2])
    with pytest.raises(RuntimeError, match=r"c must be of shape \(N, N\)"):
        tk.tsyrk_ex(torch.zeros(8, 8, dtype=bf), torch.zeros(8, 4, dtype=bf), beta=1.0)
    with pytest.raises(RuntimeError, match=r"c must be of shape \(N, N\)"):
        tk.tsyrk_ex(torch.zeros(8, 8, dtype=bf), None, beta=1.0)
    with pytest.raises(RuntimeError, match="c or c.T must be contiguous"):
        tk.tsyrk_ex(torch.zeros(8, 8, dtype=bf), torch.zeros(8, 16, dtype=bf)[:, ::2], beta=1.0)
    with pytest.raises(RuntimeError, match="out must be same shape/device/dtype"):
        tk.tsyrk_ex_small_matrix(torch.zeros(8, 8, dtype=bf), out=torch.zeros(8, 4, dtype=bf))
    with pytest.raises(RuntimeError, match="out must be contiguous"):
        tk.tsyrk_ex_small_matrix(torch.zeros(8, 8, dtype=bf), out=torch.zeros(8, 16, dtype=bf)[:, ::2])
    # batched
    with pytest.raises(TypeError, match="must be bfloat16"):
        tk.batched_tsyrk_ex(torch.zeros(2, 8, 8))
    with pytest.raises(TypeError, match="must be 3D"):
        tk.batched_tsyrk_ex(torch.zeros(8, 8, dtype=bf))
    with pytest.raises(TypeError, match="must be contiguous"):
        tk.batched_tsyrk_ex(torch.zeros(2, 8, 16, dtype=bf)[:, :, ::2])
    with pytest.raises(RuntimeError, match="must be multiples of 8"):
        tk.batched_tsyrk_ex(torch.zeros(2, 12, 8, dtype=bf))
    with pytest.raises(RuntimeError, match=r"c must be of shape \(B, N, N\)"):
        tk.batched_tsyrk_ex(torch.zeros(2, 8, 8, dtype=bf), torch.zeros(2, 8, 4, dtype=bf), beta=1.0)
    with pytest.raises(RuntimeError, match="c or c.mT must be contiguous"):
        tk.batched_tsyrk_ex(torch.zeros(2, 8, 8, dtype=bf), torch.zeros(2, 8, 16, dtype=bf)[:, :, ::2], beta=1.0)
    with pytest.raises(RuntimeError, match="out must be same shape/device/dtype"):
        tk.batched_tsyrk_ex(torch.zeros(2, 8, 8, dtype=bf), out=torch.zeros(2, 8, 4, dtype=bf))
    with pytest.raises(RuntimeError, match="out must be contiguous"):
        tk.batched_tsyrk_ex(torch.zeros(2, 8, 8, dtype=bf), out=torch.zeros(2, 8, 16, dtype=bf)[:, :, ::2])


def test_can_use_batched_tsyrk_truth_table():
    bf = torch.bfloat16
    assert tk.HAS_TRITON_340
    # CPU tensors can never take the kernel
    assert not tk.can_use_batched_tsyrk(torch.zeros(2, 8, 8, dtype=bf))
    assert not tk.can_use_batched_tsyrk(torch.zeros(8, 8, dtype=bf))


def test_registry_and_muon_constructor():
    assert registry.get_optimizer_cls("muon") is Muon and registry.get_optimizer_cls("MUON") is Muon
    assert "muon" in registry.get_optimizer_name_list()
    with pytest.raises(ValueError, match="not found in the registry"):
        registry.get_optimizer_cls("adamw")
    with pytest.raises(TypeError, match="does not accept arguments"):
        registry.get_configured_optimizer_cls("muon", not_an_arg=1)
    p = torch.nn.Parameter(torch.randn(8, 8))
    opt = registry.get_configured_optimizer_cls("muon", lr=0.1, num_ns_steps=3)([p])
    assert opt.num_ns_steps == 3 and opt.coefficient_type == "quintic" and opt.scale_mode == "spectral"
    assert opt.extra_scale_factor == 1.0 and opt.use_syrk is False
    for attr in ("num_ns_steps", "coefficient_type", "scale_mode", "extra_scale_factor", "use_syrk"):
        with pytest.raises(AttributeError, match=f"Cannot set `{attr}` post-initialization."):
            setattr(opt, attr, 1)
    with pytest.raises(ValueError, match="num_ns_steps must be at least 1, got 0"):
        Muon([p], num_ns_steps=0)
    # no CUDA device here or an unsupported one: use_syrk is switched off, not an error
    if not torch.cuda.is_available():
        assert Muon([p], use_syrk=True).use_syrk is False


class _Identity(OrthogonalizedOptimizer):
    def __init__(self, params, **kw):
        kw.setdefault("nesterov", False)
        kw.setdefault("weight_decay_method", "l2")
        kw.setdefault("fp32_matmul_prec", "highest")
        super().__init__(params, kw.pop("lr", 0.1), kw.pop("momentum", 0.0), kw.pop("weight_decay", 0.0), **kw)


@pytest.mark.parametrize("wd", [0.0, 0.1])
def test_identity_orthogonalizer_equals_sgd(wd):
    """With no orthogonalization and momentum 0 the step is plain SGD with L2 decay, bit for bit (the reference
    pins the same property, tests/test_orthogonalized_optimizer.py:63-144 there)."""
    torch.manual_seed(0)
    w = torch.randn(6, 10)
    g = [torch.randn(6, 10) for _ in range(3)]
    p1, p2 = torch.nn.Parameter(w.clone()), torch.nn.Parameter(w.clone())
    ours = _Identity([p1], lr=0.05, weight_decay=wd, scaled_orthogonalize_fn=torch.nn.Identity())
    sgd = torch.optim.SGD([p2], lr=0.05, momentum=0.0, weight_decay=wd)
    for gi in g:
        p1.grad, p2.grad = gi.clone(), gi.clone()
        ours.step()
        sgd.step()
        assert torch.equal(p1, p2)
    assert set(ours.state[p1]) == {"momentum_buffer"}


def test_step_order_hooks_and_errors():
    events = []

    class Hook:
        def pre_weight_update_inplace(self, p, update):
            events.append("hook_pre")
            return torch.tensor(7.0)

        def post_weight_update_inplace(self, p, state):
            events.append(("hook_post", float(state)))

    class Opt(_Identity):
        def pre_weight_update_fn_inplace(self, p, update):
            events.append("pre")

        def post_weight_update_fn_inplace(self, p):
            events.append("post")

        def orthogonalize(self, p, grad, **kwargs):
            events.append(("orth", torch.get_float32_matmul_precision(), sorted(kwargs)))
            return super().orthogonalize(p, grad, **kwargs)

    p = torch.nn.Parameter(torch.ones(2, 3))
    q = torch.nn.Parameter(torch.ones(2, 3))  # no grad: skipped, no state
    opt = Opt([p, q], lr=0.5, momentum=0.9, nesterov=True, fp32_matmul_prec="medium", weight_update_hook=Hook(),
              scaled_orthogonalize_fn=lambda g: 2 * g)  # fmt: skip
    p.grad = torch.ones(2, 3)
    before = torch.get_float32_matmul_precision()
    opt.step()
    assert torch.get_float32_matmul_precision() == before
    assert events == [("orth", "medium", ["lr", "momentum", "weight_decay"]), "pre", "hook_pre", "post", ("hook_post", 7.0)]
    # m = 0.1 g; nesterov u = g + 0.9 (m - g) = 0.19; update = 2u; p = 1 - 0.5 * 0.38
    assert torch.allclose(p, torch.full((2, 3), 1 - 0.5 * 0.38))
    assert q not in opt.state or len(opt.state[q]) == 0
    with pytest.raises(ValueError, match="closure is not supported"):
        opt.step(lambda: 0.0)
    r = torch.nn.Parameter(torch.ones(4))
    r.grad = torch.ones(4)
    with pytest.raises(ValueError, match="Only 2D parameters are supported."):
        _Identity([r], scaled_orthogonalize_fn=torch.nn.Identity()).step()


@pytest.mark.parametrize(
    "method,expect_p,expect_g",
    [("decoupled", 1 - 0.1 * 0.5, 1.0), ("independent", 1 - 0.1, 1.0), ("l2", 1.0, 1.0 + 0.1), ("palm", 1 - 0.1 * 0.25, 1.0)],
)
def test_weight_decay_methods(method, expect_p, expect_g):
    class Holder(mixin.WeightDecayMixin):
        weight_decay_method = method

    p, g = torch.ones(3, 3), torch.ones(3, 3)
    Holder()._apply_weight_decay_inplace(p, g, lr=0.5, weight_decay=0.1)
    assert torch.allclose(p, torch.full_like(p, expect_p)) and torch.allclose(g, torch.full_like(g, expect_g))
    Holder()._apply_weight_decay_inplace(p, g, lr=0.5, weight_decay=0.0)
    assert torch.allclose(p, torch.full_like(p, expect_p))

    class Bad(mixin.WeightDecayMixin):
        weight_decay_method = "nope"

    with pytest.raises(ValueError, match="Invalid weight decay method: nope"):
        Bad()._apply_weight_decay_inplace(p, g, 0.5, 0.1)


def test_precision_context_and_pg_helpers():
    before = torch.get_float32_matmul_precision()
    with fp32_matmul_precision("medium"):
        assert torch.get_float32_matmul_precision() == "medium"
        with pytest.raises(RuntimeError):
            with fp32_matmul_precision("high"):
                raise RuntimeError("x")
        assert torch.get_float32_matmul_precision() == "medium"
    assert torch.get_float32_matmul_precision() == before
    assert get_pg_size(None) == 1 and get_pg_rank(None) == 0


def test_fused_step_batch_plan_groups_equal_shapes_within_a_byte_budget():
    from emerging_optimizers_b200.orthogonalized_optimizers import _fused_step

    shapes = [(4096, 4096), (1024, 4096), (4096, 4096), (14336, 4096), (1024, 4096), (40, 24)]
    batches = _fused_step.plan_batches(shapes)
    assert sorted(i for b in batches for i in b) == list(range(len(shapes)))
    for b in batches:
        assert len({shapes[i] for i in b}) == 1
    assert [0, 2] in batches and [1, 4] in batches
    # a budget of one matrix splits a group into single-matrix batches
    small = _fused_step.plan_batches(shapes, max_batch_bytes=2 * 4096 * 4096)
    assert [0] in small and [2] in small and [1, 4] in small
    # CPU tensors are never eligible for the fused kernels
    p = torch.zeros(8, 8)
    assert not _fused_step.eligible(p, torch.zeros(8, 8))
    assert not _fused_step.eligible(p, None)


def test_tp_exchange_needs_a_group_and_cuda_shards(monkeypatch):
    from emerging_optimizers_b200.distributed import tensor_parallel as tp

    x = torch.zeros(8, 8, dtype=torch.bfloat16)
    assert not tp.fused_gram_available(x, None)
    assert not tp.fused_gram_available(x, object())  # CPU tensor: never
    assert tp.sharded_gram_poly(x, 1.0, 1.0, object()) is None  # likewise
    tp.clear()  # dropping the (empty) cache is harmless


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    """No fallback: if the shared library is not there, the first use raises and says how to build it."""
    from emerging_optimizers_b200 import _native

    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setenv("EO_B200_LIB", str(tmp_path / "libeo_b200.so"))
    with pytest.raises(_native.NativeLibraryError, match="no CPU or PyTorch fallback"):
        _native.lib()
    monkeypatch.delenv("EO_B200_LIB")
    monkeypatch.setattr(_native, "_lib", None)
    assert _native.lib().eo_version().decode().startswith("eo_b200")


def test_matrix_layout_detection():
    from emerging_optimizers_b200 import _native

    x = torch.zeros(6, 10)
    assert _native._mat_layout(x) == (0, 10, 0)
    assert _native._mat_layout(x.T) == (1, 10, 0)
    assert _native._mat_layout(x[:, :8]) == (0, 10, 0)  # padded rows
    b = torch.zeros(3, 6, 10)
    assert _native._mat_layout(b) == (0, 10, 60)
    assert _native._mat_layout(b.mT) == (1, 10, 60)
    assert not _native.is_matrix_layout(torch.zeros(6, 20)[:, ::2])
    assert _native.is_matrix_layout(torch.zeros(1, 7)) and _native.is_matrix_layout(torch.zeros(7, 1))


def test_padded_buffers_keep_rows_tma_addressable():
    m = muon_utils._empty_matrix((13, 21), torch.bfloat16, torch.device("cpu"))
    assert tuple(m.shape) == (13, 21) and m.stride(-1) == 1 and m.stride(-2) % 8 == 0
    b = muon_utils._empty_matrix((3, 13, 21), torch.bfloat16, torch.device("cpu"))
    assert tuple(b.shape) == (3, 13, 21) and b.stride(-2) % 8 == 0 and b.stride(0) % 8 == 0
    c = muon_utils._empty_matrix((16, 24), torch.bfloat16, torch.device("cpu"))
    assert c.is_contiguous()
    f = muon_utils._empty_matrix((5, 6), torch.float32, torch.device("cpu"))
    assert f.stride(-2) % 4 == 0


def test_a_failed_wait_of_an_earlier_call_raises_at_the_next_call(monkeypatch):
    """Every Newton-Schulz call mirrors the kernels' status word into host memory; a non-zero mirror (a kernel of
    an earlier call gave up a bounded wait) makes the next call raise, clears the word and the mirror."""
    from emerging_optimizers_b200 import _native as nat

    cleared = []
    monkeypatch.setattr(nat, "read_device_status", lambda device=None: cleared.append(device) or 0x21)
    dev = torch.device("cuda", 0)
    monkeypatch.setitem(nat._STATUS_MIRRORS, 0, torch.zeros(1, dtype=torch.int32))
    nat.raise_on_earlier_failure(dev)  # nothing recorded: passes
    nat._STATUS_MIRRORS[0][0] = 0x21
    with pytest.raises(nat.NativeLibraryError, match="0x21"):
        nat.raise_on_earlier_failure(dev)
    assert cleared == [dev] and int(nat._STATUS_MIRRORS[0][0]) == 0
    nat.raise_on_earlier_failure(dev)  # cleared: passes again


def test_layer_parallel_exchange_names():
    from emerging_optimizers_b200.distributed import LayerParallelMuon

    p = [torch.nn.Parameter(torch.zeros(8, 16)) for _ in range(4)]
    assert LayerParallelMuon(p, exchange="auto").exchange == "parameters"  # one process: a group of one
    mixed = LayerParallelMuon(p, exchange="mixed", updates_fraction=0.5, bucket_numel=128)
    assert sum(mixed._as_updates) == len(mixed.buckets) // 2 and len(mixed.buckets) == 4
    assert not any(LayerParallelMuon(p, exchange="parameters", bucket_numel=128)._as_updates)
    with pytest.raises(ValueError, match="exchange"):
        LayerParallelMuon(p, exchange="gradients")
    with pytest.raises(ValueError, match="updates_fraction"):
        LayerParallelMuon(p, exchange="mixed", updates_fraction=1.5)


@pytest.mark.parametrize("n", [8, 128, 136, 384, 1000, 2048, 4096, 8192])
@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_tensor_parallel_exchange_buffers_hold_every_tile(n, world):
    """The Gram exchange hands lower-triangle tiles (128 rows x 256 columns, 128 x 128 for n <= 128) to their owners
    round-robin; the size queries must leave a slot and a flag per (sender, tile) pair on every owner."""
    from emerging_optimizers_b200 import _native as nat

    lib = nat.lib()
    tile_n = 256 if n > 128 else 128
    tm, tn = -(-n // 128), -(-n // tile_n)
    tiles = sum(1 for i in range(tm) for j in range(tn) if i * 128 + 127 >= j * tile_n)
    slots = -(-tiles // world)  # tiles per owner
    assert lib.eo_tp_gram_flag_count(n, world) == world * slots
    assert lib.eo_tp_gram_inbox_bytes(n, world) == world * slots * 128 * tile_n * 2
    assert lib.eo_tp_gram_flag_count(0, world) == 0 and lib.eo_tp_gram_inbox_bytes(n, 0) == 0
