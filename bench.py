"""Benchmark of the Newton-Schulz orthogonalization hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (BASELINE config 4 on one device): a "step" is one full ``newton_schulz`` call -- Frobenius
normalisation, bf16 down-cast, five "simple" iterations (A = XX^T, B = bA + cA^2, X <- aX + BX) on the sm_100a
kernels and the fp32 result -- on one 8192 x 28672 fp32 matrix.  With N > 1 every rank orthogonalizes its own
matrix of that shape (layer-parallel partitioning: the matrices of a model are independent units) and the ranks
then all-gather the bf16-rounded results over NVLink, which is the one exchange step of a layer-parallel Muon
step; per-GPU work is fixed, so scaling is "weak".

Printed value: dense-equivalent TFLOP/s (4 m^2 n + 2 m^3 per iteration, the convention of the reference's own
SYRK benchmark, which credits a symmetric product like a general one) summed over all ranks.  The roofline
object credits symmetric outputs once (what the kernels actually execute) and compares with the measured
cuBLAS bf16 peak of this GPU pool.

The same JSON line carries, as further objects, the other configurations the metric names, each with its parity
check: ``muon_step`` (config 3: one Muon step over a Llama-3-8B-shaped parameter set, layer-parallel over the N
ranks), ``tp_ns`` (config 4 sharded: tensor-parallel Newton-Schulz over the N ranks, N > 1), ``per_head``
(config 5: 6400 per-head matrices divided among the ranks), ``syrk_config2`` (config 2: the batched SYRK) and
``gpu_library_baseline`` (the reference's GPU arithmetic, cuBLAS through torch, timed in the same run).

``--impl reference`` times the CPU restatement of the reference (oracle/ns_torch_cpu.py: the reference's own torch
CPU operators on all host cores) on a bounded corner block of the same matrix.
"""

from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M, N_COLS, NS_STEPS, COEFF = 8192, 28672, 5, "simple"
ABC = (3.4445, -4.7750, 2.0315)  # the "simple" tuple
CPU_SAMPLE = (2048, 7168)  # corner block timed on the host
NOMINAL_BF16_TFLOPS = 2250.0
TRAFFIC_BYTES_PER_LAUNCH = 1.95e9
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}
LAYER_SHAPES = [(4096, 4096)] * 2 + [(1024, 4096)] * 2 + [(14336, 4096)] * 2 + [(4096, 14336)]
MUON_KW = dict(lr=0.02, momentum=0.95, weight_decay=0.1, nesterov=True, weight_decay_method="decoupled",
               num_ns_steps=NS_STEPS, scale_mode="shape_scaling", coefficient_type=COEFF, fp32_matmul_prec="medium",
               use_syrk=True)  # fmt: skip
HEADS_TOTAL, HEAD_SHAPE, HEAD_CHUNK = 6400, (128, 8192), 1600


def flops(m: int, n: int, steps: int) -> tuple[float, float]:
    """(dense-equivalent, symmetric-credited) FLOPs of `steps` quintic iterations on an m x n matrix, m <= n."""
    dense = 4.0 * m * m * n + 2.0 * m**3
    sym = m * (m + 1.0) * n + m * m * (m + 1.0) + 2.0 * m * m * n
    return steps * dense, steps * sym


def load_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------------------------ CPU arm
def use_all_host_cores() -> int:
    """Let torch's CPU operators (and any BLAS behind numpy) use every core this process may run on, whatever
    OMP_NUM_THREADS the launcher exported (torch.distributed.run sets it to 1).  Returns the thread count."""
    import torch

    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(n, 1))
    try:
        from threadpoolctl import threadpool_limits

        threadpool_limits(limits=n)
    except Exception:
        pass
    return torch.get_num_threads()


def cpu_reference(steps: int, warmup: int) -> dict:
    """Time the torch-CPU restatement of the reference on the host cores; returns the cpu_baseline object."""
    import torch

    from oracle import ns_torch_cpu

    cores = use_all_host_cores()
    m, n = CPU_SAMPLE
    g = torch.Generator(device="cpu").manual_seed(3)
    x = torch.randn(m, n, generator=g, dtype=torch.float32)
    for _ in range(max(warmup, 1)):
        ns_torch_cpu.newton_schulz(x, 1, COEFF, "medium")
    times = []
    for _ in range(max(steps, 1)):
        t0 = time.perf_counter()
        ns_torch_cpu.newton_schulz(x, NS_STEPS, COEFF, "medium")
        times.append(time.perf_counter() - t0)
        if sum(times) > 25.0:
            break
    dense, _ = flops(m, n, NS_STEPS)
    total = sum(times)
    return {
        "value": dense * len(times) / total / 1e12,
        "unit": "TFLOP/s",
        "cores": int(cores),
        "kind": "port",
        "sample": f"{len(times)} x newton_schulz({m}x{n} corner block of the {M}x{N_COLS} workload, {NS_STEPS} "
        f"'{COEFF}' steps) with the reference's own CPU operators (torch bf16 matmul / addmm at precision 'medium', "
        f"{cores} threads); {total / len(times):.2f} s per call",
        "ms_per_step": 1e3 * total / len(times),
    }


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # Keep the whole run within a few minutes whatever K is.
    steps = max(1, min(args.steps, 20))
    base = cpu_reference(steps, min(args.warmup, 2))
    cfg = workload_config(args.gpus)
    cfg["timed_on_host"] = f"{CPU_SAMPLE[0]}x{CPU_SAMPLE[1]} corner block per step (bounded sample), kind: port"
    line = {
        "impl": "reference",
        "metric": "newton_schulz_tflops",
        "value": base["value"],
        "unit": "TFLOP/s",
        "n_gpus": args.gpus,
        "steps": steps,
        "warmup": args.warmup,
        "ms_per_step": base["ms_per_step"],
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int) -> dict:
    return {
        "workload": f"newton_schulz {M}x{N_COLS} fp32 in/out, {NS_STEPS} '{COEFF}' steps, bf16 tensor-core path "
        "(fp32 matmul precision 'medium', use_syrk=True)",
        "matrices_per_step": n_gpus,
        "parallelism": "single device" if n_gpus == 1 else f"layer-parallel x{n_gpus}: one matrix per rank, all-gather of "
        "the bf16 results by copy-engine pushes into symmetric memory, overlapped with the next call",
        "l2": "inputs larger than L2 (940 MB fp32 input, 470 MB bf16 iterate per matrix)",
        "flop_convention": "value: dense-equivalent 4m^2n+2m^3 per iteration; roofline: symmetric outputs counted once",
    }


# ------------------------------------------------------------------------------------------------ GPU arm
class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons while the timed region runs."""

    FIELDS = (
        "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self) -> None:
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"),
                stderr=subprocess.DEVNULL,
            )
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        try:
            with open(self.path) as f:
                for ln in f:
                    parts = [p.strip() for p in ln.split(",")]
                    if len(parts) == 7 and parts[0].replace(".", "").isdigit():
                        rows.append(parts)
            os.unlink(self.path)
        except Exception:
            pass
        if not rows:
            return out
        # keep samples taken under load (power draw above 40 % of the maximum seen)
        pw = [float(r[2]) if r[2].replace(".", "").isdigit() else 0.0 for r in rows]
        loaded = [r for r, w in zip(rows, pw) if w >= 0.4 * max(pw)] or rows
        sm = sorted(float(r[0]) for r in loaded)
        out["sm_mhz"] = sm[len(sm) // 2]
        out["sm_max_mhz"] = float(rows[0][1])
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        out["reasons"] = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in loaded)]
        out["samples"] = len(loaded)
        out["power_w_max"] = max(pw)
        return out


def bind_host_to_gpu(local_rank: int) -> str:
    """Pin this process to the CPU cores next to its GPU (NVML's affinity mask), so that pinned host buffers are
    allocated on that NUMA node and host <-> device copies of different ranks do not share one socket's memory.
    Returns a description for the config object; does nothing if NVML or the affinity call is not available."""
    try:
        import pynvml
        import torch

        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(local_rank).uuid)
        handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        allowed = os.sched_getaffinity(0)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (max(allowed) + 64) // 64)
        near = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        cpus = near & allowed
        if cpus and cpus != allowed:
            os.sched_setaffinity(0, cpus)
            return f"bound to {len(cpus)} cores near the GPU"
        if not cpus:
            return f"none of the {len(allowed)} allowed cores is near the GPU"
        return "all allowed cores are near the GPU"
    except Exception as exc:  # noqa: BLE001
        return f"not bound ({type(exc).__name__})"


class Ctx:
    """Process-group context of one bench process."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}: launch with torch.distributed.run "
                             f"--nproc-per-node {args.gpus}")  # fmt: skip
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.binding = bind_host_to_gpu(self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev, timeout=datetime.timedelta(seconds=300))
        self.group = dist.group.WORLD if self.world > 1 else None

    def barrier(self) -> None:
        import torch
        import torch.distributed as dist

        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, *vals: float) -> list[float]:
        import torch
        import torch.distributed as dist

        t = torch.tensor(list(vals), device=self.dev, dtype=torch.float64)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def close(self) -> None:
        import torch.distributed as dist

        if self.world > 1:
            dist.barrier()
            dist.destroy_process_group()


def timed(fn, warm: int, steps: int) -> float:
    """Mean milliseconds of ``fn()`` over ``steps`` calls after ``warm`` calls, CUDA events on the current stream."""
    import torch

    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def rel_fro(a, b) -> float:
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-300))


def library_newton_schulz(x, steps: int = NS_STEPS, abc=ABC):
    """The reference's GPU arithmetic for one call (muon_utils.py:216, 262-269, 370-377 there): Frobenius
    normalisation, bf16 cast, ``steps`` iterations of three library (cuBLAS) products, fp32 result.  ``x`` is fp32,
    2-D or batched 3-D; tall inputs are iterated in the wide orientation."""
    import torch

    tall = x.size(-2) > x.size(-1)
    if tall:
        x = x.mT
    X = (x / x.norm(dim=(-2, -1), keepdim=True).clamp_min(1e-15)).to(torch.bfloat16)
    a, b, c = abc
    for _ in range(steps):
        A = X @ X.mT
        if X.ndim == 3:
            B = torch.baddbmm(A, A, A, alpha=c, beta=b)
            X = torch.baddbmm(X, B, X, alpha=1.0, beta=a)
        else:
            B = torch.addmm(A, A, A, alpha=c, beta=b)
            X = torch.addmm(X, B, X, alpha=1.0, beta=a)
    X = X.to(torch.float32)
    return X.mT if tall else X


def headline_section(ctx: Ctx, args) -> dict:
    import torch
    import torch.distributed as dist

    from emerging_optimizers_b200 import _native
    from emerging_optimizers_b200.orthogonalized_optimizers import muon_utils
    from emerging_optimizers_b200.utils import fp32_matmul_precision

    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    g = torch.Generator(device="cpu").manual_seed(3 + rank)
    x_host = torch.empty(M, N_COLS, dtype=torch.float32).pin_memory()
    # Same distribution as config 4 (N(0,1)); generated in row blocks to bound host memory traffic.
    for r0 in range(0, M, 1024):
        r1 = min(r0 + 1024, M)
        x_host[r0:r1].copy_(torch.randn(r1 - r0, N_COLS, generator=g, dtype=torch.float32))
    x = x_host.to(dev, non_blocking=True)
    torch.cuda.synchronize()
    if args.batch > 0:
        if not args.kernels_only:
            raise SystemExit("--batch needs --kernels-only")
        gb = torch.Generator(device=dev).manual_seed(4)
        x = torch.randn(args.batch, M, N_COLS, generator=gb, device=dev) * 1e-3

    # Exchange buffer of the layer-parallel scheme: symmetric memory written by copy engines (no SMs taken from the
    # persistent tensor-core kernels); NCCL all-gather if symmetric memory cannot be set up on this box.
    side = torch.cuda.Stream(device=dev)
    gather_buf, peer = None, None
    slot = M * N_COLS
    if world > 1 and args.exchange == "nccl":
        gather_buf = torch.empty(world, M, N_COLS, dtype=torch.bfloat16, device=dev)
    elif world > 1:
        try:
            from emerging_optimizers_b200.distributed.peer_memory import PeerBuffer

            peer = PeerBuffer(2 * world * slot, torch.bfloat16, dev)
        except Exception as exc:  # noqa: BLE001
            if rank == 0:
                print(f"symmetric memory unavailable ({exc}); using NCCL all-gather", file=sys.stderr)
            gather_buf = torch.empty(world, M, N_COLS, dtype=torch.bfloat16, device=dev)
    exchanges = [0]

    def ns_call(inp: torch.Tensor) -> torch.Tensor:
        with fp32_matmul_precision("medium"):
            return muon_utils.newton_schulz(inp, NS_STEPS, COEFF, use_syrk=True)

    def step_device() -> torch.Tensor:
        y = ns_call(x)
        if world > 1:
            # exchange step of the layer-parallel scheme, overlapped with the next call on a side stream
            ev = torch.cuda.Event()
            ev.record()
            with torch.cuda.stream(side):
                side.wait_event(ev)
                if peer is not None:
                    base = (exchanges[0] % 2) * world * slot
                    exchanges[0] += 1
                    peer.local[base + rank * slot : base + (rank + 1) * slot].copy_(y.view(-1))  # fp32 -> bf16, lossless
                    peer.all_gather_slots(base, slot)
                else:
                    yb = y.to(torch.bfloat16)
                    dist.all_gather_into_tensor(gather_buf.view(-1), yb.view(-1))
                y.record_stream(side)
        return y

    n_warm = args.warmup if args.kernels_only else max(args.warmup, 3)
    for _ in range(n_warm):
        step_device()
    side.synchronize()
    ctx.barrier()

    sampler = ClockSampler(ctx.local_rank)
    if rank == 0 and not args.kernels_only:
        sampler.start()
        time.sleep(0.3)

    # ---- timed region 1: inputs resident in HBM -------------------------------------------------
    # The last few steps are also bracketed per library call (CUDA events on the launching stream around the 15
    # tensor-core launches of one newton_schulz call), so that the roofline figure is taken inside the sustained
    # loop, under the same clocks as ms_per_step.
    n_bracketed = 0 if args.kernels_only else min(5, args.steps)
    launches0 = _native.launch_count
    ctx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        if n_bracketed and i == args.steps - n_bracketed:
            _native.launch_timer = []
        step_device()
    torch.cuda.current_stream().wait_stream(side)
    e1.record()
    ctx.barrier()
    ms_total = e0.elapsed_time(e1)
    launches = _native.launch_count - launches0
    timer, _native.launch_timer = (_native.launch_timer or []), None
    if args.kernels_only:
        dense, sym = flops(M, N_COLS, NS_STEPS)
        nb = max(args.batch, 1)
        return {"kernels_only": True, "shape": [M, N_COLS], "batch": args.batch, "ms_per_step": ms_total / args.steps,
                "tflops_dense_eq": nb * dense * args.steps / (ms_total / 1e3) / 1e12, "gpu_launches": launches,
                "device_status": _native.read_device_status(dev)}  # fmt: skip
    call_ms = [a.elapsed_time(b) for _, a, b, _ in timer]
    kernel_launches = sum(k for _, _, _, k in timer)

    # ---- timed region 2: end to end with host buffers ------------------------------------------
    # Pinned fp32 input -> device, newton_schulz, fp32 result -> pinned host, every step; the three stages of
    # consecutive steps overlap on three streams (two input and two output buffers).
    y_host = torch.empty(M, N_COLS, dtype=torch.float32).pin_memory()
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    bufs = [torch.empty_like(x) for _ in range(2)]
    free_in = [None, None]  # event: compute that read bufs[i] has finished

    def e2e_loop(k: int) -> None:
        cur = torch.cuda.current_stream()
        for i in range(k):
            b = i % 2
            with torch.cuda.stream(s_in):
                if free_in[b] is not None:
                    s_in.wait_event(free_in[b])
                bufs[b].copy_(x_host, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            cur.wait_event(ready)
            y = ns_call(bufs[b])
            done = torch.cuda.Event()
            done.record(cur)
            free_in[b] = done
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                y_host.copy_(y, non_blocking=True)
                y.record_stream(s_out)
        cur.wait_stream(s_out)

    e2e_loop(2)
    ctx.barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    e2e_loop(args.steps)
    f1.record()
    ctx.barrier()
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else {}  # sampled over both timed regions
    status = _native.read_device_status(dev)
    ms_total, ms_e2e = ctx.max_over_ranks(ms_total, ms_e2e)
    del bufs, peer, gather_buf
    torch.cuda.empty_cache()

    dense, sym = flops(M, N_COLS, NS_STEPS)
    peaks, peak_kind = load_peaks()
    sec = ms_total / 1e3
    sustained = float(peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"])
    burst = float(peaks["bf16_tflops"])
    mean_call = sum(call_ms) / len(call_ms) if call_ms else None
    achieved = sym / (mean_call / 1e3) / 1e12 if mean_call else None
    per_call_launches = kernel_launches // max(len(call_ms), 1)
    line = {
        "metric": "newton_schulz_tflops",
        "value": dense * args.steps * world / sec / 1e12,
        "unit": "TFLOP/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": n_warm,
        "ms_per_step": ms_total / args.steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": dict(workload_config(world), host_binding=ctx.binding),
        "tflops_sym": sym * args.steps * world / sec / 1e12,
        "pct_of_measured_peak_sym": 100.0 * sym * args.steps / sec / 1e12 / sustained,
        "pct_of_nominal_peak_sym": 100.0 * sym * args.steps / sec / 1e12 / NOMINAL_BF16_TFLOPS,
        "roofline": {
            "bound": "tensor",
            "kernel": "eo_gemm_pair_kernel (the Gram SYRK, A^2 SYRK and BX GEMM launches of one newton_schulz call)",
            "achieved": achieved,
            "peak": sustained,
            "peak_kind": f"bf16_tflops_sustained ({peak_kind}): the launches are timed inside the seconds-long loop",
            "unit": "TFLOP/s",
            "frac": (achieved / sustained) if achieved else None,
            "frac_of_burst_peak": (achieved / burst) if achieved else None,
            # DRAM bytes per launch: read + write of the Gram, A^2 and BX launches of one iteration of this very
            # workload measured by ncu (2.09 + 0.60 + 3.17 GB), averaged over the three launches.  The operands
            # are 0.47 GB (X) and 0.13 GB (A, S): the excess is re-reading by later rounds of tiles.
            "traffic": TRAFFIC_BYTES_PER_LAUNCH if (M, N_COLS) == (8192, 28672) else None,
            "algorithmic_flops_per_launch": sym / per_call_launches if per_call_launches else None,
            "avg_launch_ms": mean_call / per_call_launches if mean_call and per_call_launches else None,
            "call_ms": mean_call,
            "calls_timed": len(call_ms),
            "launches_per_call": per_call_launches,
            "timed_where": "CUDA events around the tensor-core launches of the last calls of the timed loop",
            "call_ms_x_sm_mhz": (mean_call * clocks["sm_mhz"]) if mean_call and clocks.get("sm_mhz") else None,
        },
        "e2e": {
            "value": dense * args.steps * world / (ms_e2e / 1e3) / 1e12,
            "unit": "TFLOP/s",
            "ms_per_step": ms_e2e / args.steps,
            "h2d_bytes_per_step": x_host.numel() * 4 * world,
            "d2h_bytes_per_step": y_host.numel() * 4 * world,
        },
        "gpu_launches": launches,
        "clocks": clocks,
        "device_status": status,
    }
    return line


def library_section(ctx: Ctx) -> tuple[dict, dict]:
    """The reference's GPU arithmetic (torch / cuBLAS) timed beside the kernels, same device, same run: the
    headline call, and config 2 (batched SYRK 32 x 2048 x 8192 against torch.bmm, TF-eq = 2 B N^2 K / t as in the
    reference's benchmarks/bench_batched_syrk.py:89)."""
    import torch

    from emerging_optimizers_b200 import triton_kernels as tk
    from emerging_optimizers_b200.orthogonalized_optimizers import muon_utils
    from emerging_optimizers_b200.utils import fp32_matmul_precision

    dev = ctx.dev
    g = torch.Generator(device=dev).manual_seed(3)
    x = torch.randn(M, N_COLS, generator=g, device=dev)
    lib_ms = timed(lambda: library_newton_schulz(x), 2, 5)

    def ours():
        with fp32_matmul_precision("medium"):
            return muon_utils.newton_schulz(x, NS_STEPS, COEFF, use_syrk=True)

    our_ms = timed(ours, 2, 5)
    err = rel_fro(ours(), library_newton_schulz(x))
    dense, _ = flops(M, N_COLS, NS_STEPS)
    lib_ms, our_ms = ctx.max_over_ranks(lib_ms, our_ms)
    base = {
        "what": f"newton_schulz {M}x{N_COLS}, {NS_STEPS} '{COEFF}' steps with torch / cuBLAS bf16 products (the "
        "reference's GPU arithmetic), device-resident, 5 calls back to back",
        "ms_per_step": lib_ms,
        "tflops_dense_eq": dense / (lib_ms / 1e3) / 1e12,
        "this_library_ms_same_loop": our_ms,
        "speedup": lib_ms / our_ms,
        "rel_fro_this_library_vs_library_gemm": err,
    }
    del x
    B, N, K = 32, 2048, 8192
    g = torch.Generator(device=dev).manual_seed(1)
    xs = (torch.randn(B, N, K, generator=g, device=dev) / K**0.5).to(torch.bfloat16)
    syrk_ms = timed(lambda: tk.batched_tsyrk_ex(xs), 5, 20)
    bmm_ms = timed(lambda: torch.bmm(xs, xs.mT), 5, 20)
    a = tk.batched_tsyrk_ex(xs)
    want = torch.bmm(xs.float(), xs.float().mT)
    tf = 2.0 * B * N * N * K / 1e12
    syrk_ms, bmm_ms = ctx.max_over_ranks(syrk_ms, bmm_ms)
    cfg2 = {
        "what": f"batched SYRK {B} x {N} x {K} bf16, entries N(0, 1/{K}), seed 1; TF-eq = 2 B N^2 K / t",
        "ms": syrk_ms,
        "tf_eq": tf / (syrk_ms / 1e3),
        "torch_bmm_ms": bmm_ms,
        "torch_bmm_tf_eq": tf / (bmm_ms / 1e3),
        "speedup": bmm_ms / syrk_ms,
        "rel_fro_vs_fp32_accumulated": rel_fro(a, want),
        "max_rel_err": float(((a.float() - want).abs() / want.abs().clamp_min(1e-2)).max()),
        "exactly_symmetric": bool(torch.equal(a, a.mT)),
    }
    return base, cfg2


def muon_step_section(ctx: Ctx, args) -> dict:
    """BASELINE config 3: one Muon step over a Llama-3-8B-shaped parameter set (32 layers of q/o 4096x4096, k/v
    1024x4096, gate/up 14336x4096, down 4096x14336; fp32 params N(0, 0.02^2), bf16-rounded N(0, 1e-6) gradients,
    Nesterov momentum 0.95, lr 0.02, decoupled weight decay 0.1, shape_scaling, five "simple" steps), divided
    among the N ranks by LayerParallelMuon.  Total work is fixed ("strong" scaling).  Checked in the same run
    against the single-process step (every rank also runs the whole step alone: its time is ``n1_ms_same_run``,
    its parameters after three steps the reference for ``rel_fro_vs_single_process``) and, for the first step of a
    subset of matrices, against the step restated with library GEMMs."""
    import torch
    import torch.distributed as dist

    from emerging_optimizers_b200 import _native
    from emerging_optimizers_b200.distributed import LayerParallelMuon

    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    layers = args.layers
    shapes = LAYER_SHAPES * layers
    subset = sorted(set(list(range(len(LAYER_SHAPES))) + list(range(len(shapes) - len(LAYER_SHAPES), len(shapes)))))
    parity_steps = 3

    def fill(tensors, seed, scale, bf16_round):
        gen = torch.Generator(device=dev).manual_seed(seed)
        for t in tensors:
            v = torch.randn(t.shape, generator=gen, device=dev) * scale
            t.copy_(v.bfloat16().float() if bf16_round else v)

    params = [torch.nn.Parameter(torch.empty(s, device=dev)) for s in shapes]
    grads = [torch.empty(s, device=dev) for s in shapes]
    with torch.no_grad():
        fill([p.data for p in params], 3, 0.02, False)
        fill(grads, 2, 1e-3, True)
    for p, g in zip(params, grads):
        p.grad = g
    p0 = {i: params[i].detach().clone() for i in subset}

    def library_first_step(i: int) -> torch.Tensor:
        """Parameter i after the first step, restated with torch operators and library GEMMs
        (orthogonalized_optimizer.py:164-212 and muon.py:117-132 of the reference)."""
        kw = MUON_KW
        p, g = p0[i].clone(), grads[i]
        p.add_(p, alpha=-kw["weight_decay"] * kw["lr"])
        m = torch.zeros_like(g).lerp_(g, 1 - kw["momentum"])
        u = g.lerp(m, kw["momentum"])
        o = library_newton_schulz(u)
        scale = max(1, p.size(0) / p.size(1)) ** 0.5
        return p.add_(o * scale * 1.0, alpha=-kw["lr"])

    out: dict = {}
    solo_params_after = None
    if world > 1:
        # single-process step on every rank at once (a group of one rank each), for time and for parity
        solo = None
        for r in range(world):
            grp = dist.new_group([r])
            if r == rank:
                solo = grp
        opt1 = LayerParallelMuon(params, group=solo, **MUON_KW)
        ctx.barrier()
        opt1.step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(parity_steps - 1):
            opt1.step()
        e1.record()
        torch.cuda.synchronize()
        out["n1_ms_same_run"] = ctx.max_over_ranks(e0.elapsed_time(e1) / (parity_steps - 1))[0]
        solo_params_after = {i: params[i].detach().clone() for i in subset}
        del opt1
        torch.cuda.empty_cache()
        with torch.no_grad():
            fill([p.data for p in params], 3, 0.02, False)

    opt = LayerParallelMuon(params, group=ctx.group, exchange=args.lp_exchange,
                            **({"updates_fraction": args.updates_fraction} if args.lp_exchange == "mixed" else {}),
                            **({"bucket_numel": args.bucket_numel} if args.bucket_numel else {}), **MUON_KW)  # fmt: skip
    opt.step()
    torch.cuda.synchronize()
    errs = [rel_fro(params[i].detach() - p0[i], library_first_step(i) - p0[i]) for i in subset[: len(LAYER_SHAPES)]]
    out["rel_fro_update_step1_vs_library_gemm"] = ctx.max_over_ranks(max(errs))[0]
    for _ in range(parity_steps - 1):
        opt.step()
    torch.cuda.synchronize()
    if solo_params_after is not None:
        worst = max(rel_fro(params[i].detach(), solo_params_after[i]) for i in subset)
        same = all(torch.equal(params[i].detach(), solo_params_after[i]) for i in subset)
        out["rel_fro_vs_single_process"] = ctx.max_over_ranks(worst)[0]
        out["bitwise_equal_to_single_process"] = bool(ctx.max_over_ranks(0.0 if same else 1.0)[0] == 0.0)
        del solo_params_after
    out["parity_subset"] = f"the {len(subset)} matrices of the first and the last layer, after {parity_steps} steps"

    ctx.barrier()
    launches0 = _native.launch_count
    k = max(2, min(args.muon_steps, 20))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx.barrier()
    e0.record()
    for _ in range(k):
        opt.step()
    e1.record()
    ctx.barrier()
    ms = ctx.max_over_ranks(e0.elapsed_time(e1) / k)[0]
    # checksum over ranks: parameters must be identical everywhere
    chk = torch.stack([p.detach().double().sum() for p in params[:: max(1, len(params) // 32)]])
    same = True
    if world > 1:
        lo, hi = chk.clone(), chk.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        same = bool((lo == hi).all())
    dense = layers * sum(flops(min(s), max(s), NS_STEPS)[0] for s in LAYER_SHAPES)
    sym = layers * sum(flops(min(s), max(s), NS_STEPS)[1] for s in LAYER_SHAPES)
    out.update({
        "what": f"Muon step, Llama-3-8B-shaped parameter set ({layers} layers, {len(params)} matrices, "
        f"{sum(p.numel() for p in params) / 1e9:.2f} G parameters), layer-parallel x{world}, exchange of "
        f"{opt.exchange}{' (updates for %.2f of the elements)' % args.updates_fraction if args.lp_exchange == 'mixed' else ''}"
        "; strong scaling",
        "ms": ms, "steps_timed": k, "warmup_steps": parity_steps,
        "tflops_dense_eq": dense / (ms / 1e3) / 1e12, "tflops_sym": sym / (ms / 1e3) / 1e12,
        "params_identical_across_ranks": same, "gpu_launches": _native.launch_count - launches0,
        "device_status": _native.read_device_status(dev),
    })  # fmt: skip
    if "n1_ms_same_run" in out:
        out["efficiency_vs_n1"] = out["n1_ms_same_run"] / (world * ms)
    del opt, params, grads, p0
    torch.cuda.empty_cache()
    return out


def tp_section(ctx: Ctx, args) -> dict:
    """BASELINE config 4 sharded: tensor-parallel Newton-Schulz of one 8192 x 28672 matrix whose columns are sharded
    over the N ranks; per iteration the partial Gram matrices are summed inside the SYRK kernel (fused) or by an
    NCCL all-reduce behind it (nccl, timed for comparison).  Total work is fixed: "strong" scaling.  The gathered
    result is compared with single-device Newton-Schulz on the gathered matrix."""
    import torch
    import torch.distributed as dist

    from emerging_optimizers_b200 import _native
    from emerging_optimizers_b200.distributed import tensor_parallel
    from emerging_optimizers_b200.orthogonalized_optimizers import muon_utils
    from emerging_optimizers_b200.utils import fp32_matmul_precision

    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    cols = N_COLS // world
    g = torch.Generator(device=dev).manual_seed(3 + rank)
    x = torch.randn(M, cols, generator=g, device=dev)

    def call(mode: str):
        os.environ["EO_TP_GRAM"] = mode
        with fp32_matmul_precision("medium"):
            return muon_utils.newton_schulz_tp(x, NS_STEPS, COEFF, ctx.group, partition_dim=1, tp_mode="distributed",
                                               use_syrk=True)  # fmt: skip

    k = max(5, min(args.steps, 20))
    res = {}
    for mode in ("auto", "nccl"):
        ctx.barrier()
        res[mode] = ctx.max_over_ranks(timed(lambda: call(mode), 3, k))[0]
    y_fused, y_nccl = call("auto"), call("nccl")
    os.environ["EO_TP_GRAM"] = "auto"
    shards = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(shards, x)
    full = torch.cat(shards, dim=1)
    del shards
    with fp32_matmul_precision("medium"):
        y_full = muon_utils.newton_schulz(full, NS_STEPS, COEFF, use_syrk=True)
    mine = y_full[:, rank * cols : (rank + 1) * cols]
    err_fused, err_nccl = ctx.max_over_ranks(rel_fro(y_fused, mine), rel_fro(y_nccl, mine))
    ex = tensor_parallel._exchange(M, ctx.group, dev)
    dense, _ = flops(M, N_COLS, NS_STEPS)
    return {
        "what": f"tensor-parallel newton_schulz {M}x{N_COLS}, column shards of {cols}, {NS_STEPS} '{COEFF}' steps; "
        "strong scaling",
        "ms": res["auto"],
        "exchange": "SYRK + all-reduce in one kernel: "
        + ("NVSwitch multimem load-reduce / multicast stores" if ex.multicast else "peer loads / stores")
        + (", S in row blocks gathered by multicast stores" if world >= muon_utils.TP_SHARD_GRAM_POLY_MIN_WORLD else ""),
        "ms_nccl_allreduce": res["nccl"],
        "steps_timed": k,
        "tflops_dense_eq": dense / (res["auto"] / 1e3) / 1e12,
        "rel_fro_vs_single_device": err_fused,
        "rel_fro_vs_single_device_nccl": err_nccl,
        "device_status": _native.read_device_status(dev),
    }


def per_head_section(ctx: Ctx, args) -> dict:
    """BASELINE config 5: 6400 per-head matrices of 128 x 8192 (a Llama-3-70B-shaped attention stack split per
    head), divided among the N ranks (independent units, no collective), orthogonalized in chunks of up to 1600 by the
    fused small-matrix kernel.  One chunk of seeded data is reused for every chunk of a rank."""
    import torch

    from emerging_optimizers_b200 import _native
    from emerging_optimizers_b200.orthogonalized_optimizers import muon_utils
    from emerging_optimizers_b200.utils import fp32_matmul_precision

    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    heads_here = HEADS_TOTAL // world
    chunk = min(HEAD_CHUNK, heads_here)  # matrices per library call (one call runs them as one persistent kernel)
    chunks = max(1, heads_here // chunk)
    g = torch.Generator(device=dev).manual_seed(4 + rank)
    x = (torch.randn(chunk, *HEAD_SHAPE, generator=g, device=dev) * 1e-3).bfloat16().float()

    def step():
        with fp32_matmul_precision("medium"):
            for _ in range(chunks):
                y = muon_utils.newton_schulz(x, NS_STEPS, COEFF, use_syrk=True)
        return y

    ctx.barrier()
    ms = ctx.max_over_ranks(timed(step, 2, 5))[0]
    y = step()
    err = max(rel_fro(y[i], library_newton_schulz(x[i])) for i in (0, 1, chunk // 2, chunk - 1))
    err = ctx.max_over_ranks(err)[0]
    dense, _ = flops(*HEAD_SHAPE, NS_STEPS)
    total = chunks * chunk * world
    return {
        "what": f"{total} matrices of {HEAD_SHAPE[0]}x{HEAD_SHAPE[1]} ({chunks * chunk} per GPU in chunks of "
        f"{chunk}), {NS_STEPS} '{COEFF}' steps each, fp32 in/out",
        "ms": ms,
        "matrices_per_s": total / (ms / 1e3),
        "tflops_dense_eq": total * dense / (ms / 1e3) / 1e12,
        "rel_fro_vs_library_gemm": err,
        "device_status": _native.read_device_status(dev),
    }


def run_gpu_arm(args) -> None:
    ctx = Ctx(args)
    line = headline_section(ctx, args)
    if not args.kernels_only and args.sections != "headline":
        sections = [
            ("gpu_library_baseline", lambda: library_section(ctx)),
            ("muon_step", lambda: muon_step_section(ctx, args)),
            ("per_head", lambda: per_head_section(ctx, args)),
        ]
        if ctx.world > 1:
            sections.insert(2, ("tp_ns", lambda: tp_section(ctx, args)))
        for name, fn in sections:
            try:
                res = fn()
            except Exception as exc:  # noqa: BLE001  (a failed extra must not cost the headline line)
                res = {"error": f"{type(exc).__name__}: {exc}"[:400]}
                if name == "gpu_library_baseline":
                    res = (res, res)
            if name == "gpu_library_baseline":
                line["gpu_library_baseline"], line["syrk_config2"] = res
            else:
                line[name] = res
        if ctx.rank == 0:
            cpu = cpu_reference(4, 1)
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if ctx.rank == 0:
        print(json.dumps(line), flush=True)
    ctx.close()


def run_single_section(args) -> None:
    """One of the secondary workloads on its own (ad-hoc runs): prints that section's object."""
    ctx = Ctx(args)
    fn = {"muon_step": muon_step_section, "tp_ns": tp_section, "per_head": per_head_section}[args.workload]
    res = fn(ctx, args)
    if ctx.rank == 0:
        print(json.dumps(dict(res, n_gpus=ctx.world, workload=args.workload)), flush=True)
    ctx.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--shape", type=int, nargs=2, default=None, metavar=("M", "N"),
                    help="matrix shape instead of 8192 28672 (for profiler captures of a small case)")
    ap.add_argument("--batch", type=int, default=0,
                    help="with --kernels-only: run on a (BATCH, M, N) stack of matrices (per-head workload)")
    ap.add_argument("--kernels-only", action="store_true",
                    help="device-resident timing only: no end-to-end loop, CPU baseline or clock sampling, and "
                    "--warmup taken as given (for profiler captures; not a benchmark number)")
    ap.add_argument("--exchange", default="ce", choices=["ce", "nccl"],
                    help="N > 1: exchange results by copy-engine pushes into symmetric memory (default) or by NCCL")
    ap.add_argument("--workload", default="all", choices=["all", "muon_step", "tp_ns", "per_head"],
                    help="all (default): the headline line with every section; or one secondary section alone")
    ap.add_argument("--sections", default="all", choices=["all", "headline"],
                    help="headline: only the newton_schulz metric, without the secondary sections")
    ap.add_argument("--layers", type=int, default=32, help="layers of the muon_step section")
    ap.add_argument("--muon-steps", type=int, default=5, help="timed steps of the muon_step section")
    ap.add_argument("--lp-exchange", choices=["auto", "updates", "parameters", "mixed"], default="auto",
                    help="muon_step: what the layer-parallel optimizer all-gathers (auto: parameters up to four "
                    "ranks, updates beyond)")
    ap.add_argument("--updates-fraction", type=float, default=0.5,
                    help="muon_step with --lp-exchange mixed: fraction of the elements exchanged as updates")
    ap.add_argument("--bucket-numel", type=int, default=0,
                    help="muon_step: elements per rank and exchange bucket (0: the optimizer's default)")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="set a tuning knob of the native library before running (eo_set_option), e.g. gemm_pair=0; "
                    "for A/B runs and profiler captures")
    args = ap.parse_args()
    if args.option and args.impl != "reference":
        from emerging_optimizers_b200 import _native

        for item in args.option:
            name, _, value = item.partition("=")
            _native.set_option(name, int(value))
    if args.shape is not None:
        global M, N_COLS
        M, N_COLS = args.shape
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload != "all":
        run_single_section(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
