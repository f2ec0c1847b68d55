"""Benchmark of the Newton-Schulz orthogonalization hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (BASELINE config 4 on one device): a "step" is one full ``newton_schulz`` call -- Frobenius
normalisation, bf16 down-cast, five "simple" iterations (A = XX^T, B = bA + cA^2, X <- aX + BX) on the sm_100a
kernels and the fp32 result -- on one 8192 x 28672 fp32 matrix.  With N > 1 every rank orthogonalizes its own
matrix of that shape (layer-parallel partitioning: the matrices of a model are independent units) and the ranks
then all-gather the bf16-rounded results over NVLink, which is the one exchange step of a layer-parallel Muon
step; per-GPU work is fixed, so scaling is "weak".

Printed value: dense-equivalent TFLOP/s (4 m^2 n + 2 m^3 per iteration, the convention of the reference's own
SYRK benchmark, which credits a symmetric product like a general one) summed over all ranks.  The roofline
object credits symmetric outputs once (what the kernels actually execute) and compares with the measured
cuBLAS bf16 peak of this GPU pool.

``--impl reference`` times the CPU restatement of the reference (oracle/ns_oracle.py, numpy + OpenBLAS on all
host cores) on a bounded corner block of the same matrix.
"""

from __future__ import annotations

import argparse
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
CPU_SAMPLE = (2048, 7168)  # corner block timed on the host
NOMINAL_BF16_TFLOPS = 2250.0
TRAFFIC_BYTES_PER_LAUNCH = 0.67e9
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}


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
def cpu_reference(steps: int, warmup: int) -> dict:
    """Time the numpy restatement of the reference on the host cores; returns the cpu_baseline object."""
    import numpy as np

    from oracle import ns_oracle

    try:
        from threadpoolctl import threadpool_info

        cores = max([p.get("num_threads", 1) for p in threadpool_info()] or [os.cpu_count() or 1])
    except Exception:
        cores = os.cpu_count() or 1
    m, n = CPU_SAMPLE
    rng = np.random.default_rng(3)
    x = rng.standard_normal((m, n), dtype=np.float32)
    for _ in range(max(warmup, 0)):
        ns_oracle.newton_schulz(x, 1, COEFF, precision="medium")
    times = []
    for _ in range(max(steps, 1)):
        t0 = time.perf_counter()
        ns_oracle.newton_schulz(x, NS_STEPS, COEFF, precision="medium")
        times.append(time.perf_counter() - t0)
    dense, _ = flops(m, n, NS_STEPS)
    total = sum(times)
    return {
        "value": dense * len(times) / total / 1e12,
        "unit": "TFLOP/s",
        "cores": int(cores),
        "kind": "port",
        "sample": f"{len(times)} x newton_schulz({m}x{n} corner block, {NS_STEPS} '{COEFF}' steps, bf16-rounded "
        f"operands, fp32 accumulate) in numpy/OpenBLAS; {total / len(times):.2f} s per call",
        "ms_per_step": 1e3 * total / len(times),
    }


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # Keep the whole run within a few minutes whatever K is.
    steps = max(1, min(args.steps, 20))
    base = cpu_reference(steps, min(args.warmup, 2))
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
        "config": workload_config(args.gpus),
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


def run_gpu_arm(args) -> None:
    import torch
    import torch.distributed as dist

    from emerging_optimizers_b200 import _native
    from emerging_optimizers_b200.orthogonalized_optimizers import muon_utils
    from emerging_optimizers_b200.utils import fp32_matmul_precision

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

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
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0 and not args.kernels_only:
        sampler.start()
        time.sleep(0.3)

    # ---- timed region 1: inputs resident in HBM -------------------------------------------------
    launches0 = _native.launch_count
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_device()
    torch.cuda.current_stream().wait_stream(side)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = _native.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else {}
    if args.kernels_only:
        if rank == 0:
            dense, sym = flops(M, N_COLS, NS_STEPS)
            nb = max(args.batch, 1)
            print(json.dumps({"kernels_only": True, "shape": [M, N_COLS], "batch": args.batch,
                              "ms_per_step": ms_total / args.steps,
                              "tflops_dense_eq": nb * dense * args.steps / (ms_total / 1e3) / 1e12,
                              "gpu_launches": launches, "device_status": _native.read_device_status(dev)}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- per-launch timing of the tensor-core kernel (same stream, CUDA events around each launch) ----
    _native.launch_timer = []
    for _ in range(2):
        ns_call(x)
    torch.cuda.synchronize()
    kernel_ms = [a.elapsed_time(b) for _, a, b, _ in _native.launch_timer]
    names = [n for n, _, _, _ in _native.launch_timer]
    kernel_launches = sum(k for _, _, _, k in _native.launch_timer)
    _native.launch_timer = None

    # ---- timed region 2: end to end with host buffers ------------------------------------------
    # Pinned fp32 input -> device, newton_schulz, fp32 result -> pinned host, every step; the three stages of
    # consecutive steps overlap on three streams (two input and two output buffers).
    y_host = torch.empty(M, N_COLS, dtype=torch.float32).pin_memory()
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    bufs = [torch.empty_like(x) for _ in range(2)]
    free_in = [None, None]   # event: compute that read bufs[i] has finished
    outs = [None, None]

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
            outs[b] = y
        cur.wait_stream(s_out)

    e2e_loop(2)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    e2e_loop(args.steps)
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)

    status = _native.read_device_status(dev)

    # ---- reduce over ranks ------------------------------------------------------------------------
    t = torch.tensor([ms_total, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = float(t[0]), float(t[1])

    if rank == 0:
        dense, sym = flops(M, N_COLS, NS_STEPS)
        peaks, peak_kind = load_peaks()
        sec = ms_total / 1e3
        value = dense * args.steps * world / sec / 1e12
        # The timed region is seconds long, so the sustained cuBLAS figure is the denominator.
        peak = float(peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"])
        k_total_ms = sum(kernel_ms)
        n_launch = kernel_launches
        # two newton_schulz calls were timed: 2 * sym FLOP in n_launch launches of eo_gemm_kernel
        achieved = (sym * 2 / n_launch) / (k_total_ms / n_launch / 1e3) / 1e12 if n_launch else None
        by_name = {}
        for nme, ms in zip(names, kernel_ms):
            by_name.setdefault(nme, []).append(ms)
        cpu = cpu_reference(4, 1) if world == 1 else None
        line = {
            "metric": "newton_schulz_tflops",
            "value": value,
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
            "config": workload_config(world),
            "tflops_sym": sym * args.steps * world / sec / 1e12,
            "pct_of_measured_peak_sym": 100.0 * sym * args.steps / sec / 1e12 / peak,
            "pct_of_nominal_peak_sym": 100.0 * sym * args.steps / sec / 1e12 / NOMINAL_BF16_TFLOPS,
            "roofline": {
                "bound": "tensor",
                "kernel": "eo_gemm_kernel (Gram SYRK, A^2 SYRK and BX GEMM launches of one call, averaged)",
                "achieved": achieved,
                "peak": peak,
                "peak_kind": f"bf16_tflops_sustained, {peak_kind}",
                "unit": "TFLOP/s",
                "frac": (achieved / peak) if achieved else None,
                "frac_of_burst_peak": (achieved / float(peaks["bf16_tflops"])) if achieved else None,
                # DRAM bytes per launch: read + write of the Gram, A^2 and BX launches of one iteration measured by
                # ncu on 4096 x 16384 (138 + 35 + 398 MB), scaled by operand bytes to this shape and averaged over
                # the three launches.
                "traffic": TRAFFIC_BYTES_PER_LAUNCH if (M, N_COLS) == (8192, 28672) else None,
                "algorithmic_flops_per_launch": sym * 2 / n_launch if n_launch else None,
                "avg_launch_ms": k_total_ms / n_launch if n_launch else None,
                "call_ms": {k: sum(v) / len(v) for k, v in by_name.items()},
                "launches_timed": n_launch,
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
        if cpu is not None:
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_muon_step(args) -> None:
    """Secondary workload (BASELINE config 3): one Muon step over a Llama-3-8B-shaped parameter set, 32 layers of
    q/o 4096x4096, k/v 1024x4096, gate/up 14336x4096, down 4096x14336; fp32 params, bf16-rounded N(0, 1e-3)
    gradients, Nesterov momentum 0.95, lr 0.02, decoupled weight decay 0.1, shape_scaling, five "simple" steps.
    On N > 1 GPUs the matrices are divided among the ranks (layer-parallel) and the bf16 updates all-gathered;
    total work is fixed, so scaling is "strong"."""
    import torch
    import torch.distributed as dist

    from emerging_optimizers_b200 import _native
    from emerging_optimizers_b200.distributed import LayerParallelMuon

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    layers = args.layers
    layer = [(4096, 4096)] * 2 + [(1024, 4096)] * 2 + [(14336, 4096)] * 2 + [(4096, 14336)]
    g = torch.Generator(device=dev).manual_seed(2)
    params = []
    for _ in range(layers):
        for s in layer:
            p = torch.nn.Parameter(torch.randn(*s, generator=g, device=dev) * 0.02)
            p.grad = (torch.randn(*s, generator=g, device=dev) * 1e-3).bfloat16().float()
            params.append(p)
    opt = LayerParallelMuon(params, lr=0.02, momentum=0.95, weight_decay=0.1, nesterov=True,
                            weight_decay_method="decoupled", num_ns_steps=5, scale_mode="shape_scaling",
                            coefficient_type="simple", fp32_matmul_prec="medium", use_syrk=True,
                            exchange=args.lp_exchange,
                            **({"bucket_numel": args.bucket_numel} if args.bucket_numel else {}))  # fmt: skip

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 1)):
        opt.step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _native.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        opt.step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if rank == 0 else {}
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    # checksum over ranks: parameters must be identical everywhere
    chk = torch.stack([p.detach().double().sum() for p in params[:: max(1, len(params) // 16)]]).sum().reshape(1)
    same = True
    if world > 1:
        lo, hi = chk.clone(), chk.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        same = bool((lo == hi).all())
    status = _native.read_device_status(dev)
    if rank == 0:
        dense = layers * sum(flops(min(s), max(s), NS_STEPS)[0] for s in layer)
        sym = layers * sum(flops(min(s), max(s), NS_STEPS)[1] for s in layer)
        print(json.dumps({
            "metric": "muon_step_ms", "value": float(t[0]), "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 1), "ms_per_step": float(t[0]), "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"Muon step, Llama-3-8B-shaped parameter set ({layers} layers, {len(params)} matrices, "
                       f"{sum(p.numel() for p in params) / 1e9:.2f} G parameters), layer-parallel x{world}",
                       "exchange": args.lp_exchange, "l2": "parameter set far larger than L2"},
            "tflops_dense_eq": dense / (float(t[0]) / 1e3) / 1e12, "tflops_sym": sym / (float(t[0]) / 1e3) / 1e12,
            "params_identical_across_ranks": same, "gpu_launches": (_native.launch_count - launches0),
            "clocks": clocks, "device_status": status,
        }), flush=True)  # fmt: skip
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_tp_ns(args) -> None:
    """Secondary workload (BASELINE config 4): tensor-parallel Newton-Schulz of one 8192 x 28672 matrix whose
    columns are sharded over the N ranks; per iteration the partial Gram matrices are all-reduced (fused into the
    SYRK epilogue, or NCCL with --exchange nccl).  Total work is fixed: "strong" scaling."""
    import torch
    import torch.distributed as dist

    from emerging_optimizers_b200 import _native
    from emerging_optimizers_b200.orthogonalized_optimizers import muon_utils
    from emerging_optimizers_b200.utils import fp32_matmul_precision

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    os.environ["EO_TP_GRAM"] = "nccl" if args.exchange == "nccl" else "fused"
    if args.tp_shard_poly_min_world:
        muon_utils.TP_SHARD_GRAM_POLY_MIN_WORLD = args.tp_shard_poly_min_world
    cols = N_COLS // world
    g = torch.Generator(device=dev).manual_seed(3 + rank)
    x = torch.randn(M, cols, generator=g, device=dev)
    group = dist.group.WORLD if world > 1 else None

    def call():
        with fp32_matmul_precision("medium"):
            if world == 1:
                return muon_utils.newton_schulz(x, NS_STEPS, COEFF, use_syrk=True)
            return muon_utils.newton_schulz_tp(x, NS_STEPS, COEFF, group, partition_dim=1, tp_mode="distributed",
                                               use_syrk=True)  # fmt: skip

    for _ in range(max(args.warmup, 3)):
        call()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        call()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    status = _native.read_device_status(dev)
    if rank == 0:
        dense, sym = flops(M, N_COLS, NS_STEPS)
        ms = float(t[0])
        print(json.dumps({
            "metric": "tp_newton_schulz_ms", "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"tensor-parallel newton_schulz {M}x{N_COLS}, column shards of {cols}, "
                       f"{NS_STEPS} '{COEFF}' steps, Gram exchange: {args.exchange if world > 1 else 'none'}"},
            "tflops_dense_eq": dense / (ms / 1e3) / 1e12, "device_status": status,
        }), flush=True)  # fmt: skip
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
    ap.add_argument("--workload", default="newton_schulz", choices=["newton_schulz", "muon_step", "tp_ns"],
                    help="newton_schulz (default, the headline metric) or muon_step (BASELINE config 3)")
    ap.add_argument("--layers", type=int, default=32, help="layers of the muon_step workload")
    ap.add_argument("--tp-shard-poly-min-world", type=int, default=0,
                    help="tp_ns: smallest group that computes S = bA + cA^2 in row blocks per rank (0: library default)")
    ap.add_argument("--lp-exchange", choices=["updates", "parameters"], default="updates",
                    help="muon_step: what the layer-parallel optimizer all-gathers")
    ap.add_argument("--bucket-numel", type=int, default=0,
                    help="muon_step: elements per rank and exchange bucket (0: the optimizer's default)")
    args = ap.parse_args()
    if args.shape is not None:
        global M, N_COLS
        M, N_COLS = args.shape
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "muon_step":
        run_muon_step(args)
    elif args.workload == "tp_ns":
        run_tp_ns(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
