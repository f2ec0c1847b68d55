"""Host-side pieces of bench.py that need no GPU: the FLOP conventions and the clock sampler (against a fake
``nvidia-smi`` placed first on PATH)."""

import importlib.util
import os
import stat
import time

from oracle import ns_oracle


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


def test_flop_conventions_match_the_oracle():
    for m, n in ((8192, 28672), (1024, 4096), (128, 8192), (4096, 4096)):
        dense, sym = bench.flops(m, n, 5)
        assert dense == 5 * (4.0 * m * m * n + 2.0 * m**3)
        assert sym == 5 * (m * (m + 1.0) * n + m * m * (m + 1.0) + 2.0 * m * m * n)
        assert sym < dense
        want = ns_oracle.ns_flops(m, n, 5)
        assert (dense, sym) == tuple(want)
    # the headline workload: 4.398e13 dense-equivalent FLOP per call
    assert abs(bench.flops(8192, 28672, 5)[0] - 4.398e13) / 4.398e13 < 1e-3


def test_clock_sampler_summarises_samples_under_load(tmp_path, monkeypatch):
    fake = tmp_path / "nvidia-smi"
    rows = [
        "345, 1965, 180.5, Not Active, Not Active, Not Active, Not Active",  # idle sample: dropped
        "1410, 1965, 990.1, Not Active, Not Active, Not Active, Active",
        "1425, 1965, 998.7, Not Active, Not Active, Not Active, Active",
        "1395, 1965, 995.0, Not Active, Not Active, Not Active, Active",
    ]
    fake.write_text("#!/bin/sh\n" + "".join(f"echo '{r}'\n" for r in rows) + "sleep 30\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    sampler = bench.ClockSampler(0)
    sampler.start()
    time.sleep(0.5)
    out = sampler.stop()
    assert out["sm_mhz"] == 1410.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"] and out["samples"] == 3
    assert abs(out["power_w_max"] - 998.7) < 1e-6


def test_clock_sampler_without_nvidia_smi_reports_nothing(tmp_path, monkeypatch):
    monkeypatch.setenv("PATH", str(tmp_path))
    sampler = bench.ClockSampler(0)
    sampler.start()
    assert sampler.stop() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}


def test_peaks_fall_back_when_the_file_is_absent(tmp_path, monkeypatch):
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    peaks, kind = bench.load_peaks()
    assert kind == "fallback" and peaks["bf16_tflops"] == 1590.0 and peaks["hbm_gbs"] == 6650.0
