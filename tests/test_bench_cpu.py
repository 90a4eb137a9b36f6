"""Host-side pieces of ``bench.py`` that need no GPU: argument defaults and the clock sampler (run against a
stand-in ``nvidia-smi`` that prints timestamped samples)."""

import importlib.util
import os
import stat
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_defaults_finish_quickly_and_use_one_gpu(monkeypatch):
    bench = _bench()
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = bench.parse()
    assert args.gpus == 1 and args.impl == "ours" and args.warmup >= 3 and 1 <= args.steps <= 100
    assert args.graphs == "auto" and not args.no_e2e


def test_clock_sampler_keeps_only_samples_from_the_timed_region(tmp_path, monkeypatch):
    fake = tmp_path / "nvidia-smi"
    fake.write_text(
        "#!/usr/bin/env python3\n"
        "import datetime, time\n"
        "time.sleep(0.25)\n"  # NVML start-up
        "n = 0\n"
        "while True:\n"
        "    stamp = datetime.datetime.now().strftime('%Y/%m/%d %H:%M:%S.%f')[:-3]\n"
        "    clock = 900 if n < 2 else 1950\n"  # the first samples (before the timed region) show an idle clock
        "    print(f'{stamp}, 0, {clock}, 1965, 700.0, Not Active, Not Active, Not Active, Active', flush=True)\n"
        "    n += 1\n"
        "    time.sleep(0.1)\n"
    )
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    bench = _bench()
    sampler = bench.ClockSampler(0)
    t0 = time.time()
    sampler.start()
    assert time.time() - t0 >= 0.2  # waited for the first sample, i.e. for the start-up to be over
    time.sleep(0.25)  # "warm-up"
    sampler.begin()
    time.sleep(0.45)  # "timed region"
    out = sampler.stop()
    assert out["sm_mhz"] == 1950.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"] and out["samples"] >= 3


def test_clock_sampler_without_nvidia_smi(monkeypatch, tmp_path):
    monkeypatch.setenv("PATH", str(tmp_path))
    bench = _bench()
    sampler = bench.ClockSampler(0)
    sampler.start()
    sampler.begin()
    assert sampler.stop()["reasons"] == ["nvidia-smi unavailable"]
