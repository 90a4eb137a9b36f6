"""Roofline arithmetic for optimizer steps: turns a measured time into a fraction of what the hardware allows.

Denominators are measured on the machine, not nominal: a copy bandwidth (GB/s), a bf16 GEMM rate (TFLOP/s, burst and
sustained) and an NVLink rate per direction.  :func:`load_peaks` reads them from ``MEASURED_PEAKS.json`` (a file the
benchmark driver writes next to ``bench.py``) and otherwise returns documented fallback values, marking which it used.

The work models restate what each optimizer has to do at minimum:

* element-wise chain: bytes = elements x (bytes read + bytes written per element), e.g. AdamW on fp32 = 4 reads + 3
  writes = 28 B (``heavyball/utils.py:1921-1943`` is the rule being counted);
* Newton-Schulz on an ``m x n`` matrix (``m <= n``), ``steps`` iterations: ``steps * (4 m^2 n + 2 m^3)`` FLOPs as the
  reference computes it (``heavyball/utils.py:568-573``), ``steps * (3 m^2 n + m^3)`` when the symmetry of ``X X^T`` and
  of the polynomial is used;
* fp32-accurate products on the tf32 tensor cores cost three tf32 passes.
"""

from __future__ import annotations

import json
import os
from typing import Iterable, Optional, Sequence

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
NVLINK_GBS_PER_DIRECTION = 770.0  # measured peer copy on this class of machine (nominal 900)


def load_peaks(path: Optional[str] = None) -> dict:
    """Measured peaks, or the fallback set when the file does not exist.  ``source`` says which."""
    candidates = [path] if path else []
    here = os.path.dirname(os.path.abspath(__file__))
    candidates.append(os.path.join(here, "..", "..", "MEASURED_PEAKS.json"))
    candidates.append(os.path.join(os.getcwd(), "MEASURED_PEAKS.json"))
    for cand in candidates:
        if cand and os.path.exists(cand):
            try:
                with open(cand) as fh:
                    data = json.load(fh)
                out = {k: float(data[k]) for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained")}
                out["source"] = "measured"
                return out
            except (OSError, ValueError, KeyError):
                continue
    return dict(FALLBACK_PEAKS)


def newton_schulz_flops(shape: Sequence[int], steps: int = 5, symmetric: bool = True) -> float:
    if len(shape) < 2:
        return 0.0
    rows = shape[0]
    cols = 1
    for s in shape[1:]:
        cols *= s
    m, n = min(rows, cols), max(rows, cols)
    per = (3 * m * m * n + m**3) if symmetric else (4 * m * m * n + 2 * m**3)
    return float(steps * per)


def elementwise_bytes(numel: int, reads: int, writes: int, bytes_per_element: float = 4.0) -> float:
    return float(numel) * (reads + writes) * bytes_per_element


def fraction(time_ms: float, *, flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0,
             peaks: Optional[dict] = None, sustained: bool = True) -> dict:  # fmt: skip
    """Lower bound on the time of a step that needs ``flops`` bf16-equivalent tensor FLOPs, ``hbm_bytes`` of device
    memory traffic and ``nvlink_bytes`` across NVLink per GPU and direction, and the measured time as a multiple of it.
    Compute and memory phases are assumed not to overlap (they are separate kernels), NVLink to overlap with both."""
    peaks = peaks or load_peaks()
    rate = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"] * 1e12
    t_compute = flops / rate * 1e3
    t_memory = hbm_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3
    t_link = nvlink_bytes / (NVLINK_GBS_PER_DIRECTION * 1e9) * 1e3
    floor = max(t_compute + t_memory, t_link)
    return {
        "floor_ms": floor,
        "compute_floor_ms": t_compute,
        "memory_floor_ms": t_memory,
        "nvlink_floor_ms": t_link,
        "measured_ms": time_ms,
        "fraction_of_floor": (floor / time_ms) if time_ms else None,
        "peaks": peaks["source"],
    }


def muon_adamw_step(matrix_shapes: Iterable[Sequence[int]], other_numel: int, time_ms: float, *, world: int = 1,
                    ns_steps: int = 5, peaks: Optional[dict] = None) -> dict:  # fmt: skip
    """Roofline of ``SplitOpt(Muon on matrices, AdamW on the rest)``: Newton-Schulz FLOPs (symmetry used) plus the
    element-wise traffic (Muon: gradient + momentum read, momentum write, parameter read + write, and the bf16 work
    copies of the iteration; AdamW: 4 reads + 3 writes), both divided by ``world`` when the work is owner-partitioned;
    with ``world > 1`` each rank also reads its share of every peer's gradient and writes its share of the parameters to
    every peer over NVLink."""
    matrix_shapes = list(matrix_shapes)
    flops = sum(newton_schulz_flops(s, ns_steps) for s in matrix_shapes) / world
    mat_numel = sum(_numel(s) for s in matrix_shapes)
    hbm = (elementwise_bytes(mat_numel, 3, 2) + elementwise_bytes(other_numel, 4, 3)) / world
    link = 0.0
    if world > 1:
        share = (mat_numel + other_numel) / world
        link = share * 4.0 * (world - 1)  # gradient elements pulled from every peer (and the same volume pushed back)
    out = fraction(time_ms, flops=flops, hbm_bytes=hbm, nvlink_bytes=link, peaks=peaks)
    out.update(ns_flops=flops, hbm_bytes=hbm, nvlink_bytes_per_direction=link)
    return out


def _numel(shape):
    n = 1
    for s in shape:
        n *= s
    return n
