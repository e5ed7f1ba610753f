"""Measurement helpers: clock sampling during a timed region, L2 flush, rank-max timing."""
from __future__ import annotations

import shutil
import statistics
import subprocess
import tempfile
from typing import Optional

import torch

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Runs ``nvidia-smi`` in the background while a region is timed (read-only queries)."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self._proc: Optional[subprocess.Popen] = None
        self._file = None

    def start(self) -> None:
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return
        self._file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self._proc = subprocess.Popen(
            [exe, f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits",
             "-i", str(self.gpu_index), "-lms", str(self.period_ms)],
            stdout=self._file, stderr=subprocess.DEVNULL)

    def stop(self) -> dict:
        if self._proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self._proc.kill()
        self._file.flush()
        self._file.seek(0)
        sm, smax, power = [], [], []
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self._file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self._file.close()
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax),
                "power_w_max": max(power), "samples": len(sm), "reasons": sorted(reasons)}


_flush_buf = None


def flush_l2(device) -> None:
    """Overwrite a buffer larger than the 126 MB L2 so the next kernel starts cold."""
    global _flush_buf
    if _flush_buf is None or _flush_buf.device != torch.device(device):
        _flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    _flush_buf.zero_()


def max_over_ranks(value: float, device=None) -> float:
    """Maximum of ``value`` over the workers of the job (gathered over the control plane of
    the parameter server, or over ``torch.distributed`` in the baseline programs that use
    that instead)."""
    from .. import kvstore
    ctx = kvstore.context()
    if ctx is not None:
        return ctx.max_over_ranks(value)
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return value
