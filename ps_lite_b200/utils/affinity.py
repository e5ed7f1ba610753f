"""Pin the process to the CPUs next to its GPU, so that pinned host buffers and the threads
that feed the copy engines sit on the GPU's NUMA node (read-only NVML query; nothing on the
GPU is changed)."""
from __future__ import annotations

import os
from typing import Optional


def bind_to_gpu_cpus(device_index: int) -> Optional[list[int]]:
    """Restrict this process to the CPU set NVML reports as closest to ``device_index``.

    Returns the CPU list, or None when NVML or the affinity call is unavailable.  Disabled by
    ``PSB200_NO_AFFINITY=1``."""
    if os.environ.get("PSB200_NO_AFFINITY") == "1" or not hasattr(os, "sched_setaffinity"):
        return None
    try:
        import pynvml
        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        phys = device_index
        if visible:
            ids = [v.strip() for v in visible.split(",") if v.strip()]
            if device_index < len(ids) and ids[device_index].isdigit():
                phys = int(ids[device_index])
        handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
        ncpu = os.cpu_count() or 1
        words = (ncpu + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = [w * 64 + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1]
        allowed = os.sched_getaffinity(0)
        cpus = [c for c in cpus if c in allowed]
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return cpus
    except Exception:
        return None
