"""Provenance header for result files: which code, which machine, which peaks a number was measured with.

Counterpart of the reference's ``ssa.harness.stamp`` (stamp.py:35-45)."""

from __future__ import annotations

import json
import os
import platform
import subprocess
import time


def stamp() -> dict:
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = {"time": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), "host_cores": os.cpu_count(),
           "python": platform.python_version()}
    try:
        out["git"] = subprocess.run(["git", "-C", root, "rev-parse", "--short", "HEAD"], capture_output=True, text=True,
                                    timeout=5).stdout.strip() or None
    except (OSError, subprocess.SubprocessError):
        out["git"] = None
    try:
        import torch
        out["torch"] = torch.__version__
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(0)
            out["gpu"] = {"name": p.name, "capability": [p.major, p.minor], "sms": p.multi_processor_count,
                          "memory_gb": round(p.total_memory / 2 ** 30, 1)}
    except ImportError:
        pass
    pk = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        with open(pk) as fh:
            peaks = json.load(fh)
        out["peaks"] = {k: peaks.get(k) for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained")}
    return out
