"""``environment.json`` of a run: what is needed to reproduce a result or to reject it.

Retained reference surface: the file name and the top-level keys ``platform, python, pytorch, torch_cuda,
nvcc, gpu, driver, git_commit, git_status, native`` follow the reference's record
(``python/adangel/benchmark/metadata.py:21-55``) so that its tooling reads this build's runs.  Additions of
this build: the SM clock / power line sampled when the run starts (the B200 is power-limited: a number is
only comparable with its clocks beside it), the library's ABI version and the planner's environment
switches; the reference's CUTLASS revision pin has no counterpart (nothing is vendored here).
"""

from __future__ import annotations

import json
import os
import platform
import subprocess
from pathlib import Path

from ..ops.extension import native_status

_SWITCHES = ("ADG_TWO_CTA", "ADG_PDL")


def _first_output(*command: str):
    """stdout of a short command, or None when it is missing or fails."""
    try:
        done = subprocess.run(list(command), check=True, capture_output=True, text=True, timeout=10)
    except (OSError, subprocess.SubprocessError):
        return None
    return done.stdout.strip()


def _gpu_record() -> dict:
    import torch

    if not torch.cuda.is_available():
        return {}
    return {
        "name": torch.cuda.get_device_name(0),
        "compute_capability": list(torch.cuda.get_device_capability(0)),
        "device_count": torch.cuda.device_count(),
    }


def _library_record() -> dict:
    status = native_status()
    record = {"available": status.available, "reason": status.reason, "capabilities": status.capabilities}
    try:
        from ..ops import _sm100

        record["abi_version"] = int(_sm100.library().adg_abi_version())
    except OSError:
        record["abi_version"] = None
    return record


def collect_environment() -> dict:
    import torch

    smi = "nvidia-smi"
    return {
        "platform": platform.platform(),
        "python": platform.python_version(),
        "pytorch": torch.__version__,
        "torch_cuda": torch.version.cuda,
        "nvcc": _first_output("nvcc", "--version"),
        "gpu": _gpu_record(),
        "driver": _first_output(smi, "--query-gpu=driver_version", "--format=csv,noheader"),
        "clocks": _first_output(smi, "--query-gpu=clocks.sm,clocks.max.sm,power.draw,power.limit", "--format=csv,noheader"),
        "git_commit": _first_output("git", "rev-parse", "HEAD"),
        "git_status": _first_output("git", "status", "--short"),
        "native": _library_record(),
        "switches": {name: os.environ.get(name) for name in _SWITCHES},
    }


def write_environment(path: Path) -> None:
    path.write_text(json.dumps(collect_environment(), indent=2, ensure_ascii=False) + "\n", encoding="utf-8")
