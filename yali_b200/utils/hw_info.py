"""Hardware facts for reports: GPUs, NVLink configuration, peer matrix, measured peaks.
Reference counterparts: src/common/hw_info.cuh (DetectNVLinkConfig via `nvidia-smi nvlink -s`),
`collect_system_info` in scripts/sweep.py:457-507."""
from __future__ import annotations

import json
import platform
import re
import subprocess
from pathlib import Path
from typing import Dict, Optional

NVLINK = {10: (18, 50.0), 9: (18, 25.0), 8: (12, 25.0), 7: (6, 25.0)}  # compute capability major -> (links, GB/s per direction)


def _run(cmd) -> str:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, timeout=30).stdout
    except (OSError, subprocess.TimeoutExpired):
        return ""


def parse_nvlink_status(text: str) -> Dict[int, Dict[str, float]]:
    """`nvidia-smi nvlink -s` -> {gpu: {"links": n, "gbs_per_link": x}} (pure function, testable)."""
    out: Dict[int, Dict[str, float]] = {}
    gpu = None
    for line in text.splitlines():
        m = re.match(r"GPU (\d+):", line.strip())
        if m:
            gpu = int(m.group(1))
            out[gpu] = {"links": 0, "gbs_per_link": 0.0}
            continue
        m = re.match(r"Link (\d+): ([\d.]+) GB/s", line.strip())
        if m and gpu is not None:
            out[gpu]["links"] += 1
            out[gpu]["gbs_per_link"] = float(m.group(2))
    return out


def nvlink_for_capability(major: int) -> Dict[str, float]:
    links, per = NVLINK.get(min(major, 10) if major >= 10 else major, (0, 0.0))
    return {"links": links, "gbs_per_link": per, "unidirectional_gbs": links * per, "bidirectional_gbs": 2 * links * per}


def measured_peaks(repo_root: Optional[Path] = None) -> Dict[str, float]:
    root = repo_root or Path(__file__).resolve().parents[2]
    p = root / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d.get("hbm_gbs"), "bf16_tflops": d.get("bf16_tflops"),
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def system_info() -> Dict[str, object]:
    info: Dict[str, object] = {"host": platform.node(), "python": platform.python_version()}
    q = _run(["nvidia-smi", "--query-gpu=index,name,memory.total,driver_version,clocks.max.sm", "--format=csv,noheader"])
    info["gpus"] = [ln.strip() for ln in q.splitlines() if ln.strip()]
    info["nvlink"] = parse_nvlink_status(_run(["nvidia-smi", "nvlink", "-s"]))
    info["topology"] = _run(["nvidia-smi", "topo", "-m"])
    try:
        import torch
        info["torch"] = torch.__version__
        info["cuda"] = torch.version.cuda
        if torch.cuda.is_available():
            info["nccl"] = ".".join(map(str, torch.cuda.nccl.version()))
    except Exception:  # noqa: BLE001
        pass
    info["measured_peaks"] = measured_peaks()
    return info
