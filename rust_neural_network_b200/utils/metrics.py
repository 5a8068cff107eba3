"""Observability: JSON-lines metrics, a roofline calculator against the measured peaks, and a report of
the native kernel build in use. The reference only prints (rust-nn src/finetune.rs:385-392,
src/distill.rs:275-291) and returns histories as vectors; here every step can leave one machine-readable
line and the same numbers feed the HTML dashboards of `gui`.
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from pathlib import Path
from typing import Dict, Optional

import torch

ROOT = Path(__file__).resolve().parents[2]


def measured_peaks() -> Dict[str, float]:
    """Roofline denominators: the copy bandwidth and bf16 GEMM throughput recorded for this installation's GPUs in
    `MEASURED_PEAKS.json` at the repository root when that file exists, otherwise the documented fallback (`kind` says
    which)."""
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "kind": "of measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "kind": "of fallback"}


def roofline(ms: float, flops: float = 0.0, bytes_moved: float = 0.0, nvlink_bytes: float = 0.0, nvlink_gbs: float = 770.0) -> Dict[str, float]:
    """Achieved rates of one launch and their fraction of the measured peaks. The target time of a fused
    compute + collective kernel is the slowest of FLOPs / GEMM peak, bytes / HBM copy rate and NVLink bytes / link rate."""
    pk = measured_peaks()
    t = ms / 1e3
    out = {"ms": ms, "kind": pk["kind"]}
    if flops:
        out["tflops"] = flops / t / 1e12
        out["frac_of_bf16_peak"] = out["tflops"] / pk["bf16_tflops"]
    if bytes_moved:
        out["gbs"] = bytes_moved / t / 1e9
        out["frac_of_hbm_peak"] = out["gbs"] / pk["hbm_gbs"]
    target = max(flops / (pk["bf16_tflops"] * 1e12) if flops else 0.0, bytes_moved / (pk["hbm_gbs"] * 1e9) if bytes_moved else 0.0,
                 nvlink_bytes / (nvlink_gbs * 1e9) if nvlink_bytes else 0.0)
    if target > 0:
        out["roofline_ms"] = target * 1e3
        out["frac_of_roofline"] = target / t
    return out


def kernel_report() -> Dict[str, object]:
    """Which native code this process runs: library paths, target architecture, device, launch counter."""
    from .. import _native as nv
    lib_dir = Path(nv.__file__).resolve().parent / "lib"
    rep = {"arch": "sm_100a", "cuda_library": str(lib_dir / "libb200nn_cuda.so"), "host_library": str(lib_dir / "libb200nn_host.so"),
           "cuda_library_present": (lib_dir / "libb200nn_cuda.so").exists(), "host_library_present": (lib_dir / "libb200nn_host.so").exists(),
           "gemm": "tcgen05 128 x {64,128,256} x 64 bf16 / TF32 / int8 / e4m3, TMA 128B-swizzled stages, TMEM double-buffered accumulators",
           "attention": "tcgen05 flash forward (O resident in TMEM) and backward (dK/dV resident, dQ double-buffered)",
           "launches_so_far": nv.launch_count()}
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(torch.cuda.current_device())
        rep["device"] = {"name": p.name, "sms": p.multi_processor_count, "memory_gib": round(p.total_memory / 2 ** 30, 1), "cc": f"{p.major}.{p.minor}"}
    return rep


class MetricsLogger:
    """Appends one JSON object per call to `path` (and keeps them in `records`)."""

    def __init__(self, path: Optional[str] = None, rank: int = 0, echo: bool = False):
        self.path, self.rank, self.echo = path, rank, echo
        self.records = []
        self._t0 = time.time()
        if path and rank == 0:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)

    def log(self, step: int, **fields) -> dict:
        rec = {"step": int(step), "t": round(time.time() - self._t0, 4)}
        for k, v in fields.items():
            if isinstance(v, torch.Tensor):
                v = v.detach().float().cpu().tolist() if v.numel() > 1 else float(v)
            rec[k] = v
        self.records.append(rec)
        if self.rank == 0:
            if self.path:
                with open(self.path, "a") as f:
                    f.write(json.dumps(rec) + "\n")
            if self.echo:
                print(" ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in rec.items()), flush=True)
        return rec

    def losses(self):
        return [r["loss"] for r in self.records if "loss" in r]


# ----------------------------------------------------------------------------------------------- tracing
def enable_nvtx(on: bool = True) -> None:
    """Turn on NVTX ranges around this package's kernel families (gemm, flash attention, linear attention, scan, norm,
    loss, optimizer, collectives) and around the phases of `Trainer` steps. Off by default: a range costs about a
    microsecond on the host."""
    from .. import _native as nv
    nv.NVTX_ENABLED = bool(on) and torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str):
    """An NVTX range that is free when tracing is off or no GPU is present."""
    from .. import _native as nv
    if nv.NVTX_ENABLED:
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


@contextlib.contextmanager
def profile_to(path: str, with_stack: bool = False):
    """Record everything inside the block with `torch.profiler` (CPU + CUDA activities, this package's NVTX ranges as
    user annotations) and export a Chrome trace to `path`."""
    from torch.profiler import ProfilerActivity, profile
    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    from .. import _native as nv
    was = nv.NVTX_ENABLED
    enable_nvtx(True)
    try:
        with profile(activities=acts, with_stack=with_stack) as prof:
            yield prof
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        prof.export_chrome_trace(path)
    finally:
        nv.NVTX_ENABLED = was
