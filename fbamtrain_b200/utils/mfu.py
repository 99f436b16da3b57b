"""Peak-throughput table and MFU arithmetic.

The reference keeps a table of dense peak TFLOP/s per device name and precision and reports
MFU = useful FLOPs / time / peak (reference: ``tensorlib/src/mfu.cpp:25-71, 75-140``); its table
stops at Hopper.  This table adds Blackwell and keeps the older parts for completeness.  Numbers
are *dense* peaks (no 2:4 sparsity).  ``measured_peaks()`` returns this machine's measured copy
bandwidth and cuBLAS bf16 rate when a ``MEASURED_PEAKS.json`` sits next to the package's parent.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

# device-name substring -> {precision: TFLOP/s}
PEAK_TFLOPS: Dict[str, Dict[str, float]] = {
    "B200": {"bf16": 2250.0, "fp16": 2250.0, "tf32": 1125.0, "fp32": 80.0, "fp8": 4500.0},
    "GB200": {"bf16": 2500.0, "fp16": 2500.0, "tf32": 1250.0, "fp32": 80.0, "fp8": 5000.0},
    "B100": {"bf16": 1750.0, "fp16": 1750.0, "tf32": 875.0, "fp32": 60.0, "fp8": 3500.0},
    "H200": {"bf16": 989.0, "fp16": 989.0, "tf32": 494.0, "fp32": 67.0, "fp8": 1979.0},
    "H100": {"bf16": 989.0, "fp16": 989.0, "tf32": 494.0, "fp32": 67.0, "fp8": 1979.0},
    "A100": {"bf16": 312.0, "fp16": 312.0, "tf32": 156.0, "fp32": 19.5},
    "V100": {"fp16": 125.0, "fp32": 15.7},
    "RTX 4090": {"bf16": 165.2, "fp16": 165.2, "tf32": 82.6, "fp32": 82.6},
    "RTX 3090": {"bf16": 71.0, "fp16": 71.0, "tf32": 35.6, "fp32": 35.6},
}
FALLBACK_MEASURED = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peak_tflops(device_name: str, precision: str = "bf16") -> Optional[float]:
    for key, row in PEAK_TFLOPS.items():
        if key.lower() in device_name.lower():
            return row.get(precision)
    return None


def measured_peaks() -> Dict[str, float]:
    """Measured denominators for rooflines; falls back to an earlier measurement of the same part."""
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    out = dict(FALLBACK_MEASURED)
    out["source"] = "fallback"
    return out


def mfu(useful_flops: float, seconds: float, device_name: str = "B200", precision: str = "bf16") -> Optional[float]:
    peak = peak_tflops(device_name, precision)
    if not peak or seconds <= 0:
        return None
    return useful_flops / seconds / (peak * 1e12)
