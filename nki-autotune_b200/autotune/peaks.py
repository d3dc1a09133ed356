"""Roofline denominators: measured on the pool's B200s when available, else a stated fallback."""

from __future__ import annotations

import json
from pathlib import Path

# earlier measurement on the same GPU pool, used only when no measured file is present
FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
NOMINAL = {"hbm_gbs": 7700.0, "bf16_tflops": 2250.0}


def load_peaks() -> dict:
    """Peaks from ``MEASURED_PEAKS.json`` found at or above the package root, else the fallback."""
    here = Path(__file__).resolve()
    for parent in here.parents:
        cand = parent / "MEASURED_PEAKS.json"
        if cand.is_file():
            try:
                data = json.loads(cand.read_text())
                return {
                    "hbm_gbs": float(data["hbm_gbs"]),
                    "bf16_tflops": float(data["bf16_tflops"]),
                    "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                    "source": "measured",
                }
            except (ValueError, KeyError):
                break
    return dict(FALLBACK)
