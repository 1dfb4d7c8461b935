"""Samples a GPU's SM clock and throttle reasons with nvidia-smi while a timed region runs
(read-only: nothing about the GPU is changed)."""
from __future__ import annotations

import subprocess
import threading


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap,temperature.gpu")

    def __init__(self, index: int, period_s: float = 0.2):
        self.index, self.period = index, period_s
        self.rows = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                parts = [p.strip() for p in out.stdout.strip().split(",")]
                if len(parts) >= 7:
                    self.rows.append(parts)
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(6)

        def num(s):
            try:
                return float(s)
            except ValueError:
                return None

        sm = sorted(v for v in (num(r[0]) for r in self.rows) if v is not None)
        mx = [v for v in (num(r[1]) for r in self.rows) if v is not None]
        pw = [v for v in (num(r[2]) for r in self.rows) if v is not None]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in self.rows)]
        out = {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx[0] if mx else None,
               "power_w_max": max(pw) if pw else None, "reasons": reasons, "samples": len(self.rows)}
        temps = [v for v in (num(r[7]) for r in self.rows if len(r) > 7) if v is not None]
        if temps:  # die temperature at the first and the last sample, and the highest seen
            out["temp_c"] = {"first": temps[0], "last": temps[-1], "max": max(temps)}
        return out
