"""Timers: a CUDA-event timer over the launcher calls of a step, and a sampler of the GPU's clocks.

The section timer is the counterpart of the reference's backend profile sections
(crates/backend-hip/src/profile.rs:48-83): an event after every launcher call, read after the step."""
from __future__ import annotations

import statistics
import subprocess
import threading

import torch

from ..kernels import library


class SectionTimer:
    """with SectionTimer() as t: engine.step(...)   then t.sections() -> [(what, note, milliseconds)].

    An event is recorded after every launcher call; a section's time is the span between the event before it
    and its own.  Kernels that would overlap their neighbours' tails under programmatic dependent launch are
    kept apart by the events, so the times are those of serialised kernels: their shares are meaningful, their
    sum is a little above the step's own time.  Steps must run eagerly (no graph replay) to be seen."""

    def __init__(self):
        self.marks = []
        self.start = None

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()
        library.ON_LAUNCH[0] = self._on_launch
        return self

    def _on_launch(self, what, note):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append((what, note, ev))

    def __exit__(self, *exc):
        library.ON_LAUNCH[0] = None
        torch.cuda.synchronize()

    def sections(self) -> list:
        out, prev = [], self.start
        for what, note, ev in self.marks:
            out.append((what, note, prev.elapsed_time(ev)))
            prev = ev
        return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        mhz = [int(r[0]) for r in self.rows if r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}
