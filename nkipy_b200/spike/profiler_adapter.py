"""Per-call debug log around `Spike.execute` (spike/src/spike/profiler_adapter.py:18-78):
rank 0 appends PID / SOURCE / KERNEL records to ``debug_rank_0.txt``."""

from __future__ import annotations

import os
import traceback


class SpikeProfiler:
    def __init__(self, spike, log_dir: str = ".", rank: int = 0):
        self._spike = spike
        self.rank = rank
        self.path = os.path.join(log_dir, f"debug_rank_{rank}.txt")

    def execute(self, model, inputs, outputs, ntff_name: str = "", save_trace: bool = False):
        if self.rank == 0:
            frame = traceback.extract_stack(limit=3)[0]
            with open(self.path, "a") as f:
                f.write(f"PID {os.getpid()}\nSOURCE {frame.filename}:{frame.lineno}\nKERNEL {model.name} "
                        f"({model.neff_path})\n")
        return self._spike.execute(model, inputs, outputs, ntff_name, save_trace)

    def __getattr__(self, item):
        return getattr(self._spike, item)
