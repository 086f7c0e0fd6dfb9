"""Optional profilers around a few training steps, as switches of the drivers.

The reference wraps warm-up + 2-3 steps in ``torch.profiler`` and writes a chrome trace (src/executable/perf_emb.py:
275-352, dgl-ke train_pytorch.py:185-236), prints ``autograd.profiler`` tables in the DLRM driver
(dlrm_model.py:1094-1096, 1320-1332) and can run under pyinstrument.  ``StepProfiler`` is that hook for the drivers
here: give it a directory and call ``step()`` once per training step; it records ``active`` steps after ``skip``
steps, writes ``trace_rank{r}.json`` (chrome://tracing / Perfetto) and ``ops_rank{r}.txt`` (time per operator), and is
inert when no directory is given.  Numbers read from a profiled run are for finding where time goes; throughput is
never reported from one.
"""
from __future__ import annotations

import os
from typing import Optional

import torch


class StepProfiler:
    def __init__(self, out_dir: Optional[str], rank: int = 0, skip: int = 3, active: int = 3, with_stack: bool = False,
                 record_shapes: bool = False):
        self.out_dir, self.rank, self.skip, self.active = out_dir, rank, int(skip), int(active)
        self._with_stack, self._record_shapes = with_stack, record_shapes
        self._prof = None
        self._n = 0
        self.done = out_dir is None
        self.trace_file = self.table_file = None

    @property
    def enabled(self) -> bool:
        return self.out_dir is not None

    def step(self) -> None:
        """Call once per training step, after the step's work has been issued."""
        if self.done:
            return
        self._n += 1
        if self._n == self.skip:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._prof = torch.profiler.profile(activities=acts, with_stack=self._with_stack, record_shapes=self._record_shapes)
            self._prof.__enter__()
        elif self._n == self.skip + self.active:
            self.finish()

    def finish(self) -> None:
        """Stops an open recording and writes the files (also called by ``step`` when the window is over)."""
        if self._prof is None:
            self.done = True
            return
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self._prof.__exit__(None, None, None)
        os.makedirs(self.out_dir, exist_ok=True)
        self.trace_file = os.path.join(self.out_dir, f"trace_rank{self.rank}.json")
        self.table_file = os.path.join(self.out_dir, f"ops_rank{self.rank}.txt")
        self._prof.export_chrome_trace(self.trace_file)
        sort = "cuda_time_total" if torch.cuda.is_available() else "cpu_time_total"
        with open(self.table_file, "w") as f:
            f.write(self._prof.key_averages().table(sort_by=sort, row_limit=40))
        self._prof = None
        self.done = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.finish()
