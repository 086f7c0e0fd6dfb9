"""Run-to-run determinism checks: the first run records named objects, later runs compare against the record.

Role of the reference's helpers (src/executable/test/test_utils.py: ``diff_objs``, ``diff_presampling``,
``diff_forward``, which pickle tensors under ``/tmp`` and raise on the first difference), as one small class with an
explicit directory instead of fixed temporary files.

    rec = RunRecorder(os.environ.get("RECSTORE_DETERMINISM_DIR"))     # None: every check is a no-op
    rec.diff_presampling(h, r, t, neg, rank, step)                    # the sampled ids of a step
    rec.diff_forward(rows, rank, step)                                # what the embedding lookup returned
"""
from __future__ import annotations

import os
from typing import Optional

import torch


class DeterminismError(AssertionError):
    pass


class RunRecorder:
    def __init__(self, directory: Optional[str], atol: float = 0.0):
        self.dir, self.atol = directory, atol
        self.recorded = self.compared = 0
        if directory:
            os.makedirs(directory, exist_ok=True)

    def diff_objs(self, obj, name: str) -> None:
        """Stores ``obj`` under ``name`` on the first run; on later runs raises ``DeterminismError`` if it differs."""
        if not self.dir:
            return
        path = os.path.join(self.dir, "".join(c if c.isalnum() or c in "-_." else "_" for c in name) + ".pt")
        new = obj.detach().cpu() if isinstance(obj, torch.Tensor) else obj
        if not os.path.exists(path):
            torch.save(new, path)
            self.recorded += 1
            return
        old = torch.load(path, weights_only=False)
        self.compared += 1
        if isinstance(old, torch.Tensor):
            same = isinstance(new, torch.Tensor) and old.shape == new.shape and (
                torch.equal(old, new) if self.atol == 0.0 else torch.allclose(old.float(), new.float(), atol=self.atol, rtol=0.0))
        else:
            same = old == new
        if not same:
            raise DeterminismError(f"{name}: differs from the recorded run in {self.dir}")

    def diff_presampling(self, h, r, t, neg, rank: int, step: int, corrupt_head: Optional[bool] = None) -> None:
        for nm, x in (("h", h), ("r", r), ("t", t), ("neg", neg)):
            self.diff_objs(x, f"sample-{nm}-{rank}-{step}")
        if corrupt_head is not None:
            self.diff_objs(bool(corrupt_head), f"sample-side-{rank}-{step}")

    def diff_forward(self, rows, rank: int, step: int) -> None:
        self.diff_objs(rows, f"forward-{rank}-{step}")
