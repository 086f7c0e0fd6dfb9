"""Experiment harness: grids of configurations, one log directory per run, completion markers, box locks."""
from .harness import Experiment, RunResult, box_lock, expand_grid, log_succeeded  # noqa: F401
