"""``bench.py --impl reference``: the unmodified reference, if it could be installed.

The reference tree has neither ``setup.py`` nor ``pyproject.toml``, so
``pip install --target baseline/_ref <reference>`` cannot produce an installation; its native
parts additionally need third-party sources that are not in the tree, a host-name allow-list and
an sm_86 CUDA arch list.  Until an installation exists under ``baseline/_ref`` this arm reports
itself unavailable and exits 0.
"""
from __future__ import annotations

import json
import os


def main(args) -> None:
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "baseline", "_ref")
    reason = ("pip install of the reference fails: the tree has no setup.py/pyproject.toml (not installable); "
              "its CMake build needs absent third-party sources, a host-name allow-list and sm_86")
    if os.path.isdir(root) and os.listdir(root):
        reason = "baseline/_ref exists but holds no runnable reference package"
    print(json.dumps({"impl": "reference", "unavailable": reason}), flush=True)
