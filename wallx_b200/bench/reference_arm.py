"""Reference arm of the benchmark: runs the unmodified reference package installed under
``baseline/_ref`` through its own public API, or reports why it cannot."""
from __future__ import annotations

import json
import os
import sys


def unavailable(reason: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": reason}), flush=True)


def main(args) -> None:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ref_dir = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "wall_x")):
        return unavailable("baseline/_ref/wall_x is not installed on this box")
    return unavailable("reference runner not wired yet")
