"""Production defaults and the measured algorithm-selection table.

Parity: the reference's ``apply_thunderbolt_production_defaults`` sets link
profile, overlap and DDP bucket defaults without overriding what the user
already exported (mccl/tuning.py:9-28).  ``apply_nvlink_production_defaults``
is the NVLink counterpart; the old name is kept as an alias.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

_DEFAULT_TABLE = os.path.join(os.path.dirname(__file__), "tuning_table.json")


def apply_nvlink_production_defaults(training_defaults: bool = False) -> Dict[str, str]:
    """Sets defaults tuned for one NVSwitch box; existing variables win."""
    wanted = {
        "MCCL_LINK_PROFILE": "nvlink5",
        "MCCL_OVERLAP_COMM": "1",
        "MCCL_ALLREDUCE_ALGO": "auto",
    }
    if training_defaults:
        wanted["DDP_BUCKET_MB"] = "25"
        wanted["MCCL_WIRE_DTYPE"] = "bf16"
    applied = {}
    for k, v in wanted.items():
        if k not in os.environ:
            os.environ[k] = v
            applied[k] = v
    table = load_tuning_table()
    if table and "tree_below" in table and "MCCL_TREE_BELOW" not in os.environ:
        os.environ["MCCL_TREE_BELOW"] = str(int(table["tree_below"]))
        applied["MCCL_TREE_BELOW"] = os.environ["MCCL_TREE_BELOW"]
    return applied


# Name used by scripts written against the reference.
apply_thunderbolt_production_defaults = apply_nvlink_production_defaults


def load_tuning_table(path: Optional[str] = None) -> Optional[dict]:
    """Loads the JSON written by ``mccl tune`` (``MCCL_TUNING_FILE`` or the packaged default)."""
    path = path or os.environ.get("MCCL_TUNING_FILE") or _DEFAULT_TABLE
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f)


def crossover_from_sweep(rows: List[dict]) -> int:
    """Largest message size (bytes) at which one-shot is still at least as fast as the
    best bandwidth schedule, from sweep rows ``{"bytes", "algo", "us"}``."""
    by_size: Dict[int, Dict[str, float]] = {}
    for r in rows:
        by_size.setdefault(int(r["bytes"]), {})[r["algo"]] = float(r["us"])
    best = 0
    for size in sorted(by_size):
        t = by_size[size]
        if "oneshot" not in t:
            continue
        others = [v for k, v in t.items() if k != "oneshot"]
        # a tie within 3 % is noise; the crossover is the largest size at which one-shot still holds up
        if not others or t["oneshot"] <= 1.03 * min(others):
            best = size
    return best


def save_tuning_table(rows: List[dict], world: int, path: Optional[str] = None) -> str:
    path = path or os.environ.get("MCCL_TUNING_FILE") or _DEFAULT_TABLE
    table = {"world": world, "tree_below": crossover_from_sweep(rows), "rows": rows}
    with open(path, "w") as f:
        json.dump(table, f, indent=1)
    return path
