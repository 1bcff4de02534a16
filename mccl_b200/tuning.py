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


def apply_nvlink_production_defaults(training_defaults: bool = False, world: Optional[int] = None) -> Dict[str, str]:
    """Sets defaults tuned for one NVSwitch box; existing variables win.  With ``world`` (or ``WORLD_SIZE`` in the
    environment) the measured crossovers of that world size are exported."""
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
    if world is None and os.environ.get("WORLD_SIZE", "").isdigit():
        world = int(os.environ["WORLD_SIZE"])
    table = load_tuning_table()
    picked = defaults_for_world(world) if (world and table) else ({"tree_below": int(table["tree_below"])} if table and "tree_below" in table else {})
    if picked.get("tree_below") and "MCCL_TREE_BELOW" not in os.environ:
        os.environ["MCCL_TREE_BELOW"] = str(picked["tree_below"])
        applied["MCCL_TREE_BELOW"] = os.environ["MCCL_TREE_BELOW"]
    if picked.get("push_above") and "MCCL_PUSH_ABOVE" not in os.environ:
        os.environ["MCCL_PUSH_ABOVE"] = str(picked["push_above"])
        applied["MCCL_PUSH_ABOVE"] = os.environ["MCCL_PUSH_ABOVE"]
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


def policy_from_sweep(rows: List[dict]) -> List[dict]:
    """Fastest schedule per message size, from sweep rows ``{"bytes", "algo", "us"}``: a list of
    ``{"up_to": bytes, "algo": name}`` steps in increasing size (the last step covers everything larger)."""
    by_size: Dict[int, Dict[str, float]] = {}
    for r in rows:
        by_size.setdefault(int(r["bytes"]), {})[r["algo"]] = float(r["us"])
    steps: List[dict] = []
    for size in sorted(by_size):
        algo = min(by_size[size], key=by_size[size].get)
        if steps and steps[-1]["algo"] == algo:
            steps[-1]["up_to"] = size
        else:
            steps.append({"up_to": size, "algo": algo})
    return steps


def push_above_from_sweep(rows: List[dict]) -> int:
    """Smallest message size from which the fully pushed two-shot stays ahead of the plain two-shot (0: never)."""
    by_size: Dict[int, Dict[str, float]] = {}
    for r in rows:
        by_size.setdefault(int(r["bytes"]), {})[r["algo"]] = float(r["us"])
    above = 0
    for size in sorted(by_size, reverse=True):
        t = by_size[size]
        if "twoshot_push" in t and "twoshot" in t and t["twoshot_push"] < 0.97 * t["twoshot"]:
            above = size
        else:
            break
    return above


def save_tuning_table(rows: List[dict], world: int, path: Optional[str] = None) -> str:
    """Writes (or extends) the table: one entry per world size under "worlds", the newest world also at the top
    level (``tree_below`` is what ``apply_nvlink_production_defaults`` exports as ``MCCL_TREE_BELOW``)."""
    path = path or os.environ.get("MCCL_TUNING_FILE") or _DEFAULT_TABLE
    old = {}
    if os.path.exists(path):
        try:
            with open(path) as f:
                old = json.load(f)
        except Exception:  # noqa: BLE001
            old = {}
    worlds = old.get("worlds", {})
    if "world" in old and str(old["world"]) not in worlds and "tree_below" in old:
        worlds[str(old["world"])] = {"tree_below": old["tree_below"], "push_above": old.get("push_above", 0),
                                     "policy": old.get("policy", [])}
    entry = {"tree_below": crossover_from_sweep(rows), "push_above": push_above_from_sweep(rows), "policy": policy_from_sweep(rows)}
    worlds[str(world)] = entry
    table = {"world": world, **entry, "worlds": worlds, "rows": rows}
    with open(path, "w") as f:
        json.dump(table, f, indent=1)
    return path


def defaults_for_world(world: int, path: Optional[str] = None) -> Dict[str, int]:
    """``{"tree_below", "push_above"}`` measured for this world size (nearest measured size when it is missing)."""
    table = load_tuning_table(path) or {}
    worlds = table.get("worlds") or ({str(table["world"]): table} if "world" in table else {})
    if not worlds:
        return {}
    key = min(worlds, key=lambda w: abs(int(w) - world))
    e = worlds[key]
    return {"tree_below": int(e.get("tree_below", 0)), "push_above": int(e.get("push_above", 0))}
