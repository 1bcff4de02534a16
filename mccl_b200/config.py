"""One dataclass with every tunable, mirrored to environment variables.

Parity: the reference's ``DistroConfig`` (mccl/config.py:12-95) carries
node_id, num_nodes, control_port, chunk_bytes, cq_depth, connect_timeout_ms,
fast_math, shader_path, max_queue_depth and log_level, each mapped to a
``DISTRO_*`` variable, with ``from_env`` / ``from_dict`` / ``to_env`` /
``to_dict`` and range validation.  Those fields and names are kept; the
fields added here map to the ``MCCL_*`` variables the native code reads.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Any, Dict

_ENV_MAP: Dict[str, str] = {
    # reference names
    "DISTRO_NODE_ID": "node_id",
    "DISTRO_NUM_NODES": "num_nodes",
    "DISTRO_CONTROL_PORT": "control_port",
    "DISTRO_CHUNK_BYTES": "chunk_bytes",
    "DISTRO_CQ_DEPTH": "cq_depth",
    "DISTRO_CONNECT_TIMEOUT_MS": "connect_timeout_ms",
    "DISTRO_FAST_MATH": "fast_math",
    "DISTRO_SHADER_PATH": "shader_path",
    "DISTRO_MAX_QUEUE_DEPTH": "max_queue_depth",
    "DISTRO_LOG_LEVEL": "log_level",
    # names read by the native backend
    "MCCL_ALLREDUCE_ALGO": "allreduce_algo",
    "MCCL_TREE_BELOW": "tree_below",
    "MCCL_WIRE_DTYPE": "wire_dtype",
    "MCCL_NVLS": "nvls",
    "MCCL_ARENA_MB": "arena_mb",
    "MCCL_DEVICE_TIMEOUT_MS": "device_timeout_ms",
    "MCCL_TUNING_FILE": "tuning_file",
    "MCCL_BLOCKING_WAIT": "blocking_wait",
    "MCCL_MAX_CTAS": "max_ctas",
    "MCCL_SYMM_MODE": "symm_mode",
}

_ALGOS = ("auto", "ring", "tree", "butterfly", "twoshot", "oneshot", "nvls")


@dataclasses.dataclass
class DistroConfig:
    """All tunables in one place."""

    # cluster
    node_id: int = 0
    num_nodes: int = 1
    control_port: int = 29600
    # distributed memory
    chunk_bytes: int = 1 * 1024 * 1024
    cq_depth: int = 256
    connect_timeout_ms: int = 30000
    # compute
    fast_math: bool = True
    shader_path: str = ""          # kept for API parity; kernels are precompiled
    # runtime
    max_queue_depth: int = 1024
    log_level: str = "WARN"
    # collectives
    allreduce_algo: str = "auto"
    tree_below: int = 262144
    wire_dtype: str = ""           # "" (native) or "bf16"
    nvls: str = "auto"             # "auto" | "0" | "1"
    arena_mb: int = 512
    device_timeout_ms: int = 10000
    tuning_file: str = ""
    blocking_wait: bool = False
    max_ctas: int = 0
    symm_mode: str = "auto"        # "auto" | "vmm" | "ipc"

    def __post_init__(self) -> None:
        self._validate()

    def _validate(self) -> None:
        if self.node_id < 0:
            raise ValueError(f"node_id must be >= 0, got {self.node_id}")
        if self.num_nodes < 1:
            raise ValueError(f"num_nodes must be >= 1, got {self.num_nodes}")
        if self.chunk_bytes < 1:
            raise ValueError(f"chunk_bytes must be >= 1, got {self.chunk_bytes}")
        if self.allreduce_algo not in _ALGOS:
            raise ValueError(f"allreduce_algo must be one of {_ALGOS}, got {self.allreduce_algo!r}")
        if self.wire_dtype not in ("", "bf16"):
            raise ValueError(f"wire_dtype must be '' or 'bf16', got {self.wire_dtype!r}")
        if self.arena_mb < 2:
            raise ValueError(f"arena_mb must be >= 2, got {self.arena_mb}")
        if self.tree_below < 0:
            raise ValueError(f"tree_below must be >= 0, got {self.tree_below}")

    @classmethod
    def from_env(cls) -> "DistroConfig":
        cfg = cls()
        types = {f.name: f.type for f in dataclasses.fields(cls)}
        for env_key, name in _ENV_MAP.items():
            raw = os.environ.get(env_key)
            if raw is None:
                continue
            setattr(cfg, name, _coerce(raw, types[name]))
        cfg._validate()
        return cfg

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DistroConfig":
        known = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in known})

    def to_env(self) -> Dict[str, str]:
        """Exports every non-empty field to ``os.environ`` and returns what was set."""
        out: Dict[str, str] = {}
        for env_key, name in _ENV_MAP.items():
            val = getattr(self, name)
            s = ("1" if val else "0") if isinstance(val, bool) else str(val)
            if s != "":
                os.environ[env_key] = s
                out[env_key] = s
        return out

    def to_dict(self) -> Dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in dataclasses.fields(self)}


def _coerce(raw: str, target: Any) -> Any:
    if target in (bool, "bool"):
        return raw not in ("0", "false", "FALSE", "no", "NO", "")
    if target in (int, "int"):
        return int(raw)
    if target in (float, "float"):
        return float(raw)
    return raw
