"""mccl_b200: a Blackwell-native ``torch.distributed`` backend.

``import mccl_b200`` (or ``import mccl``) registers the backend, so

    dist.init_process_group(backend="mccl", ...)

works unchanged under torchrun / DDP, as with the reference package
(mccl/__init__.py:9-45).  CUDA tensors move over NVLink through hand-written
sm_100a kernels; CPU tensors move over a TCP mesh, so the whole API can be
exercised on a machine without a GPU.
"""
from __future__ import annotations

import os
import warnings

import torch  # the extension links against libtorch: import it first

from .version import COMPATIBILITY_MATRIX, __protocol_version__, __version__


def _load_native():
    here = os.path.dirname(os.path.abspath(__file__))
    so = os.path.join(here, "_C.so")
    if not os.path.exists(so):
        raise ImportError(
            "mccl_b200: the native extension mccl_b200/_C.so is missing. Build it with "
            "`python -c 'import __graft_entry__ as g; g.build()'` or `python -m mccl_b200._build` "
            "from the repository root (nvcc for sm_100a is required; no GPU is needed to build)."
        )
    from . import _C as native
    return native


_C = _load_native()


def _check_platform() -> None:
    """Warns (never fails) when CUDA collectives cannot run here; CPU tensors still work."""
    if not torch.cuda.is_available():
        return
    try:
        major, minor = torch.cuda.get_device_capability(0)
    except Exception:
        return
    if (major, minor) != (10, 0):
        warnings.warn(
            f"mccl_b200 kernels are built for sm_100a (B200); this GPU reports sm_{major}{minor}. "
            "CUDA collectives will fail to launch; CPU tensors are unaffected.",
            RuntimeWarning,
        )


_check_platform()

from ._backend import get_backend, register, set_iface_priority  # noqa: E402
from .config import DistroConfig  # noqa: E402
from .metrics import get_metrics, log_metrics, metrics_history, reset_metrics  # noqa: E402
from .tuning import apply_nvlink_production_defaults, apply_thunderbolt_production_defaults  # noqa: E402

register()

__all__ = [
    "__version__", "__protocol_version__", "COMPATIBILITY_MATRIX", "DistroConfig", "set_iface_priority",
    "register", "get_backend", "get_metrics", "reset_metrics", "log_metrics", "metrics_history",
    "apply_nvlink_production_defaults", "apply_thunderbolt_production_defaults",
]
