"""``import mccl`` — the name users of the reference package import.

Everything lives in :mod:`mccl_b200`; this module re-exports it and aliases the
sub-modules so that ``mccl.config``, ``mccl.tuning``, ``mccl.distributed`` and
``mccl._C`` resolve as they do in the reference layout.
"""
import importlib
import sys

import mccl_b200 as _impl
from mccl_b200 import *  # noqa: F401,F403
from mccl_b200 import _C, __version__, __protocol_version__  # noqa: F401

for _name in ("_backend", "config", "tuning", "version", "metrics", "check", "cli", "distributed", "parallel", "models",
              "ops", "utils"):
    sys.modules[__name__ + "." + _name] = importlib.import_module("mccl_b200." + _name)
    globals()[_name] = sys.modules[__name__ + "." + _name]
# short names for the parallelism modules
for _name, _target in (("ddp", "parallel.ddp"), ("tp", "parallel.tp"), ("pp", "parallel.pp"), ("trainer", "parallel.trainer")):
    sys.modules[__name__ + "." + _name] = importlib.import_module("mccl_b200." + _target)
    globals()[_name] = sys.modules[__name__ + "." + _name]
sys.modules[__name__ + "._C"] = _C
