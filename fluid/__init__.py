"""Compatibility package: the import paths of the reference framework (``fluid``, ``fluid.core``,
``fluid.moe``, ``fluid.attention``, ``fluid.layer``, ``fluid.setup``, ``fluid.distributed``,
``fluid.csrc``) resolve to the implementation in :mod:`fluidmoe_b200`."""
import sys as _sys
import types as _types

import fluidmoe_b200 as _f
from fluidmoe_b200 import *  # noqa: F401,F403
from fluidmoe_b200 import (_all_to_all, _all_to_all_hp2sp_forward, _all_to_all_sp2hp_forward,  # noqa: F401
                           distributed)
from fluidmoe_b200.models import attention as _attention, moe as _moe, transformer as _layer, megatron_spec as _spec
from fluidmoe_b200.parallel import comm as _comm, ddp as _ddp, p2p_backend as _p2p, schedule as _schedule
from fluidmoe_b200.parallel import scheduler as _scheduler, shmem_compat as _shmem, streams as _streams, symm as _symm
from fluidmoe_b200.ops import compat as _te_ops
from fluidmoe_b200.utils import nvtx as _nvtx, overhead_profiler as _ohp, python_profile as _pyprof

__version__ = "1.0.0"


def _module(name, *sources):
    m = _types.ModuleType(name)
    for src in sources:
        for k, v in vars(src).items():
            if not k.startswith("__"):
                setattr(m, k, v)
    _sys.modules[name] = m
    return m


core = _module("fluid.core", _comm, _schedule, _scheduler, _p2p, _nvtx)
core.comm = _module("fluid.core.comm", _comm, _schedule)
core.scheduler = _module("fluid.core.scheduler", _scheduler)
core.stream = _module("fluid.core.stream", _streams)
core.p2p_backend = _module("fluid.core.p2p_backend", _p2p)
core.nvtx = _module("fluid.core.nvtx", _nvtx)
core.nvtx.NVTX_ENABLED = _nvtx.ENABLED
core.NVTX_ENABLED = _nvtx.ENABLED
core.overhead_profiler = _module("fluid.core.overhead_profiler", _ohp)
core.python_profile = _module("fluid.core.python_profile", _pyprof)
core.te_ops = _module("fluid.core.te_ops", _te_ops)
moe = _module("fluid.moe", _moe)
moe.forward = _module("fluid.moe.forward", _moe)
moe.backward = _module("fluid.moe.backward", _moe)
for _n in ("grouped_fc1_act", "grouped_fc2", "grouped_fc2_dx", "grouped_fc1_dx"):
    setattr(moe, _n, getattr(_f, _n))
    setattr(moe.forward if _n in ("grouped_fc1_act", "grouped_fc2") else moe.backward, _n, getattr(_f, _n))
attention = _module("fluid.attention", _attention)
attention.forward = _module("fluid.attention.forward", _attention)
attention.backward = _module("fluid.attention.backward", _attention)
layer = _module("fluid.layer", _layer, _spec)
layer.transformer = _module("fluid.layer.transformer", _layer)
layer.fluid_spec = _module("fluid.layer.fluid_spec", _spec)


def _lazy_layer_class(name):
    # the Megatron module class exists only where megatron-core is installed
    if name == "FluidTransformerLayer":
        return _spec.build_fluid_transformer_layer_class()
    raise AttributeError(name)


layer.fluid_spec.__getattr__ = _lazy_layer_class
setup = _module("fluid.setup", _ddp)
csrc = _module("fluid.csrc", _symm, _shmem)
_sys.modules["fluid.distributed"] = distributed

# Export list: every public name of the implementation package plus the three underscore-prefixed
# all-to-all primitives that the reference exports by name (fluid/__init__.py:90-131).
__all__ = sorted({_k for _k in vars(_f) if not _k.startswith("_") and not isinstance(getattr(_f, _k), _types.ModuleType)}
                 | {"_all_to_all", "_all_to_all_sp2hp_forward", "_all_to_all_hp2sp_forward"})
