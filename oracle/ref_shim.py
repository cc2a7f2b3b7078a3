"""Import shim for a read-only checkout of the upstream D2DMoE code base.

TEST INFRASTRUCTURE ONLY.  This file never ships with the product path; it is
used by the golden-vector generator (tests/golden/make_golden.py) and by the
CPU tests that compare oracle/d2d_oracle.py with the real upstream modules
when a checkout is present.

The upstream package imports five third-party packages at module top
(utils.py:19-24, architectures/moe/moefication.py:7) that are not needed by
the MoE inference layer itself.  When they are missing this shim registers
empty stand-in modules for them so that
``architectures.moe.moefication`` / ``architectures.moe.moe_layers`` import.
No upstream source is copied: the modules are imported from the checkout.
"""
from __future__ import annotations

import importlib
import importlib.machinery
import os
import sys
import types
from pathlib import Path

_ENV = "D2DMOE_REFERENCE_ROOT"


def reference_root() -> Path | None:
    """Directory of the upstream checkout, or None when there is none.

    Order: the D2DMOE_REFERENCE_ROOT environment variable, then a directory
    named ``reference`` beside the repository root.
    """
    cand = []
    if os.environ.get(_ENV):
        cand.append(Path(os.environ[_ENV]))
    cand.append(Path(__file__).resolve().parents[2] / "reference")
    for c in cand:
        if (c / "architectures" / "moe" / "moefication.py").is_file():
            return c
    return None


def _stub(name: str, **attrs):
    if name in sys.modules:
        return sys.modules[name]
    try:
        if importlib.util.find_spec(name) is not None:
            return importlib.import_module(name)
    except (ImportError, ValueError):
        pass
    m = types.ModuleType(name)
    m.__spec__ = importlib.machinery.ModuleSpec(name, None)
    m.__path__ = []
    for k, v in attrs.items():
        setattr(m, k, v)
    sys.modules[name] = m
    return m


class _Anything:
    """Callable/constructible placeholder for names only used off the MoE path."""

    def __init__(self, *a, **k):
        pass

    def __call__(self, *a, **k):
        return self

    def __getattr__(self, item):
        return _Anything()


def _decorator_factory(*a, **k):
    def deco(fn):
        return fn
    return deco


_loaded = None


def load_reference():
    """Return a namespace with the upstream MoE classes, or None if no checkout.

    Attributes: MoeficationMoE, MoeficationRouter, CustomKernelExperts,
    ExecuteAllExperts, ModuleBatchedExperts, MOE_IMPL_MAP.
    """
    global _loaded
    if _loaded is not None:
        return _loaded
    root = reference_root()
    if root is None:
        return None
    # These must be imported before the stand-ins exist: transformers probes
    # optional packages with find_spec and a half-made module confuses it.
    import torch  # noqa: F401
    import torchvision  # noqa: F401
    import transformers  # noqa: F401
    try:
        import triton  # noqa: F401
    except ImportError:
        pass

    _stub("accelerate", Accelerator=_Anything, DistributedDataParallelKwargs=_Anything)
    _stub("accelerate.state", AcceleratorState=_Anything)
    _stub("accelerate.utils", PrepareForLaunch=_Anything, patch_environment=_Anything)
    _stub("fvcore")
    _stub("fvcore.nn", FlopCountAnalysis=_Anything, parameter_count=_Anything,
          flop_count_table=_Anything)
    _stub("fvcore.nn.jit_handles", elementwise_flop_counter=_decorator_factory,
          get_shape=_Anything)
    _stub("omegaconf", OmegaConf=_Anything)
    _stub("k_means_constrained", KMeansConstrained=_Anything)
    _stub("submitit")
    _stub("wandb")

    sys.path.insert(0, str(root))
    try:
        mf = importlib.import_module("architectures.moe.moefication")
        ml = importlib.import_module("architectures.moe.moe_layers")
    finally:
        # keep the path: upstream modules import lazily from each other
        pass
    ns = types.SimpleNamespace(
        root=root,
        MoeficationMoE=mf.MoeficationMoE,
        MoeficationRouter=mf.MoeficationRouter,
        CustomKernelExperts=ml.CustomKernelExperts,
        ExecuteAllExperts=ml.ExecuteAllExperts,
        ModuleBatchedExperts=ml.ModuleBatchedExperts,
        MOE_IMPL_MAP=ml.MOE_IMPL_MAP,
        moefication=mf,
        moe_layers=ml,
    )
    _loaded = ns
    return ns
