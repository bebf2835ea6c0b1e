"""Stand-ins for the third-party packages the reference's layer files import (`sigma_moe`, `aihwkit_lightning`,
`aihwkit`), so that those files can be imported UNCHANGED on top of this repository's `analog_moe.triton_src`.

Only what the layer files touch exists: the sigma-MoE base class (this package's own, written from the contract the
reference layers rely on), configuration dataclasses and enums with the reference's field names, an
`AnalogLayerBase` that does nothing, `convert_to_analog` that leaves the router Linear digital, a straight-through
`UniformQuantize`, and an `AnalogContext` placeholder.  Test infrastructure only.
"""
import importlib.util
import os
import sys
import types

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_PKG = os.path.join(ROOT, "baseline", "_ref", "analog_moe")


def reference_available() -> bool:
    return os.path.exists(os.path.join(REF_PKG, "moe_layer_aihwkit_lightning.py"))


def _module(name: str, **attrs) -> types.ModuleType:
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    parent, _, leaf = name.rpartition(".")
    if parent:
        if parent not in sys.modules:
            _module(parent)
        setattr(sys.modules[parent], leaf, m)
    return m


class _UniformQuantize(torch.autograd.Function):
    """round(w / res) * res with a straight-through gradient (what the DISCRETIZE modifiers apply)."""

    @staticmethod
    def forward(ctx, w, res, bound, inplace):
        return torch.round(w / res) * res

    @staticmethod
    def backward(ctx, g):
        return g, None, None, None


def install() -> None:
    """Registers the stand-in modules (idempotent)."""
    if "sigma_moe.moe_layer" in sys.modules and getattr(sys.modules["sigma_moe"], "_amoe_standin", False):
        return
    import analog_moe
    from analog_moe import rpu_config as R

    _module("sigma_moe", _amoe_standin=True)
    _module("sigma_moe.moe_layer", SigmaMoELayer=analog_moe.SigmaMoELayer)

    class AnalogLayerBase:
        def __init__(self, *a, **k):
            pass

    class ConfigError(Exception):
        pass

    def convert_to_analog(module, rpu_config=None, inplace=False, ensure_analog_root=False, **kw):
        return module        # the router stays a digital Linear in these tests

    _module("aihwkit_lightning.nn.modules.base", AnalogLayerBase=AnalogLayerBase)
    _module("aihwkit_lightning.simulator.configs.configs", TorchInferenceRPUConfig=R.TorchInferenceRPUConfig)
    _module("aihwkit_lightning.exceptions", ConfigError=ConfigError)
    _module("aihwkit_lightning.simulator.parameters.enums", WeightModifierType=R.WeightModifierType,
            WeightClipType=R.WeightClipType)
    _module("aihwkit_lightning.simulator.parameters", WeightModifierParameter=R.WeightModifierParameter)
    sys.modules["aihwkit_lightning.simulator.parameters"].enums = sys.modules["aihwkit_lightning.simulator.parameters.enums"]
    _module("aihwkit_lightning.nn.modules.torch_utils.torch_linear", UniformQuantize=_UniformQuantize)
    _module("aihwkit_lightning.nn.conversion", convert_to_analog=convert_to_analog)

    class AnalogContext(torch.nn.Parameter):
        def __new__(cls, layer):
            return torch.nn.Parameter.__new__(cls, torch.zeros(()), requires_grad=False)

        def __init__(self, layer):
            self.use_torch_update = True

    class RPUConfigBase:
        pass

    _module("aihwkit.nn.modules.base", AnalogLayerBase=AnalogLayerBase)
    _module("aihwkit.simulator.configs.configs", TorchInferenceRPUConfig=R.TorchInferenceRPUConfig)
    _module("aihwkit.simulator.parameters.base", RPUConfigBase=RPUConfigBase)
    _module("aihwkit.optim.context", AnalogContext=AnalogContext)
    _module("aihwkit.simulator.parameters.enums", WeightModifierType=R.WeightModifierType, WeightClipType=R.WeightClipType,
            WeightRemapType=R.WeightRemapType, BoundManagementType=R.BoundManagementType,
            NoiseManagementType=R.NoiseManagementType)
    _module("aihwkit.simulator.parameters", WeightModifierParameter=R.WeightModifierParameter,
            WeightClipParameter=R.WeightClipParameter)
    sys.modules["aihwkit.simulator.parameters"].enums = sys.modules["aihwkit.simulator.parameters.enums"]
    sys.modules["aihwkit.simulator.parameters"].base = sys.modules["aihwkit.simulator.parameters.base"]


def load_reference_layer_module(filename: str):
    """Imports baseline/_ref/analog_moe/<filename> as a submodule of THIS repository's `analog_moe` package, so that its
    `from .triton_src.cvmm import CVMM, CVMMSel, cvmm_std` binds to the CUDA library's wrappers: the layer file is the
    reference's, byte for byte; only `triton_src` underneath it is replaced."""
    install()
    import analog_moe  # noqa: F401
    name = "analog_moe._reference_" + filename[:-3]
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF_PKG, filename))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod
