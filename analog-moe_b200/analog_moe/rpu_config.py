"""Minimal configuration objects with the field names the analog sigma-MoE layers read.

The reference layers take an `aihwkit` / `aihwkit_lightning` `TorchInferenceRPUConfig`; those
packages are third-party.  The layer in this package only reads attributes, so a real
`TorchInferenceRPUConfig` works in place of these dataclasses; they exist so that the layer can
be built and tested without the third-party packages.  Field names and defaults follow what the
reference reads (moe_layer_aihwkit_lightning.py:152-181, 433-492, 524-525; the classic-aihwkit layer
additionally reads forward.{inp_bound, bound_management, is_perfect, noise_management},
mapping.max_output_size, modifier.per_batch_sample, remap.type and clip.fixed_value,
moe_layer_aihwkit.py:47-61, 163, 173, 244, 267, 324-333).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field


class WeightModifierType(enum.Enum):
    NONE = "None"
    COPY = "Copy"                    # classic aihwkit only: named by its layer, treated as NONE (moe_layer_aihwkit.py:166)
    MULT_NORMAL = "MultNormal"       # classic aihwkit only: rejected by its layer (:169-170)
    DISCRETIZE = "Discretize"
    DISCRETIZE_PER_CHANNEL = "DiscretizePerChannel"
    ADD_NORMAL = "AddNormal"
    ADD_NORMAL_PER_CHANNEL = "AddNormalPerChannel"
    DISCRETIZE_ADD_NORMAL = "DiscretizeAddNormal"
    DISCRETIZE_ADD_NORMAL_PER_CHANNEL = "DiscretizeAddNormalPerChannel"


class WeightClipType(enum.Enum):
    NONE = "None"
    FIXED_VALUE = "FixedValue"
    LAYER_GAUSSIAN = "LayerGaussian"
    LAYER_GAUSSIAN_PER_CHANNEL = "LayerGaussianPerChannel"
    AVERAGE_CHANNEL_MAX = "AverageChannelMax"


class WeightRemapType(enum.Enum):
    NONE = "None"
    LAYERWISE_SYMMETRIC = "LayerwiseSymmetric"
    CHANNELWISE_SYMMETRIC = "ChannelwiseSymmetric"


class BoundManagementType(enum.Enum):
    NONE = "None"
    ITERATIVE = "Iterative"


class NoiseManagementType(enum.Enum):
    NONE = "None"
    ABS_MAX = "AbsMax"


@dataclass
class IOParameters:
    inp_res: float = 254.0
    out_res: float = -1.0
    out_bound: float = -1.0
    out_noise: float = 0.0
    out_noise_per_channel: bool = True
    # classic-aihwkit fields
    inp_bound: float = 1.0
    bound_management: BoundManagementType = BoundManagementType.NONE
    noise_management: NoiseManagementType = NoiseManagementType.NONE


@dataclass
class AIHWKITIOParameters(IOParameters):
    """`forward` of a classic-aihwkit configuration: the presence of `is_perfect` is what CVMM.forward
    uses to tell the two parameter families apart (reference cvmm.py:727)."""
    is_perfect: bool = False


@dataclass
class InputRangeParameter:
    enable: bool = True
    learn_input_range: bool = True
    init_value: float = 3.0
    init_from_data: int = 0
    init_std_alpha: float = 3.0
    decay: float = 0.01
    input_min_percentage: float = 0.95


@dataclass
class PrePostProcessingParameter:
    input_range: InputRangeParameter = field(default_factory=InputRangeParameter)


@dataclass
class WeightModifierParameter:
    type: WeightModifierType = WeightModifierType.NONE
    res: float = 0.1
    std_dev: float = 0.0
    enable_during_test: bool = False
    per_batch_sample: bool = False


@dataclass
class WeightClipParameter:
    type: WeightClipType = WeightClipType.NONE
    sigma: float = 2.5
    fixed_value: float = -1.0


@dataclass
class WeightRemapParameter:
    type: WeightRemapType = WeightRemapType.CHANNELWISE_SYMMETRIC


@dataclass
class MappingParameter:
    max_input_size: int = -1
    max_output_size: int = -1


@dataclass
class TorchInferenceRPUConfig:
    forward: IOParameters = field(default_factory=IOParameters)
    pre_post: PrePostProcessingParameter = field(default_factory=PrePostProcessingParameter)
    modifier: WeightModifierParameter = field(default_factory=WeightModifierParameter)
    clip: WeightClipParameter = field(default_factory=WeightClipParameter)
    mapping: MappingParameter = field(default_factory=MappingParameter)
    remap: WeightRemapParameter = field(default_factory=WeightRemapParameter)


def aihwkit_rpu_config() -> TorchInferenceRPUConfig:
    """A configuration shaped like classic aihwkit's: `forward.is_perfect` exists, tile splitting is switched off
    with 0 instead of -1 (reference moe_layer_aihwkit.py:57-58)."""
    cfg = TorchInferenceRPUConfig(forward=AIHWKITIOParameters())
    cfg.mapping.max_input_size = 0
    cfg.mapping.max_output_size = 0
    return cfg
