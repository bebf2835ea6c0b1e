"""Minimal configuration objects with the field names the analog sigma-MoE layers read.

The reference layers take an `aihwkit` / `aihwkit_lightning` `TorchInferenceRPUConfig`; those
packages are third-party.  The layer in this package only reads attributes, so a real
`TorchInferenceRPUConfig` works in place of these dataclasses; they exist so that the layer can
be built and tested without the third-party packages.  Field names and defaults follow what the
reference reads (moe_layer_aihwkit_lightning.py:152-181, 433-492, 524-525).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field


class WeightModifierType(enum.Enum):
    NONE = "None"
    DISCRETIZE = "Discretize"
    DISCRETIZE_PER_CHANNEL = "DiscretizePerChannel"
    ADD_NORMAL = "AddNormal"
    ADD_NORMAL_PER_CHANNEL = "AddNormalPerChannel"
    DISCRETIZE_ADD_NORMAL = "DiscretizeAddNormal"
    DISCRETIZE_ADD_NORMAL_PER_CHANNEL = "DiscretizeAddNormalPerChannel"


class WeightClipType(enum.Enum):
    NONE = "None"
    LAYER_GAUSSIAN = "LayerGaussian"
    LAYER_GAUSSIAN_PER_CHANNEL = "LayerGaussianPerChannel"


@dataclass
class IOParameters:
    inp_res: float = 254.0
    out_res: float = -1.0
    out_bound: float = -1.0
    out_noise: float = 0.0
    out_noise_per_channel: bool = True


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


@dataclass
class WeightClipParameter:
    type: WeightClipType = WeightClipType.NONE
    sigma: float = 2.5


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
