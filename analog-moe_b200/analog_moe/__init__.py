"""B200-native analog sigma-MoE hot path: hand-written sm_100a CUDA kernels behind the
reference's `analog_moe.triton_src` Python boundary."""
from .triton_src import CVMM, CVMMSel, CVMMExt, PhiloxNoise, WeightModifier, cvmm_prepare_sel, cvmm_std  # noqa: F401
from .layers import (AnalogSigmaMoELayer, AnalogSigmaMoELayerAIHWKIT, AnalogSigmaMoELayerAIHWKITLightning,  # noqa: F401
                     MoEConifgError, SigmaMoELayer, non_traceable_to_traceable, traceable_to_non_traceable)
from .rpu_config import (TorchInferenceRPUConfig, WeightModifierType, WeightClipType, WeightRemapType,  # noqa: F401
                         BoundManagementType, NoiseManagementType, aihwkit_rpu_config)
