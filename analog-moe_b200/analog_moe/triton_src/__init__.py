from .cvmm import CVMM, CVMMSel, CVMMExt, PhiloxNoise, WeightModifier, cvmm_prepare_sel, cvmm_std  # noqa: F401
