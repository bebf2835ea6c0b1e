"""ctypes binding of libamoe_b200.so (the C ABI declared in include/amoe.h).

There is no fallback: if the shared library is missing the import fails with instructions to
build it, and every compute call raises unless the tensors live on a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import _build

F32, BF16, F16 = 0, 1, 2
PREC_BF16X1, PREC_SPLIT, PREC_FP32_SIMT, PREC_F16X1 = 0, 1, 2, 3
PRECISION_NAMES = {"bf16": PREC_BF16X1, "bf16x1": PREC_BF16X1, "split": PREC_SPLIT, "fp32": PREC_FP32_SIMT,
                   "simt": PREC_FP32_SIMT, "f16": PREC_F16X1, "f16x1": PREC_F16X1, "fp16": PREC_F16X1}

c_i32p = C.c_void_p
vp = C.c_void_p


class AmoeError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = _lib.amoe_status_string(status).decode()
        detail = _lib.amoe_last_error_string().decode()
        super().__init__(f"{where}: amoe status {status} ({msg})" + (f" [{detail}]" if detail and status == 5 else ""))


class WeightPrepassArgs(C.Structure):
    _fields_ = [
        ("w", vp), ("w_dtype", C.c_int32), ("E", C.c_int32), ("K", C.c_int32), ("N", C.c_int32),
        ("w_stride_e", C.c_int64), ("w_stride_k", C.c_int64), ("w_stride_n", C.c_int64),
        ("per_channel_scale", C.c_int32), ("noise_std", C.c_float), ("noise_per_channel", C.c_int32),
        ("discretize_res", C.c_float), ("seed", C.c_uint64), ("offset", C.c_uint32), ("step_dev", vp),
        ("col_scale", vp), ("col_inv_scale", vp), ("w_out", vp), ("fwd_hi", vp), ("fwd_lo", vp), ("bwd_hi", vp), ("bwd_lo", vp),
        ("workspace", vp), ("workspace_bytes", C.c_size_t),
        ("clip_sigma", C.c_float), ("clip_per_channel", C.c_int32), ("clip_fixed", C.c_float), ("w_clip_out", vp),
        ("expert_base", C.c_int32), ("prepared_f16", C.c_int32),
    ]


class OperandTilesArgs(C.Structure):
    _fields_ = [
        ("P", C.c_int64), ("E", C.c_int32), ("K", C.c_int32), ("precision", C.c_int32),
        ("expert_offsets", vp),
        ("a", vp), ("a_dtype", C.c_int32), ("a_stride", C.c_int64), ("a_rows", C.c_int64),
        ("a_row", vp), ("a_row_div", C.c_int32),
        ("dac", C.c_int32),
        ("ir", vp), ("ir_by_expert", C.c_int32), ("a_absmax", vp), ("inp_res", C.c_float),
        ("tile_hi", vp), ("tile_lo", vp),
        ("cache_hi", vp), ("cache_lo", vp), ("cache_scale", vp),
        ("cache_rows", C.c_int64),
        ("g_absmax_dev", vp),
        ("dev_status", vp),
        ("a_row_absmax", vp),
    ]


class CvmmArgs(C.Structure):
    _fields_ = [
        ("P", C.c_int64), ("E", C.c_int32), ("K", C.c_int32), ("N", C.c_int32), ("precision", C.c_int32),
        ("expert_offsets", vp),
        ("a", vp), ("a_dtype", C.c_int32), ("a_stride", C.c_int64), ("a_rows", C.c_int64),
        ("a_row", vp), ("a_row_div", C.c_int32), ("dst_row", vp), ("dst_rows", C.c_int64),
        ("w", vp), ("w_dtype", C.c_int32), ("w_stride_e", C.c_int64), ("w_stride_k", C.c_int64),
        ("w_stride_n", C.c_int64), ("w_hi", vp), ("w_lo", vp),
        ("ir", vp), ("ir_by_expert", C.c_int32), ("a_absmax", vp), ("inp_res", C.c_float),
        ("noise", vp), ("noise_std", C.c_float), ("seed", C.c_uint64), ("offset", C.c_uint32), ("step_dev", vp),
        ("col_scale", vp),
        ("col_inv_scale", vp), ("out_res", C.c_float), ("out_bound", C.c_float),
        ("out", vp), ("out_dtype", C.c_int32), ("out_stride", C.c_int64), ("out_codes", vp),
        ("out_row_scale", vp), ("out_row_expert", vp), ("out_relu", C.c_int32),
        ("x_ref", vp), ("x_ref_dtype", C.c_int32), ("x_ref_stride", C.c_int64), ("x_ref_rows", C.c_int64),
        ("x_ref_row", vp), ("x_ref_relu", C.c_int32),
        ("row_scale", vp), ("ir_grad", vp), ("ir_grad_relative", C.c_int32), ("ir_grad_scale", C.c_float),
        ("keep_count", vp),
        ("a_cache_hi", vp), ("a_cache_lo", vp), ("a_cache_scale", vp), ("out_cache_hi", vp), ("out_cache_lo", vp), ("cache_rows", C.c_int64),
        ("a_tile_hi", vp), ("a_tile_lo", vp),
        ("next_ir", vp), ("next_inp_res", C.c_float), ("next_codes", vp), ("out_cache_scale", vp),
        ("workspace", vp), ("workspace_bytes", C.c_size_t), ("dev_status", vp), ("a_absmax_dev", vp),
    ]


class DwArgs(C.Structure):
    _fields_ = [
        ("P", C.c_int64), ("E", C.c_int32), ("K", C.c_int32), ("N", C.c_int32), ("precision", C.c_int32),
        ("expert_offsets", vp),
        ("x", vp), ("x_dtype", C.c_int32), ("x_stride", C.c_int64), ("x_rows", C.c_int64), ("x_row", vp), ("ir", vp), ("ir_by_expert", C.c_int32),
        ("g", vp), ("g_dtype", C.c_int32), ("g_stride", C.c_int64), ("g_rows", C.c_int64), ("g_row", vp),
        ("g_div", C.c_int32), ("g_scale", vp), ("dw", vp),
        ("x_hi", vp), ("x_lo", vp), ("g_hi", vp), ("g_lo", vp), ("cache_rows", C.c_int64), ("expected_rows", C.c_int64),
        ("workspace", vp), ("workspace_bytes", C.c_size_t), ("dev_status", vp), ("g_absmax_dev", vp),
    ]


# name -> (restype, argtypes); every symbol include/amoe.h declares
SIGNATURES = {
    "amoe_version": (C.c_int, []),
    "amoe_status_string": (C.c_char_p, [C.c_int]),
    "amoe_last_error_string": (C.c_char_p, []),
    "amoe_launch_count": (C.c_ulonglong, []),
    "amoe_check_device": (C.c_int, []),
    "amoe_read_device_status": (C.c_int, [vp, C.POINTER(C.c_int32 * 4), vp]),
    "amoe_selftest_bounded_wait": (C.c_int, [vp, C.c_longlong, vp]),
    "amoe_select_sort_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int32, C.c_int32]),
    "amoe_select_sort": (C.c_int, [vp, C.c_int64, C.c_int32, C.c_int32, C.c_int32, vp, vp, vp, vp, vp, vp, vp,
                                   C.c_size_t, vp]),
    "amoe_gate_backward": (C.c_int, [vp, vp, vp, C.c_int64, C.c_int32, C.c_int32, C.c_int32, vp, vp]),
    "amoe_router_logits": (C.c_int, [vp, C.c_int32, C.c_int64, C.c_int64, C.c_int32, vp, C.c_int32, C.c_int32, vp, C.c_int32,
                                     vp, vp]),
    "amoe_router_select": (C.c_int, [vp, C.c_int32, C.c_int64, C.c_int64, C.c_int32, vp, C.c_int32, C.c_int32, vp, C.c_int32,
                                     C.c_int32, C.c_int32, vp, vp, vp, vp]),
    "amoe_sort_slots": (C.c_int, [vp, C.c_int64, C.c_int32, C.c_int32, vp, vp, vp, vp, vp, C.c_size_t, vp]),
    "amoe_router_backward_w_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int32, C.c_int32]),
    "amoe_router_backward_w": (C.c_int, [vp, C.c_int32, C.c_int64, C.c_int64, C.c_int32, vp, vp, C.c_int32, vp, vp, vp, vp,
                                         C.c_int64, C.c_int32, vp, vp, C.c_size_t, vp]),
    "amoe_combine_router": (C.c_int, [vp, C.c_int32, C.c_int64, vp, C.c_int64, C.c_int32, C.c_int32, vp, vp, C.c_int32, vp, vp,
                                      C.c_int32, C.c_int32, vp, C.c_int32, C.c_int64, vp]),
    "amoe_expert_offsets": (C.c_int, [vp, C.c_int64, C.c_int32, vp, vp, vp]),
    "amoe_weight_prepass_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "amoe_weight_prepass_clip_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "amoe_prepared_dims": (None, [C.c_int32, C.c_int32, C.POINTER(C.c_int32 * 4)]),
    "amoe_weight_prepass": (C.c_int, [C.POINTER(WeightPrepassArgs), vp]),
    "amoe_tensor_absmax": (C.c_int, [vp, C.c_int32, C.c_int64, C.c_int32, C.c_int64, vp, vp, vp]),
    "amoe_row_absmax": (C.c_int, [vp, C.c_int32, C.c_int64, C.c_int32, C.c_int64, vp, vp]),
    "amoe_cvmm_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int32]),
    "amoe_padded_rows": (C.c_int64, [C.c_int64, C.c_int32]),
    "amoe_operand_tiles": (C.c_int, [C.POINTER(OperandTilesArgs), vp]),
    "amoe_cvmm_fwd": (C.c_int, [C.POINTER(CvmmArgs), vp]),
    "amoe_cvmm_dx": (C.c_int, [C.POINTER(CvmmArgs), vp]),
    "amoe_cvmm_dw_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "amoe_cvmm_dw": (C.c_int, [C.POINTER(DwArgs), vp]),
    "amoe_cvmm_dw_workspace_bytes_tuned": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "amoe_combine": (C.c_int, [vp, C.c_int32, C.c_int64, vp, vp, C.c_int64, C.c_int32, C.c_int32, vp, C.c_int32,
                               C.c_int64, vp]),
    "amoe_combine_codes": (C.c_int, [vp, vp, vp, vp, C.c_float, vp, C.c_int64, C.c_int32, C.c_int32, vp, C.c_int32,
                                     C.c_int64, vp, vp]),
    "amoe_row_dot": (C.c_int, [vp, C.c_int32, C.c_int64, vp, vp, C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_int32,
                               vp, vp]),
    "amoe_row_dot_codes": (C.c_int, [vp, vp, vp, vp, C.c_float, vp, C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_int32,
                                     vp, vp, vp]),
    "amoe_ir_grad_reduce": (C.c_int, [vp, vp, vp, C.c_int32, C.c_float, C.c_float, vp, C.c_double, vp, C.c_int32, vp, vp]),
    "amoe_expert_std_workspace_bytes": (C.c_size_t, [C.c_int32]),
    "amoe_expert_std": (C.c_int, [vp, C.c_int32, C.c_int64, C.c_int32, C.c_int64, vp, vp, C.c_int64, C.c_int32, vp, vp,
                                  C.c_size_t, vp, vp]),
    "amoe_expert_std_static": (C.c_int, [vp, C.c_int32, C.c_int64, C.c_int32, C.c_int64, vp, vp, C.c_int64, C.c_int32, vp,
                                         vp, vp]),
    "amoe_ep_pack": (C.c_int, [vp, C.c_int32, C.c_int64, C.c_int32, vp, C.c_int32, vp, C.c_int64, vp, C.c_float, vp, vp,
                               vp, vp]),
    "amoe_invert_index": (C.c_int, [vp, C.c_int64, vp, vp]),
    "amoe_ep_local_plan": (C.c_int, [vp, C.c_int32, C.c_int32, C.c_int64, vp, vp, vp]),
    "amoe_ep_plan_ints": (C.c_int64, [C.c_int32, C.c_int32]),
    "amoe_ep_plan": (C.c_int, [vp, C.c_int32, C.c_int32, C.c_int32, vp, vp]),
    "amoe_ep_put_f16": (C.c_int, [vp, C.c_int64, C.c_int32, C.c_int64, vp, C.c_int32, vp, C.c_int64, vp, C.c_int32, vp, vp, vp,
                                  C.c_int32, C.c_int64, vp, vp]),
    "amoe_ep_share": (C.c_int, [vp, C.c_int64, vp, C.c_int64, vp, vp, C.c_int32, C.c_int32, vp, C.c_int64, vp, vp]),
    "amoe_ep_local_plan_dev": (C.c_int, [vp, C.c_int32, C.c_int32, C.c_int64, vp, vp, vp, vp]),
    "amoe_ep_put": (C.c_int, [vp, C.c_int32, C.c_int64, C.c_int32, C.c_int64, vp, C.c_int32, vp, C.c_int64, vp, C.c_int32, vp,
                              vp, C.c_int32, C.c_int64, vp, vp]),
    "amoe_ep_put_back": (C.c_int, [vp, C.c_int32, C.c_int64, C.c_int32, vp, vp, C.c_int32, C.c_int64, C.c_int64, vp, vp]),
    "amoe_ep_unpack": (C.c_int, [vp, C.c_int32, C.c_int32, vp, C.c_int64, vp, C.c_int64, vp]),
}


def _load() -> C.CDLL:
    path = os.environ.get("AMOE_LIB", _build.LIB_PATH)
    if not os.path.exists(path):
        raise ImportError(
            f"{path} not found. Build the CUDA library first: `python analog-moe_b200/analog_moe/_build.py` "
            "(needs nvcc; there is no CPU or PyTorch fallback).")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


_lib = _load()
lib = _lib


def check(status: int, where: str) -> None:
    if status != 0:
        raise AmoeError(status, where)


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"unsupported dtype {t.dtype}: the kernels take float32 or bfloat16")


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_LAUNCH_STREAM = None      # torch.cuda.Stream that overrides the current stream for library launches


def stream_ptr() -> int:
    if _LAUNCH_STREAM is not None:
        return _LAUNCH_STREAM.cuda_stream
    return torch.cuda.current_stream().cuda_stream


class launch_on:
    """Library calls inside the block are launched on `stream` while torch keeps allocating on the current
    stream: memory stays owned by the current stream, so its reuse is ordered by the join
    (`current.wait_stream(stream)`) the caller does afterwards.  The caller also orders `stream` after the
    current stream before entering (`stream.wait_stream(current)`)."""

    def __init__(self, stream):
        self.stream = stream

    def __enter__(self):
        global _LAUNCH_STREAM
        self.prev = _LAUNCH_STREAM
        _LAUNCH_STREAM = self.stream
        return self

    def __exit__(self, *exc):
        global _LAUNCH_STREAM
        _LAUNCH_STREAM = self.prev
        return False


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("analog CVMM kernels run on CUDA tensors only (no CPU path in this library)")
