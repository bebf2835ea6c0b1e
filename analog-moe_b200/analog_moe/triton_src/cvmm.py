"""Drop-in replacement for the reference's `analog_moe/triton_src/cvmm.py`.

Same public names and call signatures - `CVMMSel`, `cvmm_prepare_sel`, `cvmm_std`, `CVMM.apply`
with its eleven arguments and eleven-entry backward tuple (reference cvmm.py:19-34, 400-443,
699-897) - but every kernel behind them is a hand-written sm_100a CUDA kernel reached through the
C ABI in include/amoe.h.  There is no Triton and no CPU path: CPU tensors raise.

Extensions the reference does not have hang off one optional twelfth argument, `ext: CVMMExt`
(Philox output noise and weight modifier fused into the kernels, ADC output quantisation, the
contraction precision, a routing table computed once per layer call).  Without it the behaviour
is the reference's.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import _cabi as A
from .. import ops


@dataclass
class CVMMSel:
    """reference cvmm.py:19-28"""
    raw_sel: torch.Tensor
    sel: torch.Tensor
    sel_index: torch.Tensor
    out_index: Optional[torch.Tensor] = None
    reduction_weight: Optional[torch.Tensor] = None
    expert_offsets: Optional[torch.Tensor] = None   # [E+1] int32; filled by the select/sort kernel

    def clone(self) -> "CVMMSel":
        return CVMMSel(self.raw_sel, self.sel, self.sel_index, self.out_index, self.reduction_weight,
                       self.expert_offsets)


def cvmm_prepare_sel(sel: torch.Tensor, n_experts: int) -> CVMMSel:
    """reference cvmm.py:31-34: flatten and sort the expert ids (stable here)."""
    fsel = sel.flatten()
    ssel, sel_index = fsel.sort(stable=True)
    return CVMMSel(sel, ssel.view_as(sel), sel_index, None)


def cvmm_std(x: torch.Tensor, sel_index: torch.Tensor, sel: torch.Tensor, n_experts: int) -> torch.Tensor:
    """Per-expert std of the routed rows (reference cvmm.py:400-443)."""
    A.require_cuda(x)
    ssel = ops.i32(sel)
    off = ops.expert_offsets(ssel, n_experts)
    return ops.expert_std(x, ops.i32(sel_index), off, n_experts).to(x.dtype)


@dataclass
class PhiloxNoise:
    """Output noise generated inside the kernel: std * col_scale[e, n] * N(0,1), addressed by
    (seed, offset, destination row, column)."""
    std: float
    seed: int
    offset: int = 0
    step: Optional[torch.Tensor] = None     # int64 device scalar; the offset in effect is offset + 8*step


@dataclass
class WeightModifier:
    """ADD_NORMAL / DISCRETIZE weight modifiers applied in the weight pre-pass."""
    std_dev: float = 0.0
    per_channel: bool = True
    discretize_res: float = -1.0
    seed: int = 0
    offset: int = 0
    step: Optional[torch.Tensor] = None


@dataclass
class CVMMExt:
    noise: Optional[PhiloxNoise] = None
    modifier: Optional[WeightModifier] = None
    out_res: float = -1.0
    out_bound: float = -1.0
    scale_per_channel: bool = True          # col_scale per column (True) or per expert
    precision: Optional[int] = None         # _cabi.PREC_*; None = by dtype / AMOE_PRECISION
    expert_offsets: Optional[torch.Tensor] = None
    save_codes: bool = False                # keep ADC codes (int8) on `last_codes`
    last_codes: Optional[torch.Tensor] = field(default=None, repr=False)
    check_status: bool = False              # synchronise and raise on device-side index/wait errors
    adc_codes_path: bool = True             # with ADC and a gate-weighted reduction keep the per-slot rows as int8
                                            # codes (4x less HBM traffic); False materialises them in x.dtype


def _uses_abs_max(ir_params, io_params) -> bool:
    """Abs-max input scaling policy of reference cvmm.py:727-739."""
    if not hasattr(io_params, "is_perfect"):            # aihwkit-lightning style parameters
        return not bool(getattr(ir_params, "enable", False))
    if io_params is None or io_params.is_perfect:
        return False
    nm = io_params.noise_management
    return getattr(nm, "name", str(nm)).split(".")[-1] == "ABS_MAX"


class CVMM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, sel_index, sel, keys, inp_res, broadcasted_input_ranges=None, out_index=None,
                reduction_weight=None, out_noise=None, ir_params=None, io_params=None, ext=None):
        A.require_cuda(x, keys)
        if torch.is_autocast_enabled():
            raise RuntimeError("autocast is not supported by the B200 CVMM kernels; pass bf16 or fp32 tensors")
        ext = ext or CVMMExt()
        ops.set_tag("down" if reduction_weight is not None else "up")
        E, K, N = keys.shape
        if x.shape[-1] != K:
            raise ValueError(f"x has {x.shape[-1]} features, weights expect {K}")     # reference cvmm.py:561
        x2 = x.reshape(-1, K)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        P = sel.numel()
        dev = x.device
        precision = ext.precision if ext.precision is not None else ops.default_precision(x.dtype)
        if os.environ.get("_AIHWKIT_NO_ROUNDING", False):                              # reference cvmm.py:603-608
            assert os.environ.get("AIHWKIT_TESTING", False), "Skipping rounding but AIHWKIT_TESTING not set"
            inp_res = -1
        status = ops.new_status(dev) if ext.check_status else None

        sel_i = ops.i32(sel)
        sel_index_i = ops.i32(sel_index)
        out_index_i = None if out_index is None else ops.i32(out_index)
        offsets = ext.expert_offsets if ext.expert_offsets is not None else ops.expert_offsets(sel_i, E, status)
        ir = None if broadcasted_input_ranges is None else broadcasted_input_ranges.reshape(-1).float().contiguous()
        absmax = ops.row_absmax(x2) if _uses_abs_max(ir_params, io_params) else None

        mod = ext.modifier
        pw = ops.weight_prepass(
            keys, precision, per_channel_scale=ext.scale_per_channel,
            noise_std=mod.std_dev if mod else 0.0, noise_per_channel=mod.per_channel if mod else True,
            discretize_res=mod.discretize_res if mod else -1.0, seed=mod.seed if mod else 0,
            offset=mod.offset if mod else 0, step_dev=mod.step if mod else None, need_fwd=True, need_bwd=any(ctx.needs_input_grad[:1]) or True)

        noise_t, noise_std, seed, offset, step_dev = None, 0.0, 0, 0, None
        if isinstance(out_noise, PhiloxNoise):
            ext = CVMMExt(**{**ext.__dict__, "noise": out_noise})
        elif out_noise is not None:
            noise_t = out_noise
        if ext.noise is not None and ext.noise.std > 0:
            noise_std, seed, offset, step_dev = ext.noise.std, ext.noise.seed, ext.noise.offset, ext.noise.step

        dst = sel_index_i if out_index_i is None else out_index_i
        adc_on = ext.out_res > 0 and ext.out_bound > 0
        codes_path = adc_on and reduction_weight is not None and ext.adc_codes_path
        row_meta = {} if codes_path else None
        res, codes = ops.cvmm_fwd(
            x2, sel_index_i, dst, offsets, pw, precision, P=P, dst_rows=P, ir=ir, absmax=absmax,
            inp_res=float(inp_res), noise=noise_t, noise_std=noise_std, seed=seed, offset=offset, step_dev=step_dev,
            out_res=ext.out_res if adc_on else -1.0, out_bound=ext.out_bound if adc_on else -1.0,
            want_codes=codes_path or (adc_on and ext.save_codes), status=status, want_out=not codes_path,
            row_meta=row_meta)
        if ext.save_codes:
            ext.last_codes = codes

        res_into_reduction = None
        row_scale = row_expert = None
        adc_step = ops.adc_step(ext.out_res, ext.out_bound) if adc_on else 0.0
        if reduction_weight is not None:
            k = reduction_weight.shape[-1]
            if codes_path:
                # y[t] = sum_j gate * ((code*step)*col_scale)*row_scale, straight from the int8 codes
                row_scale, row_expert = row_meta["row_scale"], row_meta["row_expert"]
                out = ops.combine_codes(codes, pw.col_scale, row_expert, row_scale, adc_step, reduction_weight, P // k, k,
                                        out_dtype=x.dtype).view(*reduction_weight.shape[:-1], N)
            else:
                res_into_reduction = res.view(*reduction_weight.shape, N)
                out = ops.combine(res, reduction_weight, P // k, k).view(*reduction_weight.shape[:-1], N)   # cvmm.py:757-759
        else:
            out = res.view(*sel.shape, N)
        if status is not None:
            ops.raise_on_device_status(status, "CVMM.forward")

        ctx.save_for_backward(x, sel_i, sel_index_i, out_index_i, reduction_weight, ir, res_into_reduction, offsets,
                              pw.w if precision == A.PREC_FP32_SIMT else None, pw.bwd_hi, pw.bwd_lo, pw.col_scale,
                              codes if codes_path else None, row_scale, row_expert)
        ctx.meta = (E, K, N, precision, ir_params, keys.dtype, broadcasted_input_ranges.shape if ir is not None else None,
                    ext.check_status, adc_step)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (x, sel_i, sel_index_i, out_index_i, reduction_weight, ir, res_into_reduction, offsets, w_mod, bwd_hi, bwd_lo,
         col_scale, codes, row_scale, row_expert) = ctx.saved_tensors
        E, K, N, precision, ir_params, keys_dtype, ir_shape, check_status, adc_step = ctx.meta
        ops.set_tag("down" if reduction_weight is not None else "up")
        dev = x.device
        P = sel_i.numel()
        x2 = x.reshape(-1, K)
        g = grad_output.reshape(-1, N)
        if g.stride(-1) != 1:
            g = g.contiguous()
        status = ops.new_status(dev) if check_status else None
        pw = ops.PreparedWeights(E, K, N, col_scale, w=w_mod, bwd_hi=bwd_hi, bwd_lo=bwd_lo)
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[3]
        need_ir = ir is not None and ctx.needs_input_grad[5]
        down = reduction_weight is not None
        k = reduction_weight.shape[-1] if down else max(P // x2.shape[0], 1)
        rw = reduction_weight.reshape(-1).float().contiguous() if down else None

        grad_w = None
        if need_w:
            # reference cvmm.py:785-823: the outer product rw (x) g is folded into the operand load
            if down:
                grad_w = ops.cvmm_dw(x2, sel_index_i, g, sel_index_i, offsets, E, precision, P=P, ir=ir, g_div=k,
                                     g_scale=rw, status=status)
            else:
                g_row = out_index_i if out_index_i is not None else sel_index_i
                grad_w = ops.cvmm_dw(x2, sel_index_i, g, g_row, offsets, E, precision, P=P, ir=ir, status=status)
            grad_w = grad_w.to(keys_dtype)

        grad_x = grad_ir = grad_gate = None
        if need_x or need_ir:
            decay = float(getattr(ir_params, "decay", 0.0) or 0.0) if ir is not None else 0.0
            keep = torch.zeros(1, dtype=torch.int64, device=dev) if (ir is not None and decay > 0) else None
            relative = bool(getattr(ir_params, "gradient_relative", True))
            gscale = float(getattr(ir_params, "gradient_scale", 1.0)) if relative else 1.0
            if down:
                # reference cvmm.py:828-846 with bw_index = sel_index // k, output rows = sel_index
                gx, ir_slot = ops.cvmm_dx(g, sel_index_i, sel_index_i, offsets, pw, precision, P=P, dst_rows=P,
                                          a_row_div=k, x_ref=x2 if ir is not None else None,
                                          x_ref_row=sel_index_i if ir is not None else None, ir=ir, row_scale=rw,
                                          want_ir_grad=ir is not None, relative=relative, grad_scale=gscale,
                                          keep_count=keep, out_dtype=x.dtype, status=status)
                grad_x = gx.view_as(x)
            else:
                src = out_index_i if out_index_i is not None else sel_index_i
                gx, ir_slot = ops.cvmm_dx(g, src, src, offsets, pw, precision, P=P, dst_rows=P,
                                          x_ref=x2 if ir is not None else None,
                                          x_ref_row=sel_index_i if ir is not None else None, ir=ir,
                                          want_ir_grad=ir is not None, relative=relative, grad_scale=gscale,
                                          keep_count=keep, out_dtype=x.dtype, status=status)
                T = x2.shape[0]
                if P != T:
                    grad_x = ops.combine(gx, None, T, P // T).view_as(x)               # cvmm.py:890-891
                else:
                    grad_x = gx.view_as(x)
            if ir is not None:
                if decay > 0:                                                            # cvmm.py:872-878
                    pct = keep.double() / float(P * K)
                    ir_slot = ir_slot + decay * ir * (pct > ir_params.input_min_percentage).float()
                grad_ir = ir_slot.view(ir_shape)
        if down and ctx.needs_input_grad[7]:
            if codes is not None:
                d = ops.row_dot_codes(codes, col_scale, row_expert, row_scale, adc_step, g, k)
            else:
                d = ops.row_dot(res_into_reduction, g, k)                                     # cvmm.py:889
            grad_gate = d.view_as(reduction_weight).to(reduction_weight.dtype)
        if status is not None:
            ops.raise_on_device_status(status, "CVMM.backward")
        return (grad_x if need_x else None, None, None, grad_w, None, grad_ir if need_ir else None, None, grad_gate,
                None, None, None, None)
