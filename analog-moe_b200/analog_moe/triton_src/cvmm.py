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
from typing import List, Optional

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


@torch.library.custom_op("amoe::cvmm_std", mutates_args=())
def cvmm_std(x: torch.Tensor, sel_index: torch.Tensor, sel: torch.Tensor, n_experts: int) -> torch.Tensor:
    """Per-expert std of the routed rows (reference cvmm.py:400-443)."""
    A.require_cuda(x)
    ssel = ops.i32(sel)
    off = ops.expert_offsets(ssel, n_experts)
    return ops.expert_std(x, ops.i32(sel_index), off, n_experts).to(x.dtype)


@cvmm_std.register_fake
def _cvmm_std_fake(x, sel_index, sel, n_experts):
    return x.new_empty(n_experts)


@torch.library.custom_op("amoe::select_sort", mutates_args=())
def select_sort_op(logits: torch.Tensor, k: int, apply_sigmoid: bool) -> List[torch.Tensor]:
    """Gate selection and expert-contiguous slot sort (the base layer's sigmoid / top-k and cvmm_prepare_sel's sort,
    reference tests/test_moe_layer_aihwkit.py:71-76, cvmm.py:31-34) as one operator:
    [raw_sel [T,k], gate [T,k], sel [P], token_index [P], slot_index [P], expert_offsets [E+1]]."""
    r = ops.select_sort(logits, k, apply_sigmoid)
    return [r.raw_sel, r.gate, r.sel, r.token_index, r.slot_index, r.expert_offsets]


@select_sort_op.register_fake
def _select_sort_fake(logits, k, apply_sigmoid):
    E = logits.shape[-1]
    T = logits.numel() // E
    i32 = dict(dtype=torch.int32)
    new = logits.new_empty
    return [new(T, k, **i32), new(T, k, dtype=torch.float32), new(T * k, **i32), new(T * k, **i32), new(T * k, **i32),
            new(E + 1, **i32)]


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


# --------------------------------------------------------------------------- the operator boundary
# The reference registers its forward as a torch.library operator with a fake ("abstract") implementation so that
# torch.compile can trace through CVMM.apply (cvmm.py:529, 634-642).  Here both directions are operators
# (`amoe::cvmm_forward`, `amoe::cvmm_backward`): their real implementations drive the C ABI, their fake ones only
# compute shapes, and the autograd.Function below is plain tensor glue around them.  Tensors an operator does not
# produce in a given mode come back as empty (numel 0) tensors: operator outputs cannot be optional.

def _none_if_empty(t: torch.Tensor) -> Optional[torch.Tensor]:
    return t if t.numel() > 0 else None


def _empty(like: torch.Tensor, dtype=None) -> torch.Tensor:
    return like.new_empty(0, dtype=dtype or like.dtype)


def _tiles_eligible(x2: torch.Tensor, precision: int) -> bool:
    """Whether the operand pre-pass feeds this call (decided from metadata only, so that the fake implementations agree
    with the real ones): a tensor-core precision, 64-column blocks, rows that start on 16-byte boundaries."""
    esz = x2.element_size()
    return precision != A.PREC_FP32_SIMT and x2.shape[-1] % 64 == 0 and x2.stride(-1) == 1 and \
        (x2.stride(0) * esz) % 16 == 0 and (x2.storage_offset() * esz) % 16 == 0


def _prepared_weights(keys: torch.Tensor, precision: int, per_channel: bool, mod_std: float, mod_per_channel: bool,
                      mod_disc: float, mod_seed: int, mod_offset: int, mod_step: Optional[torch.Tensor],
                      training_call: bool = False):
    """Weight pre-pass, skipped when these exact weights (same storage, same version counter) were prepared before, no
    modifier changes them from call to call and the call does not train them: an inference layer pays for it once, not on
    every CVMM.apply.  A call whose weight gradient is wanted always prepares them: training loops also write weights in
    ways the version counter does not see (`p.data.add_(...)`)."""
    if mod_std > 0 or mod_disc > 0 or training_call:
        return ops.weight_prepass(keys, precision, per_channel_scale=per_channel, noise_std=mod_std,
                                  noise_per_channel=mod_per_channel, discretize_res=mod_disc, seed=mod_seed,
                                  offset=mod_offset, step_dev=mod_step, need_fwd=True, need_bwd=True)
    return ops.weight_prepass_cached(keys, precision, per_channel)


@torch.library.custom_op("amoe::cvmm_forward", mutates_args=())
def cvmm_forward_op(x: torch.Tensor, sel_index: torch.Tensor, sel: torch.Tensor, keys: torch.Tensor, inp_res: float,
                    input_ranges: Optional[torch.Tensor], out_index: Optional[torch.Tensor],
                    reduction_weight: Optional[torch.Tensor], out_noise: Optional[torch.Tensor], use_abs_max: bool,
                    expert_offsets: Optional[torch.Tensor], precision: int, scale_per_channel: bool,
                    noise_std: float, noise_seed: int, noise_offset: int, noise_step: Optional[torch.Tensor],
                    mod_std: float, mod_per_channel: bool, mod_discretize: float, mod_seed: int, mod_offset: int,
                    mod_step: Optional[torch.Tensor], out_res: float, out_bound: float, adc_codes_path: bool,
                    save_codes: bool, check_status: bool, save_operands: bool) -> List[torch.Tensor]:
    """Forward CVMM (reference cvmm.py:529-631 plus the reduction of cvmm.py:757-759).
    Returns [out, offsets, res_into_reduction, codes, row_scale, row_expert, w_mod, bwd_hi, bwd_lo, col_scale,
    x_cache_hi, x_cache_lo]; the last two (with `save_operands`) hold the clamped input rows - times the reduction
    weight, where there is one - as the weight gradient's operand."""
    A.require_cuda(x, keys)
    ops.set_tag("down" if reduction_weight is not None else "up")
    E, K, N = keys.shape
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    P = sel.numel()
    dev = x.device
    status = ops.new_status(dev) if check_status else None
    sel_i = ops.i32(sel)
    sel_index_i = ops.i32(sel_index)
    out_index_i = None if out_index is None else ops.i32(out_index)
    if expert_offsets is not None:
        offsets = expert_offsets
        offsets_out = _empty(sel_i)
    else:
        offsets = offsets_out = ops.expert_offsets(sel_i, E, status)
    ir = None if input_ranges is None else input_ranges.reshape(-1).float().contiguous()
    absmax = ops.row_absmax(x2) if use_abs_max else None
    pw = _prepared_weights(keys, precision, scale_per_channel, mod_std, mod_per_channel, mod_discretize, mod_seed,
                           mod_offset, mod_step, training_call=save_operands)
    dst = sel_index_i if out_index_i is None else out_index_i
    adc_on = out_res > 0 and out_bound > 0
    codes_path = adc_on and reduction_weight is not None and adc_codes_path
    row_meta = {} if codes_path else None
    # The DAC of the gathered rows runs as a streaming pass of its own that leaves the A operand as TMA tiles (and, for
    # the backward pass, the clamped rows as the weight gradient's operand); the tensor-core kernel runs no prologue.
    a_kw, x_cache = {}, None
    if _tiles_eligible(x2, precision):
        csc = None if reduction_weight is None else reduction_weight.reshape(-1).float().contiguous()
        tiles, x_cache = ops.operand_tiles(x2, sel_index_i, offsets, E, precision, P=P, dac=True, ir=ir, absmax=absmax,
                                           inp_res=float(inp_res), want_cache=save_operands, cache_scale=csc,
                                           status=status)
        a_kw = dict(a_tiles=tiles)
    res, codes = ops.cvmm_fwd(
        x2, sel_index_i, dst, offsets, pw, precision, P=P, dst_rows=P, ir=ir, absmax=absmax,
        inp_res=float(inp_res), noise=out_noise, noise_std=noise_std, seed=noise_seed, offset=noise_offset,
        step_dev=noise_step, out_res=out_res if adc_on else -1.0, out_bound=out_bound if adc_on else -1.0,
        want_codes=codes_path or (adc_on and save_codes), status=status, want_out=not codes_path, row_meta=row_meta,
        **a_kw)
    row_scale = row_expert = None
    if reduction_weight is not None:
        k = reduction_weight.shape[-1]
        if codes_path:
            # y[t] = sum_j gate * ((code*step)*col_scale)*row_scale, straight from the int8 codes
            row_scale, row_expert = row_meta["row_scale"], row_meta["row_expert"]
            out = ops.combine_codes(codes, pw.col_scale, row_expert, row_scale, ops.adc_step(out_res, out_bound),
                                    reduction_weight, P // k, k, out_dtype=x.dtype).view(*reduction_weight.shape[:-1], N)
            res_keep = _empty(x2)
        else:
            out = ops.combine(res, reduction_weight, P // k, k).view(*reduction_weight.shape[:-1], N)   # cvmm.py:757-759
            res_keep = res.view(*reduction_weight.shape, N)
    else:
        out = res.view(*sel.shape, N)
        res_keep = _empty(x2)
    if status is not None:
        ops.raise_on_device_status(status, "CVMM.forward")
    simt = precision == A.PREC_FP32_SIMT
    w_mod = _empty(x2)      # (every absent output is its own empty tensor: operator outputs must not alias)
    if simt and pw.w is not keys:   # the CUDA-core backward reads the (modified) weights; never hand an input back
        w_mod = pw.w
    keep_codes = codes is not None and (codes_path or save_codes)
    return [out, offsets_out, res_keep, codes if keep_codes else _empty(x2, torch.int8),
            row_scale if row_scale is not None else _empty(x2, torch.float32),
            row_expert if row_expert is not None else _empty(x2, torch.int32), w_mod,
            pw.bwd_hi if pw.bwd_hi is not None else _empty(x2, torch.bfloat16),
            pw.bwd_lo if pw.bwd_lo is not None else _empty(x2, torch.bfloat16), pw.col_scale,
            x_cache.hi if x_cache is not None else _empty(x2, torch.bfloat16),
            x_cache.lo if (x_cache is not None and x_cache.lo is not None) else _empty(x2, torch.bfloat16)]


@cvmm_forward_op.register_fake
def _cvmm_forward_fake(x, sel_index, sel, keys, inp_res, input_ranges, out_index, reduction_weight, out_noise,
                       use_abs_max, expert_offsets, precision, scale_per_channel, noise_std, noise_seed, noise_offset,
                       noise_step, mod_std, mod_per_channel, mod_discretize, mod_seed, mod_offset, mod_step, out_res,
                       out_bound, adc_codes_path, save_codes, check_status, save_operands):
    """Shapes only (reference cvmm.py:634-642)."""
    E, K, N = keys.shape
    P = sel.numel()
    new = x.new_empty
    e = new(0)
    adc_on = out_res > 0 and out_bound > 0
    codes_path = adc_on and reduction_weight is not None and adc_codes_path
    if reduction_weight is not None:
        out = new(*reduction_weight.shape[:-1], N)
        res_keep = e if codes_path else new(*reduction_weight.shape, N)
    else:
        out, res_keep = new(*sel.shape, N), e
    codes = new(P, N, dtype=torch.int8) if (codes_path or (adc_on and save_codes)) else new(0, dtype=torch.int8)
    row_scale = new(P if codes_path else 0, dtype=torch.float32)
    row_expert = new(P if codes_path else 0, dtype=torch.int32)
    offsets = new(0 if expert_offsets is not None else E + 1, dtype=torch.int32)
    simt = precision == A.PREC_FP32_SIMT
    modified = mod_std > 0 or mod_discretize > 0
    w_mod = new(E, K, N, dtype=torch.float32) if (simt and modified) else e
    _, _, kpad2, npad2 = ops.prepared_dims(K, N)
    split = precision == A.PREC_SPLIT and (keys.dtype != torch.bfloat16 or modified)
    bwd_hi = new((0,) if simt else (E, kpad2, npad2), dtype=torch.bfloat16)
    bwd_lo = new((E, kpad2, npad2) if (split and not simt) else (0,), dtype=torch.bfloat16)
    x2 = x.reshape(-1, K)
    cached = save_operands and _tiles_eligible(x2, precision)
    cshape = (K // 64, int(ops.lib.amoe_padded_rows(P, E)), 64)
    xc_hi = new(cshape if cached else (0,), dtype=torch.bfloat16)
    xc_lo = new(cshape if (cached and precision == A.PREC_SPLIT) else (0,), dtype=torch.bfloat16)
    return [out, offsets, res_keep, codes, row_scale, row_expert, w_mod, bwd_hi, bwd_lo, new(E, N, dtype=torch.float32),
            xc_hi, xc_lo]


@torch.library.custom_op("amoe::cvmm_backward", mutates_args=())
def cvmm_backward_op(grad_output: torch.Tensor, x: torch.Tensor, sel: torch.Tensor, sel_index: torch.Tensor,
                     out_index: Optional[torch.Tensor], reduction_weight: Optional[torch.Tensor],
                     input_ranges: Optional[torch.Tensor], res_into_reduction: Optional[torch.Tensor],
                     offsets: torch.Tensor, w: Optional[torch.Tensor], bwd_hi: Optional[torch.Tensor],
                     bwd_lo: Optional[torch.Tensor], col_scale: torch.Tensor, codes: Optional[torch.Tensor],
                     row_scale: Optional[torch.Tensor], row_expert: Optional[torch.Tensor], n_experts: int, N: int,
                     precision: int, decay: float, min_percentage: float, relative: bool, grad_scale: float,
                     out_res: float, out_bound: float, need_x: bool, need_w: bool, need_ir: bool, need_gate: bool, check_status: bool,
                     x_cache_hi: Optional[torch.Tensor], x_cache_lo: Optional[torch.Tensor]) -> List[torch.Tensor]:
    """Backward CVMM (reference cvmm.py:771-897).  Returns [grad_x, grad_w (fp32), grad_ir (per sorted slot), grad_gate]."""
    E = n_experts
    K = x.shape[-1]
    down = reduction_weight is not None
    adc_step = ops.adc_step(out_res, out_bound) if (out_res > 0 and out_bound > 0) else 0.0
    ops.set_tag("down" if down else "up")
    dev = x.device
    sel_i, sel_index_i = ops.i32(sel), ops.i32(sel_index)
    out_index_i = None if out_index is None else ops.i32(out_index)
    P = sel_i.numel()
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    g = grad_output.reshape(-1, N)
    if g.stride(-1) != 1:
        g = g.contiguous()
    ir = None if input_ranges is None else input_ranges.reshape(-1).float().contiguous()
    status = ops.new_status(dev) if check_status else None
    pw = ops.PreparedWeights(E, K, N, col_scale, w=w, bwd_hi=bwd_hi, bwd_lo=bwd_lo)
    k = reduction_weight.shape[-1] if down else max(P // x2.shape[0], 1)
    rw = reduction_weight.reshape(-1).float().contiguous() if down else None
    gmax = ops.grad_absmax(g, precision)        # fp16 operands: the scalar that scales the gradient rows
    grad_w = _empty(x2)
    # The upstream gradient rows, gathered per slot and converted by the operand pre-pass, serve both as the A tiles of
    # the input gradient and - with the operand the forward pass saved - as the weight gradient's operands.
    g_tiles = None
    g_row_all = sel_index_i if down or out_index_i is None else out_index_i
    if _tiles_eligible(g, precision) and (need_x or need_ir or (need_w and x_cache_hi is not None)):
        g_tiles, _ = ops.operand_tiles(g, g_row_all, offsets, E, precision, P=P, a_row_div=k if down else 1, dac=False,
                                       g_absmax=gmax, status=status)
    if need_w and g_tiles is not None and x_cache_hi is not None:
        grad_w = ops.cvmm_dw_cached(ops.OperandCache(x_cache_hi, x_cache_lo, K), g_tiles, offsets, E, precision, P=P,
                                    status=status, g_absmax=gmax)
    elif need_w:
        # reference cvmm.py:785-823: the outer product rw (x) g is folded into the operand load
        if down:
            grad_w = ops.cvmm_dw(x2, sel_index_i, g, sel_index_i, offsets, E, precision, P=P, ir=ir, g_div=k,
                                 g_scale=rw, status=status, g_absmax=gmax)
        else:
            g_row = out_index_i if out_index_i is not None else sel_index_i
            grad_w = ops.cvmm_dw(x2, sel_index_i, g, g_row, offsets, E, precision, P=P, ir=ir, status=status,
                                 g_absmax=gmax)
    grad_x = _empty(x2)
    grad_ir = _empty(x2, torch.float32)
    if need_x or need_ir:
        use_decay = ir is not None and decay > 0
        keep = torch.zeros(1, dtype=torch.int64, device=dev) if use_decay else None
        if down:
            # reference cvmm.py:828-846 with bw_index = sel_index // k, output rows = sel_index
            gx, ir_slot = ops.cvmm_dx(g, sel_index_i, sel_index_i, offsets, pw, precision, P=P, dst_rows=P,
                                      a_row_div=k, x_ref=x2 if ir is not None else None,
                                      x_ref_row=sel_index_i if ir is not None else None, ir=ir, row_scale=rw,
                                      want_ir_grad=ir is not None, relative=relative, grad_scale=grad_scale,
                                      keep_count=keep, out_dtype=x.dtype, status=status, g_absmax=gmax, a_tiles=g_tiles)
            grad_x = gx.view(x.shape)
        else:
            src = out_index_i if out_index_i is not None else sel_index_i
            gx, ir_slot = ops.cvmm_dx(g, src, src, offsets, pw, precision, P=P, dst_rows=P,
                                      x_ref=x2 if ir is not None else None,
                                      x_ref_row=sel_index_i if ir is not None else None, ir=ir,
                                      want_ir_grad=ir is not None, relative=relative, grad_scale=grad_scale,
                                      keep_count=keep, out_dtype=x.dtype, status=status, g_absmax=gmax, a_tiles=g_tiles)
            T = x2.shape[0]
            grad_x = (ops.combine(gx, None, T, P // T) if P != T else gx).view(x.shape)               # cvmm.py:890-891
        if ir is not None:
            if use_decay:                                                                   # cvmm.py:872-878
                pct = keep.double() / float(P * K)
                ir_slot = ir_slot + decay * ir * (pct > min_percentage).float()
            grad_ir = ir_slot
    grad_gate = _empty(x2, torch.float32)
    if down and need_gate:
        if codes is not None:
            grad_gate = ops.row_dot_codes(codes, col_scale, row_expert, row_scale, adc_step, g, k)
        else:
            grad_gate = ops.row_dot(res_into_reduction, g, k)                                  # cvmm.py:889
    if status is not None:
        ops.raise_on_device_status(status, "CVMM.backward")
    return [grad_x, grad_w, grad_ir, grad_gate]


@cvmm_backward_op.register_fake
def _cvmm_backward_fake(grad_output, x, sel, sel_index, out_index, reduction_weight, input_ranges, res_into_reduction,
                        offsets, w, bwd_hi, bwd_lo, col_scale, codes, row_scale, row_expert, n_experts, N, precision,
                        decay, min_percentage, relative, grad_scale, out_res, out_bound, need_x, need_w, need_ir, need_gate,
                        check_status, x_cache_hi, x_cache_lo):
    new = x.new_empty
    P, K = sel.numel(), x.shape[-1]
    has_ir = input_ranges is not None
    return [new(x.shape) if (need_x or need_ir) else new(0),
            new(n_experts, K, N, dtype=torch.float32) if need_w else new(0),
            new(P if (has_ir and (need_x or need_ir)) else 0, dtype=torch.float32),
            new(P if (reduction_weight is not None and need_gate) else 0, dtype=torch.float32)]


class CVMM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, sel_index, sel, keys, inp_res, broadcasted_input_ranges=None, out_index=None,
                reduction_weight=None, out_noise=None, ir_params=None, io_params=None, ext=None):
        ext = ext or CVMMExt()
        E, K, N = keys.shape
        if x.shape[-1] != K:
            raise ValueError(f"x has {x.shape[-1]} features, weights expect {K}")     # reference cvmm.py:561
        # Half path (reference cvmm.py:177-179, 188-189, 716): under autocast - or for fp16 tensors - the reference casts
        # both operands to fp16 whatever their storage type, accumulates in fp32 and returns fp16.  That is the fp16
        # operand precision of the tensor-core kernels; fp16 tensors cross the boundary as fp32 (an exact widening).
        half_path = torch.is_autocast_enabled() or x.dtype == torch.float16 or keys.dtype == torch.float16
        out_type = torch.float16 if half_path else x.dtype
        x_dtype_in = x.dtype
        widen = lambda t: t.float() if (t is not None and t.dtype == torch.float16) else t
        if half_path:
            x, keys_k = widen(x), widen(keys)
            broadcasted_input_ranges, reduction_weight = widen(broadcasted_input_ranges), widen(reduction_weight)
            if isinstance(out_noise, torch.Tensor):
                out_noise = widen(out_noise)
        else:
            keys_k = keys
        if ext.precision is not None:
            precision = ext.precision
        else:
            precision = A.PREC_F16X1 if (half_path and x.dtype == torch.float32) else ops.default_precision(x.dtype)
        if os.environ.get("_AIHWKIT_NO_ROUNDING", False):                              # reference cvmm.py:603-608
            assert os.environ.get("AIHWKIT_TESTING", False), "Skipping rounding but AIHWKIT_TESTING not set"
            inp_res = -1
        noise_t, pn = None, ext.noise
        if isinstance(out_noise, PhiloxNoise):
            pn = out_noise
        elif out_noise is not None:
            noise_t = out_noise
        if pn is not None and not pn.std > 0:
            pn = None
        mod = ext.modifier
        save_operands = bool(ctx.needs_input_grad[3])       # the weight gradient will want the clamped rows
        (out, offsets, res_into_reduction, codes, row_scale, row_expert, w_mod, bwd_hi, bwd_lo,
         col_scale, xc_hi, xc_lo) = cvmm_forward_op(
            x, sel_index, sel, keys_k, float(inp_res), broadcasted_input_ranges, out_index, reduction_weight, noise_t,
            _uses_abs_max(ir_params, io_params), ext.expert_offsets, precision, ext.scale_per_channel,
            float(pn.std) if pn else 0.0, int(pn.seed) if pn else 0, int(pn.offset) if pn else 0, pn.step if pn else None,
            float(mod.std_dev) if mod else 0.0, bool(mod.per_channel) if mod else True,
            float(mod.discretize_res) if mod else -1.0, int(mod.seed) if mod else 0, int(mod.offset) if mod else 0,
            mod.step if mod else None, float(ext.out_res), float(ext.out_bound), ext.adc_codes_path, ext.save_codes,
            ext.check_status, save_operands)
        if ext.save_codes:
            ext.last_codes = _none_if_empty(codes)
        if ext.expert_offsets is not None:
            offsets = ext.expert_offsets
        simt = precision == A.PREC_FP32_SIMT
        ctx.save_for_backward(x, sel, sel_index, out_index, reduction_weight, broadcasted_input_ranges,
                              res_into_reduction, offsets, w_mod, keys_k if (simt and w_mod.numel() == 0) else None,
                              bwd_hi, bwd_lo, col_scale, codes, row_scale, row_expert, xc_hi, xc_lo)
        ctx.meta = (E, N, precision, ir_params, keys.dtype, ext.check_status, float(ext.out_res), float(ext.out_bound))
        ctx.x_dtype_in = x_dtype_in
        return out if out.dtype == out_type else out.to(out_type)

    @staticmethod
    def backward(ctx, grad_output):
        (x, sel, sel_index, out_index, reduction_weight, bir, res_into_reduction, offsets, w_mod, keys_simt, bwd_hi,
         bwd_lo, col_scale, codes, row_scale, row_expert, xc_hi, xc_lo) = ctx.saved_tensors
        E, N, precision, ir_params, keys_dtype, check_status, out_res, out_bound = ctx.meta
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[3]
        need_ir = bir is not None and ctx.needs_input_grad[5]
        need_gate = reduction_weight is not None and ctx.needs_input_grad[7]
        has_ir = bir is not None
        decay = float(getattr(ir_params, "decay", 0.0) or 0.0) if has_ir else 0.0
        min_pct = float(getattr(ir_params, "input_min_percentage", 0.95)) if has_ir else 0.95
        relative = bool(getattr(ir_params, "gradient_relative", True))
        gscale = float(getattr(ir_params, "gradient_scale", 1.0)) if relative else 1.0
        w = keys_simt if keys_simt is not None else _none_if_empty(w_mod)
        if grad_output.dtype == torch.float16:
            grad_output = grad_output.float()
        grad_x, grad_w, grad_ir, grad_gate = cvmm_backward_op(
            grad_output, x, sel, sel_index, out_index, reduction_weight, bir, _none_if_empty(res_into_reduction),
            offsets, w, _none_if_empty(bwd_hi), _none_if_empty(bwd_lo), col_scale, _none_if_empty(codes),
            _none_if_empty(row_scale), _none_if_empty(row_expert), E, N, precision, decay, min_pct, relative, gscale,
            out_res, out_bound, need_x, need_w, need_ir, need_gate, check_status, _none_if_empty(xc_hi),
            _none_if_empty(xc_lo))
        return (grad_x.to(ctx.x_dtype_in) if need_x else None, None, None, grad_w.to(keys_dtype) if need_w else None, None,
                grad_ir.view(bir.shape) if need_ir else None, None,
                grad_gate.view(reduction_weight.shape).to(reduction_weight.dtype) if need_gate else None,
                None, None, None, None)
