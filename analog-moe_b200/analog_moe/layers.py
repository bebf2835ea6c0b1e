"""sigma-MoE feed-forward layer and its analog hardware-aware version on the B200 kernels.

`SigmaMoELayer` is a stand-in for the third-party base class the reference layers derive from
(`sigma_moe.moe_layer.SigmaMoELayer`): same constructor keywords and attributes, `forward`
returning `(out, aux)` and calling `compute_scores` then `cvmm_wrapper(scores, sel, self.values)`
(contract: reference moe_layer_aihwkit_lightning.py:220-233, 261-276, 384-410;
tests/test_moe_layer_aihwkit.py:60-109).  In the composed path the router matmul is a torch Linear and
everything from the gate logits onward runs in the CUDA library; the single-node step of the analog layer
(`_FusedAnalogStep`) runs the router in the library as well.

`AnalogSigmaMoELayer` mirrors the non-traceable `AnalogSigmaMoELayerAIHWKITLightning`
(moe_layer_aihwkit_lightning.py:134-543): per-expert learnable input ranges [2, E], DAC, weight
modifier, output noise, and - new here - ADC output quantisation.
"""
from __future__ import annotations

import re
from functools import partial
from typing import Callable, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from . import ops
from .rpu_config import TorchInferenceRPUConfig, WeightClipType, aihwkit_rpu_config
from .triton_src.cvmm import CVMM, CVMMExt, CVMMSel, PhiloxNoise, WeightModifier, _uses_abs_max, cvmm_std, select_sort_op


class _BroadcastInputRange(torch.autograd.Function):
    """input_range_row[sel] for the expert-sorted slot list (reference
    moe_layer_aihwkit_lightning.py:447-448).  Backward is the per-expert segment sum of the
    per-slot gradients done by the library (the slots of an expert are contiguous), instead of
    autograd's generic sort-and-accumulate indexing backward."""

    @staticmethod
    def forward(ctx, row: Tensor, sel: Tensor, offsets: Tensor) -> Tensor:
        ctx.save_for_backward(offsets)
        ctx.n_experts = row.numel()
        return row[sel.long()]

    @staticmethod
    def backward(ctx, grad: Tensor):
        (offsets,) = ctx.saved_tensors
        g = grad.reshape(-1).float().contiguous()
        return ops.ir_grad_reduce(g, offsets, None, ctx.n_experts), None, None


def _enum_name(v) -> str:
    return getattr(v, "name", str(v)).split(".")[-1]


def _is_relu(fn) -> bool:
    return fn in (F.relu, torch.relu) or isinstance(fn, nn.ReLU)


class _FusedAnalogStep(torch.autograd.Function):
    """The whole layer (router matmul excepted: it stays a torch matmul) as one autograd node that calls the
    library directly.  Same arithmetic as the composition route() -> CVMM (up) -> ReLU -> CVMM (down), with
    the glue that the composition leaves to torch folded into the kernels:

      * input ranges are read per expert inside the kernels (no per-slot broadcast tensor),
      * the ReLU runs in the up-projection's epilogue and its backward in the down-projection's input-gradient
        epilogue,
      * the input-range decay term and the per-expert sum are one reduction kernel,
      * the gate gradient goes back to the logits in one kernel.

    Reference lines as for CVMM.forward / CVMM.backward (cvmm.py:700-897) and the layer's forward
    (moe_layer_aihwkit_lightning.py:384-410, 412-517)."""

    @staticmethod
    def forward(ctx, layer, x, w_sel, keys, values, input_range):
        import os
        cfg = layer.rpu_config
        fwd, ir_p = cfg.forward, cfg.pre_post.input_range
        bsz, seq, D = x.shape
        k, E = layer.n_heads, layer.n_experts
        T = bsz * seq
        P = T * k
        x2 = x.reshape(T, D)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        precision = layer._precision(x)
        per_channel = layer._scale_per_channel()

        clip = layer._take_pending_clip()       # weight clipping left over from post_update_step, done in the pre-pass

        def prepass(w, mod, trained):
            # unchanged weights of a call that does not train them: prepared once (a training loop may write weights in
            # ways the version counter does not see, so a call that wants their gradient always prepares them)
            if mod is None and not clip and not trained:
                return ops.weight_prepass_cached(w, precision, per_channel)
            return ops.weight_prepass(
                w, precision, per_channel_scale=per_channel, noise_std=mod.std_dev if mod else 0.0,
                noise_per_channel=mod.per_channel if mod else True, discretize_res=mod.discretize_res if mod else -1.0,
                seed=mod.seed if mod else 0, offset=mod.offset if mod else 0, step_dev=mod.step if mod else None,
                need_fwd=True, need_bwd=True, **clip)

        def noise_args():
            std = layer._out_noise_std()
            if std > 0:
                return dict(noise_std=std, seed=layer.noise_seed, offset=layer._next_offset(), step_dev=layer.noise_step)
            return {}

        # The two weight pre-passes depend on nothing but the weights: they run on two streams of their own beside the
        # router matmul and the select/sort (small kernels that leave most of the GPU idle).  Side by side rather than one
        # after the other: what has not finished when the operand pre-pass and the up-projection take every SM waits
        # for them to end, and the down-projection then waits for its weights.
        nz_up = noise_args()
        mod_up = layer._weight_modifier()
        nz_dn = noise_args()
        mod_dn = layer._weight_modifier()
        main, side, side2 = torch.cuda.current_stream(), ops.side_stream(x.device), ops.side_stream(x.device, 1)
        side.wait_stream(main)
        side2.wait_stream(main)
        with ops.launch_on(side):
            ops.set_tag("up")
            pw_up = prepass(keys, mod_up, bool(ctx.needs_input_grad[3]))
            up_ready = side.record_event()      # the up-projection only waits for its own weights
        with ops.launch_on(side2):
            ops.set_tag("down")
            pw_dn = prepass(values, mod_dn, bool(ctx.needs_input_grad[4]))
        ops.set_tag("up")
        r, _ = ops.router_select(x2, w_sel, k, getattr(layer, "router_bias", None))
        inp_res = float(layer._inp_res())
        if os.environ.get("_AIHWKIT_NO_ROUNDING", False):
            assert os.environ.get("AIHWKIT_TESTING", False), "Skipping rounding but AIHWKIT_TESTING not set"
            inp_res = -1.0
        adc_on = fwd.out_res > 0 and fwd.out_bound > 0
        out_res, out_bound = (float(fwd.out_res), float(fwd.out_bound)) if adc_on else (-1.0, -1.0)
        has_ir = input_range is not None
        ir_all = input_range.detach().float().contiguous() if has_ir else None

        # ---- up-projection (+ ReLU)
        nz = nz_up
        ir_up = ir_all[0] if has_ir else None
        use_am = _uses_abs_max(ir_p, fwd)
        am_up = ops.row_absmax(x2) if use_am else None
        # operands of the two weight gradients, written while the forward kernels hold the rows anyway
        N = values.shape[-1]
        Fh = keys.shape[-1]
        cached = layer.operand_caches and ops.operand_cache_ok(precision, D, Fh, N) and \
            any(ctx.needs_input_grad[3:5])
        split = precision == ops.A.PREC_SPLIT
        pre_up = layer.operand_prepass and ops.operand_tiles_ok(x2, precision)
        xc = ops.OperandCache.empty(P, E, D, split, x.device) if (cached and not pre_up) else None
        hs = ops.OperandCache.empty(P, E, Fh, split, x.device) if cached else None
        # With input ranges and a quantising DAC the up-projection's epilogue also leaves the hidden rows as the
        # down-projection wants them (integer DAC codes as bf16 tiles, and gate * clamp(h) for its weight gradient),
        # so that the down-projection loads its A operand by TMA and runs no prologue.
        gate = r.gate if x.dtype == torch.float32 else r.gate.to(x.dtype).float()
        tiles = has_ir and inp_res >= 1.0 / 256.0 and Fh % 64 == 0 and precision != ops.A.PREC_FP32_SIMT and \
            layer.hidden_tiles          # (codes up to 256 in magnitude are exact in one bf16 term)
        hq = ops.OperandCache.empty(P, E, Fh, False, x.device) if tiles else None
        nxt = dict(next_ir=ir_all[1], next_inp_res=inp_res, next_codes=hq, out_cache=hs,
                   out_cache_scale=gate.reshape(-1) if hs is not None else None) if tiles else {}
        # The DAC of the gathered input rows runs as a streaming pass of its own (full occupancy, HBM-bound) that leaves
        # the codes as TMA tiles and the clamped rows as the weight gradient's operand; the tensor-core kernel then
        # runs no operand prologue.
        if pre_up:
            xq, xc_pre = ops.operand_tiles(x2, r.token_index, r.expert_offsets, E, precision, P=P, dac=True, ir=ir_up,
                                           ir_by_expert=True, absmax=am_up, inp_res=inp_res, want_cache=cached)
            if cached:
                xc = xc_pre
            a_kw = dict(a_tiles=xq)
        else:
            a_kw = dict(a_cache=xc)
        main.wait_event(up_ready)       # (only now: the operand pre-pass above does not read the weights)
        h, _ = ops.cvmm_fwd(x2, r.token_index, r.slot_index, r.expert_offsets, pw_up, precision, P=P, dst_rows=P,
                            ir=ir_up, ir_by_expert=True, absmax=am_up, inp_res=inp_res, out_res=out_res,
                            out_bound=out_bound, out_relu=True, **a_kw, **nxt, **nz)
        # ---- down-projection and the gate-weighted sum over k
        main.wait_stream(side)
        main.wait_stream(side2)
        ops.set_tag("down")
        nz = nz_dn
        ir_dn = ir_all[1] if has_ir else None
        am_dn = ops.row_absmax(h) if use_am else None
        # (the composition hands the gate over in the activation dtype: rounded for bf16 layers)
        if tiles:
            cache_kw = dict(a_tiles=hq)
        else:
            cache_kw = dict(a_cache=hs, a_cache_scale=gate.reshape(-1)) if cached else {}
        adc_step = ops.adc_step(out_res, out_bound) if adc_on else 0.0
        res = codes = row_scale = row_expert = None
        if adc_on:
            meta = {}
            _, codes = ops.cvmm_fwd(h, r.slot_index, r.slot_index, r.expert_offsets, pw_dn, precision, P=P, dst_rows=P,
                                    ir=ir_dn, ir_by_expert=True, absmax=am_dn, inp_res=inp_res, out_res=out_res,
                                    out_bound=out_bound, want_codes=True, want_out=False, row_meta=meta, **cache_kw,
                                    **nz)
            row_scale, row_expert = meta["row_scale"], meta["row_expert"]
            if layer.keep_codes:
                layer.last_codes = codes
            y = ops.combine_codes(codes, pw_dn.col_scale, row_expert, row_scale, adc_step, gate, T, k, out_dtype=x.dtype)
        else:
            res, _ = ops.cvmm_fwd(h, r.slot_index, r.slot_index, r.expert_offsets, pw_dn, precision, P=P, dst_rows=P,
                                  ir=ir_dn, ir_by_expert=True, absmax=am_dn, inp_res=inp_res, **cache_kw, **nz)
            y = ops.combine(res, gate, T, k)
        simt = precision == ops.A.PREC_FP32_SIMT
        ctx.save_for_backward(x2, w_sel, h, gate, r.raw_sel, r.token_index, r.slot_index, r.expert_offsets, ir_all,
                              pw_up.w if simt else None, pw_up.bwd_hi, pw_up.bwd_lo, pw_up.col_scale,
                              pw_dn.w if simt else None, pw_dn.bwd_hi, pw_dn.bwd_lo, pw_dn.col_scale,
                              codes, row_scale, row_expert, res,
                              *((xc.hi, xc.lo, hs.hi, hs.lo) if cached else (None, None, None, None)))
        ctx.operand_prepass = layer.operand_prepass
        ctx.meta = (x.shape, E, k, precision, ir_p, keys.dtype, values.dtype, adc_step, keys.shape, values.shape,
                    input_range.dtype if has_ir else None)
        return y.view(bsz, seq, N)

    @staticmethod
    def backward(ctx, gy):
        (x2, w_sel, h, gate, raw_sel, token_index, slot_index, offsets, ir_all, w_up, up_hi, up_lo, up_cs,
         w_dn, dn_hi, dn_lo, dn_cs, codes, row_scale, row_expert, res, xc_hi, xc_lo, hs_hi, hs_lo) = ctx.saved_tensors
        cached = xc_hi is not None
        x_shape, E, k, precision, ir_p, keys_dtype, values_dtype, adc_step, kshape, vshape, ir_dtype = ctx.meta
        T, D = x2.shape
        P = T * k
        Fh, N = vshape[1], vshape[2]
        need_x, need_sel, need_keys, need_values, need_ir = (ctx.needs_input_grad[i] for i in (1, 2, 3, 4, 5))
        has_ir = ir_all is not None
        need_ir = need_ir and has_ir
        g = gy.reshape(T, N)
        if g.stride(-1) != 1:
            g = g.contiguous()
        pw_up = ops.PreparedWeights(E, kshape[1], kshape[2], up_cs, w=w_up, bwd_hi=up_hi, bwd_lo=up_lo)
        pw_dn = ops.PreparedWeights(E, vshape[1], vshape[2], dn_cs, w=w_dn, bwd_hi=dn_hi, bwd_lo=dn_lo)
        decay = float(getattr(ir_p, "decay", 0.0) or 0.0) if has_ir else 0.0
        min_pct = float(getattr(ir_p, "input_min_percentage", 0.95))
        relative = bool(getattr(ir_p, "gradient_relative", True))
        gscale = float(getattr(ir_p, "gradient_scale", 1.0)) if relative else 1.0
        keeps = torch.zeros(2, dtype=torch.int64, device=x2.device) if (has_ir and decay > 0) else None
        ir_up, ir_dn = (ir_all[0], ir_all[1]) if has_ir else (None, None)

        # ---- gate gradient and the router's weight gradient: they need only the saved codes and the upstream gradient, so
        # they start at once on the second stream, beside the light kernels that open the main chain (max|gy|, the
        # operand pre-pass), instead of queueing behind the input-gradient kernels
        main, side = torch.cuda.current_stream(), ops.side_stream(x2.device)
        side.wait_stream(main)
        grad_sel = None
        with ops.launch_on(side):
            ops.set_tag("down")
            if codes is not None:
                dgate = ops.row_dot_codes(codes, dn_cs, row_expert, row_scale, adc_step, g, k)
            else:
                dgate = ops.row_dot(res, g, k)
            dgate_ready = side.record_event()
            # (routers too large for the shared-memory kernel go through torch glue on the main stream further down)
            sel_early = need_sel and ops._router_fits_smem(w_sel.shape[0], D)
            if sel_early:
                ops.set_tag("up")
                grad_sel = ops.router_backward_w(x2, dgate, gate, token_index, slot_index, offsets, w_sel.shape[0],
                                                 raw_sel=raw_sel)
        # ---- down-projection
        ops.set_tag("down")
        grad_values = None
        if need_values and not cached:
            grad_values = ops.cvmm_dw(h, slot_index, g, slot_index, offsets, E, precision, P=P, ir=ir_dn,
                                      ir_by_expert=True, g_div=k, g_scale=gate.reshape(-1),
                                      g_absmax=ops.grad_absmax(g, precision))
        split = xc_lo is not None
        # the upstream gradient rows, gathered per slot and converted by the operand pre-pass: the A tiles of the input
        # gradient below and the weight gradient's operand at once
        pre_dn = ctx.operand_prepass and ops.operand_tiles_ok(g, precision)
        gc = ops.OperandCache.empty(P, E, N, split, x2.device) if cached and need_values and not pre_dn else None
        dhc = ops.OperandCache.empty(P, E, Fh, split, x2.device) if cached and need_keys else None
        # fp16 operands: one scalar (max|gy|) scales every gradient operand of the step into fp16's normal range
        gmax = ops.grad_absmax(g, precision)
        # the hidden gradient is only needed as fp32 rows when the next kernel cannot take it as tiles
        tiles_next = dhc is not None and Fh % 64 == 0 and (need_x or need_ir)
        if pre_dn:
            gc, _ = ops.operand_tiles(g, slot_index, offsets, E, precision, P=P, a_row_div=k, dac=False, g_absmax=gmax)
            a_kw = dict(a_tiles=gc)
        else:
            a_kw = dict(a_cache=gc)
        dh, irs_dn = ops.cvmm_dx(g, slot_index, slot_index, offsets, pw_dn, precision, P=P, dst_rows=P, a_row_div=k,
                                 x_ref=h, x_ref_row=slot_index, ir=ir_dn, ir_by_expert=True, row_scale=gate.reshape(-1),
                                 want_ir_grad=has_ir, relative=relative, grad_scale=gscale,
                                 keep_count=keeps[1:] if keeps is not None else None, out_dtype=h.dtype,
                                 x_ref_relu=True, out_cache=dhc, g_absmax=gmax, want_out=not tiles_next, **a_kw)
        # ---- up-projection's input gradient (the other kernel that fills every SM), then the two weight gradients from
        # the caches on a second stream: the TMA-fed kernel runs six warps per SM and leaves registers and issue slots
        # to the streaming kernels of the main stream (gate gradient, sum over k, router), which run beside it
        ops.set_tag("up")
        grad_x = irs_up = dxr = None
        if need_x or need_ir:
            # the hidden gradient already exists as bf16 hi/lo tiles (the dW operand the kernel above wrote): TMA feeds
            # it, no gather/convert prologue
            tiles = dhc if (dhc is not None and Fh % 64 == 0) else None
            dxr, irs_up = ops.cvmm_dx(dh if dh is not None else h, slot_index, slot_index, offsets, pw_up, precision, P=P,
                                      dst_rows=P, x_ref=x2 if has_ir else None, x_ref_row=token_index if has_ir else None,
                                      ir=ir_up, ir_by_expert=True, want_ir_grad=has_ir, relative=relative,
                                      grad_scale=gscale, keep_count=keeps[:1] if keeps is not None else None,
                                      out_dtype=x2.dtype, a_tiles=tiles, g_absmax=gmax)
        grad_keys = None
        forked = cached and (need_values or need_keys)
        side2 = ops.side_stream(x2.device, 1)
        if forked:
            # each weight gradient is a TMA-fed kernel followed by the ordered sum of its partial tiles: on two streams
            # the second kernel starts while the first one's partial tiles are being summed
            side.wait_stream(main)
            side2.wait_stream(main)
            if need_values:
                with ops.launch_on(side):
                    # dW = sum_slots (gate * clamp(h))^T (x) gy: both operands straight from the caches
                    ops.set_tag("down")
                    grad_values = ops.cvmm_dw_cached(ops.OperandCache(hs_hi, hs_lo, Fh), gc, offsets, E, precision, P=P,
                                                     g_absmax=gmax)
            if need_keys:
                with ops.launch_on(side2):
                    ops.set_tag("up")
                    grad_keys = ops.cvmm_dw_cached(ops.OperandCache(xc_hi, xc_lo, D), dhc, offsets, E, precision, P=P,
                                                   g_absmax=gmax)
        elif need_keys:
            # (the hidden gradient's own magnitude scales it here: it is gathered from fp32 rows)
            grad_keys = ops.cvmm_dw(x2, token_index, dh, slot_index, offsets, E, precision, P=P, ir=ir_up,
                                    ir_by_expert=True, g_absmax=ops.grad_absmax(dh, precision))
        # ---- input-range gradients: two small reductions over the per-slot sums the input-gradient kernels left, on a
        # stream of their own beside the last large kernel of the main chain instead of behind it
        grad_ir = None
        side3 = None
        if need_ir:
            side3 = ops.side_stream(x2.device, 2)
            side3.wait_stream(main)
            grad_ir = torch.empty(2, E, dtype=torch.float32, device=x2.device)      # both rows written in place
            with ops.launch_on(side3):
                ops.set_tag("up")
                ops.ir_grad_reduce(irs_up, offsets, ir_up, E, decay, min_pct, keeps[:1] if keeps is not None else None,
                                   float(P) * D, out=grad_ir[0])
                ops.ir_grad_reduce(irs_dn, offsets, ir_dn, E, decay, min_pct, keeps[1:] if keeps is not None else None,
                                   float(P) * Fh, out=grad_ir[1])
        main.wait_event(dgate_ready)
        ops.set_tag("up")
        if need_x:
            # sum over k plus the router's own input gradient in one pass
            grad_x = ops.combine_router(dxr, T, k, dgate, gate, raw_sel, w_sel)
        # ---- router
        if need_sel and not sel_early:
            grad_sel = ops.router_backward_w(x2, dgate, gate, token_index, slot_index, offsets, w_sel.shape[0],
                                             raw_sel=raw_sel)
        if side3 is not None:
            main.wait_stream(side3)
            grad_ir = grad_ir.to(ir_dtype)
        main.wait_stream(side)
        main.wait_stream(side2)
        if grad_sel is not None:
            grad_sel = grad_sel.to(w_sel.dtype)
        if grad_values is not None:
            grad_values = grad_values.to(values_dtype)
        if grad_keys is not None:
            grad_keys = grad_keys.to(keys_dtype)
        return (None, grad_x.view(x_shape) if need_x else None, grad_sel, grad_keys, grad_values, grad_ir)


class MoEConifgError(Exception):
    """Configuration the analog sigma-MoE layers do not support (name as in the reference layers, :25/:29)."""


# --------------------------------------------------------------------------- checkpoint formats
# A non-traceable layer stores `input_range` [2, E] and a scalar `input_range_update_idx`; the reference's traceable
# mode stores one analog linear module per expert instead, each with its own `input_range` [1],
# `input_range_update_idx` [1], `x_min` [1], `x_max` [1] (reference moe_layer_aihwkit_lightning.py:33-131).

def non_traceable_to_traceable(state_dict, prefix: str) -> None:
    """In place: `input_range`/`input_range_update_idx` of a non-traceable layer as per-expert entries."""
    ir = state_dict.pop(prefix + "input_range")
    idx = state_dict.pop(prefix + "input_range_update_idx")
    for row, name in enumerate(("keys", "values")):
        for e in range(ir.shape[1]):
            base = f"{prefix}{name}.{e}."
            state_dict[base + "input_range"] = ir[row, e].reshape(1)
            state_dict[base + "input_range_update_idx"] = idx.reshape(1)
            state_dict[base + "x_min"] = torch.zeros(1, device=ir.device, dtype=ir.dtype)
            state_dict[base + "x_max"] = torch.zeros(1, device=ir.device, dtype=ir.dtype)


def traceable_to_non_traceable(state_dict, prefix: str) -> None:
    """In place: per-expert entries of a traceable checkpoint as `input_range` [2, E] and one update index."""
    pat = re.compile(rf"^{re.escape(prefix)}(keys|values)\.(\d+)\.(input_range|input_range_update_idx|x_min|x_max)$")
    found = {}
    for name in list(state_dict):
        m = pat.match(name)
        if m:
            found[(m.group(1), int(m.group(2)), m.group(3))] = name
    experts = sorted({e for (_, e, _) in found})
    rows = []
    for which in ("keys", "values"):
        rows.append(torch.cat([state_dict[found[(which, e, "input_range")]].reshape(1) for e in experts]))
    first_idx = state_dict[found[("keys", experts[0], "input_range_update_idx")]]
    for name in found.values():
        state_dict.pop(name)
    state_dict[prefix + "input_range"] = torch.stack(rows)
    state_dict[prefix + "input_range_update_idx"] = first_idx.reshape(())


def _convert_checkpoint_format(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs,
                               traceable: bool = False) -> None:
    """Load pre-hook (reference moe_layer_aihwkit_lightning.py:107-131): bring the input-range entries into the format
    of the layer that is loading them."""
    if not any("input_range" in k for k in state_dict):
        return
    is_non_traceable = prefix + "input_range" in state_dict
    if traceable and is_non_traceable:
        non_traceable_to_traceable(state_dict, prefix)
    elif not traceable and not is_non_traceable:
        traceable_to_non_traceable(state_dict, prefix)


class SigmaMoELayer(nn.Module):
    def __init__(self, d_model: int, n_experts: int, expert_size: int, k: int, dropout: float = 0.0,
                 selection_mode: str = "sigmoid", activation_after_topk: bool = False,
                 activation: Callable = F.relu, bias: bool = False, v_dim: Optional[int] = None,
                 sinkhorn_n_iters: int = 3, expert_dropout: float = 0.0, traceable: bool = False):
        super().__init__()
        if selection_mode != "sigmoid":
            raise NotImplementedError("only sigmoid gating is built")
        if traceable:
            raise NotImplementedError("traceable mode delegates to third-party per-expert modules; not built")
        self.k_dim = d_model
        self.v_dim = v_dim if v_dim is not None else d_model
        self.n_experts = n_experts
        self.expert_size = expert_size
        self.size = n_experts * expert_size
        self.dropout = dropout
        self.selection_mode = selection_mode
        self.activation_after_topk = activation_after_topk
        self.activation = activation
        self.sinkhorn_n_iters = sinkhorn_n_iters
        self.expert_dropout = expert_dropout
        self.n_heads = k
        self.traceable = traceable
        self.keys = nn.Parameter(torch.empty(n_experts, self.k_dim, expert_size))
        self.values = nn.Parameter(torch.empty(n_experts, expert_size, self.v_dim))
        self.expert_sel = nn.Linear(self.k_dim, n_experts, bias=False)
        self.bias = nn.Parameter(torch.zeros(n_experts, expert_size)) if bias else None
        self.o_bias = nn.Parameter(torch.zeros(self.v_dim)) if bias else None
        nn.init.normal_(self.keys, std=self.k_dim ** -0.5)
        nn.init.normal_(self.values, std=expert_size ** -0.5)
        nn.init.normal_(self.expert_sel.weight, std=self.k_dim ** -0.5)

    # -- the two hooks the analog layer overrides
    def cvmm_wrapper(self, inputs: Tensor, sel_indices: CVMMSel, weights: Tensor) -> Tensor:
        class _Off:
            enable = False
        return CVMM.apply(inputs, sel_indices.sel_index, sel_indices.sel, weights, -1, None, sel_indices.out_index,
                          sel_indices.reduction_weight, None, None, None,
                          CVMMExt(expert_offsets=sel_indices.expert_offsets, precision=self._precision(inputs)))

    def _precision(self, inputs: Tensor) -> int:
        return ops.default_precision(inputs.dtype)

    def compute_scores(self, inp: Tensor, index: CVMMSel, expert_scores: Optional[Tensor] = None) -> Tensor:
        if not inp.is_cuda:
            raise RuntimeError("the sigma-MoE layer runs on CUDA tensors only")
        scores = self.cvmm_wrapper(inp, index, self.keys)
        if self.bias is not None:
            scores = scores + self.bias[index.raw_sel.long()]
        scores = self.activation(scores)
        if expert_scores is not None:
            scores = scores * expert_scores[..., None]
        if self.dropout > 0:
            scores = F.dropout(scores, self.dropout, training=self.training)
        return scores

    def route(self, inp: Tensor) -> Tuple[CVMMSel, Tensor]:
        """Gate logits -> sigmoid -> top-k -> expert-sorted slot list, one kernel pipeline."""
        logits = self.expert_sel(inp)
        if getattr(self, "router_bias", None) is not None:      # fixed per-expert logit offset (skew studies)
            logits = logits + self.router_bias
        bsz, seq, _ = inp.shape
        raw_sel, _, ssel, token_index, slot_index, offsets = select_sort_op(logits.detach(), self.n_heads, True)
        raw_sel = raw_sel.view(bsz, seq, self.n_heads)
        # gate values with gradient: recompute the k picked sigmoids from the logits (tiny gather)
        gate = torch.sigmoid(logits.float()).gather(-1, raw_sel.long()).to(inp.dtype)
        sel = CVMMSel(raw_sel, ssel.view(bsz, seq, self.n_heads), token_index, slot_index, None, offsets)
        return sel, gate

    def forward(self, inp: Tensor) -> Tuple[Tensor, Tensor]:
        sel, gate = self.route(inp)
        scores = self.compute_scores(inp, sel)
        down = sel.clone()
        down.reduction_weight = gate
        down.sel_index = sel.out_index
        down.out_index = None
        out = self.cvmm_wrapper(scores, down, self.values)
        if self.o_bias is not None:
            out = out + self.o_bias
        return out, inp.new_zeros(())


class AnalogSigmaMoELayer(SigmaMoELayer):
    def __init__(self, rpu_config: Optional[TorchInferenceRPUConfig] = None, *args, precision: Optional[int] = None,
                 noise_seed: int = 0, **kwargs):
        super().__init__(*args, **kwargs)
        self.rpu_config = rpu_config if rpu_config is not None else TorchInferenceRPUConfig()
        fwd = self.rpu_config.forward
        adc_on = fwd.out_res > 0
        if adc_on and not fwd.out_bound > 0:
            raise ValueError("ADC output quantisation (out_res > 0) needs out_bound > 0")
        assert self.rpu_config.mapping.max_input_size <= 0, "max_input_size must be <= 0"   # lightning :158-160
        self.precision = precision
        self.noise_seed = noise_seed
        self.register_buffer("noise_step", torch.zeros((), dtype=torch.int64), persistent=True)
        self.register_buffer("_aux_zero", torch.zeros(()), persistent=False)
        self.fused = True          # one autograd node for the whole layer when the configuration allows it
        self.operand_caches = True  # forward / dX kernels leave bf16 copies of the dW operands (fused path)
        self.hidden_tiles = True    # the up-projection leaves the hidden rows as the down-projection's A tiles
        self.operand_prepass = True  # DAC of gathered rows as a streaming pass; the CVMM kernels load A tiles by TMA
        self.fuse_clip = False      # post_update_step only records the clipping; the next forward's weight pre-pass
                                    # clips in place while it reads the weights anyway (until then they are unclipped)
        self._pending_clip = None
        self.keep_codes = False     # keep the down-projection's ADC codes (int8, by flat slot) on `last_codes`
        self.last_codes = None
        self._noise_calls = 0
        self._register_load_state_dict_pre_hook(partial(_convert_checkpoint_format, traceable=False))
        ir = self.rpu_config.pre_post.input_range
        self.input_range = None
        if ir.enable:
            self.input_range_update_idx = nn.Parameter(torch.tensor(0.0), requires_grad=False)
            init = torch.full((2, self.n_experts), float(ir.init_value))
            if ir.learn_input_range:
                self.input_range = nn.Parameter(init)
            else:
                del self.input_range
                self.register_buffer("input_range", init)

    @classmethod
    def from_digital(cls, module: SigmaMoELayer, rpu_config: TorchInferenceRPUConfig) -> "AnalogSigmaMoELayer":
        layer = cls(rpu_config, d_model=module.k_dim, n_experts=module.n_experts, expert_size=module.expert_size,
                    k=module.n_heads, dropout=module.dropout, selection_mode=module.selection_mode,
                    activation_after_topk=module.activation_after_topk, activation=module.activation,
                    bias=module.bias is not None, v_dim=module.v_dim, sinkhorn_n_iters=module.sinkhorn_n_iters,
                    expert_dropout=module.expert_dropout, traceable=module.traceable)
        layer.load_state_dict(module.state_dict(), strict=False)
        return layer.to(module.keys.device)

    def _precision(self, inputs: Tensor) -> int:
        return self.precision if self.precision is not None else ops.default_precision(inputs.dtype)

    # -- what the two reference layers decide differently lives in these four methods
    def _inp_res(self) -> float:
        """lightning :451-456: 254 -> 2/254 = 1/127; values below 1 are a resolution already."""
        inp_res = self.rpu_config.forward.inp_res
        return (2.0 / inp_res if inp_res > 1.0 else 2.0 * inp_res) if inp_res > 0 else -1

    def _out_noise_std(self) -> float:
        """lightning :472: output noise only while training."""
        std = float(self.rpu_config.forward.out_noise)
        return std if (self.training and std > 0) else 0.0

    def _scale_per_channel(self) -> bool:
        """Per-column (True) or per-expert weight maximum as the scale of output noise and ADC (lightning :480-487)."""
        return bool(getattr(self.rpu_config.forward, "out_noise_per_channel", True))

    def _weight_modifier(self) -> Optional[WeightModifier]:
        """lightning :313-382 as parameters of the weight pre-pass.  The per-channel variants use the per-column
        maximum; the reference's lightning layer leaves ADD_NORMAL_PER_CHANNEL out of its per-channel list (:334-338)
        and so falls back to the per-expert maximum for that type, which is not reproduced here."""
        mod = self.rpu_config.modifier
        name = _enum_name(mod.type)
        if name in ("NONE", "None") or not (self.training or mod.enable_during_test):
            return None
        per_channel = name.endswith("PER_CHANNEL")
        disc = float(mod.res) if name.startswith("DISCRETIZE") else -1.0
        std = float(mod.std_dev) if "ADD_NORMAL" in name else 0.0
        return WeightModifier(std_dev=std, per_channel=per_channel, discretize_res=disc, seed=self.noise_seed,
                              offset=self._next_offset(), step=self.noise_step)

    def _next_offset(self) -> int:
        # Philox offset = call index inside the step + 8 * noise_step, where noise_step is a device
        # counter the kernels read: a CUDA graph of the step draws fresh noise on every replay, and
        # a resumed run that restores `noise_step` replays its noise.
        self._noise_calls += 1
        return self._noise_calls & 7

    def cvmm_wrapper(self, inputs: Tensor, sel_indices: CVMMSel, weights: Tensor) -> Tensor:
        cfg = self.rpu_config
        ir_p = cfg.pre_post.input_range
        bir = None
        if self.input_range is not None:
            ir_idx = 0 if inputs.ndim == 3 else 1                                   # lightning :428-429
            if self.training and ir_p.init_from_data > 0 and float(self.input_range_update_idx) < ir_p.init_from_data:   # lightning :432-445
                idx = self.input_range_update_idx
                stds = cvmm_std(inputs, sel_indices.sel_index, sel_indices.sel, self.n_experts)
                ok = stds > 0.0
                if bool(ok.any()):
                    cur = self.input_range.data[ir_idx]
                    cur[ok] = (cur[ok] * idx + ir_p.init_std_alpha * stds[ok].to(cur.dtype)) / (idx + 1)
                    self.input_range_update_idx.data += 1
                self.input_range.data = self.input_range.data.abs()
            if sel_indices.expert_offsets is not None and self.input_range.dtype == torch.float32:
                bir = _BroadcastInputRange.apply(self.input_range[ir_idx], sel_indices.sel, sel_indices.expert_offsets)
            else:
                bir = self.input_range[ir_idx][sel_indices.sel.long()]              # lightning :447-448
        inp_res = self._inp_res()
        noise = None
        std = self._out_noise_std()
        if std > 0:                                                                 # lightning :471-492
            noise = PhiloxNoise(std, self.noise_seed, self._next_offset(), self.noise_step)
        ext = CVMMExt(noise=noise, modifier=self._weight_modifier(), out_res=float(cfg.forward.out_res),
                      out_bound=float(cfg.forward.out_bound), scale_per_channel=self._scale_per_channel(),
                      precision=self._precision(inputs), expert_offsets=sel_indices.expert_offsets)
        return CVMM.apply(inputs, sel_indices.sel_index, sel_indices.sel, weights, inp_res, bir,
                          sel_indices.out_index, sel_indices.reduction_weight, None, ir_p, cfg.forward, ext)

    def _fused_ok(self, inp: Tensor) -> bool:
        """The single-node path covers the common configuration; anything else takes the composition."""
        if not self.fused or type(self).cvmm_wrapper is not AnalogSigmaMoELayer.cvmm_wrapper:
            return False
        if torch.compiler.is_compiling():
            return False          # under torch.compile the layer is the composition of traceable operators
        if self.input_range is not None and _uses_abs_max(self.rpu_config.pre_post.input_range, self.rpu_config.forward):
            return False          # input range and abs-max scaling together (classic aihwkit, noise_management=ABS_MAX)
        if not (inp.is_cuda and inp.ndim == 3 and _is_relu(self.activation)) or self.bias is not None:
            return False
        if self.dropout > 0 and self.training:
            return False
        if torch.is_autocast_enabled() or inp.dtype not in (torch.float32, torch.bfloat16):
            return False
        ir_p = self.rpu_config.pre_post.input_range
        if self.input_range is not None and self.training and ir_p.init_from_data > 0 and \
                float(self.input_range_update_idx) < ir_p.init_from_data:
            return False          # the data-driven initialisation of the input ranges runs in the composition
        return True

    def forward(self, inp: Tensor) -> Tuple[Tensor, Tensor]:
        self._noise_calls = 0
        fused = self._fused_ok(inp)
        if self._pending_clip is not None and not fused:
            c = self._take_pending_clip()
            for w in (self.keys, self.values):
                ops.clip_weights_(w.data, sigma=c["clip_sigma"], per_channel=c["clip_per_channel"],
                                  fixed_value=c["clip_fixed"])
        if fused:
            y = _FusedAnalogStep.apply(self, inp, self.expert_sel.weight, self.keys, self.values, self.input_range)
            out = (y, self._aux_zero)
        else:
            out = super().forward(inp)
        if self.training:
            self.noise_step += 1
        return out

    def post_update_step(self) -> None:
        if _enum_name(self.rpu_config.clip.type) not in ("NONE", "None"):
            self.clip_weights()

    def _clip_args(self) -> Optional[dict]:
        """lightning :519-543 as arguments of the weight pre-pass: clamp to +-sigma*std per expert (LAYER_GAUSSIAN) or
        per column (LAYER_GAUSSIAN_PER_CHANNEL)."""
        clip = self.rpu_config.clip
        name = _enum_name(clip.type)
        if name in ("NONE", "None"):
            return None
        assert clip.sigma > 0, "Clip sigma must be greater than 0"
        if name not in ("LAYER_GAUSSIAN", "LAYER_GAUSSIAN_PER_CHANNEL"):
            raise ValueError(f"Unknown clip type {clip.type}")
        return dict(clip_sigma=float(clip.sigma), clip_per_channel=name.endswith("PER_CHANNEL"), clip_fixed=-1.0)

    def _take_pending_clip(self) -> dict:
        c, self._pending_clip = self._pending_clip, None
        return c or {}

    @torch.no_grad()
    def clip_weights(self, clip=None) -> None:
        """Statistics and clamp run in the library's weight pre-pass kernels; with `fuse_clip` they wait for the
        pre-pass of the next forward."""
        args = self._clip_args()
        if args is None:
            return
        if self.fuse_clip:
            self._pending_clip = args
            return
        for w in (self.keys, self.values):
            ops.clip_weights_(w.data, sigma=args["clip_sigma"], per_channel=args["clip_per_channel"],
                              fixed_value=args["clip_fixed"])

    # -- checkpoints: the configuration travels in the state dict's metadata (lightning :545-570)
    def _save_to_state_dict(self, destination, prefix, keep_vars):
        super()._save_to_state_dict(destination, prefix, keep_vars)
        destination._metadata[prefix.split(".")[0]]["rpu_config"] = self.rpu_config

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        # a checkpoint written by the reference has no Philox step counter: keep the current one
        state_dict.setdefault(prefix + "noise_step", self.noise_step)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)
        if "rpu_config" in local_metadata:
            self.rpu_config = local_metadata["rpu_config"]


# The reference's name for the aihwkit-lightning flavour of the layer (moe_layer_aihwkit_lightning.py:134).
AnalogSigmaMoELayerAIHWKITLightning = AnalogSigmaMoELayer


class AnalogSigmaMoELayerAIHWKIT(AnalogSigmaMoELayer):
    """The classic-aihwkit flavour (reference moe_layer_aihwkit.py:28-437): same kernels, different configuration
    policy - the weight maximum that scales weight and output noise follows `remap.type`, `forward.is_perfect`
    switches quantisation and noise off, abs-max input scaling follows `forward.noise_management`, clipping knows
    FIXED_VALUE, and the configuration is stored as an `analog_tile_state` entry of the state dict."""

    def __init__(self, rpu_config: Optional[TorchInferenceRPUConfig] = None, *args, **kwargs):
        cfg = rpu_config if rpu_config is not None else aihwkit_rpu_config()
        fwd = cfg.forward
        # reference :47-61 (the two out_* asserts are gone: the ADC is implemented here)
        assert getattr(fwd, "inp_bound", 1.0) in [-1, 1.0], "inp_bound must be 1.0 or off (=-1)"
        assert cfg.mapping.max_input_size == 0, "max_input_size must be 0"
        assert getattr(cfg.mapping, "max_output_size", 0) == 0, "max_output_size must be 0"
        assert _enum_name(getattr(fwd, "bound_management", "NONE")) in ("NONE", "None"), "bound_management must be NONE"
        super().__init__(cfg, *args, **kwargs)
        # aihwkit hangs an `analog_ctx` parameter on every analog layer (reference :141-142); it carries no data the
        # kernels use, but checkpoints contain the entry
        self.analog_ctx = nn.Parameter(torch.ones(()), requires_grad=False)

    def _perfect(self) -> bool:
        return bool(getattr(self.rpu_config.forward, "is_perfect", False))

    def _remap(self) -> str:
        return _enum_name(self.rpu_config.remap.type)

    def _inp_res(self) -> float:
        return -1 if self._perfect() else super()._inp_res()                          # reference :247-249

    def _out_noise_std(self) -> float:
        return 0.0 if self._perfect() else super()._out_noise_std()                    # reference :257-261

    def _scale_per_channel(self) -> bool:
        remap = self._remap()                                                         # reference :267-282
        if remap in ("CHANNELWISE_SYMMETRIC", "NONE", "None"):
            return True
        if remap == "LAYERWISE_SYMMETRIC":
            return False
        raise MoEConifgError(f"Weight remap type {self.rpu_config.remap.type} not supported")

    def _weight_modifier(self) -> Optional[WeightModifier]:
        mod = self.rpu_config.modifier                                                # reference :144-196
        if not (self.training or mod.enable_during_test):
            return None
        if getattr(mod, "per_batch_sample", False):
            raise MoEConifgError("per_batch_sample not implemented")
        name = _enum_name(mod.type)
        if name in ("NONE", "None", "COPY"):
            return None
        if name != "ADD_NORMAL":
            raise MoEConifgError(f"Weight modifier {mod.type} not supported")
        remap = self._remap()
        if remap not in ("CHANNELWISE_SYMMETRIC", "LAYERWISE_SYMMETRIC"):
            raise MoEConifgError(f"Weight remap type {self.rpu_config.remap.type} not supported")
        return WeightModifier(std_dev=float(mod.std_dev), per_channel=remap == "CHANNELWISE_SYMMETRIC",
                              seed=self.noise_seed, offset=self._next_offset(), step=self.noise_step)

    def _clip_args(self) -> Optional[dict]:
        """reference :314-340."""
        clip = self.rpu_config.clip
        name = _enum_name(clip.type)
        if name in ("NONE", "None"):
            return None
        if name == "FIXED_VALUE":
            return dict(clip_sigma=-1.0, clip_per_channel=False, clip_fixed=float(clip.fixed_value))
        if name == "LAYER_GAUSSIAN":
            return dict(clip_sigma=float(clip.sigma), clip_per_channel=False,
                        clip_fixed=float(clip.fixed_value) if clip.fixed_value > 0 else -1.0)
        if name == "AVERAGE_CHANNEL_MAX":
            raise NotImplementedError("AVERAGE_CHANNEL_MAX not implemented")
        raise MoEConifgError(f"Unknown clip type {clip.type}")

    # -- checkpoints: the configuration is an `analog_tile_state` entry (reference :372-415)
    def load_state_dict(self, state_dict, strict: bool = True, load_rpu_config: Optional[bool] = None,
                        strict_rpu_config_check: Optional[bool] = None):
        tile_state = state_dict.pop("analog_tile_state", None)
        if load_rpu_config:
            self.rpu_config = tile_state["rpu_config"]
        if strict_rpu_config_check and not isinstance(tile_state["rpu_config"], type(self.rpu_config)) \
                and not isinstance(self.rpu_config, type(tile_state["rpu_config"])):
            raise MoEConifgError(f"RPU config mismatch: cannot replace {type(tile_state['rpu_config']).__name__} "
                                 f"with {type(self.rpu_config).__name__}")
        return super().load_state_dict(state_dict, strict)

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        SigmaMoELayer._save_to_state_dict(self, destination, prefix, keep_vars)
        destination[prefix + "analog_tile_state"] = {"rpu_config": self.rpu_config}

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        tile_state = state_dict.pop(prefix + "analog_tile_state", None)
        if tile_state is not None:
            self.rpu_config = tile_state["rpu_config"]
        state_dict.setdefault(prefix + "noise_step", self.noise_step)
        state_dict[prefix + "analog_ctx"] = self.analog_ctx.data      # whatever shape the writer's context had
        SigmaMoELayer._load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                                            unexpected_keys, error_msgs)
