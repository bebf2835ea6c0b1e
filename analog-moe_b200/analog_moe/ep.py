"""Expert-parallel analog sigma-MoE layer: experts block-partitioned over the ranks of one node, tokens
data-parallel, routed rows exchanged once each way over NVLink.

The reference is single-GPU; this module is new.  Per rank and step (`_ExpertParallelStep`, one autograd node):

  route locally (global expert ids)           amoe_router_logits, amoe_select_sort
  all-gather of the per-expert counts         amoe_ep_share, [G, E/G] int32 per rank (payload and flags in peer memory)
  plan on the device                          amoe_ep_plan, amoe_ep_local_plan_dev   (no host read)
  rows to their owners                        amoe_ep_put: stores into the owner's buffer (symmetric memory)
  up-projection -> ReLU -> down-projection    the single-GPU kernels on the rank's experts, rows addressed
                                              through local_order; operand caches for the weight gradients
  rows back (ADC codes + one scale per row)   amoe_ep_put_back, then amoe_ep_share (orders the stores, carries the
                                              experts' column scales)
  gate-weighted sum over k                    amoe_combine_codes through the inverse permutation

and the mirror image in the backward pass (gradient rows as fp16 with a scale per row: amoe_ep_put_f16).  dW and the
input-range gradients need no collective: every slot of an expert arrives at its owner.  Ordering between ranks comes
from `amoe_ep_share` launches placed after the stores: the only kernel that waits for other ranks, by polling flags in
its own memory, with a limit; every load is local.  (AMOE_EP_NCCL_SYNC=1: small NCCL collectives instead.)  Without symmetric memory (or with
AMOE_EP_NCCL=1) the rows travel by `all_to_all_single` with split sizes taken from one host read per step
(`step_plan`); `forward_composed` keeps the composition around `CVMM.apply` for other activations.  The host-side
plans are plain arithmetic on the count matrix and are tested on CPU ranks over gloo.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from . import ops
from .layers import AnalogSigmaMoELayer
from .triton_src.cvmm import CVMMSel


@dataclass
class ExchangePlan:
    send_splits: List[int]        # rows this rank sends to each rank (its sorted list, cut by owner)
    recv_splits: List[int]        # rows it receives from each rank
    recv_counts: Tensor           # [G, E_local] rows from source g for local expert e (host)
    local_sel: Tensor             # [R] local expert id per sorted position
    local_order: Tensor           # [R] index into the receive buffer per sorted position
    local_offsets: Tensor         # [E_local + 1]

    @property
    def n_recv(self) -> int:
        return int(sum(self.recv_splits))


def plan_from_counts(send_counts: Tensor, recv_counts: Tensor) -> ExchangePlan:
    """send_counts/recv_counts: [G, E_local] host integer tensors.

    The receive buffer holds, for source g = 0..G-1, that source's rows for local experts 0..E_local-1
    in order.  Sorted-by-expert order is: for e, for g, the block (g, e)."""
    G, El = recv_counts.shape
    rc = recv_counts.to(torch.int64)
    flat = rc.reshape(-1)
    starts = torch.cumsum(flat, 0) - flat                    # start of block (g, e) in the receive buffer
    starts = starts.view(G, El)
    order, sel = [], []
    for e in range(El):
        for g in range(G):
            n = int(rc[g, e])
            if n:
                order.append(torch.arange(int(starts[g, e]), int(starts[g, e]) + n, dtype=torch.int32))
                sel.append(torch.full((n,), e, dtype=torch.int32))
    empty = torch.zeros(0, dtype=torch.int32)
    offsets = torch.zeros(El + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(rc.sum(0), 0).to(torch.int32)
    return ExchangePlan([int(v) for v in send_counts.sum(1)], [int(v) for v in rc.sum(1)], recv_counts,
                        torch.cat(sel) if sel else empty, torch.cat(order) if order else empty, offsets)


def make_plan(expert_offsets: Tensor, world: int, group=None) -> ExchangePlan:
    """expert_offsets [E+1] of the local routing (any device).  One collective on the counts and one
    device->host copy."""
    E = expert_offsets.numel() - 1
    assert E % world == 0, "the number of experts must be a multiple of the number of ranks"
    counts = (expert_offsets[1:] - expert_offsets[:-1]).to(torch.int32).view(world, E // world).contiguous()
    recv = torch.empty_like(counts)
    dist.all_to_all_single(recv, counts, group=group)
    both = torch.stack([counts, recv]).cpu()                  # the one host synchronisation of the step
    return plan_from_counts(both[0], both[1])


class _AllToAllRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows: Tensor, send_splits, recv_splits, group):
        ctx.splits = (send_splits, recv_splits, group)
        out = rows.new_empty((sum(recv_splits),) + tuple(rows.shape[1:]))
        dist.all_to_all_single(out, rows.contiguous(), recv_splits, send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g: Tensor):
        send_splits, recv_splits, group = ctx.splits
        out = g.new_empty((sum(send_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), send_splits, recv_splits, group=group)
        return out, None, None, None


class _GatherSorted(torch.autograd.Function):
    """x [T, D] -> rows [P, D] in expert-sorted order; backward sums a token's k slot gradients in
    slot order (deterministic), reading the sorted rows through the inverse permutation."""

    @staticmethod
    def forward(ctx, x2: Tensor, token_index: Tensor, inv_index: Tensor, k: int):
        ctx.save_for_backward(inv_index)
        ctx.k, ctx.T = k, x2.shape[0]
        rows, _ = ops.ep_pack(x2, token_index)
        return rows

    @staticmethod
    def backward(ctx, g: Tensor):
        (inv_index,) = ctx.saved_tensors
        return ops.combine(g.contiguous(), None, ctx.T, ctx.k, row_index=inv_index), None, None, None


class _CombineSorted(torch.autograd.Function):
    """y[t] = sum_j gate[t, j] * rows[inv[t*k + j]] for rows kept in expert-sorted order
    (reference cvmm.py:757-759; backward :888-889)."""

    @staticmethod
    def forward(ctx, rows: Tensor, gate: Tensor, slot_index: Tensor, inv_index: Tensor):
        T, k = gate.shape
        ctx.save_for_backward(rows, gate, slot_index, inv_index)
        return ops.combine(rows, gate, T, k, row_index=inv_index)

    @staticmethod
    def backward(ctx, gy: Tensor):
        rows, gate, slot_index, inv_index = ctx.saved_tensors
        T, k = gate.shape
        gy = gy.contiguous()
        # d rows[i] = gate[slot_i] * gy[slot_i // k], written directly in sorted order
        drows, _ = ops.ep_pack(gy, slot_index, src_div=k, row_scale=gate.reshape(-1).float().contiguous())
        dgate = ops.row_dot(rows, gy, k, row_index=inv_index).view(T, k).to(gate.dtype)
        return drows, dgate, None, None


@dataclass
class StepPlan:
    """Host-side view of one step's exchange, from the all-gathered count matrix C[source, destination, local expert]."""
    send_n: List[int]            # rows this rank sends to each rank
    recv_n: List[int]            # rows it receives from each rank
    send_off: List[int]          # start of each destination's block in this rank's sorted slot list
    recv_off: List[int]          # start of each source's block in this rank's receive buffer
    off_in: List[int]            # start of this rank's block in each destination's receive buffer
    back_off: List[int]          # start of this rank's block in each source's sorted slot list
    p_max: int                   # largest slot count over the ranks
    recv_counts: Tensor          # [G, El] int32 on the device

    @property
    def n_recv(self) -> int:
        return int(sum(self.recv_n))


def step_plan(counts: Tensor, rank: int, group=None, expect_rows: Optional[int] = None) -> StepPlan:
    """counts [G, El]: this rank's slots per (destination rank, local expert).  One all-gather and the step's only
    device->host copy.  With `expect_rows` (the slots this rank really routes) the counts are checked on the host and
    all ranks raise `ExchangeMismatchError` together if any rank's do not add up - before a row is sent."""
    G, El = counts.shape
    flat = torch.empty(G * G * El, dtype=counts.dtype, device=counts.device)
    if counts.is_cuda:
        dist.all_gather_into_tensor(flat, counts.contiguous().view(-1), group=group)
    else:       # gloo has no all_gather_into_tensor
        parts = [torch.empty(G * El, dtype=counts.dtype) for _ in range(G)]
        dist.all_gather(parts, counts.contiguous().view(-1), group=group)
        flat = torch.cat(parts)
    gathered = flat.view(G, G, El)
    if expect_rows is not None:
        from .health import agree_or_raise, counts_consistent
        agree_or_raise(counts_consistent(gathered.cpu(), rank, expect_rows), group, "expert-parallel exchange",
                       counts.device)
    tot = gathered.sum(-1).cpu()                                  # [source, destination] row counts
    tot_l = [[int(v) for v in row] for row in tot]
    send_n = tot_l[rank]
    recv_n = [tot_l[s][rank] for s in range(G)]
    cum = lambda xs: [sum(xs[:i]) for i in range(len(xs))]
    return StepPlan(send_n, recv_n, cum(send_n), cum(recv_n),
                    [sum(tot_l[s][d] for s in range(rank)) for d in range(G)],
                    [sum(tot_l[s][d] for d in range(rank)) for s in range(G)],
                    max(sum(row) for row in tot_l), gathered[:, rank, :].contiguous())


class PeerExchange:
    """Rows travel by plain stores into the destination rank's receive buffer (symmetric memory over NVLink), written by
    the gather kernel itself: no send buffer, no separate collective, no self-copy.  Where each row goes is computed on
    the device from the all-gathered counts (`amoe_ep_plan`), so the step needs no value on the host and can be captured
    in a CUDA graph.  A `share` after the writes is the cross-rank ordering point (stream-ordered after this rank's
    writes, complete only once every rank has reached it; it can carry a small value at no extra cost).  Buffers are
    sized for the worst case (every slot of every rank routed to one rank) and reused every step; reuse across steps
    is ordered by the next step's count exchange.  One forward/backward pair may be in flight per layer."""

    def __init__(self, group, device, p_cap: int, D: int, N: int, dtype, small_bytes: int = 0):
        """`small_bytes`: the largest payload `share` will carry."""
        import torch.distributed._symmetric_memory as symm
        self.group, self.device = group, device
        self.G, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.p_cap, self.cap = p_cap, self.G * p_cap
        self.key = (p_cap, D, N, dtype)
        self.buffers = {}
        # "yc" / "ys": the down-projection's rows as ADC codes (int8, moved as N/2 two-byte elements) and one scale per row
        shapes = {"x": (self.cap, D, dtype), "g": (self.cap, N, dtype), "y": (p_cap, N, dtype), "dx": (p_cap, D, dtype),
                  "yc": (p_cap, (N + 1) // 2, torch.bfloat16), "ys": (p_cap, 1, torch.float32)}
        if dtype == torch.float32:
            # gradient rows of the fp16 precision: fp16, each scaled for its own maximum, and the maxima
            shapes.update({"g16": (self.cap, N, torch.float16), "g16m": (self.cap, 1, torch.float32)})
        for name, (rows, cols, dt) in shapes.items():
            t = symm.empty(rows, cols, dtype=dt, device=device)
            hdl = symm.rendezvous(t, group)
            self.buffers[name] = (hdl, t, int(hdl.buffer_ptrs_dev))
        self.token = torch.zeros(1, device=device)
        self.generation = 0          # forward passes that have written into the buffers
        self.status = torch.zeros(4, dtype=torch.int32, device=device)   # device status word of the exchange kernels
        # small values between the ranks (counts, a maximum, column scales) and the ordering points after the row
        # exchanges: one kernel over peer memory each (`share`) instead of a collective of the communication library
        self.peer_sync = os.environ.get("AMOE_EP_NCCL_SYNC", "0") != "1"
        self.slot_bytes = 0
        if self.peer_sync:
            self.slot_bytes = (max(small_bytes, 64) + 15) // 16 * 16
            slots = symm.empty(2 * self.G * self.slot_bytes, dtype=torch.uint8, device=device)
            flags = symm.empty(max(self.G, 4), dtype=torch.int32, device=device)
            flags.zero_()
            torch.cuda.synchronize(device)
            self._slots = (symm.rendezvous(slots, group), slots)
            self._flags = (symm.rendezvous(flags, group), flags)
            self._epoch = torch.zeros(1, dtype=torch.int32, device=device)
            torch.cuda.synchronize(device)
            dist.barrier(group)          # every rank's flags are zero before the first exchange

    def barrier(self) -> None:
        if self.peer_sync:
            self.share(None)
        else:
            dist.all_reduce(self.token, group=self.group)

    def share(self, value: Optional[Tensor]) -> Optional[Tensor]:
        """All-gather of a small tensor (the same shape on every rank) and a barrier, one kernel over peer memory; returns
        [G, *value.shape].  `None`: barrier only.  Stream-ordered, no host value, capturable."""
        if not self.peer_sync:
            if value is None:
                dist.all_reduce(self.token, group=self.group)
                return None
            out = torch.empty((self.G,) + tuple(value.shape), dtype=value.dtype, device=value.device)
            dist.all_gather_into_tensor(out, value.contiguous(), group=self.group)
            return out
        out, nbytes = None, 0
        if value is not None:
            value = value.contiguous()
            nbytes = value.numel() * value.element_size()
            if nbytes > self.slot_bytes or nbytes % 4:
                raise ValueError(f"share: {nbytes} bytes do not fit the {self.slot_bytes}-byte slots (or are not whole words)")
            out = torch.empty((self.G,) + tuple(value.shape), dtype=value.dtype, device=value.device)
        ops._call("amoe_ep_share", ops.ptr(value), nbytes, int(self._slots[0].buffer_ptrs_dev), self.slot_bytes,
                  int(self._flags[0].buffer_ptrs_dev), ops.ptr(self._epoch), self.rank, self.G, ops.ptr(out), 1 << 24,
                  ops.ptr(self.status), ops.stream_ptr())
        return out

    def check(self, where: str = "expert-parallel exchange") -> None:
        """Synchronises and raises if an exchange kernel dropped a row or saw a plan larger than its buffers."""
        ops.raise_on_device_status(self.status, where)

    def put(self, name: str, src: Tensor, index: Tensor, sel_sorted: Tensor, El: int, plan: Tensor, src_div: int = 1,
            row_scale: Optional[Tensor] = None, barrier: bool = True) -> Tensor:
        """Row src[index[i] // src_div] (* row_scale[index[i]]) of every sorted position i to the rank that owns expert
        sel_sorted[i]; returns this rank's whole receive buffer [cap, cols] (its first R rows are valid).  With
        `barrier=False` the caller issues the collective that orders the stores (one that also carries a value)."""
        hdl, buf, ptrs = self.buffers[name]
        src = src.reshape(-1, src.shape[-1])
        assert src.shape[1] == buf.shape[1] and src.dtype == buf.dtype and src.stride(-1) == 1
        ops._call("amoe_ep_put", ops.ptr(src), ops.dtype_code(src), src.stride(0), src.shape[1], src.shape[0], ops.ptr(index),
                  src_div, ops.ptr(row_scale), index.numel(), ops.ptr(sel_sorted), El, ops.ptr(plan), ptrs, self.G,
                  buf.shape[0], ops.ptr(self.status), ops.stream_ptr())
        if barrier:
            self.barrier()
        return buf

    def put_f16(self, src: Tensor, index: Tensor, sel_sorted: Tensor, El: int, plan: Tensor, src_div: int = 1,
                row_scale: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
        """`put` of fp32 gradient rows as fp16 (half the bytes over NVLink): every row scaled by the power of two of its
        own maximum.  Returns this rank's receive buffers (rows [cap, cols] fp16, maxima [cap] fp32); no barrier."""
        _, buf, ptrs = self.buffers["g16"]
        _, mbuf, mptrs = self.buffers["g16m"]
        src = src.reshape(-1, src.shape[-1])
        assert src.shape[1] == buf.shape[1] and src.dtype == torch.float32 and src.stride(-1) == 1
        ops._call("amoe_ep_put_f16", ops.ptr(src), src.stride(0), src.shape[1], src.shape[0], ops.ptr(index), src_div,
                  ops.ptr(row_scale), index.numel(), ops.ptr(sel_sorted), El, ops.ptr(plan), ptrs, mptrs, self.G, buf.shape[0],
                  ops.ptr(self.status), ops.stream_ptr())
        return buf, mbuf.view(-1)

    def put_back(self, name: str, rows: Tensor, plan: Tensor, n_own: int, barrier: bool = True) -> Tensor:
        """The first R rows of `rows` (receive order) back to their sources; returns this rank's buffer [n_own, cols]."""
        hdl, buf, ptrs = self.buffers[name]
        assert rows.shape[1] == buf.shape[1] and rows.dtype == buf.dtype and rows.stride(-1) == 1
        ops._call("amoe_ep_put_back", ops.ptr(rows), ops.dtype_code(rows), rows.stride(0), rows.shape[1], ops.ptr(plan), ptrs,
                  self.G, rows.shape[0], buf.shape[0], ops.ptr(self.status), ops.stream_ptr())
        if barrier:
            self.barrier()
        return buf[:n_own]


class _ExpertParallelStep(torch.autograd.Function):
    """The expert-parallel layer step as one autograd node: router, select/sort, one count exchange with the step's
    only host read, rows out, both projections on the owner (the same kernels and operand caches as the single-GPU
    step, rows addressed through `local_order`), rows back, gate-weighted sum; the backward mirrors it.  Needs ReLU,
    no bias, no dropout (the composition in `forward_composed` covers the rest)."""

    @staticmethod
    def forward(ctx, layer, x, w_sel, keys, values, input_range, part=0, shared=None):
        """`part`: which micro-batch of the layer call this is (selects the exchange buffers); `shared`: prepared weights
        of both projections computed once for all micro-batches (`ExpertParallelAnalogSigmaMoELayer._prepare_weights`)."""
        cfg = layer.rpu_config
        fwd, ir_p = cfg.forward, cfg.pre_post.input_range
        group, G = layer.group, layer.world
        bsz, seq, D = x.shape
        k, El = layer.n_heads, layer.n_experts
        T = bsz * seq
        P = T * k
        x2 = x.reshape(T, D)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        dev = x.device
        precision = layer._precision(x)
        per_channel = bool(getattr(fwd, "out_noise_per_channel", True))

        def prepass(w, mod):
            return ops.weight_prepass(
                w, precision, per_channel_scale=per_channel, noise_std=mod.std_dev if mod else 0.0,
                noise_per_channel=mod.per_channel if mod else True, discretize_res=mod.discretize_res if mod else -1.0,
                seed=mod.seed if mod else 0, offset=mod.offset if mod else 0, step_dev=mod.step if mod else None,
                need_fwd=True, need_bwd=True, expert_base=layer.rank * El)     # the dense layer's draws for these experts

        def noise_args():
            # output noise is addressed by the row of the local receive buffer: the rank goes into the seed, or every
            # rank would draw the same pattern
            if layer.training and fwd.out_noise > 0:
                return dict(noise_std=float(fwd.out_noise), seed=layer._rank_noise_seed(), offset=layer._next_offset(),
                            step_dev=layer.noise_step)
            return {}

        main, side = torch.cuda.current_stream(), ops.side_stream(dev)
        if shared is None:
            nz_up, mod_up = noise_args(), layer._weight_modifier()
            nz_dn, mod_dn = noise_args(), layer._weight_modifier()
            # (side by side on two streams: both done before the large kernels of the main chain take every SM)
            side2 = ops.side_stream(dev, 1)
            side.wait_stream(main)
            side2.wait_stream(main)
            with ops.launch_on(side):
                ops.set_tag("up")
                pw_up = prepass(keys, mod_up)
                up_ready = side.record_event()      # the up-projection only waits for its own weights
            with ops.launch_on(side2):
                ops.set_tag("down")
                pw_dn = prepass(values, mod_dn)
        else:
            nz_up, nz_dn = noise_args(), noise_args()
            pw_up, pw_dn, up_ready = shared["pw_up"], shared["pw_dn"], shared["up_ready"]
        ops.set_tag("up")
        r, _ = ops.router_select(x2, w_sel, k, getattr(layer, "router_bias", None))
        gate = r.gate if x.dtype == torch.float32 else r.gate.to(x.dtype).float()
        # ---- exchange plan: counts both ways, one host read
        counts = (r.expert_offsets[1:] - r.expert_offsets[:-1]).view(G, El).contiguous()
        N, Fh = values.shape[-1], keys.shape[-1]
        inv = ops.invert_index(r.slot_index)
        xchg = layer._peer_exchange(P, D, N, x.dtype, part)
        plan = send_splits = recv_splits = None
        # ---- rows to their owners
        if xchg is not None:
            # everything on the device: all-gather of the counts -> plan -> stores into the owners' buffers
            gathered = xchg.share(counts)             # [G, G, El]: source, destination, local expert
            plan = ops.ep_plan(gathered, layer.rank)
            R = xchg.cap                       # rows allocated; the kernels find the real count in the plan / offsets
            local_order, local_offsets = ops.ep_local_plan_dev(plan, G, El, R, xchg.status)
            xchg.generation += 1
            recv = xchg.put("x", x2, r.token_index, r.sel, El, plan)
        else:
            hplan = step_plan(counts, layer.rank, group, expect_rows=P)
            send_splits, recv_splits = hplan.send_n, hplan.recv_n
            R = hplan.n_recv
            local_order, local_offsets = ops.ep_local_plan(hplan.recv_counts, R)
            rows, _ = ops.ep_pack(x2, r.token_index)
            recv = rows.new_empty((R, D))
            dist.all_to_all_single(recv, rows, recv_splits, send_splits, group=group)
            del rows
        inp_res = fwd.inp_res
        inp_res = (2.0 / inp_res if inp_res > 1.0 else 2.0 * inp_res) if inp_res > 0 else -1.0
        adc_on = fwd.out_res > 0 and fwd.out_bound > 0
        out_res, out_bound = (float(fwd.out_res), float(fwd.out_bound)) if adc_on else (-1.0, -1.0)
        has_ir = input_range is not None
        ir_all = input_range.detach().float().contiguous() if has_ir else None
        main.wait_event(up_ready)
        cached = R > 0 and layer.operand_caches and ops.operand_cache_ok(precision, D, Fh, N) and \
            any(ctx.needs_input_grad[3:5])
        split = precision == ops.A.PREC_SPLIT
        pre_up = R > 0 and layer.operand_prepass and ops.operand_tiles_ok(recv, precision)
        xc = ops.OperandCache.empty(R, El, D, split, dev) if (cached and not pre_up) else None
        hs = ops.OperandCache.empty(R, El, Fh, split, dev) if cached else None
        if R > 0:
            am_up = None if has_ir else ops.row_absmax(recv)
            # the received rows go through the operand pre-pass (DAC as a streaming kernel, A tiles by TMA) like the
            # single-GPU step's; rows the pre-pass cannot take keep the in-kernel prologue
            if pre_up:
                xq, xc_pre = ops.operand_tiles(recv, local_order, local_offsets, El, precision, P=R, dac=True,
                                               ir=ir_all[0] if has_ir else None, ir_by_expert=True, absmax=am_up,
                                               inp_res=inp_res, want_cache=cached)
                if cached:
                    xc = xc_pre
                a_kw = dict(a_tiles=xq)
            else:
                a_kw = dict(a_cache=xc)
            h, _ = ops.cvmm_fwd(recv, local_order, local_order, local_offsets, pw_up, precision, P=R, dst_rows=R,
                                ir=ir_all[0] if has_ir else None, ir_by_expert=True, absmax=am_up, inp_res=inp_res,
                                out_res=out_res, out_bound=out_bound, out_relu=True, **a_kw, **nz_up)
            if shared is None:
                main.wait_stream(side)
                main.wait_stream(side2)
            else:
                main.wait_event(shared["dn_ready"])
            ops.set_tag("down")
            am_dn = None if has_ir else ops.row_absmax(h)
            # with the ADC on and the device-driven exchange the rows travel back as int8 codes + one scale per row
            codes_back = xchg is not None and adc_on and N % 16 == 0
            meta = {} if codes_back else None
            out, codes = ops.cvmm_fwd(h, local_order, local_order, local_offsets, pw_dn, precision, P=R, dst_rows=R,
                                      ir=ir_all[1] if has_ir else None, ir_by_expert=True, absmax=am_dn, inp_res=inp_res,
                                      out_res=out_res, out_bound=out_bound, a_cache=hs, want_codes=codes_back,
                                      want_out=not codes_back, row_meta=meta, **nz_dn)
        else:
            if shared is None:
                main.wait_stream(side)
                main.wait_stream(side2)
            else:
                main.wait_event(shared["dn_ready"])
            codes_back = False
            h = recv.new_zeros((0, Fh))
            out = recv.new_zeros((0, N))
        # ---- rows back, gate-weighted sum over k in slot order
        back = cs_all = scale_back = None
        adc_step = ops.adc_step(out_res, out_bound) if adc_on else 0.0
        if codes_back:
            back = xchg.put_back("yc", codes.view(torch.bfloat16), plan, P, barrier=False).view(torch.int8)
            scale_back = xchg.put_back("ys", meta["row_scale"].view(-1, 1), plan, P, barrier=False).view(-1)
            # column scales of every expert; the exchange is also the point that orders the two sets of stores above
            cs_all = xchg.share(pw_dn.col_scale.float()).view(G * El, N)
            y = ops.combine_codes(back, cs_all, r.raw_sel, scale_back, adc_step, gate, T, k, out_dtype=x.dtype,
                                  row_index=inv)
        else:
            if xchg is not None:
                back = xchg.put_back("y", out, plan, P)
            else:
                back = out.new_empty((P, N))
                dist.all_to_all_single(back, out, send_splits, recv_splits, group=group)
            y = ops.combine(back, gate, T, k, row_index=inv)
        simt = precision == ops.A.PREC_FP32_SIMT
        ctx.save_for_backward(x2, w_sel, recv, h, back, gate, r.raw_sel, r.token_index, r.slot_index, r.expert_offsets, inv, r.sel,
                              local_order, local_offsets, ir_all,
                              pw_up.w if simt else None, pw_up.bwd_hi, pw_up.bwd_lo, pw_up.col_scale,
                              pw_dn.w if simt else None, pw_dn.bwd_hi, pw_dn.bwd_lo, pw_dn.col_scale,
                              *((xc.hi, xc.lo, hs.hi, hs.lo) if cached else (None, None, None, None)), cs_all, scale_back)
        ctx.adc_step = adc_step
        ctx.operand_prepass = layer.operand_prepass
        ctx.generation = xchg.generation if xchg is not None else 0
        if layer.keep_codes:      # ADC codes of the down-projection by flat slot (parity checks)
            layer.last_codes = back[inv.long()] if codes_back else None
        ctx.meta = (x.shape, El, k, precision, ir_p, keys.dtype, values.dtype, keys.shape, values.shape,
                    input_range.dtype if has_ir else None, send_splits, recv_splits, group, plan, xchg)
        return y.view(bsz, seq, N)

    @staticmethod
    def backward(ctx, gy):
        (x2, w_sel, recv, h, back, gate, raw_sel, token_index, slot_index, offsets, inv, sel_sorted, local_order, local_offsets, ir_all,
         w_up, up_hi, up_lo, up_cs, w_dn, dn_hi, dn_lo, dn_cs, xc_hi, xc_lo, hs_hi, hs_lo, cs_all, scale_back) = ctx.saved_tensors
        (x_shape, El, k, precision, ir_p, keys_dtype, values_dtype, kshape, vshape, ir_dtype, send_splits, recv_splits,
         group, plan, xchg) = ctx.meta
        T, D = x2.shape
        P, R = T * k, recv.shape[0]
        if xchg is not None and xchg.generation != ctx.generation:
            raise RuntimeError("expert-parallel layer: a later forward pass of this layer has overwritten the exchange "
                               "buffers this backward pass reads (one forward/backward pair per layer may be in flight)")
        # rows routed to this rank: known exactly on the NCCL path; with the device-driven exchange the buffers have
        # worst-case size and the balanced share P only tunes the work split of the weight-gradient kernels
        n_rows = P if xchg is not None else R
        Fh, N = vshape[1], vshape[2]
        need_x, need_sel, need_keys, need_values, need_ir = (ctx.needs_input_grad[i] for i in (1, 2, 3, 4, 5))
        has_ir = ir_all is not None
        need_ir = need_ir and has_ir
        cached = xc_hi is not None
        dev = x2.device
        g = gy.reshape(T, N)
        if g.stride(-1) != 1:
            g = g.contiguous()
        pw_up = ops.PreparedWeights(El, kshape[1], kshape[2], up_cs, w=w_up, bwd_hi=up_hi, bwd_lo=up_lo)
        pw_dn = ops.PreparedWeights(El, vshape[1], vshape[2], dn_cs, w=w_dn, bwd_hi=dn_hi, bwd_lo=dn_lo)
        decay = float(getattr(ir_p, "decay", 0.0) or 0.0) if has_ir else 0.0
        min_pct = float(getattr(ir_p, "input_min_percentage", 0.95))
        relative = bool(getattr(ir_p, "gradient_relative", True))
        gscale = float(getattr(ir_p, "gradient_scale", 1.0)) if relative else 1.0
        keeps = torch.zeros(2, dtype=torch.int64, device=dev) if (has_ir and decay > 0) else None
        ir_up, ir_dn = (ir_all[0], ir_all[1]) if has_ir else (None, None)
        gate_flat = gate.reshape(-1)
        # ---- gate gradient and the router's weight gradient at the source: they need only what this rank saved and the
        # upstream gradient, so they run on a stream of their own beside the exchange of the gradient rows (whose kernel
        # waits on NVLink, not on the SMs).  That stream has the main chain's priority: these are large grids off the
        # critical path, and at the higher priority they held back the small kernels that follow the exchange.
        main, side, bg = torch.cuda.current_stream(), ops.side_stream(dev), ops.side_stream(dev, 2, high_priority=False)
        side.wait_stream(main)
        bg.wait_stream(main)
        grad_sel = None
        f16_peer = xchg is not None and precision == ops.A.PREC_F16X1
        if f16_peer:
            # fp16 operands need max|gate * gy| over the rows a rank receives.  Any bound shared by the ranks serves (it only
            # picks a power-of-two scale): max|gy| * max|gate| of this rank, turned into the maximum over the ranks by the
            # all-reduce that orders the stores anyway - no pass over the received rows
            with ops.launch_on(side):
                ops.set_tag("down")
                gm_g, gm_gate = ops.tensor_absmax(g), ops.tensor_absmax(gate)
                gm_ready = side.record_event()
        with ops.launch_on(bg):
            ops.set_tag("down")
            if cs_all is not None:      # `back` holds ADC codes
                dgate = ops.row_dot_codes(back, cs_all, raw_sel.reshape(-1), scale_back, ctx.adc_step, g, k, row_index=inv)
            else:
                dgate = ops.row_dot(back, g, k, row_index=inv)
            dgate_ready = bg.record_event()
            if need_sel and ops._router_fits_smem(w_sel.shape[0], D):
                ops.set_tag("up")
                grad_sel = ops.router_backward_w(x2, dgate, gate, token_index, slot_index, offsets, w_sel.shape[0],
                                                 raw_sel=raw_sel)
        # ---- gate * gy rows to the owners
        ops.set_tag("down")
        gmax = None
        g_rowmax = None
        # fp32 gradient rows of the fp16 precision cross NVLink as fp16 when everything downstream takes tiles
        g_half = (f16_peer and "g16" in xchg.buffers and ctx.operand_prepass and N % 64 == 0 and g.dtype == torch.float32
                  and (cached or not need_values) and g.data_ptr() % 16 == 0 and (g.stride(0) * 4) % 16 == 0)
        if xchg is not None:
            if g_half:
                g_recv, g_rowmax = xchg.put_f16(g, slot_index, sel_sorted, El, plan, src_div=k, row_scale=gate_flat)
            else:
                g_recv = xchg.put("g", g, slot_index, sel_sorted, El, plan, src_div=k, row_scale=gate_flat, barrier=not f16_peer)
            if f16_peer:
                main.wait_event(gm_ready)
                gmax = xchg.share(gm_g * gm_gate).max().reshape(1)
        else:
            drows, _ = ops.ep_pack(g, slot_index, src_div=k, row_scale=gate_flat)
            g_recv = drows.new_empty((R, N))
            dist.all_to_all_single(g_recv, drows, recv_splits, send_splits, group=group)
            del drows
        grad_keys = grad_values = None
        if R > 0:
            split = xc_lo is not None
            gc = ops.OperandCache.empty(R, El, N, split, dev) if cached and need_values else None
            dhc = ops.OperandCache.empty(R, El, Fh, split, dev) if cached and need_keys else None
            if xchg is None:
                gmax = ops.grad_absmax(g_recv, precision)      # fp16 operands: max|g| over the rows that arrived
            if need_values and not cached:
                grad_values = ops.cvmm_dw(h, local_order, g_recv, local_order, local_offsets, El, precision, P=R, ir=ir_dn,
                                          ir_by_expert=True, g_absmax=gmax)
            if ctx.operand_prepass and ops.operand_tiles_ok(g_recv, precision):
                gc, _ = ops.operand_tiles(g_recv, local_order, local_offsets, El, precision, P=R, dac=False, g_absmax=gmax,
                                          row_absmax=g_rowmax)
                a_kw = dict(a_tiles=gc)
            else:
                a_kw = dict(a_cache=gc)
            if g_half:
                g_recv = xchg.buffers["g"][1]       # (with tiles the kernel takes only type and shape from this argument)
            dh, irs_dn = ops.cvmm_dx(g_recv, local_order, local_order, local_offsets, pw_dn, precision, P=R, dst_rows=R,
                                     x_ref=h, x_ref_row=local_order, ir=ir_dn, ir_by_expert=True, want_ir_grad=has_ir,
                                     relative=relative, grad_scale=gscale, keep_count=keeps[1:] if keeps is not None else None,
                                     out_dtype=h.dtype, x_ref_relu=True, out_cache=dhc, g_absmax=gmax, **a_kw)
            ops.set_tag("up")
            dxr, irs_up = ops.cvmm_dx(dh, local_order, local_order, local_offsets, pw_up, precision, P=R, dst_rows=R,
                                      x_ref=recv if has_ir else None, x_ref_row=local_order if has_ir else None, ir=ir_up,
                                      ir_by_expert=True, want_ir_grad=has_ir, relative=relative, grad_scale=gscale,
                                      keep_count=keeps[:1] if keeps is not None else None, out_dtype=x2.dtype,
                                      a_tiles=dhc if (dhc is not None and Fh % 64 == 0) else None, g_absmax=gmax)
            # the two weight gradients on a second stream, beside the exchange and the streaming kernels that follow
            if cached and (need_values or need_keys):
                side.wait_stream(main)
                with ops.launch_on(side):
                    if need_values:
                        ops.set_tag("down")
                        grad_values = ops.cvmm_dw_cached(ops.OperandCache(hs_hi, hs_lo, Fh), gc, local_offsets, El, precision,
                                                         P=R, expected_rows=n_rows, g_absmax=gmax)
                    if need_keys:
                        ops.set_tag("up")
                        grad_keys = ops.cvmm_dw_cached(ops.OperandCache(xc_hi, xc_lo, D), dhc, local_offsets, El, precision,
                                                       P=R, expected_rows=n_rows, g_absmax=gmax)
            elif need_keys:
                grad_keys = ops.cvmm_dw(recv, local_order, dh, local_order, local_offsets, El, precision, P=R, ir=ir_up,
                                        ir_by_expert=True,
                                        g_absmax=ops.grad_absmax(dh, precision, plan[0:1] if xchg is not None else None))
        else:
            dxr = recv.new_zeros((0, D))
            irs_up = irs_dn = None
            if need_keys:
                grad_keys = torch.zeros(kshape, dtype=keys_dtype, device=dev)
            if need_values:
                grad_values = torch.zeros(vshape, dtype=values_dtype, device=dev)
        # ---- input-gradient rows back to the source; sum over k plus the router's term
        ops.set_tag("up")
        grad_x = None
        # The input-range decay term's threshold is one fraction over ALL routed pairs (reference cvmm.py:872-878): kept
        # elements and rows are summed over the ranks on the device (one small all-reduce, no host read), so the result is
        # the dense layer's whatever the load balance.  With rows going back through peer memory that all-reduce is also
        # the point that orders the stores.
        tot, tot_summed = None, False
        if need_ir and keeps is not None:
            tot = torch.cat([keeps, local_offsets[-1:].to(torch.int64)])     # kept (up), kept (down), rows here
        if need_x:
            if xchg is not None:
                dback = xchg.put_back("dx", dxr, plan, P, barrier=tot is None)
                if tot is not None:
                    tot = xchg.share(tot).sum(0)
                    tot_summed = True
            else:
                dback = dxr.new_empty((P, D))
                dist.all_to_all_single(dback, dxr, send_splits, recv_splits, group=group)
            main.wait_event(dgate_ready)
            grad_x = ops.combine_router(dback, T, k, dgate, gate, raw_sel, w_sel, row_index=inv).view(x_shape)
        if need_sel and grad_sel is None:
            main.wait_event(dgate_ready)
            grad_sel = ops.router_backward_w(x2, dgate, gate, token_index, slot_index, offsets, w_sel.shape[0],
                                             raw_sel=raw_sel).to(w_sel.dtype)
        grad_ir = None
        if need_ir:
            if tot is not None and not tot_summed:
                dist.all_reduce(tot, group=group)
            if R > 0:
                grad_ir = torch.stack([
                    ops.ir_grad_reduce(irs_up, local_offsets, ir_up, El, decay, min_pct,
                                       tot[0:1] if tot is not None else None, total_rows=tot[2:3] if tot is not None else None,
                                       cols=D),
                    ops.ir_grad_reduce(irs_dn, local_offsets, ir_dn, El, decay, min_pct,
                                       tot[1:2] if tot is not None else None, total_rows=tot[2:3] if tot is not None else None,
                                       cols=Fh)]).to(ir_dtype)
            else:
                grad_ir = torch.zeros(2, El, dtype=ir_dtype, device=dev)
        main.wait_stream(side)
        main.wait_stream(bg)
        if grad_sel is not None:
            grad_sel = grad_sel.to(w_sel.dtype)
        if grad_values is not None:
            grad_values = grad_values.to(values_dtype)
        if grad_keys is not None:
            grad_keys = grad_keys.to(keys_dtype)
        return (None, grad_x, grad_sel, grad_keys, grad_values, grad_ir, None, None)


class ExpertParallelAnalogSigmaMoELayer(AnalogSigmaMoELayer):
    """`n_experts` is the global number; this rank holds experts [rank*E/G, (rank+1)*E/G)."""

    def __init__(self, rpu_config=None, *args, group=None, n_experts: int, **kwargs):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert n_experts % self.world == 0
        self.n_experts_global = n_experts
        self.peer_exchange = os.environ.get("AMOE_EP_NCCL") is None    # rows by stores into peer memory (else NCCL)
        self._xchg = None
        self._xchgs = {}               # exchange buffers per micro-batch
        self._mb_streams = {}
        # Micro-batches per layer call (single-node step only): each runs on its own stream with its own exchange
        # buffers.  Off by default: measured on two B200s with 8192 tokens per GPU, two micro-batches took 1.24 ms per
        # step against 1.05 ms for one - the CVMM kernels hold every SM's registers and shared memory, so the other
        # micro-batch's exchange kernels wait for them instead of running beside them, and every kernel is paid twice.
        self.micro_batches = int(kwargs.pop("micro_batches", os.environ.get("AMOE_EP_MICRO_BATCHES", 1)))
        self.max_slots = int(kwargs.pop("max_slots", 0))
        if kwargs.get("bias"):
            raise NotImplementedError("expert-parallel layer: bias is not built")
        d_model = kwargs["d_model"]
        super().__init__(rpu_config, *args, n_experts=n_experts // self.world, **kwargs)
        # the router scores all experts and is replicated
        g = torch.Generator().manual_seed(1)
        self.expert_sel = torch.nn.Linear(d_model, n_experts, bias=False)
        with torch.no_grad():
            self.expert_sel.weight.copy_(torch.randn(n_experts, d_model, generator=g) * d_model ** -0.5)

    def _peer_exchange(self, P: int, D: int, N: int, dtype, part: int = 0) -> Optional["PeerExchange"]:
        """The symmetric-memory exchange of micro-batch `part`; None when peer access is off (`peer_exchange=False`, or
        symmetric memory could not be set up: NCCL all-to-all with one host read then).  The buffers are sized at the
        first call from the largest slot count over the ranks (one all-reduce and host read, once) or from `max_slots`."""
        if not self.peer_exchange:
            return None
        x = self._xchgs.get(part)
        if x is not None and x.key[1:] == (D, N, dtype) and P <= x.p_cap:
            return x
        if x is not None and P > x.p_cap:
            raise RuntimeError(f"expert-parallel layer: {P} slots on this rank exceed the exchange buffers ({x.p_cap}); "
                               "construct the layer with max_slots >= tokens*k of the largest batch")
        try:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("first call under stream capture")
            m = torch.tensor([max(P, self.max_slots)], dtype=torch.int64, device=self.keys.device)
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=self.group)
            small = max(self.n_experts * N * 4, self.world * self.n_experts * 4, 64)   # column scales / count matrix
            self._xchgs[part] = PeerExchange(self.group, self.keys.device, int(m.item()), D, N, dtype, small_bytes=small)
            if part == 0:
                self._xchg = self._xchgs[0]
            return self._xchgs[part]
        except Exception as exc:       # no symmetric memory on this system: say so once, use NCCL from now on
            import warnings
            warnings.warn(f"expert-parallel peer exchange unavailable ({exc!r}); using NCCL all-to-all")
            self.peer_exchange = False
            return None

    def _rank_noise_seed(self) -> int:
        return (self.noise_seed ^ (self.rank * 0x9E3779B97F4A7C15)) & (2 ** 64 - 1)

    def load_global_weights(self, keys: Tensor, values: Tensor, router: Tensor, input_range: Optional[Tensor] = None):
        El = self.n_experts
        sl = slice(self.rank * El, (self.rank + 1) * El)
        with torch.no_grad():
            self.keys.copy_(keys[sl])
            self.values.copy_(values[sl])
            self.expert_sel.weight.copy_(router)
            if input_range is not None and self.input_range is not None:
                self.input_range.copy_(input_range[:, sl])

    def forward(self, inp: Tensor) -> Tuple[Tensor, Tensor]:
        from .layers import _is_relu
        ir_p = self.rpu_config.pre_post.input_range
        single_node = self.fused and _is_relu(self.activation) and not (self.dropout > 0 and self.training) and \
            not (self.input_range is not None and self.training and ir_p.init_from_data > 0 and
                 float(self.input_range_update_idx) < ir_p.init_from_data)
        if not single_node:
            return self.forward_composed(inp)
        self._noise_calls = 0
        bsz, seq, D = inp.shape
        T = bsz * seq
        mb = self.micro_batches if (self.micro_batches > 1 and T >= 256 * self.micro_batches) else 1
        if mb == 1:
            y = _ExpertParallelStep.apply(self, inp, self.expert_sel.weight, self.keys, self.values, self.input_range,
                                          0, None)
        else:
            y = self._forward_micro_batches(inp, mb)
        if self.training:
            self.noise_step += 1
        return y, self._aux_zero

    def _prepare_weights(self, x: Tensor) -> dict:
        """Both weight pre-passes once per layer call, on the side stream (every micro-batch sees the same modified
        weights, as the whole batch does in the reference's layer, moe_layer_aihwkit_lightning.py:458-469)."""
        fwd = self.rpu_config.forward
        precision = self._precision(x)
        per_channel = bool(getattr(fwd, "out_noise_per_channel", True))
        main, side = torch.cuda.current_stream(), ops.side_stream(x.device)
        mods = [self._weight_modifier(), self._weight_modifier()]
        side.wait_stream(main)
        out = {}
        with ops.launch_on(side):
            for name, w, mod, tag in (("pw_up", self.keys, mods[0], "up"), ("pw_dn", self.values, mods[1], "down")):
                ops.set_tag(tag)
                out[name] = ops.weight_prepass(
                    w, precision, per_channel_scale=per_channel, noise_std=mod.std_dev if mod else 0.0,
                    noise_per_channel=mod.per_channel if mod else True,
                    discretize_res=mod.discretize_res if mod else -1.0, seed=mod.seed if mod else 0,
                    offset=mod.offset if mod else 0, step_dev=mod.step if mod else None, need_fwd=True, need_bwd=True,
                    expert_base=self.rank * self.n_experts)
                out["up_ready" if name == "pw_up" else "dn_ready"] = side.record_event()
        return out

    def _forward_micro_batches(self, inp: Tensor, mb: int) -> Tensor:
        bsz, seq, D = inp.shape
        T = bsz * seq
        main = torch.cuda.current_stream()
        shared = self._prepare_weights(inp)
        parts = torch.chunk(inp.reshape(1, T, D), mb, dim=1)
        outs = []
        for h, xh in enumerate(parts):
            st = self._mb_streams.get(h)
            if st is None:
                st = self._mb_streams[h] = torch.cuda.Stream(device=inp.device)
            st.wait_stream(main)
            for name in ("pw_up", "pw_dn"):        # allocated for the calling stream, read by this one until backward ends
                for t in vars(shared[name]).values():
                    if torch.is_tensor(t):
                        t.record_stream(st)
            with torch.cuda.stream(st):
                yh = _ExpertParallelStep.apply(self, xh, self.expert_sel.weight, self.keys, self.values, self.input_range,
                                               h, shared)
            outs.append((st, yh))
        for st, yh in outs:
            main.wait_stream(st)
            yh.record_stream(main)
        main.wait_stream(ops.side_stream(inp.device))
        return torch.cat([yh for _, yh in outs], dim=1).view(bsz, seq, -1)

    def forward_composed(self, inp: Tensor) -> Tuple[Tensor, Tensor]:
        """The same step composed from autograd functions around CVMM.apply (any activation, dropout)."""
        self._noise_calls = 0
        bsz, seq, D = inp.shape
        T, k = bsz * seq, self.n_heads
        logits = self.expert_sel(inp)
        if getattr(self, "router_bias", None) is not None:
            logits = logits + self.router_bias
        r = ops.select_sort(logits.detach(), k, apply_sigmoid=True)
        gate = torch.sigmoid(logits.float()).view(T, -1).gather(-1, r.raw_sel.long()).to(inp.dtype)
        plan = make_plan(r.expert_offsets, self.world, self.group)
        dev = inp.device
        inv = ops.invert_index(r.slot_index)
        rows = _GatherSorted.apply(inp.reshape(T, D), r.token_index, inv, k)
        recv = _AllToAllRows.apply(rows, plan.send_splits, plan.recv_splits, self.group)
        R = plan.n_recv
        if R > 0:
            sel = CVMMSel(None, plan.local_sel.to(dev).view(1, R, 1), plan.local_order.to(dev), None, None,
                          plan.local_offsets.to(dev))
            h = self.cvmm_wrapper(recv.view(1, R, D), sel, self.keys)            # [1, R, 1, F]
            h = self.activation(h)
            out = self.cvmm_wrapper(h, sel, self.values).reshape(R, self.v_dim)  # rows in receive order
        else:
            out = recv.new_zeros((0, self.v_dim)) + 0.0 * recv.sum()
        back = _AllToAllRows.apply(out, plan.recv_splits, plan.send_splits, self.group)
        y = _CombineSorted.apply(back, gate, r.slot_index, inv)
        if self.training:
            self.noise_step += 1
        return y.view(bsz, seq, self.v_dim), inp.new_zeros(())
