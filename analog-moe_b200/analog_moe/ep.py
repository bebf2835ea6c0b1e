"""Expert-parallel analog sigma-MoE layer: experts block-partitioned over the ranks of one node,
tokens data-parallel, one all-to-all of routed rows each way (NCCL over NVLink).

The reference is single-GPU; this module is new.  Per rank and step:

  route locally (global expert ids)          amoe_select_sort
  exchange per-expert counts                  all_to_all_single of [G, E/G] int32 + ONE host read
  gather rows in expert-sorted order          amoe_ep_pack        (contiguous block per destination rank)
  dispatch                                    all_to_all_single   (rows land in local HBM)
  up-projection -> activation -> down         the same CVMM kernels on the rank's experts
  return                                      all_to_all_single
  gate-weighted sum over k, reading the       amoe_combine with a row index
  sorted rows through the inverse permutation

dW and the input-range gradients need no collective: every slot of an expert arrives at its owner.
The exchange plan (split sizes and the regrouping of received rows by local expert) is plain host
arithmetic on the count matrix, so it is tested on CPU ranks over gloo.  Kernels only ever read
local memory.
"""
from __future__ import annotations

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


class ExpertParallelAnalogSigmaMoELayer(AnalogSigmaMoELayer):
    """`n_experts` is the global number; this rank holds experts [rank*E/G, (rank+1)*E/G)."""

    def __init__(self, rpu_config=None, *args, group=None, n_experts: int, **kwargs):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert n_experts % self.world == 0
        self.n_experts_global = n_experts
        if kwargs.get("bias"):
            raise NotImplementedError("expert-parallel layer: bias is not built")
        d_model = kwargs["d_model"]
        super().__init__(rpu_config, *args, n_experts=n_experts // self.world, **kwargs)
        # the router scores all experts and is replicated
        g = torch.Generator().manual_seed(1)
        self.expert_sel = torch.nn.Linear(d_model, n_experts, bias=False)
        with torch.no_grad():
            self.expert_sel.weight.copy_(torch.randn(n_experts, d_model, generator=g) * d_model ** -0.5)

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
