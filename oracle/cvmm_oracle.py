"""CPU oracle for the analog CVMM hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch/numpy on the CPU, the arithmetic of the
reference's conditional vector-matrix multiply (CVMM) and the analog
pre/post-processing around it.  It is the checker the CUDA kernels are compared
with; it is never the thing that is shipped or measured as the product.  Only
the tests, the smoke check and the bench's CPU-baseline leg may import it.

Parity status
-------------
* PINNED against the reference itself: every function that has a counterpart in
  the reference (`cvmm_forward`, `cvmm_dw`, `cvmm_backward`, `expert_std`,
  `prepare_sel`) is checked in the CPU test-suite against golden vectors that
  were produced by running the reference's own `CVMM.apply` forward+backward
  and `cvmm_std` under Triton's CPU interpreter (generator committed next to
  the fixtures).
* UNPINNED (the reference has no implementation, so this file *defines* them):
  ADC output quantisation (`adc_codes`), Philox-addressed noise
  (`philox_normal`), and the top-k gate select (`select_sort`), which in the
  reference's ecosystem lives in the third-party `sigma_moe` package that is
  not vendored; its behaviour is restated from the reference's naive test layer
  (tests/test_moe_layer_aihwkit.py:71-76).

Reference citations are by path inside the reference project.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch

# --------------------------------------------------------------------------- #
# Philox4x32-10 and the normal variates derived from it (definition, unpinned)
# --------------------------------------------------------------------------- #
_PHILOX_M0 = np.uint64(0xD2511F53)
_PHILOX_M1 = np.uint64(0xCD9E8D57)
_PHILOX_W0 = np.uint32(0x9E3779B9)
_PHILOX_W1 = np.uint32(0xBB67AE85)
_MASK32 = np.uint64(0xFFFFFFFF)

# Stream identifiers: the third counter word separates the consumers of one seed.
STREAM_OUT_NOISE = 0x0A0E
STREAM_WEIGHT_NOISE = 0x0B0E


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Vectorised Philox4x32 with 10 rounds (Salmon et al., SC'11).

    All arguments are broadcastable uint32 arrays; returns four uint32 arrays.
    """
    c0, c1, c2, c3 = (np.asarray(v, dtype=np.uint32) for v in (c0, c1, c2, c3))
    c0, c1, c2, c3 = np.broadcast_arrays(c0, c1, c2, c3)
    c0, c1, c2, c3 = c0.copy(), c1.copy(), c2.copy(), c3.copy()
    k0 = np.uint32(k0)
    k1 = np.uint32(k1)
    with np.errstate(over="ignore"):
        for _ in range(10):
            p0 = _PHILOX_M0 * c0.astype(np.uint64)
            p1 = _PHILOX_M1 * c2.astype(np.uint64)
            hi0 = (p0 >> np.uint64(32)).astype(np.uint32)
            lo0 = (p0 & _MASK32).astype(np.uint32)
            hi1 = (p1 >> np.uint64(32)).astype(np.uint32)
            lo1 = (p1 & _MASK32).astype(np.uint32)
            n0 = hi1 ^ c1 ^ k0
            n2 = hi0 ^ c3 ^ k1
            c0, c1, c2, c3 = n0, lo1, n2, lo0
            k0 = np.uint32((int(k0) + int(_PHILOX_W0)) & 0xFFFFFFFF)
            k1 = np.uint32((int(k1) + int(_PHILOX_W1)) & 0xFFFFFFFF)
    return c0, c1, c2, c3


def _box_muller(u_a: np.ndarray, u_b: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Two uint32 words -> two standard normals (fp32 arithmetic).  The uniforms are the 23-bit
    values (k + 0.5) * 2^-23: exact in fp32 and strictly inside (0, 1)."""
    f = np.float32(2.0 ** -23)
    ua = ((u_a >> np.uint32(9)).astype(np.float32) + np.float32(0.5)) * f
    ub = ((u_b >> np.uint32(9)).astype(np.float32) + np.float32(0.5)) * f
    r = np.sqrt(np.float32(-2.0) * np.log(ua)).astype(np.float32)
    th = (np.float32(2.0 * math.pi) * ub).astype(np.float32)
    return (r * np.cos(th)).astype(np.float32), (r * np.sin(th)).astype(np.float32)


def philox_normal(seed: int, offset: int, stream: int, rows: int, cols: int) -> torch.Tensor:
    """Standard normals addressed by (row, column).

    Element (r, c) uses counter (r, c // 4, stream, offset) and key
    (seed & 0xffffffff, seed >> 32); the four output words give the four
    columns 4*(c//4) .. 4*(c//4)+3 through two Box-Muller pairs.
    """
    quads = (cols + 3) // 4
    r = np.arange(rows, dtype=np.uint32)[:, None]
    q = np.arange(quads, dtype=np.uint32)[None, :]
    w0, w1, w2, w3 = philox4x32_10(r, q, np.uint32(stream), np.uint32(offset & 0xFFFFFFFF),
                                   seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    z0, z1 = _box_muller(w0, w1)
    z2, z3 = _box_muller(w2, w3)
    z = np.stack([z0, z1, z2, z3], axis=-1).reshape(rows, quads * 4)[:, :cols]
    return torch.from_numpy(np.ascontiguousarray(z))


def _box_muller16(w: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """One uint32 word -> two standard normals: 16-bit uniforms (k + 0.5) * 2^-16, the radius from the low half of
    the word, the angle from the high half (fp32 arithmetic)."""
    f = np.float32(2.0 ** -16)
    ua = ((w & np.uint32(0xFFFF)).astype(np.float32) + np.float32(0.5)) * f
    ub = ((w >> np.uint32(16)).astype(np.float32) + np.float32(0.5)) * f
    r = np.sqrt(np.float32(-2.0) * np.log(ua)).astype(np.float32)
    th = (np.float32(2.0 * math.pi) * ub).astype(np.float32)
    return (r * np.cos(th)).astype(np.float32), (r * np.sin(th)).astype(np.float32)


def philox_normal8(seed: int, offset: int, stream: int, rows: int, cols: int) -> torch.Tensor:
    """Standard normals addressed by (row, column), eight per Philox call: the generator of the CVMM kernels' output
    noise (this library's own definition: the reference draws its output noise from torch's generator, which no
    kernel can reproduce element by element).

    Element (r, c) uses counter (r, c // 8, stream, offset) and key (seed & 0xffffffff, seed >> 32); output word j
    gives columns 8*(c//8) + 2j and + 2j + 1 through one Box-Muller pair on its two 16-bit halves.
    """
    octs = (cols + 7) // 8
    r = np.arange(rows, dtype=np.uint32)[:, None]
    q = np.arange(octs, dtype=np.uint32)[None, :]
    ws = philox4x32_10(r, q, np.uint32(stream), np.uint32(offset & 0xFFFFFFFF), seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    zs = []
    for w in ws:
        z0, z1 = _box_muller16(w)
        zs += [z0, z1]
    z = np.stack(zs, axis=-1).reshape(rows, octs * 8)[:, :cols]
    return torch.from_numpy(np.ascontiguousarray(z))


# --------------------------------------------------------------------------- #
# Routing: gate select + expert-contiguous sort
# --------------------------------------------------------------------------- #
@dataclass
class Selection:
    """What the select/sort step produces (field names follow `CVMMSel`,
    analog_moe/triton_src/cvmm.py:19-28)."""
    raw_sel: torch.Tensor        # [T, k] int32 expert ids, unsorted
    gate: torch.Tensor           # [T, k] fp32 gate values (sigmoid of the logits)
    sel: torch.Tensor            # [P] int32 expert ids sorted ascending
    token_index: torch.Tensor    # [P] int32 token row of sorted position i
    slot_index: torch.Tensor     # [P] int32 flat (token*k + j) slot of sorted position i
    expert_offsets: torch.Tensor  # [E+1] int32 start of every expert's run


def select_sort(logits: torch.Tensor, k: int, apply_sigmoid: bool = True) -> Selection:
    """sigmoid -> top-k -> stable counting sort by expert id.

    Follows tests/test_moe_layer_aihwkit.py:71-76 (sigmoid, topk) and
    analog_moe/triton_src/cvmm.py:31-34 (flatten + sort).  Choices the reference
    leaves open are fixed here: the k picks of a token are listed by descending
    gate value, ties broken towards the lower expert id; the sort is stable, so
    inside an expert the slots stay in ascending flat-slot order.
    """
    T, E = logits.shape
    g = torch.sigmoid(logits.float()) if apply_sigmoid else logits.float()
    # descending value, lower index first on ties: sort on (-value, index)
    order = torch.argsort(-g, dim=-1, stable=True)[:, :k]
    gate = torch.gather(g, 1, order)
    raw_sel = order.to(torch.int32)
    flat = raw_sel.flatten().long()
    sel, perm = torch.sort(flat, stable=True)
    counts = torch.bincount(flat, minlength=E)
    offsets = torch.zeros(E + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
    return Selection(raw_sel, gate, sel.to(torch.int32), (perm // k).to(torch.int32),
                     perm.to(torch.int32), offsets)


def prepare_sel(sel: torch.Tensor):
    """analog_moe/triton_src/cvmm.py:31-34 with the sort made stable."""
    fsel = sel.flatten()
    ssel, idx = torch.sort(fsel.long(), stable=True)
    return ssel.view_as(sel), idx


# --------------------------------------------------------------------------- #
# DAC (input clamp + scale + quantise) and ADC
# --------------------------------------------------------------------------- #
def convert_res(res: float) -> float:
    """moe_layer_aihwkit_lightning.py:451-456: 254 -> 2/254, 1/254 -> 2/254, <=0 -> -1."""
    if res > 0:
        return 2.0 / res if res > 1.0 else 2.0 * res
    return -1.0


def dac(a: torch.Tensor, ir: Optional[torch.Tensor], absmax: Optional[torch.Tensor],
        inp_res: float) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Rows `a` [M,K] already gathered; `ir`/`absmax` are [M] per-row scalars.

    Returns (normalised operand fed to the MVM, integer codes or None).
    cvmm.py:145-172: clamp to +-ir, divide by ir, divide by abs-max, divide by
    the resolution, round half to even, multiply by the resolution - every step
    an individually rounded fp32 operation.
    """
    a = a.float()
    if ir is not None:
        r = ir.float().view(-1, 1)
        a = torch.where(a > r, r.expand_as(a), a)
        a = torch.where(a < -r, (-r).expand_as(a), a)
        a = a / r
    if absmax is not None:
        a = a / absmax.float().view(-1, 1)
    codes = None
    if inp_res > 0:
        res = torch.tensor(inp_res, dtype=torch.float32)
        codes = torch.round(a / res)
        a = codes * res
    return a, codes


def adc_step(out_res: float, out_bound: float) -> float:
    """Size of one ADC code in units of the per-column weight maximum."""
    res = 1.0 / out_res if out_res > 1.0 else out_res
    return float(np.float32(2.0) * np.float32(out_bound) * np.float32(res))


def adc_codes(acc: torch.Tensor, s_col: torch.Tensor, out_res: float, out_bound: float):
    """Definition of the ADC step (no counterpart in the reference, which asserts
    it off at moe_layer_aihwkit_lightning.py:152-157).

    `acc` [M,N] is the accumulator (+noise) in normalised-input units, `s_col`
    [M,N] or [M,1] the weight maximum that normalises the column.  All in fp32:
    v = acc * (1/s) clamped to +-out_bound; code = round-half-even(v * (1/step)),
    step = 2*out_bound*res; both reciprocals are correctly rounded fp32 values
    (1/s := 0 for an all-zero column).  Returns (codes, codes*step*s).
    """
    one = torch.tensor(1.0, dtype=torch.float32)
    step = torch.tensor(adc_step(out_res, out_bound), dtype=torch.float32)
    inv_step = one / step
    ob = torch.tensor(out_bound, dtype=torch.float32)
    s = s_col.float()
    inv_s = torch.where(s > 0, one / torch.where(s > 0, s, one), torch.zeros_like(s))
    v = acc.float() * inv_s
    v = torch.minimum(torch.maximum(v, -ob), ob)
    q = torch.round(v * inv_step)
    return q, (q * step) * s


# --------------------------------------------------------------------------- #
# Weight modifier (moe_layer_aihwkit_lightning.py:313-382, moe_layer_aihwkit.py:144-196)
# --------------------------------------------------------------------------- #
def weight_max(W: torch.Tensor, per_channel: bool) -> torch.Tensor:
    """[E,N] per-column |W| maximum, or the per-expert maximum broadcast to [E,N]."""
    E, K, N = W.shape
    if per_channel:
        return W.float().abs().amax(1)
    return W.float().reshape(E, -1).abs().amax(-1, keepdim=True).expand(E, N).contiguous()


def modify_weight(W: torch.Tensor, std_dev: float, per_channel: bool,
                  seed: int, offset: int, discretize_res: float = -1.0) -> torch.Tensor:
    """ADD_NORMAL[_PER_CHANNEL] and DISCRETIZE[_ADD_NORMAL]: W (+ quantise) + std*wmax*z.

    z for element (e, k, n) is `philox_normal` row e*K+k, column n, stream
    STREAM_WEIGHT_NOISE.  Discretisation rounds W to multiples of wmax/n_states
    (half to even) and clamps to +-wmax.
    """
    E, K, N = W.shape
    wmax = weight_max(W, per_channel).view(E, 1, N)
    out = W.float()
    if discretize_res > 0:
        n_states = max(discretize_res, 1.0 / discretize_res)
        res = wmax / torch.tensor(n_states, dtype=torch.float32)
        res_safe = torch.where(res > 0, res, torch.ones_like(res))
        out = torch.round(out / res_safe) * res_safe
        out = torch.minimum(torch.maximum(out, -wmax), wmax)
    if std_dev > 0:
        z = philox_normal(seed, offset, STREAM_WEIGHT_NOISE, E * K, N).view(E, K, N)
        out = out + (torch.tensor(std_dev, dtype=torch.float32) * wmax) * z
    return out


# --------------------------------------------------------------------------- #
# Forward CVMM (cvmm.py:98-231)
# --------------------------------------------------------------------------- #
def cvmm_forward(x: torch.Tensor, sel_index: torch.Tensor, sel: torch.Tensor, W: torch.Tensor,
                 inp_res: float = -1.0, ir_slot: Optional[torch.Tensor] = None,
                 out_index: Optional[torch.Tensor] = None, absmax: Optional[torch.Tensor] = None,
                 out_noise: Optional[torch.Tensor] = None,
                 adc: Optional[Tuple[float, float, torch.Tensor]] = None,
                 acc_dtype=torch.float64, return_codes: bool = False):
    """out[c_i,:] = ((DAC(x[r_i,:]) @ W[e_i]) + noise[c_i,:] -> ADC) * absmax[r_i] * ir_i.

    x [R,K]; sel_index/sel/ir_slot/out_index [P] in sorted-slot order; W [E,K,N];
    absmax [R] by source row; out_noise [P,N] by destination row; adc =
    (out_res, out_bound, wmax[E,N]).  Destination row c_i = out_index[i] if
    given else sel_index[i] (cvmm.py:196-205).  The contraction is accumulated
    in `acc_dtype` and rounded to fp32 once.
    """
    x = x.reshape(-1, x.shape[-1])
    sel_index = sel_index.flatten().long()
    sel = sel.flatten().long()
    P = sel.numel()
    E, K, N = W.shape
    rows = x[sel_index]
    a, in_codes = dac(rows, None if ir_slot is None else ir_slot.flatten(),
                      None if absmax is None else absmax.flatten()[sel_index], inp_res)
    dst = sel_index if out_index is None else out_index.flatten().long()
    acc = torch.empty(P, N, dtype=torch.float32)
    for e in range(E):
        m = (sel == e).nonzero().flatten()
        if m.numel():
            acc[m] = (a[m].to(acc_dtype) @ W[e].to(acc_dtype)).float()
    if out_noise is not None:
        acc = acc + out_noise.reshape(-1, N).float()[dst]
    out_codes = None
    if adc is not None:
        out_res, out_bound, wmax = adc
        out_codes, acc = adc_codes(acc, wmax.float()[sel], out_res, out_bound)
    if absmax is not None:
        acc = acc * absmax.flatten().float()[sel_index].view(-1, 1)
    if ir_slot is not None:
        acc = acc * ir_slot.flatten().float().view(-1, 1)
    out = torch.zeros(P, N, dtype=torch.float32)
    out[dst] = acc
    if return_codes:
        cd = None
        if out_codes is not None:
            cd = torch.zeros(P, N, dtype=torch.float32)
            cd[dst] = out_codes
        return out, in_codes, cd
    return out


def combine(res: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """cvmm.py:757-759: y[t,:] = sum_j gate[t,j] * res[t,j,:], accumulated in slot order."""
    T, k = gate.shape
    r = res.view(T, k, -1).float()
    y = torch.zeros(T, r.shape[-1], dtype=torch.float32)
    for j in range(k):
        y = y + gate[:, j:j + 1].float() * r[:, j]
    return y


# --------------------------------------------------------------------------- #
# dW (cvmm.py:300-397)
# --------------------------------------------------------------------------- #
def cvmm_dw(x: torch.Tensor, sel_index: torch.Tensor, sel: torch.Tensor, grads: torch.Tensor,
            n_experts: int, ir_slot: Optional[torch.Tensor] = None,
            out_index: Optional[torch.Tensor] = None, acc_dtype=torch.float64) -> torch.Tensor:
    """dW[e] = sum_{i: sel_i = e} clamp(x[r_i,:], +-ir_i)^T (x) g[b_i,:], b_i = out_index[i] or r_i.
    The input is clamped but neither scaled nor quantised (straight-through), cvmm.py:365-373."""
    x = x.reshape(-1, x.shape[-1]).float()
    g = grads.reshape(-1, grads.shape[-1]).float()
    sel_index = sel_index.flatten().long()
    sel = sel.flatten().long()
    rows = x[sel_index]
    if ir_slot is not None:
        r = ir_slot.flatten().float().view(-1, 1)
        rows = torch.where(rows > r, r.expand_as(rows), rows)
        rows = torch.where(rows < -r, (-r).expand_as(rows), rows)
    gi = g[sel_index if out_index is None else out_index.flatten().long()]
    dW = torch.zeros(n_experts, x.shape[-1], g.shape[-1], dtype=torch.float32)
    for e in range(n_experts):
        m = (sel == e).nonzero().flatten()
        if m.numel():
            dW[e] = (rows[m].to(acc_dtype).T @ gi[m].to(acc_dtype)).float()
    return dW


# --------------------------------------------------------------------------- #
# Backward of one CVMM call (cvmm.py:771-897)
# --------------------------------------------------------------------------- #
@dataclass
class IRParams:
    enable: bool = True
    decay: float = 0.0
    input_min_percentage: float = 0.95
    gradient_relative: bool = True
    gradient_scale: float = 1.0


def cvmm_backward(grad_out: torch.Tensor, x: torch.Tensor, sel_index: torch.Tensor,
                  sel: torch.Tensor, W: torch.Tensor, ir_slot: Optional[torch.Tensor],
                  out_index: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                  res_into_reduction: Optional[torch.Tensor], ir_params: Optional[IRParams],
                  acc_dtype=torch.float64):
    """Returns (dX like x, dW [E,K,N], dIR per sorted slot [P] or None, dGate [T,k] or None).

    Up-projection call (gate None):  x [T,K], grad_out [P,N] by flat slot,
    sel_index = token of sorted slot, out_index = flat slot of sorted slot.
    Down-projection call (gate given): x [P,K] by flat slot, grad_out [T,N],
    sel_index = flat slot of sorted slot, out_index None.
    """
    x2 = x.reshape(-1, x.shape[-1]).float()
    sel_index = sel_index.flatten().long()
    sel = sel.flatten().long()
    P = sel.numel()
    E, K, N = W.shape
    oi = None if out_index is None else out_index.flatten().long()
    g = grad_out.reshape(-1, N).float()
    if gate is not None:
        k = gate.shape[-1]
        gw = (gate.reshape(-1, 1).float() * g.repeat_interleave(k, 0))  # cvmm.py:789, [P,N] by flat slot
    else:
        gw = g
    dW = cvmm_dw(x2, sel_index, sel, gw, E, ir_slot, oi, acc_dtype)     # cvmm.py:812-823

    # grad_x_full, cvmm.py:828-846: same forward kernel on W^T, no DAC
    Wt = W.transpose(1, 2)
    if gate is not None:
        bw_index, bw_out = sel_index // gate.shape[-1], sel_index
    else:
        bw_index, bw_out = oi, None
    gfull = cvmm_forward(g, bw_index, sel, Wt, -1.0, None, bw_out, None, None, None, acc_dtype)  # [P,K] by flat slot

    dir_slot = None
    flat_of_sorted = sel_index if oi is None else oi
    if ir_slot is not None:
        r = ir_slot.flatten().float().view(-1, 1)
        xs = x2[sel_index]                                   # sorted order
        gs = gfull[flat_of_sorted]                           # sorted order
        if gate is not None:
            gs = gs * gate.reshape(-1, 1).float()[sel_index]  # cvmm.py:860-861
        upper = (xs >= r).float()
        lower = (xs <= -r).float()
        notclip_sorted = xs.abs() < r
        d = torch.clamp(upper * gs, max=0.0).sum(-1, keepdim=True) \
            - torch.clamp(lower * gs, min=0.0).sum(-1, keepdim=True)
        if ir_params is None or getattr(ir_params, "gradient_relative", True):
            d = d * r
            d = d * float(getattr(ir_params, "gradient_scale", 1.0) if ir_params is not None else 1.0)
        if ir_params is not None and ir_params.decay > 0:
            pct = notclip_sorted.float().mean()
            d = d + ir_params.decay * r * float(pct > ir_params.input_min_percentage)
        dir_slot = d.flatten()
        notclip_flat = torch.empty_like(notclip_sorted)
        notclip_flat[flat_of_sorted] = notclip_sorted
        gfull = gfull * notclip_flat.float()                 # cvmm.py:881

    dgate = None
    if gate is not None:
        dx = gate.reshape(-1, 1).float() * gfull             # cvmm.py:888
        T = g.shape[0]
        rr = res_into_reduction.reshape(T, gate.shape[-1], N).float()
        dgate = torch.einsum("tjn,tn->tj", rr, g)            # cvmm.py:889
    else:
        T = x2.shape[0]
        dx = gfull.view(T, P // T, K).sum(1)                 # cvmm.py:890-891
    return dx.view_as(x), dW, dir_slot, dgate


# --------------------------------------------------------------------------- #
# Per-expert std (cvmm.py:400-526)
# --------------------------------------------------------------------------- #
def expert_std(x: torch.Tensor, sel_index: torch.Tensor, sel: torch.Tensor, n_experts: int) -> torch.Tensor:
    """sigma_e = sqrt(sum_{routed rows}(x - mu_e)^2 / (n_elem_e - 1)); mu_e the mean of the routed
    rows' means.  Experts without rows give NaN (0/0), as the reference does."""
    x2 = x.reshape(-1, x.shape[-1]).double()
    rows = x2[sel_index.flatten().long()]
    sel = sel.flatten().long()
    out = torch.full((n_experts,), float("nan"), dtype=torch.float64)
    for e in range(n_experts):
        m = rows[sel == e]
        if m.numel():
            mu = m.mean(1).mean()
            out[e] = torch.sqrt(((m - mu) ** 2).sum() / (m.numel() - 1))
    return out.float()


# --------------------------------------------------------------------------- #
# Whole-layer restatement used as the CPU baseline and for the layer-level tests
# --------------------------------------------------------------------------- #
@dataclass
class LayerConfig:
    k: int
    inp_res: float = -1.0             # already converted (see convert_res)
    use_ir: bool = True
    out_noise: float = 0.0
    out_noise_per_channel: bool = True
    w_noise: float = 0.0
    w_noise_per_channel: bool = True
    out_res: float = -1.0
    out_bound: float = -1.0
    seed: int = 0
    ir_params: Optional[IRParams] = None
    act_dtype: torch.dtype = torch.float32   # storage type of activations between the kernels


def layer_forward_backward(x, w_gate, keys, values, input_range, cfg: LayerConfig, grad_y=None,
                           acc_dtype=torch.float32, logits=None):
    """One sigma-MoE analog layer, forward and (if grad_y is given) backward, on the CPU.

    Order of operations follows SigmaMoELayer.forward as restated in
    tests/test_moe_layer_aihwkit.py:60-103 and the two `cvmm_wrapper` calls in
    moe_layer_aihwkit_lightning.py:384-507: router -> sigmoid -> top-k -> sort
    -> up CVMM -> ReLU -> down CVMM with gate-weighted reduction.
    Philox offsets: 0 for the up-projection call, 1 for the down-projection.
    """
    T, D = x.shape
    E, _, F = keys.shape
    k = cfg.k
    if logits is None:
        logits = x.float() @ w_gate.float().T
    s = select_sort(logits, k)
    rnd = (lambda t: t.to(cfg.act_dtype).float()) if cfg.act_dtype != torch.float32 else (lambda t: t)
    ir_up = input_range[0][s.sel.long()] if cfg.use_ir else None
    ir_dn = input_range[1][s.sel.long()] if cfg.use_ir else None
    am_up = None if cfg.use_ir else x.float().abs().amax(-1)

    def prep(W, off):
        wmax = weight_max(W, cfg.out_noise_per_channel)
        Wm = modify_weight(W, cfg.w_noise, cfg.w_noise_per_channel, cfg.seed, off) if cfg.w_noise > 0 else W.float()
        return Wm, wmax

    Kw, kmax = prep(keys, 0)
    Vw, vmax = prep(values, 1)
    P = T * k

    def noise(off, wmax, N):
        if cfg.out_noise <= 0:
            return None
        z = philox_normal8(cfg.seed, off, STREAM_OUT_NOISE, P, N)
        return z * cfg.out_noise * wmax[s.raw_sel.flatten().long()]

    adc_up = (cfg.out_res, cfg.out_bound, kmax) if cfg.out_res > 0 else None
    adc_dn = (cfg.out_res, cfg.out_bound, vmax) if cfg.out_res > 0 else None
    h_pre = cvmm_forward(x, s.token_index, s.sel, Kw, cfg.inp_res, ir_up, s.slot_index, am_up,
                         noise(0, kmax, F), adc_up, acc_dtype)
    h_pre = rnd(h_pre)
    h = torch.relu(h_pre)
    am_dn = None if cfg.use_ir else h.abs().amax(-1)
    res = cvmm_forward(h, s.slot_index, s.sel, Vw, cfg.inp_res, ir_dn, None, am_dn,
                       noise(1, vmax, D), adc_dn, acc_dtype)
    res = rnd(res)
    y = rnd(combine(res, rnd(s.gate)))
    if grad_y is None:
        return y, None
    dh, dV, dir_dn, dgate = cvmm_backward(grad_y, h, s.slot_index, s.sel, Vw, ir_dn, None, s.gate, res,
                                          cfg.ir_params, acc_dtype)
    dh_pre = dh * (h_pre > 0).float()
    dx, dK, dir_up, _ = cvmm_backward(dh_pre, x, s.token_index, s.sel, Kw, ir_up, s.slot_index, None, None,
                                      cfg.ir_params, acc_dtype)
    dlogit = torch.zeros(T, E)
    dlogit.scatter_(1, s.raw_sel.long(), dgate * s.gate * (1 - s.gate))
    dx = dx + dlogit @ w_gate.float()
    dwg = dlogit.T @ x.float()
    d_ir = None
    if cfg.use_ir:
        d_ir = torch.zeros(2, E)
        d_ir[0].index_add_(0, s.sel.long(), dir_up)
        d_ir[1].index_add_(0, s.sel.long(), dir_dn)
    return y, dict(dx=dx, dkeys=dK, dvalues=dV, d_input_range=d_ir, dgate_w=dwg, h=h, res=res, sel=s)
