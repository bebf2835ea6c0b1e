"""Tensor-level wrappers over the C ABI.  PyTorch supplies device memory and the current stream;
all arithmetic happens in the CUDA library."""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _cabi as A
from ._cabi import lib, check, ptr, stream_ptr, dtype_code, launch_on


class Trace:
    """Sums the library's launch counter over the calls it sees and, when `timed`, brackets each call with CUDA events on the
    launching stream (used by the bench for per-kernel durations; adds event overhead)."""

    def __init__(self, timed: bool = False):
        self.timed = timed
        self.calls = []          # (name, tag, start_event, end_event)
        self.launches = 0

    def summary(self):
        torch.cuda.synchronize()
        agg = {}
        for name, tag, e0, e1 in self.calls:
            key = name if not tag else f"{name}[{tag}]"
            ms = e0.elapsed_time(e1) if e0 is not None else 0.0
            a = agg.setdefault(key, [0, 0.0])
            a[0] += 1
            a[1] += ms
        return {k: {"calls": v[0], "ms_total": v[1], "ms_avg": v[1] / v[0]} for k, v in agg.items()}


TRACE: Optional[Trace] = None
_TAG = ""
# NVTX range around every library call ("amoe_cvmm_fwd[up]", ...) for timeline tools; off unless AMOE_NVTX=1 or set here.
NVTX = os.environ.get("AMOE_NVTX", "") not in ("", "0")


def set_tag(tag: str) -> None:
    global _TAG
    _TAG = tag


def _call(name: str, *args) -> None:
    if NVTX:
        torch.cuda.nvtx.range_push(name if not _TAG else f"{name}[{_TAG}]")
        try:
            _call_traced(name, *args)
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        _call_traced(name, *args)


def _call_traced(name: str, *args) -> None:
    tr = TRACE
    if tr is None:
        check(getattr(lib, name)(*args), name)
        return
    before = lib.amoe_launch_count()
    if tr.timed:
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        st = A._LAUNCH_STREAM if A._LAUNCH_STREAM is not None else torch.cuda.current_stream()
        e0.record(st)
        check(getattr(lib, name)(*args), name)
        e1.record(st)
        tr.calls.append((name, _TAG, e0, e1))
    else:
        check(getattr(lib, name)(*args), name)
        tr.calls.append((name, _TAG, None, None))
    tr.launches += lib.amoe_launch_count() - before      # the library's own count of the kernels it launched


_SIDE_STREAMS = {}


def side_stream(device: torch.device, index: int = 0, high_priority: bool = True) -> torch.cuda.Stream:
    """Extra streams per device (`index` 0, 1, ...) for work that runs beside the main chain (the weight pre-passes, the weight
    gradients).  By default a stream has the higher priority: its kernels are few and small in thread blocks (a TMA-fed dW
    kernel is one CTA of six warps per SM), and what waits for them sits on the critical path, so their blocks should get
    the SMs ahead of the main stream's large streaming grids, which then fill in beside them.  `high_priority=False`: for
    large grids that are NOT on the critical path - at the higher priority they would hold back every small kernel of the
    main chain until their last block has been placed."""
    dev = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    key = (dev, index, high_priority)
    st = _SIDE_STREAMS.get(key)
    if st is None:
        prio = int(os.environ.get("AMOE_SIDE_PRIORITY", "-1")) if high_priority else 0
        st = _SIDE_STREAMS[key] = torch.cuda.Stream(device=dev, priority=prio)
    return st


def i32(t: torch.Tensor) -> torch.Tensor:
    """Index tensors cross the ABI as contiguous int32."""
    t = t.reshape(-1)
    if t.dtype != torch.int32:
        t = t.to(torch.int32)
    return t.contiguous()


def default_precision(dtype: torch.dtype) -> int:
    env = os.environ.get("AMOE_PRECISION")
    if env:
        return A.PRECISION_NAMES[env.lower()]
    # bf16 data: operands are exact in one bf16 term.  fp32 data: one fp16 term (about 2e-4 of the result's scale, inside
    # the 1e-3 the specification allows); "split" (bf16 hi+lo, about 2e-5) and "fp32" (CUDA cores) are the tighter modes.
    return A.PREC_BF16X1 if dtype == torch.bfloat16 else A.PREC_F16X1


def new_status(device) -> torch.Tensor:
    return torch.zeros(4, dtype=torch.int32, device=device)


def raise_on_device_status(status: torch.Tensor, where: str) -> None:
    """Synchronises; raises if a kernel recorded a bad index or a wait that ran out."""
    host = (C.c_int32 * 4)()
    code = lib.amoe_read_device_status(ptr(status), C.byref(host), stream_ptr())
    if code != 0:
        raise A.AmoeError(code, f"{where} (detail {host[1]}, {host[2]}, {host[3]})")


# --------------------------------------------------------------------------- routing
@dataclass
class Routing:
    raw_sel: torch.Tensor         # [T,k] int32
    gate: torch.Tensor            # [T,k] fp32
    sel: torch.Tensor             # [P] int32 sorted expert ids
    token_index: torch.Tensor     # [P] int32
    slot_index: torch.Tensor      # [P] int32
    expert_offsets: torch.Tensor  # [E+1] int32


def select_sort(logits: torch.Tensor, k: int, apply_sigmoid: bool = True) -> Routing:
    A.require_cuda(logits)
    logits = logits.reshape(-1, logits.shape[-1]).float().contiguous()
    T, E = logits.shape
    dev = logits.device
    P = T * k
    raw_sel = torch.empty(T, k, dtype=torch.int32, device=dev)
    gate = torch.empty(T, k, dtype=torch.float32, device=dev)
    sel = torch.empty(P, dtype=torch.int32, device=dev)
    tok = torch.empty(P, dtype=torch.int32, device=dev)
    slot = torch.empty(P, dtype=torch.int32, device=dev)
    off = torch.empty(E + 1, dtype=torch.int32, device=dev)
    nbytes = lib.amoe_select_sort_workspace_bytes(T, E, k)
    ws = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=dev)
    _call("amoe_select_sort", ptr(logits), T, E, k, int(apply_sigmoid), ptr(raw_sel), ptr(gate), ptr(sel), ptr(tok),
                               ptr(slot), ptr(off), ptr(ws), nbytes, stream_ptr())
    return Routing(raw_sel, gate, sel, tok, slot, off)


_ROUTER_SMEM_LIMIT = 200 * 1024      # the router kernels that keep the whole [E, D] weight (or its gradient) in shared memory


def _router_fits_smem(E: int, D: int) -> bool:
    return E <= 64 and ((E + 15) // 16 * 16) * D * 4 <= _ROUTER_SMEM_LIMIT


def _router_on_tensor_cores(x2: torch.Tensor, w: torch.Tensor) -> bool:
    """Routers too large for the shared-memory kernels run as one-expert CVMM calls on the tensor cores."""
    E, D = w.shape
    return not _router_fits_smem(E, D) and x2.dtype == w.dtype and D % 8 == 0 and x2.data_ptr() % 16 == 0 and \
        (x2.stride(0) * x2.element_size()) % 16 == 0


_IDENTITY_ROWS = {}


def _identity_rows(T: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """(0 .. T-1, [0, T]) as int32 device tensors: the row lists of a CVMM call whose single expert takes every row."""
    key = (T, device)
    hit = _IDENTITY_ROWS.get(key)
    if hit is None:
        if len(_IDENTITY_ROWS) >= 8:
            _IDENTITY_ROWS.pop(next(iter(_IDENTITY_ROWS)))
        hit = _IDENTITY_ROWS[key] = (torch.arange(T, dtype=torch.int32, device=device),
                                     torch.tensor([0, T], dtype=torch.int32, device=device))
    return hit


def _router_precision(x2: torch.Tensor) -> int:
    # fp32 routers: bf16 hi + lo terms (about 1e-5 of the logits' scale); bf16 routers: exact products
    return A.PREC_SPLIT if x2.dtype == torch.float32 else A.PREC_BF16X1


def router_logits(x2: torch.Tensor, w_sel: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 gate logits [T,E] of x2 [T,D] and w_sel [E,D] (rounded through bf16 when x2 is bf16)."""
    x2 = _rows(x2)
    w = w_sel.contiguous()
    T, D = x2.shape
    E = w.shape[0]
    if _router_on_tensor_cores(x2, w):
        # logits = x @ w^T as a CVMM with one expert that owns all T rows: weight [1, D, E] (a strided view, the weight
        # pre-pass reads it in place), no DAC, no noise; bf16 routers round the result through bf16 like torch's matmul
        prec = _router_precision(x2)
        pw = weight_prepass(w.t().unsqueeze(0), prec, need_fwd=True, need_bwd=False)
        rows, offsets = _identity_rows(T, x2.device)
        out, _ = cvmm_fwd(x2, rows, rows, offsets, pw, prec, P=T, dst_rows=T)
        out = out.float()
        return out if bias is None else out + bias.float()
    out = torch.empty(T, E, dtype=torch.float32, device=x2.device)
    b = None if bias is None else bias.float().contiguous()
    _call("amoe_router_logits", ptr(x2), dtype_code(x2), x2.stride(0), T, D, ptr(w), dtype_code(w), E, ptr(b),
          int(x2.dtype == torch.bfloat16), ptr(out), stream_ptr())
    return out


def router_select(x2: torch.Tensor, w_sel: torch.Tensor, k: int, bias: Optional[torch.Tensor] = None,
                  want_logits: bool = False) -> Tuple["Routing", Optional[torch.Tensor]]:
    """Router matmul, sigmoid, top-k (one kernel) and the expert-contiguous slot sort: the same result as
    select_sort(router_logits(...)).  Falls back to those two calls for routers the fused kernel does not cover."""
    x2 = _rows(x2)
    w = w_sel.contiguous()
    T, D = x2.shape
    E = w.shape[0]
    dev = x2.device
    esz = x2.element_size()
    fused = _router_fits_smem(E, D) and D % 4 == 0 and (x2.stride(0) * esz) % 16 == 0 and \
        (D * w.element_size()) % 16 == 0 and x2.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
    if not fused:
        logits = router_logits(x2, w, bias)
        return select_sort(logits, k, apply_sigmoid=True), logits
    P = T * k
    logits = torch.empty(T, E, dtype=torch.float32, device=dev) if want_logits else None
    raw_sel = torch.empty(T, k, dtype=torch.int32, device=dev)
    gate = torch.empty(T, k, dtype=torch.float32, device=dev)
    b = None if bias is None else bias.float().contiguous()
    _call("amoe_router_select", ptr(x2), dtype_code(x2), x2.stride(0), T, D, ptr(w), dtype_code(w), E, ptr(b),
          int(x2.dtype == torch.bfloat16), k, 1, ptr(logits), ptr(raw_sel), ptr(gate), stream_ptr())
    sel = torch.empty(P, dtype=torch.int32, device=dev)
    tok = torch.empty(P, dtype=torch.int32, device=dev)
    slot = torch.empty(P, dtype=torch.int32, device=dev)
    off = torch.empty(E + 1, dtype=torch.int32, device=dev)
    nbytes = lib.amoe_select_sort_workspace_bytes(T, E, k)
    ws = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=dev)
    _call("amoe_sort_slots", ptr(raw_sel), T, E, k, ptr(sel), ptr(tok), ptr(slot), ptr(off), ptr(ws), nbytes, stream_ptr())
    return Routing(raw_sel, gate, sel, tok, slot, off), logits


def router_backward_w(x2: torch.Tensor, dgate: torch.Tensor, gate: torch.Tensor, token_index: torch.Tensor,
                      slot_index: torch.Tensor, offsets: torch.Tensor, E: int, apply_sigmoid: bool = True,
                      raw_sel: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gradient [E,D] fp32 of the router weight from the gradient of the k picked gate values."""
    x2 = _rows(x2)
    T, D = x2.shape
    P = token_index.numel()
    if raw_sel is not None and not _router_fits_smem(E, D) and D % 8 == 0 and x2.data_ptr() % 16 == 0 and \
            (x2.stride(0) * x2.element_size()) % 16 == 0:
        # dW = dlogits^T @ x as a one-expert weight gradient on the tensor cores: dlogits [T,E] dense (k non-zeros per
        # row), contraction over the T rows; result [1, D, E] transposed back
        prec = _router_precision(x2)
        dl = gate_backward(dgate, gate, raw_sel, E, apply_sigmoid)
        rows, off1 = _identity_rows(T, x2.device)
        dw = cvmm_dw(x2, rows, dl, rows, off1, 1, prec, P=T)
        return dw[0].t().contiguous()
    out = torch.empty(E, D, dtype=torch.float32, device=x2.device)
    nbytes = lib.amoe_router_backward_w_workspace_bytes(P, E, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x2.device)
    _call("amoe_router_backward_w", ptr(x2), dtype_code(x2), x2.stride(0), T, D, ptr(dgate), ptr(gate), int(apply_sigmoid),
          ptr(token_index), ptr(slot_index), ptr(offsets), ptr(raw_sel), P, E, ptr(out), ptr(ws), nbytes, stream_ptr())
    return out


def combine_router(res: torch.Tensor, T: int, k: int, dgate: torch.Tensor, gate: torch.Tensor, raw_sel: torch.Tensor,
                   w_sel: torch.Tensor, apply_sigmoid: bool = True, row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """sum over k of the rows [T*k,N] plus the router's input-gradient term, [T,N] in the rows' dtype."""
    res = _rows(res)
    w = w_sel.contiguous()
    N = res.shape[1]
    y = torch.empty(T, N, dtype=res.dtype, device=res.device)
    _call("amoe_combine_router", ptr(res), dtype_code(res), res.stride(0), ptr(row_index), T, k, N, ptr(dgate), ptr(gate),
          int(apply_sigmoid), ptr(raw_sel), ptr(w), dtype_code(w), w.shape[0], ptr(y), dtype_code(y), y.stride(0),
          stream_ptr())
    return y


def gate_backward(dgate: torch.Tensor, gate: torch.Tensor, raw_sel: torch.Tensor, E: int,
                  apply_sigmoid: bool = True) -> torch.Tensor:
    """dlogits [T,E] fp32 from the gradient of the k picked gate values."""
    k = raw_sel.shape[-1]
    T = raw_sel.numel() // k
    dl = torch.empty(T, E, dtype=torch.float32, device=raw_sel.device)
    _call("amoe_gate_backward", ptr(dgate), ptr(gate), ptr(raw_sel), T, E, k, int(apply_sigmoid), ptr(dl), stream_ptr())
    return dl


def expert_offsets(sel_sorted: torch.Tensor, n_experts: int, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    sel_sorted = i32(sel_sorted)
    off = torch.empty(n_experts + 1, dtype=torch.int32, device=sel_sorted.device)
    _call("amoe_expert_offsets", ptr(sel_sorted), sel_sorted.numel(), n_experts, ptr(off), ptr(status), stream_ptr())
    return off


# --------------------------------------------------------------------------- weights
@dataclass
class PreparedWeights:
    """What the weight pre-pass leaves behind for the CVMM kernels."""
    E: int
    K: int
    N: int
    col_scale: torch.Tensor                 # [E,N] fp32
    col_inv_scale: Optional[torch.Tensor] = None   # [E,N] fp32 reciprocals
    w: Optional[torch.Tensor] = None        # [E,K,N] fp32/bf16 for the CUDA-core mode (modified weights)
    fwd_hi: Optional[torch.Tensor] = None
    fwd_lo: Optional[torch.Tensor] = None
    bwd_hi: Optional[torch.Tensor] = None
    bwd_lo: Optional[torch.Tensor] = None
    workspace: Optional[torch.Tensor] = None


def prepared_dims(K: int, N: int) -> Tuple[int, int, int, int]:
    d = (C.c_int32 * 4)()
    lib.amoe_prepared_dims(K, N, C.byref(d))
    return tuple(int(v) for v in d)


def weight_prepass(w: torch.Tensor, precision: int, *, per_channel_scale: bool = True, noise_std: float = 0.0,
                   noise_per_channel: bool = True, discretize_res: float = -1.0, seed: int = 0, offset: int = 0,
                   step_dev: Optional[torch.Tensor] = None, need_fwd: bool = True, need_bwd: bool = True,
                   need_w_out: bool = False, clip_sigma: float = -1.0, clip_per_channel: bool = False,
                   clip_fixed: float = -1.0, expert_base: int = 0) -> PreparedWeights:
    """`clip_sigma` / `clip_fixed` > 0: the weights are clipped in place first (see clip_weights_) in the same pass."""
    A.require_cuda(w)
    E, K, N = w.shape
    dev = w.device
    modified = noise_std > 0 or discretize_res > 0
    col_scale = torch.empty(E, N, dtype=torch.float32, device=dev)
    a = A.WeightPrepassArgs()
    a.w, a.w_dtype, a.E, a.K, a.N = ptr(w), dtype_code(w), E, K, N
    a.w_stride_e, a.w_stride_k, a.w_stride_n = w.stride()
    a.per_channel_scale = int(per_channel_scale)
    a.noise_std, a.noise_per_channel = float(noise_std), int(noise_per_channel)
    a.discretize_res = float(discretize_res)
    a.seed, a.offset = int(seed) & (2 ** 64 - 1), int(offset) & 0xFFFFFFFF
    a.step_dev = ptr(step_dev)
    a.expert_base = int(expert_base)
    col_inv = torch.empty(E, N, dtype=torch.float32, device=dev)
    a.col_scale = ptr(col_scale)
    a.col_inv_scale = ptr(col_inv)
    out = PreparedWeights(E, K, N, col_scale, col_inv)
    if precision == A.PREC_FP32_SIMT:
        if modified or need_w_out:
            out.w = torch.empty(E, K, N, dtype=torch.float32, device=dev)
            a.w_out = ptr(out.w)
        else:
            out.w = w
    else:
        # bf16 weights are exact in one term unless the modifier adds fp32 noise on top
        split = precision == A.PREC_SPLIT and (w.dtype != torch.bfloat16 or modified)
        a.prepared_f16 = int(precision == A.PREC_F16X1)        # (the 16-bit buffers are typed bf16 either way)
        npad, kpad, kpad2, npad2 = prepared_dims(K, N)
        if need_fwd:
            out.fwd_hi = torch.empty(E, npad, kpad, dtype=torch.bfloat16, device=dev)
            a.fwd_hi = ptr(out.fwd_hi)
            if split:
                out.fwd_lo = torch.empty_like(out.fwd_hi)
                a.fwd_lo = ptr(out.fwd_lo)
        if need_bwd:
            out.bwd_hi = torch.empty(E, kpad2, npad2, dtype=torch.bfloat16, device=dev)
            a.bwd_hi = ptr(out.bwd_hi)
            if split:
                out.bwd_lo = torch.empty_like(out.bwd_hi)
                a.bwd_lo = ptr(out.bwd_lo)
        if need_w_out:
            out.w = torch.empty(E, K, N, dtype=torch.float32, device=dev)
            a.w_out = ptr(out.w)
    clip = clip_sigma > 0 or clip_fixed > 0
    if clip:
        a.clip_sigma, a.clip_per_channel, a.clip_fixed, a.w_clip_out = float(clip_sigma), int(clip_per_channel), float(clip_fixed), ptr(w)
        nbytes = lib.amoe_weight_prepass_clip_workspace_bytes(E, K, N)
    else:
        nbytes = lib.amoe_weight_prepass_workspace_bytes(E, K, N)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    a.workspace, a.workspace_bytes = ptr(ws), nbytes
    _call("amoe_weight_prepass", C.byref(a), stream_ptr())
    out.workspace = ws       # stays alive with the result: the launch stream may differ from the allocating one
    if clip:
        forget_prepared(w)   # the weights were clamped in place
    return out


# prepared weights of unmodified weight tensors, kept while the tensor has not been written to
_PREPARED = {}


def weight_prepass_cached(w: torch.Tensor, precision: int, per_channel_scale: bool = True) -> PreparedWeights:
    """Weight pre-pass without modifier or clipping, skipped when these exact weights (same storage, same version
    counter) were prepared before: an inference layer pays for it once, not on every call.  For calls that do not train
    the weights (the callers decide): a write through `.data` does not move the version counter - `forget_prepared`
    is for those."""
    from torch.multiprocessing.reductions import StorageWeakRef
    # Inside a CUDA-graph capture the check below would be frozen into the graph: a replay after an optimizer step would
    # use stale copies.  Trainable weights are therefore always prepared inside a captured graph; frozen ones may be
    # taken from the cache there too.
    if w.requires_grad and w.is_cuda and torch.cuda.is_current_stream_capturing():
        return weight_prepass(w, precision, per_channel_scale=per_channel_scale, need_fwd=True, need_bwd=True)
    key = (w.data_ptr(), tuple(w.shape), tuple(w.stride()), w.dtype, w.device, precision, per_channel_scale)
    hit = _PREPARED.get(key)
    # valid while the storage is the one that was prepared (a freed storage's address can be handed out again) and
    # nothing has written to the tensor since
    if hit is not None and not hit[0].expired() and hit[1] == w._version:
        return hit[2]
    pw = weight_prepass(w, precision, per_channel_scale=per_channel_scale, need_fwd=True, need_bwd=True)
    if len(_PREPARED) >= 16:
        _PREPARED.pop(next(iter(_PREPARED)))
    _PREPARED[key] = (StorageWeakRef(w.untyped_storage()), w._version, pw)
    return pw


def forget_prepared(w: torch.Tensor) -> None:
    """Drops the cached prepared copies of `w`: for writes that do not move the tensor's version counter (through
    `.data`, or by a kernel of this library writing in place)."""
    ptr_ = w.data_ptr()
    for key in [k for k in _PREPARED if k[0] == ptr_]:
        del _PREPARED[key]


def clip_weights_(w: torch.Tensor, sigma: float = -1.0, per_channel: bool = False, fixed_value: float = -1.0) -> None:
    """In place: clamp w [E,K,N] to +-sigma*std (std of each expert, or of each column with `per_channel`), capped by
    `fixed_value` when that is positive; sigma <= 0 clamps to +-fixed_value.  One pass for the statistics and one for
    the clamp, both inside the weight pre-pass kernels."""
    A.require_cuda(w)
    E, K, N = w.shape
    a = A.WeightPrepassArgs()
    a.w, a.w_dtype, a.E, a.K, a.N = ptr(w), dtype_code(w), E, K, N
    a.w_stride_e, a.w_stride_k, a.w_stride_n = w.stride()
    a.per_channel_scale, a.noise_per_channel, a.discretize_res = 1, 1, -1.0
    a.clip_sigma, a.clip_per_channel, a.clip_fixed, a.w_clip_out = float(sigma), int(per_channel), float(fixed_value), ptr(w)
    nbytes = lib.amoe_weight_prepass_clip_workspace_bytes(E, K, N)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
    a.workspace, a.workspace_bytes = ptr(ws), nbytes
    _call("amoe_weight_prepass", C.byref(a), stream_ptr())
    w._amoe_workspace = ws
    forget_prepared(w)


def tensor_absmax(x2: torch.Tensor, n_rows_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """max|x| over the rows of x2 (over the first n_rows_dev[0] rows when that int32 device tensor is given) as a
    one-element fp32 device tensor: what scales the gradient operands of the fp16 precision."""
    x2 = _rows(x2)
    out = torch.empty(1, dtype=torch.float32, device=x2.device)
    _call("amoe_tensor_absmax", ptr(x2), dtype_code(x2), x2.shape[0], x2.shape[1], x2.stride(0), ptr(n_rows_dev), ptr(out),
          stream_ptr())
    return out


def grad_absmax(g2: torch.Tensor, precision: int, n_rows_dev: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """The scalar the fp16 precision needs for an upstream gradient; None for the other precisions."""
    return tensor_absmax(g2, n_rows_dev) if precision == A.PREC_F16X1 else None


def row_absmax(x2: torch.Tensor) -> torch.Tensor:
    out = torch.empty(x2.shape[0], dtype=torch.float32, device=x2.device)
    _call("amoe_row_absmax", ptr(x2), dtype_code(x2), x2.shape[0], x2.shape[1], x2.stride(0), ptr(out), stream_ptr())
    return out


# --------------------------------------------------------------------------- the CVMM itself
def _rows(t: torch.Tensor) -> torch.Tensor:
    t = t.reshape(-1, t.shape[-1])
    if t.stride(-1) != 1:
        t = t.contiguous()
    return t


def _fill_weights(a: A.CvmmArgs, pw: PreparedWeights, precision: int, backward: bool) -> None:
    if precision == A.PREC_FP32_SIMT:
        w = pw.w
        a.w, a.w_dtype = ptr(w), dtype_code(w)
        a.w_stride_e, a.w_stride_k, a.w_stride_n = w.stride()
    else:
        hi, lo = (pw.bwd_hi, pw.bwd_lo) if backward else (pw.fwd_hi, pw.fwd_lo)
        if hi is None:
            raise RuntimeError("prepared weights for this direction were not requested from weight_prepass")
        a.w_hi, a.w_lo = ptr(hi), ptr(lo)


def cvmm_fwd(x2: torch.Tensor, a_row: torch.Tensor, dst_row: torch.Tensor, offsets: torch.Tensor,
             pw: PreparedWeights, precision: int, *, P: int, dst_rows: int, a_row_div: int = 1,
             ir: Optional[torch.Tensor] = None, absmax: Optional[torch.Tensor] = None, inp_res: float = -1.0,
             noise: Optional[torch.Tensor] = None, noise_std: float = 0.0, seed: int = 0, offset: int = 0,
             step_dev: Optional[torch.Tensor] = None, out_res: float = -1.0, out_bound: float = -1.0, want_codes: bool = False,
             out_dtype: Optional[torch.dtype] = None, status: Optional[torch.Tensor] = None,
             want_out: bool = True, row_meta: Optional[dict] = None, ir_by_expert: bool = False,
             out_relu: bool = False, a_cache: Optional["OperandCache"] = None,
             a_cache_scale: Optional[torch.Tensor] = None, a_tiles: Optional["OperandCache"] = None,
             next_ir: Optional[torch.Tensor] = None, next_inp_res: float = -1.0,
             next_codes: Optional["OperandCache"] = None, out_cache: Optional["OperandCache"] = None,
             out_cache_scale: Optional[torch.Tensor] = None):
    """Returns (out or None, codes or None).  `row_meta` (a dict) receives `row_scale` [dst_rows] and
    `row_expert` [dst_rows], from which, with the codes, the output rows can be rebuilt."""
    x2 = _rows(x2)
    dev = x2.device
    out = torch.empty(dst_rows, pw.N, dtype=out_dtype or x2.dtype, device=dev) if want_out else None
    codes = torch.empty(dst_rows, pw.N, dtype=torch.int8, device=dev) if want_codes else None
    if row_meta is not None:
        row_meta["row_scale"] = torch.empty(dst_rows, dtype=torch.float32, device=dev)
        row_meta["row_expert"] = torch.empty(dst_rows, dtype=torch.int32, device=dev)
    a = A.CvmmArgs()
    a.P, a.E, a.K, a.N, a.precision = P, pw.E, pw.K, pw.N, precision
    a.expert_offsets = ptr(offsets)
    a.a, a.a_dtype, a.a_stride, a.a_rows = ptr(x2), dtype_code(x2), x2.stride(0), x2.shape[0]
    a.a_row, a.a_row_div, a.dst_row, a.dst_rows = ptr(a_row), a_row_div, ptr(dst_row), dst_rows
    _fill_weights(a, pw, precision, backward=False)
    a.ir, a.a_absmax, a.inp_res = ptr(ir), ptr(absmax), float(inp_res)
    a.ir_by_expert, a.out_relu = int(ir_by_expert), int(out_relu)
    if a_cache is not None:
        a.a_cache_hi, a.a_cache_lo, a.a_cache_scale = ptr(a_cache.hi), ptr(a_cache.lo), ptr(a_cache_scale)
        a.cache_rows = a_cache.rows
    if a_tiles is not None:          # the A operand as tiles an earlier kernel prepared (x2 only gives dtype and device)
        a.a_tile_hi, a.a_tile_lo = ptr(a_tiles.hi), ptr(a_tiles.lo)
        a.cache_rows = a_tiles.rows
    if next_codes is not None or out_cache is not None:
        a.next_ir, a.next_inp_res = ptr(next_ir), float(next_inp_res)
        if next_codes is not None:
            a.next_codes = ptr(next_codes.hi)
            a.cache_rows = next_codes.rows
        if out_cache is not None:
            a.out_cache_hi, a.out_cache_lo, a.out_cache_scale = ptr(out_cache.hi), ptr(out_cache.lo), ptr(out_cache_scale)
            a.cache_rows = out_cache.rows
    if noise is not None:
        noise = noise.reshape(-1, pw.N).float().contiguous()
        assert noise.shape[0] == dst_rows
    a.noise, a.noise_std = ptr(noise), float(noise_std)
    a.seed, a.offset = int(seed) & (2 ** 64 - 1), int(offset) & 0xFFFFFFFF
    a.step_dev = ptr(step_dev)
    a.col_scale = ptr(pw.col_scale)
    a.col_inv_scale = ptr(pw.col_inv_scale)
    a.out_res, a.out_bound = float(out_res), float(out_bound)
    if out is not None:
        a.out, a.out_dtype, a.out_stride = ptr(out), dtype_code(out), out.stride(0)
    a.out_codes = ptr(codes)
    if row_meta is not None:
        a.out_row_scale, a.out_row_expert = ptr(row_meta["row_scale"]), ptr(row_meta["row_expert"])
    a.dev_status = ptr(status)
    _call("amoe_cvmm_fwd", C.byref(a), stream_ptr())
    return out, codes


def cvmm_dx(g2: torch.Tensor, a_row: torch.Tensor, dst_row: torch.Tensor, offsets: torch.Tensor,
            pw: PreparedWeights, precision: int, *, P: int, dst_rows: int, a_row_div: int = 1,
            x_ref: Optional[torch.Tensor] = None, x_ref_row: Optional[torch.Tensor] = None,
            ir: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None, want_ir_grad: bool = False,
            relative: bool = True, grad_scale: float = 1.0, keep_count: Optional[torch.Tensor] = None,
            out_dtype: Optional[torch.dtype] = None, status: Optional[torch.Tensor] = None,
            ir_by_expert: bool = False, x_ref_relu: bool = False, a_cache: Optional["OperandCache"] = None,
            out_cache: Optional["OperandCache"] = None, a_tiles: Optional["OperandCache"] = None,
            g_absmax: Optional[torch.Tensor] = None, want_out: bool = True):
    """`a_tiles`: the A operand as an operand cache written by an earlier kernel (TMA-fed, no gather); g2 then only
    gives dtype and device.  `g_absmax`: the device scalar of the fp16 precision (see tensor_absmax).  `want_out=False`
    (with `out_cache`): only the operand cache is written."""
    g2 = _rows(g2)
    dev = g2.device
    out = torch.empty(dst_rows, pw.K, dtype=out_dtype or g2.dtype, device=dev) if want_out else None
    ir_grad = torch.empty(P, dtype=torch.float32, device=dev) if want_ir_grad else None
    a = A.CvmmArgs()
    a.P, a.E, a.K, a.N, a.precision = P, pw.E, pw.K, pw.N, precision
    a.expert_offsets = ptr(offsets)
    a.a, a.a_dtype, a.a_stride, a.a_rows = ptr(g2), dtype_code(g2), g2.stride(0), g2.shape[0]
    a.a_row, a.a_row_div, a.dst_row, a.dst_rows = ptr(a_row), a_row_div, ptr(dst_row), dst_rows
    _fill_weights(a, pw, precision, backward=True)
    a.inp_res = -1.0
    a.ir = ptr(ir)
    a.ir_by_expert, a.x_ref_relu = int(ir_by_expert), int(x_ref_relu)
    if a_cache is not None:
        a.a_cache_hi, a.a_cache_lo = ptr(a_cache.hi), ptr(a_cache.lo)
        a.cache_rows = a_cache.rows
    if out_cache is not None:
        a.out_cache_hi, a.out_cache_lo = ptr(out_cache.hi), ptr(out_cache.lo)
        a.cache_rows = out_cache.rows
    if a_tiles is not None:
        a.a_tile_hi, a.a_tile_lo = ptr(a_tiles.hi), ptr(a_tiles.lo)
        a.cache_rows = a_tiles.rows
    if out is not None:
        a.out, a.out_dtype, a.out_stride = ptr(out), dtype_code(out), out.stride(0)
    else:
        a.out_dtype, a.out_stride = dtype_code(g2), pw.K
    a.a_absmax_dev = ptr(g_absmax)
    if x_ref is not None:
        x_ref = _rows(x_ref)
        a.x_ref, a.x_ref_dtype, a.x_ref_stride, a.x_ref_row = ptr(x_ref), dtype_code(x_ref), x_ref.stride(0), ptr(x_ref_row)
        a.x_ref_rows = x_ref.shape[0]
    a.row_scale, a.ir_grad = ptr(row_scale), ptr(ir_grad)
    a.ir_grad_relative, a.ir_grad_scale = int(relative), float(grad_scale)
    a.keep_count = ptr(keep_count)
    a.dev_status = ptr(status)
    _call("amoe_cvmm_dx", C.byref(a), stream_ptr())
    return out, ir_grad


def cvmm_dw(x2: torch.Tensor, x_row: torch.Tensor, g2: torch.Tensor, g_row: torch.Tensor, offsets: torch.Tensor,
            E: int, precision: int, *, P: int, ir: Optional[torch.Tensor] = None, g_div: int = 1,
            g_scale: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
            ir_by_expert: bool = False, g_absmax: Optional[torch.Tensor] = None) -> torch.Tensor:
    x2, g2 = _rows(x2), _rows(g2)
    K, N = x2.shape[1], g2.shape[1]
    dw = torch.empty(E, K, N, dtype=torch.float32, device=x2.device)
    a = A.DwArgs()
    a.P, a.E, a.K, a.N, a.precision = P, E, K, N, precision
    a.expert_offsets = ptr(offsets)
    a.x, a.x_dtype, a.x_stride, a.x_rows, a.x_row, a.ir = ptr(x2), dtype_code(x2), x2.stride(0), x2.shape[0], ptr(x_row), ptr(ir)
    a.g, a.g_dtype, a.g_stride, a.g_rows, a.g_row = ptr(g2), dtype_code(g2), g2.stride(0), g2.shape[0], ptr(g_row)
    a.g_div, a.g_scale, a.dw = g_div, ptr(g_scale), ptr(dw)
    a.ir_by_expert = int(ir_by_expert)
    a.g_absmax_dev = ptr(g_absmax)
    nbytes = lib.amoe_cvmm_dw_workspace_bytes(P, E, K, N, precision)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x2.device) if nbytes else None
    a.workspace, a.workspace_bytes = ptr(ws), nbytes
    a.dev_status = ptr(status)
    _call("amoe_cvmm_dw", C.byref(a), stream_ptr())
    return dw


@dataclass
class OperandCache:
    """One CVMM operand as bf16 hi (+ lo) terms in padded tile-row order, written by a forward / input-gradient
    kernel and read by the weight-gradient kernel through TMA."""
    hi: torch.Tensor              # [ceil(cols/64), rows, 64] bf16
    lo: Optional[torch.Tensor]
    cols: int = 0

    @property
    def rows(self) -> int:
        return self.hi.shape[1]

    @staticmethod
    def empty(P: int, E: int, cols: int, split: bool, device) -> "OperandCache":
        rows = int(lib.amoe_padded_rows(P, E))
        hi = torch.empty((cols + 63) // 64, rows, 64, dtype=torch.bfloat16, device=device)
        return OperandCache(hi, torch.empty_like(hi) if split else None, cols)


def operand_tiles_ok(x2: torch.Tensor, precision: int) -> bool:
    """Rows the operand pre-pass can take: a tensor-core precision, 64-column blocks, 16-byte aligned rows."""
    return precision != A.PREC_FP32_SIMT and x2.shape[-1] % 64 == 0 and x2.data_ptr() % 16 == 0 and \
        (x2.stride(0) * x2.element_size()) % 16 == 0


def operand_tiles(x2: torch.Tensor, a_row: torch.Tensor, offsets: torch.Tensor, E: int, precision: int, *, P: int,
                  a_row_div: int = 1, dac: bool = True, ir: Optional[torch.Tensor] = None, ir_by_expert: bool = False,
                  absmax: Optional[torch.Tensor] = None, inp_res: float = -1.0, want_tiles: bool = True,
                  want_cache: bool = False, cache_scale: Optional[torch.Tensor] = None,
                  g_absmax: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                  row_absmax: Optional[torch.Tensor] = None):
    """The A operand of a CVMM call as TMA tiles, by a streaming pre-pass (amoe_operand_tiles).  Returns
    (tiles or None, cache or None): `tiles` goes to cvmm_fwd / cvmm_dx as `a_tiles`, `cache` (forward operands only:
    the clamped, unquantised rows) to cvmm_dw_cached.  For gradient rows (dac=False) the tiles are both.
    fp16 rows (gradient rows of the fp16 precision that arrived scaled row by row) come with `row_absmax`."""
    x2 = _rows(x2)
    K = x2.shape[-1]
    split = precision == A.PREC_SPLIT
    # integer codes up to 256 in magnitude are exact in one bf16 term; anything else in split precision takes hi + lo
    quant = dac and inp_res > 0
    tile_split = split and not (quant and inp_res >= 1.0 / 256.0) and \
        not (x2.dtype == torch.bfloat16 and dac and ir is None and absmax is None)
    # (gradient rows always carry their residual term in split precision - zeros for bf16 rows: the weight gradient
    # takes both operands with or both without one)
    tiles = OperandCache.empty(P, E, K, tile_split, x2.device) if want_tiles else None
    cache = OperandCache.empty(P, E, K, split, x2.device) if (want_cache and dac) else None
    a = A.OperandTilesArgs()
    a.P, a.E, a.K, a.precision = P, E, K, precision
    a.expert_offsets = ptr(offsets)
    a.a, a.a_stride, a.a_rows = ptr(x2), x2.stride(0), x2.shape[0]
    a.a_dtype = A.F16 if x2.dtype == torch.float16 else dtype_code(x2)
    a.a_row_absmax = ptr(row_absmax)
    a.a_row, a.a_row_div, a.dac = ptr(a_row), a_row_div, int(dac)
    a.ir, a.ir_by_expert, a.a_absmax, a.inp_res = ptr(ir), int(ir_by_expert), ptr(absmax), float(inp_res)
    if tiles is not None:
        a.tile_hi, a.tile_lo = ptr(tiles.hi), ptr(tiles.lo)
        a.cache_rows = tiles.rows
    if cache is not None:
        a.cache_hi, a.cache_lo, a.cache_scale = ptr(cache.hi), ptr(cache.lo), ptr(cache_scale)
        a.cache_rows = cache.rows
    a.g_absmax_dev = ptr(g_absmax)
    a.dev_status = ptr(status)
    _call("amoe_operand_tiles", C.byref(a), stream_ptr())
    return tiles, cache


def operand_cache_ok(precision: int, *cols: int) -> bool:
    return precision != A.PREC_FP32_SIMT and all(c % 16 == 0 for c in cols)


def cvmm_dw_cached(x_cache: OperandCache, g_cache: OperandCache, offsets: torch.Tensor, E: int, precision: int, *,
                   P: int, status: Optional[torch.Tensor] = None, expected_rows: int = 0,
                   g_absmax: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dW [E,K,N] from two operand caches ([rows,K] and [rows,N]).  `expected_rows`: the likely slot count when P is
    only an upper bound (tunes the work split)."""
    K, N = x_cache.cols, g_cache.cols
    dev = x_cache.hi.device
    dw = torch.empty(E, K, N, dtype=torch.float32, device=dev)
    a = A.DwArgs()
    a.P, a.E, a.K, a.N, a.precision = P, E, K, N, precision
    a.expert_offsets = ptr(offsets)
    a.x_hi, a.x_lo, a.g_hi, a.g_lo = ptr(x_cache.hi), ptr(x_cache.lo), ptr(g_cache.hi), ptr(g_cache.lo)
    a.cache_rows = x_cache.rows
    a.expected_rows = int(expected_rows)
    a.g_div = 1
    a.dw = ptr(dw)
    a.g_absmax_dev = ptr(g_absmax)
    nbytes = lib.amoe_cvmm_dw_workspace_bytes_tuned(P, int(expected_rows), E, K, N, precision)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None
    a.workspace, a.workspace_bytes = ptr(ws), nbytes
    a.dev_status = ptr(status)
    _call("amoe_cvmm_dw", C.byref(a), stream_ptr())
    dw._amoe_workspace = ws     # alive as long as the result: the launch stream may differ from the allocating one
    return dw


# --------------------------------------------------------------------------- reductions
def combine(res: torch.Tensor, w: Optional[torch.Tensor], T: int, k: int, out_dtype=None,
            row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    res = _rows(res)
    N = res.shape[1]
    y = torch.empty(T, N, dtype=out_dtype or res.dtype, device=res.device)
    if w is not None:
        w = w.reshape(-1).float().contiguous()
    _call("amoe_combine", ptr(res), dtype_code(res), res.stride(0), ptr(row_index), ptr(w), T, k, N, ptr(y), dtype_code(y),
                           y.stride(0), stream_ptr())
    return y


def combine_codes(codes: torch.Tensor, col_scale: torch.Tensor, raw_sel: torch.Tensor, row_mult: Optional[torch.Tensor],
                  step: float, w: Optional[torch.Tensor], T: int, k: int, out_dtype=torch.float32,
                  row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    N = codes.shape[-1]
    y = torch.empty(T, N, dtype=out_dtype, device=codes.device)
    if w is not None:
        w = w.reshape(-1).float().contiguous()
    _call("amoe_combine_codes", ptr(codes), ptr(col_scale), ptr(i32(raw_sel)), ptr(row_mult), float(step), ptr(w), T, k,
                                 N, ptr(y), dtype_code(y), y.stride(0), ptr(row_index), stream_ptr())
    return y


def row_dot(res: torch.Tensor, g: torch.Tensor, k: int, row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    res, g = _rows(res), _rows(g)
    P, N = res.shape
    d = torch.empty(P, dtype=torch.float32, device=res.device)
    _call("amoe_row_dot", ptr(res), dtype_code(res), res.stride(0), ptr(row_index), ptr(g), dtype_code(g), g.stride(0), P, k, N,
                           ptr(d), stream_ptr())
    return d


def row_dot_codes(codes: torch.Tensor, col_scale: torch.Tensor, row_expert: torch.Tensor, row_scale: torch.Tensor,
                  step: float, g: torch.Tensor, k: int, row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    g = _rows(g)
    P, N = codes.shape
    d = torch.empty(P, dtype=torch.float32, device=codes.device)
    _call("amoe_row_dot_codes", ptr(codes), ptr(col_scale), ptr(row_expert), ptr(row_scale), float(step), ptr(g),
          dtype_code(g), g.stride(0), P, k, N, ptr(d), ptr(row_index), stream_ptr())
    return d


def adc_step(out_res: float, out_bound: float) -> float:
    """2 * out_bound * res in fp32 arithmetic (the value the kernels use)."""
    f = torch.tensor
    res = (f(1.0, dtype=torch.float32) / f(out_res, dtype=torch.float32)) if out_res > 1.0 else f(out_res, dtype=torch.float32)
    return float(f(2.0, dtype=torch.float32) * f(out_bound, dtype=torch.float32) * res)


def ir_grad_reduce(ir_grad_slot: torch.Tensor, offsets: torch.Tensor, input_range: Optional[torch.Tensor], E: int,
                   decay: float = 0.0, min_percentage: float = 0.95, keep_count: Optional[torch.Tensor] = None,
                   total_elements: float = 0.0, total_rows: Optional[torch.Tensor] = None, cols: int = 0,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`total_rows` (int64 device scalar) * cols replaces `total_elements` as the denominator of the kept fraction.
    `out`: a contiguous fp32 [E] tensor (e.g. one row of a [2, E] gradient) to write into."""
    if out is None:
        out = torch.empty(E, dtype=torch.float32, device=ir_grad_slot.device)
    _call("amoe_ir_grad_reduce", ptr(ir_grad_slot), ptr(offsets), ptr(input_range), E, float(decay),
          float(min_percentage), ptr(keep_count), float(total_elements), ptr(total_rows), int(cols), ptr(out), stream_ptr())
    return out


def expert_std(x: torch.Tensor, x_row: torch.Tensor, offsets: torch.Tensor, E: int,
               status: Optional[torch.Tensor] = None) -> torch.Tensor:
    x2 = _rows(x)
    P = x_row.numel()
    out = torch.empty(E, dtype=torch.float32, device=x2.device)
    nbytes = lib.amoe_expert_std_workspace_bytes(E)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x2.device)
    _call("amoe_expert_std", ptr(x2), dtype_code(x2), x2.stride(0), x2.shape[1], x2.shape[0], ptr(x_row), ptr(offsets),
          P, E, ptr(out), ptr(ws), nbytes, ptr(status), stream_ptr())
    return out


# --------------------------------------------------------------------------- expert-parallel helpers
def ep_pack(x: torch.Tensor, src_row: torch.Tensor, ir: Optional[torch.Tensor] = None, inp_res: float = -1.0,
            src_div: int = 1, row_scale: Optional[torch.Tensor] = None):
    """Rows x[src_row[i] // src_div] (times row_scale[src_row[i]]) in the order of src_row; with `ir` and
    `inp_res` given: (int8 DAC codes, fp32 scale per row) instead."""
    x2 = _rows(x)
    P, K = src_row.numel(), x2.shape[1]
    if ir is not None and inp_res > 0:
        codes = torch.empty(P, K, dtype=torch.int8, device=x2.device)
        scale = torch.empty(P, dtype=torch.float32, device=x2.device)
        _call("amoe_ep_pack", ptr(x2), dtype_code(x2), x2.stride(0), K, ptr(src_row), src_div, None, P, ptr(ir),
              float(inp_res), None, ptr(codes), ptr(scale), stream_ptr())
        return codes, scale
    rows = torch.empty(P, K, dtype=x2.dtype, device=x2.device)
    _call("amoe_ep_pack", ptr(x2), dtype_code(x2), x2.stride(0), K, ptr(src_row), src_div, ptr(row_scale), P, None, -1.0,
          ptr(rows), None, None, stream_ptr())
    return rows, None


def ep_local_plan(recv_counts: torch.Tensor, R: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """recv_counts [G,El] int32 on the device -> (local_order [R], local_offsets [El+1])."""
    G, El = recv_counts.shape
    dev = recv_counts.device
    order = torch.empty(max(R, 1), dtype=torch.int32, device=dev)[:R]
    offsets = torch.empty(El + 1, dtype=torch.int32, device=dev)
    _call("amoe_ep_local_plan", ptr(recv_counts), G, El, R, ptr(order), ptr(offsets), stream_ptr())
    return order, offsets


def ep_plan(gathered: torch.Tensor, rank: int) -> torch.Tensor:
    """gathered [G,G,El] int32 (source, destination, local expert) -> this rank's plan (int32 device array)."""
    G, _, El = gathered.shape
    plan = torch.empty(int(lib.amoe_ep_plan_ints(G, El)), dtype=torch.int32, device=gathered.device)
    _call("amoe_ep_plan", ptr(gathered), rank, G, El, ptr(plan), stream_ptr())
    return plan


def ep_local_plan_dev(plan: torch.Tensor, G: int, El: int, cap: int,
                      status: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    order = torch.empty(cap, dtype=torch.int32, device=plan.device)
    offsets = torch.empty(El + 1, dtype=torch.int32, device=plan.device)
    _call("amoe_ep_local_plan_dev", ptr(plan), G, El, cap, ptr(order), ptr(offsets), ptr(status), stream_ptr())
    return order, offsets


def invert_index(idx: torch.Tensor) -> torch.Tensor:
    inv = torch.empty_like(idx)
    _call("amoe_invert_index", ptr(idx), idx.numel(), ptr(inv), stream_ptr())
    return inv


def ep_unpack(recv: torch.Tensor, dst_row: torch.Tensor, out_rows: int) -> torch.Tensor:
    recv = recv.contiguous()
    P, N = recv.shape
    out = (torch.empty if out_rows == P else torch.zeros)(out_rows, N, dtype=recv.dtype, device=recv.device)
    _call("amoe_ep_unpack", ptr(recv), dtype_code(recv), N, ptr(dst_row), P, ptr(out), out.stride(0), stream_ptr())
    return out
