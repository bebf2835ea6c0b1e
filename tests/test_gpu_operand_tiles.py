"""The operand pre-pass (amoe_operand_tiles) against the tensor-core kernels' own operand prologue: the same gathered
rows, the same DAC arithmetic, so a CVMM call fed by the pre-pass's tiles returns bit-identical results - forward
(quantised and normalised, with input ranges and abs-max), input gradient (converted rows, fp16 gradient scale) - and
the cache it leaves for the weight gradient gives the same dW as the cache the in-kernel prologue writes.  Routing is
ragged (one empty expert, tiles with a single row)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _routing(T, E, k, g, dev, empty=None):
    from analog_moe import ops
    logits = torch.randn(T, E, generator=g)
    logits[:, 0] += 2.0                     # a popular expert: several full tiles
    if empty is not None:
        logits[:, empty] = -1e4
    return ops.select_sort(logits.to(dev), k)


@pytest.mark.parametrize("prec_name", ["split", "f16", "bf16"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["quant_ir", "norm_ir_absmax", "plain"])
def test_forward_from_prepass_tiles_is_bit_identical(prec_name, dtype, mode):
    from analog_moe import ops, _cabi
    prec = _cabi.PRECISION_NAMES[prec_name]
    if prec_name == "f16" and dtype == torch.bfloat16:
        pytest.skip("fp16 operands are the fp32-data mode")
    dev = torch.device("cuda:0")
    T, k, K, N, E = 700, 2, 192, 128, 6
    P = T * k
    g = torch.Generator().manual_seed(7)
    r = _routing(T, E, k, g, dev, empty=3)
    x = (torch.randn(T, K, generator=g) * 1.5).to(dev).to(dtype)
    W = (torch.randn(E, K, N, generator=g) / K ** 0.5).to(dev).to(dtype)
    pw = ops.weight_prepass(W, prec)
    ir = torch.linspace(1.0, 2.5, E, device=dev) if mode != "plain" else None
    am = ops.row_absmax(x) if mode == "norm_ir_absmax" else None
    inp_res = 2.0 / 254.0 if mode == "quant_ir" else -1.0
    kw = dict(P=P, dst_rows=P, ir=ir, ir_by_expert=True, absmax=am, inp_res=inp_res, out_res=254.0, out_bound=12.0,
              want_codes=True)
    ref_cache = ops.OperandCache.empty(P, E, K, prec == _cabi.PREC_SPLIT, dev)
    want, want_codes = ops.cvmm_fwd(x, r.token_index, r.slot_index, r.expert_offsets, pw, prec, a_cache=ref_cache, **kw)
    st = ops.new_status(dev)
    tiles, cache = ops.operand_tiles(x, r.token_index, r.expert_offsets, E, prec, P=P, dac=True, ir=ir, ir_by_expert=True,
                                     absmax=am, inp_res=inp_res, want_cache=True, status=st)
    got, got_codes = ops.cvmm_fwd(x, r.token_index, r.slot_index, r.expert_offsets, pw, prec, a_tiles=tiles, **kw)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    assert torch.equal(got_codes, want_codes)
    assert torch.equal(got, want)
    # the weight-gradient operand: same dW from either cache
    gy = torch.randn(P, N, generator=g).to(dev).to(dtype)
    gmax = ops.grad_absmax(gy, prec)
    gt, _ = ops.operand_tiles(gy, r.slot_index, r.expert_offsets, E, prec, P=P, dac=False, g_absmax=gmax)
    dw_a = ops.cvmm_dw_cached(ref_cache, gt, r.expert_offsets, E, prec, P=P, g_absmax=gmax)
    dw_b = ops.cvmm_dw_cached(cache, gt, r.expert_offsets, E, prec, P=P, g_absmax=gmax)
    assert torch.equal(dw_a, dw_b)
    assert float(dw_a[3].abs().max()) == 0.0            # the empty expert


@pytest.mark.parametrize("prec_name", ["split", "f16", "bf16"])
def test_input_gradient_from_prepass_tiles_is_bit_identical(prec_name):
    from analog_moe import ops, _cabi
    prec = _cabi.PRECISION_NAMES[prec_name]
    dtype = torch.bfloat16 if prec_name == "bf16" else torch.float32
    dev = torch.device("cuda:0")
    T, k, K, N, E = 520, 4, 128, 256, 5
    P = T * k
    g = torch.Generator().manual_seed(9)
    r = _routing(T, E, k, g, dev, empty=2)
    W = (torch.randn(E, K, N, generator=g) / K ** 0.5).to(dev).to(dtype)
    pw = ops.weight_prepass(W, prec)
    h = torch.relu(torch.randn(P, K, generator=g)).to(dev).to(dtype)
    gy = (torch.randn(T, N, generator=g) * 3e-3).to(dev).to(dtype)       # small gradients: the fp16 scale matters
    ir = torch.linspace(0.8, 2.0, E, device=dev)
    gmax = ops.grad_absmax(gy, prec)
    kw = dict(P=P, dst_rows=P, a_row_div=k, x_ref=h, x_ref_row=r.slot_index, ir=ir, ir_by_expert=True,
              row_scale=r.gate.reshape(-1), want_ir_grad=True, x_ref_relu=True, g_absmax=gmax)
    want, want_ir = ops.cvmm_dx(gy, r.slot_index, r.slot_index, r.expert_offsets, pw, prec, **kw)
    st = ops.new_status(dev)
    tiles, _ = ops.operand_tiles(gy, r.slot_index, r.expert_offsets, E, prec, P=P, a_row_div=k, dac=False, g_absmax=gmax,
                                 status=st)
    got, got_ir = ops.cvmm_dx(gy, r.slot_index, r.slot_index, r.expert_offsets, pw, prec, a_tiles=tiles, **kw)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    assert torch.equal(got, want)
    # per-slot input-range gradient: a sum over the row whose order follows the split of the columns among the
    # epilogue warps, which differs between a launch with and without prologue warps
    scale = float(want_ir.abs().max())
    assert float((got_ir - want_ir).abs().max()) <= 1e-5 * scale


def test_prepass_reports_a_source_row_out_of_range():
    from analog_moe import ops, _cabi
    dev = torch.device("cuda:0")
    T, k, K, E = 256, 2, 64, 4
    P = T * k
    g = torch.Generator().manual_seed(1)
    r = _routing(T, E, k, g, dev)
    x = torch.randn(T, K, generator=g).to(dev)
    bad = r.token_index.clone()
    bad[5] = T + 3                          # beyond the rows of x: reported, written as zeros, nothing dereferenced
    st = ops.new_status(dev)
    tiles, _ = ops.operand_tiles(x, bad, r.expert_offsets, E, _cabi.PREC_F16X1, P=P, dac=True, inp_res=2.0 / 254.0,
                                 ir=torch.ones(E, device=dev), ir_by_expert=True, status=st)
    torch.cuda.synchronize()
    assert int(st[0]) == 8                  # AMOE_ERR_INDEX_RANGE
    assert float(tiles.hi[:, 5, :].float().abs().max()) == 0.0
