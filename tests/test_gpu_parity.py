"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle and against the
golden vectors produced by the reference.  Tolerances are written next to each comparison."""
import os

import numpy as np
import pytest
import torch

from oracle import cvmm_oracle as O
from test_oracle_golden import LAYER_CASES, load

pytestmark = pytest.mark.gpu

PRECS = {"simt": 2, "split": 1, "bf16x1": 0, "f16x1": 3}
# max abs error relative to max|reference| (scale floored at 1): CUDA-core fp32; bf16 hi+lo split on
# tensor cores; single bf16 pass (weights and unquantised operands rounded to 8 bits of mantissa); single fp16
# pass (11-bit significands; the specification's bound for fp32 data is 1e-3).
TOL = {"simt": 2e-5, "split": 1e-4, "bf16x1": 3e-2, "f16x1": 1e-3}


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from analog_moe import _cabi
    assert _cabi.lib.amoe_check_device() == 0, "the kernels are built for sm_100a only"
    return torch.device("cuda:0")


class IRP:
    def __init__(self, enable, decay=0.0, input_min_percentage=0.95):
        self.enable, self.decay, self.input_min_percentage = enable, decay, input_min_percentage


class IOP:
    pass


def run_layer_cuda(c, prec, dev, ext_kw=None):
    from analog_moe import CVMM, CVMMExt
    T, k, E = c["T"], c["k"], c["E"]
    sel = c["sel"].to(dev)
    perm = c["perm"].to(dev).long()
    use_ir = bool(c["use_ir"])
    x = c["x"].to(dev).view(1, T, -1).requires_grad_()
    keys = c["keys"].to(dev).requires_grad_()
    values = c["values"].to(dev).requires_grad_()
    gate = c["gate"].to(dev).view(1, T, k).requires_grad_()
    ir = c["input_range"].to(dev).requires_grad_()
    sel3 = sel.view(1, T, k)
    irp = IRP(use_ir, float(c["decay"]))
    bir_up = ir[0][sel3.long()] if use_ir else None
    bir_dn = ir[1][sel3.long()] if use_ir else None
    n_up = c["noise_up"].to(dev).unsqueeze(0) if "noise_up" in c else None
    n_dn = c["noise_dn"].to(dev).unsqueeze(0) if "noise_dn" in c else None
    ext = lambda: CVMMExt(precision=PRECS[prec], check_status=True, **(ext_kw or {}))
    h_pre = CVMM.apply(x, perm // k, sel3, keys, c["inp_res"], bir_up, perm, None, n_up, irp, IOP(), ext())
    h_pre.retain_grad()
    h = torch.relu(h_pre)
    h.retain_grad()
    y = CVMM.apply(h, perm, sel3, values, c["inp_res"], bir_dn, None, gate, n_dn, irp, IOP(), ext())
    (y * c["grad_y"].to(dev).view(1, T, -1)).sum().backward()
    out = dict(h_pre=h_pre.detach(), y=y.detach(), dh=h.grad, dh_pre=h_pre.grad, dx=x.grad, dkeys=keys.grad,
               dvalues=values.grad, dgate=gate.grad)
    if use_ir:
        out["d_input_range"] = ir.grad
    return {k_: v.float().cpu() for k_, v in out.items()}


def compare(name, prec, key, val, ref):
    val = val.reshape(ref.shape)
    if prec == "bf16x1":
        # single bf16 pass: held to a norm-wise bound (weights rounded to 8 bits of mantissa)
        rel = float((val - ref).norm() / ref.norm().clamp_min(1e-12))
        assert rel <= 1e-2, f"{name}:{key}:{prec} relative Frobenius error {rel:.3e}"
        return
    scale = max(1.0, float(ref.abs().max()))
    err = float((val - ref).abs().max())
    assert err <= TOL[prec] * scale, f"{name}:{key}:{prec} max err {err:.3e} (scale {scale:.3g})"


@pytest.mark.parametrize("name", LAYER_CASES)
def test_layer_cascade_vs_reference_golden_fp32_fma(golden_dir, dev, name):
    """Up-projection -> ReLU -> down-projection chained, forward and backward, in the CUDA-core fp32
    mode (the reference's own arithmetic), against the reference's outputs."""
    c = load(golden_dir, name)
    got = run_layer_cuda(c, "simt", dev)
    for key, val in got.items():
        compare(name, "simt", key, val, c[key])


@pytest.mark.parametrize("prec", ["split", "bf16x1", "f16x1"])
@pytest.mark.parametrize("name", LAYER_CASES)
def test_cvmm_calls_vs_reference_golden(golden_dir, dev, name, prec):
    """Each CVMM call on the reference's own inputs (the second call gets the reference's hidden
    activations and the first call's backward the reference's upstream gradient).  Chaining the two
    calls through a ReLU and a second DAC amplifies 1e-5 differences into whole quantisation steps,
    so the tensor-core modes are checked call by call."""
    from analog_moe import CVMM, CVMMExt
    c = load(golden_dir, name)
    T, k = c["T"], c["k"]
    sel3 = c["sel"].to(dev).view(1, T, k)
    perm = c["perm"].to(dev).long()
    use_ir = bool(c["use_ir"])
    irp = IRP(use_ir, float(c["decay"]))
    ir = c["input_range"].to(dev).requires_grad_()
    ext = lambda: CVMMExt(precision=PRECS[prec], check_status=True)
    # up-projection
    x = c["x"].to(dev).view(1, T, -1).requires_grad_()
    keys = c["keys"].to(dev).requires_grad_()
    n_up = c["noise_up"].to(dev).unsqueeze(0) if "noise_up" in c else None
    h_pre = CVMM.apply(x, perm // k, sel3, keys, c["inp_res"], ir[0][sel3.long()] if use_ir else None, perm, None,
                       n_up, irp, IOP(), ext())
    h_pre.backward(c["dh_pre"].to(dev).view_as(h_pre))
    compare(name, prec, "h_pre", h_pre.detach().cpu(), c["h_pre"])
    compare(name, prec, "dx", x.grad.cpu(), c["dx"])
    compare(name, prec, "dkeys", keys.grad.cpu(), c["dkeys"])
    # down-projection
    h = torch.relu(c["h_pre"]).to(dev).view(1, T, k, -1).requires_grad_()
    values = c["values"].to(dev).requires_grad_()
    gate = c["gate"].to(dev).view(1, T, k).requires_grad_()
    n_dn = c["noise_dn"].to(dev).unsqueeze(0) if "noise_dn" in c else None
    y = CVMM.apply(h, perm, sel3, values, c["inp_res"], ir[1][sel3.long()] if use_ir else None, None, gate, n_dn,
                   irp, IOP(), ext())
    y.backward(c["grad_y"].to(dev).view_as(y))
    compare(name, prec, "y", y.detach().cpu(), c["y"])
    compare(name, prec, "dh", h.grad.cpu(), c["dh"])
    compare(name, prec, "dvalues", values.grad.cpu(), c["dvalues"])
    compare(name, prec, "dgate", gate.grad.cpu(), c["dgate"])
    if use_ir:
        compare(name, prec, "d_input_range", ir.grad.cpu(), c["d_input_range"])


def rand_routing(T, E, k, seed, dev):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    s = O.select_sort(logits, k)
    return logits, s


@pytest.mark.parametrize("T,E,k", [(1, 4, 1), (7, 4, 2), (512, 8, 2), (1000, 64, 8), (4099, 16, 4), (333, 1024, 32)])
def test_select_sort(dev, T, E, k):
    from analog_moe import ops
    logits, s = rand_routing(T, E, k, T + E, dev)
    r = ops.select_sort(logits.to(dev), k)
    # bit-exact integer outputs
    assert torch.equal(r.raw_sel.cpu(), s.raw_sel)
    assert torch.equal(r.sel.cpu(), s.sel)
    assert torch.equal(r.token_index.cpu(), s.token_index)
    assert torch.equal(r.slot_index.cpu(), s.slot_index)
    assert torch.equal(r.expert_offsets.cpu(), s.expert_offsets)
    # gate values: sigmoid evaluated by expf on the device vs the host library, 1e-6 absolute
    assert torch.allclose(r.gate.cpu(), s.gate, atol=1e-6, rtol=0)
    assert torch.equal(ops.expert_offsets(r.sel, E).cpu(), s.expert_offsets)


def test_select_sort_ties_and_skew(dev):
    from analog_moe import ops
    logits = torch.zeros(64, 8)
    logits[:, 5] = 9.0          # everyone picks expert 5 first, then the lowest ids on the tie
    r = ops.select_sort(logits.to(dev), 3)
    assert torch.equal(r.raw_sel.cpu(), torch.tensor([[5, 0, 1]], dtype=torch.int32).expand(64, 3))
    off = r.expert_offsets.cpu().tolist()
    assert off == [0, 64, 128, 128, 128, 128, 192, 192, 192]


def test_dac_codes_bit_exact_with_adversarial_ties(dev):
    """Integer DAC codes must equal the oracle's bit for bit, including inputs that sit on or next to
    a rounding tie of the (x/ir)/res chain."""
    from analog_moe import ops
    res = 2.0 / 254.0
    g = torch.Generator().manual_seed(11)
    P, K = 256, 512
    ir = torch.rand(P, generator=g) * 3 + 0.3
    m = torch.randint(-127, 127, (P, K), generator=g).float()
    x = (m + 0.5) * res * ir.view(-1, 1)                       # nominal ties
    x = x + (torch.randint(-3, 4, (P, K), generator=g).float() * torch.finfo(torch.float32).eps * x.abs())
    x[::7] = torch.randn(K, generator=g) * 2                   # ordinary rows, some clipping
    _, want = O.dac(x, ir, None, res)
    codes, scale = ops.ep_pack(x.to(dev), torch.arange(P, dtype=torch.int32, device=dev), ir.to(dev), res)
    assert torch.equal(codes.cpu().float(), want), "DAC code mismatch"
    assert torch.equal(scale.cpu(), ir)


@pytest.mark.parametrize("res", [2.0 / 254.0, 2.0 / 62.0, 2.0 / 1022.0, 0.1])
def test_dac_codes_bit_exact_large_random_sample(dev, res):
    """The kernels divide with two fused multiply-adds on a correctly rounded reciprocal; this must
    reproduce IEEE division bit for bit (4M values, irregular input ranges, several resolutions)."""
    from analog_moe import ops
    g = torch.Generator().manual_seed(int(res * 1e6))
    P, K = 4096, 1024
    ir = torch.rand(P, generator=g) * 7.9 + 0.013
    ir[::3] = torch.exp(torch.randn(P, generator=g)[::3] * 2)          # a few decades of magnitudes
    x = torch.randn(P, K, generator=g) * ir.view(-1, 1) * 0.8
    x[:, ::5] = (torch.randint(-int(1 / res), int(1 / res) + 1, (P, K), generator=g).float()[:, ::5] + 0.5) \
        * res * ir.view(-1, 1)                                          # nominal ties
    _, want = O.dac(x, ir, None, res)
    if abs(want).max() > 127:
        keep = want.abs().amax(1) <= 127                                # int8 transport of ep_pack
        x, ir, want = x[keep], ir[keep], want[keep]
    if res < 1 / 127.5:
        pytest.skip("codes do not fit the int8 transport used to read them back")
    codes, _ = ops.ep_pack(x.to(dev), torch.arange(x.shape[0], dtype=torch.int32, device=dev), ir.to(dev), res)
    assert torch.equal(codes.cpu().float(), want)


@pytest.mark.parametrize("prec", ["simt", "split", "bf16x1", "f16x1"])
def test_dac_codes_through_the_gemm(dev, prec):
    """With identity weights the CVMM output is code*res*ir: the codes come back exactly."""
    from analog_moe import ops
    res = 2.0 / 254.0
    T, K, E = 300, 64, 3
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, K, generator=g) * 1.5
    logits, s = rand_routing(T, E, 1, 9, dev)
    ir_e = torch.tensor([1.0, 2.0, 0.5])
    ir = ir_e[s.sel.long()]
    W = torch.eye(K).repeat(E, 1, 1)
    _, want = O.dac(x[s.token_index.long()], ir, None, res)
    pw = ops.weight_prepass(W.to(dev), PRECS[prec])
    out, _ = ops.cvmm_fwd(x.to(dev), s.token_index.to(dev), s.slot_index.to(dev), s.expert_offsets.to(dev), pw,
                          PRECS[prec], P=T, dst_rows=T, ir=ir.to(dev), inp_res=res)
    got = out.cpu()[s.slot_index.long()] / (res * ir.view(-1, 1))
    assert torch.equal(torch.round(got), want)
    assert float((got - want).abs().max()) < 1e-3


@pytest.mark.parametrize("prec", ["simt", "split", "f16x1"])
def test_adc_codes(dev, prec):
    """ADC codes against the oracle: no mismatch away from rounding ties; near a tie (pre-rounding
    value within 1e-3 of .5, where fp32 summation order decides) at most one code apart."""
    from analog_moe import ops
    T, K, N, E, k = 200, 96, 80, 5, 2
    g = torch.Generator().manual_seed(21)
    x = torch.randn(T, K, generator=g)
    W = torch.randn(E, K, N, generator=g) / K ** 0.5
    logits, s = rand_routing(T, E, k, 3, dev)
    ir = torch.full((T * k,), 2.5)
    res = 2.0 / 254.0
    wmax = O.weight_max(W, True)
    out_w, _, codes_w = O.cvmm_forward(x, s.token_index, s.sel, W, res, ir, s.slot_index, None, None,
                                       (254.0, 12.0, wmax), return_codes=True)
    pw = ops.weight_prepass(W.to(dev), PRECS[prec])
    out, codes = ops.cvmm_fwd(x.to(dev), s.token_index.to(dev), s.slot_index.to(dev), s.expert_offsets.to(dev), pw,
                              PRECS[prec], P=T * k, dst_rows=T * k, ir=ir.to(dev), inp_res=res, out_res=254.0,
                              out_bound=12.0, want_codes=True)
    codes = codes.cpu().float()
    # pre-rounding value from the oracle, to classify ties
    acc = O.cvmm_forward(x, s.token_index, s.sel, W, res, None if False else ir, s.slot_index) / 2.5
    e_of_slot = torch.empty(T * k, dtype=torch.long)
    e_of_slot[s.slot_index.long()] = s.sel.long()
    v = acc * (1.0 / wmax[e_of_slot]) * (1.0 / O.adc_step(254.0, 12.0))
    # (fp16 weights move the pre-rounding value by up to ~2e-4 of its magnitude, i.e. a few hundredths of a code)
    tie = 5e-2 if prec == "f16x1" else 1e-3
    near_tie = ((v - torch.floor(v)) - 0.5).abs() < tie
    diff = (codes - codes_w).abs()
    assert int((diff[~near_tie] != 0).sum()) == 0
    assert float(diff.max()) <= 1.0
    assert float(near_tie.float().mean()) < 5 * tie
    same = diff == 0
    assert torch.allclose(out.cpu()[same], out_w[same], rtol=1e-6, atol=1e-6)
    assert codes.abs().max() <= 127


@pytest.mark.parametrize("prec", ["simt", "split", "f16x1"])
def test_adc_codes_path_equals_materialised_path(dev, prec):
    """Down-projection with ADC: keeping the per-slot rows as int8 codes (combine and gate gradient
    read the codes) gives bit-identical y, dX, dW, d(gate), d(input range) to materialising the rows."""
    from analog_moe import CVMM, CVMMExt
    T, k, F, D, E = 300, 3, 72, 136, 5
    g = torch.Generator().manual_seed(12)
    logits = torch.randn(T, E, generator=g)
    s = O.select_sort(logits, k)
    sel3 = s.sel.to(dev).view(1, T, k)
    outs = []
    for codes_path in (True, False):
        h = (torch.rand(1, T, k, F, generator=torch.Generator().manual_seed(3)) * 2).to(dev).requires_grad_()
        W = (torch.randn(E, F, D, generator=torch.Generator().manual_seed(4)) / F ** 0.5).to(dev).requires_grad_()
        gate = s.gate.clone().to(dev).view(1, T, k).requires_grad_()
        ir = torch.linspace(1.0, 2.0, E).to(dev).requires_grad_()
        ext = CVMMExt(precision=PRECS[prec], out_res=254.0, out_bound=12.0, adc_codes_path=codes_path, check_status=True)
        y = CVMM.apply(h, s.slot_index.to(dev).long(), sel3, W, 2.0 / 254.0, ir[sel3.long()], None, gate, None,
                       IRP(True, 0.01), IOP(), ext)
        y.backward(torch.randn(1, T, D, generator=torch.Generator().manual_seed(5)).to(dev))
        outs.append([y.detach(), h.grad, W.grad, gate.grad, ir.grad])
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_philox_noise_elementwise_and_statistics(dev):
    """The in-kernel Philox noise equals the oracle's generator element by element (1e-4: fast-math
    log/sincos), and its mean/std over a seed sweep are within 2% of the requested values."""
    from analog_moe import ops
    T, K, N, E, k = 128, 32, 64, 4, 2
    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, K, generator=g)
    W = torch.randn(E, K, N, generator=g) / K ** 0.5
    logits, s = rand_routing(T, E, k, 4, dev)
    P = T * k
    pw = ops.weight_prepass(W.to(dev), 2)
    args = (x.to(dev), s.token_index.to(dev), s.slot_index.to(dev), s.expert_offsets.to(dev), pw, 2)
    clean, _ = ops.cvmm_fwd(*args, P=P, dst_rows=P)
    e_of_slot = torch.empty(P, dtype=torch.long)
    e_of_slot[s.slot_index.long()] = s.sel.long()
    wmax = O.weight_max(W, True)[e_of_slot]
    zs = []
    for seed in range(8):
        noisy, _ = ops.cvmm_fwd(*args, P=P, dst_rows=P, noise_std=0.04, seed=1234 + seed, offset=3)
        z = ((noisy - clean).cpu() / (0.04 * wmax))
        want = O.philox_normal8(1234 + seed, 3, O.STREAM_OUT_NOISE, P, N)
        assert float((z - want).abs().max()) < 2e-3   # fp32 cancellation in (noisy-clean) on top of 1e-4
        zs.append(z)
    z = torch.stack(zs)
    assert abs(float(z.mean())) < 0.02
    assert abs(float(z.std()) - 1.0) < 0.02


@pytest.mark.parametrize("per_channel", [True, False])
def test_weight_prepass(dev, per_channel):
    from analog_moe import ops
    E, K, N = 3, 70, 52
    g = torch.Generator().manual_seed(8)
    W = torch.randn(E, K, N, generator=g) * 0.1
    pw = ops.weight_prepass(W.to(dev), 1, per_channel_scale=per_channel, noise_std=0.02, noise_per_channel=per_channel,
                            seed=77, offset=5, need_w_out=True)
    assert torch.equal(pw.col_scale.cpu(), O.weight_max(W, per_channel))
    want = O.modify_weight(W, 0.02, per_channel, 77, 5)
    assert torch.allclose(pw.w.cpu(), want, atol=2e-6, rtol=0)   # |noise| ~ 1e-2, generator agrees to 1e-4
    # prepared operand copies: hi+lo reproduces W' to 2^-16 relative; padding is zero
    npad, kpad, kpad2, npad2 = ops.prepared_dims(K, N)
    f = (pw.fwd_hi.float() + pw.fwd_lo.float()).cpu()
    assert f.shape == (E, npad, kpad)
    assert torch.allclose(f[:, :N, :K], pw.w.cpu().transpose(1, 2), rtol=2 ** -15, atol=1e-9)
    assert float(f[:, N:, :].abs().max()) == 0 and float(f[:, :, K:].abs().max()) == 0
    b = (pw.bwd_hi.float() + pw.bwd_lo.float()).cpu()
    assert b.shape == (E, kpad2, npad2)
    assert torch.allclose(b[:, :K, :N], pw.w.cpu(), rtol=2 ** -15, atol=1e-9)
    # discretisation
    pw2 = ops.weight_prepass(W.to(dev), 2, noise_per_channel=per_channel, discretize_res=0.1, need_w_out=True)
    assert torch.allclose(pw2.w.cpu(), O.modify_weight(W, 0.0, per_channel, 0, 0, 0.1), atol=1e-7, rtol=0)


def test_expert_std(golden_dir, dev):
    from analog_moe import cvmm_std
    c = load(golden_dir, "expert_std")
    k = c["k"]
    sel, perm = c["sel"].to(dev), c["perm"].to(dev).long()
    up = cvmm_std(c["x"].to(dev), perm // k, sel, c["E"])
    dn = cvmm_std(c["xs"].to(dev), perm, sel, c["E"])
    assert torch.allclose(up.cpu(), c["std_up"], rtol=2e-5, atol=0)   # fp64 accumulation here, fp32 atomics there
    assert torch.allclose(dn.cpu(), c["std_dn"], rtol=2e-5, atol=0)


@pytest.mark.parametrize("prec", ["simt", "split", "f16x1"])
def test_dw_is_deterministic_and_handles_empty_experts(dev, prec):
    from analog_moe import ops
    T, K, N, E, k = 500, 130, 72, 6, 2
    g = torch.Generator().manual_seed(31)
    x = torch.randn(T, K, generator=g)
    gr = torch.randn(T * k, N, generator=g)
    logits = torch.randn(T, E, generator=g)
    logits[:, 2] = -50.0                                   # expert 2 never selected
    s = O.select_sort(logits, k)
    ir = torch.full((T * k,), 1.0)
    want = O.cvmm_dw(x, s.token_index, s.sel, gr, E, ir, s.slot_index)
    a = [t.to(dev) for t in (x, s.token_index, gr, s.slot_index, s.expert_offsets)]
    d1 = ops.cvmm_dw(*a, E, PRECS[prec], P=T * k, ir=ir.to(dev))
    d2 = ops.cvmm_dw(*a, E, PRECS[prec], P=T * k, ir=ir.to(dev))
    assert torch.equal(d1, d2)
    assert float(d1[2].abs().max()) == 0.0
    scale = float(want.abs().max())
    assert float((d1.cpu() - want).abs().max()) <= TOL[prec] * scale


def test_dw_segmented_under_skewed_routing(dev):
    """Large slot counts take the segmented path (partial tiles + ordered reduction).  Zipf-like skew,
    one expert with no slots, sizes that are not multiples of the tile: result vs oracle, and two runs
    bit-identical."""
    from analog_moe import ops, _cabi
    T, K, N, E, k = 6000, 200, 136, 8, 2
    assert _cabi.lib.amoe_cvmm_dw_workspace_bytes(T * k, E, K, N, 1) > 0
    g = torch.Generator().manual_seed(77)
    x = torch.randn(T, K, generator=g)
    gr = torch.randn(T * k, N, generator=g)
    logits = torch.randn(T, E, generator=g) - 1.5 * torch.log(torch.arange(1, E + 1).float())
    logits[:, 5] = -50.0
    s = O.select_sort(logits, k)
    counts = (s.expert_offsets[1:] - s.expert_offsets[:-1]).float()
    assert counts.max() > 3 * counts[counts > 0].min()
    ir = torch.full((T * k,), 1.5)
    want = O.cvmm_dw(x, s.token_index, s.sel, gr, E, ir, s.slot_index)
    a = [t.to(dev) for t in (x, s.token_index, gr, s.slot_index, s.expert_offsets)]
    d1 = ops.cvmm_dw(*a, E, 1, P=T * k, ir=ir.to(dev))
    d2 = ops.cvmm_dw(*a, E, 1, P=T * k, ir=ir.to(dev))
    assert torch.equal(d1, d2)
    assert float(d1[5].abs().max()) == 0.0
    assert float((d1.cpu() - want).abs().max()) <= TOL["split"] * float(want.abs().max())


def test_index_out_of_range_is_reported_not_dereferenced(dev):
    from analog_moe import ops, _cabi
    T, K, N, E = 64, 32, 32, 2
    x = torch.randn(T, K, device=dev)
    W = torch.randn(E, K, N, device=dev)
    logits, s = rand_routing(T, E, 1, 1, dev)
    bad = s.token_index.clone()
    bad[5] = T + 1000
    st = ops.new_status(dev)
    pw = ops.weight_prepass(W, 1)
    for prec in (2, 1):
        st.zero_()
        ops.cvmm_fwd(x, bad.to(dev), s.slot_index.to(dev), s.expert_offsets.to(dev), pw if prec == 1 else
                     ops.weight_prepass(W, 2), prec, P=T, dst_rows=T, status=st)
        with pytest.raises(_cabi.AmoeError) as ei:
            ops.raise_on_device_status(st, "test")
        assert ei.value.status == 8


@pytest.mark.parametrize("prec,dtype", [("split", torch.float32), ("bf16x1", torch.bfloat16), ("f16x1", torch.float32)])
def test_layer_module_vs_oracle(dev, prec, dtype):
    """AnalogSigmaMoELayer end to end (router, select/sort, both CVMMs with DAC, ADC, backward)."""
    from analog_moe import AnalogSigmaMoELayer, TorchInferenceRPUConfig
    T, D, F, E, k = 256, 128, 64, 8, 2
    cfg = TorchInferenceRPUConfig()
    cfg.forward.inp_res = 254.0
    cfg.pre_post.input_range.init_value = 3.0
    cfg.pre_post.input_range.decay = 0.0
    torch.manual_seed(0)
    layer = AnalogSigmaMoELayer(cfg, d_model=D, n_experts=E, expert_size=F, k=k, precision=PRECS[prec]).to(dev).to(dtype)
    x = torch.randn(2, T // 2, D, device=dev, dtype=dtype, requires_grad=True)
    gy = torch.randn(2, T // 2, D, device=dev, dtype=dtype)
    layer.eval()
    y, _ = layer(x)
    (y.float() * gy.float()).sum().backward()
    f = lambda t: t.detach().float().cpu()
    lc = O.LayerConfig(k=k, inp_res=2.0 / 254.0, use_ir=True, ir_params=O.IRParams(decay=0.0), act_dtype=dtype)
    logits = f(layer.expert_sel(x.detach())).view(T, E)        # same logits, so the same experts are picked
    yo, go = O.layer_forward_backward(f(x).view(T, D), f(layer.expert_sel.weight), f(layer.keys), f(layer.values),
                                      f(layer.input_range), lc, f(gy).view(T, D), acc_dtype=torch.float64,
                                      logits=logits)
    # fp32: 1e-4 of the scale, except where the hidden activation's DAC code flips (see the call-by-call
    # test); bf16: activations are rounded to 8 bits between the calls
    tol = 2e-3 if dtype == torch.float32 else 3e-2
    if prec == "f16x1":
        # fp16 weights move a hidden activation by ~2e-4 of its scale; where that crosses a DAC rounding tie the second
        # call sees a whole quantisation step (1/127 of the range), a few per cent of the hidden units
        tol = 1e-2
    for name, got, want in [("y", f(y).view(T, D), yo), ("dx", f(x.grad).view(T, D), go["dx"]),
                            ("dkeys", f(layer.keys.grad), go["dkeys"]), ("dvalues", f(layer.values.grad), go["dvalues"]),
                            ("d_ir", f(layer.input_range.grad), go["d_input_range"]),
                            ("dgate_w", f(layer.expert_sel.weight.grad), go["dgate_w"])]:
        scale = max(1.0, float(want.abs().max()))
        err = float((got - want).abs().max())
        assert err <= tol * scale, f"{name}: {err:.3e} vs scale {scale:.3g}"


@pytest.mark.gpu
@pytest.mark.parametrize("dims", [(384, 160, 96, 8, 3), (320, 128, 128, 4, 2)])
@pytest.mark.parametrize("prec,dtype,use_ir", [("simt", torch.float32, True), ("split", torch.float32, True),
                                               ("split", torch.float32, False), ("bf16x1", torch.bfloat16, True),
                                               ("f16x1", torch.float32, True), ("f16x1", torch.float32, False)])
def test_fused_layer_step_equals_the_composition(dev, prec, dtype, use_ir, dims):
    """The single-node layer step (ReLU, per-expert input ranges, decay term and gate backward folded into the
    kernels) against the composition route() -> CVMM -> ReLU -> CVMM with every non-ideality on: same Philox
    draws, same kernels, so everything but summation-order effects of the glue must agree exactly."""
    from analog_moe import AnalogSigmaMoELayer, TorchInferenceRPUConfig, WeightModifierType
    # (the second shape has an expert size that is a multiple of 64: the up-projection's dX then takes its A tiles by TMA)
    T, D, F, E, k = dims
    cfg = TorchInferenceRPUConfig()
    cfg.forward.inp_res = 254.0
    cfg.forward.out_res = 254.0
    cfg.forward.out_bound = 12.0
    cfg.forward.out_noise = 0.03
    cfg.pre_post.input_range.enable = use_ir
    cfg.pre_post.input_range.init_value = 2.5
    cfg.pre_post.input_range.decay = 0.01
    cfg.pre_post.input_range.input_min_percentage = 0.5
    cfg.modifier.type = WeightModifierType.ADD_NORMAL_PER_CHANNEL
    cfg.modifier.std_dev = 0.02
    torch.manual_seed(3)
    layer = AnalogSigmaMoELayer(cfg, d_model=D, n_experts=E, expert_size=F, k=k, precision=PRECS[prec],
                                noise_seed=77).to(dev).to(dtype)
    layer.train()
    x0 = torch.randn(2, T // 2, D, device=dev, dtype=dtype)
    gy = torch.randn(2, T // 2, D, device=dev, dtype=dtype)
    results = {}
    for fused in (True, False):
        layer.fused = fused
        layer.noise_step.zero_()
        for p_ in layer.parameters():
            p_.grad = None
        x = x0.clone().requires_grad_()
        y, aux = layer(x)
        assert float(aux) == 0.0
        y.backward(gy)
        torch.cuda.synchronize()
        results[fused] = dict(y=y.detach().float(), dx=x.grad.float(), dkeys=layer.keys.grad.float(),
                              dvalues=layer.values.grad.float(), dsel=layer.expert_sel.weight.grad.float(),
                              dir=layer.input_range.grad.float() if use_ir else torch.zeros(1, device=dev))
    assert int(layer.noise_step) == 1
    # the gate comes from the select kernel's sigmoid in one path and from torch.sigmoid in the other (an ulp),
    # and the router's input gradient is added in a different order
    # (the weight gradients come from the cached operands, where the gate multiplies h instead of gy before the
    # bf16 hi/lo split: both factorings carry the split's own 2^-16 error)
    for key in results[True]:
        a, b = results[True][key], results[False][key]
        assert torch.isfinite(a).all(), key
        # (and the gate logits come from two different matmul kernels, so the gates differ in their last bits)
        tol = 2e-2 if dtype != torch.float32 else (3e-5 if key in ("dkeys", "dvalues") and prec != "simt" else 1e-5)
        if prec == "f16x1":
            # the fused step hands the hidden gradient on as fp16 tiles and multiplies the gate into h before the fp16
            # rounding; the composition passes fp32 rows and multiplies it into gy: 2^-12 per operand either way
            tol = 1e-5 if key == "y" else 1e-3
        scale = max(1.0, float(b.abs().max()))
        err = float((a - b).abs().max())
        assert err <= tol * scale, f"{key}: {err:.3e} vs scale {scale:.3g}"


@pytest.mark.gpu
@pytest.mark.parametrize("prec,dtype", [("split", torch.float32), ("bf16x1", torch.bfloat16), ("f16x1", torch.float32)])
def test_dw_from_operand_caches_equals_dw_from_rows(dev, prec, dtype):
    """Weight gradients computed from the bf16 operand copies that the forward / input-gradient kernels leave
    behind (TMA-fed kernel) against the kernel that gathers and converts the fp32 rows itself.  Same hi/lo terms and
    the same products; only the gate multiplies h instead of gy in the down-projection, so agreement is to rounding."""
    from analog_moe import AnalogSigmaMoELayer, TorchInferenceRPUConfig
    T, D, F, E, k = 1536, 192, 80, 6, 4        # > 4096 slots: the segmented (split-K) path; K, N not multiples of 64
    cfg = TorchInferenceRPUConfig()
    cfg.forward.inp_res = 254.0
    cfg.forward.out_res = 254.0
    cfg.forward.out_bound = 12.0
    cfg.pre_post.input_range.init_value = 2.0
    torch.manual_seed(5)
    layer = AnalogSigmaMoELayer(cfg, d_model=D, n_experts=E, expert_size=F, k=k, precision=PRECS[prec]).to(dev).to(dtype)
    with torch.no_grad():
        layer.router_bias = torch.tensor([2.0, 0.0, 0.0, -1.0, -30.0, 0.5], device=dev, dtype=dtype)   # one empty expert
    layer.eval()
    x0 = torch.randn(1, T, D, device=dev, dtype=dtype)
    gy = torch.randn(1, T, D, device=dev, dtype=dtype)
    res = {}
    for cached in (True, False):
        layer.operand_caches = cached
        for p_ in layer.parameters():
            p_.grad = None
        x = x0.clone().requires_grad_()
        y, _ = layer(x)
        y.backward(gy)
        res[cached] = [y.detach().float(), x.grad.float(), layer.keys.grad.float(), layer.values.grad.float()]
    assert torch.equal(res[True][0], res[False][0]) and torch.equal(res[True][1], res[False][1])
    for a, b in zip(res[True][2:], res[False][2:]):
        assert torch.isfinite(a).all()
        scale = float(b.abs().max())
        tol = 3e-5 if dtype == torch.float32 else 1e-2     # the split's own 2^-16, see the docstring
        if prec == "f16x1":
            tol = 5e-4                                     # fp16's 2^-12 per operand
        assert float((a - b).abs().max()) <= tol * scale
    assert float(res[True][3][4].abs().max()) == 0.0      # the expert nobody was routed to


@pytest.mark.gpu
@pytest.mark.parametrize("T,D,E,k,dtype", [(300, 136, 5, 2, torch.float32), (1000, 1024, 16, 4, torch.float32),
                                           (257, 96, 64, 8, torch.float32), (129, 70, 3, 1, torch.float32),
                                           (512, 256, 40, 4, torch.bfloat16)])
def test_router_kernels_vs_torch(dev, T, D, E, k, dtype):
    """Gate logits, router weight gradient and the fused (sum over k + router input gradient) against torch."""
    from analog_moe import ops
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, D, generator=g).to(dev).to(dtype)
    w = (torch.randn(E, D, generator=g) / D ** 0.5).to(dev).to(dtype)
    bias = torch.randn(E, generator=g).to(dev).to(dtype)
    logits = ops.router_logits(x, w, bias)
    ref = (x.double() @ w.double().t())
    if dtype == torch.bfloat16:
        ref = (ref.to(dtype).double() + bias.double()).to(dtype).double()
        assert float((logits.double() - ref).abs().max()) <= 0.04      # an ulp of bf16 at |logit| < 8
    else:
        ref = ref + bias.double()
        assert float((logits.double() - ref).abs().max()) <= 1e-5
    r = ops.select_sort(logits, k, apply_sigmoid=True)
    # the same selection with the top-k inside the router kernel: bit-identical
    r2, lg2 = ops.router_select(x, w, k, bias, want_logits=True)
    assert torch.equal(lg2, logits)
    for name in ("raw_sel", "gate", "sel", "token_index", "slot_index", "expert_offsets"):
        assert torch.equal(getattr(r2, name), getattr(r, name)), name
    dgate = torch.randn(T * k, generator=g).to(dev)
    gate = r.gate
    c = (dgate * (1 - gate.reshape(-1)) * gate.reshape(-1)).double()
    dl = torch.zeros(T, E, dtype=torch.float64, device=dev)
    dl.scatter_(1, r.raw_sel.long(), c.view(T, k))
    # weight gradient
    dw = ops.router_backward_w(x, dgate, gate, r.token_index, r.slot_index, r.expert_offsets, E)
    ref_dw = dl.t() @ x.double()
    assert float((dw.double() - ref_dw).abs().max()) <= 1e-4 * max(1.0, float(ref_dw.abs().max()))
    dw2 = ops.router_backward_w(x, dgate, gate, r.token_index, r.slot_index, r.expert_offsets, E)
    assert torch.equal(dw, dw2)                                           # fixed summation order
    dw3 = ops.router_backward_w(x, dgate, gate, r.token_index, r.slot_index, r.expert_offsets, E, raw_sel=r.raw_sel)
    assert float((dw3.double() - ref_dw).abs().max()) <= 1e-4 * max(1.0, float(ref_dw.abs().max()))   # token-major variant
    # sum over k + router term
    rows = torch.randn(T * k, D, generator=g).to(dev).to(dtype)
    y = ops.combine_router(rows, T, k, dgate, gate, r.raw_sel, w)
    ref_y = rows.double().view(T, k, D).sum(1) + dl @ w.double()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((y.double() - ref_y).abs().max()) <= tol * max(1.0, float(ref_y.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("G,E,k,dtype", [(2, 8, 2, torch.float32), (4, 16, 4, torch.float32), (8, 16, 3, torch.bfloat16)])
def test_device_driven_exchange_emulated_ranks(dev, G, E, k, dtype):
    """The expert-parallel exchange kernels with G ranks emulated on one GPU (one buffer per rank, the "peer" pointers
    are local): plan from the gathered counts, rows stored into their owners' buffers, regrouped by local expert, and
    sent back.  Checked against the host plan (`ep.step_plan` arithmetic) and as a round trip."""
    from analog_moe import ops
    from analog_moe._cabi import lib, stream_ptr
    El, D = E // G, 72
    Ts = [150 + 37 * r for r in range(G)]                      # ragged: a different token count per rank
    g = torch.Generator().manual_seed(G * 100 + E)
    xs = [torch.randn(T, D, generator=g).to(dev).to(dtype) for T in Ts]
    logits = [torch.randn(T, E, generator=g) for T in Ts]
    logits[0][:, E - 1] = -50.0                                # nobody on rank 0 picks the last expert
    routes = [ops.select_sort(l.to(dev), k) for l in logits]
    counts = torch.stack([(r.expert_offsets[1:] - r.expert_offsets[:-1]).view(G, El) for r in routes]).contiguous()  # [s,d,e]
    tot = counts.sum(-1).cpu()
    p_cap = max(T * k for T in Ts)
    cap = G * p_cap
    recv = [torch.full((cap, D), float("nan"), device=dev, dtype=dtype) for _ in range(G)]
    back = [torch.full((p_cap, D), float("nan"), device=dev, dtype=dtype) for _ in range(G)]
    recv_ptrs = torch.tensor([t.data_ptr() for t in recv], dtype=torch.int64, device=dev)
    back_ptrs = torch.tensor([t.data_ptr() for t in back], dtype=torch.int64, device=dev)
    plans = [ops.ep_plan(counts, r) for r in range(G)]
    dc = ops.dtype_code(xs[0])
    status = ops.new_status(dev)
    for r in range(G):
        st = lib.amoe_ep_put(xs[r].data_ptr(), dc, D, D, Ts[r], routes[r].token_index.data_ptr(), 1, None, Ts[r] * k,
                             routes[r].sel.data_ptr(), El, plans[r].data_ptr(), recv_ptrs.data_ptr(), G, cap,
                             status.data_ptr(), stream_ptr())
        assert st == 0
    torch.cuda.synchronize()
    for d in range(G):
        plan = plans[d].cpu()
        R = int(tot[:, d].sum())
        assert int(plan[0]) == R and int(plan[1]) == Ts[d] * k
        # receive buffer: for source s, that source's sorted rows for this rank's experts, in order
        want = []
        for s in range(G):
            lo = int(tot[s, :d].sum())
            n = int(tot[s, d])
            want.append(xs[s][routes[s].token_index[lo:lo + n].long()])
        want = torch.cat(want)
        assert torch.equal(recv[d][:R], want)
        assert torch.isnan(recv[d][R:].float()).all()          # nothing written past the rows that exist
        order, offsets = ops.ep_local_plan_dev(plans[d], G, El, cap)
        ref_order, ref_offsets = ops.ep_local_plan(counts[:, d, :].contiguous(), R)
        assert torch.equal(order[:R], ref_order) and torch.equal(offsets, ref_offsets)
        # rows regrouped by local expert really belong to that expert
        owner = torch.cat([routes[s].sel[int(tot[s, :d].sum()):int(tot[s, :d].sum()) + int(tot[s, d])] for s in range(G)])
        eo = offsets.cpu()
        for e in range(El):
            assert bool((owner[order[int(eo[e]):int(eo[e + 1])].long()] == d * El + e).all())
        st = lib.amoe_ep_put_back(recv[d].data_ptr(), dc, D, D, plans[d].data_ptr(), back_ptrs.data_ptr(), G, cap, p_cap,
                                  status.data_ptr(), stream_ptr())
        assert st == 0
    torch.cuda.synchronize()
    for r in range(G):                                         # round trip: every rank gets its sorted rows back
        P = Ts[r] * k
        assert torch.equal(back[r][:P], xs[r][routes[r].token_index.long()])
    ops.raise_on_device_status(status, "exchange")             # nothing was dropped
    # buffers too small for the plan: the kernels say so in the status word and write nothing out of bounds
    small = torch.full((8, D), float("nan"), device=dev, dtype=dtype)
    small_ptrs = torch.tensor([small.data_ptr()] * G, dtype=torch.int64, device=dev)
    st = lib.amoe_ep_put(xs[0].data_ptr(), dc, D, D, Ts[0], routes[0].token_index.data_ptr(), 1, None, Ts[0] * k,
                         routes[0].sel.data_ptr(), El, plans[0].data_ptr(), small_ptrs.data_ptr(), G, 8,
                         status.data_ptr(), stream_ptr())
    assert st == 0
    import ctypes as C
    host = (C.c_int32 * 4)()
    assert lib.amoe_read_device_status(status.data_ptr(), C.byref(host), stream_ptr()) == 8    # AMOE_ERR_INDEX_RANGE
    order = torch.full((16,), -7, dtype=torch.int32, device=dev)
    offs = torch.empty(El + 1, dtype=torch.int32, device=dev)
    status.zero_()
    assert lib.amoe_ep_local_plan_dev(plans[1].data_ptr(), G, El, 8, order.data_ptr(), offs.data_ptr(), status.data_ptr(),
                                      stream_ptr()) == 0
    assert lib.amoe_read_device_status(status.data_ptr(), C.byref(host), stream_ptr()) == 8
    assert bool((order[8:] == -7).all())                       # nothing written past the 8 rows the array holds
