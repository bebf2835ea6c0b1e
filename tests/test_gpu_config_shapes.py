"""Oracle comparisons at the shapes of the benchmark configurations (2, 3, 4, 5), where the CPU oracle cannot run in
full: forward (DAC codes, ADC codes, dequantised rows), input gradient with the clip mask, per-slot input-range gradient
and weight gradient, each against an fp64 evaluation of the oracle's definitions on a sample - 256 sorted positions for
the row-wise results, three (expert, 64 x 64 block) picks for dW, which needs every slot of the expert.

Bounds.  fp32 data, split precision: 1e-4 of the result's scale (the reference's own test tolerance).  bf16 data,
single-pass bf16: the result is stored as bf16, so each element is within 2^-7 of its row's largest magnitude (half a
bf16 ulp of the row maximum is 2^-9; the bound leaves room for the one-code ADC / rounding-tie differences described
next to the ADC contract).  ADC codes: at most one code apart, and apart only for values within 1e-3 of a rounding tie
(fp32 / bf16 accumulation order decides those); everything else is compared on the positions where the codes agree.
"""
import pytest
import torch

from oracle import cvmm_oracle as O

pytestmark = pytest.mark.gpu

CONFIGS = {
    # name: T, k, D, F, E, dtype, zipf, out_res, backward
    "c2": (8192, 4, 1024, 128, 16, torch.float32, 0.0, 254.0, True),
    "c3": (32768, 8, 2048, 256, 64, torch.bfloat16, 0.0, 254.0, False),
    "c4": (16384, 4, 1024, 128, 32, torch.float32, 1.2, 254.0, True),
    "c5": (8192, 6, 1536, 192, 48, torch.bfloat16, 0.0, 62.0, True),
}
OUT_BOUND = 12.0
RES = 2.0 / 254.0


def _close(got, want, tol, what, row_max=False):
    got, want = got.double(), want.double()
    if row_max:
        scale = want.abs().amax(-1, keepdim=True).clamp_min(1e-30)
        err = float(((got - want).abs() / scale).max())
    else:
        err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-30)
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:g}"


def _projection_check(name, tag, dev, x, a_row, dst_row, r, W, ir_e, gy, g_row, g_div, gate, dtype, out_res, backward, g):
    """One projection at full size: x [rows,K] (row of sorted position i = a_row[i]), W [E,K,N], per-expert input
    range ir_e [E], upstream gradient gy (row of position i = g_row[i] // g_div), optional gate per destination row."""
    from analog_moe import ops, _cabi
    E, K, N = W.shape
    P = r.sel.numel()
    f32 = dtype == torch.float32
    prec = _cabi.PREC_SPLIT if f32 else _cabi.PREC_BF16X1
    tol = 1e-4 if f32 else 2.0 ** -7
    pw = ops.weight_prepass(W, prec)
    out, codes = ops.cvmm_fwd(x, a_row, dst_row, r.expert_offsets, pw, prec, P=P, dst_rows=P, ir=ir_e, ir_by_expert=True,
                              inp_res=RES, out_res=out_res, out_bound=OUT_BOUND, want_codes=True)
    # ---- forward on a sample of sorted positions
    ns = 256
    idx = torch.randperm(P, generator=g)[:ns]
    sel_c, arow_c, drow_c = r.sel.cpu().long(), a_row.cpu().long(), dst_row.cpu().long()
    e_of = sel_c[idx]
    xc, Wc, ir_c = x.float().cpu(), W.float().cpu(), ir_e.cpu()
    rows = xc[arow_c[idx]]
    a, _ = O.dac(rows, ir_c[e_of], None, RES)                     # quantised, normalised input (code * res)
    acc = torch.einsum("pk,pkn->pn", a.double(), Wc[e_of].double()).float()
    wmax = O.weight_max(Wc, True)[e_of]
    q, deq = O.adc_codes(acc, wmax, out_res, OUT_BOUND)
    got_q = codes.cpu()[drow_c[idx]].float()
    dq = (got_q - q).abs()
    assert float(dq.max()) <= 1.0, f"{name}/{tag}: ADC codes more than one apart"
    # where they differ the pre-rounding value sits next to a tie
    step = O.adc_step(out_res, OUT_BOUND)
    v = (acc / wmax).clamp(-OUT_BOUND, OUT_BOUND) / step
    frac = (v - torch.floor(v) - 0.5).abs()
    assert bool((frac[dq > 0] < 1e-2).all()), f"{name}/{tag}: code differs away from a rounding tie"
    ok = dq == 0
    assert float(ok.float().mean()) > 0.995
    want = deq * ir_c[e_of][:, None]
    got = out.float().cpu()[drow_c[idx]]
    if f32:
        assert torch.allclose(got[ok], want[ok], rtol=1e-5, atol=1e-6), f"{name}/{tag}: dequantised rows"
    else:
        w_b = want.to(torch.bfloat16).float()
        _close(torch.where(ok, got, w_b), w_b, tol, f"{name}/{tag}: forward rows", row_max=True)
    if not backward:
        return
    # ---- input gradient, clip mask, per-slot input-range gradient on the same sample
    rs = gate.reshape(-1) if gate is not None else None
    dx, ir_slot = ops.cvmm_dx(gy, g_row, dst_row, r.expert_offsets, pw, prec, P=P, dst_rows=P, a_row_div=g_div,
                              x_ref=x, x_ref_row=a_row, ir=ir_e, ir_by_expert=True, row_scale=rs, want_ir_grad=True,
                              relative=True, grad_scale=1.0)
    gc = gy.float().cpu()
    grow_c = g_row.cpu().long()
    g_rows = gc[grow_c[idx] // g_div]
    full = torch.einsum("pn,pkn->pk", g_rows.double(), Wc[e_of].double())
    if rs is not None:
        full = full * rs.cpu().double()[drow_c[idx]][:, None]
    irs = ir_c[e_of].double()[:, None]
    xr = rows.double()
    up, low, keep = xr >= irs, xr <= -irs, xr.abs() < irs
    want_ir = ((up * full).clamp(max=0).sum(-1) - (low * full).clamp(min=0).sum(-1)) * irs[:, 0]      # cvmm.py:863-870
    want_dx = (full * keep).float()
    got_dx = dx.float().cpu()[drow_c[idx]]
    if f32:
        _close(got_dx, want_dx, tol, f"{name}/{tag}: dX")
    else:
        _close(got_dx, want_dx.to(torch.bfloat16).float(), tol, f"{name}/{tag}: dX", row_max=True)
    _close(ir_slot.cpu()[idx], want_ir.float(), 1e-4 if f32 else 1e-3, f"{name}/{tag}: per-slot input-range gradient")
    # ---- weight gradient: three (expert, block) picks, every slot of the expert
    dw = ops.cvmm_dw(x, a_row, gy, g_row, r.expert_offsets, E, prec, P=P, ir=ir_e, ir_by_expert=True, g_div=g_div,
                     g_scale=rs).cpu()
    off = r.expert_offsets.cpu()
    cnt = off[1:] - off[:-1]
    picks = [int(cnt.argmax()), int(cnt.argmin()), int(torch.randint(0, E, (1,), generator=g))]
    for e in picks:
        lo, hi = int(off[e]), int(off[e + 1])
        k0 = int(torch.randint(0, max(K - 63, 1), (1,), generator=g))
        n0 = int(torch.randint(0, max(N - 63, 1), (1,), generator=g))
        if hi == lo:
            assert float(dw[e].abs().max()) == 0.0
            continue
        xe = xc[arow_c[lo:hi]][:, k0:k0 + 64].double().clamp(-float(ir_c[e]), float(ir_c[e]))
        ge = gc[grow_c[lo:hi] // g_div][:, n0:n0 + 64].double()
        if rs is not None:
            ge = ge * rs.cpu().double()[grow_c[lo:hi]][:, None]
        want_dw = xe.T @ ge
        scale = float(dw[e].abs().max())
        err = float((dw[e, k0:k0 + 64, n0:n0 + 64].double() - want_dw).abs().max())
        assert err <= (1e-4 if f32 else 2.0 ** -7) * scale, f"{name}/{tag}: dW[{e}] block err {err:.3e} vs scale {scale:.3g}"


@pytest.mark.parametrize("name", list(CONFIGS))
def test_config_shape_against_the_oracle_on_a_sample(name):
    from analog_moe import ops
    T, k, D, F, E, dtype, zipf, out_res, backward = CONFIGS[name]
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(17)
    logits = torch.randn(T, E, generator=g)
    if zipf:
        logits = logits - zipf * 1.6 * torch.log(torch.arange(1, E + 1).float())
    r = ops.select_sort(logits.to(dev), k)
    P = T * k
    mk = lambda *s, scale=1.0: (torch.randn(*s, generator=g) * scale).to(dev).to(dtype)
    x = mk(T, D)
    keys, values = mk(E, D, F, scale=D ** -0.5), mk(E, F, D, scale=F ** -0.5)
    ir = torch.stack([torch.linspace(2.0, 3.5, E), torch.linspace(1.0, 2.5, E)]).to(dev)
    # up-projection: rows by token, results by flat slot; upstream gradient per slot
    gh = mk(P, F)
    _projection_check(name, "up", dev, x, r.token_index, r.slot_index, r, keys, ir[0], gh, r.slot_index, 1, None, dtype,
                      out_res, backward, g)
    # down-projection: hidden rows by flat slot, upstream gradient per token (k slots share a row), gate per slot
    h = torch.relu(mk(P, F))
    gy = mk(T, D)
    gate = r.gate if dtype == torch.float32 else r.gate.to(dtype).float()
    _projection_check(name, "down", dev, h, r.slot_index, r.slot_index, r, values, ir[1], gy, r.slot_index, k, gate,
                      dtype, out_res, backward, g)


def test_output_noise_statistics_over_32_seeds():
    """Noise gate of the specification: over the seed sweep 0..31 the error the output noise adds has mean 0 and the
    configured standard deviation within 2 %.  Shapes of configuration 2's down-projection on one 128-row tile per
    expert and more (2048 slots, F = 128 -> D = 1024), split precision, 8-bit ADC off so that the error is the noise
    itself; the statistic is the reference test's (tests/test_moe_layer_aihwkit.py:112-177): the per-row standard
    deviation of (noisy - clean), averaged over rows, here normalised by out_noise * wmax[e, n] * ir."""
    from analog_moe import ops, _cabi
    dev = torch.device("cuda:0")
    T, k, D, F, E = 512, 4, 1024, 128, 16
    P = T * k
    g = torch.Generator().manual_seed(3)
    r = ops.select_sort(torch.randn(T, E, generator=g).to(dev), k)
    h = torch.relu(torch.randn(P, F, generator=g)).to(dev)
    W = (torch.randn(E, F, D, generator=g) / F ** 0.5).to(dev)
    ir = torch.full((E,), 3.0, device=dev)
    prec = _cabi.PREC_SPLIT
    pw = ops.weight_prepass(W, prec)
    std = 0.04
    kw = dict(P=P, dst_rows=P, ir=ir, ir_by_expert=True, inp_res=RES)
    clean, _ = ops.cvmm_fwd(h, r.slot_index, r.slot_index, r.expert_offsets, pw, prec, **kw)
    scale = (std * pw.col_scale[r.raw_sel.long().view(-1)] * 3.0)           # [P, D] by flat slot
    row_std, row_mean = [], []
    for seed in range(32):
        noisy, _ = ops.cvmm_fwd(h, r.slot_index, r.slot_index, r.expert_offsets, pw, prec, noise_std=std, seed=seed,
                                offset=1, **kw)
        z = (noisy - clean) / scale
        row_std.append(float(z.std(-1).mean()))
        row_mean.append(float(z.mean()))
    sweep_std = sum(row_std) / len(row_std)
    sweep_mean = sum(row_mean) / len(row_mean)
    assert abs(sweep_std - 1.0) <= 0.02, sweep_std
    assert abs(sweep_mean) <= 0.02, sweep_mean
    assert max(abs(s - 1.0) for s in row_std) <= 0.02          # every single seed as well
    assert len({round(s, 6) for s in row_std}) > 16             # the seeds really draw different noise
