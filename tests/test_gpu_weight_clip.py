"""Weight clipping (reference moe_layer_aihwkit_lightning.py:509-543, moe_layer_aihwkit.py:303-340) inside the weight
pre-pass kernels, against the reference's torch formulas: clamp to +-sigma * std per expert (LAYER_GAUSSIAN), per
column (LAYER_GAUSSIAN_PER_CHANNEL), capped by or equal to a fixed value (classic flavour).  torch.std is the
unbiased sample standard deviation; the kernels accumulate sums and sums of squares in fp64, so the bound - and with it
every clamped element - agrees to fp32 rounding."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(got, want, what, tol=2e-6):
    # the bound itself agrees with torch's to an ulp or two (fp64 sums here, fp32 there), and with it every clamped element
    # (bf16 weights: the clamped value is rounded to bf16, so an ulp of the bound can become a bf16 ulp)
    diff = (got - want).abs()
    assert float(diff.max()) <= tol * float(want.abs().max()), what


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clip_against_the_reference_formulas(dtype):
    from analog_moe import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(2)
    E, K, N = 5, 200, 136
    w0 = (torch.randn(E, K, N, generator=g) * torch.linspace(0.5, 2.0, E).view(E, 1, 1)).to(dev).to(dtype)
    sigma = 1.7
    tol = 2e-6 if dtype == torch.float32 else 2.0 ** -7
    # per expert
    w = w0.clone()
    ops.clip_weights_(w, sigma=sigma)
    b = sigma * w0.float().std((1, 2), keepdim=True)
    _check(w.float(), w0.float().clamp(-b, b).to(dtype).float(), "LAYER_GAUSSIAN", tol)
    assert float((w != w0).float().mean()) > 0.05            # something was clipped
    # per column
    w = w0.clone()
    ops.clip_weights_(w, sigma=sigma, per_channel=True)
    b = sigma * w0.float().std(1, keepdim=True)
    _check(w.float(), w0.float().clamp(-b, b).to(dtype).float(), "LAYER_GAUSSIAN_PER_CHANNEL", tol)
    # fixed value, and sigma capped by a fixed value (classic flavour)
    w = w0.clone()
    ops.clip_weights_(w, fixed_value=0.8)
    _check(w.float(), w0.float().clamp(-0.8, 0.8), "FIXED_VALUE", tol)
    w = w0.clone()
    ops.clip_weights_(w, sigma=sigma, fixed_value=1.1)
    b = (sigma * w0.float().std((1, 2), keepdim=True)).clamp(max=1.1)
    _check(w.float(), w0.float().clamp(-b, b).to(dtype).float(), "LAYER_GAUSSIAN capped", tol)


def test_clip_fused_into_the_weight_prepass_and_the_layer_hook():
    """The same clamp as part of the pre-pass that prepares the weights for the next forward pass: the weight tensor
    is clamped in place and the prepared copies are those of the clamped weights; `post_update_step` of a layer with
    a clip type set does it for keys and values."""
    from analog_moe import ops, _cabi, AnalogSigmaMoELayer, TorchInferenceRPUConfig, WeightClipType
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(3)
    E, K, N = 4, 128, 64
    w0 = torch.randn(E, K, N, generator=g).to(dev)
    w = w0.clone()
    pw = ops.weight_prepass(w, _cabi.PREC_SPLIT, clip_sigma=2.0)
    b = 2.0 * w0.std((1, 2), keepdim=True)
    want = w0.clamp(-b, b)
    _check(w, want, "in-place clamp by the pre-pass")
    ref = ops.weight_prepass(want.contiguous(), _cabi.PREC_SPLIT)
    assert torch.equal(pw.fwd_hi, ref.fwd_hi) or float((pw.fwd_hi.float() - ref.fwd_hi.float()).abs().max()) < 1e-2
    assert torch.allclose(pw.col_scale, ref.col_scale, rtol=1e-6)
    cfg = TorchInferenceRPUConfig()
    cfg.clip.type, cfg.clip.sigma = WeightClipType.LAYER_GAUSSIAN, 1.5
    torch.manual_seed(0)
    layer = AnalogSigmaMoELayer(cfg, d_model=64, n_experts=4, expert_size=64, k=2).to(dev).train()
    k0, v0 = layer.keys.data.clone(), layer.values.data.clone()
    layer.post_update_step()
    x = torch.randn(1, 64, 64, device=dev)
    layer(x)                                   # a pending clip runs with the next forward's weight pre-pass
    for got, w_ in ((layer.keys.data, k0), (layer.values.data, v0)):
        bb = 1.5 * w_.std((1, 2), keepdim=True)
        _check(got, w_.clamp(-bb, bb), "post_update_step")
