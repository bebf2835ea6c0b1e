"""The reference's own Triton kernels on the same GPU, beside the CUDA library.

baseline/_ref holds the reference package as pip installed it; its `analog_moe/triton_src/cvmm.py` is imported by
path (it needs none of the third-party packages).  Two checks:

* integer DAC codes.  With identity weights the output of a quantising forward is `code * res * ir`, so the codes both
  implementations form are observable exactly.  The reference's GPU build divides with the approximate `div.full.f32`,
  this library with IEEE-exact quotients, so they may differ on inputs whose quotient sits within a few ulp of a
  rounding tie - and nowhere else.  The test counts the differences inside and outside that near-tie set and asserts
  zero outside.
* forward + backward of the two chained CVMM calls (fp32, quantised, input ranges) against the reference's result on
  the GPU, at the reference's own test tolerances.
"""
import importlib.util
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_CVMM = os.path.join(ROOT, "baseline", "_ref", "analog_moe", "triton_src", "cvmm.py")


def load_reference_cvmm():
    name = "_reference_triton_cvmm"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, REF_CVMM)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


needs_ref = pytest.mark.skipif(not os.path.exists(REF_CVMM), reason="baseline/_ref is not installed")


class IR:
    def __init__(self, enable=True, decay=0.0, input_min_percentage=0.95):
        self.enable, self.decay, self.input_min_percentage = enable, decay, input_min_percentage


class IO:
    pass


@needs_ref
def test_dac_codes_against_the_reference_triton_kernel():
    from analog_moe import CVMM, CVMMExt, ops, _cabi
    ref = load_reference_cvmm()
    dev = torch.device("cuda:0")
    T, k, K, E = 4096, 2, 128, 8
    res = 2.0 / 254.0
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(1, T, K, generator=g) * 1.3).to(dev)
    # some inputs exactly on rounding ties of the first expert's grid, to make the near-tie set non-empty
    ir_vals = torch.linspace(0.75, 3.0, E)
    x[0, :64, :] = ((torch.arange(64 * K).view(64, K) % 250 - 125).float() + 0.5).to(dev) * res * float(ir_vals[0])
    r = ops.select_sort(torch.randn(T, E, generator=g).to(dev), k)
    sel3 = r.sel.view(1, T, k).long()
    eye = torch.eye(K, device=dev).repeat(E, 1, 1).contiguous()
    bir = ir_vals.to(dev)[sel3]
    tok, slot = r.token_index.long(), r.slot_index.long()
    with torch.no_grad():
        theirs = ref.CVMM.apply(x, tok, sel3, eye, res, bir, slot, None, None, IR(), IO())
        codes = {}
        for name, prec in (("split", _cabi.PREC_SPLIT), ("simt", _cabi.PREC_FP32_SIMT)):
            mine = CVMM.apply(x, tok, sel3, eye, res, bir, slot, None, None, IR(), IO(), CVMMExt(precision=prec))
            codes[name] = mine
    torch.cuda.synchronize()
    # decode: out[slot, j] = code * res * ir(slot)
    scale = (res * ir_vals.to(dev)[r.raw_sel.long()]).view(1, T, k, 1)      # out rows are flat slots (token, j)
    dec = lambda o: torch.round(o / scale).to(torch.int32)
    c_ref = dec(theirs)
    assert float((theirs / scale - c_ref).abs().max()) < 1e-3          # the decode is unambiguous
    # near-tie set, from an fp64 evaluation of the quotient
    xs = x[0].double()[:, None, :].expand(T, k, K)
    irs = ir_vals.double().to(dev)[r.raw_sel.long()].view(T, k, 1)
    q = (xs.clamp(-irs, irs) / irs) / res
    near = ((q - torch.floor(q)) - 0.5).abs() < 1e-4
    for name, mine in codes.items():
        c = dec(mine)
        diff = (c != c_ref).view(T, k, K)
        inside = int((diff & near).sum())
        outside = int((diff & ~near).sum())
        print(f"DAC codes vs reference Triton kernel [{name}]: {int(diff.sum())} of {diff.numel()} differ "
              f"({inside} within 1e-4 of a rounding tie, {outside} elsewhere; near-tie set holds {int(near.sum())})")
        assert outside == 0
        assert int((c - c_ref).abs().max()) <= 1


@needs_ref
def test_layer_path_against_the_reference_on_the_gpu():
    """Two chained CVMM.apply calls with a ReLU, forward + backward, fp32: this library (split precision and CUDA-core
    fp32) against the reference's Triton kernels run right here.  Tolerances are the reference's own
    (tests/test_moe_layer_aihwkit.py:267-306): 1e-4 forward / dW / dIR, 1e-3 dX, of the scale.  The up-projection and
    the down-projection are compared call by call on the reference's intermediate tensor: a 1e-6 difference in a hidden
    activation that sits on a DAC rounding tie becomes a whole quantisation step downstream."""
    from analog_moe import CVMM, CVMMExt, ops, _cabi
    ref = load_reference_cvmm()
    dev = torch.device("cuda:0")
    T, k, D, F, E = 1024, 4, 256, 128, 8
    res = 2.0 / 254.0
    g = torch.Generator().manual_seed(5)
    mk = lambda *s, scale=1.0: (torch.randn(*s, generator=g) * scale).to(dev)
    x0, keys0, values0 = mk(1, T, D), mk(E, D, F, scale=D ** -0.5), mk(E, F, D, scale=F ** -0.5)
    gy = mk(1, T, D)
    r = ops.select_sort(mk(T, E), k)
    sel3 = r.sel.view(1, T, k).long()
    gate0 = r.gate.view(1, T, k)
    ir0 = torch.stack([torch.linspace(1.0, 2.5, E), torch.linspace(0.8, 2.0, E)]).to(dev)
    tok, slot = r.token_index.long(), r.slot_index.long()
    irp = IR(True, decay=0.01)

    def run(apply, ext, h_in=None):
        x, keys, values = x0.clone().requires_grad_(), keys0.clone().requires_grad_(), values0.clone().requires_grad_()
        gate, ir = gate0.clone().requires_grad_(), ir0.clone().requires_grad_()
        e = (ext,) if ext is not None else ()
        h_pre = apply(x, tok, sel3, keys, res, ir[0][sel3], slot, None, None, irp, IO(), *e)
        h = torch.relu(h_pre) if h_in is None else h_in.clone().requires_grad_()
        y = apply(h, slot, sel3, values, res, ir[1][sel3], None, gate, None, irp, IO(), *e)
        if h_in is None:
            (y * gy).sum().backward()
            return dict(h=h.detach(), y=y.detach(), dx=x.grad, dkeys=keys.grad, dvalues=values.grad, dgate=gate.grad,
                        dir=ir.grad)
        # second call on a given hidden tensor: its own gradients only
        y.backward(gy)
        return dict(y=y.detach(), dh=h.grad, dvalues=values.grad, dgate=gate.grad, dir_dn=ir.grad[1])

    def run_up(apply, ext, grad_h):
        x, keys, ir = x0.clone().requires_grad_(), keys0.clone().requires_grad_(), ir0.clone().requires_grad_()
        e = (ext,) if ext is not None else ()
        h_pre = apply(x, tok, sel3, keys, res, ir[0][sel3], slot, None, None, irp, IO(), *e)
        h_pre.backward(grad_h)
        return dict(dx=x.grad, dkeys=keys.grad, dir_up=ir.grad[0])

    want = run(ref.CVMM.apply, None)
    want_dn = run(ref.CVMM.apply, None, h_in=want["h"])
    grad_h = want_dn["dh"] * (want["h"] > 0).float()
    want_up = run_up(ref.CVMM.apply, None, grad_h)
    torch.cuda.synchronize()

    def close(a, b, tol, what):
        # The reference's GPU build rounds a few near-tie inputs to the neighbouring DAC code (approximate division,
        # counted in the test above); each such input moves the outputs it feeds by one quantisation step times a
        # weight.  So: all but a thousandth of the elements within `tol`, and nothing further off than 5e-3.
        scale = max(1.0, float(b.abs().max()))
        err = (a - b).abs() / scale
        frac = float((err > tol).float().mean())
        assert frac <= 1e-3, f"{what}: {frac:.2e} of the elements differ by more than {tol:g} of the scale"
        assert float(err.max()) <= 5e-3, f"{what}: max {float(err.max()):.3e} of the scale"

    for name, prec in (("split", _cabi.PREC_SPLIT), ("simt", _cabi.PREC_FP32_SIMT)):
        ext = CVMMExt(precision=prec)
        got = run(CVMM.apply, ext)
        close(got["h"], want["h"], 1e-4, f"{name}: hidden")
        got_dn = run(CVMM.apply, ext, h_in=want["h"])
        close(got_dn["y"], want_dn["y"], 1e-4, f"{name}: y")
        close(got_dn["dh"], want_dn["dh"], 1e-3, f"{name}: dh")
        close(got_dn["dvalues"], want_dn["dvalues"], 1e-4, f"{name}: dvalues")
        close(got_dn["dgate"], want_dn["dgate"], 1e-4, f"{name}: dgate")
        close(got_dn["dir_dn"], want_dn["dir_dn"], 1e-4, f"{name}: d_input_range[1]")
        got_up = run_up(CVMM.apply, ext, grad_h)
        close(got_up["dx"], want_up["dx"], 1e-3, f"{name}: dx")
        close(got_up["dkeys"], want_up["dkeys"], 1e-4, f"{name}: dkeys")
        close(got_up["dir_up"], want_up["dir_up"], 1e-4, f"{name}: d_input_range[0]")
