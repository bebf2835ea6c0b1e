"""Generate the golden vectors under tests/golden/ from the reference implementation.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's `analog_moe/triton_src/cvmm.py` by file path and runs
its own `CVMM.apply` (forward and backward) and `cvmm_std` on CPU tensors with
Triton's interpreter (`TRITON_INTERPRET=1`).  Three shims are applied from the
outside, none of which changes the reference's arithmetic:

* `Tensor.cuda()` returns the tensor itself (the reference hard-codes `.cuda()`
  for its `-1` sentinels);
* the autotuned kernels are launched through their undecorated `.fn` with one
  fixed tile configuration (the autotuner needs a GPU driver);
* `libdevice.rint` is given an interpreter implementation (`numpy.rint`, i.e.
  round half to even, the same function).

The outputs are stored as compressed `.npz` files together with the inputs, so
the tests need neither the reference nor Triton.
"""
import importlib.util
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton.language as tl  # noqa: E402
from triton.runtime.interpreter import TensorHandle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    spec = importlib.util.spec_from_file_location(
        "ref_cvmm", os.path.join(root, "analog_moe", "triton_src", "cvmm.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    torch.Tensor.cuda = lambda self, *a, **k: self

    def _rint(x, _semantic=None, _builder=None):
        return tl.tensor(TensorHandle(np.rint(x.handle.data), x.handle.dtype), x.type)
    tl.extra.cuda.libdevice.rint = _rint

    class Fixed:
        def __init__(self, auto, **meta):
            self.fn, self.meta = auto.fn, meta

        def __getitem__(self, grid):
            def launch(*args, **kw):
                kw = dict(kw)
                kw.update(self.meta)
                g = grid(self.meta) if callable(grid) else grid
                return self.fn[g](*args, **kw)
            return launch

    mod.cvmm_kernel = Fixed(mod.cvmm_kernel, BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, BLOCK_SIZE_K=32, GROUP_SIZE_M=8)
    mod.cvmm_backward_kernel3 = Fixed(mod.cvmm_backward_kernel3, BLOCK_SIZE_M=32, BLOCK_SIZE_N=32,
                                      BLOCK_SIZE_K=16, GROUP_SIZE_M=8, K_BLOCKS=4)
    mod.cvmm_mean_kernel = Fixed(mod.cvmm_mean_kernel, BLOCK_SIZE_M=32)
    # One column block covers the row, so the reference's repeated-work grid factor is 1.
    mod.cvmm_center_and_square_kernel = Fixed(mod.cvmm_center_and_square_kernel, BLOCK_SIZE_M=32, BLOCK_SIZE_N=512)
    return mod


class IR:
    def __init__(self, enable=True, decay=0.0, input_min_percentage=0.95):
        self.enable, self.decay, self.input_min_percentage = enable, decay, input_min_percentage


class IO:
    pass


def routing(T, E, k, seed, zipf=False):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    if zipf:
        logits = logits - 1.5 * torch.log(torch.arange(1, E + 1).float())
    gate, idx = torch.sigmoid(logits).topk(k, dim=-1)
    ssel, perm = torch.sort(idx.flatten(), stable=True)
    return gate, idx.int(), ssel.int(), perm


def layer_case(ref, name, T, k, D, F, E, inp_res, use_ir, seed, decay=0.0, noise=0.0, zipf=False,
               ir_values=None, empty_expert=False):
    """Two CVMM.apply calls with a ReLU in between (the layer's hot path), forward + backward."""
    g = torch.Generator().manual_seed(seed + 1000)
    gate, raw_sel, ssel, perm = routing(T, E, k, seed, zipf)
    if empty_expert:
        # route everything that went to expert 1 to expert 0 instead
        raw_sel = torch.where(raw_sel == 1, torch.zeros_like(raw_sel), raw_sel)
        ssel, perm = torch.sort(raw_sel.flatten().long(), stable=True)
        ssel = ssel.int()
    x = torch.randn(1, T, D, generator=g).requires_grad_()
    keys = (torch.randn(E, D, F, generator=g) / D ** 0.5).requires_grad_()
    values = (torch.randn(E, F, D, generator=g) / F ** 0.5).requires_grad_()
    gate = gate.clone().view(1, T, k).requires_grad_()
    grad_y = torch.randn(1, T, D, generator=g)
    if ir_values is None:
        ir_values = torch.stack([torch.linspace(1.0, 2.5, E), torch.linspace(0.8, 2.0, E)])
    input_range = ir_values.clone().requires_grad_()
    sel3 = ssel.view(1, T, k)
    ir_p = IR(enable=use_ir, decay=decay)
    n_up = n_dn = None
    if noise > 0:
        n_up = torch.randn(1, T, k, F, generator=g) * noise
        n_dn = torch.randn(1, T, k, D, generator=g) * noise
    bir_up = input_range[0][sel3.long()] if use_ir else None
    bir_dn = input_range[1][sel3.long()] if use_ir else None
    h_pre = ref.CVMM.apply(x, perm // k, sel3, keys, inp_res, bir_up, perm, None, n_up, ir_p, IO())
    h_pre.retain_grad()
    h = torch.relu(h_pre)
    h.retain_grad()
    y = ref.CVMM.apply(h, perm, sel3, values, inp_res, bir_dn, None, gate, n_dn, ir_p, IO())
    (y * grad_y).sum().backward()
    out = dict(
        T=T, k=k, D=D, F=F, E=E, inp_res=inp_res, use_ir=int(use_ir), decay=decay,
        x=x.detach()[0], keys=keys.detach(), values=values.detach(), gate=gate.detach()[0],
        raw_sel=raw_sel, sel=ssel, perm=perm.int(), grad_y=grad_y[0], input_range=ir_values,
        h_pre=h_pre.detach()[0], y=y.detach()[0], dh=h.grad[0], dh_pre=h_pre.grad[0],
        dx=x.grad[0], dkeys=keys.grad, dvalues=values.grad, dgate=gate.grad[0],
    )
    if use_ir:
        out["d_input_range"] = input_range.grad
    if noise > 0:
        out["noise_up"], out["noise_dn"] = n_up[0], n_dn[0]
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        **{k_: (v.numpy() if torch.is_tensor(v) else np.asarray(v)) for k_, v in out.items()})
    print(name, "y", float(y.abs().mean()), "dx", float(x.grad.abs().mean()))


def std_case(ref, name, T, k, D, E, seed):
    g = torch.Generator().manual_seed(seed)
    _, raw_sel, ssel, perm = routing(T, E, k, seed)
    x = torch.randn(T, D, generator=g) * torch.linspace(0.5, 2.0, T).view(-1, 1) + 0.1
    std_up = ref.cvmm_std(x, perm // k, ssel, E)
    xs = torch.randn(T * k, D, generator=g)
    std_dn = ref.cvmm_std(xs, perm, ssel, E)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), T=T, k=k, D=D, E=E, x=x.numpy(), xs=xs.numpy(),
                        sel=ssel.numpy(), perm=perm.int().numpy(), std_up=std_up.numpy(), std_dn=std_dn.numpy())
    print(name, std_up)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference>")
    ref = load_reference(sys.argv[1])
    q = 2.0 / 254.0
    # reference-test shape (tests/test_moe_layer_aihwkit.py:211-216) with input ranges 1+e (:248-263)
    ir_1pe = torch.stack([torch.arange(1.0, 5.0), torch.arange(1.0, 5.0)])
    layer_case(ref, "ref_test_shape_ir_fp", 100, 2, 128, 64, 4, -1, True, seed=0, ir_values=ir_1pe)
    layer_case(ref, "ref_test_shape_absmax_fp", 100, 2, 128, 64, 4, -1, False, seed=0)
    layer_case(ref, "small_ir_quant", 96, 2, 64, 32, 4, q, True, seed=1)
    layer_case(ref, "small_ir_quant_decay", 96, 2, 64, 32, 4, q, True, seed=2, decay=0.01,
               ir_values=torch.full((2, 4), 3.5))
    layer_case(ref, "small_absmax_quant", 80, 3, 48, 40, 5, q, False, seed=3)
    layer_case(ref, "small_ir_quant_noise", 64, 2, 64, 32, 4, q, True, seed=4, noise=0.05)
    layer_case(ref, "ragged_zipf_empty", 77, 3, 40, 24, 6, q, True, seed=5, zipf=True, empty_expert=True)
    # benchmark config 1: d_model=256, E=8, F=64, k=2, 512 tokens, 8-bit DAC, input range 3.0
    layer_case(ref, "config1", 512, 2, 256, 64, 8, q, True, seed=0, ir_values=torch.full((2, 8), 3.0))
    std_case(ref, "expert_std", 120, 2, 96, 5, seed=7)


if __name__ == "__main__":
    main()
