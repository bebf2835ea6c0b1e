"""Routers too large for the shared-memory kernels (E * D * 4 bytes > 200 KiB: the benchmark configurations 3 and 5) run
their matmul and their weight gradient as one-expert CVMM calls on the tensor cores.  Checked against torch in fp64:
fp32 routers to 2e-5 of the result's scale (bf16 hi + lo terms), bf16 routers to the bf16 rounding of the result."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("E,D,dtype", [(64, 2048, torch.float32), (48, 1536, torch.bfloat16), (48, 1536, torch.float32)])
def test_large_router_forward_and_weight_gradient(E, D, dtype):
    from analog_moe import ops
    dev = torch.device("cuda:0")
    assert not ops._router_fits_smem(E, D)
    T, k = 3000, 4
    g = torch.Generator().manual_seed(4)
    x = torch.randn(T, D, generator=g).to(dev).to(dtype)
    w = (torch.randn(E, D, generator=g) / D ** 0.5).to(dev).to(dtype)
    assert ops._router_on_tensor_cores(x, w)
    logits = ops.router_logits(x, w)
    want = x.double() @ w.double().t()
    scale = float(want.abs().max())
    if dtype == torch.float32:
        assert float((logits.double() - want).abs().max()) <= 2e-5 * scale
    else:
        assert float((logits.double() - want.to(torch.bfloat16).double()).abs().max()) <= 2.0 ** -7 * scale
    # the routing built on those logits: select + sort as one call, every index in range, offsets consistent
    r, lg = ops.router_select(x, w, k)
    assert lg is not None and int(r.expert_offsets[-1]) == T * k
    # weight gradient: dlogits has k non-zeros per row
    dgate = torch.randn(T, k, generator=g).to(dev)
    dw = ops.router_backward_w(x, dgate, r.gate, r.token_index, r.slot_index, r.expert_offsets, E, raw_sel=r.raw_sel)
    dl = torch.zeros(T, E, dtype=torch.float64, device=dev)
    gt = r.gate.double()
    dl.scatter_(1, r.raw_sel.long(), dgate.double() * gt * (1.0 - gt))
    want_dw = dl.t() @ x.double()
    tol = 2e-5 if dtype == torch.float32 else 2.0 ** -7
    assert dw.shape == (E, D)
    assert float((dw.double() - want_dw).abs().max()) <= tol * float(want_dw.abs().max())
