"""The allocation-free entry point amoe_expert_std_static against amoe_expert_std.

Some hosts cannot call cudaMalloc once they are up (all device memory belongs to their own arena,
or they sit on a path where an allocation's device-wide synchronisation is not allowed), so they
cannot lend the library a workspace.  This entry point keeps its accumulators in an array inside
the library image instead.  The test calls both entry points through the C ABI on the same inputs,
twice in a row with different data (the second call finds the first call's sums in the array and
must clear them), and expects the same numbers from both, to the tolerance the regular
per-expert-std test uses (relative 2e-5).  Collected last so that a failure here cannot mask
another test under `-x`.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, x, x_row, off, E, use_static):
    P, K = x_row.numel(), x.shape[1]
    out = torch.full((E,), -1.0, dtype=torch.float32, device=x.device)
    stream = torch.cuda.current_stream().cuda_stream
    if use_static:
        rc = lib.amoe_expert_std_static(x.data_ptr(), 0, x.stride(0), K, x.shape[0], x_row.data_ptr(), off.data_ptr(),
                                        P, E, out.data_ptr(), None, stream)
    else:
        nbytes = lib.amoe_expert_std_workspace_bytes(E)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        rc = lib.amoe_expert_std(x.data_ptr(), 0, x.stride(0), K, x.shape[0], x_row.data_ptr(), off.data_ptr(), P, E,
                                 out.data_ptr(), ws.data_ptr(), nbytes, None, stream)
    assert rc == 0, lib.amoe_status_string(rc)
    torch.cuda.synchronize()
    return out.cpu()


def test_static_scratch_entry_point_matches_workspace_entry_point():
    from analog_moe import _cabi, ops
    lib = _cabi.lib
    dev = torch.device("cuda:0")
    E, k = 7, 2
    for call, (T, K, seed) in enumerate([(300, 96, 1), (190, 64, 2)]):
        g = torch.Generator().manual_seed(seed)
        x = (torch.randn(T, K, generator=g) * (1 + call) + 0.25).to(dev)
        logits = torch.randn(T, E, generator=g)
        logits[:, 3] = -40.0                      # one expert without rows: NaN from both entry points
        r = ops.select_sort(logits.to(dev), k)
        want = _both(lib, x, r.token_index, r.expert_offsets, E, use_static=False)
        got = _both(lib, x, r.token_index, r.expert_offsets, E, use_static=True)
        assert torch.isnan(want[3]) and torch.isnan(got[3])
        ok = ~torch.isnan(want)
        assert torch.allclose(got[ok], want[ok], rtol=2e-5, atol=0), (call, got, want)


def test_static_scratch_entry_point_rejects_too_many_experts():
    from analog_moe import _cabi
    lib = _cabi.lib
    dev = torch.device("cuda:0")
    x = torch.zeros(4, 8, device=dev)
    idx = torch.zeros(4, dtype=torch.int32, device=dev)
    off = torch.zeros(5000, dtype=torch.int32, device=dev)
    out = torch.zeros(5000, device=dev)
    rc = lib.amoe_expert_std_static(x.data_ptr(), 0, 8, 8, 4, idx.data_ptr(), off.data_ptr(), 4, 4097, out.data_ptr(), None,
                                    None)
    assert rc == 1
    assert b"4096" in lib.amoe_last_error_string()
