"""The CPU oracle against golden vectors produced by the reference's own
CVMM.apply / cvmm_std (see tests/golden/make_golden.py)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import cvmm_oracle as O

LAYER_CASES = ["ref_test_shape_ir_fp", "ref_test_shape_absmax_fp", "small_ir_quant", "small_ir_quant_decay",
               "small_absmax_quant", "small_ir_quant_noise", "ragged_zipf_empty", "config1"]


def load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return {k: (torch.from_numpy(z[k]) if z[k].ndim else z[k].item()) for k in z.files}


def run_oracle_layer(c, acc_dtype=torch.float64):
    T, k, E = c["T"], c["k"], c["E"]
    sel, perm = c["sel"].long(), c["perm"].long()
    use_ir = bool(c["use_ir"])
    ir_up = c["input_range"][0][sel] if use_ir else None
    ir_dn = c["input_range"][1][sel] if use_ir else None
    irp = O.IRParams(enable=use_ir, decay=float(c["decay"]))
    x = c["x"]
    am_up = None if use_ir else x.abs().amax(-1)
    h_pre = O.cvmm_forward(x, perm // k, sel, c["keys"], c["inp_res"], ir_up, perm, am_up,
                           c.get("noise_up"), None, acc_dtype)
    h = torch.relu(h_pre)
    am_dn = None if use_ir else h.abs().amax(-1)
    res = O.cvmm_forward(h, perm, sel, c["values"], c["inp_res"], ir_dn, None, am_dn,
                         c.get("noise_dn"), None, acc_dtype)
    y = O.combine(res, c["gate"])
    dh, dV, dir_dn, dgate = O.cvmm_backward(c["grad_y"], h, perm, sel, c["values"], ir_dn, None, c["gate"], res,
                                            irp, acc_dtype)
    dh_pre = dh * (h_pre > 0).float()
    dx, dK, dir_up, _ = O.cvmm_backward(dh_pre, x, perm // k, sel, c["keys"], ir_up, perm, None, None, irp, acc_dtype)
    out = dict(h_pre=h_pre, y=y, dh=dh, dh_pre=dh_pre, dx=dx, dkeys=dK, dvalues=dV, dgate=dgate)
    if use_ir:
        d = torch.zeros(2, E)
        d[0].index_add_(0, sel, dir_up)
        d[1].index_add_(0, sel, dir_dn)
        out["d_input_range"] = d
    return out


@pytest.mark.parametrize("name", LAYER_CASES)
def test_layer_cases(golden_dir, name):
    c = load(golden_dir, name)
    got = run_oracle_layer(c)
    for key, val in got.items():
        ref = c[key]
        scale = max(1.0, float(ref.abs().max()))
        err = float((val.reshape(ref.shape) - ref).abs().max())
        # fp32 accumulation-order noise of the reference's tiled FMA vs the oracle's fp64 accumulate
        assert err <= 2e-5 * scale, f"{name}:{key} max err {err} (scale {scale})"


def test_dac_codes_are_integers_and_bitexact(golden_dir):
    c = load(golden_dir, "small_ir_quant")
    sel, perm, k = c["sel"].long(), c["perm"].long(), c["k"]
    rows = c["x"][perm // k]
    a, codes = O.dac(rows, c["input_range"][0][sel], None, c["inp_res"])
    assert torch.equal(codes, torch.round(codes))
    assert codes.abs().max() <= 127
    assert torch.equal(a, codes * torch.tensor(c["inp_res"], dtype=torch.float32))


def test_expert_std(golden_dir):
    c = load(golden_dir, "expert_std")
    k = c["k"]
    sel, perm = c["sel"].long(), c["perm"].long()
    up = O.expert_std(c["x"], perm // k, sel, c["E"])
    dn = O.expert_std(c["xs"], perm, sel, c["E"])
    assert torch.allclose(up, c["std_up"], rtol=2e-5, atol=0)
    assert torch.allclose(dn, c["std_dn"], rtol=2e-5, atol=0)


def test_select_sort_matches_torch_topk():
    torch.manual_seed(3)
    logits = torch.randn(257, 16)
    s = O.select_sort(logits, 4)
    val, idx = torch.sigmoid(logits).topk(4, dim=-1)
    assert torch.equal(s.raw_sel.long(), idx)
    assert torch.equal(s.gate, val)
    assert torch.equal(s.sel.long(), torch.sort(idx.flatten(), stable=True)[0])
    assert torch.equal(s.slot_index.long() // 4, s.token_index.long())
    assert int(s.expert_offsets[-1]) == 257 * 4


def test_philox_known_answer():
    # Random123 known-answer vectors for philox4x32-10
    out = O.philox4x32_10(0, 0, 0, 0, 0, 0)
    assert [int(v) for v in out] == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    out = O.philox4x32_10(0xffffffff, 0xffffffff, 0xffffffff, 0xffffffff, 0xffffffff, 0xffffffff)
    assert [int(v) for v in out] == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    out = O.philox4x32_10(0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344, 0xa4093822, 0x299f31d0)
    assert [int(v) for v in out] == [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_box_muller_extreme_words_are_finite():
    for a in (0, 0xFFFFFFFF, 0x80000000):
        for b in (0, 0xFFFFFFFF):
            z0, z1 = O._box_muller(np.array([a], dtype=np.uint32), np.array([b], dtype=np.uint32))
            assert np.isfinite(z0).all() and np.isfinite(z1).all()
            assert abs(float(z0[0])) < 6.0 and abs(float(z1[0])) < 6.0


def test_output_noise_generator_moments_and_range():
    """Eight normals per Philox call from 16-bit uniforms: moments of a standard normal, |z| bounded by
    sqrt(2 ln 2^17), finite for every word."""
    z = O.philox_normal8(1234, 0, O.STREAM_OUT_NOISE, 2048, 256)
    assert abs(float(z.mean())) < 5e-3
    assert abs(float(z.std()) - 1.0) < 5e-3
    assert abs(float((z ** 4).mean()) - 3.0) < 5e-2
    assert float(z.abs().max()) <= (2 * np.log(2.0 ** 17)) ** 0.5 + 1e-3
    for w in (0, 0xFFFFFFFF, 0x0000FFFF, 0xFFFF0000):
        z0, z1 = O._box_muller16(np.array([w], dtype=np.uint32))
        assert np.isfinite(z0).all() and np.isfinite(z1).all()
    # columns 0..7 of a row come from one counter, column 8 from the next
    a = O.philox_normal8(7, 1, O.STREAM_OUT_NOISE, 4, 16)
    b = O.philox_normal8(7, 1, O.STREAM_OUT_NOISE, 4, 9)
    assert torch.equal(a[:, :9], b)


def test_philox_normal_moments():
    z = O.philox_normal(1234, 0, O.STREAM_OUT_NOISE, 2048, 256)
    assert abs(float(z.mean())) < 5e-3
    assert abs(float(z.std()) - 1.0) < 5e-3
    assert abs(float((z ** 4).mean()) - 3.0) < 5e-2
