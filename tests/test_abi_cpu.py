"""CPU-side checks of the boundary: the library loads without a GPU driver, exports every symbol
the header declares, and the host-side argument validation answers without touching a device."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "amoe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(amoe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from analog_moe import _cabi
    syms = header_symbols()
    assert len(syms) >= 20
    for s in syms:
        assert hasattr(_cabi.lib, s), f"{s} declared in include/amoe.h but not exported"
        assert s in _cabi.SIGNATURES, f"{s} has no ctypes signature"
    assert set(_cabi.SIGNATURES) == set(syms)


def test_status_strings_and_version():
    from analog_moe import _cabi
    assert _cabi.lib.amoe_version() >= 100
    assert _cabi.lib.amoe_status_string(0) == b"ok"
    for code in range(1, 10):
        assert _cabi.lib.amoe_status_string(code) not in (b"ok", b"unknown status")


def test_struct_layout_matches_header():
    """Field order of the ctypes structures follows the C structs (names, in order)."""
    from analog_moe import _cabi
    text = open(os.path.join(ROOT, "include", "amoe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for cname, cls in (("amoe_cvmm_args", _cabi.CvmmArgs), ("amoe_dw_args", _cabi.DwArgs),
                       ("amoe_weight_prepass_args", _cabi.WeightPrepassArgs)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), text, flags=re.S).group(1)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            parts = decl.split(",")
            names.append(re.findall(r"(\w+)\s*$", parts[0].strip())[0])
            names += [p.strip().lstrip("*") for p in parts[1:]]
        assert names == [f[0] for f in cls._fields_], cname


def test_host_validation_without_gpu():
    from analog_moe import _cabi
    lib = _cabi.lib
    assert lib.amoe_select_sort(None, 0, 4, 2, 1, None, None, None, None, None, None, None, 0, None) == 1
    assert lib.amoe_select_sort(None, 8, 4, 2, 1, None, None, None, None, None, None, None, 0, None) == 3
    assert lib.amoe_select_sort(None, 8, 4, 8, 1, None, None, None, None, None, None, None, 0, None) == 1  # k > E
    a = _cabi.CvmmArgs()
    assert lib.amoe_cvmm_fwd(ctypes.byref(a), None) == 1
    a.P, a.E, a.K, a.N = 16, 2, 8, 8
    assert lib.amoe_cvmm_fwd(ctypes.byref(a), None) == 3
    d = _cabi.DwArgs()
    assert lib.amoe_cvmm_dw(ctypes.byref(d), None) == 1
    assert lib.amoe_select_sort_workspace_bytes(1024, 16, 4) == (16 * 16 + 16) * 4   # 16 chunks of 256 slots x 16 experts + totals
    assert lib.amoe_expert_std_workspace_bytes(8) == 8 * 3 * 8


def test_cpu_tensors_are_refused():
    from analog_moe import CVMM
    x = torch.randn(1, 4, 8)
    keys = torch.randn(2, 8, 8)
    sel = torch.zeros(1, 4, 1, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA"):
        CVMM.apply(x, torch.arange(4), sel, keys, -1)


def test_prepared_dims():
    from analog_moe import ops
    assert ops.prepared_dims(1024, 128) == (128, 1024, 1024, 128)
    assert ops.prepared_dims(40, 24) == (32, 64, 48, 64)
