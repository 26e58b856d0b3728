"""The C-ABI boundary, checked without a GPU: the library loads, exports every symbol the header
declares, its structs have the layout the Python mirror assumes, host-side validation follows
ruy/validate.h, and nothing pretends to work when there is no device."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

import ruy_b200
from ruy_b200 import _abi, cases
from ruy_b200._lib import LIB_PATH, lib
from ruy_b200.api import Layout, Matrix, MulParams, Order, make_simple_layout

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ruy_b200.h")


def _declared():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"RUYB200_API [\w\s\*]+?\b(ruyb200_\w+)\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared()
    assert len(names) >= 27
    out = subprocess.check_output(["nm", "-D", "--defined-only", LIB_PATH], text=True)
    exported = set(re.findall(r" T (ruyb200_\w+)", out))
    assert set(names) <= exported, sorted(set(names) - exported)
    assert set(names) == set(_abi.PROTOTYPES), "Python prototypes and header disagree"
    lib()  # loads, declares prototypes, checks the ABI version


def test_struct_layout_matches_c(tmp_path):
    src = tmp_path / "sizes.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "ruy_b200.h"\nint main(){printf("%zu %zu %zu %zu %zu %zu\\n",'
                   "sizeof(ruyb200_matrix),sizeof(ruyb200_mul_params),sizeof(ruyb200_mul_desc),"
                   "offsetof(ruyb200_mul_desc,params),offsetof(ruyb200_mul_params,clamp_min),"
                   "offsetof(ruyb200_matrix,order));return 0;}\n")
    exe = tmp_path / "sizes"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    got = [int(v) for v in subprocess.check_output([str(exe)], text=True).split()]
    want = [C.sizeof(_abi.MatrixDesc), C.sizeof(_abi.MulParamsDesc), C.sizeof(_abi.MulDesc), _abi.MulDesc.params.offset,
            _abi.MulParamsDesc.clamp_min.offset, _abi.MatrixDesc.order.offset]
    assert got == want


def test_header_is_plain_c_and_cxx(tmp_path):
    for comp, ext, std in (("gcc", "c", "-std=c99"), ("g++", "cc", "-std=c++14")):
        f = tmp_path / f"inc.{ext}"
        f.write_text('#include "ruy_b200.h"\nint main(void){return RUYB200_ABI_VERSION - 1;}\n')
        subprocess.check_call([comp, std, "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), "-c",
                               str(f), "-o", str(tmp_path / "inc.o")])


def _mk(rows=4, depth=5, cols=3, lhs="int8", rhs="int8", dst="int8"):
    c = cases.random_case(rows, depth, cols, lhs, rhs, dst, seed=1)
    lhs_m, rhs_m, p, dst_m, keep = c.bind(c.new_dst())
    return lhs_m, rhs_m, p, dst_m, keep


def test_validate_accepts_ruys_type_matrix():
    combos = [("float32",) * 3, ("float64", "float32", "float32"), ("float32", "float64", "float64"), ("uint8", "uint8", "uint8"), ("int8", "int8", "int8"), ("int8", "int8", "uint8"),
              ("int8", "uint8", "int8"), ("uint8", "uint8", "int16"), ("int8", "int8", "int32"), ("int8", "uint8", "int32"),
              ("int8", "int16", "int16"), ("int16", "int8", "int16")]
    for l, r, d in combos:
        lhs, rhs, p, dst, keep = _mk(lhs=l, rhs=r, dst=d)
        assert ruy_b200.validate(lhs, rhs, p, dst) == _abi.OK, (l, r, d, lib().ruyb200_last_error())


def test_validate_zero_point_rules():
    # ruy/validate.h:33-38: float zero points must be 0
    lhs, rhs, p, dst, keep = _mk(lhs="float32", rhs="float32", dst="float32")
    lhs.zero_point = 1
    assert ruy_b200.validate(lhs, rhs, p, dst) == _abi.ERR_INVALID
    lhs, rhs, p, dst, keep = _mk(lhs="float64", rhs="float32", dst="float32")
    assert p.accum == "float64"
    rhs.zero_point = 1
    assert ruy_b200.validate(lhs, rhs, p, dst) == _abi.ERR_INVALID
    lhs, rhs, p, dst, keep = _mk(lhs="float64", rhs="float32", dst="float32")
    p.accum = "int32"       # a double operand with an integer accumulator is outside ruy's type space
    assert ruy_b200.validate(lhs, rhs, p, dst) == _abi.ERR_UNSUPPORTED
    # ruy/validate.h:47-57: 16-bit inputs need every zero point to be 0
    lhs, rhs, p, dst, keep = _mk(lhs="int8", rhs="int16", dst="int16")
    dst.zero_point = 3
    assert ruy_b200.validate(lhs, rhs, p, dst) == _abi.ERR_INVALID
    # ruy/validate.h:59-65: both zero points at the lowest value only for uint8 x uint8
    lhs, rhs, p, dst, keep = _mk()
    lhs.zero_point, rhs.zero_point = -128, -128
    assert ruy_b200.validate(lhs, rhs, p, dst) == _abi.ERR_INVALID
    lhs, rhs, p, dst, keep = _mk(lhs="uint8", rhs="uint8", dst="uint8")
    lhs.zero_point, rhs.zero_point = 0, 0
    assert ruy_b200.validate(lhs, rhs, p, dst) == _abi.OK


def test_validate_shapes_strides_and_multiplier_preconditions():
    lhs, rhs, p, dst, keep = _mk()
    rhs.layout = Layout(rhs.layout.rows + 1, rhs.layout.cols, rhs.layout.stride + 1, rhs.layout.order)
    assert ruy_b200.validate(lhs, rhs, p, dst) == _abi.ERR_INVALID
    lhs, rhs, p, dst, keep = _mk()
    dst.layout = Layout(dst.layout.rows, dst.layout.cols, dst.layout.rows - 1, Order.kColMajor)
    assert ruy_b200.validate(lhs, rhs, p, dst) == _abi.ERR_INVALID
    lhs, rhs, p, dst, keep = _mk()
    p.multiplier_exponent = -32  # ruy/apply_multiplier.cc:51 (RUY_CHECK_GE(shift, -31))
    assert ruy_b200.validate(lhs, rhs, p, dst) == _abi.ERR_INVALID
    lhs, rhs, p, dst, keep = _mk()
    p.multiplier_fixedpoint = -5
    assert ruy_b200.validate(lhs, rhs, p, dst) == _abi.ERR_INVALID
    lhs, rhs, p, dst, keep = _mk()
    lhs.data = np.zeros(lhs.data.size, np.float32)  # float x int8 is outside ruy's type space
    lhs.zero_point = 0
    assert ruy_b200.validate(lhs, rhs, p, dst) == _abi.ERR_UNSUPPORTED


def test_defaults_follow_ruy():
    # ruy/mul_params_test.cc:26-73, ruy/matrix_test.cc:23-95
    p = MulParams("int32", "uint8")
    assert (p.multiplier_fixedpoint, p.multiplier_exponent, p.bias) == (0, 0, None)
    assert (p.clamp_min, p.clamp_max) == (0, 255)
    assert p.channel_dimension == ruy_b200.ChannelDimension.kRow
    assert p.perchannel_buffers_capacity_rounding == 1
    f = MulParams("float32", "float32")
    assert f.clamp_min == -np.inf and f.clamp_max == np.inf
    m = Matrix()
    assert m.zero_point == 0 and m.cache_policy == ruy_b200.CachePolicy.kNeverCache
    lay = make_simple_layout(3, 5, Order.kRowMajor)
    assert (lay.rows, lay.cols, lay.stride) == (3, 5, 5)
    assert make_simple_layout(3, 5, Order.kColMajor).stride == 3
    assert int(ruy_b200.kDefaultPaths) == 0x71


def test_no_device_means_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = C.c_void_p()
    rc = lib().ruyb200_ctx_create(0, C.byref(h))
    assert rc == _abi.ERR_NO_DEVICE and not h
    with pytest.raises(ruy_b200.RuyError):
        ruy_b200.Context(0)
