"""The header-only C++ front end (include/ruy/*.h): code written like the reference's example program
(example/example.cc:21-182) must compile unchanged, abort loudly when there is no GPU, and on a GPU produce
what the oracle produces."""
import os
import subprocess

import numpy as np
import pytest

import util
from ruy_b200 import cases
from ruy_b200._lib import LIB_PATH
from ruy_b200.api import Layout, Order

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "shim_example.cc")


def _build(tmp_path):
    exe = str(tmp_path / "shim_example")
    libdir = os.path.dirname(LIB_PATH)
    subprocess.check_call(["g++", "-std=c++14", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), SRC, "-o", exe,
                           "-L", libdir, "-lruy_b200", f"-Wl,-rpath,{libdir}"])
    return exe


def test_example_compiles_against_the_drop_in_headers_and_needs_a_gpu(tmp_path):
    import torch
    exe = _build(tmp_path)
    if torch.cuda.is_available():
        pytest.skip("a device is present; the run is checked by the gpu test")
    p = subprocess.run([exe], capture_output=True, text=True)
    assert p.returncode != 0 and "no CUDA device" in p.stderr   # loud failure, no CPU fallback


def _expected():
    rm, cm = Layout(2, 2, 2, Order.kRowMajor), Layout(2, 2, 2, Order.kColMajor)
    f = np.array([1, 2, 3, 4], np.float32)
    i8 = np.array([1, 2, 3, 4], np.int8)
    mfp, mexp = np.array([3 << 28, 5 << 28], np.int32), np.array([1, -2], np.int32)
    cs = {
        "float": cases.MulCase("f", f, rm, 0, f.copy(), cm, 0, "float32", cm),
        "float_bias_clamp": cases.MulCase("fb", f, rm, 0, f.copy(), cm, 0, "float32", cm, 0, np.array([1, 0], np.float32),
                                          clamp=(0.0, 15.0)),
        "double_lhs_float_rhs": cases.MulCase("d", np.array([1.5, 2, 3, 4], np.float64), rm, 0, np.array([1, 2, 3, 4.25], np.float32),
                                              cm, 0, "float32", cm, 0, np.array([0.5, -1], np.float64), clamp=(-np.inf, 20.0)),
        "uint8_asymmetric": cases.MulCase("u8", np.array([124, 125, 126, 127], np.uint8), rm, 125,
                                          np.array([129, 130, 131, 132], np.uint8), cm, 132, "uint8", cm, 129, None, 1 << 30, 0),
        "int8_perchannel": cases.MulCase("pc", i8, rm, 0, i8.copy(), cm, 0, "int8", cm, 0, None, mfp, mexp),
        "int8_raw_accumulators": cases.MulCase("raw", i8, rm, 0, i8.copy(), cm, 0, "int32", cm),
        "int8_times_int16": cases.MulCase("i16", i8, rm, 0, np.array([1000, 2000, 3000, 4000], np.int16), cm, 0, "int16", cm, 0,
                                          None, mfp, mexp),
    }
    # destinations are column-major 2x2: the program prints storage order
    return {k: util.run_oracle(c).T.reshape(-1).astype(np.float64) for k, c in cs.items()}


@pytest.mark.gpu
def test_example_runs_on_the_gpu_and_matches_the_oracle(tmp_path):
    exe = _build(tmp_path)
    out = subprocess.run([exe], capture_output=True, text=True, check=True).stdout
    got = {line.split()[0]: [float(v) for v in line.split()[1:]] for line in out.strip().splitlines()}
    for name, want in _expected().items():
        assert np.array_equal(np.array(got[name]), want), (name, got[name], want)
    assert got["last_used_path"] == [0x40]           # most significant default path, as ruy reports on an AVX-512 host
    assert got["enabled_paths"] == [0x1] and got["max_num_threads"] == [4]
    assert got["advisory"] == [1]   # the last mul had 2-entry per-channel buffers: ruy would have re-allocated them
