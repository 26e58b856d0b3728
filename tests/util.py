"""Shared helpers for the tests: run one MulCase through each implementation."""
import ctypes as C

import numpy as np

import oracle as oracle_pkg
from ruy_b200 import _abi
from ruy_b200.api import Rounding, make_desc, mul, mul_async


def run_oracle(case, rounding=Rounding.kReference, wide_float=False):
    """The C restatement; returns the logical rows x cols result."""
    dst = case.new_dst()
    lhs, rhs, p, d, keep = case.bind(dst)
    desc = make_desc(lhs, rhs, p, d)
    rc = oracle_pkg.oracle().ruy_oracle_mul(C.byref(desc), int(rounding), int(wide_float))
    assert rc == 0, rc
    return case.dst_view(dst).copy()


def run_reference(case, path=0, threads=1, reference_mul=False, ctx=None):
    """The compiled reference (ruy::Mul on `path`, or ruy::ReferenceMul); None if it is not built."""
    ref = oracle_pkg.reference()
    if ref is None:
        return None
    dst = case.new_dst()
    lhs, rhs, p, d, keep = case.bind(dst)
    desc = make_desc(lhs, rhs, p, d)
    if reference_mul:
        assert ref.ruy_ref_reference_mul(C.byref(desc)) == 0
    else:
        own = ctx is None
        if own:
            ctx = ref.ruy_ref_ctx_create(int(path), threads)
        try:
            assert ref.ruy_ref_mul(ctx, C.byref(desc)) == 0
        finally:
            if own:
                ref.ruy_ref_ctx_destroy(ctx)
    return case.dst_view(dst).copy()


def run_gpu(case, ctx, where="device", rounding=Rounding.kFromPath, sentinel=None, use_async=False):
    """The CUDA library through the C ABI.  where='device': operands resident in HBM (torch
    tensors); where='host': numpy arrays, staged by the library."""
    if where == "host":
        dst = case.new_dst(fill=sentinel)
        lhs, rhs, p, d, keep = case.bind(dst, rounding=rounding)
        mul(lhs, rhs, p, ctx, d)
        return case.dst_view(dst).copy(), dst
    import torch
    dev = torch.device("cuda", 0)
    host = case.new_dst(fill=sentinel)
    dst = torch.from_numpy(host).to(dev)
    lhs, rhs, p, d, keep = case.bind(dst, device=dev, rounding=rounding)
    torch.cuda.synchronize()
    if use_async:
        mul_async(lhs, rhs, p, ctx, d)
        ctx.sync()
    else:
        mul(lhs, rhs, p, ctx, d)
    out = dst.cpu().numpy()
    return case.dst_view(out).copy(), out


def padding_untouched(case, storage, sentinel):
    """True when the elements of a strided dst storage that are not part of the matrix still
    hold the sentinel (the kernel wrote nothing outside the logical matrix)."""
    lay = case.dst_layout
    s = np.asarray(storage)
    from ruy_b200.api import Order
    if lay.order == Order.kColMajor:
        pad = s.reshape(lay.cols, lay.stride)[:, lay.rows:]
    else:
        pad = s.reshape(lay.rows, lay.stride)[:, lay.cols:]
    return bool(np.all(pad == sentinel))


def x86_rounding_for(case):
    """The rounding ruy's x86 paths apply to this case: their SIMD kernels cover 8-bit operands and
    int8 x int16; an int16 LHS (after the operand swap that a row-major destination causes) falls
    back to the standard C++ kernel, i.e. to the reference rounding."""
    from ruy_b200.api import Order
    lhs_dtype = case.lhs.dtype if case.dst_layout.order == Order.kColMajor else case.rhs.dtype
    return Rounding.kReference if lhs_dtype == np.int16 else Rounding.kX86
