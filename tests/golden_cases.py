"""The named, seeded cases whose reference outputs are committed under tests/golden/.

Shared by the generator (tests/golden/make_golden.py, which runs the compiled reference)
and by the tests that replay them against the C oracle and the CUDA library."""
import numpy as np

from ruy_b200 import cases
from ruy_b200.api import ChannelDimension


def golden_cases():
    out = []
    out.append(cases.config0())                                   # benchmark config 0
    out.append(cases.config0(exps=(-17, -13)))                    # non-saturating variant
    out.append(cases.config0(dst="int32"))
    for shape in [(50, 50, 50), (17, 301, 9), (256, 64, 1)]:      # config 1 small shapes
        out.append(cases.config1(shape))
    out.extend(cases.config2(n=16384, seed=0, first=0, count=6))   # first muls of config 2
    out.append(cases.config3(rows=192, depth=256, cols=160, dst="int32"))
    out.append(cases.config3(rows=192, depth=256, cols=160, dst="int8"))
    out.append(cases.config4(4, batch=1))                         # 1024 x 512 x 49, uint8
    # ruy's type matrix (ruy/BUILD:1195-1207) on ragged shapes, all storage orders, padded strides
    types = [("uint8", "uint8", "uint8"), ("int8", "int8", "int8"), ("int8", "int8", "uint8"),
             ("int8", "uint8", "int8"), ("uint8", "uint8", "int16"), ("int8", "int8", "int32"),
             ("int8", "uint8", "int32"), ("int8", "int16", "int16"), ("int16", "int8", "int16")]
    orders = ["RCC", "CCC", "RRC", "CRC", "RCR", "CCR", "RRR", "CRR"]
    for t, (l, r, d) in enumerate(types):
        for o, ords in enumerate(orders):
            if (t + o) % 3:
                continue
            out.append(cases.random_case(33 + t, 70 + 3 * o, 17 + 2 * t, l, r, d, orders=ords, extra_stride=(o % 2),
                                         perchannel=bool((t + o) % 2),
                                         channel=ChannelDimension.kCol if o % 3 == 0 else ChannelDimension.kRow,
                                         seed=100 + t * 8 + o))
    out.append(cases.random_case(5, 5001, 4, "int8", "int8", "int8", seed=7))          # deep
    out.append(cases.random_case(1, 32767, 1, "uint8", "uint8", "uint8", seed=8))      # deepest ruy tests
    out.append(cases.random_case(64, 3, 65, "int8", "int8", "int8", seed=9))           # shallow
    out.append(cases.random_case(37, 43, 1, "uint8", "uint8", "uint8", seed=10))       # matrix * vector
    out.append(cases.random_case(40, 40, 40, "float32", "float32", "float32", orders="CRR", extra_stride=1, seed=11))
    # ruy's two mixed floating-point cases, double accumulator (ruy/BUILD:1195-1207)
    out.append(cases.random_case(33, 70, 17, "float64", "float32", "float32", orders="RCC", extra_stride=1, seed=12))
    out.append(cases.random_case(29, 65, 40, "float32", "float64", "float64", orders="CRR", seed=13,
                                 channel=ChannelDimension.kCol))
    # a few columns against a wide operand (the register-level MMA form of the narrow kernel: whole steps of 256 bytes
    # of depth plus a tail, wide rows left over past the last 16, one and two tiles of 8 narrow rows, the narrow side
    # as either operand) and operands that must be packed first (rows off the 16-byte grid; width-contiguous storage)
    out.append(cases.random_case(1030, 4112, 5, "int8", "uint8", "int8", orders="RCC", perchannel=True, symmetric=False, seed=14))
    out.append(cases.random_case(1500, 784, 13, "uint8", "int8", "int8", orders="RCR", perchannel=True,
                                 channel=ChannelDimension.kCol, symmetric=False, seed=15))
    out.append(cases.random_case(3, 2064, 1100, "int8", "int8", "int16", orders="RCC", symmetric=False, seed=16))
    out.append(cases.random_case(129, 4100, 96, "int8", "int8", "int8", orders="RCC", extra_stride=3, perchannel=True,
                                 symmetric=False, seed=17))
    out.append(cases.random_case(300, 260, 200, "uint8", "uint8", "uint8", orders="CRC", extra_stride=1, symmetric=False, seed=18))
    names = [c.name for c in out]
    assert len(set(names)) == len(names), "golden case names must be unique"
    return out


def requant_extreme_cases():
    """Multiplier exponents on both sides of every fast-path boundary of the epilogues (total shift 24..61), multipliers
    at the ends of their range, biases large enough to wrap or to leave the small-addend path, degenerate clamps and
    extreme destination zero points; per-tensor and per-channel along either destination dimension."""
    exps = (7, 1, 0, -1, -2, -13, -14, -15, -19, -20, -21, -30)
    mfps = (1 << 30, (1 << 31) - 1, 1518500250)
    out = []
    for i, e in enumerate(exps):
        c = cases.random_case(70, 48, 90, "int8", "uint8", "int8", orders="RCC", symmetric=False, seed=100 + i)
        c.mfp, c.mexp = mfps[i % 3], e
        if e > -8:
            # small accumulators, so that multipliers near and above one do not saturate every output
            r2 = np.random.default_rng(50 + i)
            c.lhs = (c.lhs_zp + r2.integers(-1, 1, size=c.lhs.shape, endpoint=True)).astype(c.lhs.dtype)
            c.rhs = (c.rhs_zp + r2.integers(-2, 2, size=c.rhs.shape, endpoint=True)).clip(0, 255).astype(c.rhs.dtype)
            c.bias = r2.integers(-3, 3, size=c.bias.shape, endpoint=True).astype(np.int32)
        if e <= -15:
            # large biases, so that multipliers far below one still produce a spread of outputs
            r2 = np.random.default_rng(70 + i)
            mag = min(1 << (6 - e), 1 << 30)
            c.bias = r2.integers(-mag, mag, size=c.bias.shape, endpoint=True).astype(np.int32)
        c.dst_zp = (-128, 127, 3)[i % 3]
        c.name += f"_pt_e{e}"
        out.append(c)
    rng = np.random.default_rng(7)
    for j, (orders, channel) in enumerate((("RCC", ChannelDimension.kRow), ("RCC", ChannelDimension.kCol),
                                            ("RCR", ChannelDimension.kRow), ("RCR", ChannelDimension.kCol))):
        c = cases.random_case(70, 48, 90, "uint8", "uint8", "uint8", orders=orders, symmetric=False, perchannel=True,
                              channel=channel, seed=200 + j)
        nch = 70 if channel == ChannelDimension.kRow else 90
        c.mexp = rng.choice(exps, size=nch).astype(np.int32)
        c.mfp = rng.choice(mfps, size=nch).astype(np.int32)
        b = rng.integers(-20000, 20000, size=nch).astype(np.int64)
        b[::7] = (1 << 30) + 5
        b[3::7] = -(1 << 30) - 9
        b[5::11] = (1 << 31) - 1
        c.bias = b.astype(np.int32)
        c.clamp = (5, 5) if j == 3 else c.clamp
        c.name += f"_pc{j}"
        out.append(c)
    return out
