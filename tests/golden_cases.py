"""The named, seeded cases whose reference outputs are committed under tests/golden/.

Shared by the generator (tests/golden/make_golden.py, which runs the compiled reference)
and by the tests that replay them against the C oracle and the CUDA library."""
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
    names = [c.name for c in out]
    assert len(set(names)) == len(names), "golden case names must be unique"
    return out
