"""The cubic that the attention kernels can use for 2^x on the FMA pipe (``mb::poly_exp2`` in
mist_b200/csrc/common.cuh), replayed in float32 on the CPU with the constants read from the source."""
import os
import re

import numpy as np

SRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "mist_b200", "csrc", "common.cuh")


def _constants():
    body = open(SRC).read()
    body = body[body.index("float poly_exp2(float x)"):]
    body = body[:body.index("return")]
    c3, c2 = re.search(r"fmaf\(([0-9.]+)f, f, ([0-9.]+)f\)", body).groups()
    c1, c0 = re.findall(r"fmaf\(p, f, ([0-9.]+)f\)", body)
    magic = re.search(r"x \+ ([0-9.]+)f;", body).group(1)
    clamp = re.search(r"fmaxf\(x, (-[0-9.]+)f\)", body).group(1)
    return [np.float32(v) for v in (c0, c1, c2, c3)], np.float32(magic), np.float32(clamp)


def poly_exp2(x):
    c, magic, clamp = _constants()
    x = np.maximum(x.astype(np.float32), clamp)
    t = (x + magic).astype(np.float32)
    f = (x - (t - magic).astype(np.float32)).astype(np.float32)
    p = (c[3] * f + c[2]).astype(np.float32)
    p = (p * f + c[1]).astype(np.float32)
    p = (p * f + c[0]).astype(np.float32)
    e = (t.view(np.int32).astype(np.int64) << 23) & 0xFFFFFFFF
    bits = (p.view(np.int32).astype(np.int64) + e) & 0xFFFFFFFF
    return bits.astype(np.uint32).view(np.float32)


def test_cubic_exp2_is_far_below_bf16_rounding():
    x = np.linspace(-60.0, 9.0, 1_500_001).astype(np.float32)
    rel = np.abs(poly_exp2(x) / np.exp2(x.astype(np.float64)) - 1.0)
    assert rel.max() < 1.0e-4           # bf16 rounds at 3.9e-3
    f = poly_exp2(np.array([-0.5, 0.5, 0.0], dtype=np.float32))
    assert abs(f[0] * f[1] - 1.0) < 2e-4 and abs(f[2] - 1.0) < 1e-4


def test_cubic_exp2_of_masked_scores_is_negligible():
    tiny = poly_exp2(np.array([-np.inf, -1e30, -125.0, -300.0], dtype=np.float32))
    assert np.all(tiny > 0) and np.all(tiny < 1e-37)      # 2^-125 instead of an exact zero


def test_magic_constant_leaves_only_the_integer_in_the_shifted_bits():
    _, magic, _ = _constants()
    assert (int(magic.view(np.int32)) << 23) & 0xFFFFFFFF == 0
