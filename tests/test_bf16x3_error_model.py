"""Numerics of the `bf16x3` precision, restated in numpy (no GPU): both operands are split into
hi = bf16(v) and lo = bf16(v - hi) (round to nearest even) and the product keeps hi*hi + hi*lo + lo*hi.
The dropped terms (lo*lo and the two residuals v - hi - lo) bound the relative Frobenius error of a
product of N(0,1) data near 5e-6, inside the 1e-5 bound of the fp32-class modes; the GPU tests hold the
kernels to the same bound (tests/gpu_util.py: TOL)."""
import numpy as np


def bf16_round(v):
    """float32 -> nearest bf16 (ties to even), returned as float32."""
    bits = np.ascontiguousarray(v, dtype=np.float32).view(np.uint32)
    rounded = (bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return rounded.view(np.float32)


def split(v):
    hi = bf16_round(v)
    lo = bf16_round((v - hi).astype(np.float32))
    return hi, lo


def test_the_difference_is_exact_and_the_residual_is_below_two_to_the_minus_17():
    rng = np.random.default_rng(0)
    v = (rng.standard_normal(1 << 16) * np.exp(rng.uniform(-20, 20, 1 << 16))).astype(np.float32)
    hi, lo = split(v)
    # v - hi is exactly representable in fp32 (computed in float64 and in float32: same value)
    assert np.array_equal((v.astype(np.float64) - hi.astype(np.float64)).astype(np.float32), v - hi)
    residual = np.abs(v.astype(np.float64) - hi.astype(np.float64) - lo.astype(np.float64))
    assert np.all(residual <= np.abs(v.astype(np.float64)) * 2.0 ** -17)
    assert np.all(np.abs(lo) <= np.abs(v) * 2.0 ** -8)


def test_three_products_stay_inside_the_fp32_class_bound():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((256, 512)).astype(np.float32)
    w = (rng.standard_normal((384, 512)) * 0.02).astype(np.float32)
    xh, xl = (a.astype(np.float64) for a in split(x))
    wh, wl = (a.astype(np.float64) for a in split(w))
    got = xh @ wh.T + xh @ wl.T + xl @ wh.T
    want = x.astype(np.float64) @ w.astype(np.float64).T
    err = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert 1e-6 < err < 7e-6, err   # measured on the GPU kernels: 4.5e-6 ... 4.7e-6
