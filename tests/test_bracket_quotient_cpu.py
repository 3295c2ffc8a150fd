"""The quantizer does not divide in its common path: it converts the two products
x * y(1 - 2^-21) and x * y(1 + 2^-21), y = RN(1/t), and accepts their codes when they agree.
This file replays that rule in float32 numpy arithmetic and checks it against the code of the
exact quotient RN(x / t) - on random operands and on operands placed within a few ulps of
every E2M1 rounding boundary, where a wrong rule would show first."""
import numpy as np

from oracle import ck_oracle as oc

Y_HI = np.float32(1.0 + 2.0 ** -21)
Y_LO = np.float32(1.0 - 2.0 ** -21)
BOUNDARIES = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)


def _codes(q: np.ndarray) -> np.ndarray:
    return oc.f32_to_e2m1(np.clip(q, np.float32(-6.0), np.float32(6.0)))


def _bracket(x: np.ndarray, t: np.ndarray):
    y = (np.float32(1.0) / t).astype(np.float32)          # correctly rounded reciprocal
    hi = _codes((x * (y * Y_HI).astype(np.float32)).astype(np.float32))
    lo = _codes((x * (y * Y_LO).astype(np.float32)).astype(np.float32))
    return hi, lo


def _check(x: np.ndarray, t: np.ndarray) -> float:
    exact = _codes((x / t).astype(np.float32))
    hi, lo = _bracket(x, t)
    agree = hi == lo
    assert np.array_equal(hi[agree], exact[agree]), "agreeing bracket codes differ from the exact quotient's code"
    return 1.0 - agree.mean()


def _bf16(x: np.ndarray) -> np.ndarray:
    return oc.bf16_bits_to_f32(oc.f32_to_bf16_bits(x.astype(np.float32)))


def test_random_operands():
    rng = np.random.default_rng(0)
    x = _bf16(rng.standard_normal(2_000_000) * 3.0)
    t = (np.exp(rng.uniform(-8.0, 3.0, x.size))).astype(np.float32)
    miss = _check(x, t)
    assert miss < 1e-3  # the exact path is rare on random data
    xs = x.copy()
    xs[::7] = 0.0
    xs[3::7] = -0.0
    _check(xs, t)  # signed zeros keep their sign through the products


def test_operands_next_to_every_rounding_boundary():
    rng = np.random.default_rng(1)
    n = 200_000
    t = (np.exp(rng.uniform(-6.0, 2.0, n))).astype(np.float32)
    for b in BOUNDARIES:
        target = (t * b).astype(np.float32)
        bits = target.view(np.uint32)
        for delta in range(-6, 7):            # float32 inputs a few ulps around t * boundary
            x = (bits.astype(np.int64) + delta).astype(np.uint32).view(np.float32)
            _check(x, t)
            _check(-x, t)
        # bf16 inputs: the nearest representable values on both sides
        xb = _bf16(target)
        for step in (-1, 0, 1):
            xb_s = (oc.f32_to_bf16_bits(xb).astype(np.int32) + step).astype(np.uint16)
            _check(oc.bf16_bits_to_f32(xb_s), t)


def test_divisors_with_extreme_significands():
    """Divisors whose significand is all ones or a power of two, where a reciprocal is least accurate."""
    rng = np.random.default_rng(2)
    exps = rng.integers(-20, 10, 50_000)
    for mant in (0x7FFFFF, 0x000000, 0x000001, 0x400000, 0x7FFFFE):
        t = ((exps + 127).astype(np.uint32) << np.uint32(23) | np.uint32(mant)).view(np.float32)
        for b in BOUNDARIES:
            for delta in (-2, -1, 0, 1, 2):
                x = ((t * b).astype(np.float32).view(np.uint32).astype(np.int64) + delta).astype(np.uint32).view(np.float32)
                _check(x, t)
