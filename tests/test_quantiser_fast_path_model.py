"""The TORCHREF activation quantiser on the GPU replaces x / scale by x * (1 / scale) wherever that cannot change
the rounded integer, and keeps the division otherwise (quantize4_torchref_fast in csrc/common.cuh: the product is
clamped to +-127 first, rounded by adding 1.5 * 2^23, and the division decides when it lies within 1e-4 of a
half-integer).  This is
a float32 model of that rule in numpy (IEEE single operations, as the device code uses round-to-nearest
intrinsics), checked against the exact statement clamp(rint(x / scale), +-127) of tests/test_moe_w8a8.py:40-43
on random rows and on inputs placed on the rounding boundaries.  The device code itself is compared with the
oracle bit for bit in the GPU tests."""
from __future__ import annotations

import numpy as np


def _exact(v, scale):
    return np.clip(np.rint((v / scale).astype(np.float32)), -127, 127)


def _fast(v, scale):
    inverse = (np.float32(1.0) / scale).astype(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        raw = (v * inverse).astype(np.float32)
    product = np.fmax(np.fmin(raw, np.float32(127.0)), np.float32(-127.0))  # fminf / fmaxf: NaN ends at +127
    nearest = np.rint(product)
    distance = np.abs((product - nearest).astype(np.float32))
    slow = distance > np.float32(0.4999)
    return np.where(slow, _exact(v, scale), nearest), slow


def _fast_groups_of_four(v, scale):
    """The device takes the division for all four values of a group when any of them is near a boundary, and reads the
    integer out of (product + 1.5 * 2^23)'s low mantissa byte."""
    inverse = (np.float32(1.0) / scale).astype(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        raw = (v * inverse).astype(np.float32)
    product = np.fmax(np.fmin(raw, np.float32(127.0)), np.float32(-127.0))
    shifted = (product + np.float32(12582912.0)).astype(np.float32)
    nearest = (shifted - np.float32(12582912.0)).astype(np.float32)
    distance = np.abs((product - nearest).astype(np.float32))
    slow = np.repeat((distance.reshape(-1, 4) > np.float32(0.4999)).any(axis=1), 4)
    low_byte = (shifted.view(np.uint32) & np.uint32(0xFF)).astype(np.uint8).view(np.int8).astype(np.float32)
    return np.where(slow, _exact(v, scale), low_byte)


def _to_bf16(v):
    bits = v.astype(np.float32).view(np.uint32)
    rounded = (bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return rounded.view(np.float32)


def test_fast_path_equals_division_on_random_rows():
    rng = np.random.default_rng(7)
    count = 2_000_000
    amax = np.maximum(np.abs(rng.standard_normal(count)).astype(np.float32) * np.float32(rng.uniform(1e-3, 50)), np.float32(1e-6))
    v = _to_bf16(amax * rng.uniform(-1, 1, count).astype(np.float32))
    scale = np.maximum((amax / np.float32(127.0)).astype(np.float32), np.float32(1e-30))
    fast, slow = _fast(v, scale)
    assert np.array_equal(fast, _exact(v, scale))
    assert np.array_equal(_fast_groups_of_four(v, scale), _exact(v, scale))
    assert slow.mean() < 1e-3  # the division is the rare case


def test_fast_path_equals_division_on_rounding_boundaries():
    rng = np.random.default_rng(8)
    count = 2_000_000
    scale = (np.abs(rng.standard_normal(count)).astype(np.float32) * np.float32(0.05) + np.float32(1e-4)).astype(np.float32)
    half = rng.integers(-128, 128, count).astype(np.float32) + np.float32(0.5)
    for nudge in (0, 1, -1, 2, -2):
        v = (half * scale).astype(np.float32)
        v = (v.view(np.int32) + np.int32(nudge)).view(np.float32)  # the boundary value and its neighbours in float32
        fast, _ = _fast(v, scale)
        assert np.array_equal(fast, _exact(v, scale))
        assert np.array_equal(_fast_groups_of_four(v, scale), _exact(v, scale))


def test_fast_path_handles_zero_rows_and_overflow():
    scale = np.full(4, 1e-30, dtype=np.float32)  # the clamp of an all-zero row
    v = np.array([0.0, 1e-31, -1e-28, 3e-29], dtype=np.float32)
    fast, _ = _fast(v, scale)
    assert np.array_equal(fast, _exact(v, scale))
    assert np.array_equal(_fast_groups_of_four(v, scale), _exact(v, scale))
    big = np.array([1e30, -1e30, np.inf, np.nan], dtype=np.float32)  # clamped before the rounding: +-127 without the division
    fast, slow = _fast(big, np.full(4, 1e-3, dtype=np.float32))
    assert not slow.any() and np.array_equal(fast, np.array([127, -127, 127, 127], dtype=np.float32))
    assert np.array_equal(_fast_groups_of_four(big, np.full(4, 1e-3, dtype=np.float32)), fast)
