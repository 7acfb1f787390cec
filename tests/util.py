"""Helpers shared by the tests."""
import numpy as np

from bunker_b200 import runtime as R


def dev(a: np.ndarray) -> R.DeviceBuffer:
    return R.DeviceBuffer.from_numpy(np.ascontiguousarray(a))


def same_bits(a: np.ndarray, b: np.ndarray) -> bool:
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    return a.shape == b.shape and a.dtype.itemsize == b.dtype.itemsize and \
        np.array_equal(a.view(np.uint8), b.view(np.uint8))


def assert_same_bits(got: np.ndarray, want: np.ndarray, what: str = ""):
    if not same_bits(got, want):
        g = np.ascontiguousarray(got).reshape(-1)
        w = np.ascontiguousarray(want).reshape(-1)
        bad = np.nonzero(g.view(f"u{g.dtype.itemsize}") != w.view(f"u{w.dtype.itemsize}"))[0]
        i = int(bad[0])
        raise AssertionError(f"{what}: {bad.size}/{g.size} elements differ; first at {i}: got {g[i]!r} want {w[i]!r}")


def rel_err(got, want) -> float:
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))
