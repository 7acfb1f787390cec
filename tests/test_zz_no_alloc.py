"""The allocation-free argmax entry point against the ordinary one.

Some users of this library cannot hand it a scratch buffer: their device memory was budgeted once at
start-up, or they call from a place where cudaMalloc is not allowed (it stalls the device and is illegal
while a stream is being captured), or another runtime owns all device memory.  bkArgmaxStatic serves
them from an array compiled into the library.  This file runs last so that a failure here cannot hide
the result of any other test.
"""
import ctypes as C

import numpy as np
import pytest

from bunker_b200 import ops
from bunker_b200 import runtime as R
from tests.util import assert_same_bits, dev

pytestmark = pytest.mark.gpu


def test_static_scratch_argmax_matches_bkargmax_twice_in_a_row(bk):
    B, V = 5, 151936
    rng = np.random.default_rng(2024)
    idx_a, val_a = R.DeviceBuffer(B * 4), R.DeviceBuffer(B * 4)
    idx_b, val_b = R.DeviceBuffer(B * 4), R.DeviceBuffer(B * 4)
    scratch = R.DeviceBuffer.zeros(ops.argmax_scratch_bytes(B))
    lib = R.cu()
    for call in range(2):                      # the second call finds the first call's leftovers in the array
        logits = rng.normal(0, 4, (B, V)).astype(np.float32)
        logits[0, 17] = logits[0, 90000] = 99.0          # tie: lowest index
        logits[1, V - 1] = 77.0 + call                    # maximum in the last chunk
        dl = dev(logits)
        ops.argmax(dl.ptr, V, B, idx_a.ptr, val_a.ptr, scratch.ptr)
        rc = lib.bkArgmaxStatic(C.c_uint64(dl.ptr), V, B, C.c_uint64(idx_b.ptr), C.c_uint64(val_b.ptr))   # through the C ABI
        assert rc == 0, R.last_error()
        want_i, got_i = idx_a.download(np.int32, (B,)), idx_b.download(np.int32, (B,))
        assert np.array_equal(got_i, want_i) and got_i[0] == 17 and got_i[1] == V - 1
        assert_same_bits(val_b.download(np.float32, (B,)), val_a.download(np.float32, (B,)), f"call {call}")
        dl.free()


def test_static_scratch_argmax_rejects_oversized_batch(bk):
    lib = R.cu()
    rc = lib.bkArgmaxStatic(C.c_uint64(256), 1000, 65, C.c_uint64(256), C.c_uint64(256))
    assert rc == R.BK_ERR_ARG and "at most 64" in R.last_error()
