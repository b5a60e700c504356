"""The allocation-free argmax entry point (vb_op_sample_argmax_static).

Some callers cannot give the library a scratch buffer or allocate one: a runner that handed all device memory
to its arenas before serving started, or a host language binding that is not allowed to call cudaMalloc.  For
them the library carries its own small scratch.  This test calls the entry point through the C ABI twice in a
row (the built-in scratch is shared and keeps the previous call's contents) and compares with the ordinary
entry point, which must agree exactly -- indices are integers.  It runs last so that a failure here does not
hide the rest of the suite; it passes alone in a fresh process as well as after the other tests.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_argmax_matches_scratch_version_twice(vb, oracle):
    from velox_b200.engine import DeviceBuffer
    lib = vb.load()
    n = 152064
    first = oracle.fill_normal(n, 77, 1, 1.0)
    second = oracle.fill_normal(n, 77, 2, 1.0)
    second[[5, 90000, n - 1]] = 40.0            # ties across stage-1 blocks: the lowest index wins
    small = np.float32([0.5, -1.0, 0.5])          # a much shorter row after a long one: stale candidates must not leak
    for lg in (first, second, small):
        m = lg.size
        d_logits = DeviceBuffer.from_numpy(lg)
        out_a, out_b = DeviceBuffer(4), DeviceBuffer(4)
        nbytes = lib.vb_op_scratch_bytes(1, 32, 1, m)
        scratch = DeviceBuffer(nbytes)
        vb.check(lib.vb_op_sample_argmax(out_a.ptr, d_logits.ptr, m, scratch.ptr, nbytes, None))
        vb.check(lib.vb_op_sample_argmax_static(out_b.ptr, d_logits.ptr, m, None))
        a = int(out_a.to_numpy(np.uint32, (1,))[0])
        b = int(out_b.to_numpy(np.uint32, (1,))[0])
        assert a == b == oracle.lib().vo_sample_argmax_f32(lg.ctypes.data_as(C.c_void_p), m)


def test_static_argmax_rejects_oversized_rows(vb):
    from velox_b200.engine import DeviceBuffer
    lib = vb.load()
    buf = DeviceBuffer(64)
    rc = lib.vb_op_sample_argmax_static(buf.ptr, buf.ptr, (1 << 20) + 1, None)
    assert rc == vb.ERR_INVALID
    assert b"exceeds" in lib.vb_last_error()
    assert lib.vb_op_sample_argmax_static(None, buf.ptr, 4, None) == vb.ERR_INVALID
