"""The C-ABI shared library loads without a GPU, exports every symbol the header declares, and its entry
points fail with a status code (never a crash) when there is no device or the arguments are bad."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "velox_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vb_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(vb):
    decl = declared_symbols()
    assert len(decl) >= 40
    assert sorted(vb.SIGNATURES) == decl, "velox_b200/lib.py must bind exactly the functions of include/velox_b200.h"


def test_library_exports_every_declared_symbol(vb):
    lib = C.CDLL(vb.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), "libvelox_b200.so does not export %s" % name


def test_struct_layout(vb):
    assert C.sizeof(vb.ModelDesc) == 4 * (1 + 9 + 2 + 11 + 8)


def test_errors_are_status_codes(vb):
    lib = vb.load()
    assert lib.vb_version() >= 1
    h = C.c_void_p()
    assert lib.vb_create(None, 0, C.byref(h)) == vb.ERR_INVALID
    assert b"null" in lib.vb_last_error()
    d = vb.ModelDesc()
    d.struct_bytes = 12
    assert lib.vb_create(C.byref(d), 0, C.byref(h)) == vb.ERR_INVALID
    assert lib.vb_decode_step(None) == vb.ERR_INVALID
    assert lib.vb_op_matmul(None, None, None, None, 0, 8, 8, 1, None) == vb.ERR_INVALID
    assert lib.vb_op_sample_argmax(None, None, 0, None, 0, None) == vb.ERR_INVALID
    with pytest.raises(vb.VeloxError):
        vb.check(lib.vb_op_rope(None, 1, 3, 0, 10000.0, None))


def test_no_device_fails_loudly(vb):
    """Without a GPU every compute entry point reports a CUDA error: there is no CPU fallback."""
    lib = vb.load()
    n = C.c_int32(-1)
    rc = lib.vb_device_count(C.byref(n))
    if rc == vb.OK and n.value > 0:
        pytest.skip("a GPU is present")
    from velox_b200.engine import Engine
    from helpers import TINY
    with pytest.raises(vb.VeloxError):
        Engine(TINY, max_seq_len=32)
    x = np.zeros(8, dtype=np.float32)
    p = x.ctypes.data_as(C.c_void_p)
    assert lib.vb_op_matmul(p, p, p, None, vb.FMT_F32, 8, 1, 1, None) in (vb.ERR_CUDA, vb.ERR_OOM)
