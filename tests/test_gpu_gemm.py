"""Multi-row products on the tcgen05 tensor cores (vb_op_matmul_rows, the prefill path) against the CPU checker."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

FMTS = ["f32", "f16", "bf16", "q4g32", "q4g64ref", "i8pc"]


@pytest.fixture(scope="module")
def dev(vb):
    from velox_b200.engine import DeviceBuffer
    return DeviceBuffer


def code(oracle, name):
    return {"f32": oracle.FMT_F32, "f16": oracle.FMT_F16, "bf16": oracle.FMT_BF16, "q4g32": oracle.FMT_Q4G32,
            "q4g64ref": oracle.FMT_Q4G64REF, "i8pc": oracle.FMT_I8PC}[name]


def run_rows(vb, dev, data, scales, c, x, in_dim, out_dim):
    lib = vb.load()
    n_rows = x.shape[0]
    ws_bytes = lib.vb_op_matmul_rows_workspace_bytes(in_dim, out_dim, n_rows)
    ws = dev(ws_bytes + 1024)
    ws_ptr = C.c_void_p((ws.ptr.value + 1023) // 1024 * 1024)
    dw, dx, dy = dev.from_numpy(data), dev.from_numpy(x), dev(n_rows * out_dim * 4)
    ds = dev.from_numpy(scales) if scales is not None else None
    vb.check(lib.vb_op_matmul_rows(dy.ptr, dx.ptr, dw.ptr, ds.ptr if ds else None, c, in_dim, out_dim, n_rows, ws_ptr, ws_bytes, None))
    vb.check(lib.vb_dev_sync())
    return dy.to_numpy(np.float32, (n_rows, out_dim))


# (in_dim, out_dim, rows): ragged tiles in every direction, K that ends inside a 64-element stage, one row, many tiles
SHAPES = [(64, 5, 3), (96, 128, 1), (576, 1536, 130), (4096, 300, 257), (1536, 576, 128), (1024, 256, 512)]


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("shape", SHAPES)
def test_matmul_rows_parity(vb, oracle, dev, fmt, shape):
    in_dim, out_dim, n_rows = shape
    if fmt == "q4g64ref" and in_dim % 64:
        pytest.skip("format needs in_dim % 64 == 0")
    c = code(oracle, fmt)
    w = oracle.fill_normal(out_dim * in_dim, 15, 1, 0.02).reshape(out_dim, in_dim)
    data, scales = oracle.quantize(w, c)
    x = oracle.fill_normal(n_rows * in_dim, 15, 2, 1.0).reshape(n_rows, in_dim)
    got = run_rows(vb, dev, data, scales, c, x, in_dim, out_dim)
    scale = np.sqrt(in_dim) * 0.02
    # 1. the kernel's own arithmetic restated in float64: decode batches (up to 32 rows) multiply single fp16 operands;
    #    larger chunks multiply x, and weights fp16 cannot hold exactly, as fp16 hi + lo parts, i.e. the fp32 values
    split = n_rows > 32
    xh = (x if split else x.astype(np.float16)).astype(np.float64)
    if fmt == "i8pc":
        wh = data.astype(np.float64)
        want16 = (xh @ wh.T) * scales.view(np.float16).astype(np.float64)[None, :]
    else:
        wd = oracle.dequantize(data, scales, c, out_dim, in_dim)
        wh = (wd if split else wd.astype(np.float16)).astype(np.float64)
        want16 = xh @ wh.T
    assert np.max(np.abs(got - want16)) <= 1e-4 * scale + 1e-6  # fp32 accumulation in the tensor cores only
    # 2. the reference's fp32 product: the two operand roundings to fp16 (2^-11 relative each) stay far below the
    #    2e-2 logit bound
    for r in (0, n_rows // 2, n_rows - 1):
        want = oracle.matvec(x[r], data, scales, c, in_dim, out_dim)
        assert np.max(np.abs(got[r] - want)) <= 3e-3 * scale


def test_matmul_rows_inputs_beyond_fp16_range(vb, oracle, dev):
    """Rows of x with values around 1e5 (un-normalised activations of a real checkpoint can get there): the chunk path carries
    them as fp16 hi + lo halves (exact up to 2 x 65504), the decode-batch path saturates; neither produces infinities."""
    in_dim, out_dim = 512, 256
    c = oracle.FMT_Q4G32
    w = oracle.fill_normal(out_dim * in_dim, 21, 1, 0.02).reshape(out_dim, in_dim)
    data, scales = oracle.quantize(w, c)
    for n_rows in (64, 8):
        x = oracle.fill_normal(n_rows * in_dim, 21, 2, 1.0).reshape(n_rows, in_dim)
        x[1, 7], x[1, 300], x[n_rows - 1, 0] = 1.0e5, -9.5e4, 1.2e5
        got = run_rows(vb, dev, data, scales, c, x, in_dim, out_dim)
        assert np.all(np.isfinite(got))
        if n_rows > 32:  # hi + lo halves hold these values exactly: the product agrees with the fp32 reference
            for r in (1, n_rows - 1, 5):
                want = oracle.matvec(x[r], data, scales, c, in_dim, out_dim)
                assert np.max(np.abs(got[r] - want)) <= 1e-3 * max(1.0, float(np.max(np.abs(want))))
        else:            # one fp16 half: the outliers are clamped to 65504, the other rows are untouched
            want = oracle.matvec(x[5], data, scales, c, in_dim, out_dim)
            assert np.max(np.abs(got[5] - want)) <= 3e-3 * np.sqrt(in_dim) * 0.02
            xc = np.clip(x[1], -65504.0, 65504.0)
            want = oracle.matvec(xc, data, scales, c, in_dim, out_dim)
            assert np.max(np.abs(got[1] - want)) <= 2e-3 * float(np.max(np.abs(want)))


def test_matmul_rows_linearity_at_full_size(vb, oracle, dev):
    """Llama-3-8B down-projection shape, 512 rows: (x1 + x2) W = x1 W + x2 W up to rounding, and a spot check of rows."""
    in_dim, out_dim, n_rows = 14336, 4096, 512
    c = oracle.FMT_Q4G32
    w = oracle.fill_normal(out_dim * in_dim, 16, 1, 0.02).reshape(out_dim, in_dim)
    data, scales = oracle.quantize(w, c)
    x1 = oracle.fill_normal(n_rows * in_dim, 16, 2, 1.0).reshape(n_rows, in_dim).astype(np.float16).astype(np.float32)
    x2 = oracle.fill_normal(n_rows * in_dim, 16, 3, 1.0).reshape(n_rows, in_dim).astype(np.float16).astype(np.float32)
    xs = ((x1.astype(np.float64) + x2.astype(np.float64)) / 2).astype(np.float16).astype(np.float32)
    y1, y2, ys = (run_rows(vb, dev, data, scales, c, x, in_dim, out_dim) for x in (x1, x2, xs))
    scale = np.sqrt(in_dim) * 0.02
    assert np.max(np.abs((y1 + y2) / 2 - ys)) <= 2e-3 * scale
    for r in (0, 300, 511):
        want = oracle.matvec(x1[r], data, scales, c, in_dim, out_dim)
        assert np.max(np.abs(y1[r] - want)) <= 3e-3 * scale


def test_matmul_rows_bad_arguments(vb, dev):
    lib = vb.load()
    b = dev(8 << 20)
    base = (b.ptr.value + 1023) // 1024 * 1024
    p, p16 = C.c_void_p(base), C.c_void_p(base + 16)
    assert lib.vb_op_matmul_rows(p, p, p, None, vb.FMT_F32, 8, 0, 1, p, 6 << 20, None) == vb.OK
    assert lib.vb_op_matmul_rows(p, p, p, None, vb.FMT_F32, 8, 4, 0, p, 6 << 20, None) == vb.OK
    assert lib.vb_op_matmul_rows(p, p, p, None, vb.FMT_F32, 12, 4, 1, p, 6 << 20, None) == vb.ERR_INVALID  # in_dim % 8
    assert lib.vb_op_matmul_rows(p, p, p, None, vb.FMT_Q4G32, 64, 4, 1, p, 6 << 20, None) == vb.ERR_INVALID  # no scales
    assert lib.vb_op_matmul_rows(p, p, p, None, vb.FMT_F32, 64, 4, 1, p16, 6 << 20, None) == vb.ERR_INVALID  # alignment
    assert lib.vb_op_matmul_rows(p, p, p, None, vb.FMT_F32, 64, 4, 1, p, 64, None) == vb.ERR_INVALID  # workspace too small
