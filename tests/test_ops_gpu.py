"""Parity of the direct C-ABI kernels (through intent_ir_b200.ops, i.e. ctypes) against the
CPU oracle on the same seeded inputs: bit-exact for boolean results, within the oracle's
inferred tolerances (verify/tolerances.py figures, written out below) for floating point."""

import numpy as np
import pytest

from intent_ir_b200.ir import IntentFunction
from oracle import execute_intent, infer_tolerances
from oracle.diff import compare_outputs

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _graph(op, attrs, in_shape, out_shape, out_dtype="f32", in_dtype="f32"):
    return IntentFunction.from_json_dict({
        "name": f"one_{op}",
        "tensors": {"x": {"dtype": in_dtype, "shape": list(in_shape), "layout": "row_major"},
                    "y": {"dtype": out_dtype, "shape": list(out_shape), "layout": "row_major"}},
        "ops": [{"op": op, "inputs": ["x"], "output": "y", "attrs": attrs}], "outputs": ["y"]})


def _agree(got: np.ndarray, want: np.ndarray, atol: float, rtol: float):
    """The oracle's own comparison (diff_runner.py:357-418).  That comparison rejects any NaN
    (it tests the non-finite values with ``np.array_equal``, for which NaN != NaN), so NaN
    positions are first checked to coincide exactly and then neutralised on both sides;
    infinities still have to match in place and sign."""
    got, want = np.asarray(got), np.asarray(want)
    if got.dtype.kind == "f" or want.dtype.kind == "f":
        gn, wn = np.isnan(got), np.isnan(want)
        assert np.array_equal(gn, wn), "NaN pattern differs"
        if gn.any():
            got, want = np.where(gn, 0, got), np.where(wn, 0, want)
    d = compare_outputs({"y": want}, {"y": got}, ["y"], {"atol": atol, "rtol": rtol})
    assert d.ok, (d.summary, d.max_abs_err, d.first_bad_index)


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


# ---------------------------------------------------------------- reductions ----------------

def test_reduce_any_baseline_case_bit_exact():
    from intent_ir_b200 import ops
    rng = np.random.default_rng(0)
    mask = rng.random((16, 256)) < 0.05
    x = np.where(mask, rng.standard_normal((16, 256), dtype=np.float32), np.float32(0))
    x[3] = 0  # an all-zero row
    want = execute_intent(_graph("reduce_any", {"dims": [1]}, ["M", "N"], ["M"], "bool"), {"x": x})["y"]
    got = ops.reduce(_dev(x), "any", [1]).cpu().numpy()
    assert got.dtype == np.bool_ and np.array_equal(got, want)


def test_reduce_any_non_finite_and_signed_zero_rows(golden_edges):
    from intent_ir_b200 import ops
    x = golden_edges["x"]
    got = ops.reduce(_dev(x), "any", [1]).cpu().numpy()
    assert np.array_equal(got, golden_edges["reduce_any"])
    got = ops.reduce(_dev(x), "max", [1]).cpu().numpy()
    assert np.array_equal(got, golden_edges["reduce_max"], equal_nan=True)


@pytest.mark.parametrize("shape,dims", [
    ((1, 1), [1]), ((7, 3), [1]), ((5, 17), [1]), ((33, 256), [1]), ((9, 1000), [1]), ((4, 4096), [1]),
    ((3, 5000), [1]), ((2, 70001), [1]), ((64, 33), [0]), ((6, 40, 9), [1]), ((3, 5, 7, 11), [2, 3]),
    ((4, 6, 8), [0, 1]), ((5, 6), [0, 1]), ((2049, 2), [0]),
    # many short rows: several rows per warp (8 or 16 lanes each)
    ((5000, 4), [1]), ((4097, 8), [1]), ((6001, 60), [1]), ((4096, 64), [1]), ((7777, 100), [1]), ((5003, 128), [1]), ((4100, 132), [1]),
])
@pytest.mark.parametrize("kind", ["sum", "max", "any"])
def test_reduce_matches_oracle(shape, dims, kind):
    from intent_ir_b200 import ops
    rng = np.random.default_rng(hash((shape, tuple(dims), kind)) % 2**32)
    x = rng.standard_normal(shape, dtype=np.float32)
    if kind == "any":
        x = np.where(rng.random(shape) < 0.002, x, np.float32(0))
    sym = [f"D{i}" for i in range(len(shape))]
    out_sym = [s for i, s in enumerate(sym) if i not in dims]
    want = execute_intent(_graph(f"reduce_{kind}", {"dims": dims}, sym, out_sym, "bool" if kind == "any" else "f32"), {"x": x})["y"]
    got = ops.reduce(_dev(x), kind, dims).cpu().numpy()
    assert got.shape == np.asarray(want).shape
    if kind == "any":
        assert np.array_equal(got, want)
    else:
        _agree(got, want, 1e-3, 1e-3)  # reduce_sum / reduce_max: (1e-3, 1e-3)


def test_reduce_sum_scale_and_keepdims():
    from intent_ir_b200 import ops
    x = np.random.default_rng(1).standard_normal((12, 50), dtype=np.float32)
    got = ops.reduce(_dev(x), "sum", [1], keepdims=True, scale=1.0 / 50).cpu().numpy()
    assert got.shape == (12, 1)
    _agree(got, x.sum(axis=1, keepdims=True) * (1.0 / 50), 1e-3, 1e-3)


def test_reduce_empty_and_errors():
    from intent_ir_b200 import ops
    from intent_ir_b200.errors import B200LoweringError, B200RuntimeError
    assert ops.reduce(torch.empty((0, 8), device="cuda"), "sum", [1]).shape == (0,)
    got = ops.reduce(torch.empty((4, 0), device="cuda"), "sum", [1]).cpu().numpy()
    assert np.array_equal(got, np.zeros(4, np.float32))
    with pytest.raises(B200LoweringError):
        ops.reduce(torch.zeros((2, 3, 4), device="cuda"), "sum", [0, 2])
    with pytest.raises(B200RuntimeError):
        ops.reduce(torch.zeros((2, 3)), "sum", [1])  # host tensor


# ---------------------------------------------------------------- softmax -------------------

@pytest.mark.parametrize("shape", [(1, 1), (3, 2), (7, 37), (16, 128), (5, 129), (64, 1000), (9, 1024), (33, 2048),
                                   (17, 4096), (3, 4100), (4, 8192), (2, 16384), (3, 20000), (2, 3, 50)])
def test_softmax_matches_oracle(shape):
    from intent_ir_b200 import ops
    x = 3 * np.random.default_rng(shape[-1]).standard_normal(shape, dtype=np.float32)
    sym = [f"D{i}" for i in range(len(shape))]
    g = _graph("softmax", {"axis": -1}, sym, sym)
    want = execute_intent(g, {"x": x})["y"]
    got = ops.softmax(_dev(x)).cpu().numpy()
    tol = infer_tolerances(g).to_dict()
    assert tol == {"atol": 1e-4, "rtol": 1e-4}
    _agree(got, want, **tol)
    assert np.allclose(got.sum(axis=-1), 1.0, atol=1e-5)


def test_softmax_non_finite_rows(golden_edges):
    from intent_ir_b200 import ops
    got = ops.softmax(_dev(golden_edges["x"])).cpu().numpy()
    _agree(got, golden_edges["softmax"], 1e-4, 1e-4)  # compare_outputs demands identical NaN patterns


def test_softmax_aux_outputs_and_bf16():
    from intent_ir_b200 import ops
    x = 2 * np.random.default_rng(3).standard_normal((11, 300), dtype=np.float32)
    xd = _dev(x)
    mx = torch.empty(11, device="cuda")
    sm = torch.empty(11, device="cuda")
    ops.softmax(xd, row_max=mx, row_sum=sm)
    assert np.array_equal(mx.cpu().numpy(), x.max(axis=1))
    _agree(sm.cpu().numpy(), np.exp(x - x.max(axis=1, keepdims=True)).sum(axis=1), 1e-3, 1e-3)
    xb = xd.to(torch.bfloat16)
    got = ops.softmax(xb).float().cpu().numpy()
    xr = xb.float().cpu().numpy()
    e = np.exp(xr - xr.max(axis=1, keepdims=True))
    _agree(got, e / e.sum(axis=1, keepdims=True), 1e-3, 1e-3)  # bf16 visible: floor (1e-3, 1e-3)


# ---------------------------------------------------------------- normalisation -------------

def _ln_ref(x, w, b, eps=1e-5):
    mean = x.mean(axis=-1, keepdims=True, dtype=np.float64)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    rstd = 1.0 / np.sqrt(var + eps)
    y = (x - mean) * rstd
    if w is not None:
        y = y * w
    if b is not None:
        y = y + b
    return y, mean[..., 0], rstd[..., 0]


@pytest.mark.parametrize("shape", [(1, 2), (5, 3), (16, 128), (7, 129), (40, 1000), (9, 1024), (6, 2050), (33, 4096),
                                   (3, 8192), (2, 16384), (3, 32768), (2, 40004), (2, 131072), (1, 140000)])
def test_layernorm_matches_oracle_arithmetic(shape):
    from intent_ir_b200 import ops
    rng = np.random.default_rng(shape[1])
    x = rng.standard_normal(shape, dtype=np.float32) + np.float32(0.5)
    w = rng.uniform(0.5, 1.5, shape[1]).astype(np.float32)
    b = (0.1 * rng.standard_normal(shape[1])).astype(np.float32)
    y, mean, rstd = ops.layernorm(_dev(x), _dev(w), _dev(b), 1e-5)
    wy, wm, wr = _ln_ref(x, w, b)
    _agree(y.cpu().numpy(), wy, 1e-3, 1e-3)  # reduce_sum + rsqrt chain: capped at (1e-3, 1e-3)
    _agree(mean.cpu().numpy(), wm, 1e-3, 1e-3)
    _agree(rstd.cpu().numpy(), wr, 1e-3, 1e-3)


def test_layernorm_shift_relation_and_non_finite():
    from intent_ir_b200 import ops
    rng = np.random.default_rng(5)
    x = rng.standard_normal((8, 512), dtype=np.float32)
    w = rng.standard_normal(512, dtype=np.float32)
    b = rng.standard_normal(512, dtype=np.float32)
    y0, m0, r0 = ops.layernorm(_dev(x), _dev(w), _dev(b))
    y1, m1, r1 = ops.layernorm(_dev(x + np.float32(100.0)), _dev(w), _dev(b))  # a one-pass variance fails this
    _agree(y1.cpu().numpy(), y0.cpu().numpy(), 1e-3, 1e-3)
    _agree(m1.cpu().numpy(), m0.cpu().numpy() + 100.0, 1e-3, 1e-3)
    _agree(r1.cpu().numpy(), r0.cpu().numpy(), 1e-3, 1e-3)
    x[0, 0] = np.nan
    x[1, 0], x[1, 1] = np.inf, -np.inf
    y, m, r = ops.layernorm(_dev(x), _dev(w), _dev(b))
    with np.errstate(all="ignore"):
        wy, wm, wr = _ln_ref(x, w, b)
    _agree(y.cpu().numpy(), wy, 1e-3, 1e-3)
    _agree(m.cpu().numpy(), wm, 1e-3, 1e-3)


@pytest.mark.parametrize("n,c,hw,g", [(1, 2, 2, 2), (2, 8, 16, 4), (3, 6, 5, 3), (2, 32, 49, 8), (2, 64, 256, 8),
                                      (2, 16, 4096, 2), (1, 8, 4097, 2), (1, 4, 70000, 1)])
def test_groupnorm_matches_oracle_arithmetic(n, c, hw, g):
    from intent_ir_b200 import ops
    rng = np.random.default_rng(n * 1000 + c + hw)
    x = rng.standard_normal((n, c, hw), dtype=np.float32)
    w = rng.standard_normal(c, dtype=np.float32)
    b = rng.standard_normal(c, dtype=np.float32)
    y, mean, rstd = ops.groupnorm(_dev(x), _dev(w), _dev(b), g, 1e-5)
    x4 = x.reshape(n, g, c // g, hw).astype(np.float64)
    m = x4.mean(axis=(2, 3), keepdims=True)
    v = ((x4 - m) ** 2).mean(axis=(2, 3), keepdims=True)
    r = 1.0 / np.sqrt(v + 1e-5)
    wy = ((x4 - m) * r).reshape(n, c, hw) * w[None, :, None] + b[None, :, None]
    _agree(y.cpu().numpy(), wy, 1e-3, 1e-3)
    _agree(mean.cpu().numpy(), m.reshape(n, g), 1e-3, 1e-3)
    _agree(rstd.cpu().numpy(), r.reshape(n, g), 1e-3, 1e-3)


# ---------------------------------------------------------------- matmul --------------------

def _bf16_round(a):
    return torch.from_numpy(a).to(torch.bfloat16).float().numpy()


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 128), (256, 512, 256), (300, 264, 72), (1, 8, 8),
                                   (130, 520, 1000), (512, 1024, 4096)])
@pytest.mark.parametrize("transpose_b", [False, True])
def test_gemm_tensor_core_path(m, n, k, transpose_b):
    from intent_ir_b200 import ops
    rng = np.random.default_rng(m + n + k)
    a = _bf16_round((0.5 * rng.standard_normal((m, k))).astype(np.float32))
    b = _bf16_round((0.5 * rng.standard_normal((k, n))).astype(np.float32))
    bias = _bf16_round((0.1 * rng.standard_normal(n)).astype(np.float32))
    want = np.maximum(a.astype(np.float64) @ b.astype(np.float64) + bias, 0)
    bd = _dev(np.ascontiguousarray(b.T) if transpose_b else b, torch.bfloat16)
    got = ops.gemm_bias_act(_dev(a, torch.bfloat16), bd, _dev(bias, torch.bfloat16), "relu", transpose_b)
    ops.check_device_status()
    _agree(got.float().cpu().numpy(), want, 2e-2, 2e-2)  # matmul: (2e-2, 2e-2)
    got32 = ops.gemm_bias_act(_dev(a, torch.bfloat16), bd, None, "none", transpose_b, out_dtype=torch.float32)
    ops.check_device_status()
    _agree(got32.cpu().numpy(), a.astype(np.float64) @ b.astype(np.float64), 1e-3, 1e-3)


@pytest.mark.parametrize("m,n,k", [(32, 48, 16), (1, 1, 1), (65, 67, 33), (7, 200, 129)])
def test_gemm_fma_path_f32(m, n, k):
    from intent_ir_b200 import ops
    rng = np.random.default_rng(k)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32)
    got = ops.gemm_bias_act(_dev(a), _dev(b), _dev(bias), "relu")
    _agree(got.cpu().numpy(), np.maximum(a @ b + bias, 0), 1e-4, 1e-4)
    got = ops.gemm_bias_act(_dev(a), _dev(np.ascontiguousarray(b.T)), None, "none", transpose_b=True)
    _agree(got.cpu().numpy(), a @ b, 1e-4, 1e-4)


def test_gemm_known_answer_all_ones():
    from intent_ir_b200 import ops
    # the reference's tests/test_diff_runner.py: all-ones GEMM + bias + ReLU = K + 1
    for dt, k in ((torch.float32, 3), (torch.bfloat16, 64)):
        a = torch.ones((128, k), dtype=dt, device="cuda")
        b = torch.ones((k, 256), dtype=dt, device="cuda")
        bias = torch.ones(256, dtype=dt, device="cuda")
        got = ops.gemm_bias_act(a, b, bias, "relu")
        ops.check_device_status()
        assert torch.all(got.float() == k + 1.0)


def test_transpose2d():
    from intent_ir_b200 import ops
    x = np.random.default_rng(0).standard_normal((70, 33), dtype=np.float32)
    assert np.array_equal(ops.transpose2d(_dev(x)).cpu().numpy(), x.T)


def test_direct_c_entry_points_through_ctypes():
    """Every convenience entry point of the header, called with raw pointers."""
    import ctypes as C

    from intent_ir_b200 import _lib

    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(9)
    x = rng.standard_normal((12, 96), dtype=np.float32)
    xd = _dev(x)
    y = torch.empty_like(xd)
    assert lib.ib200_softmax(xd.data_ptr(), y.data_ptr(), None, None, _lib.F32, 12, 96, stream) == 0
    e = np.exp(x - x.max(axis=1, keepdims=True))
    _agree(y.cpu().numpy(), e / e.sum(axis=1, keepdims=True), 1e-4, 1e-4)
    flags = torch.empty(12, dtype=torch.bool, device="cuda")
    z = _dev(np.where(rng.random((12, 96)) < 0.02, x, np.float32(0)))
    assert lib.ib200_reduce_any_f32(z.data_ptr(), flags.data_ptr(), 12, 96, stream) == 0
    assert np.array_equal(flags.cpu().numpy(), (z.cpu().numpy() != 0).any(axis=1))
    w, b = _dev(rng.standard_normal(96, dtype=np.float32)), _dev(rng.standard_normal(96, dtype=np.float32))
    mean, rstd = torch.empty(12, device="cuda"), torch.empty(12, device="cuda")
    assert lib.ib200_layernorm(xd.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), _lib.F32, 12, 96, 1e-5, stream) == 0
    wy, wm, wr = _ln_ref(x, w.cpu().numpy(), b.cpu().numpy())
    _agree(y.cpu().numpy(), wy, 1e-3, 1e-3)
    _agree(mean.cpu().numpy(), wm, 1e-3, 1e-3)
    g = _dev(rng.standard_normal((2, 6, 16), dtype=np.float32))
    gy = torch.empty_like(g)
    gm, gr = torch.empty(4, device="cuda"), torch.empty(4, device="cuda")
    w6, b6 = _dev(np.ones(6, np.float32)), _dev(np.zeros(6, np.float32))
    assert lib.ib200_groupnorm(g.data_ptr(), w6.data_ptr(), b6.data_ptr(), gy.data_ptr(), gm.data_ptr(), gr.data_ptr(), _lib.F32, 2, 6, 16, 2, 1e-5, stream) == 0
    g4 = g.cpu().numpy().reshape(2, 2, 48).astype(np.float64)
    _agree(gm.cpu().numpy(), g4.mean(axis=2).reshape(4), 1e-3, 1e-3)
    assert lib.ib200_check_status(None, stream) == 0  # the library's own status word is clean
    assert lib.ib200_groupnorm(g.data_ptr(), None, None, gy.data_ptr(), None, None, _lib.F32, 2, 6, 16, 4, 1e-5, stream) == _lib.ERR_INVALID
    assert b"multiple" in lib.ib200_last_error()


@pytest.mark.parametrize("shape", [(1, 1), (7, 5), (64, 60), (33, 1024), (5, 3, 1000), (6, 4099), (2, 16384)])
@pytest.mark.parametrize("shared", [False, True])
def test_softmax_masked_direct_entry(shape, shared):
    from intent_ir_b200 import ops
    rng = np.random.default_rng(shape[-1] + shared)
    x = 3 * rng.standard_normal(shape, dtype=np.float32)
    mask = rng.random(shape[-1:] if shared else shape) > 0.5
    if not shared and x.ndim == 2 and shape[0] > 1:
        mask[1] = False
    got = ops.softmax_masked(_dev(x), torch.from_numpy(mask).cuda(), -1e9).cpu().numpy()
    xm = np.where(mask, x, np.float32(-1e9))
    e = np.exp(xm - xm.max(axis=-1, keepdims=True))
    _agree(got, e / e.sum(axis=-1, keepdims=True), 1e-4, 1e-4)
    as_bytes = ops.softmax_masked(_dev(x), torch.from_numpy(mask.astype(np.uint8)).cuda(), -1e9).cpu().numpy()
    assert np.array_equal(as_bytes, got)


def test_softmax_masked_rejects_what_it_does_not_cover():
    from intent_ir_b200 import ops
    from intent_ir_b200.errors import B200LoweringError, B200RuntimeError
    x = torch.zeros(2, 20000, device="cuda")
    with pytest.raises(B200LoweringError):
        ops.softmax_masked(x, torch.ones(2, 20000, dtype=torch.bool, device="cuda"), 0.0)  # rows above 16384 elements
    with pytest.raises(B200RuntimeError):
        ops.softmax_masked(x[:, :8].contiguous(), torch.ones(3, dtype=torch.bool, device="cuda"), 0.0)
    with pytest.raises(B200RuntimeError):
        ops.softmax_masked(x[:, :8].contiguous().half(), torch.ones(8, dtype=torch.bool, device="cuda"), 0.0)


@pytest.mark.parametrize("shape,dims", [((2, 200000), [1]), ((1, 70001), [1]), ((50000, 64), [0]), ((3, 7000, 128), [1]), ((9000, 12), [0]),
                                        ((300, 700), [0, 1])])
@pytest.mark.parametrize("kind", ["sum", "max", "any"])
def test_reduce_with_scratch_matches_the_unsplit_kernels(shape, dims, kind):
    from intent_ir_b200 import _lib, ops
    x = np.random.default_rng(len(shape) + shape[-1]).standard_normal(shape).astype(np.float32)
    if kind == "any":
        x[np.abs(x) < 3.5] = 0
    xd = _dev(x)
    lib = _lib.load()
    outer = int(np.prod(shape[: dims[0]], dtype=np.int64))
    red = int(np.prod(shape[dims[0]: dims[-1] + 1], dtype=np.int64))
    inner = int(np.prod(shape[dims[-1] + 1:], dtype=np.int64))
    assert lib.ib200_reduce_scratch_bytes(outer, red, inner) > 0
    split = ops.reduce(xd, kind, dims).cpu().numpy()
    plain = ops.reduce(xd, kind, dims, split=False).cpu().numpy()
    want = {"sum": np.sum, "max": np.max, "any": lambda a, axis: np.any(a != 0, axis=axis)}[kind](x, axis=tuple(dims))
    if kind == "sum":
        _agree(split, want, 1e-3, 1e-4)
        _agree(plain, want, 1e-3, 1e-4)
    else:
        assert np.array_equal(split, want) and np.array_equal(plain, want)
    assert np.array_equal(split, ops.reduce(xd, kind, dims).cpu().numpy())  # the same bits on every run


def test_reduce_ws_falls_back_without_enough_scratch_and_checks_alignment():
    from intent_ir_b200 import _lib
    lib = _lib.load()
    x = torch.ones(1, 1 << 20, device="cuda")
    out = torch.zeros(1, device="cuda")
    need = lib.ib200_reduce_scratch_bytes(1, 1 << 20, 1)
    assert need > 0 and lib.ib200_reduce_scratch_bytes(4096, 4096, 1) == 0
    small = torch.empty(256, dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert lib.ib200_reduce_ws(x.data_ptr(), out.data_ptr(), _lib.F32, _lib.F32,
                               _lib.REDUCE_SUM, 1, 1 << 20, 1, 1.0, small.data_ptr(), 256, s) == _lib.OK
    assert float(out.cpu()) == float(1 << 20)
    big = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    assert lib.ib200_reduce_ws(x.data_ptr(), out.data_ptr(), 0, 0, _lib.REDUCE_SUM, 1, 1 << 20, 1, 1.0, big.data_ptr() + 4, need, s) != _lib.OK


# ---- the bounded-wait error path, with the failure injected from the host -------------------------------
# No kernel is made to wait: the status word a kernel would have written is written by a host copy.

def test_device_wait_status_surfaces_as_an_exception_and_clears():
    from intent_ir_b200 import ops
    from intent_ir_b200.errors import B200RuntimeError

    a = _dev(np.ones((128, 64), np.float32)).to(torch.bfloat16)
    b = _dev(np.ones((64, 128), np.float32)).to(torch.bfloat16)
    ops.gemm_bias_act(a, b, None, "none")
    ops.check_device_status()  # clean
    ops.status_word().fill_(4)  # "epilogue waiting for a finished accumulator"
    with pytest.raises(B200RuntimeError) as e:
        ops.check_device_status()
    assert "bounded device wait expired" in str(e.value) and "epilogue" in str(e.value)
    c = ops.gemm_bias_act(a, b, None, "none")  # the word was cleared: the next launch is judged on its own
    ops.check_device_status()
    assert float(c.float().min()) == float(c.float().max()) == 64.0
    from intent_ir_b200 import _lib

    lib = _lib.load()
    word = torch.full((1,), 2, dtype=torch.int32, device="cuda")
    assert lib.ib200_check_status(word.data_ptr(), torch.cuda.current_stream().cuda_stream) == _lib.ERR_DEVICE_WAIT
    assert b"MMA issuer" in lib.ib200_last_error()
    word.fill_(77)
    assert lib.ib200_check_status(word.data_ptr(), torch.cuda.current_stream().cuda_stream) == _lib.ERR_DEVICE_WAIT
    assert b"unknown site" in lib.ib200_last_error()


def test_plan_status_word_surfaces_through_check_plan_status(golden_graphs):
    import json as _json

    from intent_ir_b200 import runtime
    from intent_ir_b200.errors import B200RuntimeError
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel

    js = _json.loads(_json.dumps(golden_graphs["matmul_bias_relu2d"]["intent"]))
    for name in ("A", "B", "bias", "C"):
        js["tensors"][name]["dtype"] = "bf16"
    low = lower_intent_to_b200_kernel(js, shape_bindings={"M": 128, "N": 128, "K": 64})
    assert low.status_offset >= 0
    ins = {"A": np.ones((128, 64), np.float32), "B": np.ones((64, 128), np.float32), "bias": np.zeros(128, np.float32)}
    assert float(runtime.run_lowered(low, ins)["C"].max()) == 64.0
    ws = next(w for k, w in runtime._WORKSPACES.items() if k[0] == low.io_spec["plan_id"])
    base = runtime._aligned_ptr(ws) - ws.data_ptr() + low.status_offset
    ws[base: base + 4].view(torch.int32).fill_(1)  # "producer waiting for a free ring stage"
    with pytest.raises(B200RuntimeError) as e:
        runtime.check_plan_status(low)
    assert "ring stage" in str(e.value) and "-5" in str(e.value)
    assert float(runtime.run_lowered(low, ins)["C"].max()) == 64.0  # cleared: the plan runs and checks clean again
    # a plan whose scratch left the cache can no longer be checked, and says so
    for key in [k for k in runtime._WORKSPACES if k[0] == low.io_spec["plan_id"]]:
        del runtime._WORKSPACES[key]
    with pytest.raises(B200RuntimeError) as e:
        runtime.check_plan_status(low)
    assert "can no longer be read" in str(e.value)


# ---- tensor cores for every float operand type, and the K-split tail --------------------------------------

@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 264, 72), (1, 8, 8), (130, 520, 1000), (512, 1024, 2048)])
@pytest.mark.parametrize("transpose_b", [False, True])
def test_gemm_f16_operands_on_tensor_cores(m, n, k, transpose_b):
    from intent_ir_b200 import ops
    rng = np.random.default_rng(m + n + k + 1)
    a = (0.5 * rng.standard_normal((m, k))).astype(np.float16).astype(np.float32)
    b = (0.5 * rng.standard_normal((k, n))).astype(np.float16).astype(np.float32)
    bias = (0.1 * rng.standard_normal(n)).astype(np.float16).astype(np.float32)
    want = np.maximum(a.astype(np.float64) @ b.astype(np.float64) + bias, 0)
    bd = _dev(np.ascontiguousarray(b.T) if transpose_b else b, torch.float16)
    got = ops.gemm_bias_act(_dev(a, torch.float16), bd, _dev(bias, torch.float16), "relu", transpose_b)
    ops.check_device_status()
    assert got.dtype == torch.float16
    _agree(got.float().cpu().numpy(), want, 2e-2, 2e-2)
    got32 = ops.gemm_bias_act(_dev(a, torch.float16), bd, None, "none", transpose_b, out_dtype=torch.float32)
    ops.check_device_status()
    _agree(got32.cpu().numpy(), a.astype(np.float64) @ b.astype(np.float64), 1e-3, 1e-3)  # f16 products are exact in fp32


@pytest.mark.parametrize("m,n,k", [(128, 256, 32), (128, 256, 64), (300, 264, 72), (1, 8, 8), (130, 520, 1000), (512, 1024, 2048)])
@pytest.mark.parametrize("transpose_b", [False, True])
def test_gemm_f32_operands_as_tf32(m, n, k, transpose_b):
    from intent_ir_b200 import ops
    rng = np.random.default_rng(m + n + k + 2)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = (rng.standard_normal((k, n), dtype=np.float32) / np.sqrt(k)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(n)).astype(np.float32)
    want = np.maximum(a.astype(np.float64) @ b.astype(np.float64) + bias, 0)
    bd = _dev(np.ascontiguousarray(b.T) if transpose_b else b)
    got = ops.gemm_bias_act(_dev(a), bd, _dev(bias), "relu", transpose_b, allow_tf32=True)
    ops.check_device_status()
    _agree(got.cpu().numpy(), want, 2e-2, 2e-2)  # the verifier's matmul tolerance
    # TF32 keeps 10 mantissa bits: the result must differ from the exact-FMA kernel's, or the flag did nothing
    exact = ops.gemm_bias_act(_dev(a), bd, _dev(bias), "relu", transpose_b)
    _agree(exact.cpu().numpy(), want, 1e-4, 1e-4)
    if k >= 64:
        assert not torch.equal(got, exact)
    # operands exactly representable in TF32 give the exact product
    a8 = np.round(a * 8) / 8
    b8 = np.round(b * 64) / 64
    b8d = _dev(np.ascontiguousarray(b8.T if transpose_b else b8).astype(np.float32))
    got8 = ops.gemm_bias_act(_dev(a8.astype(np.float32)), b8d, None, "none", transpose_b, allow_tf32=True)
    _agree(got8.cpu().numpy(), a8.astype(np.float64) @ b8.astype(np.float64), 1e-5, 1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("m,n,k,transpose_b", [(128 * 20, 256 * 10, 2048, False),  # 200 tiles: one full round + 52 tiles split in two
                                                (128 * 5, 256 * 6, 4096, True),     # 30 tiles, all split in four
                                                (640 + 3, 1536 - 8, 2048 + 8, False),  # ragged M, N, K
                                                (4096, 4096, 2048, False)])         # 512 tiles: three rounds + 68 split in two
def test_gemm_tail_tiles_split_along_k(dtype, m, n, k, transpose_b):
    from intent_ir_b200 import _lib, ops
    rng = np.random.default_rng(m + n + k + 3)
    a = _bf16_round(rng.standard_normal((m, k)).astype(np.float32) * 0.5)
    b = _bf16_round((rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32))
    bias = _bf16_round((0.1 * rng.standard_normal(n)).astype(np.float32))
    lib = _lib.load()
    code = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}[dtype]
    tf32 = dtype == torch.float32
    assert lib.ib200_gemm_scratch_bytes(code, code, m, n, k, 1, _lib.GEMM_ONE_CTA | (_lib.GEMM_ALLOW_TF32 if tf32 else 0)) > 0
    ad, bd, biasd = _dev(a, dtype), _dev(np.ascontiguousarray(b.T) if transpose_b else b, dtype), _dev(bias, dtype)
    split = ops.gemm_bias_act(ad, bd, biasd, "relu", transpose_b, allow_tf32=tf32, split_tail=True, cta_pairs=False)
    ops.check_device_status()
    whole = ops.gemm_bias_act(ad, bd, biasd, "relu", transpose_b, allow_tf32=tf32, split_tail=False, cta_pairs=False)
    ops.check_device_status()
    again = ops.gemm_bias_act(ad, bd, biasd, "relu", transpose_b, allow_tf32=tf32, split_tail=True, cta_pairs=False)  # tickets were left at zero
    ops.check_device_status()
    assert torch.equal(split, again)  # slices are added in slice order: the same bits on every run
    want = np.maximum(a.astype(np.float64) @ b.astype(np.float64) + bias, 0)
    _agree(split.float().cpu().numpy(), want, 2e-2, 2e-2)
    _agree(whole.float().cpu().numpy(), want, 2e-2, 2e-2)
    # bf16 / f16 products are exact and both kernels accumulate in fp32: split and whole agree to accumulation order
    assert float((split.float() - whole.float()).abs().max()) <= (2e-2 if dtype != torch.float32 else 1e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("m,n,k,transpose_b", [(256, 256, 64, False), (256, 256, 512, True), (512, 768, 1024, False), (300, 264, 72, False),
                                                (130, 520, 1000, True), (1, 8, 8, False), (2048, 2048, 2048, False), (4096, 1024, 512, True),
                                                (2560, 2048, 256, False), (2500, 2056, 136, True)])  # (the last two leave a short last round)
def test_gemm_on_cta_pairs(dtype, m, n, k, transpose_b):
    """tcgen05 cta_group::2: two CTAs share a 256 x 256 tile, each staging half of the operands."""
    from intent_ir_b200 import ops
    rng = np.random.default_rng(m + n + k + 4)
    a = _bf16_round((0.5 * rng.standard_normal((m, k))).astype(np.float32))
    b = _bf16_round((rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32))
    bias = _bf16_round((0.1 * rng.standard_normal(n)).astype(np.float32))
    tf32 = dtype == torch.float32
    ad, bd, biasd = _dev(a, dtype), _dev(np.ascontiguousarray(b.T) if transpose_b else b, dtype), _dev(bias, dtype)
    got = ops.gemm_bias_act(ad, bd, biasd, "relu", transpose_b, allow_tf32=tf32, cta_pairs=True)
    ops.check_device_status()
    want = np.maximum(a.astype(np.float64) @ b.astype(np.float64) + bias, 0)
    _agree(got.float().cpu().numpy(), want, 2e-2, 2e-2)
    if not tf32 or transpose_b:  # (a [K,N] TF32 operand needs scratch for its transpose, which split_tail=False withholds)
        lone = ops.gemm_bias_act(ad, bd, biasd, "relu", transpose_b, allow_tf32=tf32, split_tail=False, cta_pairs=False)
        ops.check_device_status()
        # products of bf16-representable values are exact in every operand kind and both kernels accumulate in fp32 in
        # K order: the pair kernel gives the one-CTA kernel's bits
        assert torch.equal(got, lone)
    # the last round's tiles as half-width units (taken when they fill at most half of the pairs): the same bits again
    narrow = ops.gemm_bias_act(ad, bd, biasd, "relu", transpose_b, allow_tf32=tf32, cta_pairs=True, narrow_tail=True)
    ops.check_device_status()
    assert torch.equal(got, narrow)
