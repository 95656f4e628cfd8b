"""End-to-end parity through the drop-in boundary: IntentIR JSON -> lower_intent_to_b200_kernel
-> run_b200_kernel (ctypes -> C ABI -> sm_100a kernels) against

  * the reference interpreter's own outputs (tests/golden, generated from the reference), and
  * the CPU oracle's run_diff over generated edge-size cases,

bit-exact for boolean / integer results and within the oracle's inferred tolerances
(verify/tolerances.py) for floating point.  The tests read like the reference's
tests/backends/cuda/test_cuda_backend_smoke.py."""

import json
import os

import numpy as np
import pytest

from intent_ir_b200.ir import IntentFunction
from oracle import TestCase, execute_intent, generate_cases, infer_tolerances, run_diff
from oracle.diff import compare_outputs, derive_bindings

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
with open(os.path.join(GOLDEN, "intents.json")) as _f:
    _GRAPHS = json.load(_f)
KEYS = sorted(_GRAPHS)


def _lower_and_run(intent, bindings, inputs):
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel
    from intent_ir_b200.runtime import run_b200_kernel

    lowered = lower_intent_to_b200_kernel(intent, shape_bindings=bindings)
    return run_b200_kernel(kernel_name=lowered.kernel_name, cuda_src=lowered.cuda_src, io_spec=lowered.io_spec,
                           launch=lowered.launch, bindings=lowered.bindings, inputs_np=inputs,
                           output_names=lowered.output_names), lowered


def _agree(got, want, tol, name=""):
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    if want.dtype == np.bool_ or want.dtype.kind in "iu":
        assert np.array_equal(got.astype(want.dtype), want), f"{name}: exact mismatch"
        return
    gn, wn = np.isnan(got), np.isnan(want)
    assert np.array_equal(gn, wn), f"{name}: NaN pattern differs"
    if gn.any():
        got, want = np.where(gn, 0, got), np.where(wn, 0, want)
    d = compare_outputs({"y": want}, {"y": got}, ["y"], tol)
    assert d.ok, (name, d.summary, d.max_abs_err, d.first_bad_index)


@pytest.mark.parametrize("key", KEYS)
def test_golden_graph_matches_reference_interpreter(key, golden_graphs, golden_vectors, golden_verdicts):
    g = golden_graphs[key]
    intent = IntentFunction.from_json_dict(g["intent"])
    inputs = {n: golden_vectors[f"{key}/in/{n}"] for n in g["inputs"]}
    out, lowered = _lower_and_run(intent, g["shapes"], inputs)
    tol = golden_verdicts[key]["tol_decl"]
    for name in g["outputs"]:
        _agree(out[name], golden_vectors[f"{key}/out/{name}"], tol, f"{key}/{name}")
    for name in inputs:  # the runner returns inputs as well (frontends/cuda/runtime.py:1028)
        assert name in out


@pytest.mark.parametrize("key", ["any_kernel_dim", "softmax_inner", "softmax_inner__cuda_pipeline_form", "layer_norm_persistent",
                                 "layer_norm_persistent__cuda_pipeline_form", "group_norm_kernel", "matmul_bias_relu2d",
                                 "add_bias2d", "where2d", "row_sum", "row_max", "clamp2d", "rms_norm2d", "mlp2d",
                                 "masked_softmax2d", "layer_norm_residual2d", "transpose2d", "grouped_row_sum2d"])
def test_run_diff_over_generated_edge_cases(key, golden_graphs):
    """verify.diff_runner.run_diff with the B200 backend as run_ref_fn, over the deterministic
    edge-size grid of verify.gen_cases ({1,2,3} U {t-1,t,t+1,2t+1} per axis)."""
    from intent_ir_b200.backend import make_run_ref_fn

    g = golden_graphs[key]
    intent = IntentFunction.from_json_dict(g["intent"])
    base = dict(g["shapes"])
    cases = []
    for c in generate_cases(intent, limit=24, seed=7):
        shapes = {**base, **c.shapes}
        if key == "group_norm_kernel":
            shapes["C"] = shapes["num_groups"] * shapes["group_size"]  # the generator varies both freely
        if key == "grouped_row_sum2d":
            shapes["N"] = shapes["group_size"] * max(1, shapes["N"] // shapes["group_size"])
        cases.append(TestCase(shapes=shapes, dtypes={}, seed=c.seed + len(cases)))
    cases.append(TestCase(shapes=base, dtypes={}, seed=1))
    run = make_run_ref_fn(intent)
    diffs, cex = run_diff(intent, run, cases, tolerances=infer_tolerances(intent).to_dict())
    bad = [(c.case.shapes, c.diff.summary, c.diff.max_abs_err) for c in cex]
    assert not bad, bad[:3]
    assert len(diffs) == len(cases) and all(d.ok for d in diffs)


def test_mismatching_runner_is_caught():
    """The reference's tests/test_diff_runner.py:55-70 with the backend in the loop: corrupt
    one output element after the GPU run and the diff must produce a counterexample."""
    from intent_ir_b200.backend import make_run_ref_fn

    intent = IntentFunction.from_json_dict(_GRAPHS["matmul_bias_relu2d"]["intent"])
    run = make_run_ref_fn(intent)

    def corrupted(case):
        io = run(case)
        io["C"] = io["C"].copy()
        io["C"][0, 0] += 5.0
        return io

    diffs, cex = run_diff(intent, corrupted, [TestCase(shapes={"M": 4, "N": 8, "K": 8}, dtypes={}, seed=0)])
    assert not diffs[0].ok and cex


# ---- the reference's backend smoke tests, against this backend -----------------------------

def _smoke(js, bindings, inputs):
    out, _ = _lower_and_run(IntentFunction.from_json_dict(js), bindings, inputs)
    return out


def _t(shape, dtype="f32"):
    return {"dtype": dtype, "shape": shape, "layout": "row_major"}


def test_smoke_matmul_matches_numpy():
    js = {"name": "mm_smoke", "tensors": {"A": _t(["M", "K"]), "B": _t(["K", "N"]), "C": _t(["M", "N"])},
          "ops": [{"op": "matmul", "inputs": ["A", "B"], "output": "C", "attrs": {}}], "outputs": ["C"],
          "parallel_axes": ["M", "N"], "schedule": {"tile_m": 8, "tile_n": 16, "tile_k": 16, "parallel_axes": ["M", "N"]}}
    M, N, K = 32, 48, 16
    rng = np.random.default_rng(0)
    A, B = rng.standard_normal((M, K), dtype=np.float32), rng.standard_normal((K, N), dtype=np.float32)
    got = _smoke(js, {"M": M, "N": N, "K": K}, {"A": A, "B": B})["C"]
    np.testing.assert_allclose(got, A @ B, rtol=1e-4, atol=1e-4)


def test_smoke_fused_elementwise_broadcast_relu():
    js = {"name": "ew_smoke", "tensors": {"A": _t(["M", "N"]), "B": _t(["N"]), "T": _t(["M", "N"]), "Out": _t(["M", "N"])},
          "ops": [{"op": "add", "inputs": ["A", "B"], "output": "T", "attrs": {}},
                  {"op": "relu", "inputs": ["T"], "output": "Out", "attrs": {}}], "outputs": ["Out"]}
    rng = np.random.default_rng(0)
    A, B = rng.standard_normal((8, 16), dtype=np.float32), rng.standard_normal(16, dtype=np.float32)
    got = _smoke(js, {"M": 8, "N": 16}, {"A": A, "B": B})["Out"]
    np.testing.assert_allclose(got, np.maximum(A + B[None, :], 0), rtol=1e-5, atol=1e-5)


def test_smoke_transpose_row_sum_row_max_any():
    rng = np.random.default_rng(0)
    A = rng.standard_normal((16, 8), dtype=np.float32)
    js = {"name": "tr", "tensors": {"A": _t(["M", "N"]), "B": _t(["N", "M"])},
          "ops": [{"op": "transpose", "inputs": ["A"], "output": "B", "attrs": {"perm": [1, 0]}}], "outputs": ["B"]}
    assert np.array_equal(_smoke(js, {"M": 16, "N": 8}, {"A": A})["B"], A.T)
    for op, ref in (("reduce_sum", A.sum(axis=1)), ("reduce_max", A.max(axis=1))):
        js = {"name": op, "tensors": {"A": _t(["M", "N"]), "S": _t(["M"])},
              "ops": [{"op": op, "inputs": ["A"], "output": "S", "attrs": {"dims": [1]}}], "outputs": ["S"]}
        np.testing.assert_allclose(_smoke(js, {"M": 16, "N": 8}, {"A": A})["S"], ref, rtol=1e-6, atol=1e-6)
    Z = rng.integers(0, 2, size=(8, 8)).astype(np.float32) * (rng.random((8, 8)) < 0.2)
    js = {"name": "any", "tensors": {"A": _t(["M", "N"]), "z": _t([]), "T": _t(["M", "N"], "i1"), "Out": _t(["M"], "i1")},
          "ops": [{"op": "const", "inputs": [], "output": "z", "attrs": {"value": 0.0}},
                  {"op": "ne", "inputs": ["A", "z"], "output": "T", "attrs": {}},
                  {"op": "reduce_any", "inputs": ["T"], "output": "Out", "attrs": {"dims": [1]}}], "outputs": ["Out"]}
    got = _smoke(js, {"M": 8, "N": 8}, {"A": Z.astype(np.float32)})["Out"]
    assert got.dtype == np.bool_ and np.array_equal(got, np.any(Z != 0, axis=1))


# ---- headline configurations at full size ------------------------------------------------------------------

def test_config_reduce_any_16x256(golden_graphs):
    intent = IntentFunction.from_json_dict(golden_graphs["any_kernel_dim"]["intent"])
    rng = np.random.default_rng(0)
    x = np.where(rng.random((16, 256)) < 0.05, rng.standard_normal((16, 256), dtype=np.float32), np.float32(0))
    out, lowered = _lower_and_run(intent, {"M": 16, "N": 256}, {"inp": x})
    assert lowered.n_launches == 1
    assert np.array_equal(out["out"], execute_intent(intent, {"inp": x})["out"])


def test_config_softmax_4096x4096(golden_graphs):
    intent = IntentFunction.from_json_dict(golden_graphs["softmax_inner"]["intent"])
    x = 3 * np.random.default_rng(1).standard_normal((4096, 4096), dtype=np.float32)
    out, lowered = _lower_and_run(intent, {"M": 4096, "N": 4096}, {"input_ptr": x})
    assert [s["kernel"] for s in lowered.steps] == ["softmax"]
    want = execute_intent(intent, {"input_ptr": x})["output_ptr"]
    _agree(out["output_ptr"], want, {"atol": 1e-4, "rtol": 1e-4}, "softmax")  # 1-op softmax: (1e-4, 1e-4)


def test_config_layernorm_8192x4096(golden_graphs):
    intent = IntentFunction.from_json_dict(golden_graphs["layer_norm_persistent"]["intent"])
    rng = np.random.default_rng(2)
    M, N = 8192, 4096
    x = rng.standard_normal((M, N), dtype=np.float32)
    w = rng.uniform(0.5, 1.5, N).astype(np.float32)
    b = (0.1 * rng.standard_normal(N)).astype(np.float32)
    out, lowered = _lower_and_run(intent, {"M": M, "N": N}, {"in_ptr": x, "weight_ptr": w, "bias_ptr": b})
    assert [s["kernel"] for s in lowered.steps] == ["layernorm"]
    # the oracle on the whole tensor, at the verifier's own tolerance for this graph ...
    with np.errstate(all="ignore"):
        want = execute_intent(intent, {"in_ptr": x, "weight_ptr": w, "bias_ptr": b}, {"M": M, "N": N})
    tol = infer_tolerances(intent).to_dict()
    _agree(out["out_ptr"], want["out_ptr"], tol, "y")
    _agree(out["out_mean_ptr"], want["out_mean_ptr"], tol, "mean")
    _agree(out["out_rstd_ptr"], want["out_rstd_ptr"], tol, "rstd")
    # ... and size-independent properties on all of them: (y - b)/w has zero mean and unit variance
    z = (out["out_ptr"].astype(np.float64) - b) / w
    assert np.abs(z.mean(axis=1)).max() < 1e-4
    assert np.abs(z.var(axis=1) - 1.0).max() < 1e-3
    assert np.allclose(out["out_mean_ptr"], x.mean(axis=1, dtype=np.float64), atol=1e-5)


def test_config_groupnorm_32x256x4096(golden_graphs):
    intent = IntentFunction.from_json_dict(golden_graphs["group_norm_kernel"]["intent"])
    rng = np.random.default_rng(4)
    shapes = {"N": 32, "C": 256, "HW": 4096, "num_groups": 32}
    x = rng.standard_normal((32, 256, 4096), dtype=np.float32)
    w = rng.standard_normal(256, dtype=np.float32)
    b = rng.standard_normal(256, dtype=np.float32)
    out, lowered = _lower_and_run(intent, shapes, {"X": x, "W": w, "B": b})
    assert [s["kernel"] for s in lowered.steps] == ["groupnorm"]
    with np.errstate(all="ignore"):  # the oracle on all 32 samples
        want = execute_intent(intent, {"X": x, "W": w, "B": b}, derive_bindings(shapes))
    tol = infer_tolerances(intent).to_dict()
    _agree(out["Y"], want["Y"], tol, "Y")
    _agree(out["Mean"], want["Mean"], tol, "Mean")
    _agree(out["Rstd"], want["Rstd"], tol, "Rstd")
    x4 = x.reshape(32, 32, 8 * 4096)
    assert np.allclose(out["Mean"], x4.mean(axis=2, dtype=np.float64), atol=1e-5)
    assert np.allclose(out["Rstd"], 1.0 / np.sqrt(x4.var(axis=2, dtype=np.float64) + 1e-5), rtol=1e-4)


def test_config_matmul_bias_relu_bf16_4096(golden_graphs):
    from intent_ir_b200.backend import round_to_bf16

    js = json.loads(json.dumps(golden_graphs["matmul_bias_relu2d"]["intent"]))
    for name in ("A", "B", "bias", "C"):
        js["tensors"][name]["dtype"] = "bf16"
    js["ops"][0]["attrs"] = {"accum_dtype": "f32"}
    intent = IntentFunction.from_json_dict(js)
    rng = np.random.default_rng(3)
    n = 4096
    A = round_to_bf16(0.02 * rng.standard_normal((n, n), dtype=np.float32))
    B = round_to_bf16(0.02 * rng.standard_normal((n, n), dtype=np.float32))
    bias = round_to_bf16(0.1 * rng.standard_normal(n, dtype=np.float32))
    out, lowered = _lower_and_run(intent, {"M": n, "N": n, "K": n}, {"A": A, "B": B, "bias": bias})
    assert [s["kernel"] for s in lowered.steps] == ["gemm+bias+relu(cta pairs)"]  # 256 x 256 tiles on pairs of CTAs (tcgen05 cta_group::2)
    want = execute_intent(intent, {"A": A, "B": B, "bias": bias})["C"]  # float32-carried bf16 values
    tol = infer_tolerances(intent).to_dict()
    assert tol == {"atol": 2e-2, "rtol": 2e-2}
    _agree(out["C"], want, tol, "C")
    # tighter than the verifier asks: bf16 rounding of an fp32-accumulated result
    assert np.abs(out["C"] - want).max() <= 2.0 ** -8 * np.abs(want).max() + 1e-6


# ---- error behaviour ---------------------------------------------------------------------------

def _t0(shape, dtype="f32"):
    return {"dtype": dtype, "shape": shape, "layout": "row_major"}


@pytest.mark.parametrize("name,js", [
    ("rank-1", {"name": "m", "tensors": {"a": _t0(["M"]), "b": _t0(["M", "N"]), "y": _t0(["N"])},
                "ops": [{"op": "matmul", "inputs": ["a", "b"], "output": "y"}], "outputs": ["y"]}),
    ("gather", {"name": "g", "tensors": {"x": _t0(["M", "N"]), "i": _t0(["M"], "i32"), "y": _t0(["M"])},
                "ops": [{"op": "gather", "inputs": ["x", "i"], "output": "y"}], "outputs": ["y"]}),  # fewer index tensors than data axes
])
def test_uncovered_graphs_fail_loudly(name, js):
    from intent_ir_b200.errors import B200LoweringError
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel

    with pytest.raises(B200LoweringError) as e:
        lower_intent_to_b200_kernel(IntentFunction.from_json_dict(js), shape_bindings={"S": 4, "B": 2, "H": 2, "D": 8, "D2": 4, "M": 8, "N": 8})
    assert name in str(e.value)


def test_gather_wraps_negative_indices_and_fills_out_of_range(golden_graphs):
    js = json.loads(json.dumps(golden_graphs["gather2d"]["intent"]))
    js["ops"][0]["attrs"] = {"other_value": -1.0}
    rng = np.random.default_rng(0)
    A = rng.standard_normal((7, 9), dtype=np.float32)
    row = rng.integers(-9, 9, size=32).astype(np.int32)
    col = rng.integers(-11, 11, size=32).astype(np.int32)
    out, _ = _lower_and_run(IntentFunction.from_json_dict(js), {"M": 7, "N": 9, "L": 32}, {"inp": A, "row_idx": row, "col_idx": col})
    want = np.full(32, -1.0, np.float32)
    for i in range(32):
        if -7 <= row[i] < 7 and -9 <= col[i] < 9:
            want[i] = A[row[i], col[i]]  # numpy semantics where numpy accepts the index
    assert np.array_equal(out["out"], want)


def test_missing_input_and_wrong_shape_raise(golden_graphs):
    from intent_ir_b200.errors import B200RuntimeError
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel
    from intent_ir_b200.runtime import run_b200_kernel

    g = golden_graphs["add2d"]
    lowered = lower_intent_to_b200_kernel(IntentFunction.from_json_dict(g["intent"]), shape_bindings={"M": 4, "N": 4})
    kw = dict(kernel_name=lowered.kernel_name, cuda_src="", io_spec=lowered.io_spec, launch=lowered.launch,
              bindings=lowered.bindings, output_names=lowered.output_names)
    with pytest.raises(B200RuntimeError, match="missing input"):
        run_b200_kernel(inputs_np={"A": np.zeros((4, 4), np.float32)}, **kw)
    with pytest.raises(B200RuntimeError, match="shape"):
        run_b200_kernel(inputs_np={"A": np.zeros((4, 5), np.float32), "B": np.zeros((4, 4), np.float32)}, **kw)


@pytest.mark.parametrize("m,n,dtype", [(2048, 2048, "f32"), (1536, 4100, "f32"), (3000, 1024, "bf16"), (1031, 2053, "f32"),
                                         (1000, 520, "f16"), (77, 36, "bf16"), (515, 1027, "bf16")])
def test_large_broadcast_chain_matches_oracle(m, n, dtype):
    """Large enough for the 16-elements-per-thread staging (and a ragged shape that is not)."""
    from intent_ir_b200.backend import round_to_bf16

    t = lambda s, d=dtype: {"dtype": d, "shape": s, "layout": "row_major"}  # noqa: E731
    js = {"name": "chain", "tensors": {"x": t(["M", "N"]), "col": t(["N"]), "row": t(["M", 1]), "y": t(["M", "N"], "f32")},
          "ops": [{"op": "mul", "inputs": ["x", "col"], "output": "a"}, {"op": "add", "inputs": ["a", "row"], "output": "b"},
                  {"op": "mul", "inputs": ["b"], "output": "c", "attrs": {"mul_factor": 0.5}},
                  {"op": "sub", "inputs": ["c", "col"], "output": "d"}, {"op": "mul", "inputs": ["d", "d"], "output": "e"},
                  {"op": "max", "inputs": ["e", "x"], "output": "y"}], "outputs": ["y"]}
    intent = IntentFunction.from_json_dict(js)
    rng = np.random.default_rng(m + n)
    q = {"bf16": round_to_bf16, "f16": lambda a: a.astype(np.float16).astype(np.float32), "f32": lambda a: a}[dtype]
    ins = {"x": q(rng.standard_normal((m, n), dtype=np.float32)), "col": q(rng.standard_normal(n, dtype=np.float32)),
           "row": q(rng.standard_normal((m, 1), dtype=np.float32))}
    out, lowered = _lower_and_run(intent, {"M": m, "N": n}, ins)
    assert lowered.n_launches == 1
    want = execute_intent(intent, ins, {"M": m, "N": n})["y"]
    _agree(out["y"], want, infer_tolerances(intent).to_dict(), "y")


def test_softmax_bf16_input_f32_output(golden_graphs):
    from intent_ir_b200.backend import round_to_bf16

    js = json.loads(json.dumps(golden_graphs["softmax_inner"]["intent"]))
    js["tensors"]["input_ptr"]["dtype"] = "bf16"
    intent = IntentFunction.from_json_dict(js)
    x = round_to_bf16(3 * np.random.default_rng(8).standard_normal((300, 31), dtype=np.float32))
    out, lowered = _lower_and_run(intent, {"M": 300, "N": 31}, {"input_ptr": x})
    assert [s["kernel"] for s in lowered.steps] == ["softmax"]
    want = execute_intent(intent, {"input_ptr": x})["output_ptr"]
    assert (want > 0.5).any()  # the regime a bf16 result could not meet
    _agree(out["output_ptr"], want, infer_tolerances(intent).to_dict(), "softmax bf16->f32")


# ---- stage-C style checks through the same runner (verify/metamorphic.py) --------------------

def _runner(key, golden_graphs):
    from intent_ir_b200.backend import make_run_ref_fn

    intent = IntentFunction.from_json_dict(golden_graphs[key]["intent"])
    return intent, make_run_ref_fn(intent)


def test_metamorphic_relations(golden_graphs):
    rng = np.random.default_rng(12)
    # any: invariant under a column permutation (metamorphic.py:309-329)
    intent, run = _runner("any_kernel_dim", golden_graphs)
    x = np.where(rng.random((40, 300)) < 0.01, np.float32(1), np.float32(0))
    base = run(TestCase(shapes={"M": 40, "N": 300}, dtypes={}, seed=0, inputs={"inp": x}))["out"]
    perm = run(TestCase(shapes={"M": 40, "N": 300}, dtypes={}, seed=0, inputs={"inp": x[:, rng.permutation(300)]}))["out"]
    assert np.array_equal(base, perm) and base.any() and not base.all()
    # softmax: shift invariance and column reversal (:360-420)
    intent, run = _runner("softmax_inner", golden_graphs)
    x = rng.standard_normal((33, 500), dtype=np.float32)
    case = lambda a: TestCase(shapes={"M": 33, "N": 500}, dtypes={}, seed=0, inputs={"input_ptr": a})  # noqa: E731
    y0 = run(case(x))["output_ptr"]
    assert np.allclose(run(case(x + np.float32(0.37)))["output_ptr"], y0, atol=1e-4, rtol=1e-4)
    assert np.allclose(run(case(x[:, ::-1].copy()))["output_ptr"][:, ::-1], y0, atol=1e-6, rtol=1e-6)
    # layernorm / groupnorm: Y and rstd invariant under a shift of the input, mean shifts (:330-358, :460-482)
    intent, run = _runner("layer_norm_persistent", golden_graphs)
    w, b = rng.standard_normal(700, dtype=np.float32), rng.standard_normal(700, dtype=np.float32)
    x = rng.standard_normal((20, 700), dtype=np.float32)
    case = lambda a: TestCase(shapes={"M": 20, "N": 700}, dtypes={}, seed=0, inputs={"in_ptr": a, "weight_ptr": w, "bias_ptr": b})  # noqa: E731
    o0, o1 = run(case(x)), run(case(x + np.float32(0.37)))
    assert np.allclose(o0["out_ptr"], o1["out_ptr"], atol=1e-3, rtol=1e-3)
    assert np.allclose(o0["out_mean_ptr"] + 0.37, o1["out_mean_ptr"], atol=1e-3) and np.allclose(o0["out_rstd_ptr"], o1["out_rstd_ptr"], rtol=1e-3)
    intent, run = _runner("group_norm_kernel", golden_graphs)
    shapes = {"N": 3, "C": 16, "HW": 4608, "num_groups": 2}  # rows of 36864 elements: the clustered kernel
    x = rng.standard_normal((3, 16, 4608), dtype=np.float32)
    w, b = rng.standard_normal(16, dtype=np.float32), rng.standard_normal(16, dtype=np.float32)
    case = lambda a: TestCase(shapes=shapes, dtypes={}, seed=0, inputs={"X": a, "W": w, "B": b})  # noqa: E731
    o0, o1 = run(case(x)), run(case(x + np.float32(0.37)))
    assert np.allclose(o0["Y"], o1["Y"], atol=1e-3, rtol=1e-3)
    assert np.allclose(o0["Mean"] + 0.37, o1["Mean"], atol=1e-3) and np.allclose(o0["Rstd"], o1["Rstd"], rtol=1e-3)


def test_bounded_exhaustive_tiny_domains(golden_graphs):
    """Every input over a tiny domain, as verify/metamorphic.py:664-701 enumerates them."""
    from itertools import product

    def sweep(key, shapes, name, shape, domain, fixed):
        intent, run = _runner(key, golden_graphs)
        cases = [TestCase(shapes=shapes, dtypes={}, seed=0, inputs={**fixed, name: np.array(v, np.float32).reshape(shape)})
                 for v in product(domain, repeat=int(np.prod(shape)))]
        diffs, cex = run_diff(intent, run, cases, tolerances=infer_tolerances(intent).to_dict())
        assert len(diffs) == len(cases) and all(d.ok for d in diffs), [(c.case.inputs[name].tolist(), c.diff.summary) for c in cex[:3]]

    sweep("any_kernel_dim", {"M": 2, "N": 3}, "inp", (2, 3), [0.0, 1.0], {})
    sweep("softmax_inner", {"M": 1, "N": 2}, "input_ptr", (1, 2), [-1.0, 0.0, 1.0], {})
    one2 = np.ones(2, np.float32)
    sweep("layer_norm_persistent", {"M": 1, "N": 2}, "in_ptr", (1, 2), [-1.0, 0.0, 1.0], {"weight_ptr": one2, "bias_ptr": 0 * one2})
    sweep("group_norm_kernel", {"N": 1, "C": 2, "HW": 2, "num_groups": 2}, "X", (1, 2, 2), [-1.0, 0.0, 1.0], {"W": one2, "B": 0 * one2})


def test_bound_graphed_and_pipelined_launchers_agree_with_the_plain_runner(golden_graphs):
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel
    from intent_ir_b200.runtime import HostPipeline, bind_lowered, graph_lowered, run_lowered

    intent = IntentFunction.from_json_dict(golden_graphs["mlp2d"]["intent"])  # a multi-kernel plan with a workspace
    shapes = {"M": 64, "K": 96, "H": 192, "N": 48}
    lowered = lower_intent_to_b200_kernel(intent, shape_bindings=shapes)
    assert lowered.n_launches > 1 and lowered.workspace_bytes > 0
    rng = np.random.default_rng(2)
    specs, outs = lowered.io_spec["tensors"], lowered.output_names

    def inputs():
        return {n: rng.standard_normal([int(d) for d in specs[n]["shape"]]).astype(np.float32)
                for n in lowered.io_spec["arg_names"] if n not in outs}

    a, b = inputs(), inputs()
    want_a, want_b = run_lowered(lowered, a), run_lowered(lowered, b)
    dev = {k: torch.from_numpy(v).cuda() for k, v in a.items()}
    launch, res = bind_lowered(lowered, dev)
    launch()
    torch.cuda.synchronize()
    for n in outs:
        assert np.array_equal(res[n].cpu().numpy(), want_a[n])
    replay, gres = graph_lowered(lowered, dev)
    for k, v in b.items():
        dev[k].copy_(torch.from_numpy(v))
    replay()
    torch.cuda.synchronize()
    for n in outs:
        assert np.array_equal(gres[n].cpu().numpy(), want_b[n])
    pipe = HostPipeline(lowered, depth=2)
    host_in = [{k: torch.from_numpy(v).pin_memory() for k, v in d.items()} for d in (a, b, a)]
    host_out = [{n: torch.empty([int(d) for d in specs[n]["shape"]], dtype=torch.float32).pin_memory() for n in outs} for _ in range(3)]
    for i in range(3):
        pipe.submit(host_in[i], host_out[i])
    pipe.wait()
    for i, want in enumerate((want_a, want_b, want_a)):
        for n in outs:
            assert np.array_equal(host_out[i][n].numpy(), want[n]), (i, n)


@pytest.mark.parametrize("key,primary,shapes", [
    ("softmax_inner", "input_ptr", {"M": 9, "N": 300}),
    ("layer_norm_persistent", "in_ptr", {"M": 9, "N": 300}),
    ("group_norm_kernel", "X", {"N": 2, "C": 8, "HW": 40, "num_groups": 2}),
    ("matmul_bias_relu2d", "A", {"M": 16, "N": 24, "K": 40}),
    ("add_bias2d", "inp", {"M": 9, "N": 300}),
    ("row_max", "inp", {"M": 9, "N": 300}),
])
def test_numerical_stability_probes(key, primary, shapes, golden_graphs):
    """The three probes of verify/numerical_stability.py:136-164 — a NaN, a +Inf/-Inf pair and a
    1e4 scale injected into the primary input — with NaN positions compared explicitly (the
    reference's comparison cannot accept any NaN) and everything else through the oracle."""
    from intent_ir_b200.backend import default_inputs, make_run_ref_fn

    intent = IntentFunction.from_json_dict(golden_graphs[key]["intent"])
    bindings = derive_bindings(shapes)
    base = default_inputs(intent, bindings, seed=4)
    run = make_run_ref_fn(intent)
    tol = infer_tolerances(intent).to_dict()
    probes = {}
    m = base[primary].copy(); m.reshape(-1)[0] = np.nan; probes["nan"] = m
    m = base[primary].copy(); m.reshape(-1)[0] = np.inf; m.reshape(-1)[1] = -np.inf; probes["inf"] = m
    probes["scale_1e4"] = (base[primary] * np.float32(1e4)).astype(np.float32)
    for tag, arr in probes.items():
        ins = {**base, primary: arr}
        got = run(TestCase(shapes=shapes, dtypes={}, seed=4, inputs=ins))
        with np.errstate(all="ignore"):
            want = execute_intent(intent, ins, bindings)
        for name in intent.outputs:
            _agree(got[name], want[name], tol, f"{key}/{tag}/{name}")


def test_mutants_are_killed(golden_graphs):
    """verify/mutation.py in miniature: the interpreter runs a wrong variant of the graph, the
    backend runs the original, and the diff must reject every mutant."""
    from intent_ir_b200.backend import make_run_ref_fn

    def mutate(js, fn):
        js = json.loads(json.dumps(js))
        fn(js)
        return IntentFunction.from_json_dict(js)

    ln = golden_graphs["layer_norm_persistent"]["intent"]
    mm = golden_graphs["matmul_bias_relu2d"]["intent"]
    sm = golden_graphs["softmax_inner__cuda_pipeline_form"]["intent"]
    mutants = [
        (ln, {"M": 8, "N": 64}, lambda j: j["ops"][6]["attrs"].update(value=1e-1)),                      # eps
        (ln, {"M": 8, "N": 64}, lambda j: j["ops"][2].update(inputs=list(reversed(j["ops"][2]["inputs"])))),  # mean - x
        (ln, {"M": 8, "N": 64}, lambda j: j["ops"][13].update(op="sub")),                                # - bias
        (mm, {"M": 8, "N": 16, "K": 24}, lambda j: j["ops"][3].update(op="abs")),                         # relu -> abs
        (mm, {"M": 8, "N": 16, "K": 24}, lambda j: j["ops"][2].update(op="sub")),                         # - bias
        (sm, {"M": 8, "N": 64}, lambda j: j["ops"][6].update(op="mul")),                                  # div -> mul
    ]
    for original, shapes, fn in mutants:
        run = make_run_ref_fn(IntentFunction.from_json_dict(original))
        mutant = mutate(original, fn)
        diffs, cex = run_diff(mutant, run, [TestCase(shapes=shapes, dtypes={}, seed=3)], tolerances=infer_tolerances(mutant).to_dict())
        assert not diffs[0].ok and cex, mutant.ops


# ---- pipeline report artefacts replayed on the GPU (scripts/backend_codegen_smoke.py:81-218) -------

@pytest.mark.parametrize("key", ["softmax_inner", "group_norm_kernel", "_attn_fwd", "layer_norm_persistent", "any_kernel_dim",
                                 "rms_norm_residual2d", "masked_softmax2d", "mlp2d"])
def test_artifact_replay(key, tmp_path, golden_graphs, golden_vectors):
    from intent_ir_b200.artifacts import run_artifact

    g = golden_graphs[key]
    report = {"baseline": {"shapes": g["shapes"], "seed": 0}, "intent": g["intent"], "intent_expanded": g["intent"]}
    (tmp_path / f"{key}.json").write_text(json.dumps(report))
    arrays = {n: golden_vectors[f"{key}/in/{n}"] for n in g["inputs"]}
    arrays.update({n: golden_vectors[f"{key}/out/{n}"] for n in g["outputs"]})
    np.savez(tmp_path / f"{key}.baseline.npz", **arrays)
    res = run_artifact(str(tmp_path / f"{key}.json"))
    assert res["ok"], res
    # a corrupted recording must be reported, output by output
    arrays[g["outputs"][0]] = np.where(arrays[g["outputs"][0]].astype(np.float32) > -1e30, 1, 0).astype(arrays[g["outputs"][0]].dtype) \
        if arrays[g["outputs"][0]].dtype != np.bool_ else ~arrays[g["outputs"][0]]
    np.savez(tmp_path / f"{key}.baseline.npz", **arrays)
    res = run_artifact(str(tmp_path / f"{key}.json"))
    assert not res["ok"] and g["outputs"][0] in res["failed"]


# ---- rope, dropout and the int8 image ops against the reference interpreter's recorded outputs (tests/golden/make_golden_ops.py) ----

with open(os.path.join(os.path.dirname(__file__), "golden", "op_intents.json")) as _f:
    _OP_GRAPHS = json.load(_f)


@pytest.mark.parametrize("key", sorted(_OP_GRAPHS))
def test_single_op_kernels_are_bit_exact(key):
    g = _OP_GRAPHS[key]
    with np.load(os.path.join(os.path.dirname(__file__), "golden", "op_vectors.npz")) as z:
        ins = {n: z[f"{key}/in/{n}"] for n in g["inputs"]}
        want = {n: z[f"{key}/out/{n}"] for n in g["outputs"]}
    intent = IntentFunction.from_json_dict(g["intent"])
    out, lowered = _lower_and_run(intent, g["shapes"], ins)
    assert [s["kernel"] for s in lowered.steps] == [key.split("_")[0]]
    for n, w in want.items():
        assert out[n].dtype == w.dtype and np.array_equal(out[n], w), (key, n)


def test_dropout_mask_statistics_and_scaling_at_size():
    """4M elements: the keep fraction matches 1 - p, kept values are exactly x / (1 - p), and the
    mask equals the oracle's Philox stream."""
    js = {"name": "dropout", "tensors": {"x": _t0(["M"]), "p": _t0([]), "seed": _t0([], "i64"), "y": _t0(["M"])},
          "ops": [{"op": "dropout", "inputs": ["x", "p", "seed"], "output": "y"}], "outputs": ["y"]}
    intent = IntentFunction.from_json_dict(js)
    m = 1 << 22
    x = np.random.default_rng(3).standard_normal(m, dtype=np.float32) + 3.0
    ins = {"x": x, "p": np.array(0.3, np.float32), "seed": np.array(2 ** 33 + 17, np.int64)}
    out, _ = _lower_and_run(intent, {"M": m}, ins)
    want = execute_intent(intent, ins, {"M": m})["y"]
    assert np.array_equal(out["y"], want)
    assert abs((out["y"] != 0).mean() - 0.7) < 2e-3


def test_rope_and_dropout_inside_larger_graphs():
    js = {"name": "g", "tensors": {"x": _t0(["S", "B", "H", "D"]), "c": _t0(["S", "D2"]), "s": _t0(["S", "D2"]), "p": _t0([]),
                                   "seed": _t0([], "i32"), "y": _t0(["S", "B", "H", "D"])},
          "ops": [{"op": "mul", "inputs": ["x"], "output": "x2", "attrs": {"mul_factor": 0.5}},
                  {"op": "rope", "inputs": ["x2", "c", "s"], "output": "r"},
                  {"op": "dropout", "inputs": ["r", "p", "seed"], "output": "d", "attrs": {"n_rounds": 7}},
                  {"op": "relu", "inputs": ["d"], "output": "y"}], "outputs": ["y"]}
    intent = IntentFunction.from_json_dict(js)
    rng = np.random.default_rng(9)
    shapes = {"S": 5, "B": 2, "H": 3, "D": 16, "D2": 8}
    ang = rng.uniform(-3, 3, (5, 8))
    ins = {"x": rng.standard_normal((5, 2, 3, 16), dtype=np.float32), "c": np.cos(ang).astype(np.float32), "s": np.sin(ang).astype(np.float32),
           "p": np.array(0.25, np.float32), "seed": np.array(77, np.int32)}
    out, lowered = _lower_and_run(intent, shapes, ins)
    want = execute_intent(intent, ins, shapes)["y"]
    assert np.array_equal(out["y"], want), [s["kernel"] for s in lowered.steps]


def test_image_ops_at_size_and_in_a_chain():
    """correlation -> resize -> warp on a [8, 96, 160] int8 image: every stage integer-exact."""
    t = _t0
    js = {"name": "img", "tensors": {"a": t(["C", "H", "W"], "i8"), "b": t(["C", "H", "W"], "i8"), "sh": t([], "i32"), "off": t(["H2", "W2"], "i16"),
                                     "corr": t(["OC", "H", "W"], "i8"), "up": t(["OC", "H2", "W2"], "i8"), "out": t(["OC", "H2", "W2"], "i8")},
          "ops": [{"op": "correlation", "inputs": ["a", "b", "sh"], "output": "corr"},
                  {"op": "resize", "inputs": ["corr"], "output": "up", "attrs": {"hw_fl": 7}},
                  {"op": "warp", "inputs": ["up", "off"], "output": "out"}], "outputs": ["out", "corr"]}
    intent = IntentFunction.from_json_dict(js)
    rng = np.random.default_rng(12)
    shapes = {"C": 8, "H": 96, "W": 160, "OC": 5, "H2": 192, "W2": 320}
    ins = {"a": rng.integers(-128, 128, (8, 96, 160)).astype(np.int8), "b": rng.integers(-128, 128, (8, 96, 160)).astype(np.int8),
           "sh": np.array(6, np.int32), "off": rng.integers(-1024, 1024, (192, 320)).astype(np.int16)}
    out, lowered = _lower_and_run(intent, shapes, ins)
    assert [s["kernel"] for s in lowered.steps] == ["correlation", "resize", "warp"]
    want = execute_intent(intent, ins, shapes)
    for n in ("out", "corr"):
        assert out[n].dtype == np.int8 and np.array_equal(out[n], want[n]), n


@pytest.mark.parametrize("m,n", [(7, 64), (33, 1000), (64, 4096), (16, 8192), (40, 20000), (24, 40000), (20, 100000), (12, 20000), (3, 200000),
                                 (5, 4099)])
@pytest.mark.parametrize("residual", [False, True])
def test_rms_norm_through_every_norm_kernel_variant(m, n, residual, golden_graphs):
    """rms-norm runs on the row-normalisation kernels with the mean fixed at zero: warp, block, pipelined
    cluster, one-shot cluster and (for a handful of long rows) segmented variants, with and without a residual
    sum in front."""
    key = "rms_norm_residual2d" if residual else "rms_norm2d"
    intent = IntentFunction.from_json_dict(golden_graphs[key]["intent"])
    rng = np.random.default_rng(n + m)
    ins = {"inp": (2.0 + rng.standard_normal((m, n))).astype(np.float32), "weight": rng.uniform(0.5, 1.5, n).astype(np.float32)}
    if residual:
        ins["residual"] = rng.standard_normal((m, n)).astype(np.float32)
        ins["bias"] = rng.standard_normal(n).astype(np.float32)
    out, lowered = _lower_and_run(intent, {"M": m, "N": n}, ins)
    assert lowered.steps[-1]["kernel"] in ("rmsnorm", "residual+rmsnorm", "rmsnorm(segmented)")
    assert (lowered.steps[-1]["kernel"] == "rmsnorm(segmented)") == (n > 16384 and m * 8 < 148)
    if residual:  # rows up to 16384 elements are summed inside the norm kernel, longer ones by a kernel in front of it
        assert (len(lowered.steps) == 1) == (n <= 16384), [s["kernel"] for s in lowered.steps]
    want = execute_intent(intent, ins, {"M": m, "N": n})
    tol = infer_tolerances(intent).to_dict()
    for name in intent.outputs:
        _agree(out[name], want[name], tol, name)
    # a row of zeros stays finite (rstd = 1/sqrt(eps)) and an Inf poisons only its own row
    ins["inp"][0] = 0.0
    if m > 1:
        ins["inp"][1, 0] = np.inf
    if residual:
        ins["residual"][:2] = 0.0
    out, _ = _lower_and_run(intent, {"M": m, "N": n}, ins)
    with np.errstate(all="ignore"):
        want = execute_intent(intent, ins, {"M": m, "N": n})
    for name in intent.outputs:
        w, g = np.asarray(want[name]), out[name]
        assert np.array_equal(np.isnan(w), np.isnan(g)), name
        assert np.allclose(np.nan_to_num(g, nan=0.0, posinf=0.0, neginf=0.0), np.nan_to_num(w, nan=0.0, posinf=0.0, neginf=0.0), rtol=1e-3, atol=1e-3), name


def test_seeded_sweep_over_every_graph_family():
    """96 seeded cases over all fourteen graph families (random extents with the verifier's edge sizes, f32 and
    bf16) lowered, run on the GPU and diffed by the oracle's run_diff, exactly as `bench.py --workload sweep` does."""
    from intent_ir_b200.sweep import ALL_KINDS, generate_sweep_cases, run_sweep

    cases = generate_sweep_cases(96, base_seed=4242, max_elements=1 << 18, kinds=ALL_KINDS)
    recs = run_sweep(cases, diff_fn=run_diff, tolerances_fn=infer_tolerances, case_type=TestCase)
    bad = [(r["kind"], r["shapes"], r["summary"]) for r in recs if not r["ok"]]
    assert len(recs) == 96 and not bad, bad
    assert {r["kind"] for r in recs} == set(ALL_KINDS)


@pytest.mark.parametrize("rounds", [1, 5, 13])
def test_dropout_with_other_round_counts(rounds):
    js = {"name": "dropout", "tensors": {"x": _t0(["M"]), "p": _t0([]), "seed": _t0([], "i32"), "y": _t0(["M"])},
          "ops": [{"op": "dropout", "inputs": ["x", "p", "seed"], "output": "y", "attrs": {"n_rounds": rounds}}], "outputs": ["y"]}
    intent = IntentFunction.from_json_dict(js)
    ins = {"x": np.random.default_rng(rounds).standard_normal(5000, dtype=np.float32), "p": np.array(0.4, np.float32), "seed": np.array(-3, np.int32)}
    out, _ = _lower_and_run(intent, {"M": 5000}, ins)
    assert np.array_equal(out["y"], execute_intent(intent, ins, {"M": 5000})["y"])


@pytest.mark.parametrize("m,n", [(5001, 64), (4099, 32), (1000, 17), (7, 8), (3001, 60), (2, 3), (1025, 33)])
@pytest.mark.parametrize("key,xname", [("softmax_inner", "input_ptr"), ("layer_norm_persistent", "in_ptr"), ("rms_norm2d", "inp")])
def test_short_rows_share_a_warp(key, xname, m, n, golden_graphs):
    """Rows of at most 64 elements run 2 or 4 to a warp; row counts that do not fill the last warp included."""
    intent = IntentFunction.from_json_dict(golden_graphs[key]["intent"])
    rng = np.random.default_rng(m * 131 + n)
    ins = {xname: (1.5 * rng.standard_normal((m, n))).astype(np.float32)}
    for name in golden_graphs[key]["inputs"]:
        if name != xname:
            ins[name] = rng.uniform(0.5, 1.5, n).astype(np.float32)
    out, _ = _lower_and_run(intent, {"M": m, "N": n}, ins)
    want = execute_intent(intent, ins, {"M": m, "N": n})
    tol = infer_tolerances(intent).to_dict()
    for name in intent.outputs:
        _agree(out[name], want[name], tol, name)


# ---- softmax with a where-mask applied on load --------------------------------------------

def _masked_softmax_graph(full_mask, fill):
    mshape = ["M", "N"] if full_mask else ["N"]
    ops = []
    if not full_mask:
        ops.append({"op": "broadcast_in_dim", "inputs": ["mask"], "output": "m2", "attrs": {"broadcast_dims": [1], "out_shape": ["M", "N"]}})
    ops += [{"op": "const", "inputs": [], "output": "neg", "attrs": {"value": fill, "dtype": "f32"}},
            {"op": "where", "inputs": ["mask" if full_mask else "m2", "x", "neg"], "output": "xm"},
            {"op": "softmax", "inputs": ["xm"], "output": "y", "attrs": {"axis": -1}}]
    return {"name": "msm", "tensors": {"x": _t(["M", "N"]), "mask": _t(mshape, "bool"), "m2": _t(["M", "N"], "bool"), "y": _t(["M", "N"])},
            "ops": ops, "outputs": ["y"]}


@pytest.mark.parametrize("m,n", [(1, 1), (5, 1), (1, 9), (5, 7), (16, 64), (4099, 24), (37, 60), (33, 1000), (9, 4099), (3, 16384), (2, 20000)])
@pytest.mark.parametrize("full_mask", [False, True])
def test_softmax_applies_the_mask_while_loading(m, n, full_mask):
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel
    from intent_ir_b200.runtime import run_lowered

    intent = IntentFunction.from_json_dict(_masked_softmax_graph(full_mask, -1e9))
    rng = np.random.default_rng(m * 31 + n)
    x = rng.standard_normal((m, n)).astype(np.float32) * 3
    mask = rng.random((m, n) if full_mask else (n,)) > 0.4
    if full_mask and m > 1:
        mask[1, :] = False  # a row with everything masked: uniform over the fill value
        mask[m - 1, :] = True
    low = lower_intent_to_b200_kernel(intent, shape_bindings={"M": m, "N": n})
    kernels = [s["kernel"] for s in low.steps]
    assert kernels == (["softmax+mask"] if n <= 16384 else kernels), kernels
    got = run_lowered(low, {"x": x, "mask": mask})["y"]
    want = execute_intent(intent, {"x": x, "mask": mask}, shape_bindings={"M": m, "N": n})["y"]
    assert np.allclose(got, want, rtol=1e-5, atol=1e-7), float(np.abs(got - want).max())
    assert np.allclose(got.sum(axis=1), 1.0, atol=1e-4)
    keep = np.broadcast_to(mask, (m, n))
    live = keep.any(axis=1)
    assert np.all(got[live][~keep[live]] == 0.0)  # exp(-1e9 - max) is exactly zero


def test_masked_softmax_keeps_an_infinite_fill_and_a_consumer_of_the_masked_scores():
    """-inf as the fill gives NaN rows where nothing is kept, as in numpy; a graph that also
    returns the masked scores cannot drop them, so the mask stays a step of its own."""
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel
    from intent_ir_b200.runtime import run_lowered

    js = _masked_softmax_graph(True, float("-inf"))
    rng = np.random.default_rng(5)
    x = rng.standard_normal((6, 50)).astype(np.float32)
    mask = rng.random((6, 50)) > 0.5
    mask[2, :] = False
    intent = IntentFunction.from_json_dict(js)
    low = lower_intent_to_b200_kernel(intent, shape_bindings={"M": 6, "N": 50})
    got = run_lowered(low, {"x": x, "mask": mask})["y"]
    with np.errstate(all="ignore"):
        want = execute_intent(intent, {"x": x, "mask": mask}, shape_bindings={"M": 6, "N": 50})["y"]
    assert np.allclose(got, want, rtol=1e-5, atol=1e-7, equal_nan=True)
    assert np.isnan(got[2]).all() and np.isfinite(np.delete(got, 2, axis=0)).all()

    js2 = _masked_softmax_graph(True, -1e9)
    js2["outputs"] = ["y", "xm"]
    js2["tensors"]["xm"] = _t(["M", "N"])
    intent2 = IntentFunction.from_json_dict(js2)
    low2 = lower_intent_to_b200_kernel(intent2, shape_bindings={"M": 6, "N": 50})
    assert "softmax+mask" not in [s["kernel"] for s in low2.steps]
    got2 = run_lowered(low2, {"x": x, "mask": mask})
    want2 = execute_intent(intent2, {"x": x, "mask": mask}, shape_bindings={"M": 6, "N": 50})
    assert np.array_equal(got2["xm"], want2["xm"]) and np.allclose(got2["y"], want2["y"], rtol=1e-5, atol=1e-7)


# ---- few long rows: the reduction is split over many CTAs ----------------------------------

def _reduce_graph(op, shape_syms, dims, dtype="f32"):
    out_shape = [s for i, s in enumerate(shape_syms) if i not in dims]
    return {"name": "r", "tensors": {"x": _t(shape_syms, dtype), "y": _t(out_shape, "bool" if op == "reduce_any" else "f32")},
            "ops": [{"op": op, "inputs": ["x"], "output": "y", "attrs": {"dims": dims}}], "outputs": ["y"]}


@pytest.mark.parametrize("op", ["reduce_sum", "reduce_max", "reduce_any"])
@pytest.mark.parametrize("m,n", [(1, 65536), (1, 1 << 22), (3, 100003), (7, 262147), (40, 70000), (295, 65537)])
def test_few_long_rows_are_split_over_the_gpu(op, m, n):
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel
    from intent_ir_b200.runtime import run_lowered

    intent = IntentFunction.from_json_dict(_reduce_graph(op, ["M", "N"], [1]))
    rng = np.random.default_rng(m + n)
    x = rng.standard_normal((m, n)).astype(np.float32)
    if op == "reduce_any":
        x[:] = 0
        x[0, n - 1] = 2.0  # only the last segment of the first row sees a non-zero
        if m > 2:
            x[2, 17] = float("nan")
    if op == "reduce_max" and m > 1:
        x[1, n // 2] = float("nan")  # np.max propagates it
    low = lower_intent_to_b200_kernel(intent, shape_bindings={"M": m, "N": n})
    assert [s["kernel"] for s in low.steps] == [op + "(split rows)"]
    with np.errstate(all="ignore"):
        want = execute_intent(intent, {"x": x}, shape_bindings={"M": m, "N": n})["y"]
    first = run_lowered(low, {"x": x})["y"]
    again = run_lowered(low, {"x": x})["y"]  # same scratch area a second time; same bits
    assert np.array_equal(first, again, equal_nan=True)
    if op == "reduce_sum":
        _agree(first, want, infer_tolerances(intent).to_dict(), "split sum")  # what the verifier grants: 1e-3 + 1e-3 |ref|
    else:
        assert np.array_equal(first, want, equal_nan=True)


def test_whole_tensor_reductions_and_split_rows_inside_a_graph():
    """sum over both axes is one row of M*N elements; a split reduction feeding later ops."""
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel
    from intent_ir_b200.runtime import run_lowered

    js = {"name": "g", "tensors": {"x": _t(["M", "N"]), "tot": _t([]), "y": _t(["M", "N"])},
          "ops": [{"op": "reduce_sum", "inputs": ["x"], "output": "tot", "attrs": {"dims": [0, 1]}},
                  {"op": "sub", "inputs": ["x", "tot"], "output": "y"}], "outputs": ["tot", "y"]}
    intent = IntentFunction.from_json_dict(js)
    x = np.random.default_rng(9).random((300, 1000)).astype(np.float32)
    low = lower_intent_to_b200_kernel(intent, shape_bindings={"M": 300, "N": 1000})
    assert "reduce_sum(split rows)" in [s["kernel"] for s in low.steps]
    got = run_lowered(low, {"x": x})
    want = execute_intent(intent, {"x": x}, shape_bindings={"M": 300, "N": 1000})
    assert np.allclose(got["tot"], want["tot"], rtol=1e-5)
    assert np.allclose(got["y"], want["y"], rtol=1e-5, atol=2e-2)


@pytest.mark.parametrize("op", ["reduce_sum", "reduce_max", "reduce_any"])
@pytest.mark.parametrize("shape,dims", [((100000, 64), [0]), ((65536, 1024), [0]), ((5000, 4), [0]), ((333, 8), [0]), ((70000, 132), [0]),
                                        ((3, 9000, 64), [1]), ((2, 4097, 20), [1]), ((40000, 6), [0]), ((17, 50, 4096), [0, 1])])
def test_reductions_over_leading_axes_are_split_over_the_gpu(op, shape, dims):
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel
    from intent_ir_b200.runtime import run_lowered

    syms = [f"D{i}" for i in range(len(shape))]
    bind = dict(zip(syms, shape))
    intent = IntentFunction.from_json_dict(_reduce_graph(op, syms, dims))
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal(shape).astype(np.float32)
    if op == "reduce_any":
        x[:] = 0
        x[(shape[0] - 1,) + (0,) * (len(shape) - 2) + (shape[-1] - 1,)] = 1.0
        x[(0,) * (len(shape) - 1) + (1,)] = float("nan")
    if op == "reduce_max":
        x[(shape[0] // 2,) + (0,) * (len(shape) - 1)] = float("nan")
    low = lower_intent_to_b200_kernel(intent, shape_bindings=bind)
    kernels = [s["kernel"] for s in low.steps]
    assert kernels == ([op + "(split columns)"] if shape[-1] % 4 == 0 else [op]), kernels
    with np.errstate(all="ignore"):
        want = execute_intent(intent, {"x": x}, shape_bindings=bind)["y"]
    first = run_lowered(low, {"x": x})["y"]
    again = run_lowered(low, {"x": x})["y"]
    assert first.shape == want.shape and np.array_equal(first, again, equal_nan=True)
    if op == "reduce_sum":
        _agree(first, want, infer_tolerances(intent).to_dict(), "split column sum")
    else:
        assert np.array_equal(first, want, equal_nan=True)


# ---- few, very long rows: segments over the whole GPU --------------------------------------------------------

@pytest.mark.parametrize("m,n,dtype", [(4, 1 << 20, "f32"), (1, 20000, "f32"), (3, 100003, "f32"), (2, 65536 + 4, "bf16"), (300, 1 << 17, "f32")])
def test_softmax_over_few_very_long_rows_is_segmented(m, n, dtype, golden_graphs):
    from intent_ir_b200.backend import round_to_bf16

    js = json.loads(json.dumps(golden_graphs["softmax_inner"]["intent"]))
    js["tensors"]["input_ptr"]["dtype"] = dtype  # a 16-bit input with an f32 result, as the sweep declares it
    intent = IntentFunction.from_json_dict(js)
    rng = np.random.default_rng(m + n)
    x = 3 * rng.standard_normal((m, n), dtype=np.float32)
    if dtype == "bf16":
        x = round_to_bf16(x)
    x[0, : n // 3] = -np.inf  # whole segments of -inf beside finite ones: exact zeros, no NaN
    if m > 1:
        x[1, n - 1] = 40.0  # the row maximum sits in the last segment
    if m > 2:
        x[2, 12345] = np.nan  # numpy: the whole row becomes NaN
    if m > 3:
        x[3, :] = -np.inf  # numpy: all NaN
    out, lowered = _lower_and_run(intent, {"M": m, "N": n}, {"input_ptr": x})
    assert [s["kernel"] for s in lowered.steps] == ["softmax(segmented)"]
    with np.errstate(all="ignore"):
        want = execute_intent(intent, {"input_ptr": x}, {"M": m, "N": n})["output_ptr"]
    _agree(out["output_ptr"], want, infer_tolerances(intent).to_dict(), "segmented softmax")
    assert np.all(out["output_ptr"][0, : n // 3] == 0)
    again, _ = _lower_and_run(intent, {"M": m, "N": n}, {"input_ptr": x})
    assert np.array_equal(out["output_ptr"], again["output_ptr"], equal_nan=True)  # a fixed folding order: the same bits every run


@pytest.mark.parametrize("m,n", [(4, 1 << 20), (2, 40000), (3, 100003), (1, 131072 + 8)])
def test_layernorm_over_few_very_long_rows_is_segmented(m, n, golden_graphs):
    intent = IntentFunction.from_json_dict(golden_graphs["layer_norm_persistent"]["intent"])
    rng = np.random.default_rng(m * 7 + n)
    x = (rng.standard_normal((m, n), dtype=np.float32) * np.float32(2.0) + np.float32(5.0)).astype(np.float32)  # a mean far from zero
    x[0, : n // 2] += np.float32(100.0)  # segment means far apart: the merge of segment moments has to carry it
    w = rng.uniform(0.5, 1.5, n).astype(np.float32)
    b = (0.1 * rng.standard_normal(n)).astype(np.float32)
    ins = {"in_ptr": x, "weight_ptr": w, "bias_ptr": b}
    out, lowered = _lower_and_run(intent, {"M": m, "N": n}, ins)
    assert [s["kernel"] for s in lowered.steps] == ["layernorm(segmented)"]
    with np.errstate(all="ignore"):
        want = execute_intent(intent, ins, {"M": m, "N": n})
    tol = infer_tolerances(intent).to_dict()
    for name in ("out_ptr", "out_mean_ptr", "out_rstd_ptr"):
        _agree(out[name], want[name], tol, name)
    x64 = x.astype(np.float64)
    assert np.allclose(out["out_mean_ptr"], x64.mean(axis=1), rtol=1e-6)
    assert np.allclose(out["out_rstd_ptr"], 1.0 / np.sqrt(x64.var(axis=1) + 1e-5), rtol=1e-5)


def test_rmsnorm_and_groupnorm_over_very_long_rows_are_segmented(golden_graphs):
    rng = np.random.default_rng(5)
    intent = IntentFunction.from_json_dict(golden_graphs["rms_norm2d"]["intent"])
    m, n = 2, 300000
    ins = {"inp": rng.standard_normal((m, n), dtype=np.float32), "weight": rng.uniform(0.5, 1.5, n).astype(np.float32)}
    out, lowered = _lower_and_run(intent, {"M": m, "N": n}, ins)
    assert [s["kernel"] for s in lowered.steps] == ["rmsnorm(segmented)"]
    want = execute_intent(intent, ins, {"M": m, "N": n})
    for name in intent.outputs:
        _agree(out[name], want[name], infer_tolerances(intent).to_dict(), name)
    # one group of 8 channels x 65536 positions: rows of 512 Ki elements with a per-channel affine
    gn = IntentFunction.from_json_dict(golden_graphs["group_norm_kernel"]["intent"])
    shapes = {"N": 2, "C": 16, "HW": 65536, "num_groups": 2}
    ins = {"X": rng.standard_normal((2, 16, 65536), dtype=np.float32), "W": rng.standard_normal(16, dtype=np.float32), "B": rng.standard_normal(16, dtype=np.float32)}
    out, lowered = _lower_and_run(gn, shapes, ins)
    assert [s["kernel"] for s in lowered.steps] == ["groupnorm(segmented)"]
    want = execute_intent(gn, ins, derive_bindings(shapes))
    for name in gn.outputs:
        _agree(out[name], want[name], infer_tolerances(gn).to_dict(), name)


# ---- f64 tensors and 32- / 64-bit integers: exact, through the double-valued elementwise kernel ------------------

def test_f64_elementwise_graph_matches_numpy_to_the_last_bit():
    js = {"name": "f64_chain", "tensors": {"a": _t(["M", "N"], "f64"), "b": _t(["N"], "f64"), "y": _t(["M", "N"], "f64"), "z": _t(["M", "N"], "f64")},
          "ops": [{"op": "add", "inputs": ["a", "b"], "output": "s"},
                  {"op": "mul", "inputs": ["s"], "output": "y", "attrs": {"mul_factor": 1.0000000001}},
                  {"op": "sub", "inputs": ["y", "a"], "output": "d"},
                  {"op": "max", "inputs": ["d", "b"], "output": "z"}], "outputs": ["y", "z"]}
    intent = IntentFunction.from_json_dict(js)
    rng = np.random.default_rng(8)
    a = 1.0 + 1e-12 * rng.standard_normal((37, 53))  # differences far below f32 resolution
    b = 1e-9 * rng.standard_normal(53)
    b[3] = np.nan
    out, lowered = _lower_and_run(intent, {"M": 37, "N": 53}, {"a": a, "b": b})
    assert all(s["kernel"].endswith("(f64 lanes)") for s in lowered.steps)
    want = execute_intent(intent, {"a": a, "b": b}, {"M": 37, "N": 53})
    for name in ("y", "z"):
        assert out[name].dtype == np.float64 and want[name].dtype == np.float64
        assert np.array_equal(out[name], want[name], equal_nan=True), name
    assert len(np.unique(out["y"])) > 1000  # the values really differ below f32 resolution


@pytest.mark.parametrize("dt,np_dt,big", [("i32", np.int32, 1 << 30), ("i64", np.int64, 1 << 45)])
def test_integer_elementwise_arithmetic_is_exact_beyond_2_to_24(dt, np_dt, big):
    js = {"name": "int_chain", "tensors": {"a": _t(["M", "N"], dt), "b": _t(["N"], dt), "s": _t(["M", "N"], dt), "p": _t(["M", "N"], dt),
                                           "lt": _t(["M", "N"], "bool"), "w": _t(["M", "N"], dt)},
          "ops": [{"op": "add", "inputs": ["a", "b"], "output": "s"},
                  {"op": "mul", "inputs": ["b"], "output": "b3", "attrs": {"mul_factor": 3}},
                  {"op": "sub", "inputs": ["a", "b3"], "output": "p"},
                  {"op": "lt", "inputs": ["a", "s"], "output": "lt"},
                  {"op": "where", "inputs": ["lt", "s", "p"], "output": "w"}], "outputs": ["s", "p", "lt", "w"]}
    intent = IntentFunction.from_json_dict(js)
    rng = np.random.default_rng(9)
    a = (big + rng.integers(-1000, 1000, size=(19, 40))).astype(np_dt)  # neighbours differ by 1: f32 lanes would merge them
    b = rng.integers(-5, 6, size=40).astype(np_dt)
    a[0, :4] = [(1 << 24) + 1, (1 << 24) + 3, -(1 << 24) - 1, 0]
    out, lowered = _lower_and_run(intent, {"M": 19, "N": 40}, {"a": a, "b": b})
    assert all(s["kernel"].endswith("(f64 lanes)") for s in lowered.steps)
    want = execute_intent(intent, {"a": a, "b": b}, {"M": 19, "N": 40})
    for name in ("s", "p", "lt", "w"):
        assert np.array_equal(out[name].astype(np.int64), np.asarray(want[name]).astype(np.int64)), name
    assert out["s"].dtype == np_dt and out["lt"].dtype == np.bool_


def test_iota_index_arithmetic_over_a_large_extent_is_exact():
    """Flattened indices of a [5000, 4000] tensor run to 2*10^7, past the 2^24 an f32 lane counts to."""
    js = {"name": "flat_index", "tensors": {"y": _t(["M", "N"], "i32")},
          "ops": [{"op": "iota", "inputs": [], "output": "r", "attrs": {"shape": ["M", "N"], "axis": 0, "dtype": "i32"}},
                  {"op": "iota", "inputs": [], "output": "c", "attrs": {"shape": ["M", "N"], "axis": 1, "dtype": "i32"}},
                  {"op": "mul", "inputs": ["r"], "output": "rn", "attrs": {"mul_factor": 4000}},
                  {"op": "add", "inputs": ["rn", "c"], "output": "y"}], "outputs": ["y"]}
    intent = IntentFunction.from_json_dict(js)
    out, lowered = _lower_and_run(intent, {"M": 5000, "N": 4000}, {})
    assert np.array_equal(out["y"].astype(np.int64).ravel(), np.arange(5000 * 4000, dtype=np.int64))


# ---- graph forms the interpreter takes with any axis -----------------------------------------------------------

@pytest.mark.parametrize("shape,axis,dtype", [((4, 100, 64), 1, "f32"), ((40, 64), 0, "f32"), ((3, 7, 5, 33), 2, "f32"), ((2, 1, 300, 17), -2, "bf16"),
                                              ((1, 2, 3), 0, "f32"), ((16, 2048, 8), 1, "f32")])
def test_softmax_over_a_non_trailing_axis(shape, axis, dtype):
    from intent_ir_b200.backend import round_to_bf16

    syms = [f"D{i}" for i in range(len(shape))]
    js = {"name": "sm_axis", "tensors": {"x": _t(syms, dtype), "y": _t(syms, "f32")},
          "ops": [{"op": "softmax", "inputs": ["x"], "output": "y", "attrs": {"axis": axis}}], "outputs": ["y"]}
    intent = IntentFunction.from_json_dict(js)
    bind = dict(zip(syms, shape))
    x = 3 * np.random.default_rng(sum(shape)).standard_normal(shape).astype(np.float32)
    if dtype == "bf16":
        x = round_to_bf16(x)
    if x.size > 10:
        x.reshape(-1)[3] = -np.inf
    out, lowered = _lower_and_run(intent, bind, {"x": x})
    with np.errstate(all="ignore"):
        want = execute_intent(intent, {"x": x}, bind)["y"]
    _agree(out["y"], want, infer_tolerances(intent).to_dict(), "softmax axis")
    assert np.allclose(out["y"].sum(axis=axis), 1.0, atol=1e-4)


@pytest.mark.parametrize("op", ["reduce_sum", "reduce_max", "reduce_any"])
@pytest.mark.parametrize("shape,dims,keepdims", [((4, 10, 6, 8), [0, 2], False), ((4, 10, 6, 8), [1, 3], True), ((3, 5, 7, 2, 9), [0, 2, 4], False),
                                                 ((33, 1, 17, 65), [0, 2], False), ((2, 3, 4), [0, 2], True), ((64, 300, 5, 128), [0, 2], False)])
def test_reductions_over_non_adjacent_axes(op, shape, dims, keepdims):
    syms = [f"D{i}" for i in range(len(shape))]
    out_shape = [1 if i in dims else s for i, s in enumerate(syms) if keepdims or i not in dims]
    js = {"name": "r", "tensors": {"x": _t(syms), "y": _t(out_shape, "bool" if op == "reduce_any" else "f32")},
          "ops": [{"op": op, "inputs": ["x"], "output": "y", "attrs": {"dims": dims, "keepdims": keepdims}}], "outputs": ["y"]}
    intent = IntentFunction.from_json_dict(js)
    bind = dict(zip(syms, shape))
    rng = np.random.default_rng(sum(shape) + len(dims))
    x = rng.standard_normal(shape).astype(np.float32)
    if op == "reduce_any":
        x = np.where(rng.random(shape) < 0.02, x, np.float32(0))
    if op == "reduce_max":
        x.reshape(-1)[5] = np.nan
    out, lowered = _lower_and_run(intent, bind, {"x": x})
    assert len(lowered.steps) >= 2 or 1 in shape
    with np.errstate(all="ignore"):
        want = execute_intent(intent, {"x": x}, bind)["y"]
    _agree(out["y"], want, infer_tolerances(intent).to_dict(), op)


def test_scaled_sum_over_three_separate_axes():
    js = {"name": "r3", "tensors": {"x": _t(["A", "B", "C", "D", "E"]), "y": _t(["B", "D"])},
          "ops": [{"op": "reduce_sum", "inputs": ["x"], "output": "y", "attrs": {"dims": [0, 2, 4], "scale": "1.0/(A*C*E)"}}], "outputs": ["y"]}
    intent = IntentFunction.from_json_dict(js)
    bind = {"A": 4, "B": 10, "C": 6, "D": 8, "E": 3}
    x = np.random.default_rng(3).standard_normal((4, 10, 6, 8, 3)).astype(np.float32)
    out, lowered = _lower_and_run(intent, bind, {"x": x})
    assert [s["kernel"] for s in lowered.steps] == ["reduce_sum"] * 3
    want = execute_intent(intent, {"x": x}, bind)["y"]
    _agree(out["y"], want, infer_tolerances(intent).to_dict(), "mean over three axes")
    assert np.allclose(out["y"], x.mean(axis=(0, 2, 4)), atol=1e-5)


def test_compiled_in_chains_give_the_interpreters_bits():
    """The benchmark chains run as straight-line kernels; same expressions per opcode as the instruction loop, so the
    results equal the oracle's bit for bit (as every elementwise program's do)."""
    import bench

    for name in ("chain", "dag"):
        js, _, _, _, _, _ = bench.workload(name)
        intent = IntentFunction.from_json_dict(js)
        for m, n in ((64, 128), (33, 260), (257, 4096)):
            rng = np.random.default_rng(m + n)
            ins = {"x": rng.standard_normal((m, n), dtype=np.float32), "col": rng.standard_normal(n, dtype=np.float32),
                   "row": rng.standard_normal((m, 1), dtype=np.float32)}
            ins["x"][0, 0] = np.nan
            out, lowered = _lower_and_run(intent, {"M": m, "N": n}, ins)
            # (the interpreter's attribute operand `mul_factor` is a float64 scalar, so under numpy 2 its result is float64;
            # the last addition then rounds once more on the way to the declared f32 — which is the f32 result)
            want = np.asarray(execute_intent(intent, ins, {"M": m, "N": n})["y"]).astype(np.float32)
            assert np.array_equal(out["y"], want, equal_nan=True), (name, m, n)


@pytest.mark.parametrize("m,n", [(7, 64), (33, 1000), (64, 4096), (16, 8192), (40, 20000), (24, 40000), (5, 4099)])
@pytest.mark.parametrize("where", ["inside", "after"])
def test_relu_inside_a_normalisation_rides_in_the_norm_kernel(m, n, where, golden_graphs):
    """rms-norm with relu(x̂)·w and layernorm followed by a ReLU: one norm kernel, checked against the oracle."""
    rng = np.random.default_rng(m + n)
    if where == "inside":
        t = lambda s: {"dtype": "f32", "shape": s, "layout": "row_major"}  # noqa: E731
        js = {"name": "rms_relu", "tensors": {"x": t(["M", "N"]), "w": t(["N"]), "y": t(["M", "N"]), "rstd": t(["M"])},
              "ops": [{"op": "mul", "inputs": ["x", "x"], "output": "sq"},
                      {"op": "reduce_sum", "inputs": ["sq"], "output": "ss", "attrs": {"dims": [1], "keepdims": True, "scale": "1.0/N"}},
                      {"op": "add", "inputs": ["ss"], "output": "ve", "attrs": {"addend": 1e-5}},
                      {"op": "rsqrt", "inputs": ["ve"], "output": "r1"},
                      {"op": "reshape", "inputs": ["r1"], "output": "rstd", "attrs": {"shape": ["M"]}},
                      {"op": "mul", "inputs": ["x", "r1"], "output": "xn"},
                      {"op": "relu", "inputs": ["xn"], "output": "xr"},
                      {"op": "mul", "inputs": ["xr", "w"], "output": "y"}], "outputs": ["y", "rstd"]}
        ins = {"x": rng.standard_normal((m, n), dtype=np.float32), "w": rng.uniform(-1.5, 1.5, n).astype(np.float32)}
        label = "rmsnorm+relu"
    else:
        js = json.loads(json.dumps(golden_graphs["layer_norm_persistent"]["intent"]))
        out = js["outputs"][0]
        for o in js["ops"]:
            if o["output"] == out:
                o["output"] = "pre_relu"
        js["tensors"]["pre_relu"] = dict(js["tensors"][out])
        js["ops"].append({"op": "relu", "inputs": ["pre_relu"], "output": out})
        ins = {"in_ptr": rng.standard_normal((m, n), dtype=np.float32), "weight_ptr": rng.uniform(-1.5, 1.5, n).astype(np.float32),
               "bias_ptr": (0.3 * rng.standard_normal(n)).astype(np.float32)}
        label = "layernorm+relu"
    intent = IntentFunction.from_json_dict(js)
    out_, lowered = _lower_and_run(intent, {"M": m, "N": n}, ins)
    assert [s["kernel"] for s in lowered.steps] == [label]
    want = execute_intent(intent, ins, {"M": m, "N": n})
    tol = infer_tolerances(intent).to_dict()
    for name in intent.outputs:
        _agree(out_[name], want[name], tol, name)
    main = out_[intent.outputs[0]]
    assert (main == 0).mean() > 0.2 or where == "inside"  # the ReLU really clipped something


# ---- row programs that are also compiled in (rowfuse.cu): every launch shape against the oracle ----

@pytest.mark.parametrize("key", ["_attn_fwd", "flash_attention2d"])
@pytest.mark.parametrize("kv", [16, 200, 1024, 1028, 4096, 8200, 250])
def test_compiled_in_attention_softmax_rows(key, kv, golden_graphs):
    """The scale + mask + softmax between an attention's two products is one fused row program whose phases are
    also compiled into the kernel.  Row lengths cover one warp per row (up to 1024), 128 and 512 threads per
    row, rows that end inside a pass, and a length that is no multiple of 4 (which runs decoded)."""
    g = golden_graphs[key]
    intent = IntentFunction.from_json_dict(g["intent"])
    shapes = dict(g["shapes"], KV_CTX=kv, Q_CTX=24)
    rng = np.random.default_rng(kv)
    dims = lambda name: tuple(shapes[d] if isinstance(d, str) else d for d in g["intent"]["tensors"][name]["shape"])  # noqa: E731
    ins = {n: rng.standard_normal(dims(n), dtype=np.float32) for n in g["inputs"]}
    ins["sm_scale"] = np.array([0.25], dtype=np.float32)
    if "attn_mask" in ins:
        ins["attn_mask"] = np.where(rng.random(dims("attn_mask")) < 0.2, -1e9, 0.0).astype(np.float32)
    out, lowered = _lower_and_run(intent, shapes, ins)
    fused = [s for s in lowered.steps if "row_program" in s]
    assert len(fused) == 1 and fused[0]["row_program"]["compiled_in"] == (kv % 4 == 0), [s["kernel"] for s in lowered.steps]
    with np.errstate(all="ignore"):
        want = execute_intent(intent, ins, shapes)
    tol = infer_tolerances(intent).to_dict()
    for name in g["outputs"]:
        _agree(out[name], want[name], tol, f"{key}/{name}/kv={kv}")


@pytest.mark.parametrize("m,n", [(64, 512), (300, 4096), (16, 8192), (9, 1000), (5, 4100)])
def test_compiled_in_rms_row_program(m, n):
    """rms-norm with |x| between the normalisation and the weight: nothing dedicated matches, so it runs as a
    fused row program, one of those compiled in; rstd is the graph's second output."""
    t = lambda shape: {"dtype": "f32", "shape": shape, "layout": "row_major"}  # noqa: E731
    js = {"name": "rms_abs", "tensors": {"x": t(["M", "N"]), "w": t(["N"]), "y": t(["M", "N"]), "rstd": t(["M"])},
          "ops": [{"op": "mul", "inputs": ["x", "x"], "output": "sq"},
                  {"op": "reduce_sum", "inputs": ["sq"], "output": "ss", "attrs": {"dims": [1], "keepdims": True, "scale": "1.0/N"}},
                  {"op": "add", "inputs": ["ss"], "output": "ve", "attrs": {"addend": 1e-5}},
                  {"op": "rsqrt", "inputs": ["ve"], "output": "r1"},
                  {"op": "reshape", "inputs": ["r1"], "output": "rstd", "attrs": {"shape": ["M"]}},
                  {"op": "mul", "inputs": ["x", "r1"], "output": "xn"},
                  {"op": "abs", "inputs": ["xn"], "output": "xr"},
                  {"op": "mul", "inputs": ["xr", "w"], "output": "y"}], "outputs": ["y", "rstd"]}
    intent = IntentFunction.from_json_dict(js)
    rng = np.random.default_rng(n)
    ins = {"x": rng.standard_normal((m, n), dtype=np.float32), "w": rng.uniform(0.5, 1.5, n).astype(np.float32)}
    out, lowered = _lower_and_run(intent, {"M": m, "N": n}, ins)
    fused = [s for s in lowered.steps if "row_program" in s]
    assert len(lowered.steps) == 1 and fused and fused[0]["row_program"]["compiled_in"]
    want = execute_intent(intent, ins, {"M": m, "N": n})
    tol = infer_tolerances(intent).to_dict()
    for name in ("y", "rstd"):
        _agree(out[name], want[name], tol, f"rms_abs/{name}/{m}x{n}")
