"""The CPU oracle against the reference's own outputs (tests/golden, written by
tests/golden/make_golden.py from the reference checkout): interpreter values bit for bit,
tolerances, generated case shapes and run_diff verdicts."""

import json
import os

import numpy as np
import pytest

from intent_ir_b200.ir import IntentFunction
from oracle import TestCase, execute_intent, generate_cases, infer_tolerances, run_diff
from oracle.diff import derive_bindings

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
with open(os.path.join(GOLDEN, "intents.json")) as _f:
    KEYS = sorted(json.load(_f))


def _io(key, graphs, vectors):
    g = graphs[key]
    ins = {n: vectors[f"{key}/in/{n}"] for n in g["inputs"]}
    outs = {n: vectors[f"{key}/out/{n}"] for n in g["outputs"]}
    return IntentFunction.from_json_dict(g["intent"]), g["shapes"], ins, outs


@pytest.mark.parametrize("key", KEYS)
def test_interpreter_reproduces_reference_bits(key, golden_graphs, golden_vectors):
    intent, shapes, ins, outs = _io(key, golden_graphs, golden_vectors)
    with np.errstate(all="ignore"):
        got = execute_intent(intent, ins, shape_bindings=derive_bindings(shapes))
    for name, want in outs.items():
        g = np.asarray(got[name])
        assert g.shape == want.shape, name
        assert g.dtype == want.dtype, (name, g.dtype, want.dtype)
        assert np.array_equal(g, want, equal_nan=g.dtype.kind == "f"), name


@pytest.mark.parametrize("key", KEYS)
def test_json_round_trip_matches_reference_serialisation(key, golden_graphs):
    js = golden_graphs[key]["intent"]
    assert IntentFunction.from_json_dict(js).to_json_dict() == js


@pytest.mark.parametrize("key", KEYS)
def test_tolerances_cases_and_verdicts(key, golden_graphs, golden_vectors, golden_verdicts):
    intent, shapes, ins, outs = _io(key, golden_graphs, golden_vectors)
    v = golden_verdicts[key]
    assert infer_tolerances(intent).to_dict() == v["tol_decl"]
    assert infer_tolerances(intent, ref_out={**ins, **outs}).to_dict() == v["tol_ref_out"]
    assert [c.shapes for c in generate_cases(intent, limit=12, seed=3)] == v["cases"]

    honest = lambda case: {**ins, **outs}  # noqa: E731
    d, cex = run_diff(intent, honest, [TestCase(shapes=shapes, dtypes={}, seed=0)])
    assert (d[0].ok, d[0].summary, len(cex)) == (v["honest"]["ok"], v["honest"]["summary"], v["honest"]["n_cex"])

    def corrupt(case):
        io = dict(honest(case))
        first = intent.outputs[0]
        a = np.array(io[first], copy=True)
        if a.dtype == bool:
            a.reshape(-1)[0] = ~a.reshape(-1)[0]
        else:
            a.reshape(-1)[-1] += 1.0
        io[first] = a
        return io

    d, cex = run_diff(intent, corrupt, [TestCase(shapes=shapes, dtypes={}, seed=0)])
    w = v["corrupt"]
    assert (d[0].ok, d[0].summary, len(cex)) == (w["ok"], w["summary"], w["n_cex"])
    assert (list(d[0].first_bad_index) if d[0].first_bad_index else None) == w["first_bad_index"]
    if w["max_abs_err"] is not None:
        assert d[0].max_abs_err == pytest.approx(w["max_abs_err"], rel=1e-12)


def _one_op(op, attrs, out_dtype="f32", out_shape=("M", "N")):
    return IntentFunction.from_json_dict({
        "name": f"edge_{op}",
        "tensors": {"x": {"dtype": "f32", "shape": ["M", "N"], "layout": "row_major"},
                    "y": {"dtype": out_dtype, "shape": list(out_shape), "layout": "row_major"}},
        "ops": [{"op": op, "inputs": ["x"], "output": "y", "attrs": attrs}], "outputs": ["y"]})


@pytest.mark.parametrize("tag,intent", [
    ("softmax", _one_op("softmax", {"axis": -1})),
    ("reduce_any", _one_op("reduce_any", {"dims": [1]}, "bool", ("M",))),
    ("reduce_max", _one_op("reduce_max", {"dims": [1]}, "f32", ("M",))),
    ("reduce_sum", _one_op("reduce_sum", {"dims": [1]}, "f32", ("M",))),
    ("relu", _one_op("relu", {})),
    ("exp", _one_op("exp", {})),
    ("rsqrt", _one_op("rsqrt", {})),
])
def test_non_finite_probes(tag, intent, golden_edges):
    with np.errstate(all="ignore"):
        got = np.asarray(execute_intent(intent, {"x": golden_edges["x"]})["y"])
    want = golden_edges[tag]
    assert got.dtype == want.dtype
    assert np.array_equal(got, want, equal_nan=want.dtype.kind == "f")


def test_known_answers_from_the_reference_tests():
    # tests/test_diff_runner.py:35-43 of the reference: all-ones GEMM + bias + ReLU = K + 1.
    js = {"name": "mm", "tensors": {
        "A": {"dtype": "f32", "shape": ["M", "K"], "layout": "row_major"},
        "B": {"dtype": "f32", "shape": ["K", "N"], "layout": "row_major"},
        "bias": {"dtype": "f32", "shape": ["N"], "layout": "row_major"},
        "C": {"dtype": "f32", "shape": ["M", "N"], "layout": "row_major"}},
        "ops": [{"op": "matmul", "inputs": ["A", "B"], "output": "Y"},
                {"op": "broadcast_in_dim", "inputs": ["bias"], "output": "bias2d",
                 "attrs": {"out_shape": ["M", "N"], "broadcast_dims": [1]}},
                {"op": "add", "inputs": ["Y", "bias2d"], "output": "Z"},
                {"op": "relu", "inputs": ["Z"], "output": "C"}], "outputs": ["C"]}
    intent = IntentFunction.from_json_dict(js)
    M, K, N = 2, 3, 4
    out = execute_intent(intent, {"A": np.ones((M, K), np.float32), "B": np.ones((K, N), np.float32),
                                  "bias": np.ones(N, np.float32)})
    assert out["C"].shape == (M, N) and np.all(out["C"] == K + 1.0)
    cases = generate_cases(intent, limit=3, seed=0)
    assert len(cases) == 3 and all({"M", "N", "K"} <= set(c.shapes) for c in cases)

    # :55-70: a runner that returns a wrong C must yield a counterexample.
    def wrong(case):
        m, k, n = case.shapes["M"], case.shapes["K"], case.shapes["N"]
        return {"A": np.ones((m, k), np.float32), "B": np.ones((k, n), np.float32),
                "bias": np.ones(n, np.float32), "C": np.full((m, n), 999.0, np.float32)}

    diffs, cex = run_diff(intent, wrong, [TestCase(shapes={"M": 2, "K": 2, "N": 2}, seed=0, dtypes={})])
    assert len(diffs) == 1 and not diffs[0].ok and cex


def test_tolerance_known_answers():
    # tests/test_tolerances.py of the reference: softmax-only f32 is tighter than 1e-3,
    # matmul is looser.
    soft = _one_op("softmax", {"axis": -1})
    assert infer_tolerances(soft).atol < 1e-3
    mm = IntentFunction.from_json_dict({"name": "m", "tensors": {
        "A": {"dtype": "f32", "shape": ["M", "K"]}, "B": {"dtype": "f32", "shape": ["K", "N"]},
        "C": {"dtype": "f32", "shape": ["M", "N"]}},
        "ops": [{"op": "matmul", "inputs": ["A", "B"], "output": "C"}], "outputs": ["C"]})
    assert infer_tolerances(mm).atol > 1e-3


# ---- rope, dropout, correlation, resize, warp (tests/golden/make_golden_ops.py) ----------------------
with open(os.path.join(GOLDEN, "op_intents.json")) as _f:
    OP_KEYS = sorted(json.load(_f))


@pytest.fixture(scope="module")
def op_golden():
    with open(os.path.join(GOLDEN, "op_intents.json")) as f:
        graphs = json.load(f)
    with np.load(os.path.join(GOLDEN, "op_vectors.npz")) as z:
        return graphs, {k: z[k] for k in z.files}


@pytest.mark.parametrize("key", OP_KEYS)
def test_interpreter_reproduces_single_op_kernel_bits(key, op_golden):
    graphs, vectors = op_golden
    g = graphs[key]
    intent = IntentFunction.from_json_dict(g["intent"])
    ins = {n: vectors[f"{key}/in/{n}"] for n in g["inputs"]}
    with np.errstate(all="ignore"):
        got = execute_intent(intent, ins, shape_bindings=g["shapes"])
    for n in g["outputs"]:
        want = vectors[f"{key}/out/{n}"]
        have = np.asarray(got[n])
        assert have.shape == want.shape and have.dtype == want.dtype, n
        assert np.array_equal(have, want, equal_nan=True), n
