"""The planner's elementwise programs, checked without a GPU: the micro-op programs in the plan
description (operand strides over the collapsed extents, slots, immediates, stores) are executed by the
numpy emulator in tests/rowprog_emulator.py and compared with the oracle -- bit for bit on the fuzz
graphs, whose dyadic inputs make every exact op exact on both sides."""

import json

import numpy as np
import pytest

from intent_ir_b200.bindings import derive_bindings
from intent_ir_b200.ir import IntentFunction
from intent_ir_b200.lowering import plan_json
from intent_ir_b200.sweep import case_inputs, generate_sweep_cases
from oracle import execute_intent, infer_tolerances
from oracle.diff import compare_outputs
from tests.rowprog_emulator import run_plan_description
from tests.test_fuzz_gpu import _inputs, random_elementwise_graph


def _emulate(js, ins, bindings):
    desc = plan_json(js, bindings)
    kernels = [s["kernel"] for s in desc["steps"]]
    if not all("program" in s or "row_program" in s for s in desc["steps"]):
        pytest.skip(f"plan has steps the emulator does not cover: {kernels}")
    intent = IntentFunction.from_json_dict(json.loads(json.dumps(js)))
    with np.errstate(all="ignore"):
        want = execute_intent(intent, ins, shape_bindings=bindings)
    return intent, desc, want, run_plan_description(desc, ins), kernels


@pytest.mark.parametrize("seed", range(40))
def test_fuzzed_dags_mean_what_the_oracle_computes(seed):
    """Random DAGs over x[M,N], col[N], row[M,1], lead[1,N] and a scalar, with reused values and a float and a
    boolean result, at shapes with and without vectorisable inner extents."""
    rng = np.random.default_rng(seed)
    m, n = [(1, 1), (3, 5), (7, 64), (33, 100), (16, 256), (5, 1028), (600, 9)][seed % 7]
    js = random_elementwise_graph(rng, int(rng.integers(2, 14)))
    ins = _inputs(rng, m, n)
    intent, desc, want, got, kernels = _emulate(js, ins, {"M": m, "N": n})
    for name in intent.outputs:
        w, g = np.asarray(want[name]), got[name]
        assert g.shape == w.shape, (name, kernels)
        if w.dtype == np.bool_:
            assert np.array_equal(g.astype(bool), w), (name, kernels)
        else:
            assert np.array_equal(g.astype(np.float32), w.astype(np.float32), equal_nan=True), (name, kernels)


def test_sweep_chains_mean_what_the_oracle_computes():
    """The broadcast add / mul chains of the verification sweep (2-6 ops, f32 and bf16 declarations) at small sizes."""
    cases = [c for c in generate_sweep_cases(300, base_seed=1000, max_elements=1 << 12) if c.kind == "chain"][:24]
    assert len(cases) >= 12
    for c in cases:
        bind = derive_bindings(dict(c.shapes))
        ins = case_inputs(c)
        intent, desc, want, got, kernels = _emulate(c.intent, ins, bind)
        tol = infer_tolerances(intent).to_dict()
        for name in intent.outputs:
            d = compare_outputs({"y": np.asarray(want[name])}, {"y": got[name].astype(np.float32)}, ["y"], tol)
            assert d.ok, (c.case_id, c.dtype, c.shapes, d.summary, kernels)


ELEMENTWISE_GOLDEN = ["add2d", "add_bias2d", "clamp2d", "exp2d", "floor2d", "where2d", "copy2d_divmod", "any_const_ne"]


@pytest.mark.parametrize("key", ELEMENTWISE_GOLDEN)
def test_recorded_elementwise_graphs_reproduce_the_reference_outputs(key, golden_graphs, golden_vectors):
    """The reference's own elementwise graphs on its recorded inputs: the emulated plan gives the recorded outputs."""
    if key not in golden_graphs:
        pytest.skip("not recorded")
    g = golden_graphs[key]
    ins = {n: golden_vectors[f"{key}/in/{n}"] for n in g["inputs"]}
    bind = derive_bindings(dict(g["shapes"]))
    intent, desc, want, got, kernels = _emulate(g["intent"], ins, bind)
    for n in g["outputs"]:
        ref = golden_vectors[f"{key}/out/{n}"]
        if ref.dtype == np.bool_:
            assert np.array_equal(got[n].astype(bool), ref), (n, kernels)
        else:
            assert np.allclose(got[n].astype(np.float32), ref.astype(np.float32), rtol=1e-5, atol=1e-6, equal_nan=True), (n, kernels)


def test_wide_integer_program_is_exact_above_2_pow_24():
    """32-bit integers beyond float32's 24 bits run on double lanes with full-precision immediates."""
    js = {"name": "wide", "tensors": {k: {"dtype": "i32", "shape": ["M", "N"]} for k in ("x", "y", "z")},
          "ops": [{"op": "add", "inputs": ["x", "y"], "output": "t"},
                  {"op": "const", "inputs": [], "output": "c", "attrs": {"value": 16777217, "dtype": "i32"}},
                  {"op": "add", "inputs": ["t", "c"], "output": "z"}], "outputs": ["z"]}
    rng = np.random.default_rng(3)
    ins = {"x": rng.integers(1 << 24, 1 << 29, (5, 12)).astype(np.int32), "y": rng.integers(1 << 24, 1 << 29, (5, 12)).astype(np.int32)}
    intent, desc, want, got, kernels = _emulate(js, ins, {"M": 5, "N": 12})
    assert desc["steps"][0]["program"]["wide"] == 1 and desc["steps"][0]["program"]["instr"][-1]["imm"] == 16777217
    assert np.array_equal(got["z"].astype(np.int64), np.asarray(want["z"]).astype(np.int64))
