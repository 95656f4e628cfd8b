"""Whole plans, checked without a GPU.  The plan description names, step by step, the kernels, their extents and
the buffers they are given; tests/rowprog_emulator.py restates the kernels' contracts in numpy and runs the plan.
What is checked is everything the planner decides -- pattern matching, views and strides, transposes around
non-trailing axes, the order of reductions over separate axes, scratch buffers, affine indexing, fused epilogues --
against the reference's recorded outputs and against the oracle.  The kernels themselves are checked on the GPU."""

import json

import numpy as np
import pytest

from intent_ir_b200.bindings import derive_bindings
from intent_ir_b200.errors import B200LoweringError
from intent_ir_b200.ir import IntentFunction
from intent_ir_b200.lowering import plan_json
from intent_ir_b200.sweep import case_inputs, generate_sweep_cases
from oracle import execute_intent, infer_tolerances
from oracle.diff import compare_outputs
from tests.rowprog_emulator import run_plan_description

with open(__file__.rsplit("/", 1)[0] + "/golden/intents.json") as _f:
    _KEYS = sorted(json.load(_f))


def _t(shape, dtype="f32"):
    return {"dtype": dtype, "shape": list(shape), "layout": "row_major"}


def _agree(got, want, tol, what):
    want = np.asarray(want)
    got = np.asarray(got).reshape(want.shape)
    if want.dtype == np.bool_:
        assert np.array_equal(got.astype(bool), want), what
    else:
        d = compare_outputs({"y": want}, {"y": got.astype(np.float32)}, ["y"], tol)
        assert d.ok, (what, d.summary)


def _plan_and_emulate(js, bind, ins):
    desc = plan_json(js, bind)
    covered = all("program" in s or "row_program" in s or "args" in s for s in desc["steps"])
    if not covered:
        pytest.skip(f"the emulator does not cover {[s['kernel'] for s in desc['steps']]}")
    with np.errstate(all="ignore"):
        return desc, run_plan_description(desc, ins)


@pytest.mark.parametrize("key", _KEYS)
def test_recorded_graphs_plan_to_the_recorded_outputs(key, golden_graphs, golden_vectors):
    """Every graph recorded from the reference, at its recorded shapes, on its recorded inputs."""
    g = golden_graphs[key]
    ins = {n: golden_vectors[f"{key}/in/{n}"] for n in g["inputs"]}
    intent = IntentFunction.from_json_dict(g["intent"])
    desc, got = _plan_and_emulate(g["intent"], derive_bindings(dict(g["shapes"])), ins)
    tol = infer_tolerances(intent).to_dict()
    for n in g["outputs"]:
        _agree(got[n], golden_vectors[f"{key}/out/{n}"], tol, (key, n, [s["kernel"] for s in desc["steps"]]))


def test_sweep_families_plan_to_what_the_oracle_computes():
    """The verification sweep's graph families (headline and extra ones) at small seeded sizes, f32 and bf16."""
    from intent_ir_b200.sweep import ALL_KINDS

    seen = {}
    for c in generate_sweep_cases(260, base_seed=4242, max_elements=1 << 12, kinds=ALL_KINDS):
        if seen.get((c.kind, c.dtype), 0) >= 3 or c.kind in ("rope", "dropout", "image"):
            continue
        seen[(c.kind, c.dtype)] = seen.get((c.kind, c.dtype), 0) + 1
        bind = derive_bindings(dict(c.shapes))
        ins = case_inputs(c)
        intent = IntentFunction.from_json_dict(c.intent)
        desc = plan_json(c.intent, bind)
        with np.errstate(all="ignore"):
            got = run_plan_description(desc, ins)
            want = execute_intent(intent, ins, shape_bindings=bind)
        tol = infer_tolerances(intent).to_dict()
        for n in intent.outputs:
            _agree(got[n], want[n], tol, (c.kind, c.dtype, c.shapes, n, [s["kernel"] for s in desc["steps"]]))
    assert len({k for k, _ in seen}) >= 10, seen


@pytest.mark.parametrize("shape,axis", [((4, 100, 64), 1), ((40, 64), 0), ((3, 7, 5, 33), 2), ((2, 1, 300, 17), -2), ((1, 2, 3), 0), ((5, 8), -1)])
def test_softmax_over_any_axis(shape, axis):
    syms = [f"D{i}" for i in range(len(shape))]
    js = {"name": "sm_axis", "tensors": {"x": _t(syms), "y": _t(syms)},
          "ops": [{"op": "softmax", "inputs": ["x"], "output": "y", "attrs": {"axis": axis}}], "outputs": ["y"]}
    bind = dict(zip(syms, shape))
    x = 3 * np.random.default_rng(sum(shape)).standard_normal(shape).astype(np.float32)
    if x.size > 10:
        x.reshape(-1)[3] = -np.inf
    intent = IntentFunction.from_json_dict(js)
    desc, got = _plan_and_emulate(js, bind, {"x": x})
    with np.errstate(all="ignore"):
        want = execute_intent(intent, {"x": x}, bind)["y"]
    _agree(got["y"], want, infer_tolerances(intent).to_dict(), [s["kernel"] for s in desc["steps"]])


@pytest.mark.parametrize("op", ["reduce_sum", "reduce_max", "reduce_any"])
@pytest.mark.parametrize("shape,dims,keepdims", [((4, 10, 6, 8), [0, 2], False), ((4, 10, 6, 8), [1, 3], True), ((3, 5, 7, 2, 9), [0, 2, 4], False),
                                                 ((33, 1, 17, 65), [0, 2], False), ((2, 3, 4), [0, 2], True), ((6, 7), [0], False), ((6, 7), [0, 1], True)])
def test_reductions_over_any_set_of_axes(op, shape, dims, keepdims):
    syms = [f"D{i}" for i in range(len(shape))]
    out_shape = [1 if i in dims else s for i, s in enumerate(syms) if keepdims or i not in dims]
    js = {"name": "r", "tensors": {"x": _t(syms), "y": _t(out_shape, "bool" if op == "reduce_any" else "f32")},
          "ops": [{"op": op, "inputs": ["x"], "output": "y", "attrs": {"dims": dims, "keepdims": keepdims}}], "outputs": ["y"]}
    bind = dict(zip(syms, shape))
    rng = np.random.default_rng(sum(shape) + len(dims))
    x = rng.standard_normal(shape).astype(np.float32)
    if op == "reduce_any":
        x = np.where(rng.random(shape) < 0.05, x, np.float32(0))
    intent = IntentFunction.from_json_dict(js)
    desc, got = _plan_and_emulate(js, bind, {"x": x})
    with np.errstate(all="ignore"):
        want = execute_intent(intent, {"x": x}, bind)["y"]
    _agree(got["y"], want, infer_tolerances(intent).to_dict(), (op, [s["kernel"] for s in desc["steps"]]))


def test_damaged_graphs_that_still_plan_keep_the_oracles_meaning(golden_graphs):
    """Seeded structural damage to the recorded graphs: most is refused; what still plans (a changed axis, attribute,
    operand or shape that happens to be valid) must compute what the oracle computes for the damaged graph -- nothing
    is silently read as something else.  (A result is stored with its declared type, which the interpreter does not
    model: results whose declaration was damaged, or that no longer hold the declared kind of value, are left out.)"""
    import copy
    import random

    junk = [None, True, -1, 0, 2, 3, 1.5, "", "f16", "i32", "bool", "f32", "softmax", "add", "mul", "max", "exp", "relu", [], [0], [1], [-1], [0, 1],
            "M", "N", ["M"], ["N"], ["M", "N"], ["N", "M"], [1, "N"], ["M", 1]]
    symbols = "M N K C HW num_groups Z Q_CTX KV_CTX HEAD_DIM q_numhead kv_numhead B H W D S".split()
    np_of = {"f32": np.float32, "f16": np.float16, "bf16": np.float32, "i32": np.int32, "i64": np.int64, "bool": np.bool_, "i8": np.int8,
             "u8": np.uint8, "f64": np.float64, "i16": np.int16}

    def paths(o, p=()):
        if p:
            yield p
        for k in (o if isinstance(o, dict) else range(len(o)) if isinstance(o, list) else ()):
            yield from paths(o[k], p + (k,))

    keys = sorted(golden_graphs)
    agreed = refused = 0
    for i in range(700):
        rng = random.Random(i)
        original = golden_graphs[keys[i % len(keys)]]["intent"]
        js = copy.deepcopy(original)
        for _ in range(rng.choice([1, 1, 2])):
            p = rng.choice(list(paths(js)))
            parent = js
            for k in p[:-1]:
                parent = parent[k]
            if rng.random() < 0.15:
                del parent[p[-1]]
            else:
                parent[p[-1]] = copy.deepcopy(rng.choice(junk))
        bind = {s: rng.choice([1, 2, 3, 4, 6, 8, 16]) for s in symbols}
        try:
            desc = plan_json(js, bind)
        except B200LoweringError:
            refused += 1
            continue
        if not all("program" in s or "row_program" in s or "args" in s for s in desc["steps"]):
            continue
        spec, outs = desc["io_spec"]["tensors"], desc["output_names"]
        if any((js.get("tensors", {}).get(n) or {}).get("dtype") != (original["tensors"].get(n) or {}).get("dtype") for n in outs):
            continue
        nrng = np.random.default_rng(i)
        ins = {}
        for n in desc["io_spec"]["arg_names"]:
            if n not in outs:
                t = spec[n]
                a = nrng.integers(0, 2, t["shape"]) if t["dtype"][0] in "iub" else nrng.integers(-8, 9, t["shape"]) / 4.0
                ins[n] = np.asarray(a).astype(np_of[t["dtype"]])
        try:
            with np.errstate(all="ignore"):
                want = execute_intent(IntentFunction.from_json_dict(js), ins, dict(desc["bindings"]))
        except Exception:
            continue  # (the interpreter has no answer to compare with)
        with np.errstate(all="ignore"):
            got = run_plan_description(desc, ins)
        for n in outs:
            w, g = np.asarray(want[n]), np.asarray(got[n])
            assert g.shape == w.shape, (i, n)
            if w.dtype.kind != np.dtype(np_of[spec[n]["dtype"]]).kind:
                continue  # (the damage made an op compute another kind of value than the result is declared to hold)
            if w.dtype == np.bool_:
                assert np.array_equal(g.astype(bool), w), (i, keys[i % len(keys)], n)
            else:
                assert np.allclose(g.astype(np.float64), w.astype(np.float64), rtol=1e-4, atol=1e-5, equal_nan=True), (i, keys[i % len(keys)], n)
        agreed += 1
    assert refused > 400 and agreed > 40, (refused, agreed)


@pytest.mark.parametrize("what,shapes", [("softmax", {"M": 4, "N": 1 << 18}), ("layernorm", {"M": 3, "N": 200_000}), ("reduce_sum", {"M": 2, "N": 1 << 19}),
                                         ("reduce_max", {"M": 70_000, "N": 5}), ("matmul_bias_relu", {"M": 300, "N": 40, "K": 2000}),
                                         ("groupnorm", {"N": 2, "C": 8, "HW": 70_000, "num_groups": 2})])
def test_plans_of_shapes_that_take_the_split_forms(what, shapes):
    """Few very long rows (segments over the whole GPU, scratch in the workspace), tall column reductions, a product
    with a long K: the planner's choices for such shapes change kernels and add scratch buffers, not meaning."""
    from intent_ir_b200 import sweep

    maker = {"softmax": lambda: sweep.g_softmax("f32"), "layernorm": sweep.g_layernorm, "groupnorm": sweep.g_groupnorm,
             "reduce_sum": lambda: sweep.g_reduce("reduce_sum", "f32"), "reduce_max": lambda: sweep.g_reduce("reduce_max", "f32"),
             "matmul_bias_relu": lambda: sweep.g_matmul("f32")}[what]
    js = maker()
    bind = derive_bindings(dict(shapes))
    intent = IntentFunction.from_json_dict(js)
    rng = np.random.default_rng(7)
    desc = plan_json(js, bind)
    spec, outs = desc["io_spec"]["tensors"], desc["output_names"]
    ins = {n: rng.standard_normal(spec[n]["shape"]).astype(np.float32) for n in desc["io_spec"]["arg_names"] if n not in outs}
    with np.errstate(all="ignore"):
        got = run_plan_description(desc, ins)
        want = execute_intent(intent, ins, shape_bindings=bind)
    tol = infer_tolerances(intent).to_dict()
    for n in intent.outputs:
        _agree(got[n], want[n], tol, (what, n, [s["kernel"] for s in desc["steps"]], desc["workspace_bytes"]))


@pytest.mark.parametrize("seed", range(24))
@pytest.mark.parametrize("finish", ["transcendental", "reduce", "softmax_matmul"])
def test_fuzzed_graphs_with_tails_plan_to_what_the_oracle_computes(seed, finish):
    """Random DAGs finished by exp / rsqrt / div, by row, column and any-reductions, or by a softmax and a product with
    its own transpose: the exact part bit for bit, the rest within the verifier's tolerances."""
    from tests.test_fuzz_gpu import _inputs, random_elementwise_graph

    rng = np.random.default_rng(1000 + seed)
    m, n = [(2, 3), (9, 40), (17, 128), (64, 257), (130, 72)][seed % 5]
    js = random_elementwise_graph(rng, int(rng.integers(1, 9)), finish=finish)
    intent = IntentFunction.from_json_dict(js)
    ins = _inputs(rng, m, n)
    with np.errstate(all="ignore"):
        want = execute_intent(intent, ins, {"M": m, "N": n})
    desc, got = _plan_and_emulate(js, {"M": m, "N": n}, ins)
    tol = infer_tolerances(intent).to_dict()
    for name in intent.outputs:
        w, g = np.asarray(want[name]), np.asarray(got[name])
        assert g.shape == w.shape, (seed, name)
        if w.dtype == np.bool_ or name in ("Y", "P", "A"):
            assert np.array_equal(g.astype(w.dtype), w, equal_nan=w.dtype.kind == "f"), (seed, finish, name, [s["kernel"] for s in desc["steps"]])
        else:
            _agree(g, w, tol, (seed, finish, name, [s["kernel"] for s in desc["steps"]]))
