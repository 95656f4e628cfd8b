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


def _random_graph(rng):
    """A chain of up to six random ops over a tensor of rank 1-4 with literal extents: elementwise ops against tensors
    of the same shape, broadcast vectors and constants, reductions over any subset of axes, softmax over any axis,
    permutations, reshapes (merging, splitting, with a -1), broadcasts into a new axis, products with a weight
    (plain or transposed) and comparisons feeding a `where`."""
    grid = lambda shape, hi=8: (rng.integers(-hi, hi + 1, size=shape) / 4.0).astype(np.float32)  # noqa: E731
    shape = [int(rng.choice([1, 2, 3, 4, 5, 7, 8, 16, 33])) for _ in range(int(rng.integers(1, 5)))]
    tensors, ins, ops = {"x": _t(shape)}, {"x": grid(shape)}, []
    cur, known = "x", {"x": list(shape)}

    def emit(op, inputs, attrs=None):
        nonlocal cur
        out = f"v{len(ops)}"
        ops.append({"op": op, "inputs": inputs, "output": out, **({"attrs": attrs} if attrs else {})})
        cur = out
        known[out] = list(shape)

    for _ in range(int(rng.integers(1, 7))):
        kind = rng.choice(["unary", "same", "vector", "attr", "reduce", "softmax", "transpose", "reshape", "broadcast", "matmul", "where"])
        if kind == "unary":
            emit(str(rng.choice(["relu", "abs", "exp", "floor"])), [cur])
        elif kind == "same":
            emit(str(rng.choice(["add", "sub", "mul", "max", "min"])), [cur, str(rng.choice([n for n, s in known.items() if s == shape]))])
        elif kind == "vector" and shape:
            name, vs = f"w{len(ops)}", [shape[-1]] if rng.random() < 0.6 else [c if rng.random() < 0.5 else 1 for c in shape]
            tensors[name], ins[name] = _t(vs), grid(vs)
            emit(str(rng.choice(["add", "sub", "mul", "max"])), [cur, name] if rng.random() < 0.7 else [name, cur])
        elif kind == "attr":
            op, key = [("add", "addend"), ("sub", "subtract"), ("mul", "mul_factor"), ("max", "other"), ("min", "other")][int(rng.integers(0, 5))]
            emit(op, [cur], {key: float(rng.choice([-1.5, -0.25, 0.5, 2.0]))})
        elif kind == "reduce" and shape:
            r = len(shape)
            dims = sorted(int(d) for d in rng.choice(r, size=int(rng.integers(1, r + 1)), replace=False))
            keep = bool(rng.random() < 0.5)
            shown = [d - r for d in dims] if rng.random() < 0.3 else dims
            shape = [1 if i in dims else s for i, s in enumerate(shape) if keep or i not in dims]
            emit(str(rng.choice(["reduce_sum", "reduce_max", "reduce_any"])), [cur], {"dims": shown, "keepdims": keep})
        elif kind == "softmax" and shape:
            emit("softmax", [cur], {"axis": int(rng.integers(-len(shape), len(shape)))})
        elif kind == "transpose" and len(shape) >= 2:
            perm = [int(p) for p in rng.permutation(len(shape))]
            shape = [shape[p] for p in perm]
            emit("transpose", [cur], {"perm": perm})
        elif kind == "reshape" and shape:
            if len(shape) >= 2 and rng.random() < 0.6:
                i = int(rng.integers(0, len(shape) - 1))
                new = shape[:i] + [shape[i] * shape[i + 1]] + shape[i + 2:]
            else:
                i = int(rng.integers(0, len(shape)))
                factors = [a for a in (2, 3, 4) if shape[i] % a == 0]
                if not factors or len(shape) >= 5:
                    continue
                a = int(rng.choice(factors))
                new = shape[:i] + [a, shape[i] // a] + shape[i + 1:]
            asked = list(new)
            if rng.random() < 0.3:
                asked[int(rng.integers(0, len(new)))] = -1
            shape = new
            emit("reshape", [cur], {"shape": asked})
        elif kind == "broadcast" and len(shape) <= 3:
            pos = int(rng.integers(0, len(shape) + 1))
            shape = shape[:pos] + [int(rng.choice([2, 3, 5]))] + shape[pos:]
            emit("broadcast_in_dim", [cur], {"out_shape": list(shape), "broadcast_dims": [i for i in range(len(shape)) if i != pos]})
        elif kind == "matmul" and len(shape) in (3, 4) and rng.random() < 0.7:  # batched, the weight shared or per batch
            name, n2 = f"b{len(ops)}", int(rng.choice([1, 3, 8]))
            bs = (shape[:-2] if rng.random() < 0.5 else []) + [shape[-1], n2]
            tensors[name], ins[name] = _t(bs), grid(bs, 4)
            shape = shape[:-1] + [n2]
            emit("matmul", [cur, name])
        elif kind == "matmul" and len(shape) == 2:
            name, n2, tb = f"b{len(ops)}", int(rng.choice([1, 3, 8, 17])), bool(rng.random() < 0.4)
            bs = [n2, shape[1]] if tb else [shape[1], n2]
            tensors[name], ins[name] = _t(bs), grid(bs, 4)
            shape = [shape[0], n2]
            emit("matmul", [cur, name], {"transpose_b": True} if tb else None)
        elif kind == "where" and shape:
            value = cur
            emit("const", [], {"value": 0.25, "dtype": "f32"})
            const = cur
            emit(str(rng.choice(["gt", "lt", "ne", "ge"])), [value, const])
            emit("where", [cur, value, const])
    if cur == "x":
        emit("relu", ["x"])
    return {"name": "random_graph", "tensors": tensors, "ops": ops, "outputs": [cur]}, ins


@pytest.mark.parametrize("block", range(6))
def test_random_graphs_plan_to_what_the_oracle_computes(block):
    """50 seeded random graphs per block: the plan, run step by step, agrees with the oracle within the verifier's
    tolerances (non-finite results: the same pattern, and the finite part within tolerance).  The result is declared
    with the shape and kind of value the interpreter gives; graphs numpy itself refuses (boolean subtraction, a maximum
    over nothing) are passed over, and so are the few the planner refuses by name."""
    ran = 0
    for seed in range(50 * block, 50 * block + 50):
        js, ins = _random_graph(np.random.default_rng(seed))
        last = js["outputs"][0]
        js["tensors"][last] = _t([1])  # (a placeholder: validation wants the output declared)
        try:
            with np.errstate(all="ignore"):
                want = np.asarray(execute_intent(IntentFunction.from_json_dict(json.loads(json.dumps(js))), ins, {})[last])
        except (TypeError, ValueError):
            continue
        if want.dtype == np.float64:  # (constants promote the interpreter's values; the declared type is f32)
            with np.errstate(over="ignore"):
                want = want.astype(np.float32)
        js["tensors"][last] = _t(want.shape, "bool" if want.dtype == np.bool_ else "f32")
        intent = IntentFunction.from_json_dict(json.loads(json.dumps(js)))
        try:
            desc = plan_json(js, {})
        except B200LoweringError as e:
            assert "non-float tensor" in str(e) or "boolean tensors" in str(e), (seed, str(e))
            continue
        kernels = [s["kernel"] for s in desc["steps"]]
        if not all("program" in s or "row_program" in s or "args" in s for s in desc["steps"]):
            continue
        with np.errstate(all="ignore"):
            got = np.asarray(run_plan_description(desc, ins)[js["outputs"][0]])
        what = (seed, [(o["op"], o.get("attrs")) for o in js["ops"]], js["tensors"]["x"]["shape"], kernels)
        assert list(got.shape) == list(want.shape), what
        if want.dtype == np.bool_:
            assert np.array_equal(got.astype(bool), want), what
            ran += 1
            continue
        finite = np.isfinite(want)
        if finite.all():
            _agree(got, want.astype(np.float32), infer_tolerances(intent).to_dict(), what)
        else:
            assert np.array_equal(np.isnan(want), np.isnan(got)) and np.array_equal(want[np.isinf(want)], got[np.isinf(want)]), what
            assert np.allclose(got[finite].astype(np.float32), want[finite], rtol=1e-3, atol=1e-3), what
        ran += 1
    assert ran >= 40


@pytest.mark.parametrize("m,n,k", [(5, 3, 0), (0, 3, 4), (5, 0, 4), (0, 0, 0)])
def test_products_with_an_empty_axis(m, n, k):
    """An empty contraction gives the bias (through the ReLU), empty results give nothing; none of them is a batch."""
    from intent_ir_b200 import sweep

    js = sweep.g_matmul("f32")
    rng = np.random.default_rng(m + 7 * n + 49 * k)
    ins = {"A": rng.standard_normal((m, k)).astype(np.float32), "B": rng.standard_normal((k, n)).astype(np.float32),
           "bias": rng.standard_normal((n,)).astype(np.float32)}
    desc, got = _plan_and_emulate(js, {"M": m, "N": n, "K": k}, ins)
    assert desc["steps"][0]["kernel"].startswith("gemm") and desc["steps"][0]["args"]["batch"] <= 1
    want = np.maximum(ins["A"] @ ins["B"] + ins["bias"], 0)
    assert np.array_equal(np.asarray(got["C"]).reshape(m, n), want)


def test_boolean_values_follow_numpy_through_arithmetic_and_sums():
    """`add` / `max` of two boolean tensors is "or", `mul` / `min` is "and" (the results stay boolean); the sum of
    booleans counts (an integer), so arithmetic on counts is arithmetic again; subtracting booleans is refused."""
    base = {"name": "b", "tensors": {"x": _t(["M", "N"]), "y": _t(["M", "N"])}, "outputs": ["y"]}
    x = (np.random.default_rng(5).integers(-1, 2, (6, 9)) / 2.0).astype(np.float32)

    def run(ops, out_shape, out_dtype="f32"):
        js = json.loads(json.dumps(base))
        js["ops"] = [{"op": "const", "inputs": [], "output": "z", "attrs": {"value": 0.0, "dtype": "f32"}},
                     {"op": "gt", "inputs": ["x", "z"], "output": "p"}, {"op": "lt", "inputs": ["x", "z"], "output": "q"}] + ops
        js["tensors"]["y"] = _t(out_shape, out_dtype)
        intent = IntentFunction.from_json_dict(js)
        desc, got = _plan_and_emulate(js, {"M": 6, "N": 9}, {"x": x})
        with np.errstate(all="ignore"):
            want = np.asarray(execute_intent(intent, {"x": x}, {"M": 6, "N": 9})["y"])
        return np.asarray(got["y"]).reshape(want.shape), want

    for op in ("add", "max", "mul", "min"):
        got, want = run([{"op": op, "inputs": ["p", "q"], "output": "pq"}, {"op": op, "inputs": ["pq", "p"], "output": "y"}], ["M", "N"], "bool")
        assert want.dtype == np.bool_ and np.array_equal(got.astype(bool), want), op
    got, want = run([{"op": "add", "inputs": ["p", "p"], "output": "pp"}, {"op": "add", "inputs": ["pp"], "output": "y", "attrs": {"addend": 2.0}}], ["M", "N"])
    assert np.array_equal(got.astype(np.float64), want.astype(np.float64))  # True + True is True, plus 2.0 is 3.0
    try:  # (counting booleans is refused where no fused row program takes it; where it plans, it counts)
        got, want = run([{"op": "reduce_any", "inputs": ["p"], "output": "a", "attrs": {"dims": [1]}},
                         {"op": "reduce_sum", "inputs": ["a"], "output": "c", "attrs": {"dims": [0]}},
                         {"op": "add", "inputs": ["c", "c"], "output": "y"}], [])
        assert want.dtype.kind == "i" and np.array_equal(got.astype(np.int64), want.astype(np.int64))
    except B200LoweringError as e:
        assert "non-float tensor" in str(e)
    with pytest.raises(B200LoweringError, match="boolean tensors"):
        run([{"op": "sub", "inputs": ["p", "q"], "output": "y"}], ["M", "N"])
