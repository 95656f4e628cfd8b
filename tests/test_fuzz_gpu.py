"""Seeded random IntentIR graphs through the whole path (planner -> micro-op programs, reductions,
softmax, matmul) against the CPU oracle.  Elementwise arithmetic that is exactly rounded on both
sides (add / sub / mul / max / min / abs / relu, comparisons, boolean logic, where) must agree
bit for bit; graphs that end in exp / rsqrt / div / reductions are held to the oracle's inferred
tolerances."""

import numpy as np
import pytest

from intent_ir_b200.ir import IntentFunction
from oracle import execute_intent, infer_tolerances
from oracle.diff import compare_outputs

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

EXACT_BIN = ["add", "sub", "mul", "max", "min"]
EXACT_UN = ["abs", "relu", "identity"]
CMP = ["lt", "le", "gt", "ge", "ne"]


def _t(shape, dtype="f32"):
    return {"dtype": dtype, "shape": list(shape), "layout": "row_major"}


def random_elementwise_graph(rng, n_ops, finish=None):
    """A DAG over x[M,N], col[N], row[M,1], lead[1,N], s[] with reuse of intermediates and up to three
    outputs (float, bool, and an optional transcendental tail)."""
    tensors = {"x": _t(["M", "N"]), "col": _t(["N"]), "row": _t(["M", 1]), "lead": _t([1, "N"]), "s": _t([])}
    floats, bools, ops = ["x", "col", "row", "lead", "s"], [], []
    full_float = ["x"]  # values known to have the full [M,N] shape
    full = {"x"}

    def fresh(prefix):
        return f"{prefix}{len(ops)}"

    for _ in range(n_ops):
        kind = rng.choice(["bin", "bin", "bin", "un", "cmp", "logic", "where", "attr"])
        if kind == "bin":
            a, b = rng.choice(floats), rng.choice(floats)
            out = fresh("f")
            ops.append({"op": str(rng.choice(EXACT_BIN)), "inputs": [str(a), str(b)], "output": out})
            floats.append(out)
            if a in full or b in full:
                full.add(out); full_float.append(out)
        elif kind == "un":
            a = rng.choice(floats)
            out = fresh("f")
            ops.append({"op": str(rng.choice(EXACT_UN)), "inputs": [str(a)], "output": out})
            floats.append(out)
            if a in full:
                full.add(out); full_float.append(out)
        elif kind == "attr":
            a = rng.choice(floats)
            op, key = [("add", "addend"), ("sub", "subtract"), ("mul", "mul_factor"), ("max", "other"), ("min", "other")][int(rng.integers(0, 5))]
            out = fresh("f")
            ops.append({"op": op, "inputs": [str(a)], "output": out, "attrs": {key: float(rng.choice([-1.5, -0.25, 0.5, 2.0]))}})
            floats.append(out)
            if a in full:
                full.add(out); full_float.append(out)
        elif kind == "cmp":
            a, b = rng.choice(floats), rng.choice(floats)
            out = fresh("b")
            ops.append({"op": str(rng.choice(CMP)), "inputs": [str(a), str(b)], "output": out})
            bools.append(out)
            if a in full or b in full:
                full.add(out)
        elif kind == "logic" and bools:
            if rng.random() < 0.3:
                a = rng.choice(bools)
                out = fresh("b")
                ops.append({"op": "not", "inputs": [str(a)], "output": out})
                if a in full:
                    full.add(out)
            else:
                a, b = rng.choice(bools), rng.choice(bools)
                out = fresh("b")
                ops.append({"op": str(rng.choice(["and", "or"])), "inputs": [str(a), str(b)], "output": out})
                if a in full or b in full:
                    full.add(out)
            bools.append(out)
        elif kind == "where" and bools:
            c, a, b = rng.choice(bools), rng.choice(floats), rng.choice(floats)
            out = fresh("f")
            ops.append({"op": "where", "inputs": [str(c), str(a), str(b)], "output": out})
            floats.append(out)
            if c in full or a in full or b in full:
                full.add(out); full_float.append(out)
    outputs = []
    # a full-shape float output that keeps several of the walk's values live
    live = [f for f in dict.fromkeys(reversed(full_float)) if f != "x"][:4]
    ops.append({"op": "add", "inputs": ["x", str(rng.choice(floats))], "output": "yf"})
    y = "yf"
    for i, f in enumerate(live):
        ops.append({"op": "add" if i % 2 == 0 else "max", "inputs": [y, f], "output": f"yl{i}"})
        y = f"yl{i}"
    ops.append({"op": "identity", "inputs": [y], "output": "Y"})
    tensors["Y"] = _t(["M", "N"])
    outputs.append("Y")
    full_bools = [b for b in bools if b in full]
    if full_bools:
        ops.append({"op": "identity", "inputs": [str(full_bools[-1])], "output": "P"})
        tensors["P"] = _t(["M", "N"], "bool")
        outputs.append("P")
    if finish == "transcendental":
        ops += [{"op": "min", "inputs": ["Y"], "output": "yc", "attrs": {"other": 3.0}},
                {"op": "exp", "inputs": ["yc"], "output": "ye"},
                {"op": "add", "inputs": ["ye"], "output": "yp", "attrs": {"addend": 0.5}},
                {"op": "rsqrt", "inputs": ["yp"], "output": "yr"},
                {"op": "div", "inputs": ["yr", "yp"], "output": "Z"}]
        tensors["Z"] = _t(["M", "N"])
        outputs.append("Z")
    elif finish == "reduce":
        ops += [{"op": "reduce_sum", "inputs": ["Y"], "output": "S", "attrs": {"dims": [1]}},
                {"op": "reduce_max", "inputs": ["Y"], "output": "Mx", "attrs": {"dims": [0], "keepdims": True}}]
        tensors["S"] = _t(["M"])
        tensors["Mx"] = _t([1, "N"])
        outputs += ["S", "Mx"]
        if full_bools:
            ops.append({"op": "reduce_any", "inputs": ["P"], "output": "A", "attrs": {"dims": [1]}})
            tensors["A"] = _t(["M"], "bool")
            outputs.append("A")
    elif finish == "softmax_matmul":
        ops += [{"op": "max", "inputs": ["Y"], "output": "yl", "attrs": {"other": -8.0}},
                {"op": "min", "inputs": ["yl"], "output": "yh", "attrs": {"other": 8.0}},
                {"op": "softmax", "inputs": ["yh"], "output": "sm", "attrs": {"axis": -1}},
                {"op": "matmul", "inputs": ["sm", "yh"], "output": "Q", "attrs": {"transpose_b": True}}]
        tensors["Q"] = _t(["M", "M"])
        outputs.append("Q")
    return {"name": "fuzz", "tensors": tensors, "ops": ops, "outputs": outputs}


def _inputs(rng, m, n):
    # small dyadic values: sums and products stay exactly representable, so ties in max / min /
    # comparisons resolve identically on both sides
    grid = lambda shape: (rng.integers(-8, 9, size=shape) / 4.0).astype(np.float32)  # noqa: E731
    return {"x": grid((m, n)), "col": grid((n,)), "row": grid((m, 1)), "lead": grid((1, n)), "s": grid(())}


@pytest.mark.parametrize("seed", range(40))
def test_random_elementwise_dags_are_bit_exact(seed):
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel
    from intent_ir_b200.runtime import run_lowered

    rng = np.random.default_rng(seed)
    m, n = [(1, 1), (3, 5), (7, 64), (33, 100), (16, 256), (5, 1028), (600, 9)][seed % 7]
    js = random_elementwise_graph(rng, int(rng.integers(2, 14)))
    intent = IntentFunction.from_json_dict(js)
    ins = _inputs(rng, m, n)
    with np.errstate(all="ignore"):
        want = execute_intent(intent, ins, {"M": m, "N": n})
    lowered = lower_intent_to_b200_kernel(intent, shape_bindings={"M": m, "N": n})
    got = run_lowered(lowered, ins)
    for name in intent.outputs:
        w = np.asarray(want[name])
        assert got[name].shape == w.shape, (seed, name)
        assert np.array_equal(got[name], w.astype(got[name].dtype), equal_nan=got[name].dtype.kind == "f"), \
            (seed, name, [o["op"] for o in js["ops"]], [s["kernel"] for s in lowered.steps])


@pytest.mark.parametrize("seed", range(24))
@pytest.mark.parametrize("finish", ["transcendental", "reduce", "softmax_matmul"])
def test_random_graphs_with_tails_within_tolerance(seed, finish):
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel
    from intent_ir_b200.runtime import run_lowered

    rng = np.random.default_rng(1000 + seed)
    m, n = [(2, 3), (9, 40), (17, 128), (64, 257), (130, 72)][seed % 5]
    js = random_elementwise_graph(rng, int(rng.integers(1, 9)), finish=finish)
    intent = IntentFunction.from_json_dict(js)
    ins = _inputs(rng, m, n)
    with np.errstate(all="ignore"):
        want = execute_intent(intent, ins, {"M": m, "N": n})
    lowered = lower_intent_to_b200_kernel(intent, shape_bindings={"M": m, "N": n})
    got = run_lowered(lowered, ins)
    tol = infer_tolerances(intent).to_dict()
    for name in intent.outputs:
        w, g = np.asarray(want[name]), got[name]
        assert g.shape == w.shape, (seed, name)
        if w.dtype == np.bool_ or name in ("Y", "P", "A"):
            assert np.array_equal(g, w.astype(g.dtype)), (seed, finish, name)
        else:
            d = compare_outputs({"y": w}, {"y": g}, ["y"], tol)
            assert d.ok, (seed, finish, name, d.summary, d.max_abs_err, [s["kernel"] for s in lowered.steps])
