"""The planner's row-fusion pass, checked without a GPU: the fused row programs it emits are
executed by a numpy emulator (tests/rowprog_emulator.py) and compared with the oracle and with
the reference's golden outputs."""

import json

import numpy as np
import pytest

from intent_ir_b200.ir import IntentFunction
from intent_ir_b200.lowering import plan_json
from oracle import execute_intent, infer_tolerances
from oracle.diff import compare_outputs, derive_bindings
from tests.rowprog_emulator import run_plan_description
from tests.test_fuzz_gpu import _inputs, random_elementwise_graph

FUSED_GOLDEN = ["masked_softmax2d"]


def _check(intent, ins, bindings, expect_single=True):
    desc = plan_json(intent, bindings)
    kernels = [s["kernel"] for s in desc["steps"]]
    if expect_single:
        assert len(kernels) == 1 and kernels[0].startswith("rowfused"), kernels
    elif not all(k.startswith("rowfused") for k in kernels):
        pytest.skip(f"plan has unfused steps: {kernels}")
    with np.errstate(all="ignore"):
        want = execute_intent(intent, ins, shape_bindings=bindings)
    got = run_plan_description(desc, ins)
    tol = infer_tolerances(intent).to_dict()
    for name in intent.outputs:
        w, g = np.asarray(want[name]), got[name]
        assert g.shape == w.shape, name
        if w.dtype == np.bool_:
            assert np.array_equal(g.astype(bool), w), name
        else:
            d = compare_outputs({"y": w}, {"y": g.astype(np.float32)}, ["y"], tol)
            assert d.ok, (name, d.summary, kernels)
    return desc


@pytest.mark.parametrize("key", FUSED_GOLDEN)
def test_golden_graphs_fuse_into_one_row_program(key, golden_graphs, golden_vectors):
    """The reference's masked softmax with a per-row shift added before the mask: a softmax does
    not see a shift of its row, and masked entries underflow to zero either way, so the
    reference's recorded output still applies; the plain graph goes to the softmax kernel's own
    mask path and would not exercise a row program."""
    g = json.loads(json.dumps(golden_graphs[key]))
    js = g["intent"]
    js["tensors"]["row"] = _t(["M", 1])
    js["tensors"]["shifted"] = _t(["M", "N"])
    where = next(o for o in js["ops"] if o["op"] == "where")
    js["ops"].insert(js["ops"].index(where), {"op": "add", "inputs": [where["inputs"][1], "row"], "output": "shifted"})
    where["inputs"][1] = "shifted"
    intent = IntentFunction.from_json_dict(js)
    ins = {n: golden_vectors[f"{key}/in/{n}"] for n in g["inputs"]}
    ins["row"] = np.linspace(-2.0, 2.0, g["shapes"]["M"], dtype=np.float32).reshape(-1, 1)
    desc = _check(intent, ins, derive_bindings(g["shapes"]))
    got = run_plan_description(desc, ins)
    for n in g["outputs"]:
        want = golden_vectors[f"{key}/out/{n}"]
        assert np.allclose(got[n].astype(np.float32), want.astype(np.float32), rtol=1e-4, atol=1e-5, equal_nan=True), n


def _t(shape, dtype="f32"):
    return {"dtype": dtype, "shape": list(shape), "layout": "row_major"}


def _rms(m, n):
    """rms-norm with |x| between the scaling and the weight, so that no dedicated norm kernel's pattern applies (a ReLU
    there rides in the norm kernel)"""
    return {"name": "rms", "tensors": {"x": _t(["M", "N"]), "w": _t(["N"]), "y": _t(["M", "N"]), "rstd": _t(["M"])},
            "ops": [{"op": "mul", "inputs": ["x", "x"], "output": "sq"},
                    {"op": "reduce_sum", "inputs": ["sq"], "output": "ss", "attrs": {"dims": [1], "keepdims": True}},
                    {"op": "div", "inputs": ["ss"], "output": "ms", "attrs": {"divisor": "N"}},
                    {"op": "add", "inputs": ["ms"], "output": "me", "attrs": {"addend": 1e-5}},
                    {"op": "rsqrt", "inputs": ["me"], "output": "r1"},
                    {"op": "reshape", "inputs": ["r1"], "output": "rstd", "attrs": {"shape": ["M"]}},
                    {"op": "mul", "inputs": ["x", "r1"], "output": "xn"},
                    {"op": "abs", "inputs": ["xn"], "output": "xr"},
                    {"op": "mul", "inputs": ["xr", "w"], "output": "y"}], "outputs": ["y", "rstd"]}


def _log_softmax(m, n):
    return {"name": "lsm", "tensors": {"x": _t(["M", "N"]), "y": _t(["M", "N"])},
            "ops": [{"op": "reduce_max", "inputs": ["x"], "output": "mx", "attrs": {"dims": [1], "keepdims": True}},
                    {"op": "sub", "inputs": ["x", "mx"], "output": "xs"},
                    {"op": "exp", "inputs": ["xs"], "output": "e"},
                    {"op": "reduce_sum", "inputs": ["e"], "output": "se", "attrs": {"dims": [1], "keepdims": True}},
                    {"op": "div", "inputs": ["e", "se"], "output": "p"},
                    {"op": "mul", "inputs": ["p", "xs"], "output": "y"}], "outputs": ["y"]}


def _masked_softmax_rowstats(m, n):
    return {"name": "msm", "tensors": {"x": _t(["M", "N"]), "mask": _t(["M", "N"], "bool"), "row": _t(["M", 1]), "y": _t(["M", "N"]),
                                       "cnt": _t(["M"]), "anyneg": _t(["M"], "bool")},
            "ops": [{"op": "const", "inputs": [], "output": "neg", "attrs": {"value": -1e9, "dtype": "f32"}},
                    {"op": "add", "inputs": ["x", "row"], "output": "xr"},
                    {"op": "where", "inputs": ["mask", "xr", "neg"], "output": "xm"},
                    {"op": "softmax", "inputs": ["xm"], "output": "y", "attrs": {"axis": -1}},
                    {"op": "cast", "inputs": ["mask"], "output": "mf", "attrs": {"to": "f32"}},
                    {"op": "reduce_sum", "inputs": ["mf"], "output": "cnt", "attrs": {"dims": [1]}},
                    {"op": "const", "inputs": [], "output": "zero", "attrs": {"value": 0.0, "dtype": "f32"}},
                    {"op": "lt", "inputs": ["xr", "zero"], "output": "isneg"},
                    {"op": "reduce_any", "inputs": ["isneg"], "output": "anyneg", "attrs": {"dims": [1]}}],
            "outputs": ["y", "cnt", "anyneg"]}


@pytest.mark.parametrize("m,n", [(1, 8), (4, 64), (5, 7), (16, 16), (3, 130), (2, 1028)])
@pytest.mark.parametrize("build", [_rms, _log_softmax, _masked_softmax_rowstats])
def test_synthetic_row_graphs(build, m, n):
    js = build(m, n)
    intent = IntentFunction.from_json_dict(js)
    rng = np.random.default_rng(m * 1000 + n)
    ins = {}
    for name in intent.external_inputs() if hasattr(intent, "external_inputs") else []:
        t = js["tensors"][name]
        shape = [{"M": m, "N": n}.get(d, d) for d in t["shape"]]
        ins[name] = (rng.random(shape) > 0.3) if t["dtype"] == "bool" else rng.standard_normal(shape).astype(np.float32)
    _check(intent, ins, {"M": m, "N": n}, expect_single=False)


@pytest.mark.parametrize("seed", range(12))
@pytest.mark.parametrize("finish", ["reduce", "softmax_matmul"])
def test_fuzzed_graphs_keep_their_meaning_when_fused(seed, finish):
    """The fuzz graphs' row parts (a chain, then row reductions or a softmax) fuse; whatever is
    fused must leave every later consumer and every output unchanged.  Only plans that are
    fused end to end can be emulated here; the GPU suite runs all of them."""
    rng = np.random.default_rng(1000 + seed)
    m, n = [(2, 3), (9, 40), (17, 128), (4, 260), (13, 72)][seed % 5]
    js = random_elementwise_graph(rng, int(rng.integers(1, 9)), finish=finish)
    # keep only the row-wise tail so that the whole plan can fuse
    if finish == "reduce":
        js["ops"] = [o for o in js["ops"] if o["output"] != "Mx"]
        js["outputs"] = [o for o in js["outputs"] if o != "Mx"]
    else:
        js["ops"] = [o for o in js["ops"] if o["op"] != "matmul"]
        js["outputs"] = [o for o in js["outputs"] if o != "Q"] + ["sm"]
        js["tensors"]["sm"] = _t(["M", "N"])
    js["tensors"] = {k: v for k, v in js["tensors"].items() if k not in ("Mx", "Q")}
    intent = IntentFunction.from_json_dict(json.loads(json.dumps(js)))
    _check(intent, _inputs(rng, m, n), {"M": m, "N": n}, expect_single=False)
