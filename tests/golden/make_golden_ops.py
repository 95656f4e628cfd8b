"""Golden vectors for the single-op kernels `rope`, `dropout`, `correlation`, `resize` and `warp`, from the reference checkout.

    python tests/golden/make_golden_ops.py /path/to/intent_ir

Records the outputs of the reference's own ``verify.interpreter.execute_intent``
(interpreter.py:455-477 rope, :303-329 and :697-742 dropout with its Philox-4x32 keep mask) for
seeded inputs into ``op_vectors.npz``; the graphs themselves go to ``op_intents.json``.  The
keep mask of dropout is pure integer arithmetic, so these vectors pin it bit for bit; so are the
int8 image ops (:330-454).
"""

from __future__ import annotations

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def _t(shape, dtype="f32"):
    return {"dtype": dtype, "shape": list(shape), "layout": "row_major"}


def rope_graph():
    return {"name": "rope4d", "tensors": {"x": _t(["S", "B", "H", "D"]), "cos": _t(["S", "D2"]), "sin": _t(["S", "D2"]), "y": _t(["S", "B", "H", "D"])},
            "ops": [{"op": "rope", "inputs": ["x", "cos", "sin"], "output": "y"}], "outputs": ["y"]}


def dropout_graph(seed_dtype="i32", n_rounds=None, rank2=False):
    shape = ["M", "N"] if rank2 else ["M"]
    attrs = {} if n_rounds is None else {"n_rounds": n_rounds}
    return {"name": "dropout", "tensors": {"x": _t(shape), "p": _t([]), "seed": _t([], seed_dtype), "y": _t(shape)},
            "ops": [{"op": "dropout", "inputs": ["x", "p", "seed"], "output": "y", "attrs": attrs}], "outputs": ["y"]}


def image_graph(op, attrs=None):
    if op == "correlation":
        return {"name": "correlation", "tensors": {"src0": _t(["C", "H", "W"], "i8"), "src1": _t(["C", "H", "W"], "i8"), "out_shift": _t([], "i32"),
                                                   "out": _t(["OC", "H", "W"], "i8")},
                "ops": [{"op": "correlation", "inputs": ["src0", "src1", "out_shift"], "output": "out"}], "outputs": ["out"]}
    if op == "resize":
        return {"name": "resize", "tensors": {"src": _t(["C", "H", "W"], "i8"), "out": _t(["C", "OH", "OW"], "i8")},
                "ops": [{"op": "resize", "inputs": ["src"], "output": "out", "attrs": attrs or {}}], "outputs": ["out"]}
    return {"name": "warp", "tensors": {"src": _t(["C", "H", "W"], "i8"), "offset": _t(["H", "W"], "i16"), "out": _t(["C", "H", "W"], "i8")},
            "ops": [{"op": "warp", "inputs": ["src", "offset"], "output": "out"}], "outputs": ["out"]}


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from intent_ir.ir import IntentFunction
    from verify.interpreter import execute_intent

    rng = np.random.default_rng(2024)
    graphs, vectors = {}, {}

    def record(key, js, shapes, inputs):
        intent = IntentFunction.from_json_dict(js)
        with np.errstate(all="ignore"):
            out = execute_intent(intent, inputs, shape_bindings=shapes)
        graphs[key] = {"intent": intent.to_json_dict(), "shapes": shapes, "inputs": list(inputs), "outputs": list(intent.outputs)}
        for n, v in inputs.items():
            vectors[f"{key}/in/{n}"] = np.asarray(v)
        for n in intent.outputs:
            vectors[f"{key}/out/{n}"] = np.asarray(out[n])

    for i, (s, b, h, d) in enumerate([(4, 1, 2, 8), (7, 2, 3, 6), (16, 2, 4, 64), (3, 1, 1, 2)]):
        ang = rng.uniform(-3.2, 3.2, (s, d // 2))
        record(f"rope_{i}", rope_graph(), {"S": s, "B": b, "H": h, "D": d, "D2": d // 2},
               {"x": rng.standard_normal((s, b, h, d), dtype=np.float32), "cos": np.cos(ang).astype(np.float32), "sin": np.sin(ang).astype(np.float32)})

    cases = [("i32", None, False, 1000, 0.1, 1234), ("i32", None, False, 4099, 0.5, 7), ("i64", None, True, (33, 65), 0.25, 2 ** 40 + 12345),
             ("i64", None, False, 257, 0.9, -5), ("i32", 7, False, 512, 0.3, 99), ("i32", 0, False, 130, 0.3, 99),
             ("i32", None, False, 64, 0.0, 3), ("i32", None, False, 64, 1.0, 3), ("i32", None, False, 64, 1.5, 3), ("i32", None, False, 64, -0.5, 3)]
    for i, (sd, rounds, rank2, shape, p, seed) in enumerate(cases):
        shp = shape if rank2 else (shape,)
        shapes = {"M": shp[0], "N": shp[1]} if rank2 else {"M": shp[0]}
        record(f"dropout_{i}", dropout_graph(sd, rounds, rank2), shapes,
               {"x": rng.standard_normal(shp, dtype=np.float32), "p": np.array(p, np.float32),
                "seed": np.array(seed, np.int64 if sd == "i64" else np.int32)})

    i8 = lambda shape: rng.integers(-128, 128, size=shape, dtype=np.int64).astype(np.int8)  # noqa: E731
    for i, (c, h, w, oc, shift) in enumerate([(4, 5, 16, 3, 2), (8, 3, 40, 8, 5), (1, 1, 7, 8, 0), (3, 6, 130, 5, 7)]):
        record(f"correlation_{i}", image_graph("correlation"), {"C": c, "H": h, "W": w, "OC": oc},
               {"src0": i8((c, h, w)), "src1": i8((c, h, w)), "out_shift": np.array(shift, np.int32)})
    for i, (c, h, w, fl) in enumerate([(2, 4, 6, None), (3, 7, 33, 7), (1, 1, 1, 7), (2, 5, 9, 4)]):
        record(f"resize_{i}", image_graph("resize", None if fl is None else {"hw_fl": fl}), {"C": c, "H": h, "W": w, "OH": 2 * h, "OW": 2 * w},
               {"src": i8((c, h, w))})
    for i, (c, h, w) in enumerate([(2, 3, 16), (3, 5, 100), (1, 2, 200), (4, 1, 1)]):
        off = rng.integers(-(3 << 8), 3 << 8, size=(h, w)).astype(np.int16)
        if i == 2:
            off = rng.integers(-32768, 32768, size=(h, w)).astype(np.int16)  # every wrap-around
        record(f"warp_{i}", image_graph("warp"), {"C": c, "H": h, "W": w}, {"src": i8((c, h, w)), "offset": off})

    with open(os.path.join(HERE, "op_intents.json"), "w") as f:
        json.dump(graphs, f, indent=1, sort_keys=True)
    np.savez_compressed(os.path.join(HERE, "op_vectors.npz"), **vectors)
    print(f"wrote {len(graphs)} graphs, {len(vectors)} arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden_ops.py /path/to/intent_ir")
    main(sys.argv[1])
