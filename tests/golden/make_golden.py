"""Generate the golden fixtures in this directory from the reference checkout.

Run once, where the reference is available:

    python tests/golden/make_golden.py /path/to/intent_ir

It imports the reference's own ``verify.interpreter.execute_intent``,
``verify.diff_runner.run_diff``, ``verify.tolerances.infer_tolerances`` and
``verify.gen_cases.generate_cases`` and records what THEY return, so that the CPU oracle
under ``oracle/`` can be checked against the reference on machines that do not have it:

* ``../../intent_ir_b200/config_graphs.json`` — the subset of ``intents.json`` the benchmark runs;
* ``intents.json``      — IntentIR graphs (``IntentFunction.to_json_dict``) of the reference's
                          deterministic kernel specs and hand-written variants, with the
                          case shapes used;
* ``vectors.npz``       — per graph: seeded inputs, the derived bindings, and every output of
                          the reference interpreter;
* ``edge_cases.npz``    — NaN / ±Inf / −0 / denormal probes through the reference interpreter;
* ``verdicts.json``     — per graph: ``infer_tolerances`` (with and without ``ref_out``),
                          ``generate_cases`` shapes, and the ``run_diff`` verdict for an honest
                          and for a corrupted runner.
"""

from __future__ import annotations

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from intent_ir.ir import IntentFunction
    from pipeline.cuda.core import _deterministic_fallback_intent_for
    from pipeline.tilelang.core import coverage_kernel_specs
    from verify.diff_runner import run_diff
    from verify.gen_cases import TestCase, generate_cases
    from verify.interpreter import execute_intent
    from verify.tolerances import infer_tolerances

    sys.path.insert(0, os.path.join(HERE, "..", ".."))
    from oracle.diff import derive_bindings  # symbol derivation only; values come from the reference

    small = {
        "group_norm_kernel": {"N": 2, "C": 8, "HW": 16, "num_groups": 4},
        "flash_attention2d": {"Q_CTX": 16, "KV_CTX": 16, "HEAD_DIM": 16},
        "gather2d": {"M": 8, "N": 8, "L": 32},
    }

    graphs, vectors, verdicts = {}, {}, {}

    def record(key, intent, shapes, io, *, runner=None):
        bindings = derive_bindings(shapes)
        produced = {o.output for o in intent.ops}
        ext = [n for o in intent.ops for n in o.inputs if n in intent.tensors and n not in produced]
        inputs = {n: np.asarray(io[n]) for n in dict.fromkeys(ext) if n in io}
        with np.errstate(all="ignore"):
            outs = execute_intent(intent, inputs, shape_bindings=bindings)
        graphs[key] = {"intent": intent.to_json_dict(), "shapes": shapes,
                       "inputs": sorted(inputs), "outputs": list(intent.outputs)}
        for n, a in inputs.items():
            vectors[f"{key}/in/{n}"] = a
        for n, a in outs.items():
            vectors[f"{key}/out/{n}"] = np.asarray(a)
        v = {
            "tol_decl": infer_tolerances(intent).to_dict(),
            "tol_ref_out": infer_tolerances(intent, ref_out={**inputs, **outs}).to_dict(),
            "cases": [{k: int(x) for k, x in c.shapes.items()} for c in generate_cases(intent, limit=12, seed=3)],
        }
        honest = lambda case: {**inputs, **{k: np.asarray(x) for k, x in outs.items()}}  # noqa: E731
        d, cex = run_diff(intent, honest, [TestCase(shapes=shapes, dtypes={}, seed=0)])
        v["honest"] = {"ok": d[0].ok, "summary": d[0].summary, "n_cex": len(cex)}

        def corrupt(case):
            io2 = honest(case)
            first = intent.outputs[0]
            a = np.array(io2[first], copy=True)
            if a.dtype == bool:
                a.reshape(-1)[0] = ~a.reshape(-1)[0]
            else:
                a.reshape(-1)[-1] += 1.0
            io2[first] = a
            return io2

        d, cex = run_diff(intent, corrupt, [TestCase(shapes=shapes, dtypes={}, seed=0)])
        v["corrupt"] = {"ok": d[0].ok, "summary": d[0].summary, "n_cex": len(cex),
                        "first_bad_index": [int(i) for i in d[0].first_bad_index] if d[0].first_bad_index else None,
                        "max_abs_err": None if not np.isfinite(d[0].max_abs_err) else float(d[0].max_abs_err)}
        verdicts[key] = v

    for spec in coverage_kernel_specs():
        if spec.name == "upsample_bicubic2d_aa":
            continue
        intent = spec.intent_builder()
        shapes = dict(small.get(spec.name, spec.canonical_shapes))
        io = spec.runner(TestCase(shapes=shapes, dtypes={}, seed=11))
        if spec.name == "clamp2d":  # the spec's runner returns (1,) for rank-0 lo/hi
            io = {k: (np.asarray(v).reshape(()) if k in ("lo", "hi") else v) for k, v in io.items()}
        record(spec.name, intent, shapes, io)

    rng = np.random.default_rng(5)
    for name, shapes in (("softmax_inner", {"M": 5, "N": 37}), ("layer_norm_persistent", {"M": 6, "N": 40})):
        intent = _deterministic_fallback_intent_for(name)
        x = rng.standard_normal((shapes["M"], shapes["N"]), dtype=np.float32) * 2
        io = {"input_ptr": x} if name == "softmax_inner" else {
            "in_ptr": x, "weight_ptr": rng.standard_normal(shapes["N"], dtype=np.float32),
            "bias_ptr": rng.standard_normal(shapes["N"], dtype=np.float32)}
        record(f"{name}__cuda_pipeline_form", intent, shapes, io)

    hand = {
        "softmax_like_rowvec": ({
            "name": "softmax_like",
            "tensors": {n: {"dtype": "f32", "shape": s, "layout": "row_major"} for n, s in
                        {"X": ["M", "N"], "mx": ["M"], "Xc": ["M", "N"], "E": ["M", "N"], "sm": ["M"],
                         "out": ["M", "N"]}.items()},
            "ops": [
                {"op": "reduce_max", "inputs": ["X"], "output": "mx", "attrs": {"axis": [1], "keepdims": False}},
                {"op": "sub", "inputs": ["X", "mx"], "output": "Xc"},
                {"op": "exp", "inputs": ["Xc"], "output": "E"},
                {"op": "reduce_sum", "inputs": ["E"], "output": "sm", "attrs": {"axis": [1], "keepdims": False}},
                {"op": "div", "inputs": ["E", "sm"], "output": "out"}],
            "outputs": ["out"]}, {"M": 4, "N": 4}, lambda s: {"X": rng.standard_normal((4, 4), dtype=np.float32)}),
        "any_const_ne": ({
            "name": "any_dim",
            "tensors": {"A": {"dtype": "f32", "shape": ["M", "N"], "layout": "row_major"},
                        "z": {"dtype": "f32", "shape": [], "layout": "row_major"},
                        "T": {"dtype": "i1", "shape": ["M", "N"], "layout": "row_major"},
                        "Out": {"dtype": "i1", "shape": ["M"], "layout": "row_major"}},
            "ops": [{"op": "const", "inputs": [], "output": "z", "attrs": {"value": 0.0}},
                    {"op": "ne", "inputs": ["A", "z"], "output": "T", "attrs": {}},
                    {"op": "reduce_any", "inputs": ["T"], "output": "Out", "attrs": {"dims": [1]}}],
            "outputs": ["Out"]}, {"M": 8, "N": 8},
            lambda s: {"A": (rng.random((8, 8)) < 0.1).astype(np.float32)}),
        "reduce_forms": ({
            "name": "reduce_forms",
            "tensors": {"X": {"dtype": "f32", "shape": ["A", "B", "C"], "layout": "row_major"},
                        "s0": {"dtype": "f32", "shape": ["B", "C"], "layout": "row_major"},
                        "s12": {"dtype": "f32", "shape": ["A", 1, 1], "layout": "row_major"},
                        "mneg": {"dtype": "f32", "shape": ["A", "B"], "layout": "row_major"},
                        "sall": {"dtype": "f32", "shape": [], "layout": "row_major"},
                        "sscaled": {"dtype": "f32", "shape": ["A", "B"], "layout": "row_major"},
                        "anyleg": {"dtype": "bool", "shape": ["A", "C"], "layout": "row_major"}},
            "ops": [{"op": "reduce_sum", "inputs": ["X"], "output": "s0", "attrs": {"dims": [0]}},
                    {"op": "reduce_sum", "inputs": ["X"], "output": "s12", "attrs": {"dims": [1, 2], "keepdims": True}},
                    {"op": "reduce_max", "inputs": ["X"], "output": "mneg", "attrs": {"axis": -1}},
                    {"op": "reduce_sum", "inputs": ["X"], "output": "sall", "attrs": {"reduce_dims": [0]}},
                    {"op": "reduce_sum", "inputs": ["X"], "output": "sscaled", "attrs": {"dims": [2], "scale": "1.0/C"}},
                    {"op": "reduce_sum", "inputs": ["X"], "output": "anyleg", "attrs": {"dims": [1], "reduction_type": "any"}}],
            "outputs": ["s0", "s12", "mneg", "sall", "sscaled", "anyleg"]}, {"A": 3, "B": 5, "C": 7},
            lambda s: {"X": rng.standard_normal((3, 5, 7), dtype=np.float32)}),
        "scalar_attr_forms": ({
            "name": "scalar_attr_forms",
            "tensors": {"X": {"dtype": "f32", "shape": ["M", "N"], "layout": "row_major"},
                        "Y": {"dtype": "f32", "shape": ["M", "N"], "layout": "row_major"}},
            "ops": [{"op": "div", "inputs": ["X"], "output": "a", "attrs": {"divisor": "N"}},
                    {"op": "add", "inputs": ["a"], "output": "b", "attrs": {"addend": "0.25"}},
                    {"op": "sub", "inputs": ["b"], "output": "c", "attrs": {"subtract": 1.5}},
                    {"op": "const", "inputs": [], "output": "k", "attrs": {"value": "1.0/(N**0.5)", "dtype": "f32"}},
                    {"op": "mul", "inputs": ["c"], "output": "d", "attrs": {"mul_factor": "k"}},
                    {"op": "max", "inputs": ["d"], "output": "e", "attrs": {"other": -0.5}},
                    {"op": "mul", "inputs": ["e", "k"], "output": "f"},
                    {"op": "abs", "inputs": ["f"], "output": "g"},
                    {"op": "floor", "inputs": ["g"], "output": "h"},
                    {"op": "min", "inputs": ["f", "h"], "output": "Y"}],
            "outputs": ["Y"]}, {"M": 4, "N": 6},
            lambda s: {"X": 9 * rng.standard_normal((4, 6), dtype=np.float32)}),
        "bool_cast_forms": ({
            "name": "bool_cast_forms",
            "tensors": {"X": {"dtype": "f32", "shape": ["M", "N"], "layout": "row_major"},
                        "Y": {"dtype": "f32", "shape": ["M", "N"], "layout": "row_major"},
                        "P": {"dtype": "bool", "shape": ["M", "N"], "layout": "row_major"},
                        "Q": {"dtype": "f32", "shape": ["N", "M"], "layout": "row_major"},
                        "I": {"dtype": "i32", "shape": ["M", "N"], "layout": "row_major"}},
            "ops": [{"op": "lt", "inputs": ["X", "Y"], "output": "a"},
                    {"op": "ge", "inputs": ["X", "Y"], "output": "b"},
                    {"op": "not", "inputs": ["b"], "output": "nb"},
                    {"op": "and", "inputs": ["a", "nb"], "output": "c"},
                    {"op": "le", "inputs": ["X", "Y"], "output": "d"},
                    {"op": "or", "inputs": ["c", "d"], "output": "P"},
                    {"op": "where", "inputs": ["P", "X", "Y"], "output": "w"},
                    {"op": "transpose", "inputs": ["w"], "output": "Q", "attrs": {"perm": [1, 0]}},
                    {"op": "cast", "inputs": ["w"], "output": "I", "attrs": {"to": "i32"}}],
            "outputs": ["P", "Q", "I"]}, {"M": 3, "N": 5},
            lambda s: {"X": 4 * rng.standard_normal((3, 5), dtype=np.float32),
                       "Y": 4 * rng.standard_normal((3, 5), dtype=np.float32)}),
        "matmul_transposed_epilogue": ({
            "name": "matmul_te",
            "tensors": {"A": {"dtype": "f32", "shape": ["K", "M"], "layout": "row_major"},
                        "B": {"dtype": "f32", "shape": ["N", "K"], "layout": "row_major"},
                        "bias": {"dtype": "f32", "shape": ["N"], "layout": "row_major"},
                        "C": {"dtype": "f32", "shape": ["M", "N"], "layout": "row_major"}},
            "ops": [{"op": "identity", "inputs": ["bias"], "output": "bias_v"},
                    {"op": "matmul", "inputs": ["A", "B"], "output": "C",
                     "attrs": {"transpose_a": True, "transpose_b": True, "accum_dtype": "f32",
                               "epilogue": {"op": "relu", "inputs": [{"op": "add", "inputs": ["$x", "bias_v"]}]}}}],
            "outputs": ["C"]}, {"M": 5, "N": 6, "K": 7},
            lambda s: {"A": rng.standard_normal((7, 5), dtype=np.float32),
                       "B": rng.standard_normal((6, 7), dtype=np.float32),
                       "bias": rng.standard_normal(6, dtype=np.float32)}),
    }
    for key, (js, shapes, gen) in hand.items():
        record(key, IntentFunction.from_json_dict(js), shapes, gen(shapes))

    # ---- edge cases: one row each, through the single-op graphs -------------------------------
    def one_op(op, attrs, out_dtype="f32", out_shape=("M", "N")):
        return IntentFunction.from_json_dict({
            "name": f"edge_{op}",
            "tensors": {"x": {"dtype": "f32", "shape": ["M", "N"], "layout": "row_major"},
                        "y": {"dtype": out_dtype, "shape": list(out_shape), "layout": "row_major"}},
            "ops": [{"op": op, "inputs": ["x"], "output": "y", "attrs": attrs}], "outputs": ["y"]})

    nan, inf = np.float32(np.nan), np.float32(np.inf)
    probes = np.array([
        [1, 2, inf, 4], [1, nan, 2, 3], [-inf, -inf, -inf, -inf], [1, -inf, 2, 3],
        [0, -0.0, 0, 0], [0, nan, 0, 0], [0, 1e-45, 0, 0], [-1, nan, inf, -inf], [1, 2, 3, 4],
    ], dtype=np.float32)
    edge = {"x": probes}
    with np.errstate(all="ignore"):
        for tag, intent in (
            ("softmax", one_op("softmax", {"axis": -1})),
            ("reduce_any", one_op("reduce_any", {"dims": [1]}, "bool", ("M",))),
            ("reduce_max", one_op("reduce_max", {"dims": [1]}, "f32", ("M",))),
            ("reduce_sum", one_op("reduce_sum", {"dims": [1]}, "f32", ("M",))),
            ("relu", one_op("relu", {})),
            ("exp", one_op("exp", {})),
            ("rsqrt", one_op("rsqrt", {})),
        ):
            edge[tag] = np.asarray(execute_intent(intent, {"x": probes})["y"])

    with open(os.path.join(HERE, "intents.json"), "w") as f:
        json.dump(graphs, f, indent=1, sort_keys=True)
    # the benchmark configurations' graphs also ship inside the package (bench.py and the smoke entry read them there)
    config_keys = ["any_kernel_dim", "softmax_inner", "layer_norm_persistent", "group_norm_kernel", "matmul_bias_relu2d", "add_bias2d",
                   "rms_norm2d", "layer_norm_residual2d", "masked_softmax2d"]
    with open(os.path.join(HERE, "..", "..", "intent_ir_b200", "config_graphs.json"), "w") as f:
        json.dump({k: graphs[k]["intent"] for k in config_keys}, f, indent=0, sort_keys=True)
    with open(os.path.join(HERE, "verdicts.json"), "w") as f:
        json.dump(verdicts, f, indent=1, sort_keys=True)
    np.savez_compressed(os.path.join(HERE, "vectors.npz"), **vectors)
    np.savez_compressed(os.path.join(HERE, "edge_cases.npz"), **edge)
    print(f"wrote {len(graphs)} graphs, {len(vectors)} arrays, {len(edge) - 1} edge probes; numpy {np.__version__}")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("INTENTIR_REF", ""))


def validation_cases():
    """Graphs that the reference's IntentFunction.from_json_dict must accept or reject."""
    T = lambda shape, dtype="f32", **kw: dict({"dtype": dtype, "shape": shape, "layout": "row_major"}, **kw)  # noqa: E731
    base = {"name": "g", "tensors": {"x": T(["M", "N"]), "y": T(["M", "N"])},
            "ops": [{"op": "relu", "inputs": ["x"], "output": "y"}], "outputs": ["y"]}

    def variant(**patch):
        import copy
        g = copy.deepcopy(base)
        for k, v in patch.items():
            g[k] = v
        return g

    op = lambda **kw: [dict({"op": "relu", "inputs": ["x"], "output": "y"}, **kw)]  # noqa: E731
    return {
        "ok_minimal": base,
        "ok_outputs_default": {k: v for k, v in base.items() if k != "outputs"},
        "ok_layout_dense": variant(tensors={"x": T(["M", "N"], layout="dense"), "y": T(["M", "N"])}),
        "ok_reduce_dims_alias": variant(tensors={"x": T(["M", "N"]), "y": T(["M"])}, ops=op(op="reduce_sum", attrs={"reduce_dims": [1]})),
        "ok_reduce_axis_int": variant(tensors={"x": T(["M", "N"]), "y": T(["M"])}, ops=op(op="reduce_max", attrs={"axis": 1})),
        "ok_div_scalar_attr": variant(ops=op(op="div", attrs={"divisor": "N"})),
        "bad_unknown_op": variant(ops=op(op="frobnicate")),
        "bad_undefined_input": variant(ops=op(inputs=["nope"])),
        "bad_duplicate_output": variant(ops=op() + op()),
        "bad_empty_ops": variant(ops=[]),
        "bad_output_undeclared": variant(outputs=["zzz"]),
        "bad_dtype": variant(tensors={"x": T(["M"], "f8"), "y": T(["M"])}),
        "bad_layout": variant(tensors={"x": T(["M"], layout="zigzag"), "y": T(["M"])}),
        "bad_shape_type": variant(tensors={"x": T([1.5]), "y": T(["M"])}),
        "bad_reduce_no_dims": variant(ops=op(op="reduce_sum", attrs={})),
        "bad_reduce_dims_type": variant(ops=op(op="reduce_sum", attrs={"dims": ["N"]})),
        "bad_softmax_no_axis": variant(ops=op(op="softmax", attrs={})),
        "bad_softmax_axis_type": variant(ops=op(op="softmax", attrs={"axis": "1"})),
        "bad_matmul_arity": variant(ops=op(op="matmul")),
        "bad_matmul_accum": variant(ops=op(op="matmul", inputs=["x", "x"], attrs={"accum_dtype": "f8"})),
        "bad_matmul_epilogue_op": variant(ops=op(op="matmul", inputs=["x", "x"], attrs={"epilogue": {"op": "erf", "inputs": ["$x"]}})),
        "bad_const_inputs": variant(ops=op(op="const", attrs={"value": 1})),
        "bad_const_no_value": variant(ops=op(op="const", inputs=[], attrs={})),
        "bad_cast_no_to": variant(ops=op(op="cast", attrs={"dtype": "f16"})),
        "bad_identity_attrs": variant(ops=op(op="identity", attrs={"slice": [0, 1]})),
        "bad_add_arity": variant(ops=op(op="add")),
        "bad_where_arity": variant(ops=op(op="where", inputs=["x", "x"])),
        "bad_broadcast_no_shape": variant(ops=op(op="broadcast_in_dim", attrs={"broadcast_dims": [0]})),
        "bad_broadcast_dims_type": variant(ops=op(op="broadcast_in_dim", attrs={"out_shape": ["M", "N"], "broadcast_dims": ["a"]})),
        "bad_transpose_perm": variant(ops=op(op="transpose", attrs={"perm": []})),
        "bad_reshape_shape": variant(ops=op(op="reshape", attrs={})),
        "bad_iota_axis": variant(ops=op(op="iota", inputs=[], attrs={"shape": ["M"], "dimension": 0})),
        "bad_layout_cast_to": variant(ops=op(op="layout_cast", attrs={})),
        "bad_parallel_axes": variant(parallel_axes=["Q"]),
        "bad_axis_role": variant(axis_roles={"M": "diagonal"}),
        "bad_schedule_mismatch": variant(parallel_axes=["M"], schedule={"tile_m": 16, "parallel_axes": ["N"]}),
        "bad_tensors_type": variant(tensors=[]),
        "bad_op_attrs_type": variant(ops=op(attrs=[1])),
    }


def write_validation(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from intent_ir.ir import IntentFunction, IntentIRValidationError

    out = {}
    for key, js in validation_cases().items():
        try:
            IntentFunction.from_json_dict(js)
            out[key] = {"json": js, "ok": True, "message": None}
        except IntentIRValidationError as e:
            out[key] = {"json": js, "ok": False, "message": str(e).splitlines()[0]}
    with open(os.path.join(HERE, "validation.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print(f"wrote {len(out)} validation cases ({sum(1 for v in out.values() if not v['ok'])} rejected)")


if __name__ == "__main__":
    write_validation(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("INTENTIR_REF", ""))
