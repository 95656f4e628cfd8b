"""Host-side logic that needs no GPU: the C-ABI library loads and exports every declared
symbol, graph validation agrees with the reference, the planner lowers the reference's own
graphs to the expected kernels, bindings / expression handling, the registry idiom, and the
loud failure of the execution path when there is no CUDA device."""

import ctypes
import json
import os
import re

import numpy as np
import pytest

from intent_ir_b200 import _lib, registry
from intent_ir_b200.bindings import derive_bindings, eval_expression, normalise_bindings, resolve_expressions
from intent_ir_b200.errors import B200LoweringError, B200RuntimeError
from intent_ir_b200.ir import IntentFunction, IntentIRValidationError
from intent_ir_b200.lowering import lower_intent_to_b200_kernel, plan_json

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "intentir_b200.h")).read()
    declared = set(re.findall(r"IB200_API[^;(]*?\b(ib200_\w+)\s*\(", header))
    assert declared and declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert _lib.load().ib200_version() >= 100


def test_validation_agrees_with_reference():
    with open(os.path.join(ROOT, "tests", "golden", "validation.json")) as f:
        cases = json.load(f)
    for key, c in cases.items():
        try:
            IntentFunction.from_json_dict(c["json"])
            got = (True, None)
        except IntentIRValidationError as e:
            got = (False, str(e).splitlines()[0])
        assert got == (c["ok"], c["message"]), key


EXPECTED_KERNELS = {
    "any_kernel_dim": ["reduce_any"], "any_const_ne": ["reduce_any"],
    "softmax_inner": ["softmax"], "softmax_inner__cuda_pipeline_form": ["softmax"], "softmax_like_rowvec": ["softmax"],
    "layer_norm_persistent": ["layernorm"], "layer_norm_persistent__cuda_pipeline_form": ["layernorm"],
    "group_norm_kernel": ["groupnorm"], "matmul_bias_relu2d": ["gemm+bias+relu"], "matmul_relu2d": ["gemm+relu"],
    "row_sum": ["reduce_sum"], "row_max": ["reduce_max"], "transpose2d": ["transpose2d"], "gather2d": ["gather"],
    "_attn_fwd": ["gemm", "rowfused(2 steps, 4 phases)", "gemm"],  # scale + mask + softmax in one row program
    "masked_softmax2d": ["softmax+mask"], "rms_norm2d": ["rmsnorm"],
    "rms_norm_residual2d": ["residual+rmsnorm"],  # inp + residual + bias summed by the norm kernel as it loads each row
    "layer_norm_residual2d": ["residual+layernorm"],
    "mlp2d": ["gemm+bias+relu", "gemm+bias"], "matmul_transposed_epilogue": ["transpose2d", "gemm+bias+relu"],  # epilogues folded per GEMM
}


@pytest.mark.parametrize("key", sorted(EXPECTED_KERNELS))
def test_planner_picks_the_fused_kernel(key, golden_graphs):
    g = golden_graphs[key]
    d = plan_json(g["intent"], g["shapes"])
    assert [s["kernel"] for s in d["steps"]] == EXPECTED_KERNELS[key]
    assert d["cuda_src"] == "" and d["kernel_name"] == g["intent"]["name"]
    assert d["output_names"] == g["outputs"]
    # io_spec lists external inputs (first use) then outputs, with concrete shapes
    assert d["io_spec"]["arg_names"][-len(g["outputs"]):] == g["outputs"]
    assert sorted(d["io_spec"]["arg_names"][: -len(g["outputs"])]) == sorted(g["inputs"])


def test_planner_fuses_elementwise_chains_into_one_pass(golden_graphs):
    for key, n_in in (("add_bias2d", 2), ("where2d", 2), ("clamp2d", 3), ("scalar_attr_forms", 1), ("rowmask_where2d", 2)):
        g = golden_graphs[key]
        d = plan_json(g["intent"], g["shapes"])
        assert len(d["steps"]) == 1 and d["steps"][0]["kernel"].startswith("elementwise("), (key, d["steps"])
        assert f"{n_in} in, 1 out" in d["steps"][0]["kernel"]
        assert d["workspace_bytes"] == 0


def test_planner_general_path_and_workspace(golden_graphs):
    g = golden_graphs["matmul_fused_epilogue2d"]  # an epilogue the GEMM kernel cannot absorb
    d = plan_json(g["intent"], g["shapes"])
    kinds = [s["kernel"].split("(")[0] for s in d["steps"]]
    assert kinds == ["gemm", "elementwise"]
    assert d["workspace_bytes"] > 0 and d["status_offset"] >= 0


def test_planner_rejects_what_it_does_not_cover(golden_graphs):
    conv = {"name": "r", "tensors": {n: {"dtype": "f32", "shape": s} for n, s in {"x": ["S", "D"], "w": ["D", "D"], "y": ["S", "D"]}.items()},
            "ops": [{"op": "conv2d", "inputs": ["x", "w"], "output": "y"}], "outputs": ["y"]}
    with pytest.raises((B200LoweringError, IntentIRValidationError), match="conv2d"):
        plan_json(conv, {"S": 4, "D": 8})
    rope = {"name": "r", "tensors": {n: {"dtype": "f32", "shape": s} for n, s in
                                      {"x": ["S", "B", "H", "D"], "c": ["S", "D2"], "s": ["S", "D2"], "y": ["S", "B", "H", "D"]}.items()},
            "ops": [{"op": "rope", "inputs": ["x", "c", "s"], "output": "y"}], "outputs": ["y"]}
    assert [s["kernel"] for s in plan_json(rope, {"S": 4, "B": 1, "H": 2, "D": 8, "D2": 4})["steps"]] == ["rope"]
    with pytest.raises(B200LoweringError, match="cos/sin shape mismatch"):
        plan_json(rope, {"S": 4, "B": 1, "H": 2, "D": 8, "D2": 3})
    g = golden_graphs["softmax_inner"]
    with pytest.raises(B200LoweringError, match="unbound symbolic dim"):
        plan_json(g["intent"], {"M": 4})
    with pytest.raises(B200LoweringError, match="invalid IntentIR graph"):
        plan_json({"name": "x", "tensors": {}, "ops": []}, {})
    # extents that are no extents, a consumed output that nothing produces, attributes of the wrong kind
    add = golden_graphs["add2d"]["intent"]
    for bad, why in (([-1], "negative extent"), ([1.5, "N"], "invalid dimension type|bad dim"), ([2**31, 2**31], "larger than 2\\^40 elements")):
        damaged = json.loads(json.dumps(add))
        for t in damaged["tensors"].values():
            t["shape"] = bad
        with pytest.raises(B200LoweringError, match=why):
            plan_json(damaged, {"M": 4, "N": 8})
    with pytest.raises(B200LoweringError, match="not an extent"):
        plan_json(add, {"M": -4, "N": 8})
    form = json.loads(json.dumps(golden_graphs["softmax_inner__cuda_pipeline_form"]["intent"]))
    op = next(o for o in form["ops"] if o["output"] == "row_sum_ptr")
    op["output"] = "elsewhere"
    form["tensors"]["elsewhere"] = dict(form["tensors"]["row_sum_ptr"])
    with pytest.raises(B200LoweringError, match="consumed but no op produces it"):
        plan_json(form, {"M": 4, "N": 8})
    rows = json.loads(json.dumps(golden_graphs["row_sum"]["intent"]))
    rows["ops"][0]["attrs"]["keepdims"] = "yes"
    with pytest.raises(B200LoweringError, match="keepdims must be a boolean"):
        plan_json(rows, {"M": 4, "N": 8})
    tr = json.loads(json.dumps(golden_graphs["transpose2d"]["intent"]))
    tr["ops"][0]["attrs"]["perm"] = [1, 1]
    with pytest.raises(B200LoweringError, match="repeated axis"):
        plan_json(tr, {"M": 4, "N": 8})


def test_lowered_record_mirrors_the_reference_fields(golden_graphs):
    g = golden_graphs["softmax_inner"]
    low = lower_intent_to_b200_kernel(IntentFunction.from_json_dict(g["intent"]),
                                      shape_bindings={"M": 8, "N": 100, "SOFTMAX_THREADS": 128, "ALLOW_TF32": True, "junk": "x"})
    assert low.kernel_name == "softmax_inner" and low.cuda_src == ""
    assert set(low.io_spec) >= {"arg_names", "tensors", "scalars"}
    assert low.io_spec["tensors"]["input_ptr"] == {"dtype": "f32", "shape": [8, 100]}
    assert low.output_names == ["output_ptr"]
    assert low.bindings["M"] == 8 and low.bindings["ALLOW_TF32"] == 1 and "junk" not in low.bindings
    assert len(low.launch.grid) == 3 and len(low.launch.block) == 3
    again = lower_intent_to_b200_kernel(IntentFunction.from_json_dict(g["intent"]), shape_bindings={"M": 8, "N": 100,
                                        "SOFTMAX_THREADS": 128, "ALLOW_TF32": True})
    assert again is low  # plans are cached per (graph, bindings)


def test_reference_style_intent_object_is_accepted(golden_graphs):
    class Foreign:  # stands in for the reference's IntentFunction: anything with to_json_dict()
        def __init__(self, js):
            self._js = js

        def to_json_dict(self):
            return self._js

    g = golden_graphs["row_sum"]
    low = lower_intent_to_b200_kernel(Foreign(g["intent"]), shape_bindings=g["shapes"])
    assert [s["kernel"] for s in low.steps] == ["reduce_sum"]


def test_bindings_rules():
    assert normalise_bindings({"M": 4, "f": 2.0, "g": 2.5, "t": True, "s": "7", "bad": "x", "n": None}) == \
        {"M": 4, "f": 2, "g": 2.5, "t": 1, "s": 7}
    d = derive_bindings({"N": 16, "C": 64, "HW": 16, "num_groups": 4})
    assert d["group_size"] == 16 and d["num_elements"] == 256 and d["G"] == 1
    d = derive_bindings({"batch": 3, "HEAD_DIM": 64, "group": 2})
    assert d["Z"] == 3 and d["HEAD_DIM_DIV2"] == 32 and d["num_groups"] == 2
    assert eval_expression("1.0/(HEAD_DIM**0.5)", {"HEAD_DIM": 64}) == 0.125
    with pytest.raises(ValueError):
        eval_expression("__import__('os').system('true')", {})
    js = {"tensors": {"x": {}}, "ops": [{"op": "const", "inputs": [], "output": "c", "attrs": {"value": "1.0/N"}},
                                         {"op": "reduce_sum", "inputs": ["x"], "output": "s", "attrs": {"dims": [1], "scale": "1.0/N"}},
                                         {"op": "const", "inputs": [], "output": "e", "attrs": {"value": "eps"}}]}
    out = resolve_expressions(js, {"N": 4})
    assert out["ops"][0]["attrs"]["value"] == 0.25 and out["ops"][1]["attrs"]["scale"] == 0.25
    assert out["ops"][2]["attrs"]["value"] == "eps" and js["ops"][0]["attrs"]["value"] == "1.0/N"


def test_registry_idiom():
    backend = registry.get("b200")
    assert backend.name == "b200" and registry.get("b200") is backend
    with pytest.raises(KeyError, match="backend not registered: triton"):
        registry.get("triton")

    class Other:
        name = "other"

    registry.register(Other)
    assert registry.get("other") is Other


def test_no_cpu_fallback(golden_graphs):
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    g = golden_graphs["add2d"]
    low = lower_intent_to_b200_kernel(g["intent"], shape_bindings=g["shapes"])  # planning is host-only
    from intent_ir_b200.runtime import run_b200_kernel

    with pytest.raises(B200RuntimeError, match="no CPU path"):
        run_b200_kernel(io_spec=low.io_spec, inputs_np={"A": np.zeros((16, 16), np.float32), "B": np.zeros((16, 16), np.float32)})


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "intent_ir_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", text, re.M), f


# ---- pipeline report artefacts (scripts/backend_codegen_smoke.py:81-146) --------------------------

def _write_artifact(tmp_path, key, golden_graphs, golden_vectors, rename=None, expanded=True):
    g = golden_graphs[key]
    report = {"baseline": {"shapes": g["shapes"], "seed": 0}, "intent": g["intent"], "intent_expanded": g["intent"] if expanded else None}
    (tmp_path / f"{key}.json").write_text(json.dumps(report))
    arrays = {n: golden_vectors[f"{key}/in/{n}"] for n in g["inputs"]}
    arrays.update({n: golden_vectors[f"{key}/out/{n}"] for n in g["outputs"]})
    for old, new in (rename or {}).items():
        arrays[new] = arrays.pop(old)
    np.savez(tmp_path / f"{key}.baseline.npz", **arrays)
    return str(tmp_path / f"{key}.json")


def test_artifact_loader_reads_report_and_baseline(tmp_path, golden_graphs, golden_vectors):
    from intent_ir_b200.artifacts import SMOKE_TOLERANCES, load_artifact

    path = _write_artifact(tmp_path, "softmax_inner", golden_graphs, golden_vectors, rename={"input_ptr": "input", "output_ptr": "out"})
    art = load_artifact(path)
    assert art.kernel == "softmax_inner" and art.inputs == ["input_ptr"] and art.outputs == ["output_ptr"]
    assert art.tolerances == SMOKE_TOLERANCES["softmax_inner"]
    # recorded under other spellings, reachable under the graph's names
    assert np.array_equal(art.baseline["input_ptr"], golden_vectors["softmax_inner/in/input_ptr"])
    assert np.array_equal(art.baseline["output_ptr"], golden_vectors["softmax_inner/out/output_ptr"])
    assert art.bindings == golden_graphs["softmax_inner"]["shapes"]

    path = _write_artifact(tmp_path, "group_norm_kernel", golden_graphs, golden_vectors, expanded=False)
    art = load_artifact(path)
    assert art.bindings["group_size"] * art.bindings["num_groups"] == art.bindings["C"]
    assert art.bindings["num_elements"] == art.bindings["group_size"] * art.bindings["HW"]


def test_artifact_loader_errors(tmp_path):
    from intent_ir_b200.artifacts import load_artifact
    from intent_ir_b200.errors import B200RuntimeError

    (tmp_path / "k.json").write_text(json.dumps({"baseline": {"shapes": {}}}))
    with pytest.raises(B200RuntimeError, match="neither intent_expanded nor intent"):
        load_artifact(str(tmp_path / "k.json"))
    (tmp_path / "k2.json").write_text(json.dumps({"intent": {"name": "k2", "tensors": {"x": {"dtype": "f32", "shape": [2], "layout": "row_major"},
                                                                                 "y": {"dtype": "f32", "shape": [2], "layout": "row_major"}},
                                                             "ops": [{"op": "relu", "inputs": ["x"], "output": "y"}], "outputs": ["y"]}}))
    with pytest.raises(B200RuntimeError, match="missing baseline npz"):
        load_artifact(str(tmp_path / "k2.json"))


def test_plan_ids_stay_unique_when_the_plan_cache_evicts(golden_graphs):
    """Workspaces are cached per plan id: an id handed out twice would give a plan another plan's scratch."""
    g = golden_graphs["add2d"]["intent"]
    ids = set()
    for m in range(1, 560):  # more plans than the cache holds
        ids.add(lower_intent_to_b200_kernel(g, shape_bindings={"M": m, "N": 8}).io_spec["plan_id"])
    assert len(ids) == 559


def test_reduce_scratch_sizes_and_plan_labels_agree():
    """ib200_reduce_scratch_bytes is a host computation: shapes that fill the GPU by themselves need no
    scratch, few long rows take the fixed row area, narrow leading-axis reductions an area that grows
    with the number of segments; the plan builder marks exactly the shapes that get scratch."""
    from intent_ir_b200 import _lib
    from intent_ir_b200.lowering import plan_json

    lib = _lib.load()
    need = lambda o, r, i: int(lib.ib200_reduce_scratch_bytes(o, r, i))  # noqa: E731
    assert need(4096, 4096, 1) == 0 and need(16, 256, 1) == 0 and need(4, 65535, 1) == 0 and need(296, 65536, 1) == 0
    assert need(1, 1 << 26, 1) == need(295, 65536, 1) == 8192
    assert need(1, 40000, 6) == 0  # inner extent not a multiple of 4: the scalar tiles, unsplit
    assert need(1, 1 << 20, 64) > need(1, 1 << 10, 64) > 0
    assert need(1, 8, 64) == 0 and need(0, 5, 4) == 0 and need(1 << 20, 64, 128) == 0

    def graph(dims):
        t = lambda sh, dt="f32": {"dtype": dt, "shape": sh, "layout": "row_major"}  # noqa: E731
        out = [s for k, s in enumerate(["M", "N"]) if k not in dims]
        return {"name": "r", "tensors": {"x": t(["M", "N"]), "y": t(out)},
                "ops": [{"op": "reduce_sum", "inputs": ["x"], "output": "y", "attrs": {"dims": dims}}], "outputs": ["y"]}

    for (m, n, dims, o, r, i) in [(1, 1 << 20, [1], 1, 1 << 20, 1), (4096, 4096, [1], 4096, 4096, 1), (1 << 16, 64, [0], 1, 1 << 16, 64),
                                  (300, 1000, [0, 1], 1, 300000, 1), (40000, 6, [0], 1, 40000, 6)]:
        d = plan_json(graph(dims), {"M": m, "N": n})
        label = d["steps"][0]["kernel"]
        if need(o, r, i):
            assert label == ("reduce_sum(split rows)" if i == 1 else "reduce_sum(split columns)"), (m, n, label)
            assert d["workspace_bytes"] >= need(o, r, i)
        else:
            assert label == "reduce_sum" and d["workspace_bytes"] == 0, (m, n, label)


def test_packaged_config_graphs_are_the_recorded_reference_graphs(golden_graphs):
    """bench.py and smoke() read their graphs from the package; they must be the graphs recorded from
    the reference's builders, not a drifting copy."""
    from intent_ir_b200.config_graphs import config_graph, config_graphs

    packaged = config_graphs()
    assert set(packaged) >= {"any_kernel_dim", "softmax_inner", "layer_norm_persistent", "group_norm_kernel", "matmul_bias_relu2d"}
    for key, js in packaged.items():
        assert js == golden_graphs[key]["intent"], key
    config_graph("softmax_inner")["name"] = "edited"  # callers get copies
    assert config_graph("softmax_inner")["name"] != "edited"
    with pytest.raises(KeyError):
        config_graph("no_such_graph")


def test_registry_keeps_the_reason_a_builtin_backend_failed_to_import(monkeypatch):
    monkeypatch.setitem(registry._LAZY, "broken", "intent_ir_b200.no_such_module")
    with pytest.raises(KeyError) as e:
        registry.get("broken")
    assert "no_such_module" in str(e.value) and isinstance(e.value.__cause__, ImportError)


def test_gemm_plans_cover_every_float_operand_type(golden_graphs):
    """bf16 and f16 products always lower to the tensor-core GEMM, f32 products only under the reference's
    ALLOW_TF32 binding (intentir_to_cuda.py:577-578); a last, mostly empty round of tiles gets scratch for the
    K split."""
    from intent_ir_b200.lowering import plan_json

    def graph(dt):
        js = json.loads(json.dumps(golden_graphs["matmul_bias_relu2d"]["intent"]))
        for name in ("A", "B", "bias", "C"):
            js["tensors"][name]["dtype"] = dt
        return js

    for dt in ("bf16", "f16"):
        d = plan_json(graph(dt), {"M": 256, "N": 256, "K": 128})
        assert [s["kernel"] for s in d["steps"]] == ["gemm+bias+relu"] and d["io_spec"]["tensors"]["C"]["dtype"] == dt
    assert [s["kernel"] for s in plan_json(graph("f32"), {"M": 256, "N": 256, "K": 128})["steps"]] == ["gemm+bias+relu"]
    assert [s["kernel"] for s in plan_json(graph("f32"), {"M": 256, "N": 256, "K": 128, "ALLOW_TF32": 1})["steps"]] == ["gemm+bias+relu(tf32)"]
    assert [s["kernel"] for s in plan_json(graph("f32"), {"M": 256, "N": 250, "K": 128, "ALLOW_TF32": 1})["steps"]] == ["gemm+bias+relu"]  # ragged N: FMA
    big = plan_json(graph("bf16"), {"M": 4096, "N": 4096, "K": 4096})  # large products: 256 x 256 tiles on pairs of CTAs, no scratch
    assert [s["kernel"] for s in big["steps"]] == ["gemm+bias+relu(cta pairs)"]
    lib = _lib.load()
    assert lib.ib200_gemm_scratch_bytes(_lib.BF16, _lib.BF16, 4096, 4096, 4096, 0, 0) == 0
    # one row of tiles (M = 128 leaves a pair's second CTA without rows): 40 tiles on 148 SMs, three K slices each
    flat = plan_json(graph("bf16"), {"M": 128, "N": 10240, "K": 4096})
    assert [s["kernel"] for s in flat["steps"]] == ["gemm+bias+relu(split tail)"]
    need = lib.ib200_gemm_scratch_bytes(_lib.BF16, _lib.BF16, 128, 10240, 4096, 0, 0)
    assert need == 256 + 40 * 16 + 256 + 40 * 3 * 128 * 256 * 4 and flat["workspace_bytes"] >= need
    # the one-CTA kernel forced onto 4096^3: 512 tiles, 68 tail tiles, two slices each
    assert lib.ib200_gemm_scratch_bytes(_lib.BF16, _lib.BF16, 4096, 4096, 4096, 0, _lib.GEMM_ONE_CTA) == 256 + 68 * 16 + 256 + 68 * 2 * 128 * 256 * 4
    assert lib.ib200_gemm_scratch_bytes(_lib.F32, _lib.F32, 4096, 4096, 4096, 0, 0) == 0  # exact FMA path: no tiles to split
    # TF32 takes B as [N,K]: a [K,N] operand needs room for its transpose on top of the split area
    tf = _lib.GEMM_ALLOW_TF32
    assert lib.ib200_gemm_scratch_bytes(_lib.F32, _lib.F32, 4096, 4096, 4096, 0, tf) == lib.ib200_gemm_scratch_bytes(_lib.F32, _lib.F32, 4096, 4096, 4096, 1, tf) + 4096 * 4096 * 4 == 4096 * 4096 * 4
    assert lib.ib200_gemm_scratch_bytes(_lib.BF16, _lib.BF16, 128 * 37, 256 * 4, 4096, 0, 0) == 0  # 148 tiles: a full round


def test_f64_and_wide_integer_chains_take_the_double_valued_kernel():
    """The elementwise kernels carry values in f32 lanes, which hold neither f64 nor integers above 2^24:
    programs that touch f64 / i32 / i64 tensors are marked for the double-valued kernel (and stay out of the
    f32 row programs)."""
    from intent_ir_b200.lowering import plan_json

    def t(shape, dt):
        return {"dtype": dt, "shape": shape, "layout": "row_major"}

    def kernels(dt_in, dt_out, op="add"):
        js = {"name": "g", "tensors": {"a": t(["M", "N"], dt_in), "b": t(["N"], dt_in), "y": t(["M", "N"], dt_out)},
              "ops": [{"op": op, "inputs": ["a", "b"], "output": "y"}], "outputs": ["y"]}
        return [s["kernel"] for s in plan_json(js, {"M": 8, "N": 16})["steps"]]

    assert kernels("f64", "f64") == ["elementwise(1 ops, 2 in, 1 out)(f64 lanes)"]
    assert kernels("i32", "i32", "mul") == ["elementwise(1 ops, 2 in, 1 out)(f64 lanes)"]
    assert kernels("i64", "bool", "lt") == ["elementwise(1 ops, 2 in, 1 out)(f64 lanes)"]
    assert kernels("f32", "f32") == ["elementwise(1 ops, 2 in, 1 out)"]
    assert kernels("i8", "i8") == ["elementwise(1 ops, 2 in, 1 out)"]  # 8- and 16-bit integers are exact in f32 lanes


def test_recurring_elementwise_chains_are_compiled_in(golden_graphs):
    """Linear chains run from registers; the ones that recur (the benchmark chains, bias / activation epilogues,
    clamps, selects) are also compiled in as straight-line kernels, found by the signature of their register code.
    Anything else keeps the run-time instruction loop."""
    from intent_ir_b200.lowering import plan_json

    def programs(js, bind):
        return [s["program"] for s in plan_json(js, bind)["steps"] if "program" in s]

    import bench

    for name in ("chain", "dag"):
        js, bind = bench.workload(name)[:2]
        (prog,) = programs(js, bind)
        assert prog["compiled_in"] == 1 and prog["register_code"].startswith("n3 b4 r2"), (name, prog["register_code"])
    for key in ("add_bias2d", "add2d", "relu2d", "exp2d", "where2d", "clamp2d", "rowmask_where2d", "floor2d", "copy2d_divmod"):
        g = golden_graphs[key]
        shapes = {k: 8 * v for k, v in g["shapes"].items()}
        progs = programs(g["intent"], shapes)
        assert progs and all(p["compiled_in"] == 1 for p in progs), (key, [p["register_code"] for p in progs])
    # an arbitrary chain is still a register-path program, run by the instruction loop
    t = lambda s: {"dtype": "f32", "shape": s, "layout": "row_major"}  # noqa: E731
    js = {"name": "odd", "tensors": {"x": t(["M", "N"]), "c": t(["N"]), "y": t(["M", "N"])},
          "ops": [{"op": "sub", "inputs": ["x", "c"], "output": "a"}, {"op": "abs", "inputs": ["a"], "output": "b"},
                  {"op": "min", "inputs": ["b", "c"], "output": "y"}], "outputs": ["y"]}
    (prog,) = programs(js, {"M": 64, "N": 128})
    assert prog["compiled_in"] == 0 and prog["register_code"]


def test_recurring_row_programs_are_compiled_in(golden_graphs):
    """The softmax between an attention's products (additive-mask and causal forms) and an rms-norm with |x| inside
    fuse into row programs whose phases the row kernel also holds as compiled-in tables; the plan description
    says so.  A row length that is no multiple of 4 runs decoded."""
    for key in ("_attn_fwd", "flash_attention2d", "masked_attention2d"):
        g = golden_graphs[key]
        fused = [s for s in plan_json(g["intent"], g["shapes"])["steps"] if "row_program" in s]
        assert len(fused) == 1 and fused[0]["row_program"]["compiled_in"] is True, key
        odd = [s for s in plan_json(g["intent"], dict(g["shapes"], KV_CTX=18))["steps"] if "row_program" in s]
        assert odd and odd[0]["row_program"]["compiled_in"] is False, key
    t = lambda shape: {"dtype": "f32", "shape": shape, "layout": "row_major"}  # noqa: E731
    rms = {"name": "rms_abs", "tensors": {"x": t(["M", "N"]), "w": t(["N"]), "y": t(["M", "N"]), "rstd": t(["M"])},
           "ops": [{"op": "mul", "inputs": ["x", "x"], "output": "sq"},
                   {"op": "reduce_sum", "inputs": ["sq"], "output": "ss", "attrs": {"dims": [1], "keepdims": True, "scale": "1.0/N"}},
                   {"op": "add", "inputs": ["ss"], "output": "ve", "attrs": {"addend": 1e-5}},
                   {"op": "rsqrt", "inputs": ["ve"], "output": "r1"},
                   {"op": "reshape", "inputs": ["r1"], "output": "rstd", "attrs": {"shape": ["M"]}},
                   {"op": "mul", "inputs": ["x", "r1"], "output": "xn"},
                   {"op": "abs", "inputs": ["xn"], "output": "xr"},
                   {"op": "mul", "inputs": ["xr", "w"], "output": "y"}], "outputs": ["y", "rstd"]}
    steps = plan_json(rms, {"M": 64, "N": 4096})["steps"]
    assert len(steps) == 1 and steps[0]["row_program"]["compiled_in"] is True


def test_planner_answers_damaged_graphs_with_a_status_code(golden_graphs):
    """The stateless C entry takes text from outside the process: whatever is wrong with it — missing or
    retyped fields, absurd extents, truncated text — the answer is a status code (planned, unsupported or
    invalid), never a fault.  Seeded structural damage to every recorded reference graph."""
    import copy
    import random

    lib = _lib.load()
    junk = [None, True, -1, 0, 2**31, 2**40, 2**62, -2**40, 1.5, "", "zz", "i64", "softmax", [], {}, [[]], ["a"], [1, 2, 3], {"a": 1}, 1e308, "M"]
    symbols = "M N K C HW num_groups Z Q_CTX KV_CTX HEAD_DIM q_numhead kv_numhead B H W D S".split()

    def paths(o, p=()):
        if p:
            yield p
        for k in (o if isinstance(o, dict) else range(len(o)) if isinstance(o, list) else ()):
            yield from paths(o[k], p + (k,))

    def damage(o, rng):
        o = copy.deepcopy(o)
        for _ in range(rng.choice([1, 1, 2, 3])):
            p = rng.choice(list(paths(o)))
            parent = o
            for k in p[:-1]:
                parent = parent[k]
            if rng.random() < 0.3:
                del parent[p[-1]]
            else:
                parent[p[-1]] = copy.deepcopy(rng.choice(junk))
        return o

    buf = ctypes.create_string_buffer(1 << 20)
    seen = set()
    keys = sorted(golden_graphs)
    for i in range(600):
        rng = random.Random(i)
        text = json.dumps(damage(golden_graphs[keys[i % len(keys)]]["intent"], rng))
        if i % 20 == 0:
            text = text[: rng.randrange(len(text))]
        bind = {s: rng.choice([1, 2, 3, 7, 64, 100, 4096] + ([0, -1, 2**33] if i % 5 == 0 else [])) for s in symbols}
        seen.add(lib.ib200_plan_json(text.encode(), json.dumps(bind).encode(), buf, len(buf)))
    assert seen <= {_lib.OK, _lib.ERR_UNSUPPORTED, _lib.ERR_INVALID}, seen
    assert _lib.ERR_INVALID in seen and _lib.OK in seen
    # the Python entry in front of it: a plan or B200LoweringError, whatever the parser tripped over
    for i in range(300):
        rng = random.Random(10_000 + i)
        graph = damage(golden_graphs[keys[i % len(keys)]]["intent"], rng)
        bind = {s: rng.choice([1, 2, 3, 64, 4096] + ([0, -1, "x", None, 1.5] if i % 5 == 0 else [])) for s in symbols}
        try:
            plan_json(graph, bind)
        except B200LoweringError:
            pass


def test_direct_entries_refuse_arguments_that_cannot_be_meant():
    """Negative extents, extents whose product no device holds (or that wrap), unknown type / kind / activation
    codes, null operands and a negative mask stride are answered before anything is launched: the codes are
    INVALID or UNSUPPORTED, never the CUDA error a launch attempt gives on a machine without a device.  Empty
    tensors are fine and launch nothing."""
    lib = _lib.load()
    p = ctypes.c_void_p(0x7F0000000000)  # stands for a device address; nothing on the host dereferences it
    refused = {_lib.ERR_INVALID, _lib.ERR_UNSUPPORTED}

    def calls(r, c):
        return [lib.ib200_softmax(p, p, None, None, _lib.F32, r, c, None),
                lib.ib200_softmax_io(p, p, None, None, _lib.BF16, _lib.F32, r, c, None),
                lib.ib200_softmax_masked(p, p, 0, -1e9, p, None, None, r, c, None),
                lib.ib200_layernorm(p, p, p, p, None, None, _lib.F32, r, c, 1e-5, None),
                lib.ib200_norm_rows(p, p, p, p, None, None, _lib.F32, _lib.F32, r, c, 1, max(c, 1), 1e-5, None),
                lib.ib200_reduce(p, p, _lib.F32, _lib.F32, _lib.REDUCE_SUM, r, c, 1, 1.0, None),
                lib.ib200_reduce(p, p, _lib.F32, _lib.F32, _lib.REDUCE_MAX, 1, r, c, 1.0, None),
                lib.ib200_reduce_any_f32(p, p, r, c, None),
                lib.ib200_gemm_bias_act(p, p, None, p, _lib.BF16, _lib.BF16, r, c, 8, 0, _lib.ACT_RELU, None, None),
                lib.ib200_gemm_bias_act(p, p, None, p, _lib.F32, _lib.F32, 8, r, c, 0, _lib.ACT_NONE, None, None),
                lib.ib200_transpose2d(p, p, 4, r, c, None),
                lib.ib200_groupnorm(p, p, p, p, None, None, _lib.F32, r, c, 16, 1, 1e-5, None)]

    for r, c in ((-1, 16), (4, -5), (1 << 40, 1 << 40), (1 << 62, 4), (4, 1 << 62), (1 << 21, 1 << 20)):
        assert set(calls(r, c)) <= refused, (r, c, calls(r, c))
    for r, c in ((0, 16), (0, 0)):  # (the maximum over an empty axis has no identity: that one call is refused)
        got = calls(r, c)
        assert got[6] == (_lib.ERR_INVALID if c else _lib.OK) and set(got[:6] + got[7:]) == {_lib.OK}, (r, c, got)
    for code in (-1, 99):
        assert lib.ib200_softmax(p, p, None, None, code, 4, 16, None) in refused
        assert lib.ib200_layernorm(p, p, p, p, None, None, code, 4, 16, 1e-5, None) in refused
        assert lib.ib200_reduce(p, p, code, _lib.F32, _lib.REDUCE_SUM, 4, 16, 1, 1.0, None) in refused
        assert lib.ib200_reduce(p, p, _lib.F32, _lib.F32, code, 4, 16, 1, 1.0, None) in refused
        assert lib.ib200_gemm_bias_act(p, p, None, p, code, _lib.F32, 8, 8, 8, 0, _lib.ACT_NONE, None, None) in refused
        assert lib.ib200_gemm_bias_act(p, p, None, p, _lib.F32, _lib.F32, 8, 8, 8, 0, code, None, None) in refused
        assert lib.ib200_transpose2d(p, p, code, 4, 4, None) in refused
    assert lib.ib200_softmax(None, p, None, None, _lib.F32, 4, 16, None) == _lib.ERR_INVALID
    assert lib.ib200_layernorm(p, p, p, None, None, None, _lib.F32, 4, 16, 1e-5, None) == _lib.ERR_INVALID
    assert lib.ib200_reduce(p, None, _lib.F32, _lib.F32, _lib.REDUCE_SUM, 4, 16, 1, 1.0, None) == _lib.ERR_INVALID
    assert lib.ib200_gemm_bias_act(None, p, None, p, _lib.F32, _lib.F32, 8, 8, 8, 0, _lib.ACT_NONE, None, None) == _lib.ERR_INVALID
    assert lib.ib200_groupnorm(p, p, p, p, None, None, _lib.F32, 2, 8, 16, 3, 1e-5, None) == _lib.ERR_INVALID
    assert lib.ib200_groupnorm(p, p, p, p, None, None, _lib.F32, 2, 8, 16, 0, 1e-5, None) == _lib.ERR_INVALID
    assert lib.ib200_norm_rows(p, p, p, p, None, None, _lib.F32, _lib.F32, 4, 16, 1, 0, 1e-5, None) == _lib.ERR_INVALID
    assert lib.ib200_softmax_masked(p, p, -3, -1e9, p, None, None, 4, 16, None) == _lib.ERR_INVALID
    assert lib.ib200_plan_launch(None, None, 0, None, 0, None) == _lib.ERR_INVALID
    assert lib.ib200_plan_json(None, None, None, 0) == _lib.ERR_INVALID
