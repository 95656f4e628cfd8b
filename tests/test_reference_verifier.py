"""The reference's own classes and verifier driving this backend.

Everything here imports the reference (``intent_ir``, ``verify``; for the CPU tier also its
``pipeline.tilelang.core`` kernel specs) from ``$INTENTIR_REF``, ``baseline/_ref`` (written by
``oracle/install_reference.py``) or the path BASELINE.json names, and is skipped where none of
them exists.

* CPU tier: real ``IntentFunction`` objects from the reference's deterministic builders are
  handed to ``lower_intent_to_b200_kernel`` / ``plan_json`` / ``make_run_ref_fn`` as objects —
  the drop-in promise of the boundary (``intentir_to_cuda.py:2047-2052`` takes the same object).
* GPU tier: ``verify.diff_runner.run_diff``, ``verify.metamorphic.run_metamorphic_suite`` /
  ``run_bounded_exhaustive``, ``verify.numerical_stability.run_numerical_stability_suite`` and
  ``verify.mutation.run_mutation_kill`` are called unchanged with ``make_run_ref_fn(intent)``
  as their ``run_ref_fn``, on the benchmark configurations' graphs.  Their verdicts must equal
  the verdicts the same suites give an *exact* runner (the reference interpreter itself): the
  CUDA backend must be indistinguishable from it at the suites' tolerances.
"""

import os

import numpy as np
import pytest

from intent_ir_b200.backend import make_run_ref_fn
from intent_ir_b200.config_graphs import config_graph
from intent_ir_b200.errors import B200LoweringError
from intent_ir_b200.lowering import lower_intent_to_b200_kernel, plan_json
from oracle.reference import import_reference, reference_root

pytestmark = pytest.mark.skipif(reference_root() is None, reason="no checkout of the reference on this machine")


@pytest.fixture(scope="module")
def ref():
    return import_reference()


def _specs(ref):
    try:
        import importlib

        return importlib.import_module("pipeline.tilelang.core").coverage_kernel_specs()
    except Exception as e:  # the trimmed install has no kernel specs (they import the TileLang kernels)
        pytest.skip(f"the reference's kernel specs are not importable here: {type(e).__name__}: {e}")


# graphs the backend refuses on purpose (a macro op outside the hot path)
REFUSED = {"upsample_bicubic2d_aa"}


def test_reference_intent_objects_lower_as_objects(ref):
    seen = 0
    for spec in _specs(ref):
        intent = spec.intent_builder()
        assert isinstance(intent, ref.IntentFunction)
        shapes = dict(spec.canonical_shapes)
        if spec.name in REFUSED:
            with pytest.raises(B200LoweringError):
                lower_intent_to_b200_kernel(intent, shape_bindings=shapes)
            continue
        lowered = lower_intent_to_b200_kernel(intent, shape_bindings=shapes)
        described = plan_json(intent, shapes)
        assert lowered.output_names == list(intent.outputs) and lowered.cuda_src == ""
        assert [s["kernel"] for s in described["steps"]] == [s["kernel"] for s in lowered.steps] and lowered.steps
        # every external input and output of the reference object is an argument of the plan
        produced = {op.output for op in intent.ops}
        external = {n for op in intent.ops for n in op.inputs if n in intent.tensors and n not in produced}
        assert external | set(intent.outputs) <= set(lowered.io_spec["arg_names"]), spec.name
        run = make_run_ref_fn(intent, input_gen=spec.runner)  # construction only: no device here
        assert callable(run)
        seen += 1
    assert seen >= 25


def test_reference_checker_returns_the_reference_functions(ref, monkeypatch):
    from intent_ir_b200.sweep import reference_checker

    monkeypatch.setenv("INTENTIR_REF", ref.root)
    run_diff, infer_tolerances, case_type = reference_checker()
    assert run_diff is ref.run_diff and infer_tolerances is ref.infer_tolerances and case_type is ref.TestCase
    monkeypatch.setenv("INTENTIR_REF", os.path.join(ref.root, "no_such_dir"))
    with pytest.raises(RuntimeError):
        reference_checker()


def test_reference_run_diff_accepts_an_exact_runner_built_from_our_graphs(ref):
    """The packaged configuration graphs load into the reference's own IntentFunction and pass its
    run_diff when the runner is exact — the harness below is sound before a GPU is involved."""
    intent = ref.IntentFunction.from_json_dict(config_graph("softmax_inner"))
    diffs, cex = ref.run_diff(intent, _exact_runner(ref, intent), [ref.TestCase(shapes={"M": 5, "N": 33}, dtypes={}, seed=1)])
    assert diffs[0].ok and not cex


# ---- helpers -----------------------------------------------------------------------------------

def _bindings(shapes):
    from intent_ir_b200.bindings import derive_bindings

    return derive_bindings(dict(shapes))


def _exact_runner(ref, intent):
    """run_ref_fn whose outputs come from the reference interpreter: what a perfect backend looks like."""
    from intent_ir_b200.backend import default_inputs
    from intent_ir_b200.ir import as_intent

    ours = as_intent(intent)
    ext = ours.external_inputs()

    def run(case):
        b = _bindings(case.shapes)
        ins = default_inputs(ours, b, getattr(case, "seed", 0))
        if getattr(case, "inputs", None):
            ins.update({k: np.asarray(v) for k, v in case.inputs.items() if k in ext})
        with np.errstate(all="ignore"):
            outs = ref.execute_intent(intent, ins, shape_bindings=b)
        return {**ins, **{k: np.asarray(v) for k, v in outs.items()}}

    return run


CONFIGS = {
    "any_kernel_dim": {"M": 16, "N": 256},
    "softmax_inner": {"M": 64, "N": 1000},
    "layer_norm_persistent": {"M": 48, "N": 512},
    "group_norm_kernel": {"N": 2, "C": 32, "HW": 256, "num_groups": 4},
    "matmul_bias_relu2d": {"M": 96, "N": 80, "K": 64},
}


# ---- GPU tier ----------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("key", sorted(CONFIGS))
def test_reference_run_diff_with_the_cuda_backend(ref, key):
    intent = ref.IntentFunction.from_json_dict(config_graph(key))
    cases = [ref.TestCase(shapes=dict(CONFIGS[key]), dtypes={}, seed=s) for s in (0, 1)]
    extra = [c for c in ref.generate_cases(intent, limit=6, seed=3)] if key != "group_norm_kernel" else []
    diffs, cex = ref.run_diff(intent, make_run_ref_fn(intent), cases + extra, tolerances=ref.infer_tolerances(intent).to_dict())
    assert len(diffs) == len(cases) + len(extra)
    assert all(d.ok for d in diffs), [d.summary for d in diffs if not d.ok]
    assert not cex


@pytest.mark.gpu
@pytest.mark.parametrize("key", ["any_kernel_dim", "softmax_inner", "layer_norm_persistent", "group_norm_kernel"])
def test_reference_metamorphic_and_bounded_suites(ref, key):
    intent = ref.IntentFunction.from_json_dict(config_graph(key))
    base = ref.TestCase(shapes=dict(CONFIGS[key]), dtypes={}, seed=4)
    mm = ref.metamorphic
    got = mm.run_metamorphic_suite(key, intent, make_run_ref_fn(intent), base_case=base)
    want = mm.run_metamorphic_suite(key, intent, _exact_runner(ref, intent), base_case=base)
    assert [(r.relation, r.ok) for r in got.results] == [(r.relation, r.ok) for r in want.results], [r.detail for r in got.results]
    assert got.ok and len(got.results) >= 1 and got.results[0].relation != "(none)"
    be = mm.run_bounded_exhaustive(key, intent, make_run_ref_fn(intent))
    assert be.ok and be.checked == be.total and be.total in (64, 81, 9), (be.detail, be.first_failure_summary)


@pytest.mark.gpu
@pytest.mark.parametrize("key", sorted(CONFIGS))
def test_reference_numerical_stability_suite(ref, key):
    """NaN / +-Inf / x1e4 probes.  The reference's comparison rejects any NaN in an output (NaN != NaN under
    ``np.array_equal``), so some probes fail for every runner, an exact one included: the verdicts are
    recorded as they come and must be the exact runner's."""
    intent = ref.IntentFunction.from_json_dict(config_graph(key))
    base = ref.TestCase(shapes=dict(CONFIGS[key]), dtypes={}, seed=4)
    suite = ref.numerical_stability.run_numerical_stability_suite
    got = suite(key, intent, make_run_ref_fn(intent), base_case=base)
    want = suite(key, intent, _exact_runner(ref, intent), base_case=base)
    assert not got.skipped and got.input == want.input
    assert [(r.name, r.ok) for r in got.results] == [(r.name, r.ok) for r in want.results], [(r.name, r.summary) for r in got.results]
    assert len(got.results) == 3


@pytest.mark.gpu
@pytest.mark.parametrize("key", ["softmax_inner", "layer_norm_persistent", "matmul_bias_relu2d"])
def test_reference_mutation_kill(ref, key):
    """The verifier's teeth, with this backend as the trusted side: mutated graphs are diffed against the
    CUDA results of the unmutated graph.  Mutant by mutant, the outcome must be the one an exact runner gives."""
    intent = ref.IntentFunction.from_json_dict(config_graph(key))
    shapes = dict(CONFIGS[key])
    cases = [ref.TestCase(shapes=shapes, dtypes={}, seed=s) for s in (0, 1)]
    kw = dict(intent=intent, diff_cases=cases, metamorphic_base_case=cases[0], n_mutants=12, seed=0)
    got = ref.mutation.run_mutation_kill(key, run_ref_fn=make_run_ref_fn(intent), **kw)
    want = ref.mutation.run_mutation_kill(key, run_ref_fn=_exact_runner(ref, intent), **kw)
    assert [(o.mutant_id, o.mutation_type, o.killed_by) for o in got.outcomes] == [(o.mutant_id, o.mutation_type, o.killed_by) for o in want.outcomes]
    assert got.total >= 6 and got.killed >= 1
