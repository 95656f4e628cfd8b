"""Oracle differential runner — TEST INFRASTRUCTURE.  Restates ``verify/diff_runner.py``.

``run_diff(intent, run_ref_fn, cases, constraints, tolerances, stop_on_first_fail)``
(diff_runner.py:37-275): for every case call the runner (it returns inputs AND outputs),
alias its keys onto the graph's tensor names (:278-354), derive the extra symbols the
interpreter needs (``Z``/``batch``, ``num_groups``, ``group_size``, ``num_elements``, ``G``,
``HEAD_DIM_*``; :101-140), feed only the true external inputs (:142-189), insist that their
shapes equal the declared ones (:194-241), execute the graph on the CPU and compare
(:357-418): booleans exactly, non-finite values by identical pattern and value, everything
else per element in float64 against ``atol + rtol·|ref|``; shapes may differ only by unit
dimensions (:421-490).

Macro expansion (:48) is the identity for every graph on this path: the only macro op,
``upsample_bicubic2d_aa``, is out of scope and is rejected with the same
"macro expansion error" result shape.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple

import numpy as np

from .cases import TestCase
from .interpreter import execute_intent
from .tolerances import infer_tolerances

__all__ = ["DiffResult", "Counterexample", "run_diff", "compare_outputs", "derive_bindings", "with_io_aliases"]


@dataclass
class DiffResult:
    ok: bool
    max_abs_err: float
    max_rel_err: float
    first_bad_index: Optional[Tuple[int, ...]]
    summary: str


@dataclass
class Counterexample:
    case: TestCase
    diff: DiffResult
    intent_json: Dict[str, Any]
    facts_summary: Optional[Dict[str, Any]]
    hints: List[str]


def _fail(summary: str) -> DiffResult:
    return DiffResult(False, 0.0, 0.0, None, summary)


# ---- names ----------------------------------------------------------------------

_SHORT = {"i": "input", "o": "output", "x": "input", "y": "output", "w": "weight", "b": "bias",
          "in": "input", "out": "output"}


def _canon(name: str) -> str:
    s = str(name).strip().strip("_").lower()
    if s.startswith("ptr_"):
        s = s[4:]
    if s.endswith("_ptr"):
        s = s[:-4]
    if s.endswith("ptr") and len(s) > 3:
        s = s[:-3]
    return _SHORT.get(s, s).replace("_", "")


def with_io_aliases(intent, io: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
    out = dict(io)
    by_canon: Dict[str, List[str]] = {}
    for key in io:
        by_canon.setdefault(_canon(key), []).append(key)
    for name in set(intent.tensors) | set(intent.outputs):
        if name in out:
            continue
        canon = _canon(name)
        keys = by_canon.get(canon) or []
        if len(keys) == 1:
            out[name] = io[keys[0]]
        elif keys:
            pick = next((k for k in keys if str(k).lower() == str(name).lower()), None)
            if pick is None and canon in io:
                pick = canon
            out[name] = io[pick if pick is not None else keys[0]]
        elif len(canon) >= 3:
            cands = [k for k in io if canon in _canon(k)]
            if len(cands) == 1:
                out[name] = io[cands[0]]
    return out


# ---- bindings -----------------------------------------------------------------------

def derive_bindings(shapes: Dict[str, int]) -> Dict[str, int]:
    b = dict(shapes)
    if "batch" in b and "Z" not in b:
        b["Z"] = b["batch"]
    if "Z" in b and "batch" not in b:
        b["batch"] = b["Z"]
    if "group" in b and "num_groups" not in b:
        b["num_groups"] = b["group"]
    if "num_groups" in b and "C" in b and "group_size" not in b:
        g, c = int(b["num_groups"]), int(b["C"])
        if g <= 0:
            raise ValueError(f"invalid num_groups: {g}")
        b["group_size"] = c // g if c % g == 0 else (c + g - 1) // g
    if "group_size" in b and "HW" in b and "num_elements" not in b:
        b["num_elements"] = int(b["group_size"]) * int(b["HW"])
    if "N" in b and "group_size" in b and "G" not in b:
        n, gs = int(b["N"]), int(b["group_size"])
        if gs > 0 and n % gs == 0:
            b["G"] = n // gs
    if "HEAD_DIM" in b and int(b["HEAD_DIM"]) > 0:
        half = int(b["HEAD_DIM"]) // 2
        for alias in ("HEAD_DIM_DIV2", "HEAD_DIM_DIV_2", "HEAD_DIM_HALF", "HEAD_DIM_MID"):
            b.setdefault(alias, half)
    return b


def _declared_shape(tensor, bindings) -> Optional[Tuple[int, ...]]:
    dims = []
    for d in tensor.shape:
        if d.kind == "const":
            dims.append(int(d.value))
        elif bindings.get(d.value) is not None:
            dims.append(bindings[d.value])
        else:
            return None
    return tuple(dims)


_SCALAR_NP = {"f16": np.float16, "f64": np.float64, "i32": np.int32, "i64": np.int64, "i8": np.int8,
              "u8": np.uint8, "bool": np.bool_}


# ---- comparison -------------------------------------------------------------------------

def _drop_units(arr: np.ndarray, target: Tuple[int, ...]) -> Optional[np.ndarray]:
    have = tuple(arr.shape)
    if len(have) < len(target):
        return None
    drop, j = [], 0
    for i, d in enumerate(have):
        if j < len(target) and d == target[j]:
            j += 1
        elif d == 1:
            drop.append(i)
        else:
            return None
    if j != len(target) or not drop:
        return None
    out = np.squeeze(arr, axis=tuple(drop))
    return out if tuple(out.shape) == tuple(target) else None


def _add_units(arr: np.ndarray, target: Tuple[int, ...]) -> Optional[np.ndarray]:
    have = tuple(arr.shape)
    if len(have) > len(target):
        return None
    i = 0
    for d in target:
        if i < len(have) and have[i] == d:
            i += 1
        elif d != 1:
            return None
    if i != len(have):
        return None
    return arr.reshape(target)


def compare_outputs(pred: Dict[str, np.ndarray], ref: Dict[str, np.ndarray], outputs: List[str], tol) -> DiffResult:
    worst_abs = worst_rel = 0.0
    bad = None
    atol, rtol = float(tol.get("atol", 1e-3)), float(tol.get("rtol", 1e-3))
    for name in outputs:
        if name not in ref:
            return DiffResult(False, worst_abs, worst_rel, bad, f"reference missing output {name}")
        if name not in pred:
            return DiffResult(False, worst_abs, worst_rel, bad, f"missing output {name}")
        r, p = ref[name], pred[name]
        if p.shape != r.shape:
            q = _drop_units(p, r.shape)
            if q is None:
                q = _add_units(p, r.shape)
            if q is None:
                return DiffResult(False, worst_abs, worst_rel, bad, f"shape mismatch for {name}: {p.shape} vs {r.shape}")
            p = q
        if r.dtype == bool or p.dtype == bool:
            differ = np.not_equal(p.astype(bool), r.astype(bool))
            if differ.any():
                where = tuple(np.unravel_index(np.argmax(differ.astype(np.int32)), differ.shape))
                return DiffResult(False, float("inf"), float("inf"), where, f"mismatch in {name} (bool)")
            continue
        p_bad, r_bad = ~np.isfinite(p), ~np.isfinite(r)
        if p_bad.any() or r_bad.any():
            if not np.array_equal(p_bad, r_bad):
                return DiffResult(False, float("inf"), float("inf"), None, f"non-finite pattern mismatch in {name}")
            if not np.array_equal(p[p_bad], r[r_bad]):
                return DiffResult(False, float("inf"), float("inf"), None, f"non-finite values mismatch in {name}")
        finite = ~(p_bad | r_bad)
        abs_err = np.zeros(r.shape, np.float64)
        rel_err = np.zeros(r.shape, np.float64)
        r64 = r.astype(np.float64, copy=False)
        if finite.any():
            p64 = p.astype(np.float64, copy=False)
            abs_err[finite] = np.abs(p64[finite] - r64[finite])
            rel_err[finite] = abs_err[finite] / (np.abs(r64[finite]) + 1e-8)
        worst_abs = max(worst_abs, float(abs_err.max()) if abs_err.size else 0.0)
        worst_rel = max(worst_rel, float(rel_err.max()) if rel_err.size else 0.0)
        limit = atol + rtol * np.abs(r64)
        over = (abs_err > limit) & finite
        if over.any():
            margin = np.where(over, abs_err - limit, -np.inf)
            bad = tuple(np.unravel_index(int(np.argmax(margin)), margin.shape))
            return DiffResult(False, worst_abs, worst_rel, bad, f"mismatch in {name}")
    return DiffResult(True, worst_abs, worst_rel, bad, "ok")


# ---- the runner ------------------------------------------------------------------------------

def run_diff(
    intent,
    run_ref_fn: Callable[[TestCase], Dict[str, np.ndarray]],
    cases: Iterable[TestCase],
    constraints=None,
    tolerances=None,
    stop_on_first_fail: bool = False,
) -> Tuple[List[DiffResult], List[Counterexample]]:
    tol = None if tolerances is None else dict(tolerances)
    cases = list(cases)
    diffs: List[DiffResult] = []
    cexs: List[Counterexample] = []

    def record(case, diff, hints):
        diffs.append(diff)
        if not diff.ok:
            cexs.append(Counterexample(case, diff, intent.to_json_dict(), None, hints))

    if any(op.op == "upsample_bicubic2d_aa" for op in intent.ops):
        d = _fail("macro expansion error: NotImplementedError: upsample_bicubic2d_aa is outside this oracle")
        first = cases[0] if cases else TestCase(shapes={}, dtypes={}, seed=0)
        return [d for _ in cases], [Counterexample(first, d, intent.to_json_dict(), None,
                                                   ["fix compiler macro expansion (not an LLM issue)"])]

    produced = {op.output for op in intent.ops if op.output}
    consumed = {n for op in intent.ops for n in op.inputs}
    external = {n for n in consumed if n in intent.tensors and n not in produced}

    for case in cases:
        try:
            io = run_ref_fn(case)
        except Exception as e:
            record(case, _fail(f"ref runner error: {type(e).__name__}: {e}"), [
                "reference runner failed (likely out-of-contract shapes or missing required inputs)",
                "try reducing case sizes or regenerating in-contract cases from contract assumptions",
            ])
            if stop_on_first_fail:
                break
            continue
        io = with_io_aliases(intent, io)
        if tol is None:
            tol = infer_tolerances(intent, ref_out=io).to_dict()
        bindings = derive_bindings(case.shapes)
        inputs = {k: v for k, v in io.items() if k in external}
        for name in sorted(n for n in external if n not in inputs):
            t = intent.tensors.get(name)
            if t is None or t.shape:
                continue
            if case.inputs and name in case.inputs:
                inputs[name] = np.asarray(case.inputs[name])
            elif name == "sm_scale" and bindings.get("HEAD_DIM") is not None and int(bindings["HEAD_DIM"]) > 0:
                inputs[name] = np.array(1.0 / np.sqrt(float(bindings["HEAD_DIM"])), dtype=np.float32)
            elif name in bindings:
                inputs[name] = np.array(bindings[name], dtype=_SCALAR_NP.get(str(t.dtype), np.float32))

        problem = None
        for name, arr in inputs.items():
            if name not in intent.tensors:
                continue
            want = _declared_shape(intent.tensors[name], bindings)
            if want is None:
                problem = (_fail(f"unbound symbols in input shape for {name}: intent shape={intent.tensors[name].shape}"),
                           ["ensure all input tensor dims are bound by case shapes (e.g., N/C/HW), and keep original view"])
                break
            if tuple(arr.shape) != tuple(want):
                problem = (_fail(f"input shape mismatch for {name}: ref {arr.shape} vs intent {want}"),
                           ["keep original input view; if you need grouped/view shapes, add intent.reshape/broadcast_in_dim ops"])
                break
        if problem is not None:
            record(case, *problem)
            if stop_on_first_fail:
                break
            continue

        try:
            with np.errstate(all="ignore"):
                pred = execute_intent(intent, inputs, shape_bindings=bindings)
            diff = compare_outputs(pred, io, intent.outputs, tol)
        except Exception as e:
            diff = _fail(f"interpreter error: {type(e).__name__}: {e}")
        record(case, diff, ["check missing ops/reshape/broadcast or wrong reduce axes"])
        if not diff.ok and stop_on_first_fail:
            break
    return diffs, cexs
