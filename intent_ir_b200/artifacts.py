"""Pipeline report artefacts as input to the B200 backend.

The reference's pipelines leave, per kernel, a report ``<kernel>.json`` (with ``intent`` /
``intent_expanded``, ``baseline.shapes``, ``tolerances``; pipeline/tilelang/core.py:2223-2300)
and the recorded baseline tensors ``<kernel>.baseline.npz``.  Its backend smoke script
(scripts/backend_codegen_smoke.py:81-218) replays such a pair through a backend: load the
expanded graph, complete the shape bindings, feed the recorded inputs, compare the outputs
with the recorded ones under a per-kernel tolerance.  ``load_artifact`` / ``run_artifact`` are
that replay for this backend, so existing artefact directories can be pointed at it as they are.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

import numpy as np

from .bindings import derive_bindings
from .errors import B200RuntimeError
from .ir import IntentFunction

# backend_codegen_smoke.py:147-155: (atol, rtol) per kernel, 1e-3 / 1e-3 otherwise
SMOKE_TOLERANCES: Dict[str, Tuple[float, float]] = {
    "any_kernel_dim": (0.0, 0.0), "group_norm_kernel": (1e-3, 1e-3), "_attn_fwd": (1e-2, 1e-2),
    "softmax_inner": (1e-3, 1e-3), "layer_norm_persistent": (1e-3, 1e-3), "upsample_bicubic2d_aa": (1e-3, 1e-3),
}
_SHORT_NAMES = {"i": "input", "o": "output", "x": "input", "y": "output", "w": "weight", "b": "bias", "in": "input", "out": "output"}


def _canonical(name: str) -> str:
    s = str(name).strip().strip("_").lower()
    if s.startswith("ptr_"):
        s = s[4:]
    if s.endswith("_ptr"):
        s = s[:-4]
    if s.endswith("ptr") and len(s) > 3:
        s = s[:-3]
    return _SHORT_NAMES.get(s, s).replace("_", "")


def alias_io(intent: IntentFunction, io: Mapping[str, np.ndarray]) -> Dict[str, np.ndarray]:
    """Make recorded tensors reachable under the graph's tensor names (``input`` vs ``input_ptr``
    vs ``x`` ...), the matching rule of verify/diff_runner.py:313-371."""
    out = dict(io)
    groups: Dict[str, List[str]] = {}
    for key in io:
        groups.setdefault(_canonical(key), []).append(key)
    for name in set(intent.tensors) | set(intent.outputs):
        if name in out:
            continue
        canon = _canonical(name)
        keys = groups.get(canon) or []
        if len(keys) == 1:
            out[name] = io[keys[0]]
        elif keys:
            same = [k for k in keys if str(k).lower() == str(name).lower()]
            out[name] = io[same[0] if same else (canon if canon in io else keys[0])]
        elif len(canon) >= 3:
            partial = [k for k in io if canon in _canonical(k)]
            if len(partial) == 1:
                out[name] = io[partial[0]]
    return out


@dataclass
class Artifact:
    kernel: str
    intent: IntentFunction
    bindings: Dict[str, Any]
    baseline: Dict[str, np.ndarray]
    inputs: List[str]
    outputs: List[str]
    tolerances: Tuple[float, float]


def load_artifact(report_path: str, baseline_path: Optional[str] = None) -> Artifact:
    """Read ``<kernel>.json`` and ``<kernel>.baseline.npz`` (next to it unless given)."""
    with open(report_path, encoding="utf-8") as f:
        report = json.load(f)
    graph = report.get("intent_expanded") if isinstance(report.get("intent_expanded"), dict) else report.get("intent")
    if not isinstance(graph, dict):
        raise B200RuntimeError(f"{report_path}: report carries neither intent_expanded nor intent")
    intent = IntentFunction.from_json_dict(graph)
    kernel = os.path.basename(report_path)[: -len(".json")] if report_path.endswith(".json") else intent.name
    if baseline_path is None:
        baseline_path = os.path.join(os.path.dirname(report_path), f"{kernel}.baseline.npz")
    if not os.path.exists(baseline_path):
        raise B200RuntimeError(f"missing baseline npz: {baseline_path}")
    with np.load(baseline_path, allow_pickle=False) as z:
        baseline = alias_io(intent, {k: z[k] for k in z.files})
    shapes = (report.get("baseline") or {}).get("shapes") if isinstance(report.get("baseline"), dict) else None
    bindings = derive_bindings(dict(shapes or {}))
    inputs = intent.external_inputs()
    return Artifact(kernel=kernel, intent=intent, bindings=bindings, baseline=baseline, inputs=inputs,
                    outputs=list(intent.outputs), tolerances=SMOKE_TOLERANCES.get(kernel, (1e-3, 1e-3)))


def run_artifact(report_path: str, baseline_path: Optional[str] = None, device: str = "cuda") -> Dict[str, Any]:
    """Replay one artefact on the GPU; returns ``{"kernel", "ok", "max_abs_err", "failed", "kernels"}``."""
    from .lowering import lower_intent_to_b200_kernel
    from .runtime import run_lowered

    art = load_artifact(report_path, baseline_path)
    for name in art.inputs + art.outputs:
        if name not in art.baseline:
            raise B200RuntimeError(f"baseline missing {'input' if name in art.inputs else 'output'} {name} for {art.kernel}")
    lowered = lower_intent_to_b200_kernel(art.intent, shape_bindings=art.bindings)
    got = run_lowered(lowered, {n: np.asarray(art.baseline[n]) for n in art.inputs}, device=device)
    atol, rtol = art.tolerances
    failed, worst = [], 0.0
    for name in art.outputs:
        want = np.asarray(art.baseline[name])
        have = np.asarray(got[name])
        if have.shape != want.shape:
            have = have.reshape(want.shape) if have.size == want.size else have
        if have.shape != want.shape:
            failed.append(name)
            continue
        if want.dtype == np.bool_ or have.dtype == np.bool_:
            ok = bool(np.array_equal(have.astype(bool), want.astype(bool)))
        else:
            a, b = have.astype(np.float64), want.astype(np.float64)
            with np.errstate(all="ignore"):
                err = np.abs(a - b)
            finite = np.isfinite(err)
            worst = max(worst, float(err[finite].max()) if finite.any() else 0.0)
            ok = bool(np.allclose(a, b, atol=atol, rtol=rtol, equal_nan=True))
        if not ok:
            failed.append(name)
    return {"kernel": art.kernel, "ok": not failed, "max_abs_err": worst, "failed": failed,
            "kernels": [s["kernel"] for s in lowered.steps]}
