"""Oracle tolerances — TEST INFRASTRUCTURE.  Restates ``verify/tolerances.py`` of the
reference (``_OP_TOL_F32`` :34-47, ``infer_tolerances`` :68-129): a kernel-level
``(atol, rtol)`` picked from the op mix and the dtypes seen.

Rule, in order: start at (1e-4, 1e-4); take the max over per-op floors {softmax 1e-4,
exp / rsqrt 3e-4, reduce_sum / reduce_max 1e-3, matmul 2e-2, reduce_any 0}; with more than
one matmul raise to 2e-2·(1 + 0.5·(n−1)); if any f16/bf16 is visible (numpy dtypes of
``ref_out`` when given, else the declared dtype strings) floor at 1e-3; (0, 0) falls back
to (1e-3, 1e-3); finally cap at 1e-3, or at the matmul figure when a matmul is present.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Optional

import numpy as np

__all__ = ["Tolerances", "infer_tolerances"]

_FLOORS = {"softmax": 1e-4, "exp": 3e-4, "rsqrt": 3e-4, "matmul": 2e-2, "reduce_sum": 1e-3,
           "reduce_max": 1e-3, "reduce_any": 0.0}
_LEGACY = 1e-3


@dataclass(frozen=True)
class Tolerances:
    atol: float
    rtol: float

    def to_dict(self) -> Dict[str, float]:
        return {"atol": float(self.atol), "rtol": float(self.rtol)}


def _kind_of(dt) -> str:
    d = np.dtype(dt)
    for name, ref in (("f16", np.float16), ("f32", np.float32), ("f64", np.float64), ("bool", np.bool_)):
        if d == ref:
            return name
    return "int" if np.issubdtype(d, np.integer) else str(d)


def infer_tolerances(intent, *, ref_out: Optional[Mapping[str, np.ndarray]] = None) -> Tolerances:
    n_matmul = sum(1 for op in intent.ops if op.op == "matmul")
    level = max([1e-4] + [_FLOORS[op.op] for op in intent.ops if op.op in _FLOORS])
    matmul_level = 2e-2 * (1.0 + 0.5 * max(0, n_matmul - 1))
    if n_matmul > 1:
        level = max(level, matmul_level)

    seen = set()
    if ref_out is not None:
        for name in set(intent.outputs) | set(intent.tensors):
            if name in ref_out:
                try:
                    seen.add(_kind_of(np.asarray(ref_out[name]).dtype))
                except Exception:
                    pass
    else:
        seen = {str(t.dtype) for t in intent.tensors.values()}
    if "f16" in seen or "bf16" in seen:
        level = max(level, _LEGACY)
    if level == 0.0:
        return Tolerances(_LEGACY, _LEGACY)
    cap = max(_LEGACY, matmul_level) if n_matmul > 0 else _LEGACY
    level = min(max(level, 0.0), cap)
    return Tolerances(level, level)
