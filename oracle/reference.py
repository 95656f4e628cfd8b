"""Locating and importing the reference's own verifier — TEST INFRASTRUCTURE.

``reference_root()`` returns the first of ``$INTENTIR_REF``, ``BASELINE.json``'s
``reference_path`` (a full checkout, where the build machine has one) and ``baseline/_ref``
(the verifier packages copied by ``oracle/install_reference.py``) that holds an importable
``verify`` package, or None.  ``import_reference()`` puts it first on ``sys.path``
and returns the modules the tests and the benchmark use.
"""

from __future__ import annotations

import importlib
import json
import os
import sys
from types import SimpleNamespace
from typing import Optional

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_root() -> Optional[str]:
    candidates = [os.environ.get("INTENTIR_REF")]
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            candidates.append(json.load(f).get("reference_path"))
    except Exception:
        pass
    candidates.append(os.path.join(ROOT, "baseline", "_ref"))
    for c in candidates:
        if c and os.path.isfile(os.path.join(c, "verify", "diff_runner.py")) and os.path.isfile(os.path.join(c, "intent_ir", "ir", "ir_types.py")):
            return os.path.abspath(c)
    return None


def import_reference(root: Optional[str] = None) -> SimpleNamespace:
    """The reference's modules: ``.root, .IntentFunction, .execute_intent, .run_diff, .infer_tolerances,
    .TestCase, .generate_cases, .metamorphic, .numerical_stability, .mutation``.  Raises ImportError when
    no checkout is found."""
    root = root or reference_root()
    if root is None:
        raise ImportError("no checkout of the reference: set INTENTIR_REF or run oracle/install_reference.py where one exists")
    if root not in sys.path:
        sys.path.insert(0, root)
    mod = importlib.import_module
    ir, interp, dr = mod("intent_ir.ir"), mod("verify.interpreter"), mod("verify.diff_runner")
    tol, gc = mod("verify.tolerances"), mod("verify.gen_cases")
    return SimpleNamespace(root=root, IntentFunction=ir.IntentFunction, execute_intent=interp.execute_intent, run_diff=dr.run_diff,
                           infer_tolerances=tol.infer_tolerances, TestCase=gc.TestCase, generate_cases=gc.generate_cases,
                           metamorphic=mod("verify.metamorphic"), numerical_stability=mod("verify.numerical_stability"),
                           mutation=mod("verify.mutation"))
