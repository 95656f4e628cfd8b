"""Put the reference's own verifier where the GPU box can import it — TEST INFRASTRUCTURE.

    python oracle/install_reference.py [/path/to/intent_ir]

The reference is pure Python on this path.  Its checkout exists only on the build machine, so this
recipe copies the packages the verification path needs — ``intent_ir/{ir,macros,ops}``, ``verify/``
and ``pipeline/{__init__,interfaces,registry,run}.py`` — unmodified into ``baseline/_ref/`` at the
repository root.  That folder is git-ignored (reference sources never enter this repository's
history) but travels with a working copy, so that the GPU tests can hand the CUDA backend to the
reference's ``run_diff`` / ``run_metamorphic_suite`` / ``run_bounded_exhaustive`` /
``run_numerical_stability_suite`` / ``run_mutation_kill`` themselves, and ``bench.py --impl
reference`` can time the reference's ``verify.interpreter.execute_intent`` rather than the port.
Nothing in the shipped package reads the folder; ``oracle.reference_root()`` finds it for the
tests and the benchmark.
"""

from __future__ import annotations

import json
import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEST = os.path.join(ROOT, "baseline", "_ref")
PACKAGES = ["intent_ir/__init__.py", "intent_ir/diagnostics.py", "intent_ir/ir", "intent_ir/macros", "intent_ir/ops", "verify",
            "pipeline/__init__.py", "pipeline/interfaces.py", "pipeline/registry.py", "pipeline/run.py"]


def default_source() -> str:
    with open(os.path.join(ROOT, "BASELINE.json")) as f:
        return json.load(f).get("reference_path", "")


def install(src: str, dest: str = DEST) -> str:
    """Copy the verification packages of the checkout at ``src`` into ``dest``; returns ``dest``."""
    if not os.path.isdir(os.path.join(src, "verify")):
        raise FileNotFoundError(f"{src!r} is not a checkout of the reference (no verify/ package)")
    if os.path.isdir(dest):
        shutil.rmtree(dest)
    for rel in PACKAGES:
        a, b = os.path.join(src, rel), os.path.join(dest, rel)
        if not os.path.exists(a):
            continue
        os.makedirs(os.path.dirname(b), exist_ok=True)
        if os.path.isdir(a):
            shutil.copytree(a, b, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
        else:
            shutil.copy2(a, b)
    with open(os.path.join(dest, "INSTALLED_FROM"), "w") as f:
        f.write(os.path.abspath(src) + "\n")
    return dest


if __name__ == "__main__":
    print(install(sys.argv[1] if len(sys.argv) > 1 else default_source()))
