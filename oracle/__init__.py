"""CPU oracle for the IntentIR execution path — TEST INFRASTRUCTURE, not product.

A numpy restatement of the reference's verifier (``verify/interpreter.py``,
``verify/diff_runner.py``, ``verify/tolerances.py``, ``verify/gen_cases.py``), pinned to
the reference by the golden vectors under ``tests/golden/``.  Only the tests, the smoke
entry and the benchmark's CPU-baseline / reference arm may import it; the shipped
package never does.
"""

from .cases import TestCase, generate_cases  # noqa: F401
from .diff import Counterexample, DiffResult, compare_outputs, run_diff  # noqa: F401
from .interpreter import execute_intent, execute_intent_env  # noqa: F401
from .tolerances import Tolerances, infer_tolerances  # noqa: F401
