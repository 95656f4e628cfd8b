"""intent_ir_b200 — a B200 (sm_100a) execution backend for IntentIR graphs."""

from .errors import B200LoweringError, B200RuntimeError  # noqa: F401
from .ir import IntentFunction, IntentIRValidationError, as_intent  # noqa: F401

__all__ = ["IntentFunction", "IntentIRValidationError", "as_intent", "B200LoweringError", "B200RuntimeError"]
