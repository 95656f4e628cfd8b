"""The ``b200`` backend object and the verifier hook.

``make_run_ref_fn(intent, input_gen)`` builds the one callable the reference's verifier
needs — ``run_ref_fn: Callable[[TestCase], Dict[str, np.ndarray]]`` of
``verify.diff_runner.run_diff`` (diff_runner.py:37-44) and of the metamorphic / stability
suites — backed by the B200 kernels: it takes the shapes from ``case.shapes``, honours
``case.inputs`` overrides (verify/metamorphic.py:133-139, numerical_stability.py:136-141),
seeds generated inputs from ``case.seed``, runs the lowered plan and returns inputs and
outputs under the graph's own tensor names.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, Mapping, Optional

import numpy as np

from . import registry
from .bindings import derive_bindings
from .ir import IntentFunction, as_intent
from .lowering import B200LoweredKernel, lower_intent_to_b200_kernel

_NP_OF = {"f32": np.float32, "bf16": np.float32, "f16": np.float32, "f64": np.float64, "i32": np.int32, "i64": np.int64,
          "i8": np.int8, "i16": np.int16, "u8": np.uint8, "bool": np.bool_, "i1": np.bool_}


def round_to_bf16(a: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bfloat16 (ties to even), keeping float32 storage:
    how bf16-declared inputs are made exactly representable on both sides of a diff."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32)
    rounded = ((bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)).astype(np.uint32)
    out = rounded.view(np.float32).copy()
    nan = np.isnan(a)
    if nan.any():
        out[nan] = np.nan
    return out


def default_inputs(intent: IntentFunction, bindings: Mapping[str, Any], seed: int) -> Dict[str, np.ndarray]:
    """Seeded inputs for every external tensor: N(0,1) for floats (bf16/f16 values rounded to
    bf16), {0,1} for booleans, small non-negative integers for integer types."""
    rng = np.random.default_rng(int(seed))
    out: Dict[str, np.ndarray] = {}
    for name in intent.external_inputs():
        t = intent.tensors[name]
        shape = tuple(int(bindings[d.value]) if d.kind == "sym" else int(d.value) for d in t.shape)
        dt = _NP_OF[t.dtype]
        if t.dtype in ("f32", "f64"):
            out[name] = rng.standard_normal(shape).astype(dt)
        elif t.dtype in ("bf16", "f16"):
            out[name] = round_to_bf16(rng.standard_normal(shape).astype(np.float32))
        elif t.dtype in ("bool", "i1"):
            out[name] = rng.integers(0, 2, size=shape).astype(np.bool_)
        else:
            out[name] = rng.integers(0, 4, size=shape).astype(dt)
    return out


class B200Backend:
    name = "b200"

    def lower(self, intent, shape_bindings: Mapping[str, Any], schedule_override=None) -> B200LoweredKernel:
        return lower_intent_to_b200_kernel(intent, shape_bindings=shape_bindings, schedule_override=schedule_override)

    def run(self, lowered: B200LoweredKernel, inputs_np: Mapping[str, np.ndarray]) -> Dict[str, np.ndarray]:
        from .runtime import run_lowered  # torch is imported only when something runs

        return run_lowered(lowered, inputs_np)

    def make_run_ref_fn(self, intent, input_gen: Optional[Callable[[Any], Dict[str, np.ndarray]]] = None):
        return make_run_ref_fn(intent, input_gen)


def make_run_ref_fn(intent, input_gen: Optional[Callable[[Any], Dict[str, np.ndarray]]] = None):
    """``input_gen(case)`` may return any subset of the inputs (and may return extra keys,
    e.g. a numpy reference runner that also returns outputs: only the graph's external
    inputs are used).  Missing inputs are generated from ``case.seed``."""
    fn = as_intent(intent)
    ext = fn.external_inputs()

    def run(case) -> Dict[str, np.ndarray]:
        bindings = derive_bindings(dict(case.shapes))
        lowered = lower_intent_to_b200_kernel(fn, shape_bindings=bindings)
        given: Dict[str, np.ndarray] = {}
        if input_gen is not None:
            given.update({k: v for k, v in input_gen(case).items() if k in ext})
        if getattr(case, "inputs", None):
            given.update({k: np.asarray(v) for k, v in case.inputs.items() if k in ext})
        if any(n not in given for n in ext):
            for k, v in default_inputs(fn, bindings, getattr(case, "seed", 0)).items():
                given.setdefault(k, v)
        for n in ext:  # scalar tensors may arrive as (1,) arrays
            want = tuple(int(bindings[d.value]) if d.kind == "sym" else int(d.value) for d in fn.tensors[n].shape)
            if np.asarray(given[n]).shape != want and np.asarray(given[n]).size == 1 and int(np.prod(want, dtype=np.int64)) == 1:
                given[n] = np.asarray(given[n]).reshape(want)
        from .runtime import run_lowered

        return run_lowered(lowered, given)

    return run


registry.register(B200Backend())
