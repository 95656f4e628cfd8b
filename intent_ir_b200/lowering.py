"""Lowering: IntentIR graph + concrete bindings -> a launchable plan.

Mirrors the reference entry point
``lower_intent_to_cuda_kernel(intent, *, shape_bindings, schedule_override=None) ->
CudaLoweredKernel`` (backends/cuda/codegen/intentir_to_cuda.py:2047-2052, dataclass :27-35):
same arguments, same record fields (``kernel_name, cuda_src, io_spec, launch, output_names,
bindings``), same failure mode (a ``RuntimeError`` subclass naming what is unsupported).
The work is done by the C++ planner behind ``ib200_plan_create``; ``cuda_src`` is empty
because nothing is generated — plans select pre-compiled sm_100a kernels.  Upper-case tuning
knobs that the reference carries inside ``shape_bindings`` (``SOFTMAX_THREADS``, ``WMMA_*``,
``CUDA_*``, ``ALLOW_TF32`` ...) are accepted and ignored.
"""

from __future__ import annotations

import ctypes as C
import itertools
import json
import threading
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

from . import _lib
from .bindings import derive_bindings, normalise_bindings, resolve_expressions
from .errors import B200LoweringError
from .ir import IntentIRValidationError, as_intent

__all__ = ["B200Launch", "B200LoweredKernel", "lower_intent_to_b200_kernel", "plan_json"]


@dataclass(frozen=True)
class B200Launch:
    """Field-compatible with the reference's ``CudaLaunch`` (frontends/cuda/runtime.py:27-31).
    Informational only: grids are chosen per kernel inside the library."""

    grid: Tuple[int, int, int]
    block: Tuple[int, int, int]
    shared_mem: int = 0


class _PlanHandle:
    """Owns one ``ib200_plan_t*``."""

    def __init__(self, ptr: int):
        self.ptr = ptr

    def __del__(self):
        try:
            if self.ptr:
                _lib.load().ib200_plan_destroy(self.ptr)
        except Exception:
            pass
        self.ptr = None


@dataclass(frozen=True)
class B200LoweredKernel:
    kernel_name: str
    cuda_src: str
    io_spec: Dict[str, Any]
    launch: B200Launch
    output_names: List[str]
    bindings: Dict[str, Any]
    # extras beyond the reference record
    steps: List[Dict[str, Any]] = field(default_factory=list)
    workspace_bytes: int = 0
    status_offset: int = -1  # byte offset of the GEMM status word inside the workspace, or -1
    plan: Optional[_PlanHandle] = field(default=None, compare=False, repr=False)

    @property
    def arg_names(self) -> List[str]:
        return list(self.io_spec["arg_names"])

    @property
    def n_launches(self) -> int:
        return len(self.steps)


_CACHE: "OrderedDict[Tuple[str, str], B200LoweredKernel]" = OrderedDict()
_CACHE_LIMIT = 512
_PLAN_SERIAL = itertools.count()
_LOCK = threading.Lock()
_BY_ID: Dict[str, B200LoweredKernel] = {}


def _raise(rc: int, what: str) -> None:
    raise B200LoweringError(f"B200 lowering unsupported for intent: {what}: {_lib.last_error()}")


def _prepare(intent, shape_bindings) -> Tuple[str, str, Dict[str, Any]]:
    # A graph whose fields have the wrong type trips over itself somewhere in the parser (a list where a name is
    # expected, a number where a list is): to the caller that is an invalid graph like any other.
    try:
        fn = as_intent(intent)
    except (IntentIRValidationError, TypeError, ValueError, KeyError, AttributeError) as e:
        raise B200LoweringError(f"invalid IntentIR graph: {e}") from e
    try:
        bindings = derive_bindings(normalise_bindings(shape_bindings))
    except (TypeError, ValueError, AttributeError) as e:
        raise B200LoweringError(f"invalid shape bindings: {e}") from e
    try:
        js = resolve_expressions(fn.to_json_dict(), bindings)
    except (TypeError, ValueError, KeyError, AttributeError) as e:
        raise B200LoweringError(str(e)) from e
    # only the numeric bindings travel; tuning knobs are harmless extra symbols
    return json.dumps(js, allow_nan=True), json.dumps(bindings, sort_keys=True), bindings


def plan_json(intent, shape_bindings: Mapping[str, Any]) -> Dict[str, Any]:
    """The stateless C entry point ``ib200_plan_json``: graph JSON in, plan JSON out."""
    intent_s, bind_s, _ = _prepare(intent, shape_bindings)
    lib = _lib.load()
    cap = 1 << 16
    while True:
        buf = C.create_string_buffer(cap)
        rc = lib.ib200_plan_json(intent_s.encode(), bind_s.encode(), buf, cap)
        if rc == _lib.ERR_BUFFER and cap < (1 << 26):
            cap *= 4
            continue
        if rc != _lib.OK:
            _raise(rc, "plan_json")
        return json.loads(buf.value.decode())


def lower_intent_to_b200_kernel(intent, *, shape_bindings: Mapping[str, Any], schedule_override=None) -> B200LoweredKernel:
    """Lower ``intent`` under ``shape_bindings``.  ``schedule_override`` is accepted for
    signature compatibility; schedules are non-semantic hints and the kernels choose their
    own tiling."""
    intent_s, bind_s, bindings = _prepare(intent, shape_bindings)
    key = (intent_s, bind_s)
    with _LOCK:
        hit = _CACHE.get(key)
        if hit is not None:
            _CACHE.move_to_end(key)
            return hit
    lib = _lib.load()
    handle = C.c_void_p()
    rc = lib.ib200_plan_create(intent_s.encode(), bind_s.encode(), C.byref(handle))
    if rc != _lib.OK:
        _raise(rc, f"name={json.loads(intent_s).get('name')}")
    plan = _PlanHandle(handle.value)
    cap = 1 << 16
    while True:
        buf = C.create_string_buffer(cap)
        rc = lib.ib200_plan_describe(plan.ptr, buf, cap)
        if rc == _lib.ERR_BUFFER and cap < (1 << 26):
            cap *= 4
            continue
        if rc != _lib.OK:
            _raise(rc, "plan_describe")
        break
    d = json.loads(buf.value.decode())
    plan_id = f"{d['kernel_name']}#{next(_PLAN_SERIAL)}"  # never reused, even after cache eviction
    io_spec = dict(d["io_spec"])
    io_spec["plan_id"] = plan_id
    lowered = B200LoweredKernel(
        kernel_name=d["kernel_name"],
        cuda_src=d.get("cuda_src", ""),
        io_spec=io_spec,
        launch=B200Launch(tuple(d["launch"]["grid"]), tuple(d["launch"]["block"]), int(d["launch"]["shared_mem"])),
        output_names=list(d["output_names"]),
        bindings=dict(bindings),
        steps=list(d.get("steps", [])),
        workspace_bytes=int(d.get("workspace_bytes", 0)),
        status_offset=int(d.get("status_offset", -1)),
        plan=plan,
    )
    with _LOCK:
        _BY_ID[plan_id] = lowered
        _CACHE[key] = lowered
        while len(_CACHE) > _CACHE_LIMIT:
            _, old = _CACHE.popitem(last=False)
            _BY_ID.pop(old.io_spec.get("plan_id"), None)
    return lowered


def lookup_plan(io_spec: Mapping[str, Any]) -> B200LoweredKernel:
    pid = io_spec.get("plan_id") if isinstance(io_spec, Mapping) else None
    with _LOCK:
        hit = _BY_ID.get(pid)
    if hit is None:
        raise B200LoweringError("io_spec does not name a live plan: pass the io_spec returned by lower_intent_to_b200_kernel")
    return hit
