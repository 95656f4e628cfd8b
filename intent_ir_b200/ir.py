"""IntentIR graph types for the B200 backend: JSON in, validated graph out.

Host-side mirror of the reference's ``intent_ir/ir/ir_types.py``:

* wire format and field names of ``IntentFunction.to_json_dict`` /
  ``from_json_dict`` (ir_types.py:223-291): ``name, tensors{dtype, shape,
  layout}, ops[{op, inputs, output, attrs}], outputs, parallel_axes,
  schedule, axis_roles, meta, contract``;
* the op set of ``intent_ir/ops/opset.py:19-78``;
* the per-op arity / attribute rules of ``_validate_op_attrs``
  (ir_types.py:536-763) and the SSA rules of ``_validate_ops``
  (ir_types.py:476-533), raising :class:`IntentIRValidationError` in the same
  situations.

The classes expose the attributes the reference's verifier reads
(``intent.tensors[name].shape[i].kind/.value``, ``intent.ops[i].op/.inputs/
.output/.attrs``, ``intent.outputs``, ``intent.schedule.tile_*``), so a graph
built here can be handed to ``verify.diff_runner.run_diff`` unchanged, and a
reference ``IntentFunction`` can be handed to this backend (anything with
``to_json_dict()`` is accepted by :func:`as_intent`).

Schedule, axis roles, meta and contract are carried but never interpreted:
they are non-semantic (docs/FORMAL_SEMANTICS.md:128-135).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional

__all__ = [
    "IntentIRValidationError",
    "Dim",
    "TensorLayout",
    "TensorType",
    "Op",
    "ScheduleSketch",
    "IntentFunction",
    "as_intent",
    "CORE_OPS",
    "SUPPORTED_OPS",
    "SUPPORTED_DTYPES",
]


class IntentIRValidationError(Exception):
    """Raised when an IntentIR graph violates the schema or the SSA rules."""


SUPPORTED_DTYPES = frozenset(
    {"f16", "bf16", "f32", "f64", "i8", "i16", "u8", "i1", "i32", "i64", "bool"}
)

# intent_ir/ops/opset.py:19-63
CORE_OPS = frozenset(
    {
        "matmul", "softmax", "dropout", "correlation", "resize", "warp", "rope",
        "add", "sub", "mul", "div", "max", "min",
        "ne", "lt", "le", "gt", "ge", "and", "or", "not",
        "exp", "relu", "rsqrt", "abs", "floor", "cast", "where",
        "iota", "gather", "identity", "const",
        "reduce_sum", "reduce_any", "reduce_max",
        "broadcast_in_dim", "transpose", "reshape", "layout_cast",
    }
)
# conv2d is schema-legal but not executable; upsample_bicubic2d_aa is a macro
# (opset.py:65-78).
SUPPORTED_OPS = CORE_OPS | {"conv2d", "upsample_bicubic2d_aa"}

_LAYOUT_KINDS = ("row_major", "col_major", "blocked", "custom")
_AXIS_ROLES = ("spatial", "reduction", "batch", "channel")
_EPILOGUE_OPS = frozenset(
    {"add", "sub", "mul", "div", "relu", "exp", "max", "min", "ne", "sigmoid", "tanh",
     "gelu", "clip", "identity", "cast", "rsqrt"}
)
# one-input form of a binary op and the attribute that carries the second
# operand (interpreter.py:215-226).
SCALAR_ATTR_OF = {
    "div": "divisor", "add": "addend", "sub": "subtract", "mul": "mul_factor",
    "max": "other", "min": "other",
}


@dataclass(frozen=True)
class Dim:
    kind: str  # "sym" | "const"
    value: Any  # str for sym, int for const


@dataclass(frozen=True)
class TensorLayout:
    kind: str = "row_major"
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class TensorType:
    dtype: str
    shape: List[Dim]
    layout: TensorLayout = field(default_factory=TensorLayout)


@dataclass
class Op:
    op: str
    inputs: List[str]
    output: str
    attrs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ScheduleSketch:
    tile_m: Any = None
    tile_n: Any = None
    tile_k: Any = None
    vec_width: Any = None
    pipeline_depth: Any = None
    axis_bindings: Dict[str, str] = field(default_factory=dict)
    vec_axis: Optional[str] = None
    parallel_axes: List[str] = field(default_factory=list)
    memory_hint: Dict[str, Any] = field(default_factory=dict)


def _fail(msg: str) -> None:
    raise IntentIRValidationError(msg)


def _dim(x: Any) -> Dim:
    if isinstance(x, bool):
        _fail(f"invalid dimension type: {type(x)}")
    if isinstance(x, int):
        return Dim("const", x)
    if isinstance(x, str):
        return Dim("sym", x)
    _fail(f"invalid dimension type: {type(x)}")


def _layout(x: Any) -> TensorLayout:
    if isinstance(x, str):
        if x in ("scalar", "dense"):  # informal tags accepted by the reference
            return TensorLayout("row_major", {})
        if x not in ("row_major", "col_major"):
            _fail(f"unsupported layout: {x}")
        return TensorLayout(x, {})
    if not isinstance(x, dict):
        _fail("layout must be string or object")
    kind, params = x.get("kind"), x.get("params", {})
    if kind not in _LAYOUT_KINDS:
        _fail(f"unsupported layout kind: {kind}")
    if not isinstance(params, dict):
        _fail("layout.params must be an object")
    return TensorLayout(kind, params)


def _tensor(name: str, data: Any) -> TensorType:
    if not isinstance(data, dict):
        _fail(f"tensor {name} must be an object")
    dtype = data.get("dtype")
    if dtype not in SUPPORTED_DTYPES:
        _fail(f"tensors.{name}.dtype unsupported: {dtype}")
    shape = data.get("shape")
    if not isinstance(shape, list):
        _fail(f"tensors.{name}.shape must be a list")
    return TensorType(dtype, [_dim(d) for d in shape], _layout(data.get("layout", "row_major")))


def _op(data: Any) -> Op:
    if not isinstance(data, dict):
        _fail("each op must be an object")
    name, inputs, output = data.get("op"), data.get("inputs") or [], data.get("output")
    attrs = data.get("attrs", {})
    if not isinstance(name, str):
        _fail("op.op must be a string")
    if not isinstance(inputs, list):
        _fail(f"op.inputs must be a list for op {name}")
    if not isinstance(output, str):
        _fail(f"op.output must be a string for op {name}")
    if attrs is None:
        attrs = {}
    if not isinstance(attrs, dict):
        _fail(f"op.attrs must be an object for op {name}")
    return Op(name, list(inputs), output, attrs)


# ---- per-op attribute rules -------------------------------------------------

_ARITY_1 = ("abs", "floor", "not", "exp", "relu", "rsqrt")
_ARITY_2 = ("lt", "le", "gt", "ge", "and", "or", "ne")
_FIXED_ARITY = {
    "matmul": (2, "matmul requires 2 inputs (A, B)"),
    "cast": (1, "cast requires 1 input"),
    "where": (3, "where requires 3 inputs (cond, x, y)"),
    "dropout": (3, "dropout requires 3 inputs (X, p, seed)"),
    "correlation": (3, "correlation requires 3 inputs (src0, src1, out_shift)"),
    "resize": (1, "resize requires 1 input (src)"),
    "warp": (2, "warp requires 2 inputs (src, offset)"),
    "rope": (3, "rope requires 3 inputs (input, cos, sin)"),
    "identity": (1, "identity requires 1 input"),
    "softmax": (1, "softmax requires 1 input"),
    "broadcast_in_dim": (1, "broadcast_in_dim requires 1 input"),
    "transpose": (1, "transpose requires 1 input"),
    "reshape": (1, "reshape requires 1 input"),
    "layout_cast": (1, "layout_cast requires 1 input"),
    "upsample_bicubic2d_aa": (1, "upsample_bicubic2d_aa requires 1 input (the input tensor)"),
}


def _check_epilogue(node: Any, path: str) -> None:
    if isinstance(node, str):
        return
    if not isinstance(node, dict):
        _fail(f"{path} must be string or object")
    if node.get("op") not in _EPILOGUE_OPS:
        _fail(f"{path}.op unsupported: {node.get('op')}")
    if not isinstance(node.get("inputs"), list):
        _fail(f"{path}.inputs must be list")
    for i, child in enumerate(node["inputs"]):
        _check_epilogue(child, f"{path}.inputs[{i}]")


def _check_op(op: Op, idx: int) -> None:
    a, kind, n_in = op.attrs or {}, op.op, len(op.inputs)
    where = f"op[{idx}]"
    if kind in _FIXED_ARITY and n_in != _FIXED_ARITY[kind][0]:
        _fail(f"{where} {_FIXED_ARITY[kind][1]}")
    if kind in _ARITY_1 and n_in != 1:
        _fail(f"{where} {kind} requires 1 input")
    if kind in _ARITY_2 and n_in != 2:
        _fail(f"{where} {kind} requires 2 inputs")

    if kind == "matmul":
        acc = a.get("accum_dtype")
        if acc is not None and acc not in SUPPORTED_DTYPES:
            _fail(f"{where}.attrs.accum_dtype unsupported: {acc}")
        if "epilogue" in a:
            _check_epilogue(a["epilogue"], f"{where}.attrs.epilogue")
    elif kind == "const":
        if op.inputs:
            _fail(f"{where} const requires 0 inputs")
        if "value" not in a:
            _fail(f"{where} const requires attrs.value")
        if a.get("dtype") is not None and a["dtype"] not in SUPPORTED_DTYPES:
            _fail(f"{where}.attrs.dtype unsupported: {a['dtype']}")
    elif kind == "cast":
        to = a.get("to")
        if to is None:
            hint = " (not attrs.dtype)" if "dtype" in a else ""
            _fail(f"{where} cast requires attrs.to{hint}")
        if to not in SUPPORTED_DTYPES:
            _fail(f"{where} cast.to unsupported: {to}")
    elif kind == "iota":
        if op.inputs:
            _fail(f"{where} iota requires 0 inputs")
        shape, axis = a.get("shape"), a.get("axis")
        if axis is None and "dimension" in a:
            _fail(f"{where} iota requires attrs.axis (not attrs.dimension)")
        if not isinstance(shape, list) or not shape:
            _fail(f"{where} iota.shape must be non-empty list")
        for d in shape:
            _dim(d)
        if axis is None:
            _fail(f"{where} iota requires attrs.axis")
        if not isinstance(axis, int):
            _fail(f"{where} iota.axis must be int, got {type(axis).__name__}")
        if a.get("dtype", "i32") not in SUPPORTED_DTYPES:
            _fail(f"{where} iota.dtype unsupported: {a.get('dtype')}")
    elif kind == "gather":
        if n_in < 2:
            _fail(f"{where} gather requires data + index tensors")
    elif kind == "dropout":
        if a.get("n_rounds") is not None and not isinstance(a["n_rounds"], int):
            _fail(f"{where} dropout.attrs.n_rounds must be int when provided")
    elif kind == "resize":
        if a.get("hw_fl") is not None and not isinstance(a["hw_fl"], int):
            _fail(f"{where} resize.attrs.hw_fl must be int when provided")
    elif kind == "identity":
        if a:
            _fail(f"{where} identity must not have attrs (slice/assign_slice unsupported)")
    elif kind in SCALAR_ATTR_OF:
        if n_in == 2 or (n_in == 1 and SCALAR_ATTR_OF[kind] in a):
            return
        _fail(f"{where} {kind} requires 2 inputs (or 1+scalar attr)")
    elif kind in ("reduce_sum", "reduce_max", "reduce_any"):
        if n_in != 1:
            _fail(f"{where} {kind} requires 1 input")
        dims = a.get("dims")
        if dims is None:
            dims = a.get("reduce_dims")
        if dims is None:
            dims = a.get("axis")
            if isinstance(dims, int):
                dims = [dims]
        if dims is None:
            _fail(f"{where} {kind} requires dims or axis")
        if not isinstance(dims, list) or not dims or not all(isinstance(x, int) for x in dims):
            _fail(f"{where} {kind}.dims must be list[int]")
    elif kind == "softmax":
        axis = a.get("axis")
        if axis is None:
            _fail(f"{where} softmax requires axis")
        if not isinstance(axis, int):
            _fail(f"{where} softmax.axis must be int, got {type(axis).__name__}")
        if a.get("stable") is not None and not isinstance(a["stable"], bool):
            _fail(f"{where}.attrs.stable must be bool when provided")
    elif kind == "broadcast_in_dim":
        out_shape, bdims = a.get("out_shape"), a.get("broadcast_dims")
        if not isinstance(out_shape, list) or not out_shape:
            _fail(f"{where} broadcast_in_dim.out_shape must be non-empty list")
        for d in out_shape:
            _dim(d)
        if not isinstance(bdims, list):
            _fail(f"{where} broadcast_in_dim.broadcast_dims must be a list")
        for j, v in enumerate(bdims):
            if not isinstance(v, int):
                _fail(f"{where} broadcast_in_dim.broadcast_dims[{j}] must be int")
    elif kind == "transpose":
        perm = a.get("perm")
        if not isinstance(perm, list) or not perm or not all(isinstance(p, int) for p in perm):
            _fail(f"{where} transpose.perm must be list of int")
    elif kind == "reshape":
        shape = a.get("shape")
        if not isinstance(shape, list) or not shape:
            _fail(f"{where} reshape.shape must be non-empty list")
        for d in shape:
            _dim(d)
    elif kind == "layout_cast":
        if not isinstance(a.get("to"), str):
            _fail(f"{where} layout_cast.to must be string")


@dataclass
class IntentFunction:
    name: str
    tensors: Dict[str, TensorType]
    ops: List[Op]
    outputs: List[str]
    contract: Any = None
    parallel_axes: List[str] = field(default_factory=list)
    schedule: Optional[ScheduleSketch] = None
    meta: Dict[str, Any] = field(default_factory=dict)
    axis_roles: Dict[str, str] = field(default_factory=dict)

    # -- JSON -----------------------------------------------------------------
    @classmethod
    def from_json_dict(cls, data: Mapping[str, Any]) -> "IntentFunction":
        tensors_json = data.get("tensors") or {}
        if not isinstance(tensors_json, dict):
            _fail("tensors must be an object")
        ops_json = data.get("ops") or []
        if not isinstance(ops_json, list):
            _fail("ops must be a list")
        ops = [_op(o) for o in ops_json]
        outputs = data.get("outputs")
        if outputs is None:
            outputs = [ops[-1].output] if ops else []
        if not isinstance(outputs, list):
            _fail("outputs must be a list if provided")
        schedule = None
        if data.get("schedule") is not None:
            s = data["schedule"]
            if not isinstance(s, dict):
                _fail("schedule must be an object")
            schedule = ScheduleSketch(
                s.get("tile_m"), s.get("tile_n"), s.get("tile_k"), s.get("vec_width"),
                s.get("pipeline_depth"), s.get("axis_bindings") or {}, s.get("vec_axis"),
                s.get("parallel_axes") or [], s.get("memory_hint") or {},
            )
        parallel_axes = data.get("parallel_axes") or []
        if schedule and schedule.parallel_axes:
            parallel_axes = schedule.parallel_axes
        meta = dict(data["meta"]) if isinstance(data.get("meta"), dict) else {}
        contract = data.get("contract")
        if contract is None and isinstance(meta.get("contract"), dict):
            contract = meta.pop("contract")
        fn = cls(
            name=data.get("name") or data.get("kernel_type") or "intent_fn",
            tensors={k: _tensor(k, v) for k, v in tensors_json.items()},
            ops=ops,
            outputs=list(outputs),
            contract=contract if isinstance(contract, dict) else None,
            parallel_axes=list(parallel_axes),
            schedule=schedule,
            meta=meta,
            axis_roles=dict(data.get("axis_roles") or {}),
        )
        fn.validate()
        return fn

    def to_json_dict(self) -> Dict[str, Any]:
        def layout_json(l: TensorLayout) -> Any:
            if l.kind in ("row_major", "col_major") and not l.params:
                return l.kind
            return {"kind": l.kind, "params": dict(l.params)}

        out: Dict[str, Any] = {
            "name": self.name,
            "tensors": {
                k: {"dtype": t.dtype, "shape": [d.value for d in t.shape], "layout": layout_json(t.layout)}
                for k, t in self.tensors.items()
            },
            "ops": [
                dict({"op": o.op, "inputs": list(o.inputs), "output": o.output},
                     **({"attrs": o.attrs} if o.attrs else {}))
                for o in self.ops
            ],
            "outputs": list(self.outputs),
            "parallel_axes": list(self.parallel_axes),
        }
        if self.contract is not None:
            out["contract"] = dict(self.contract)
        if self.schedule is not None:
            s = self.schedule
            out["schedule"] = {
                "tile_m": s.tile_m, "tile_n": s.tile_n, "tile_k": s.tile_k, "vec_width": s.vec_width,
                "pipeline_depth": s.pipeline_depth, "axis_bindings": dict(s.axis_bindings),
                "vec_axis": s.vec_axis, "parallel_axes": list(s.parallel_axes),
                "memory_hint": dict(s.memory_hint),
            }
        if self.axis_roles:
            out["axis_roles"] = dict(self.axis_roles)
        if self.meta:
            out["meta"] = dict(self.meta)
        return out

    # -- validation -----------------------------------------------------------
    def validate(self) -> None:
        for name, t in self.tensors.items():
            if t.dtype not in SUPPORTED_DTYPES:
                _fail(f"tensors.{name}.dtype unsupported: {t.dtype}")
            for i, d in enumerate(t.shape):
                if not isinstance(d, Dim):
                    _fail(f"tensors.{name}.shape[{i}] is not a Dim")
                if d.kind == "const" and not isinstance(d.value, int):
                    _fail(f"tensors.{name}.shape[{i}] const must be int")
                if d.kind == "sym" and not isinstance(d.value, str):
                    _fail(f"tensors.{name}.shape[{i}] sym must be str")
            if t.layout.kind not in _LAYOUT_KINDS:
                _fail(f"tensors.{name}.layout unsupported: {t.layout.kind}")
            if t.layout.kind == "blocked":
                if not t.layout.params:
                    _fail(f"tensors.{name}.layout blocked requires params")
                for k, v in t.layout.params.items():
                    if not isinstance(v, int):
                        _fail(f"tensors.{name}.layout.params[{k}] must be int for blocked layout")
        for axis, role in self.axis_roles.items():
            if role not in _AXIS_ROLES:
                _fail(f"axis_roles.{axis} role unsupported: {role}")
        if not self.ops:
            _fail("ops must not be empty")
        known, produced = set(self.tensors), set()
        for idx, op in enumerate(self.ops):
            if op.op not in SUPPORTED_OPS:
                _fail(f"op[{idx}].op unsupported: {op.op}")
            for inp in op.inputs:
                if inp not in known:
                    _fail(
                        f"Error: op[{idx}] '{op.op}' references undefined tensor '{inp}'\n"
                        f"Note: Available tensors at this point: {sorted(known)}"
                    )
            _check_op(op, idx)
            if op.output in produced:
                _fail(f"op[{idx}].output duplicates previous op output: {op.output}")
            produced.add(op.output)
            known.add(op.output)
        if not self.outputs:
            _fail("outputs must not be empty")
        for i, out in enumerate(self.outputs):
            if out not in self.tensors:
                _fail(f"outputs[{i}] not found in tensors: {out}")
        shape_axes = {d.value for t in self.tensors.values() for d in t.shape if d.kind == "sym"}
        for i, ax in enumerate(self.parallel_axes):
            if not isinstance(ax, str):
                _fail(f"parallel_axes[{i}] must be string")
            if shape_axes and ax not in shape_axes:
                _fail(f"parallel_axes[{i}] not found in any tensor shape: {ax}")
        if self.schedule is not None:
            s = self.schedule
            for k in ("tile_m", "tile_n", "tile_k", "vec_width", "pipeline_depth"):
                v = getattr(s, k)
                if v is not None and not isinstance(v, (int, str)):
                    _fail(f"schedule.{k} must be int/str/None")
            if s.parallel_axes and list(s.parallel_axes) != list(self.parallel_axes):
                _fail("schedule.parallel_axes must match function.parallel_axes when both are set")

    # -- helpers used by the backend -------------------------------------------
    def external_inputs(self) -> List[str]:
        """Declared tensors consumed by ops and produced by none, in first-use
        order (the set ``run_diff`` feeds to the interpreter, diff_runner.py:142-147)."""
        produced = {o.output for o in self.ops}
        seen: List[str] = []
        for o in self.ops:
            for n in o.inputs:
                if n in self.tensors and n not in produced and n not in seen:
                    seen.append(n)
        return seen


def as_intent(obj: Any) -> IntentFunction:
    """Accept this module's IntentFunction, a reference IntentFunction (anything
    with ``to_json_dict``) or a JSON dict."""
    if isinstance(obj, IntentFunction):
        return obj
    if hasattr(obj, "to_json_dict"):
        return IntentFunction.from_json_dict(obj.to_json_dict())
    if isinstance(obj, Mapping):
        return IntentFunction.from_json_dict(obj)
    raise TypeError(f"cannot interpret {type(obj).__name__} as an IntentIR graph")
