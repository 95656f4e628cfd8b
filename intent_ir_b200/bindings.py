"""Shape bindings: what the caller passes, what the graph needs.

``normalise_bindings`` applies the reference's rule for ``shape_bindings`` values
(backends/cuda/codegen/intentir_to_cuda.py:2059-2072): bools and ints stay ints, anything
float-like becomes an int when integral else a float, everything else is dropped.

``derive_bindings`` adds the symbols the reference's ``run_diff`` derives before it runs
the interpreter (verify/diff_runner.py:101-140) — ``Z``/``batch``, ``num_groups`` from
``group``, ``group_size = C / num_groups``, ``num_elements = group_size * HW``,
``G = N / group_size`` and the ``HEAD_DIM_*`` halves — because a backend runner only sees
``case.shapes`` and has to arrive at the same graph the interpreter executes.

``resolve_expressions`` replaces the attribute strings that the interpreter evaluates as
Python expressions over the bindings (``const.value`` such as ``"1.0/(HEAD_DIM**0.5)"``,
interpreter.py:521-544; ``reduce_sum.scale`` such as ``"1.0/N"``, :646-673) with numbers,
so that the C++ planner only ever sees numbers, value names and bound symbols.
"""

from __future__ import annotations

import ast
import copy
import operator
from typing import Any, Dict, Mapping

_BIN = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv,
        ast.FloorDiv: operator.floordiv, ast.Mod: operator.mod, ast.Pow: operator.pow}
_UN = {ast.UAdd: operator.pos, ast.USub: operator.neg}


def normalise_bindings(shape_bindings: Mapping[str, Any]) -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    for k, v in dict(shape_bindings).items():
        if isinstance(v, bool):
            out[str(k)] = int(v)
        elif isinstance(v, int):
            out[str(k)] = int(v)
        else:
            try:
                f = float(v)
            except Exception:
                continue
            out[str(k)] = int(f) if f.is_integer() else f
    return out


def derive_bindings(shapes: Mapping[str, Any]) -> Dict[str, Any]:
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
        for alias in ("HEAD_DIM_DIV2", "HEAD_DIM_DIV_2", "HEAD_DIM_HALF", "HEAD_DIM_MID"):
            b.setdefault(alias, int(b["HEAD_DIM"]) // 2)
    return b


def eval_expression(text: str, bindings: Mapping[str, Any]) -> float:
    """Arithmetic over bound symbols: + - * / // % ** and parentheses, nothing else."""

    def ev(node):
        if isinstance(node, ast.Expression):
            return ev(node.body)
        if isinstance(node, ast.Constant) and isinstance(node.value, (int, float)) and not isinstance(node.value, bool):
            return node.value
        if isinstance(node, ast.Name):
            if node.id in bindings:
                return bindings[node.id]
            raise ValueError(f"unbound symbol {node.id!r}")
        if isinstance(node, ast.BinOp) and type(node.op) in _BIN:
            return _BIN[type(node.op)](ev(node.left), ev(node.right))
        if isinstance(node, ast.UnaryOp) and type(node.op) in _UN:
            return _UN[type(node.op)](ev(node.operand))
        raise ValueError(f"unsupported syntax in expression {text!r}")

    return float(ev(ast.parse(text, mode="eval")))


def _is_number_text(s: str) -> bool:
    try:
        float(s)
        return True
    except Exception:
        return False


def resolve_expressions(intent_json: Dict[str, Any], bindings: Mapping[str, Any]) -> Dict[str, Any]:
    """A copy of the graph JSON in which expression strings have become numbers."""
    js = copy.deepcopy(intent_json)
    produced = set(js.get("tensors", {}))
    for op in js.get("ops", []):
        attrs = op.get("attrs") or {}
        kind = op.get("op")
        if kind == "const" and isinstance(attrs.get("value"), str):
            v = attrs["value"]
            if v.startswith("placeholder:"):
                raise ValueError(f"placeholder const is not a valid semantic value: {v}")
            if v not in produced and v not in bindings and not _is_number_text(v) and v != "eps":
                try:
                    attrs["value"] = eval_expression(v, bindings)
                except Exception:
                    raise ValueError(f"unresolved const value: {v}") from None
        if kind == "reduce_sum" and isinstance(attrs.get("scale"), str):
            v = attrs["scale"]
            scope = dict(bindings)
            if "num_elements" not in scope and isinstance(scope.get("group_size"), int) and isinstance(scope.get("HW"), int):
                scope["num_elements"] = scope["group_size"] * scope["HW"]
            if v in scope:
                attrs["scale"] = float(scope[v])
            else:
                try:
                    attrs["scale"] = eval_expression(v, scope)
                except Exception as e:
                    raise ValueError(f"unresolved reduce scale: {v}") from e
        produced.add(op.get("output"))
    return js
