"""The seeded verification sweep: many (graph, shapes, seed) cases, each lowered, run on the
GPU and diffed against the CPU interpreter, sharded over the GPUs of one box.

This is the reference's "Task5 cases + diff" stage (``generate_cases`` ->
``run_diff(intent, run_ref_fn, cases)``, pipeline/triton/core.py:2552-2602,
verify/diff_runner.py:37-275) turned into a batch job:

* cases are independent, so case ``i`` goes to rank ``i % world`` — one process per GPU, no
  device-side communication at all; each rank appends one JSON record per case to its own
  JSONL shard (restart skips the ids already recorded) and rank 0 merges the shards with a
  host-side gather;
* a failing case never stops the sweep: exceptions from lowering, from the GPU run or from
  the checker become failed records, the way ``pipeline/run.py:60-79`` isolates per-kernel
  errors;
* large row-independent cases can be split on their leading axis into sub-cases so that both
  the GPU work and the CPU checking of one big case spread over ranks.

The checker is injected: ``run_sweep(..., diff_fn=run_diff, tolerances_fn=infer_tolerances,
case_type=TestCase)`` takes the reference's own ``verify`` functions (or anything with the
same signatures).  ``reference_checker()`` imports them from a reference checkout named by
``$INTENTIR_REF``; this module never falls back to a checker of its own.
"""

from __future__ import annotations

import importlib
import json
import os
import sys
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from .backend import round_to_bf16

__all__ = ["SweepCase", "generate_sweep_cases", "split_rows", "run_sweep", "merge_records", "reference_checker", "KINDS",
           "CheckerPool", "partition_cases", "estimate_cost"]

EDGE_SIZES = (1, 2, 3, 7, 8, 15, 16, 17, 31, 32, 33)
KINDS = ("reduce_any", "reduce_sum", "reduce_max", "softmax", "layernorm", "groupnorm", "matmul_bias_relu", "chain")
# the graphs either side of the headline path: normalisation variants, masked softmax, the single-op kernels
EXTRA_KINDS = ("rmsnorm", "layernorm_residual", "masked_softmax", "rope", "dropout", "image")
ALL_KINDS = KINDS + EXTRA_KINDS


@dataclass
class SweepCase:
    case_id: int
    kind: str
    dtype: str
    shapes: Dict[str, int]
    seed: int
    intent: Dict[str, Any] = field(repr=False, default_factory=dict)
    elements: int = 0  # size of the largest tensor, for load balancing and memory caps


# ---- graph templates (IntentIR JSON, the wire format of intent_ir/ir/ir_types.py:273-291) ---------

def _t(shape, dtype="f32"):
    return {"dtype": dtype, "shape": list(shape), "layout": "row_major"}


def g_reduce(kind: str, dtype: str) -> Dict[str, Any]:
    out_dt = "bool" if kind == "reduce_any" else "f32"
    return {"name": f"sweep_{kind}", "tensors": {"inp": _t(["M", "N"], dtype), "out": _t(["M"], out_dt)},
            "ops": [{"op": kind, "inputs": ["inp"], "output": "out", "attrs": {"dims": [1], "keepdims": False}}],
            "outputs": ["out"]}


def g_softmax(dtype: str) -> Dict[str, Any]:
    # f32 result even for bf16 inputs: a bf16 probability above 0.5 carries a rounding error of up to
    # 2^-9 and cannot meet the verifier's 1e-3 + 1e-3*|y|
    return {"name": "sweep_softmax", "tensors": {"inp": _t(["M", "N"], dtype), "out": _t(["M", "N"], "f32")},
            "ops": [{"op": "softmax", "inputs": ["inp"], "output": "out", "attrs": {"axis": -1}}], "outputs": ["out"]}


def g_layernorm() -> Dict[str, Any]:
    ops = [
        {"op": "reduce_sum", "inputs": ["x"], "output": "s", "attrs": {"dims": [1], "keepdims": True}},
        {"op": "div", "inputs": ["s"], "output": "mu", "attrs": {"divisor": "N"}},
        {"op": "sub", "inputs": ["x", "mu"], "output": "d"},
        {"op": "mul", "inputs": ["d", "d"], "output": "sq"},
        {"op": "reduce_sum", "inputs": ["sq"], "output": "vs", "attrs": {"dims": [1], "keepdims": True}},
        {"op": "div", "inputs": ["vs"], "output": "var", "attrs": {"divisor": "N"}},
        {"op": "const", "inputs": [], "output": "eps", "attrs": {"value": 1e-5, "dtype": "f32"}},
        {"op": "add", "inputs": ["var", "eps"], "output": "ve"},
        {"op": "rsqrt", "inputs": ["ve"], "output": "rs"},
        {"op": "mul", "inputs": ["d", "rs"], "output": "xh"},
        {"op": "broadcast_in_dim", "inputs": ["w"], "output": "wb", "attrs": {"out_shape": ["M", "N"], "broadcast_dims": [1]}},
        {"op": "broadcast_in_dim", "inputs": ["b"], "output": "bb", "attrs": {"out_shape": ["M", "N"], "broadcast_dims": [1]}},
        {"op": "mul", "inputs": ["xh", "wb"], "output": "sc"},
        {"op": "add", "inputs": ["sc", "bb"], "output": "y"},
        {"op": "reshape", "inputs": ["mu"], "output": "mean", "attrs": {"shape": ["M"]}},
        {"op": "reshape", "inputs": ["rs"], "output": "rstd", "attrs": {"shape": ["M"]}},
    ]
    return {"name": "sweep_layernorm",
            "tensors": {"x": _t(["M", "N"]), "w": _t(["N"]), "b": _t(["N"]), "y": _t(["M", "N"]), "mean": _t(["M"]), "rstd": _t(["M"])},
            "ops": ops, "outputs": ["y", "mean", "rstd"]}


def g_groupnorm() -> Dict[str, Any]:
    g4 = ["N", "num_groups", 1, 1]
    ops = [
        {"op": "reshape", "inputs": ["X"], "output": "X4", "attrs": {"shape": ["N", "num_groups", "group_size", "HW"]}},
        {"op": "reduce_sum", "inputs": ["X4"], "output": "s", "attrs": {"dims": [2, 3], "keepdims": True}},
        {"op": "div", "inputs": ["s"], "output": "mu", "attrs": {"divisor": "num_elements"}},
        {"op": "sub", "inputs": ["X4", "mu"], "output": "d"},
        {"op": "mul", "inputs": ["d", "d"], "output": "sq"},
        {"op": "reduce_sum", "inputs": ["sq"], "output": "vs", "attrs": {"dims": [2, 3], "keepdims": True}},
        {"op": "div", "inputs": ["vs"], "output": "var", "attrs": {"divisor": "num_elements"}},
        {"op": "const", "inputs": [], "output": "eps", "attrs": {"value": 1e-5, "dtype": "f32"}},
        {"op": "add", "inputs": ["var", "eps"], "output": "ve"},
        {"op": "rsqrt", "inputs": ["ve"], "output": "rs"},
        {"op": "mul", "inputs": ["d", "rs"], "output": "xh4"},
        {"op": "reshape", "inputs": ["xh4"], "output": "xh", "attrs": {"shape": ["N", "C", "HW"]}},
        {"op": "broadcast_in_dim", "inputs": ["W"], "output": "W3", "attrs": {"out_shape": ["N", "C", "HW"], "broadcast_dims": [1]}},
        {"op": "broadcast_in_dim", "inputs": ["B"], "output": "B3", "attrs": {"out_shape": ["N", "C", "HW"], "broadcast_dims": [1]}},
        {"op": "mul", "inputs": ["xh", "W3"], "output": "sc"},
        {"op": "add", "inputs": ["sc", "B3"], "output": "Y"},
        {"op": "reshape", "inputs": ["mu"], "output": "Mean", "attrs": {"shape": ["N", "num_groups"]}},
        {"op": "reshape", "inputs": ["rs"], "output": "Rstd", "attrs": {"shape": ["N", "num_groups"]}},
    ]
    tensors = {"X": _t(["N", "C", "HW"]), "W": _t(["C"]), "B": _t(["C"]), "Y": _t(["N", "C", "HW"]),
               "Mean": _t(["N", "num_groups"]), "Rstd": _t(["N", "num_groups"]), "mu": _t(g4), "rs": _t(g4)}
    return {"name": "sweep_groupnorm", "tensors": tensors, "ops": ops, "outputs": ["Y", "Mean", "Rstd"]}


def g_matmul(dtype: str) -> Dict[str, Any]:
    return {"name": "sweep_matmul_bias_relu",
            "tensors": {"A": _t(["M", "K"], dtype), "B": _t(["K", "N"], dtype), "bias": _t(["N"], dtype), "C": _t(["M", "N"], dtype)},
            "ops": [{"op": "matmul", "inputs": ["A", "B"], "output": "mm", "attrs": {"accum_dtype": "f32"}},
                    {"op": "broadcast_in_dim", "inputs": ["bias"], "output": "b2", "attrs": {"out_shape": ["M", "N"], "broadcast_dims": [1]}},
                    {"op": "add", "inputs": ["mm", "b2"], "output": "mb"},
                    {"op": "relu", "inputs": ["mb"], "output": "C"}],
            "outputs": ["C"]}


def g_chain(rng: np.random.Generator, dtype: str) -> Dict[str, Any]:
    """2..6 add/mul ops over x[M,N] with [N], [M,1] and scalar operands; output f32."""
    n_ops = int(rng.integers(2, 7))
    tensors = {"x": _t(["M", "N"], dtype), "col": _t(["N"], dtype), "row": _t(["M", 1], dtype), "y": _t(["M", "N"])}
    ops, cur = [], "x"
    for i in range(n_ops):
        op = "add" if rng.random() < 0.5 else "mul"
        out = "y" if i == n_ops - 1 else f"t{i}"
        which = int(rng.integers(0, 3))
        if which == 0:
            ops.append({"op": op, "inputs": [cur, "col"], "output": out})
        elif which == 1:
            ops.append({"op": op, "inputs": [cur, "row"], "output": out})
        else:
            key = "addend" if op == "add" else "mul_factor"
            ops.append({"op": op, "inputs": [cur], "output": out, "attrs": {key: float(np.round(rng.uniform(-1.5, 1.5), 3))}})
        cur = out
    if not any("col" in o["inputs"] for o in ops):  # keep every declared input in use
        ops[0] = {"op": ops[0]["op"], "inputs": ["x", "col"], "output": ops[0]["output"]}
    if not any("row" in o["inputs"] for o in ops):
        ops[-1] = {"op": ops[-1]["op"], "inputs": [ops[-1]["inputs"][0], "row"], "output": "y"}
    return {"name": "sweep_chain", "tensors": tensors, "ops": ops, "outputs": ["y"]}


def g_rmsnorm() -> Dict[str, Any]:
    """y = x * rsqrt(mean(x^2) + 1e-5) * w, rstd returned (the chain of pipeline/tilelang/core.py:735-776)."""
    return {"name": "sweep_rmsnorm", "tensors": {"x": _t(["M", "N"]), "w": _t(["N"]), "y": _t(["M", "N"]), "rstd": _t(["M"])},
            "ops": [{"op": "mul", "inputs": ["x", "x"], "output": "sq"},
                    {"op": "reduce_sum", "inputs": ["sq"], "output": "ss", "attrs": {"dims": [1], "keepdims": True, "scale": "1.0/N"}},
                    {"op": "add", "inputs": ["ss"], "output": "ve", "attrs": {"addend": 1e-5}},
                    {"op": "rsqrt", "inputs": ["ve"], "output": "r1"},
                    {"op": "reshape", "inputs": ["r1"], "output": "rstd", "attrs": {"shape": ["M"]}},
                    {"op": "mul", "inputs": ["x", "r1"], "output": "xn"},
                    {"op": "mul", "inputs": ["xn", "w"], "output": "y"}], "outputs": ["y", "rstd"]}


def g_layernorm_residual() -> Dict[str, Any]:
    """layernorm of x + r (pipeline/tilelang/core.py:1426): the residual sum is computed first."""
    g = g_layernorm()
    g = {**g, "name": "sweep_layernorm_residual", "tensors": {**g["tensors"], "r": _t(["M", "N"]), "x0": _t(["M", "N"])}}
    ops = [dict(o, inputs=["z" if i == "x" else i for i in o["inputs"]]) for o in g["ops"]]
    g["ops"] = [{"op": "add", "inputs": ["x0", "r"], "output": "z"}] + ops
    del g["tensors"]["x"]
    return g


def g_masked_softmax() -> Dict[str, Any]:
    """softmax(where(mask[N], x, -1e9)) along the row (pipeline/tilelang/core.py:1050-1076)."""
    return {"name": "sweep_masked_softmax", "tensors": {"x": _t(["M", "N"]), "mask": _t(["N"], "bool"), "y": _t(["M", "N"])},
            "ops": [{"op": "const", "inputs": [], "output": "neg", "attrs": {"value": -1e9, "dtype": "f32"}},
                    {"op": "broadcast_in_dim", "inputs": ["mask"], "output": "m2", "attrs": {"out_shape": ["M", "N"], "broadcast_dims": [1]}},
                    {"op": "where", "inputs": ["m2", "x", "neg"], "output": "xm"},
                    {"op": "softmax", "inputs": ["xm"], "output": "y", "attrs": {"axis": -1}}], "outputs": ["y"]}


def g_rope() -> Dict[str, Any]:
    return {"name": "sweep_rope", "tensors": {"x": _t(["S", "B", "H", "D"]), "cos": _t(["S", "D2"]), "sin": _t(["S", "D2"]), "y": _t(["S", "B", "H", "D"])},
            "ops": [{"op": "rope", "inputs": ["x", "cos", "sin"], "output": "y"}], "outputs": ["y"]}


def g_dropout(rounds: int) -> Dict[str, Any]:
    return {"name": "sweep_dropout", "tensors": {"x": _t(["M", "N"]), "p": _t([]), "seed": _t([], "i64"), "y": _t(["M", "N"])},
            "ops": [{"op": "dropout", "inputs": ["x", "p", "seed"], "output": "y", "attrs": {"n_rounds": rounds}}], "outputs": ["y"]}


def g_image() -> Dict[str, Any]:
    """correlation -> 2x resize -> warp on int8 planes (verify/interpreter.py:330-454)."""
    return {"name": "sweep_image",
            "tensors": {"a": _t(["C", "H", "W"], "i8"), "b": _t(["C", "H", "W"], "i8"), "sh": _t([], "i32"), "off": _t(["H2", "W2"], "i16"),
                        "corr": _t(["OC", "H", "W"], "i8"), "up": _t(["OC", "H2", "W2"], "i8"), "out": _t(["OC", "H2", "W2"], "i8")},
            "ops": [{"op": "correlation", "inputs": ["a", "b", "sh"], "output": "corr"},
                    {"op": "resize", "inputs": ["corr"], "output": "up", "attrs": {"hw_fl": 7}},
                    {"op": "warp", "inputs": ["up", "off"], "output": "out"}], "outputs": ["out", "corr"]}


# ---- case generation ------------------------------------------------------------------------------------

def _dim(rng: np.random.Generator, hi: int = 4096) -> int:
    if rng.random() < 0.25:
        t = int(rng.choice((16, 32, 64, 128, 256, 1024)))
        return int(min(hi, rng.choice(EDGE_SIZES + (t - 1, t, t + 1, 2 * t + 1))))
    return int(rng.integers(1, hi + 1))


def _fit(dims: List[int], cap: int) -> List[int]:
    """Halve the extents in turn (first one first) until their product is at most ``cap``."""
    dims = [max(1, int(d)) for d in dims]
    i = 0
    while int(np.prod(dims, dtype=np.int64)) > cap and any(d > 1 for d in dims):
        if dims[i % len(dims)] > 1:
            dims[i % len(dims)] //= 2
        i += 1
    return dims


def generate_sweep_cases(n_cases: int, base_seed: int = 1000, max_elements: int = 1 << 24,
                         canonical_groupnorm_every: int = 0, kinds: Sequence[str] = KINDS) -> List[SweepCase]:
    """Deterministic: case ``i`` is a function of ``base_seed + i`` only.  Every free extent is
    uniform in [1, 4096] mixed with the edge sizes of verify/gen_cases.py ({1,2,3}, t-1, t, t+1,
    2t+1); dtypes are f32 or bf16; ``max_elements`` caps the largest tensor of a case."""
    out: List[SweepCase] = []
    for i in range(n_cases):
        seed = base_seed + i
        rng = np.random.default_rng(seed)
        kind = kinds[int(rng.integers(0, len(kinds)))]
        dtype = "bf16" if rng.random() < 0.3 else "f32"
        if kind in ("reduce_any", "reduce_sum", "reduce_max", "softmax", "chain"):
            m, n = _fit([_dim(rng), _dim(rng)], max_elements)
            shapes = {"M": m, "N": n}
            intent = g_softmax(dtype) if kind == "softmax" else g_chain(rng, dtype) if kind == "chain" else g_reduce(kind, dtype)
            elements = m * n
        elif kind in ("layernorm", "rmsnorm", "layernorm_residual", "masked_softmax", "dropout"):
            dtype = "f32"
            m, n = _fit([_dim(rng), _dim(rng)], max_elements)
            intent = {"layernorm": g_layernorm, "rmsnorm": g_rmsnorm, "layernorm_residual": g_layernorm_residual,
                      "masked_softmax": g_masked_softmax}[kind]() if kind != "dropout" else g_dropout(int(rng.choice((7, 10))))
            shapes, elements = {"M": m, "N": n}, m * n
        elif kind == "rope":
            dtype = "f32"
            seq, heads, half = _fit([_dim(rng, 1024), int(rng.integers(1, 17)), int(rng.integers(1, 65))], max_elements // 2)
            shapes = {"S": seq, "B": int(rng.integers(1, 3)), "H": heads, "D": 2 * half, "D2": half}
            intent, elements = g_rope(), seq * shapes["B"] * heads * 2 * half
        elif kind == "image":
            dtype = "i8"
            c, h, w = _fit([int(rng.integers(1, 9)), _dim(rng, 128), _dim(rng, 300)], max_elements // 16)
            oc = int(rng.integers(1, min(8, w + 1) + 1))
            shapes = {"C": c, "H": h, "W": w, "OC": oc, "H2": 2 * h, "W2": 2 * w}
            intent, elements = g_image(), 4 * oc * h * w
        elif kind == "groupnorm":
            dtype = "f32"
            if canonical_groupnorm_every and i % canonical_groupnorm_every == 0:
                shapes = {"N": 32, "C": 256, "HW": 4096, "num_groups": 32}
            else:
                groups, gs = int(rng.integers(1, 33)), int(rng.integers(1, 17))
                hw, nb, gs, groups = _fit([_dim(rng), int(rng.integers(1, 9)), gs, groups], max_elements)
                shapes = {"N": nb, "C": groups * gs, "HW": hw, "num_groups": groups}
            intent = g_groupnorm()
            elements = shapes["N"] * shapes["C"] * shapes["HW"]
        else:  # matmul_bias_relu
            m, n, k = _dim(rng, 2048), _dim(rng, 2048), _dim(rng, 2048)
            if dtype == "bf16":  # the tensor-core path wants 16-byte rows; other shapes also run (FMA path)
                if rng.random() < 0.7:
                    n, k = max(8, n // 8 * 8), max(8, k // 8 * 8)
            shapes, intent, elements = {"M": m, "N": n, "K": k}, g_matmul(dtype), max(m * k, k * n, m * n)
        out.append(SweepCase(case_id=i, kind=kind, dtype=dtype, shapes=shapes, seed=seed, intent=intent, elements=elements))
    return out


_ROW_AXIS = {"reduce_any": "M", "reduce_sum": "M", "reduce_max": "M", "softmax": "M", "layernorm": "M", "chain": "M",
             "matmul_bias_relu": "M", "groupnorm": "N", "rmsnorm": "M", "layernorm_residual": "M", "masked_softmax": "M"}


def split_rows(case: SweepCase, parts: int, id_stride: int = 1 << 20) -> List[SweepCase]:
    """Split a case on its leading independent axis into up to ``parts`` sub-cases (rows of
    every kind here are independent; matmul replicates B).  Sub-case ``j`` gets the id
    ``case_id + (j+1)*id_stride`` and its own seed."""
    axis = _ROW_AXIS[case.kind]
    rows = case.shapes[axis]
    parts = max(1, min(parts, rows))
    if parts == 1:
        return [case]
    base, extra = divmod(rows, parts)
    subs = []
    for j in range(parts):
        r = base + (1 if j < extra else 0)
        shapes = dict(case.shapes)
        shapes[axis] = r
        subs.append(SweepCase(case_id=case.case_id + (j + 1) * id_stride, kind=case.kind, dtype=case.dtype, shapes=shapes,
                              seed=case.seed * 131 + j, intent=case.intent, elements=case.elements * r // max(rows, 1)))
    return subs


_POOL = 1 << 16


def _u16(rng, n: int) -> np.ndarray:
    """n uniform 16-bit integers, four to a raw 64-bit draw."""
    return rng.bit_generator.random_raw((n + 3) // 4).view(np.uint16)[:n]


_CHUNK = 1 << 16  # elements generated at a time: the index and the gathered values stay in the core's cache


def _round_bf16_in_place(a: np.ndarray) -> None:
    """backend.round_to_bf16 on finite float32 values, without a second array."""
    bits = a.view(np.uint32)
    bits += np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    bits &= np.uint32(0xFFFF0000)


def _normal(rng, shape, scale=None, bf16: bool = False, out: Optional[np.ndarray] = None) -> np.ndarray:
    """Standard-normal float32 values of the given shape, times ``scale``, rounded to bf16 on request, written
    into ``out`` (a C-contiguous float32 array of that shape) when one is given.  Large tensors draw their
    elements, independently and uniformly, from 65536 normal variates generated for this tensor: the inputs of
    a sweep case cost the host as much as interpreting the graph when every element goes through the ziggurat
    (52 ms against 18 ms for 4 Mi elements), and a check of a kernel is indifferent to the difference.  The
    tensor is produced 64 Ki elements at a time (the same random stream as in one piece), scaled and rounded
    while the piece is in cache."""
    shape = (shape,) if np.isscalar(shape) else tuple(shape)
    n = int(np.prod(shape, dtype=np.int64))
    if out is None or out.shape != shape or out.dtype != np.float32 or not out.flags.c_contiguous:
        out = np.empty(shape, np.float32)
    flat = out.reshape(-1)

    def finish(piece):
        if scale is not None:
            piece *= np.float32(scale)
        if bf16:
            _round_bf16_in_place(piece)

    if n <= 4 * _POOL:
        if n:
            rng.standard_normal(out=flat, dtype=np.float32)
            finish(flat)
        return out
    pool = rng.standard_normal(_POOL, dtype=np.float32)
    for a in range(0, n, _CHUNK):
        b = min(n, a + _CHUNK)
        np.take(pool, _u16(rng, b - a), out=flat[a:b], mode="clip")  # (every index is in range; 'raise' would buffer the output)
        finish(flat[a:b])
    return out


def case_inputs(case: SweepCase, dest: Optional[Callable[[str, tuple], Optional[np.ndarray]]] = None) -> Dict[str, np.ndarray]:
    """Seeded inputs with the value distributions of the benchmark configurations; bf16 tensors
    are float32 arrays holding bf16-representable values.  ``dest(name, shape)`` may hand out the float32
    array a large tensor is to be generated into (the checker processes' shared-memory arena)."""
    rng = np.random.default_rng(case.seed)
    s = case.shapes
    b16 = case.dtype == "bf16"
    q = round_to_bf16 if b16 else (lambda a: a)
    k = case.kind

    def normal(name, shape, scale=None, rounded=b16):
        shape = (shape,) if np.isscalar(shape) else tuple(shape)
        return _normal(rng, shape, scale, rounded, dest(name, shape) if dest else None)

    if k in ("reduce_any",):
        m, n = s["M"], s["N"]
        x = normal("inp", (m, n), rounded=False)
        flat = x.reshape(-1)
        for a in range(0, m * n, _CHUNK):  # about one element in twenty is non-zero
            piece = flat[a:a + _CHUNK]
            piece[_u16(rng, piece.size) >= 3277] = 0
        if b16:
            _round_bf16_in_place(flat)
        return {"inp": x}
    if k in ("reduce_sum", "reduce_max"):
        return {"inp": normal("inp", (s["M"], s["N"]))}
    if k == "softmax":
        return {"inp": normal("inp", (s["M"], s["N"]), 3)}
    if k == "chain":
        return {"x": normal("x", (s["M"], s["N"])), "col": normal("col", s["N"]), "row": normal("row", (s["M"], 1))}
    if k == "layernorm":
        return {"x": normal("x", (s["M"], s["N"]), rounded=False), "w": rng.uniform(0.5, 1.5, s["N"]).astype(np.float32),
                "b": (0.1 * rng.standard_normal(s["N"])).astype(np.float32)}
    if k == "groupnorm":
        return {"X": normal("X", (s["N"], s["C"], s["HW"]), rounded=False), "W": normal("W", s["C"], rounded=False),
                "B": normal("B", s["C"], rounded=False)}
    if k == "matmul_bias_relu":
        sc = np.float32(1.0 / np.sqrt(max(s["K"], 1)))
        return {"A": normal("A", (s["M"], s["K"])), "B": normal("B", (s["K"], s["N"]), sc), "bias": normal("bias", s["N"], 0.1)}
    if k == "rmsnorm":
        return {"x": normal("x", (s["M"], s["N"]), rounded=False), "w": rng.uniform(0.5, 1.5, s["N"]).astype(np.float32)}
    if k == "layernorm_residual":
        return {"x0": normal("x0", (s["M"], s["N"]), rounded=False), "r": normal("r", (s["M"], s["N"]), rounded=False),
                "w": rng.uniform(0.5, 1.5, s["N"]).astype(np.float32), "b": (0.1 * rng.standard_normal(s["N"])).astype(np.float32)}
    if k == "masked_softmax":
        mask = rng.random(s["N"]) > 0.2
        mask[int(rng.integers(0, s["N"]))] = True  # at least one column survives
        return {"x": normal("x", (s["M"], s["N"]), 3, rounded=False), "mask": mask}
    if k == "rope":
        ang = rng.uniform(-np.pi, np.pi, (s["S"], s["D2"]))
        return {"x": normal("x", (s["S"], s["B"], s["H"], s["D"]), rounded=False), "cos": np.cos(ang).astype(np.float32),
                "sin": np.sin(ang).astype(np.float32)}
    if k == "dropout":
        return {"x": normal("x", (s["M"], s["N"]), rounded=False), "p": np.array(rng.choice((0.1, 0.25, 0.5)), np.float32),
                "seed": np.array(int(rng.integers(-2 ** 40, 2 ** 40)), np.int64)}
    if k == "image":
        i8 = lambda shape: rng.integers(-128, 128, size=shape).astype(np.int8)  # noqa: E731
        return {"a": i8((s["C"], s["H"], s["W"])), "b": i8((s["C"], s["H"], s["W"])), "sh": np.array(int(rng.integers(0, 9)), np.int32),
                "off": rng.integers(-1024, 1024, size=(s["H2"], s["W2"])).astype(np.int16)}
    raise ValueError(f"unknown sweep kind {k}")


# ---- the driver -------------------------------------------------------------------------------------------

def reference_checker() -> Tuple[Callable, Callable, type]:
    """(run_diff, infer_tolerances, TestCase) imported from the reference checkout at
    ``$INTENTIR_REF``.  Raises if it is not there: the sweep has no checker of its own."""
    root = os.environ.get("INTENTIR_REF")
    if not root or not os.path.isdir(root):
        raise RuntimeError("set INTENTIR_REF to a checkout of the reference (its verify/ package is the checker), "
                           "or pass diff_fn / tolerances_fn / case_type explicitly")
    if root not in sys.path:
        sys.path.insert(0, root)
    dr = importlib.import_module("verify.diff_runner")
    tol = importlib.import_module("verify.tolerances")
    gc = importlib.import_module("verify.gen_cases")
    return dr.run_diff, tol.infer_tolerances, gc.TestCase


def _load_shard(path: str) -> Dict[int, Dict[str, Any]]:
    """Records already in a JSONL shard, by case id (a torn last line is ignored)."""
    done: Dict[int, Dict[str, Any]] = {}
    if os.path.exists(path):
        with open(path) as f:
            for line in f:
                try:
                    rec = json.loads(line)
                    done[int(rec["case_id"])] = rec
                except Exception:
                    pass
    return done


# CPU milliseconds per million elements for input generation + interpreter + comparison, measured with the
# numpy checker on one host thread; only the ratios matter (they order and balance the work)
_COST_MS_PER_MEL = {"reduce_any": 22.0, "reduce_sum": 16.0, "reduce_max": 16.0, "softmax": 52.0, "chain": 85.0, "layernorm": 78.0,
                    "groupnorm": 46.0, "rmsnorm": 60.0, "layernorm_residual": 95.0, "masked_softmax": 60.0, "rope": 50.0,
                    "dropout": 120.0, "image": 40.0}


def estimate_cost(case: SweepCase) -> float:
    """Rough host cost of one case in milliseconds (the sweep is bound by the CPU checker)."""
    s = case.shapes
    if case.kind == "matmul_bias_relu":
        m, n, k = s["M"], s["N"], s["K"]
        return 0.3 + 16.0 * (m * k + k * n) / 1e6 + 30.0 * m * n / 1e6 + m * n * k / 3e7  # BLAS on one thread: ~60 GFLOP/s
    return 0.3 + _COST_MS_PER_MEL.get(case.kind, 60.0) * case.elements / 1e6


def partition_cases(cases: Sequence[SweepCase], world: int, how: str = "mod") -> List[List[int]]:
    """Positions of ``cases`` per rank, computed identically by every rank from the case list alone — no
    communication.  ``"mod"``: case i -> rank i % world.  ``"lpt"``: longest estimated case first onto the
    least loaded rank.  ``"deal"``: the same longest-first rule applied family by family (ties go to the
    rank with the smaller total), so that every rank holds an equal share of EACH graph family: within a
    family the estimate is proportional to the element count and reliable, while the weights between families
    (which depend on the checker and the host) no longer matter for the balance."""
    world = max(1, int(world))
    if how == "mod":
        return [list(range(r, len(cases), world)) for r in range(world)]
    parts: List[List[int]] = [[] for _ in range(world)]
    if how == "lpt":
        order = sorted(range(len(cases)), key=lambda i: (-estimate_cost(cases[i]), i))
        load = [0.0] * world
        for i in order:
            r = min(range(world), key=lambda q: (load[q], q))
            parts[r].append(i)
            load[r] += estimate_cost(cases[i])
        return parts
    if how != "deal":
        raise ValueError(f"unknown partition {how!r}")
    by_kind: Dict[str, List[int]] = {}
    for i, c in enumerate(cases):
        by_kind.setdefault(c.kind, []).append(i)
    total = [0.0] * world
    for kind in sorted(by_kind):
        mine = [0.0] * world  # this family's load per rank
        for i in sorted(by_kind[kind], key=lambda j: (-estimate_cost(cases[j]), j)):
            r = min(range(world), key=lambda q: (mine[q], total[q], q))
            parts[r].append(i)
            mine[r] += estimate_cost(cases[i])
            total[r] += estimate_cost(cases[i])
    return [sorted(p) for p in parts]


# graph families whose result has the row axis at full size: checked in blocks of about this many elements
_BLOCK_KINDS = ("softmax", "layernorm", "chain", "groupnorm", "rmsnorm", "layernorm_residual", "masked_softmax")
_BLOCK_ELEMENTS = 1 << 16
_BLOCK_MIN = 2  # cases of fewer than this many blocks are checked whole
# matmul: a block of rows of A meets all of B again, so its blocks are larger (B is streamed once per block, a tenth of
# the block's product at 128 rows) and only results of more than a million elements are cut
_MATMUL_BLOCK_ELEMENTS = 1 << 18
_MATMUL_MIN_RESULT = 1 << 20


def _row_blocks(case: SweepCase) -> List[Tuple[int, int]]:
    """Row ranges for checking a large case block by block; empty when the case is checked whole (small cases and
    reductions, whose results are small)."""
    rows = int(case.shapes.get(_ROW_AXIS.get(case.kind, ""), 0))
    if case.kind == "matmul_bias_relu":
        width = int(case.shapes.get("N", 0))
        if rows * width < _MATMUL_MIN_RESULT:
            return []
        step = max(64, _MATMUL_BLOCK_ELEMENTS // max(1, width))
    elif case.kind in _BLOCK_KINDS and case.elements >= _BLOCK_MIN * _BLOCK_ELEMENTS:
        step = max(1, _BLOCK_ELEMENTS // max(1, case.elements // max(rows, 1)))
    else:
        return []
    return [(a, min(rows, a + step)) for a in range(0, rows, step)] if step < rows else []


def _rows_of(case: SweepCase, name: str, arr, axis: str, a: int, b: int):
    """Rows a..b-1 of a tensor of the case (a view), or the tensor itself when it does not carry the row axis."""
    decl = case.intent.get("tensors", {}).get(name, {}).get("shape")
    arr = np.asarray(arr)
    if not decl or arr.ndim != len(decl):
        return arr
    return arr[tuple(slice(a, b) if d == axis else slice(None) for d in decl)]


def _check_case(case: SweepCase, runner_of: Callable, diff_fn: Callable, tolerances_fn: Callable, case_type: type,
                intent_from_json: Callable, rank: int) -> Dict[str, Any]:
    """One case through the verifier: ``runner_of(intent, case, timing)`` gives the ``run_ref_fn`` handed
    to ``diff_fn`` (it may record the device's share of its time as ``timing["device"]``).  Every failure
    (lowering, device, checker) becomes a failed record."""
    t0 = time.perf_counter()
    rec: Dict[str, Any] = {"case_id": case.case_id, "kind": case.kind, "dtype": case.dtype, "shapes": case.shapes, "rank": rank}
    try:
        intent = intent_from_json(case.intent)
        timing: Dict[str, float] = {}
        backend_fn = runner_of(intent, case, timing)

        def timed(c, _fn=backend_fn, _t=timing):
            t = time.perf_counter()
            try:
                return _fn(c)
            finally:
                _t["gpu"] = time.perf_counter() - t

        tol = tolerances_fn(intent).to_dict()
        whole = case_type(shapes=dict(case.shapes), dtypes={}, seed=case.seed)
        blocks = _row_blocks(case)
        if not blocks:
            diffs, _ = diff_fn(intent, timed, [whole], tolerances=tol)
            d = diffs[0]
            ok, summary, max_abs, max_rel = bool(d.ok), d.summary, d.max_abs_err, d.max_rel_err
        else:
            # The device runs the case whole, once; the verifier then checks it block of rows by block of rows (rows are
            # independent in these graph families), so that the interpreter's and the comparator's temporaries stay in
            # the core's cache instead of streaming 16-32 MB arrays through host memory a dozen times per case.
            io = timed(whole)
            ok, summary, max_abs, max_rel = True, "ok", 0.0, 0.0
            axis = _ROW_AXIS[case.kind]
            for a, b in blocks:
                part = {k: _rows_of(case, k, v, axis, a, b) for k, v in io.items()}
                diffs, _ = diff_fn(intent, lambda c, _p=part: _p, [case_type(shapes=dict(case.shapes, **{axis: b - a}), dtypes={}, seed=case.seed)],
                                   tolerances=tol)
                d = diffs[0]
                max_abs, max_rel = max(max_abs, d.max_abs_err), max(max_rel, d.max_rel_err)
                if not d.ok and ok:
                    ok, summary = False, f"{d.summary} (rows {a}..{b - 1})"
        rec.update(ok=ok, summary=summary, max_abs=float(max_abs) if np.isfinite(max_abs) else None,
                   max_rel=float(max_rel) if np.isfinite(max_rel) else None, t_gpu=timing.get("device", timing.get("gpu")),
                   t_runner=timing.get("gpu"), t_inputs=timing.get("inputs"))
    except Exception as e:  # lowering, GPU or checker failure: a failed record, not a dead sweep
        rec.update(ok=False, summary=f"{type(e).__name__}: {e}"[:300], max_abs=None, max_rel=None, t_gpu=None)
    rec["t_total"] = time.perf_counter() - t0
    return rec


# ---- checker processes ------------------------------------------------------------------------------------
#
# The sweep is bound by the host: generating a case's inputs, interpreting the graph with numpy and comparing
# in float64 cost 10-100 ms per case, the GPU run well under one.  With ``workers`` > 0 a rank therefore keeps
# its GPU in one process (the one that called run_sweep) and does the host work in ``workers`` child processes:
# a child generates the inputs into a shared-memory arena, asks the parent to run the plan on them (the parent
# uploads straight from the arena and downloads the results into it), then interprets and compares while the
# parent serves the other children.  The verifier is unchanged: each child calls ``diff_fn(intent, run_ref_fn,
# [case])`` with a ``run_ref_fn`` that happens to do its device work in the parent.

_NP_OUT = {"f32": np.float32, "bf16": np.float32, "f16": np.float32, "f64": np.float64, "i32": np.int32, "i64": np.int64,
           "i8": np.int8, "i16": np.int16, "u8": np.uint8, "bool": np.bool_, "i1": np.bool_}


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class _Arena:
    """A shared-memory block owned by one checker process, grown on demand."""

    def __init__(self):
        self.shm = None

    def ensure(self, nbytes: int):
        from multiprocessing import shared_memory

        if self.shm is None or self.shm.size < nbytes:
            self.close()
            self.shm = shared_memory.SharedMemory(create=True, size=max(_align(nbytes, 1 << 20), 8 << 20))
        return self.shm

    def close(self):
        if self.shm is not None:
            for step in (self.shm.close, self.shm.unlink):  # (close refuses while views are alive; the name is removed all the same)
                try:
                    step()
                except Exception:
                    pass
            self.shm = None


def _exchange(conn, shm, case: SweepCase, c, layout_in, layout_out, inputs, timing):
    """Ask the parent to run the case on the arena's arrays; returns inputs and outputs as the verifier wants them."""
    conn.send(("run", case.case_id, case.intent, dict(c.shapes), shm.name, layout_in, layout_out))
    reply = conn.recv()
    if reply[0] != "ok":
        raise RuntimeError(reply[1])
    if timing is not None:
        timing["device"] = reply[2]
    result = dict(inputs)
    for name, dts, shape, o in layout_out:
        sent = reply[1].get(name)
        result[name] = sent if sent is not None else np.ndarray(shape, np.dtype(dts), buffer=shm.buf, offset=o)
    return result


def _run_copying(conn, arena: _Arena, intent, case: SweepCase, c, inputs, outs, timing):
    """The plain form: inputs that live in private memory are copied into an arena sized for exactly this case."""
    inputs = {k: np.array(v, copy=True) for k, v in inputs.items()}  # (some may be views of the arena that is about to be replaced)
    layout_in, layout_out, off = [], [], 0
    for k, v in inputs.items():
        layout_in.append((k, v.dtype.str, tuple(v.shape), off))
        off = _align(off + max(v.nbytes, 1))
    for name, dt, shape in outs:
        layout_out.append((name, dt.str, shape, off))
        off = _align(off + max(int(np.prod(shape, dtype=np.int64)) * dt.itemsize, 1))
    shm = arena.ensure(off)
    for (k, _, shape, o), v in zip(layout_in, inputs.values()):
        np.ndarray(shape, v.dtype, buffer=shm.buf, offset=o)[...] = v
    return _exchange(conn, shm, case, c, layout_in, layout_out, inputs, timing)


def _remote_runner(conn, arena: _Arena, intent, case: SweepCase, timing: Optional[Dict[str, float]] = None):
    """``run_ref_fn`` for one case, run inside a checker process: inputs are generated here, the device
    work happens in the parent."""
    from .bindings import derive_bindings

    def run(c):
        t_start = time.perf_counter()
        bind = derive_bindings(dict(c.shapes))
        outs = []
        out_bytes = 0
        for name in intent.outputs:
            t = intent.tensors[name]
            shape = tuple(int(bind[d.value]) if d.kind == "sym" else int(d.value) for d in t.shape)
            dt = np.dtype(_NP_OUT[t.dtype])
            outs.append((name, dt, shape))
            out_bytes += _align(max(int(np.prod(shape, dtype=np.int64)) * dt.itemsize, 1))
        # Large inputs are generated straight into the arena (no copy afterwards), so the arena is sized first: every
        # declared tensor that is not an output counts as a possible input (intermediates that a graph declares only
        # make the bound generous), plus room for the small ones; an input that does not fit after all is generated in
        # private memory and copied, as small ones are.
        in_bytes = 1 << 20
        for name, t in intent.tensors.items():
            if name not in intent.outputs:
                dims = [bind.get(d.value) if d.kind == "sym" else d.value for d in t.shape]
                if any(v is None for v in dims):
                    continue  # (a symbol only the planner derives: not an input)
                numel = int(np.prod([int(v) for v in dims] or [1], dtype=np.int64))
                in_bytes += _align(np.dtype(_NP_OUT.get(t.dtype, np.float64)).itemsize * numel)
        shm = arena.ensure(in_bytes + out_bytes)
        room = shm.size - out_bytes
        layout_in, placed, off = [], {}, 0

        def dest(name, shape):
            nonlocal off
            nbytes = 4 * int(np.prod(shape, dtype=np.int64))
            if nbytes < (1 << 16) or off + _align(nbytes) > room or name in placed:
                return None
            view = np.ndarray(shape, np.float32, buffer=shm.buf, offset=off)
            placed[name] = off
            off = _align(off + nbytes)
            return view

        inputs = case_inputs(case, dest)
        if getattr(c, "inputs", None):
            inputs.update({k: np.asarray(v) for k, v in c.inputs.items()})
        inputs = {k: np.ascontiguousarray(v) if np.ndim(v) else np.asarray(v) for k, v in inputs.items()}
        for k, v in inputs.items():
            at = placed.get(k)
            if at is not None and v.dtype == np.float32 and v.ctypes.data == np.ndarray(v.shape, np.float32, buffer=shm.buf, offset=at).ctypes.data:
                layout_in.append((k, v.dtype.str, tuple(v.shape), at))  # already in place
                continue
            if off + _align(max(v.nbytes, 1)) > room:  # (never seen: the bound above is generous) grow and start over without placement
                return _run_copying(conn, arena, intent, case, c, inputs, outs, timing)
            layout_in.append((k, v.dtype.str, tuple(v.shape), off))
            np.ndarray(v.shape, v.dtype, buffer=shm.buf, offset=off)[...] = v
            off = _align(off + max(v.nbytes, 1))
        layout_out = []
        off = room
        for name, dt, shape in outs:
            layout_out.append((name, dt.str, shape, off))
            off = _align(off + max(int(np.prod(shape, dtype=np.int64)) * dt.itemsize, 1))
        inputs = {k: np.ndarray(shape, np.dtype(dts), buffer=shm.buf, offset=o) for k, dts, shape, o in layout_in}
        if timing is not None:
            timing["inputs"] = time.perf_counter() - t_start
        return _exchange(conn, shm, case, c, layout_in, layout_out, inputs, timing)

    return run


def _checker_main(conn, checker, intent_from_json, rank: int, cpus: Optional[Sequence[int]]) -> None:
    """Body of a checker process: cases in, records out, device work delegated to the parent."""
    if cpus:
        try:
            os.sched_setaffinity(0, set(cpus))
        except Exception:
            pass
    diff_fn, tolerances_fn, case_type = checker
    arena = _Arena()
    try:
        conn.send(("ready",))
        while True:
            msg = conn.recv()
            if msg[0] == "stop":
                break
            if msg[0] == "prime":  # have the arena at its working size, pages present, before the cases come
                shm = arena.ensure(int(msg[1]))
                try:  # (reserve first: touching pages the filesystem cannot back would end the process)
                    os.posix_fallocate(shm._fd, 0, shm.size)
                    np.frombuffer(shm.buf, np.uint8)[:] = 0
                    conn.send(("primed", shm.name, shm.size))
                except Exception:
                    conn.send(("not primed",))
                continue
            case = msg[1]
            rec = _check_case(case, lambda intent, cs, timing: _remote_runner(conn, arena, intent, cs, timing), diff_fn, tolerances_fn,
                              case_type, intent_from_json, rank)
            conn.send(("done", rec))
    except (EOFError, KeyboardInterrupt):
        pass
    finally:
        arena.close()


class _Served:
    """Parent-side view of the arenas of the checker processes (attached once per block)."""

    def __init__(self):
        self.blocks: Dict[str, Any] = {}
        self.owner: Dict[str, Any] = {}

    def views(self, name: str, layout, owner=None):
        from multiprocessing import shared_memory

        shm = self.blocks.get(name)
        if shm is None:
            for stale in [n for n, o in self.owner.items() if owner is not None and o is owner]:  # that process grew its arena: the old block is gone
                try:
                    self.blocks.pop(stale).close()
                except Exception:
                    pass
                del self.owner[stale]
            shm = shared_memory.SharedMemory(name=name)
            self.blocks[name] = shm
            self.owner[name] = owner
        return {k: np.ndarray(shape, np.dtype(dts), buffer=shm.buf, offset=o) for k, dts, shape, o in layout}

    def drop_owner(self, owner):
        """The process behind ``owner`` is gone without cleaning up: remove its blocks."""
        for name in [n for n, o in self.owner.items() if o is owner]:
            shm = self.blocks.pop(name)
            del self.owner[name]
            try:
                shm.close()
                shm.unlink()
            except Exception:
                pass

    def close(self):
        for shm in self.blocks.values():
            try:
                shm.close()
            except Exception:
                pass
        self.blocks.clear()
        self.owner.clear()


class _Shapes:
    """The part of a verifier ``TestCase`` a runner reads."""

    def __init__(self, shapes, seed=0):
        self.shapes, self.seed, self.inputs, self.dtypes = shapes, seed, None, {}


def _device_run_b200(intent_json, shapes, ins: Dict[str, np.ndarray], outs: Dict[str, np.ndarray]) -> Dict[str, Any]:
    """Parent side of one request on the B200 backend: lower (cached), upload from the arena, launch,
    download into the arena."""
    from .bindings import derive_bindings
    from .lowering import lower_intent_to_b200_kernel
    from .runtime import run_lowered

    lowered = lower_intent_to_b200_kernel(intent_json, shape_bindings=derive_bindings(dict(shapes)))
    return run_lowered(lowered, ins, out=outs)


def host_allocator_settings() -> None:
    """Allocator settings for processes that interpret graphs with numpy, applied to this process and (through
    the environment) to every process started after this call.

    A case allocates a dozen fresh arrays of up to 32 MiB: inputs, the interpreter's intermediates, the
    comparator's float64 copies.  (1) numpy marks such blocks MADV_HUGEPAGE, and where transparent huge pages
    are set to compact on such faults the first touch of every block stalls in the kernel (measured: 1.5 s
    against 0.05 s for a three-op graph over 4 Mi elements, a sweep's interpreter time 18 s against 3 s); with
    many processes the stalls also contend with each other.  So: no huge-page advice.  (2) glibc gives blocks
    above its mmap threshold back to the system at once and trims the heap, so every case faults its pages in
    again; with the threshold at its maximum (32 MiB), no trimming and a padded heap top the pages are reused
    (a further 30 % off a case's host time)."""
    tunables = {"MALLOC_MMAP_THRESHOLD_": 32 << 20, "MALLOC_TRIM_THRESHOLD_": 1 << 34, "MALLOC_TOP_PAD_": 256 << 20}
    os.environ.setdefault("NUMPY_MADVISE_HUGEPAGE", "0")
    for k, v in tunables.items():
        os.environ.setdefault(k, str(v))
    try:  # this process read its environment long ago
        from numpy._core.multiarray import _set_madvise_hugepage

        _set_madvise_hugepage(os.environ["NUMPY_MADVISE_HUGEPAGE"] != "0")
    except Exception:
        pass
    try:
        import ctypes

        libc = ctypes.CDLL("libc.so.6")
        for param, k in ((-3, "MALLOC_MMAP_THRESHOLD_"), (-1, "MALLOC_TRIM_THRESHOLD_"), (-2, "MALLOC_TOP_PAD_")):  # M_MMAP_THRESHOLD, M_TRIM_THRESHOLD, M_TOP_PAD
            libc.mallopt(ctypes.c_int(param), ctypes.c_int(min(int(os.environ[k]), (1 << 31) - 1)))
    except Exception:
        pass


def rank_cpu_share(cpus: Sequence[int], local_rank: int, ranks_per_host: int = 8, sysfs: str = "/sys/devices/system/cpu") -> Tuple[List[int], int]:
    """The logical CPUs of one rank out of `cpus` (the process's affinity), and how many hardware threads share a
    core there.  Every rank gets ``len(cpus) // ranks_per_host`` of them whatever the number of ranks running.

    Logical CPUs are ordered core by core first (package, core id, cpu number, read from the topology files), so
    that a share is made of whole cores: Linux numbers the second hardware thread of core k as ``k + cores``, and
    consecutive CPU numbers would give a rank alone four cores with idle sibling threads but, with all ranks
    running, two cores' worth of throughput shared with another rank's threads.  Where the topology cannot be read
    the CPU numbers decide."""

    def where(cpu: int) -> Tuple[int, int, int]:
        ids = []
        for name in ("physical_package_id", "core_id"):
            try:
                with open(os.path.join(sysfs, f"cpu{cpu}", "topology", name)) as f:
                    ids.append(int(f.read().strip()))
            except (OSError, ValueError):
                ids.append(-1)
        return (ids[0], ids[1] if ids[1] >= 0 else cpu, cpu)

    placed = sorted((where(c) for c in cpus))
    ordered = [w[2] for w in placed]
    per_core: Dict[Tuple[int, int], int] = {}
    for w in placed:
        per_core[w[:2]] = per_core.get(w[:2], 0) + 1
    smt = max(per_core.values()) if per_core else 1
    share = max(1, len(ordered) // max(1, ranks_per_host))
    mine = ordered[local_rank * share:(local_rank + 1) * share]
    return (mine or ordered), smt


class CheckerPool:
    """``workers`` checker processes of one rank and the loop that serves their device requests."""

    def __init__(self, workers: int, checker: Tuple[Callable, Callable, type], intent_from_json: Callable, rank: int = 0,
                 cpus: Optional[Sequence[int]] = None):
        import multiprocessing as mp

        ctx = mp.get_context("spawn")  # never fork a process that holds a CUDA context
        self.rank, self.procs, self.conns = rank, [], []
        host_allocator_settings()
        for _ in range(max(1, int(workers))):
            a, b = ctx.Pipe()
            p = ctx.Process(target=_checker_main, args=(b, checker, intent_from_json, rank, list(cpus) if cpus else None), daemon=True)
            p.start()
            b.close()
            self.procs.append(p)
            self.conns.append(a)
        for c in self.conns:  # imports done, ready for cases
            if not c.poll(120) or c.recv()[0] != "ready":
                raise RuntimeError("a checker process did not start")
        self.served = _Served()

    def prime(self, arena_bytes: int) -> None:
        """Every checker process brings its shared-memory arena to ``arena_bytes`` and touches it, and this process
        maps and touches it too.  A sweep then starts with its arenas in place instead of every process of every rank
        faulting tens of thousands of fresh pages in at the same moment (cases that need more still grow theirs)."""
        for c in self.conns:
            c.send(("prime", int(arena_bytes)))
        for c in self.conns:
            try:
                if not c.poll(120):
                    continue
                msg = c.recv()
                if msg[0] == "primed":
                    view = self.served.views(msg[1], [("all", "|u1", (int(msg[2]),), 0)], c)["all"]
                    int(view[::4096].sum())
            except (EOFError, OSError):
                pass  # (run() reports a process that died)

    def run(self, cases: Sequence[SweepCase], device_run: Callable, on_record: Optional[Callable] = None) -> List[Dict[str, Any]]:
        """Check ``cases`` (handed out in the given order, one in flight per process); returns the records
        in that order.  ``device_run(intent_json, shapes, ins, outs)`` runs the graph on arrays that live in
        a child's arena and returns the outputs it could not write in place (or all of them)."""
        from multiprocessing.connection import wait

        todo = list(range(len(cases)))[::-1]
        inflight: Dict[Any, int] = {}
        recs: Dict[int, Dict[str, Any]] = {}
        live = list(self.conns)

        def feed(c):
            if todo:
                i = todo.pop()
                inflight[c] = i
                c.send(("case", cases[i]))

        for c in live:
            feed(c)
        while inflight:
            for c in wait(list(inflight)):
                i = inflight[c]
                try:
                    msg = c.recv()
                except (EOFError, OSError):  # the process died: its case fails, the others carry on
                    case = cases[i]
                    recs[i] = {"case_id": case.case_id, "kind": case.kind, "dtype": case.dtype, "shapes": case.shapes, "rank": self.rank,
                               "ok": False, "summary": "checker process died", "max_abs": None, "max_rel": None, "t_gpu": None, "t_total": None}
                    if on_record:
                        on_record(recs[i])
                    del inflight[c]
                    live.remove(c)
                    self.served.drop_owner(c)
                    if not live and todo:
                        raise RuntimeError("every checker process died")
                    continue
                if msg[0] == "run":
                    _, _, intent_json, shapes, shm_name, layout_in, layout_out = msg
                    try:
                        t = time.perf_counter()
                        ins = self.served.views(shm_name, layout_in, c)
                        outs = self.served.views(shm_name, layout_out, c)
                        extra = device_run(intent_json, shapes, ins, outs) or {}
                        send = {}
                        for k, v in extra.items():
                            if k in outs and v is not outs[k]:
                                v = np.asarray(v)
                                if v.shape == outs[k].shape and v.dtype == outs[k].dtype:
                                    outs[k][...] = v
                                elif v.size == outs[k].size and v.dtype == outs[k].dtype:
                                    outs[k][...] = v.reshape(outs[k].shape)
                                else:
                                    send[k] = v  # not what the graph declares: the checker should see it as it is
                        c.send(("ok", send, time.perf_counter() - t))
                    except Exception as e:
                        c.send(("err", f"{type(e).__name__}: {e}"[:300]))
                elif msg[0] == "done":
                    recs[i] = msg[1]
                    if on_record:
                        on_record(msg[1])
                    del inflight[c]
                    feed(c)
        return [recs[i] for i in range(len(cases))]

    def close(self):
        for c in self.conns:
            try:
                c.send(("stop",))
            except Exception:
                pass
        for p in self.procs:
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()
        self.served.close()
        for c in self.conns:
            c.close()


def run_sweep(cases: Iterable[SweepCase], *, diff_fn: Callable, tolerances_fn: Callable, case_type: type,
              rank: int = 0, world: int = 1, out_dir: Optional[str] = None, make_runner: Optional[Callable] = None,
              intent_from_json: Optional[Callable] = None, workers: int = 0, partition: str = "mod",
              pool: Optional[CheckerPool] = None, cpus: Optional[Sequence[int]] = None) -> List[Dict[str, Any]]:
    """Run this rank's share of ``cases`` and return its records, those found in the rank's shard file
    from an earlier run included (``"resumed": True``).  ``partition``: see :func:`partition_cases`.
    ``make_runner(intent, input_gen)`` defaults to the B200 backend's ``make_run_ref_fn``;
    ``intent_from_json`` to this package's ``IntentFunction``.

    ``workers`` = 0 checks every case in this process, one after the other.  ``workers`` > 0 (or a
    ready ``pool``) keeps the device in this process and checks in that many child processes, the
    largest cases first; the checker functions and ``intent_from_json`` must then be importable
    (module-level) because they travel to the children by name."""
    if intent_from_json is None:
        from .ir import IntentFunction

        intent_from_json = IntentFunction.from_json_dict
    cases = list(cases)
    mine = [cases[i] for i in partition_cases(cases, world, partition)[rank]]
    shard, done = None, {}
    if out_dir:
        os.makedirs(out_dir, exist_ok=True)
        shard = os.path.join(out_dir, f"sweep.rank{rank}.jsonl")
        done = _load_shard(shard)
    fh = open(shard, "a") if shard else None

    def on_record(rec):
        if fh:
            fh.write(json.dumps(rec) + "\n")
            fh.flush()

    fresh = [c for c in mine if c.case_id not in done]
    try:
        if workers > 0 or pool is not None:
            if make_runner is None:
                device_run = _device_run_b200
            else:
                def device_run(intent_json, shapes, ins, outs, _mk=make_runner):
                    intent = intent_from_json(intent_json)
                    return {k: v for k, v in _mk(intent, lambda c: ins)(_Shapes(shapes)).items() if k in outs}
            own = pool is None
            if own:
                pool = CheckerPool(workers, (diff_fn, tolerances_fn, case_type), intent_from_json, rank, cpus)
            try:
                order = sorted(range(len(fresh)), key=lambda i: (-estimate_cost(fresh[i]), i))
                got = pool.run([fresh[i] for i in order], device_run, on_record)
                new = {fresh[i].case_id: r for i, r in zip(order, got)}
            finally:
                if own:
                    pool.close()
        else:
            if make_runner is None:
                from .backend import make_run_ref_fn as make_runner
            new = {}
            for case in fresh:
                rec = _check_case(case, lambda intent, cs, timing: make_runner(intent, lambda c, _cs=cs: case_inputs(_cs)), diff_fn,
                                  tolerances_fn, case_type, intent_from_json, rank)
                new[case.case_id] = rec
                on_record(rec)
    finally:
        if fh:
            fh.close()
    return [new[c.case_id] if c.case_id in new else dict(done[c.case_id], resumed=True) for c in mine]


def merge_records(per_rank: Sequence[Sequence[Dict[str, Any]]]) -> Dict[str, Any]:
    """Host-side gather: one summary from every rank's records."""
    rows = sorted((r for part in per_rank for r in part), key=lambda r: r["case_id"])
    by_kind: Dict[str, Dict[str, int]] = {}
    for r in rows:
        k = by_kind.setdefault(r["kind"], {"cases": 0, "ok": 0})
        k["cases"] += 1
        k["ok"] += int(bool(r["ok"]))
    return {"cases": len(rows), "ok": sum(int(bool(r["ok"])) for r in rows), "by_kind": by_kind,
            "failed": [{"case_id": r["case_id"], "kind": r["kind"], "shapes": r["shapes"], "summary": r["summary"]} for r in rows if not r["ok"]][:20]}
