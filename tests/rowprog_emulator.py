"""A numpy emulator of the fused row programs the planner emits (intent_ir_b200/csrc/row_program.h),
driven by the readable dump in the plan description.  It lets the CPU-only tests check the
planner's fusion pass -- slot and scalar allocation, liveness, reduction sinks, which results
reach global memory -- against the oracle without a GPU.  Test infrastructure only."""

from __future__ import annotations

from typing import Dict

import numpy as np

ACC, IMM, NODST, ROWSCALAR, NONE = 0x80, 0x81, 0xFF, 0x40, 0xFF

_NP = {"f32": np.float32, "bf16": np.float32, "f16": np.float16, "i32": np.int32, "i64": np.int64, "bool": np.bool_,
       "u8": np.uint8, "i8": np.int8, "i16": np.int16, "f64": np.float64}
_SIZE = {"f32": 4, "bf16": 2, "f16": 2, "i32": 4, "i64": 8, "bool": 1, "u8": 1, "i8": 1, "i16": 2, "f64": 8}


def _apply(op, a, b):
    f = np.float32
    with np.errstate(all="ignore"):
        if op == "mov": return a
        if op == "add": return a + b
        if op == "sub": return a - b
        if op == "mul": return a * b
        if op == "div": return a / b
        if op == "max": return np.maximum(a, b)
        if op == "min": return np.minimum(a, b)
        if op == "relu": return np.maximum(a, f(0))
        if op == "exp": return np.exp(a)
        if op == "rsqrt": return f(1) / np.sqrt(a)
        if op == "abs": return np.abs(a)
        if op == "floor": return np.floor(a)
        if op in ("ne", "lt", "le", "gt", "ge"):
            return {"ne": np.not_equal, "lt": np.less, "le": np.less_equal, "gt": np.greater, "ge": np.greater_equal}[op](a, b).astype(f)
        if op == "and": return ((a != 0) & (b != 0)).astype(f)
        if op == "or": return ((a != 0) | (b != 0)).astype(f)
        if op == "not": return (a == 0).astype(f)
        if op == "to_bool": return (a != 0).astype(f)
        if op == "to_int": return np.trunc(a)
        if op == "round_f16": return a.astype(np.float16).astype(f)
        if op == "rsub": return b - a
        if op == "rdiv": return b / a
        if op == "loadb": return b
    raise ValueError(f"emulator: op {op}")


def _store(values, dtype):
    if dtype == "bool":
        return values != 0
    if dtype in ("i32", "i64", "i8", "i16", "u8"):
        return np.trunc(values).astype(_NP[dtype])
    if dtype == "f16":
        return values.astype(np.float16)
    if dtype == "f64":
        return values.astype(np.float64)
    if dtype == "bf16":  # bf16 buffers are float32 arrays here, holding values rounded to bf16 (nearest even) as a store rounds them
        bits = np.ascontiguousarray(values, np.float32).view(np.uint32).astype(np.uint64)
        rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32)
        return np.where(np.isnan(values), np.float32(np.nan), rounded)
    return values.astype(np.float32)


def run_row_program(prog: dict, buffers: Dict[int, np.ndarray], buffer_table: list) -> None:
    """Execute one fused step; `buffers` maps buffer id -> flat numpy array and is updated in place."""
    rows, cols = int(prog["rows"]), int(prog["cols"])
    once_done = set()
    slots: Dict[int, np.ndarray] = {}
    for row in range(rows):
        S = np.full(32, np.nan, np.float32)
        for pi, ph in enumerate(prog["phases"]):
            for ld in ph["loads"]:
                S[ld["scalar"]] = np.float32(buffers[ld["buffer"]][ld["offset"] + row * ld["row_stride"]])
            scalar = ph["domain"] == "scalar"
            width = 1 if scalar else cols
            for k, inp in enumerate(ph["inputs"]):
                if inp["once"]:
                    if (pi, k) in once_done:
                        continue
                    once_done.add((pi, k))
                idx = inp["offset"] + row * inp["row_stride"] + np.arange(cols) * inp["col_stride"]
                slots[inp["slot"]] = idx.astype(np.float32) if inp["iota"] else buffers[inp["buffer"]][idx].astype(np.float32)
            acc = np.zeros(width, np.float32)

            def get(code, imm):
                if code == ACC: return acc
                if code == IMM: return np.full(width, imm, np.float32)
                if code >= ROWSCALAR: return np.full(width, S[code - ROWSCALAR], np.float32)
                assert not scalar, "slot operand in a scalar phase"
                return slots[code]

            for ins in ph["instr"]:
                imm = np.float32(ins["imm"])
                if ins["op"] == "where":
                    acc = np.where(get(ins["a"], imm) != 0, get(ins["b"], imm), get(ins["c"], imm)).astype(np.float32)
                else:
                    acc = np.asarray(_apply(ins["op"], get(ins["a"], imm), get(ins["b"], imm)), np.float32)
                if ins["dst"] != NODST:
                    if scalar:
                        S[ins["dst"] - ROWSCALAR] = acc[0]
                    else:
                        slots[ins["dst"]] = acc.copy()
            for out in ph["outputs"]:
                v = get(out["src"], np.float32(0))
                if out["reduce"]:
                    kind = out["reduce"] - 1
                    with np.errstate(all="ignore"):
                        r = v.sum(dtype=np.float32) if kind == 0 else v.max() if kind == 1 else np.float32((v != 0).any())
                    r = np.float32(r * np.float32(out["scale"]))
                    S[out["scalar"]] = r
                    if out["buffer"] >= 0:
                        _write(buffers, buffer_table, out["buffer"], row * out["row_stride"], np.asarray([r]), out["dtype"])
                elif scalar:
                    if out["scalar"] != NONE:
                        S[out["scalar"]] = v[0]
                    if out["buffer"] >= 0:
                        _write(buffers, buffer_table, out["buffer"], row * out["row_stride"], v[:1], out["dtype"])
                elif out["buffer"] >= 0:
                    _write(buffers, buffer_table, out["buffer"], row * out["row_stride"], v, out["dtype"])


def _write(buffers, table, buf, start, values, dtype):
    if buf not in buffers:
        t = table[buf]
        n = int(t["bytes"]) // _SIZE[t["dtype"]]
        buffers[buf] = np.zeros(n, _NP[t["dtype"]])
    buffers[buf][start:start + len(values)] = _store(values, dtype)


def run_elementwise_program(step: dict, buffers: Dict[int, np.ndarray], buffer_table: list) -> None:
    """Execute one elementwise step (intent_ir_b200/csrc/ew_program.h): every output element reads each operand at
    ``offset + sum(coordinate * stride)`` over the step's extents (an iota operand's value IS that number), runs the
    micro-ops with the result of the previous one as the accumulator, and stores slots or the accumulator.  Values
    are float32, or float64 when the step runs on the double-valued kernel."""
    prog = step["program"]
    ext = [int(e) for e in step["extents"]]
    lane = np.float64 if prog.get("wide") else np.float32
    total = int(np.prod(ext, dtype=np.int64))
    coords = np.unravel_index(np.arange(total, dtype=np.int64), ext) if total else [np.zeros(0, np.int64)] * len(ext)
    slots: Dict[int, np.ndarray] = {}
    for k, inp in enumerate(prog["inputs"]):
        idx = np.full(total, int(inp["offset"]), np.int64)
        for c, st in zip(coords, inp["strides"]):
            idx += c * int(st)
        slots[k] = idx.astype(lane) if inp["iota"] else np.asarray(buffers[inp["buffer"]])[idx].astype(lane)
    acc = np.zeros(total, lane)

    def get(code, imm):
        if code == ACC: return acc
        if code == IMM: return np.full(total, imm, lane)
        return slots[code]

    for ins in prog["instr"]:
        imm = lane(ins["imm"])
        if ins["op"] == "where":
            acc = np.where(get(ins["a"], imm) != 0, get(ins["b"], imm), get(ins["c"], imm)).astype(lane)
        elif ins["op"] == "round_bf16":
            bits = get(ins["a"], imm).astype(np.float32).view(np.uint32).astype(np.uint64)
            bits = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
            acc = bits.view(np.float32).astype(lane)
        else:
            acc = np.asarray(_apply(ins["op"], get(ins["a"], imm), get(ins["b"], imm))).astype(lane)
        if ins["dst"] != NODST:
            slots[ins["dst"]] = acc.copy()
    for out in prog["outputs"]:
        _write(buffers, buffer_table, out["buffer"], 0, get(out["src"], lane(0)), out["dtype"])


def _buffer(buffers, table, i):
    """Buffer ``i`` as a flat array, created (zeros) when nothing has written it yet."""
    if i not in buffers:
        t = table[i]
        buffers[i] = np.zeros(int(t["bytes"]) // _SIZE[t["dtype"]], _NP[t["dtype"]])
    return buffers[i]


def run_kernel_step(step: dict, buffers: Dict[int, np.ndarray], table: list) -> None:
    """The contracts of the reduce / softmax / normalisation / product / transpose launchers (include/intentir_b200.h
    and the step executor of intent_ir_b200/csrc/plan.cu), restated in numpy on the step's buffers."""
    a, d = step["args"], [int(v) for v in step["extents"]]
    f = np.float32
    src = [(_buffer(buffers, table, i) if i >= 0 else None) for i in a["in"]]

    def put(slot, values, dtype):
        if a["out"][slot] >= 0:
            _write(buffers, table, a["out"][slot], 0, np.asarray(values).reshape(-1), dtype)

    with np.errstate(all="ignore"):
        if a["kind"] == "reduce":
            outer, red, inner = d[0], d[1], d[2]
            x = src[0][:outer * red * inner].astype(f).reshape(outer, red, inner)
            k = a["reduce_kind"]
            r = x.sum(axis=1, dtype=f) * f(a["scale"]) if k == 0 else x.max(axis=1) if k == 1 else (x != 0).any(axis=1).astype(f)
            put(0, r, a["dtype2"])
        elif a["kind"] == "softmax":
            rows, cols = d[0], d[1]
            x = src[0][:rows * cols].astype(f).reshape(rows, cols)
            if a["reduce_kind"]:
                stride = int(a["aff_inner"])
                m = np.stack([src[1][r * stride:r * stride + cols] for r in range(rows)]) if rows else np.zeros((0, cols))
                x = np.where(m != 0, x, f(a["other"]))
            mx = x.max(axis=1, keepdims=True) if cols else np.zeros((rows, 1), f)
            e = np.exp(x - mx)
            sm = e.sum(axis=1, keepdims=True, dtype=f)
            put(0, e / sm, a["dtype2"])
            put(1, mx, "f32")
            put(2, sm, "f32")
        elif a["kind"] == "norm":
            rows, cols = d[0], d[1]
            x = src[0][:rows * cols].astype(f).reshape(rows, cols)
            for j, rid in enumerate(a["residual"]):
                r = _buffer(buffers, table, rid).astype(f)
                x = x + (r[:rows * cols].reshape(rows, cols) if j == 0 else r[:cols][None, :])
            mean = x.mean(axis=1, keepdims=True, dtype=f) if a["act"] else np.zeros((rows, 1), f)
            xc = x - mean
            rstd = f(1) / np.sqrt((xc * xc).mean(axis=1, keepdims=True, dtype=f) + f(a["eps"]))
            lin = np.arange(rows * cols, dtype=np.int64).reshape(rows, cols)
            idx = (lin // int(a["aff_inner"])) % int(a["aff_period"])
            t = xc * rstd
            if a["flags"] == 1:
                t = np.maximum(t, f(0))
            if src[1] is not None:
                t = t * src[1].astype(f)[idx]
            if src[2] is not None:
                t = t + src[2].astype(f)[idx]
            if a["flags"] == 2:
                t = np.maximum(t, f(0))
            put(0, t, a["dtype"])
            put(1, mean, "f32")
            put(2, rstd, "f32")
        elif a["kind"] == "gemm":
            m, n, k = d[0], d[1], d[2]
            sa, sb, sc = [int(v) for v in a["batch_stride"]]
            out = _buffer(buffers, table, a["out"][0])
            for bi in range(int(a["batch"])):
                A = src[0][bi * sa:bi * sa + m * k].astype(f).reshape(m, k)
                B = src[1][bi * sb:bi * sb + n * k].astype(f)
                B = B.reshape(n, k).T if a["transpose_b"] else B.reshape(k, n)
                c = A @ B
                if src[2] is not None:
                    c = c + src[2].astype(f)[:n][None, :]
                if a["act"] == 1:
                    c = np.maximum(c, f(0))
                out[bi * sc:bi * sc + m * n] = _store(c.reshape(-1), a["dtype2"])
        elif a["kind"] == "gather":  # out[l] = data[idx0[l], idx1[l], ...]; negative indices wrap once, positions outside read `other`
            n = d[0]
            off, inside = np.zeros(n, np.int64), np.ones(n, bool)
            for ib, dim, stride in zip(a["index"], a["dim"], a["stride"]):
                i = _buffer(buffers, table, ib)[:n].astype(np.int64)
                i = np.where(i < 0, i + int(dim), i)
                inside &= (i >= 0) & (i < int(dim))
                off += i * int(stride)
            data = src[0]
            vals = np.where(inside, data[np.where(inside, off, 0)], data.dtype.type(a["other"]))
            out = _buffer(buffers, table, a["out"][0])
            out[:n] = vals
        elif a["kind"] == "transpose":
            rows, cols = d[0], d[1]
            out = _buffer(buffers, table, a["out"][0])
            out[:rows * cols] = src[0][:rows * cols].reshape(rows, cols).T.reshape(-1)
        else:
            raise ValueError(f"emulator: step kind {a['kind']}")


def run_plan_description(desc: dict, inputs: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
    """Run a plan step by step (fused row programs, elementwise programs, and the reduce / softmax / normalisation /
    product / transpose kernels by their contracts); returns the declared outputs by name."""
    table = desc["buffers"]
    names = desc["io_spec"]["arg_names"]
    buffers: Dict[int, np.ndarray] = {}
    for i, t in enumerate(table):
        if t["arg"] >= 0 and names[t["arg"]] in inputs:
            buffers[i] = np.ascontiguousarray(inputs[names[t["arg"]]]).reshape(-1)
    for st in desc["steps"]:
        if "row_program" in st:
            run_row_program(st["row_program"], buffers, table)
        elif "program" in st:
            run_elementwise_program(st, buffers, table)
        elif "args" in st:
            run_kernel_step(st, buffers, table)
        else:
            raise ValueError(f"emulator does not cover {st['kernel']}")
    out = {}
    for name in desc["output_names"]:
        i = next(k for k, t in enumerate(table) if t["arg"] >= 0 and names[t["arg"]] == name)
        shape = desc["io_spec"]["tensors"][name]["shape"]
        out[name] = buffers[i].reshape(shape)
    return out
