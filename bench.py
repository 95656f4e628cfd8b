"""Benchmark of the IntentIR hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Default workload: BASELINE configs[1], row softmax f32 [4096,4096] (one step = one launch of
the lowered plan over one [4096,4096] batch).  Prints ONE JSON line:

  metric / value : achieved HBM GB/s = algorithmic bytes (read x once + write y once) / time,
                   whole job over all N ranks, inputs resident in HBM, CUDA-event timed (median of
                   5 repeats of max(K, 200) launches), max over ranks;
  e2e            : the same metric through the public host-buffer API (pinned host tensors,
                   H2D + plan + D2H inside the timed region); e2e_numpy: the same step through
                   run_b200_kernel with pageable numpy arrays, the call run_diff makes;
  roofline       : the softmax kernel against the measured copy bandwidth of this pool;
  cpu_baseline   : the CPU interpreter on the same workload, one host thread;
  ops            : the other BASELINE configurations at one GPU, each with its own fraction of the
                   measured peak (layernorm, groupnorm and matmul last);
  sweep          : the seeded verification sweep — a fixed list of cases sharded over the ranks,
                   each lowered, run on the GPU and diffed against the interpreter by checker
                   processes — as verified cases per second of wall time.

`--impl reference` times the reference's own CPU implementation of the path
(verify/interpreter.py from the reference's verifier packages when they are installed beside
this file, else the numpy port under oracle/) with all host threads, on the same config.

`--workload sweep` runs the sweep alone (`--sweep-total`, `--sweep-out`).

Multi-GPU: one process per GPU under torchrun; rows / cases are sharded, no data-path
collective; only the timing reduction and the final host-side gather use torch.distributed.
"""

from __future__ import annotations

import os

# Thread budget, fixed before numpy loads: every process of this benchmark runs BLAS / OpenMP on one
# thread; host parallelism is the processes and threads started below.  A rank's budget is
# cores // 8 whatever the number of ranks, so that one rank alone and eight ranks together work
# with the same share of the host.
for _k in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS", "NUMEXPR_NUM_THREADS"):
    os.environ[_k] = "1"
# Both arms interpret graphs with numpy on fresh arrays of tens of MiB; with numpy's huge-page advice the first
# touch of every such array stalls in the kernel's compaction (intent_ir_b200.sweep.host_allocator_settings has
# the measurement).  Set here, before numpy loads, so that this process and every process it starts run alike.
os.environ.setdefault("NUMPY_MADVISE_HUGEPAGE", "0")

import argparse  # noqa: E402
import json  # noqa: E402
import re  # noqa: E402
import sys  # noqa: E402
import tempfile  # noqa: E402
import threading  # noqa: E402
import time  # noqa: E402

import numpy as np  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# the ncu summary that holds each workload's DRAM counters (dram__bytes_read.sum / dram__bytes_write.sum rows)
PROFILE_OF = {"softmax": "softmax_block_f32_4096x4096.md", "layernorm": "norm_block_layernorm_f32_8192x4096.md",
              "groupnorm": "norm_pipe_groupnorm_f32_32x256x4096.md", "matmul": "gemm_tcgen05_pair_bf16_4096x4096x4096.md",
              "chain": "ew_kernel_static_chain4_f32_8192x4096.md", "dag": "ew_kernel_static_dag6_f32_8192x4096.md",
              "rmsnorm": "norm_block_rmsnorm_f32_8192x4096.md", "rmsnorm_relu": "norm_block_rmsnorm_relu_f32_8192x4096.md",
              "rowprog": "row_kernel_static_rms_abs_f32_8192x4096.md", "rope": "rope_kernel_f32_8192x2x16x128.md",
              "masked_softmax": "softmax_block_masked_f32_4096x4096.md", "reduce_sum_all": "reduce_rows_split_sum_f32_8192x8192.md",
              "column_sum": "reduce_cols_vec_sum_f32_65536x1024.md", "reduce_any_large": "reduce_rows_block_any_f32_16384x4096.md", "softmax_long": "softmax_resident_f32_4x1Mi.md",
              "layernorm_long": "norm_resident_f32_4x1Mi.md"}


def host_cores() -> list:
    try:
        return sorted(os.sched_getaffinity(0))
    except Exception:
        return list(range(os.cpu_count() or 1))


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def ncu_traffic(workload_name):
    """DRAM bytes per launch (read + write) from the committed ncu summary of this workload's kernel, or None."""
    name = PROFILE_OF.get(workload_name)
    path = os.path.join(ROOT, "profiles", name) if name else None
    if not path or not os.path.exists(path):
        return None
    unit = {"byte": 1, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    total = 0.0
    with open(path) as f:
        text = f.read()
    for counter in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
        m = re.search(r"\|\s*" + re.escape(counter) + r"\s*\|\s*([0-9.,]+)\s*\|\s*(\w+)\s*\|", text)
        if not m or m.group(2) not in unit:
            return None
        total += float(m.group(1).replace(",", "")) * unit[m.group(2)]
    return int(total)


# ---------------------------------------------------------------- workloads --------------------

def bf16_graph(js):
    js = json.loads(json.dumps(js))
    for name in ("A", "B", "bias", "C"):
        js["tensors"][name]["dtype"] = "bf16"
    js["ops"][0]["attrs"] = {"accum_dtype": "f32"}
    return js


def _t(shape, dtype="f32"):
    return {"dtype": dtype, "shape": shape, "layout": "row_major"}


def chain_graph():
    return {"name": "bcast_chain", "tensors": {"x": _t(["M", "N"]), "col": _t(["N"]), "row": _t(["M", 1]), "y": _t(["M", "N"])},
            "ops": [{"op": "mul", "inputs": ["x", "col"], "output": "a"},
                    {"op": "add", "inputs": ["a", "row"], "output": "b"},
                    {"op": "mul", "inputs": ["b"], "output": "c", "attrs": {"mul_factor": 0.5}},
                    {"op": "add", "inputs": ["c", "col"], "output": "y"}], "outputs": ["y"]}


def workload(name):
    """-> (intent json, bindings, input generator(rng) -> dict of numpy arrays, algorithmic bytes, flops, label)"""
    from intent_ir_b200.config_graphs import config_graph as g

    if name == "softmax":
        m = n = 4096
        return (g("softmax_inner"), {"M": m, "N": n},
                lambda r: {"input_ptr": 3 * r.standard_normal((m, n), dtype=np.float32)},
                2 * m * n * 4, 0, "row softmax f32 [4096,4096] (BASELINE configs[1])")
    if name == "layernorm":
        m, n = 8192, 4096
        return (g("layer_norm_persistent"), {"M": m, "N": n},
                lambda r: {"in_ptr": r.standard_normal((m, n), dtype=np.float32),
                           "weight_ptr": r.uniform(0.5, 1.5, n).astype(np.float32),
                           "bias_ptr": (0.1 * r.standard_normal(n)).astype(np.float32)},
                2 * m * n * 4 + 2 * n * 4 + 2 * m * 4, 0, "layernorm f32 [8192,4096]+mean,rstd (configs[2])")
    if name == "groupnorm":
        nn, c, hw, grp = 32, 256, 4096, 32
        return (g("group_norm_kernel"), {"N": nn, "C": c, "HW": hw, "num_groups": grp},
                lambda r: {"X": r.standard_normal((nn, c, hw), dtype=np.float32), "W": r.standard_normal(c, dtype=np.float32),
                           "B": r.standard_normal(c, dtype=np.float32)},
                2 * nn * c * hw * 4 + 2 * c * 4 + 2 * nn * grp * 4, 0, "groupnorm f32 [32,256,64*64] G=32 (configs[4])")
    if name in ("matmul", "matmul_f32", "matmul_f16"):
        n = 4096
        from intent_ir_b200.backend import round_to_bf16
        js = g("matmul_bias_relu2d")
        dt = {"matmul": "bf16", "matmul_f16": "f16", "matmul_f32": "f32"}[name]
        if dt != "f32":
            js = bf16_graph(js)
            for t in ("A", "B", "bias", "C"):
                js["tensors"][t]["dtype"] = dt
        esz = 4 if dt == "f32" else 2
        label = {"matmul": "matmul+bias+ReLU bf16 4096^3, f32 accumulate (configs[3])", "matmul_f16": "matmul+bias+ReLU f16 4096^3",
                 "matmul_f32": "matmul+bias+ReLU f32 4096^3 (tf32 tensor cores)"}[name]
        bind = {"M": n, "N": n, "K": n}
        if dt == "f32":
            bind["ALLOW_TF32"] = 1  # the reference's opt-in binding (intentir_to_cuda.py:577-578); without it f32 stays on exact FMA
        return (js, bind,
                lambda r: {"A": round_to_bf16(0.02 * r.standard_normal((n, n), dtype=np.float32)),
                           "B": round_to_bf16(0.02 * r.standard_normal((n, n), dtype=np.float32)),
                           "bias": round_to_bf16(0.1 * r.standard_normal(n, dtype=np.float32))},
                3 * n * n * esz + esz * n, 2 * n ** 3, label)
    if name == "reduce_any":
        m, n = 16, 256
        return (g("any_kernel_dim"), {"M": m, "N": n},
                lambda r: {"inp": np.where(r.random((m, n)) < 0.05, r.standard_normal((m, n), dtype=np.float32), np.float32(0))},
                m * n * 4 + m, 0, "reduce_any f32 [16,256] (configs[0]; latency-bound)")
    if name == "reduce_any_large":
        m, n = 16384, 4096
        return (g("any_kernel_dim"), {"M": m, "N": n},
                lambda r: {"inp": np.where(r.random((m, n)) < 0.05, r.standard_normal((m, n), dtype=np.float32), np.float32(0))},
                m * n * 4 + m, 0, "reduce_any f32 [16384,4096]")
    if name == "chain":
        m, n = 8192, 4096
        return (chain_graph(), {"M": m, "N": n},
                lambda r: {"x": r.standard_normal((m, n), dtype=np.float32), "col": r.standard_normal(n, dtype=np.float32),
                           "row": r.standard_normal((m, 1), dtype=np.float32)},
                2 * m * n * 4 + n * 4 + m * 4, 0, "broadcast mul/add chain, 4 ops, f32 [8192,4096]")
    if name == "rmsnorm":
        m, n = 8192, 4096
        return (g("rms_norm2d"), {"M": m, "N": n},
                lambda r: {"inp": r.standard_normal((m, n), dtype=np.float32), "weight": r.uniform(0.5, 1.5, n).astype(np.float32)},
                2 * m * n * 4 + n * 4 + m * 4, 0, "rms-norm f32 [8192,4096]+rstd")
    if name == "layernorm_residual":
        m, n = 8192, 4096
        return (g("layer_norm_residual2d"), {"M": m, "N": n},
                lambda r: {"inp": r.standard_normal((m, n), dtype=np.float32), "residual": r.standard_normal((m, n), dtype=np.float32),
                           "weight": r.uniform(0.5, 1.5, n).astype(np.float32), "bias": (0.1 * r.standard_normal(n)).astype(np.float32)},
                3 * m * n * 4 + 2 * n * 4 + 2 * m * 4, 0, "residual add + layernorm f32 [8192,4096]")
    if name == "masked_softmax":
        m = n = 4096
        return (g("masked_softmax2d"), {"M": m, "N": n},
                lambda r: {"inp": 3 * r.standard_normal((m, n), dtype=np.float32), "mask": r.random(n) > 0.2},
                2 * m * n * 4 + n, 0, "masked softmax f32 [4096,4096], column mask")
    if name == "dag":
        m, n = 8192, 4096
        js = {"name": "ew_dag", "tensors": {"x": _t(["M", "N"]), "col": _t(["N"]), "row": _t(["M", 1]), "y": _t(["M", "N"])},
              "ops": [{"op": "mul", "inputs": ["x", "col"], "output": "a"}, {"op": "add", "inputs": ["a", "row"], "output": "b"},
                      {"op": "sub", "inputs": ["x", "col"], "output": "c"}, {"op": "mul", "inputs": ["b", "c"], "output": "d"},
                      {"op": "max", "inputs": ["x", "row"], "output": "e"}, {"op": "add", "inputs": ["d", "e"], "output": "y"}], "outputs": ["y"]}
        return (js, {"M": m, "N": n},
                lambda r: {"x": r.standard_normal((m, n), dtype=np.float32), "col": r.standard_normal(n, dtype=np.float32),
                           "row": r.standard_normal((m, 1), dtype=np.float32)},
                2 * m * n * 4 + n * 4 + m * 4, 0, "elementwise DAG with reused values, 6 ops, f32 [8192,4096]")
    if name in ("rowprog", "rmsnorm_relu"):
        # rms-norm with an activation between the normalisation and the weight.  With a ReLU the norm kernel takes it
        # (an activation hook); with |x| nothing dedicated matches and the graph runs as one fused row program
        m, n = 8192, 4096
        inner = "relu" if name == "rmsnorm_relu" else "abs"
        js = {"name": "rms_" + inner, "tensors": {"x": _t(["M", "N"]), "w": _t(["N"]), "y": _t(["M", "N"]), "rstd": _t(["M"])},
              "ops": [{"op": "mul", "inputs": ["x", "x"], "output": "sq"},
                      {"op": "reduce_sum", "inputs": ["sq"], "output": "ss", "attrs": {"dims": [1], "keepdims": True, "scale": "1.0/N"}},
                      {"op": "add", "inputs": ["ss"], "output": "ve", "attrs": {"addend": 1e-5}},
                      {"op": "rsqrt", "inputs": ["ve"], "output": "r1"},
                      {"op": "reshape", "inputs": ["r1"], "output": "rstd", "attrs": {"shape": ["M"]}},
                      {"op": "mul", "inputs": ["x", "r1"], "output": "xn"},
                      {"op": inner, "inputs": ["xn"], "output": "xr"},
                      {"op": "mul", "inputs": ["xr", "w"], "output": "y"}], "outputs": ["y", "rstd"]}
        return (js, {"M": m, "N": n},
                lambda r: {"x": r.standard_normal((m, n), dtype=np.float32), "w": r.uniform(0.5, 1.5, n).astype(np.float32)},
                2 * m * n * 4 + n * 4 + m * 4, 0,
                "rms-norm with a ReLU inside, f32 [8192,4096] (norm kernel)" if inner == "relu"
                else "rms-norm with |x| inside, f32 [8192,4096] (fused row program)")
    if name == "rope":
        sq, b, h, d = 8192, 2, 16, 128
        js = {"name": "rope", "tensors": {"x": _t(["S", "B", "H", "D"]), "cos": _t(["S", "D2"]), "sin": _t(["S", "D2"]), "y": _t(["S", "B", "H", "D"])},
              "ops": [{"op": "rope", "inputs": ["x", "cos", "sin"], "output": "y"}], "outputs": ["y"]}

        def gen(r):
            ang = r.uniform(-np.pi, np.pi, (sq, d // 2))
            return {"x": r.standard_normal((sq, b, h, d), dtype=np.float32), "cos": np.cos(ang).astype(np.float32), "sin": np.sin(ang).astype(np.float32)}
        return (js, {"S": sq, "B": b, "H": h, "D": d, "D2": d // 2}, gen, 2 * sq * b * h * d * 4 + 2 * sq * (d // 2) * 4, 0,
                "rope f32 [8192,2,16,128], bit-exact")
    if name == "dropout":
        m, n = 8192, 4096
        js = {"name": "dropout", "tensors": {"x": _t(["M", "N"]), "p": _t([]), "seed": _t([], "i64"), "y": _t(["M", "N"])},
              "ops": [{"op": "dropout", "inputs": ["x", "p", "seed"], "output": "y"}], "outputs": ["y"]}
        return (js, {"M": m, "N": n},
                lambda r: {"x": r.standard_normal((m, n), dtype=np.float32), "p": np.array(0.1, np.float32), "seed": np.array(1234, np.int64)},
                2 * m * n * 4, 0, "dropout f32 [8192,4096], 10 Philox rounds, bit-exact mask")
    if name in ("reduce_sum_all", "column_sum"):
        m, n = (8192, 8192) if name == "reduce_sum_all" else (65536, 1024)
        whole = name == "reduce_sum_all"
        js = {"name": name, "tensors": {"x": _t(["M", "N"]), "y": _t([] if whole else ["N"])},
              "ops": [{"op": "reduce_sum", "inputs": ["x"], "output": "y", "attrs": {"dims": [0, 1] if whole else [0]}}], "outputs": ["y"]}
        return (js, {"M": m, "N": n}, lambda r: {"x": r.standard_normal((m, n), dtype=np.float32)}, m * n * 4 + (4 if whole else n * 4), 0,
                "sum of a whole f32 [8192,8192] tensor" if whole else "sum over the leading axis of f32 [65536,1024]")
    if name == "copy_long":
        m, n = 4, 1 << 20
        js = {"name": "copy", "tensors": {"x": _t(["M", "N"]), "y": _t(["M", "N"])},
              "ops": [{"op": "identity", "inputs": ["x"], "output": "y"}], "outputs": ["y"]}
        return (js, {"M": m, "N": n}, lambda r: {"x": r.standard_normal((m, n), dtype=np.float32)}, 2 * m * n * 4, 0,
                "copy f32 [4,1Mi]: the yardstick for the two long-row workloads")
    if name in ("softmax_long", "layernorm_long"):
        m, n = 4, 1 << 20
        if name == "softmax_long":
            return (g("softmax_inner"), {"M": m, "N": n}, lambda r: {"input_ptr": 3 * r.standard_normal((m, n), dtype=np.float32)},
                    2 * m * n * 4, 0, "row softmax f32 [4,1Mi]: few very long rows")
        return (g("layer_norm_persistent"), {"M": m, "N": n},
                lambda r: {"in_ptr": r.standard_normal((m, n), dtype=np.float32), "weight_ptr": r.uniform(0.5, 1.5, n).astype(np.float32),
                           "bias_ptr": (0.1 * r.standard_normal(n)).astype(np.float32)},
                2 * m * n * 4 + 2 * n * 4 + 2 * m * 4, 0, "layernorm f32 [4,1Mi]: few very long rows")
    raise SystemExit(f"unknown workload {name}")


# the per-op table, least important first: a reader that keeps only the end of the line keeps the BASELINE configurations
OPS_ORDER = ("reduce_any", "reduce_any_large", "column_sum", "reduce_sum_all", "dropout", "rope", "rowprog", "rmsnorm_relu", "dag", "chain", "masked_softmax",
             "layernorm_residual", "rmsnorm", "copy_long", "softmax_long", "layernorm_long", "matmul_f32", "matmul_f16", "layernorm", "groupnorm", "matmul")


# ---------------------------------------------------------------- clocks -----------------------

class ClockSampler:
    """Polls SM clock and throttle reasons through NVML (read-only) while kernels run."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------- timing -----------------------

REPEATS = 5
MIN_LAUNCHES = 200


def device_sets(lowered, gen, n_sets, seed):
    import torch

    from intent_ir_b200.ops import TORCH_OF_DTYPE

    rng = np.random.default_rng(seed)
    specs = lowered.io_spec["tensors"]
    sets = []
    for _ in range(n_sets):
        ins = {k: torch.from_numpy(np.asarray(v, order="C")).cuda().to(TORCH_OF_DTYPE[specs[k]["dtype"]]) for k, v in gen(rng).items()}
        outs = {k: torch.empty([int(d) for d in specs[k]["shape"]], dtype=TORCH_OF_DTYPE[specs[k]["dtype"]], device="cuda")
                for k in lowered.output_names}
        sets.append((ins, outs))
    return sets


def time_plan(lowered, sets, launches, warmup, barrier=None, repeats=1):
    """CUDA-event time of `launches` launches, rotating through buffer sets whose combined footprint exceeds
    L2, `repeats` times over (each repeat bracketed by a synchronise, and by the barrier when there is one).
    Returns the list of per-repeat milliseconds."""
    import torch

    from intent_ir_b200.runtime import bind_lowered, check_plan_status

    bound = [bind_lowered(lowered, ins, outs)[0] for ins, outs in sets]  # validated once per buffer set
    for i in range(warmup):
        bound[i % len(bound)]()
    times = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        if barrier:
            barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(launches):
            bound[i % len(bound)]()
        end.record()
        torch.cuda.synchronize()
        if barrier:
            barrier()
        times.append(start.elapsed_time(end))
    check_plan_status(lowered)
    return times


def sets_needed(bytes_per_set):
    return max(2, min(16, int(np.ceil(4 * L2_BYTES / max(bytes_per_set, 1)))))


def measure_op(name, steps, warmup, peaks):
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel

    js, bind, gen, nbytes, flops, label = workload(name)
    lowered = lower_intent_to_b200_kernel(js, shape_bindings=bind)
    sets = device_sets(lowered, gen, sets_needed(nbytes), seed=11)
    n = max(steps, MIN_LAUNCHES if nbytes >= (1 << 20) and not flops else 100)
    per = float(np.median(time_plan(lowered, sets, n, warmup, repeats=REPEATS))) / n
    out = {"w": label, "us": round(per * 1e3, 2), "k": "+".join(s["kernel"] for s in lowered.steps)[:60]}
    if per * 1e3 < 40.0 and not flops:  # short enough for the host's launch cost to show: the same plan replayed from a CUDA graph
        import torch

        from intent_ir_b200.runtime import graph_lowered

        replay, _ = graph_lowered(lowered, sets[0][0], sets[0][1])
        for _ in range(warmup):
            replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            replay()
        e1.record()
        torch.cuda.synchronize()
        out["us_graph_replay"] = round(e0.elapsed_time(e1) / n * 1e3, 2)  # one buffer set: L2-warm for small tensors
    if flops:
        tf = flops / (per * 1e-3) / 1e12
        out.update({"tflops": round(tf, 1), "frac": round(tf / peaks["bf16_tflops"], 3),
                    "frac_sustained": round(tf / peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]), 3)})
        # the figure above comes from ~50 ms of back-to-back products, i.e. under the board's power cap; the burst
        # peak it is divided by is a short run on an idle chip, so the same regime is measured too: a dozen launches
        # after a pause (median of five such bursts)
        bursts = []
        for _ in range(REPEATS):
            time.sleep(0.2)
            bursts.append(time_plan(lowered, sets, 12, 2)[0] / 12)
        tb = flops / (float(np.median(bursts)) * 1e-3) / 1e12
        out.update({"tflops_burst": round(tb, 1), "frac_burst": round(tb / peaks["bf16_tflops"], 3)})
    else:
        gbs = nbytes / (per * 1e-3) / 1e9
        out.update({"gbs": round(gbs, 1), "frac": round(gbs / peaks["hbm_gbs"], 3)})
        if name == "dropout":
            out["bound"] = "int-mul"  # ~20 32x32->64 multiplies per element by construction of the Philox stream: not an HBM-bound kernel
    return out


# ---------------------------------------------------------------- CPU side ---------------------

def cpu_interpreter():
    """(execute_intent, IntentFunction.from_json_dict, kind): the reference's own interpreter when its verifier
    packages are importable on this machine, else the numpy port."""
    try:
        from oracle.reference import import_reference

        ref = import_reference()
        return ref.execute_intent, ref.IntentFunction.from_json_dict, "reference"
    except ImportError:
        from intent_ir_b200.ir import IntentFunction
        from oracle import execute_intent

        return execute_intent, IntentFunction.from_json_dict, "port"


class CpuArm:
    """The CPU interpreter on a workload, its rows split over `threads` host threads (numpy releases the GIL)."""

    def __init__(self, js, bind_full, gen, row_key, threads):
        from concurrent.futures import ThreadPoolExecutor

        self.execute, from_json, self.kind = cpu_interpreter()
        self.intent = from_json(js)
        self.bind = dict(bind_full)
        self.full = gen(np.random.default_rng(11))
        self.rows = self.full[row_key].shape[0]
        self.chunks = [c for c in np.array_split(np.arange(self.rows), max(1, threads)) if len(c)]
        self.pool = ThreadPoolExecutor(max_workers=len(self.chunks))

    def _work(self, idx):
        ins = {k: (v[idx[0]: idx[-1] + 1] if v.ndim and v.shape[0] == self.rows else v) for k, v in self.full.items()}
        b = dict(self.bind)
        b["M"] = len(idx)
        with np.errstate(all="ignore"):
            return self.execute(self.intent, ins, b)

    def step(self) -> float:
        t0 = time.perf_counter()
        list(self.pool.map(self._work, self.chunks))
        return time.perf_counter() - t0


# ---------------------------------------------------------------- sweep ------------------------

SWEEP_TOTAL = 2048          # cases of the sweep block: the same list at every N (strong scaling), >= 256 per rank at N = 8
SWEEP_MAX_ELEMENTS = 1 << 22


def sweep_checker(which):
    """-> (diff_fn, tolerances_fn, case_type, intent_from_json, label)"""
    if which in ("auto", "reference"):
        try:
            from oracle.reference import import_reference

            ref = import_reference()
            return ref.run_diff, ref.infer_tolerances, ref.TestCase, ref.IntentFunction.from_json_dict, "reference verify.diff_runner.run_diff"
        except ImportError:
            if which == "reference":
                raise
    from intent_ir_b200.ir import IntentFunction
    from oracle import TestCase, infer_tolerances, run_diff

    return run_diff, infer_tolerances, TestCase, IntentFunction.from_json_dict, "oracle port of run_diff"


def run_sweep_block(rank, world, local, dist, total, out_dir=None, checker="auto", groupnorm_every=0, max_elements=SWEEP_MAX_ELEMENTS):
    """The verification sweep on `total` seeded cases (base seed 1000), dealt to the ranks family by family in order of
    estimated cost; each rank keeps its GPU in this process and checks in child processes, all pinned to the
    rank's own `threads_per_rank` logical CPUs.  Wall-clock, max over ranks.  Returns the block on
    rank 0, None elsewhere."""
    import torch

    from intent_ir_b200.sweep import CheckerPool, generate_sweep_cases, merge_records, rank_cpu_share, run_sweep

    cores = host_cores()
    budget = max(1, len(cores) // 8)
    mine, smt = rank_cpu_share(cores, local)  # whole cores: the same hardware whether the other ranks run or not
    try:
        os.sched_setaffinity(0, set(mine))
    except Exception:
        mine = []
    # The rank's processes are pinned to its `budget` cores, so the cores bound what the rank can use whatever the
    # number of processes: as many checker processes as cores, and the GPU-serving parent (busy about a seventh of
    # the time) shares them.  Without pinning the parent counts as one of the budget.
    workers = budget if mine else max(1, budget - 1)
    diff_fn, tol_fn, case_type, from_json, label = sweep_checker(checker)
    chk = dict(diff_fn=diff_fn, tolerances_fn=tol_fn, case_type=case_type, intent_from_json=from_json)
    pool = CheckerPool(workers, (diff_fn, tol_fn, case_type), from_json, rank, mine)
    try:
        # untimed: imports, first plans, and the arenas and heaps of every process at their working size (a few of the
        # largest kind of case per checker process), so that the timed cases do not start with all ranks' processes
        # faulting their memory in at once
        pool.prime(3 * 4 * max_elements)
        warm = generate_sweep_cases(4 * workers, base_seed=10, max_elements=1 << 16)
        warm += [c for c in generate_sweep_cases(64, base_seed=20, max_elements=max_elements) if 2 * c.elements >= max_elements][:2 * workers]
        run_sweep(warm, pool=pool, **chk)
        cases = generate_sweep_cases(total, base_seed=1000, max_elements=max_elements, canonical_groupnorm_every=groupnorm_every)
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        t0 = time.perf_counter()
        records = run_sweep(cases, rank=rank, world=world, out_dir=out_dir, partition="deal", pool=pool, **chk)
        torch.cuda.synchronize()
        dt_own = time.perf_counter() - t0
    finally:
        pool.close()
        try:
            os.sched_setaffinity(0, set(cores))
        except Exception:
            pass
    dt = dt_own
    gathered = [records]
    if dist:
        t = torch.tensor([dt_own], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t[0])
        gathered = [None] * world if rank == 0 else None
        dist.gather_object((records, dt_own), gathered, dst=0)
        if rank == 0:
            rank_s = [round(g[1], 2) for g in gathered]
            gathered = [g[0] for g in gathered]
    else:
        rank_s = [round(dt_own, 2)]
    if rank != 0:
        return None
    summary = merge_records(gathered)
    gpu_s = sum((r.get("t_gpu") or 0.0) for part in gathered for r in part)
    host_s = sum((r.get("t_total") or 0.0) for part in gathered for r in part)  # checker-process time, device wait included
    n_rec = max(1, sum(len(part) for part in gathered))
    cps = summary["ok"] / dt
    block = {"cases_per_s": round(cps, 2), "cases": summary["cases"], "ok": summary["ok"], "wall_s": round(dt, 2), "rank_wall_s": rank_s,
             "scaling": "strong", "partition": "longest estimated case first, family by family", "max_elements": max_elements, "base_seed": 1000,
             "threads_per_rank": budget, "pinned_to_cores": bool(mine), "checker_processes_per_rank": workers, "host_cores": len(cores), "hw_threads_per_core": smt, "blas_threads": 1,
             "checker": label, "gpu_busy_fraction": round(gpu_s / (dt * world), 4),
             # where the time goes: the checker processes' share of the wall clock, and a case's cost on the host and on the GPU
             "checker_busy_fraction": round(host_s / (dt * world * workers), 3), "host_ms_per_case": round(1e3 * host_s / n_rec, 1),
             "gpu_ms_per_case": round(1e3 * gpu_s / n_rec, 2),
             "inputs_ms_per_case": round(1e3 * sum((r.get("t_inputs") or 0.0) for part in gathered for r in part) / n_rec, 2),
             "failed": summary["failed"][:3],
             "by_kind": {k: f"{v['ok']}/{v['cases']}" for k, v in summary["by_kind"].items()}}
    # the one-rank figure of the same case list on the same host, when an N = 1 run left it behind
    note = os.path.join(tempfile.gettempdir(), f"ib200_sweep_n1_{total}_{max_elements}_{budget}.json")
    try:
        if world == 1:
            with open(note, "w") as f:
                json.dump({"cases_per_s": cps}, f)
        elif os.path.exists(note):
            with open(note) as f:
                cps1 = float(json.load(f)["cases_per_s"])
            block["cases_per_s_n1"] = round(cps1, 2)
            block["efficiency"] = round(cps / (world * cps1), 3)
    except Exception:
        pass
    return block


# ---------------------------------------------------------------- main -------------------------

_RESULT_FD = None


def reserve_stdout():
    """stdout carries exactly one JSON line.  Libraries (NCCL's version banner, for one) print there too, so
    everything else written to file descriptor 1 from here on goes to stderr and the line is written to the
    descriptor saved now."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(obj) -> None:
    data = (json.dumps(obj) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        sys.stdout.flush()
        os.write(_RESULT_FD, data)


def config_of(label, n_sets, nbytes):
    """The same description from both arms (the GPU arm and --impl reference)."""
    return {"workload": label, "per_gpu": "one full batch per rank per step (rows sharded, no collective)",
            "l2": f"GPU arm: {n_sets} rotating buffer sets, {n_sets * nbytes >> 20} MiB > {L2_BYTES >> 20} MiB L2"}


def main():
    reserve_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="softmax")
    ap.add_argument("--no-ops", action="store_true", help="skip the per-op table (other BASELINE configs)")
    ap.add_argument("--no-sweep", action="store_true", help="skip the verification-sweep block")
    ap.add_argument("--profile", action="store_true", help="timed launches only (for ncu captures): no clock probe, e2e, CPU arm, per-op table or sweep")
    ap.add_argument("--sweep-total", type=int, default=SWEEP_TOTAL, help="cases of the sweep (the same list at every N)")
    ap.add_argument("--sweep-out", default=None, help="directory for the per-rank JSONL shards of --workload sweep (restart resumes)")
    ap.add_argument("--sweep-groupnorm-every", type=int, default=0, help="every n-th groupnorm case is the canonical [32,256,4096]/32")
    ap.add_argument("--sweep-max-elements", type=int, default=SWEEP_MAX_ELEMENTS)
    ap.add_argument("--checker", default="auto", choices=["auto", "reference", "oracle"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    from intent_ir_b200.sweep import host_allocator_settings

    host_allocator_settings()  # both arms, and every process started from here on

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    peaks, peak_kind = load_peaks()

    sweep_only = args.workload == "sweep"
    js, bind, gen, nbytes, flops, label = workload("softmax" if sweep_only else args.workload)
    row_key = {"softmax": "input_ptr", "layernorm": "in_ptr", "chain": "x", "reduce_any": "inp", "reduce_any_large": "inp"}.get(args.workload)
    rows_full = bind.get("M", 1)
    n_sets = sets_needed(nbytes)

    if args.impl == "reference":
        if rank != 0:
            return
        threads = len(host_cores())
        if row_key is None:
            emit(({"impl": "reference", "unavailable": f"no row-sharded CPU arm for workload {args.workload}"}))
            return
        arm = CpuArm(js, bind, gen, row_key, threads)
        for _ in range(args.warmup):
            arm.step()
        t_all = time.perf_counter()
        times = []
        for _ in range(args.steps):
            times.append(arm.step())
            if time.perf_counter() - t_all > 240:
                break
        per = float(np.median(times))
        value = nbytes / per / 1e9
        sample = (f"all {rows_full} rows per step split over {len(arm.chunks)} threads, median of {len(times)} steps; "
                  + ("the reference's verify/interpreter.py" if arm.kind == "reference" else "numpy port of verify/interpreter.py") + f", numpy {np.__version__}")
        emit(({
            "impl": "reference", "metric": "hbm_gbs", "value": round(value, 3), "unit": "GB/s", "n_gpus": args.gpus,
            "steps": len(times), "warmup": args.warmup, "ms_per_step": round(per * 1e3, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_of(label, n_sets, nbytes),
            "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": len(arm.chunks), "kind": arm.kind, "sample": sample},
            "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    # NCCL announces its version on stdout at the first collective unless told otherwise; stdout is for the JSON line
    if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
        os.environ["NCCL_DEBUG"] = "WARN"
    import torch

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local)
    barrier, dist = None, None
    if world > 1:
        import torch.distributed as dist

        # NCCL for the barrier and the timing reduction, gloo for the host-side gather of the sweep's records
        dist.init_process_group("cpu:gloo,cuda:nccl", device_id=torch.device("cuda", local))
        barrier = lambda: (dist.barrier(), torch.cuda.synchronize())  # noqa: E731

    if sweep_only:
        block = run_sweep_block(rank, world, local, dist, args.sweep_total, out_dir=args.sweep_out, checker=args.checker,
                                groupnorm_every=args.sweep_groupnorm_every, max_elements=args.sweep_max_elements)
        if rank == 0:
            emit(({"metric": "verified_cases_per_s", "value": block["cases_per_s"], "unit": "cases/s", "n_gpus": world, "steps": block["cases"],
                   "warmup": 0, "ms_per_step": round(block["wall_s"] / max(block["cases"], 1) * 1e3, 3), "higher_is_better": True,
                   "scaling": "strong", "vs_baseline": None, "dtype": "f32/bf16", "data": "synthetic",
                   "config": {"workload": f"verification sweep: {block['cases']} seeded cases (base seed 1000), mixed reduce/softmax/layernorm/"
                                          f"groupnorm/matmul/chain, dims in [1,4096], f32/bf16, <= {args.sweep_max_elements} elements per tensor",
                              "timing": "wall clock, max over ranks"},
                   "sweep": block}))
        if dist:
            dist.destroy_process_group()
        return

    from intent_ir_b200.lowering import lower_intent_to_b200_kernel
    from intent_ir_b200.runtime import HostPipeline, run_b200_kernel, run_lowered_pinned

    lowered = lower_intent_to_b200_kernel(js, shape_bindings=bind)
    sets = device_sets(lowered, gen, n_sets, seed=11 + rank)

    launches = max(args.steps, MIN_LAUNCHES)
    repeats = 1 if args.profile else REPEATS
    if args.profile:
        launches = args.steps
    sampler = ClockSampler(local)
    sampler.start()
    times = time_plan(lowered, sets, launches, args.warmup, barrier, repeats=repeats)
    # keep the clocks record meaningful for short runs: the same launches, untimed, for ~0.3 s
    t0 = time.perf_counter()
    while not args.profile and time.perf_counter() - t0 < 0.3:
        time_plan(lowered, sets, 50, 0)
    clocks = sampler.stop()
    if args.profile:
        emit(({"profile_run": True, "workload": label, "ms_per_step": times[0] / launches, "kernels": [s["kernel"] for s in lowered.steps]}))
        return

    # ---- end to end: pinned host buffers, H2D + plan + D2H per step ------------------------
    from intent_ir_b200.ops import TORCH_OF_DTYPE

    specs = lowered.io_spec["tensors"]
    host_in = {k: v.cpu().pin_memory() for k, v in sets[0][0].items()}
    host_out = {k: torch.empty([int(d) for d in specs[k]["shape"]], dtype=TORCH_OF_DTYPE[specs[k]["dtype"]]).pin_memory()
                for k in lowered.output_names}
    e2e_steps = max(3, min(args.steps, 20))
    pipe = HostPipeline(lowered, depth=2)
    host_outs = [host_out, {k: torch.empty_like(v).pin_memory() for k, v in host_out.items()}]
    for i in range(3):
        pipe.submit(host_in, host_outs[i % 2])
    pipe.wait()
    run_lowered_pinned(lowered, host_in, host_out)  # the blocking single-call form stays exercised
    if barrier:
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(pipe._compute)  # first upload starts on the compute stream ...
    for i in range(e2e_steps):
        pipe.submit(host_in, host_outs[i % 2])  # every step uploads its inputs and downloads its result
    e1.record(pipe._download)  # ... the last download ends on the download stream
    pipe.wait()
    e2e_ms = e0.elapsed_time(e1)
    h2d = sum(t.numel() * t.element_size() for t in host_in.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out.values())

    # the reference-shaped call: run_b200_kernel with pageable numpy arrays (what run_diff's run_ref_fn does per case)
    np_in = {k: v.numpy().copy() for k, v in host_in.items()} if not flops else None
    np_ms = None
    if np_in is not None:
        call = dict(kernel_name=lowered.kernel_name, cuda_src="", io_spec=lowered.io_spec, launch=lowered.launch, bindings=lowered.bindings,
                    inputs_np=np_in, output_names=lowered.output_names)
        run_b200_kernel(**call)
        if barrier:
            barrier()
        t0 = time.perf_counter()
        for _ in range(3):
            run_b200_kernel(**call)
        np_ms = (time.perf_counter() - t0) / 3 * 1e3

    ms = float(np.median(times))
    if world > 1:
        t = torch.tensor([ms, e2e_ms, np_ms or 0.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, np_ms = float(t[0]), float(t[1]), (float(t[2]) or None)

    per_ms = ms / launches
    if flops:
        metric, unit = "tflops", "TFLOP/s"
        value = world * flops / (per_ms * 1e-3) / 1e12
        e2e_value = world * flops / (e2e_ms / e2e_steps * 1e-3) / 1e12
        per_gpu = value / world
        roof = {"bound": "tensor", "achieved": round(per_gpu, 2), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": round(per_gpu / peaks["bf16_tflops"], 4), "traffic": ncu_traffic(args.workload)}
    else:
        metric, unit = "hbm_gbs", "GB/s"
        value = world * nbytes / (per_ms * 1e-3) / 1e9
        e2e_value = world * nbytes / (e2e_ms / e2e_steps * 1e-3) / 1e9
        per_gpu = value / world
        roof = {"bound": "hbm", "achieved": round(per_gpu, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(per_gpu / peaks["hbm_gbs"], 4), "traffic": ncu_traffic(args.workload)}
    roof["peak_kind"] = f"of {peak_kind}"
    roof["kernel"] = lowered.steps[0]["kernel"]
    roof["algorithmic_bytes_per_launch"] = nbytes

    line = {
        "metric": metric, "value": round(value, 2), "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(per_ms, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if flops else "f32", "data": "synthetic",
        "config": config_of(label, n_sets, nbytes),
        "timing": {"launches_per_repeat": launches, "repeats": repeats, "stat": "median of repeats, max over ranks",
                   "repeat_us_per_launch": [round(t / launches * 1e3, 2) for t in times]},
        "e2e": {"value": round(e2e_value, 2), "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                "api": "HostPipeline.submit/wait, pinned host tensors"},
        "gpu_launches": launches * repeats * lowered.n_launches * world,
        "clocks": clocks,
        "roofline": roof,
    }
    if np_ms:
        line["e2e_numpy"] = {"value": round(world * nbytes / (np_ms * 1e-3) / 1e9, 2), "unit": unit, "ms_per_step": round(np_ms, 2),
                             "api": "run_b200_kernel, pageable numpy arrays in and out, synchronous"}
    if rank == 0 and world == 1:
        if row_key is not None:
            arm = CpuArm(js, bind, gen, row_key, 1)
            arm.step()
            best = min(arm.step() for _ in range(3))
            line["cpu_baseline"] = {"value": round(nbytes / best / 1e9, 3), "unit": "GB/s", "cores": 1, "kind": arm.kind,
                                    "sample": f"all {rows_full} rows, best of 3, numpy {np.__version__}, host has {len(host_cores())} cores"}
        if not args.no_ops:
            ops = {}
            for name in OPS_ORDER:
                if name == args.workload:
                    continue
                try:
                    ops[name] = measure_op(name, max(20, min(args.steps, 100)), max(3, min(args.warmup, 10)), peaks)
                except Exception as e:  # one workload failing to lower must not lose the line
                    ops[name] = {"error": f"{type(e).__name__}: {e}"[:120]}
            line["ops"] = ops
    if not args.no_sweep:
        block = run_sweep_block(rank, world, local, dist, args.sweep_total, checker=args.checker)
        if rank == 0:
            line["sweep"] = block
    if rank == 0:
        emit((line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
