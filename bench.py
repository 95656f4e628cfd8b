"""Benchmark of the IntentIR hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Default workload: BASELINE configs[1], row softmax f32 [4096,4096] (one step = one launch of
the lowered plan over one [4096,4096] batch).  Prints ONE JSON line:

  metric / value : achieved HBM GB/s = algorithmic bytes (read x once + write y once) / time,
                   whole job over all N ranks, inputs resident in HBM, CUDA-event timed, max
                   over ranks;
  e2e            : the same metric through the public host-buffer API (pinned host tensors,
                   H2D + plan + D2H inside the timed region);
  roofline       : the softmax kernel against the measured copy bandwidth of this pool;
  cpu_baseline   : the CPU oracle (numpy restatement of the reference interpreter) on a bounded
                   sample of the same workload, on this host's cores;
  ops            : the other BASELINE configurations at one GPU (layernorm, groupnorm,
                   matmul+bias+ReLU bf16, reduce_any, a broadcast add/mul chain), each with
                   its own roofline fraction.

`--impl reference` times the reference's own CPU implementation of the path — here the
oracle port of verify/interpreter.py, because the reference is Python and is not present on
the GPU box — with all host threads, on the same config, metric and unit.

`--workload sweep` runs a bounded sample of the seeded verification sweep (cases sharded
across ranks, each diffed against the CPU oracle) and reports verified cases/s.

Multi-GPU: one process per GPU under torchrun; rows / cases are sharded, no data-path
collective; only the timing reduction and the final host-side gather use torch.distributed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram bytes per launch from the ncu capture summarised in profiles/ (read + write); None = not captured
NCU_TRAFFIC = {"softmax": 89600000, "layernorm": 220300000, "groupnorm": 215200000, "matmul": 79500000, "chain": 223500000,
               "rmsnorm": 217900000, "rowprog": 223600000, "rope": 224200000, "masked_softmax": 87800000, "reduce_sum_all": 273400000,
               "column_sum": 275900000}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def graphs():
    with open(os.path.join(ROOT, "tests", "golden", "intents.json")) as f:
        return json.load(f)


# ---------------------------------------------------------------- workloads --------------------

def bf16_graph(js):
    js = json.loads(json.dumps(js))
    for name in ("A", "B", "bias", "C"):
        js["tensors"][name]["dtype"] = "bf16"
    js["ops"][0]["attrs"] = {"accum_dtype": "f32"}
    return js


def chain_graph():
    t = lambda s: {"dtype": "f32", "shape": s, "layout": "row_major"}  # noqa: E731
    return {"name": "bcast_chain", "tensors": {"x": t(["M", "N"]), "col": t(["N"]), "row": t(["M", 1]), "y": t(["M", "N"])},
            "ops": [{"op": "mul", "inputs": ["x", "col"], "output": "a"},
                    {"op": "add", "inputs": ["a", "row"], "output": "b"},
                    {"op": "mul", "inputs": ["b"], "output": "c", "attrs": {"mul_factor": 0.5}},
                    {"op": "add", "inputs": ["c", "col"], "output": "y"}], "outputs": ["y"]}


def workload(name):
    """-> (intent json, bindings, input generator(rng) -> dict of numpy arrays, algorithmic bytes, flops, label)"""
    g = graphs()
    if name == "softmax":
        m = n = 4096
        return (g["softmax_inner"]["intent"], {"M": m, "N": n},
                lambda r: {"input_ptr": 3 * r.standard_normal((m, n), dtype=np.float32)},
                2 * m * n * 4, 0, "row softmax f32 [4096,4096] (BASELINE configs[1])")
    if name == "layernorm":
        m, n = 8192, 4096
        return (g["layer_norm_persistent"]["intent"], {"M": m, "N": n},
                lambda r: {"in_ptr": r.standard_normal((m, n), dtype=np.float32),
                           "weight_ptr": r.uniform(0.5, 1.5, n).astype(np.float32),
                           "bias_ptr": (0.1 * r.standard_normal(n)).astype(np.float32)},
                2 * m * n * 4 + 2 * n * 4 + 2 * m * 4, 0, "layernorm f32 [8192,4096] + mean, rstd (configs[2])")
    if name == "groupnorm":
        nn, c, hw, grp = 32, 256, 4096, 32
        return (g["group_norm_kernel"]["intent"], {"N": nn, "C": c, "HW": hw, "num_groups": grp},
                lambda r: {"X": r.standard_normal((nn, c, hw), dtype=np.float32), "W": r.standard_normal(c, dtype=np.float32),
                           "B": r.standard_normal(c, dtype=np.float32)},
                2 * nn * c * hw * 4 + 2 * c * 4 + 2 * nn * grp * 4, 0, "groupnorm f32 [32,256,64*64], 32 groups (configs[4])")
    if name == "matmul":
        n = 4096
        from intent_ir_b200.backend import round_to_bf16
        return (bf16_graph(g["matmul_bias_relu2d"]["intent"]), {"M": n, "N": n, "K": n},
                lambda r: {"A": round_to_bf16(0.02 * r.standard_normal((n, n), dtype=np.float32)),
                           "B": round_to_bf16(0.02 * r.standard_normal((n, n), dtype=np.float32)),
                           "bias": round_to_bf16(0.1 * r.standard_normal(n, dtype=np.float32))},
                3 * n * n * 2 + 2 * n, 2 * n ** 3, "matmul+bias+ReLU bf16 4096^3, fp32 accumulate (configs[3])")
    if name == "reduce_any":
        m, n = 16, 256
        return (g["any_kernel_dim"]["intent"], {"M": m, "N": n},
                lambda r: {"inp": np.where(r.random((m, n)) < 0.05, r.standard_normal((m, n), dtype=np.float32), np.float32(0))},
                m * n * 4 + m, 0, "reduce_any f32 [16,256] (configs[0]; latency-bound)")
    if name == "reduce_any_large":
        m, n = 16384, 4096
        return (g["any_kernel_dim"]["intent"], {"M": m, "N": n},
                lambda r: {"inp": np.where(r.random((m, n)) < 0.05, r.standard_normal((m, n), dtype=np.float32), np.float32(0))},
                m * n * 4 + m, 0, "reduce_any f32 [16384,4096] (supplementary bandwidth point)")
    if name == "chain":
        m, n = 8192, 4096
        return (chain_graph(), {"M": m, "N": n},
                lambda r: {"x": r.standard_normal((m, n), dtype=np.float32), "col": r.standard_normal(n, dtype=np.float32),
                           "row": r.standard_normal((m, 1), dtype=np.float32)},
                2 * m * n * 4 + n * 4 + m * 4, 0, "broadcast mul/add chain, 4 ops, f32 [8192,4096]")
    if name == "rmsnorm":
        m, n = 8192, 4096
        return (g["rms_norm2d"]["intent"], {"M": m, "N": n},
                lambda r: {"inp": r.standard_normal((m, n), dtype=np.float32), "weight": r.uniform(0.5, 1.5, n).astype(np.float32)},
                2 * m * n * 4 + n * 4 + m * 4, 0, "rms-norm f32 [8192,4096] + rstd (pipeline/tilelang/core.py:735)")
    if name == "layernorm_residual":
        m, n = 8192, 4096
        return (g["layer_norm_residual2d"]["intent"], {"M": m, "N": n},
                lambda r: {"inp": r.standard_normal((m, n), dtype=np.float32), "residual": r.standard_normal((m, n), dtype=np.float32),
                           "weight": r.uniform(0.5, 1.5, n).astype(np.float32), "bias": (0.1 * r.standard_normal(n)).astype(np.float32)},
                3 * m * n * 4 + 2 * n * 4 + 2 * m * 4, 0, "residual add + layernorm f32 [8192,4096] + mean, rstd (pipeline/tilelang/core.py:1426)")
    if name == "masked_softmax":
        m = n = 4096
        return (g["masked_softmax2d"]["intent"], {"M": m, "N": n},
                lambda r: {"inp": 3 * r.standard_normal((m, n), dtype=np.float32), "mask": r.random(n) > 0.2},
                2 * m * n * 4 + n, 0, "masked softmax f32 [4096,4096], column mask (pipeline/tilelang/core.py:1050)")
    if name == "dag":
        m, n = 8192, 4096
        t = lambda sh: {"dtype": "f32", "shape": sh, "layout": "row_major"}  # noqa: E731
        js = {"name": "ew_dag", "tensors": {"x": t(["M", "N"]), "col": t(["N"]), "row": t(["M", 1]), "y": t(["M", "N"])},
              "ops": [{"op": "mul", "inputs": ["x", "col"], "output": "a"}, {"op": "add", "inputs": ["a", "row"], "output": "b"},
                      {"op": "sub", "inputs": ["x", "col"], "output": "c"}, {"op": "mul", "inputs": ["b", "c"], "output": "d"},
                      {"op": "max", "inputs": ["x", "row"], "output": "e"}, {"op": "add", "inputs": ["d", "e"], "output": "y"}], "outputs": ["y"]}
        return (js, {"M": m, "N": n},
                lambda r: {"x": r.standard_normal((m, n), dtype=np.float32), "col": r.standard_normal(n, dtype=np.float32),
                           "row": r.standard_normal((m, 1), dtype=np.float32)},
                2 * m * n * 4 + n * 4 + m * 4, 0, "elementwise DAG with reused values (6 ops, two register temporaries), f32 [8192,4096]")
    if name == "rowprog":
        m, n = 8192, 4096
        t = lambda sh: {"dtype": "f32", "shape": sh, "layout": "row_major"}  # noqa: E731
        js = {"name": "rms_relu", "tensors": {"x": t(["M", "N"]), "w": t(["N"]), "y": t(["M", "N"]), "rstd": t(["M"])},
              "ops": [{"op": "mul", "inputs": ["x", "x"], "output": "sq"},
                      {"op": "reduce_sum", "inputs": ["sq"], "output": "ss", "attrs": {"dims": [1], "keepdims": True, "scale": "1.0/N"}},
                      {"op": "add", "inputs": ["ss"], "output": "ve", "attrs": {"addend": 1e-5}},
                      {"op": "rsqrt", "inputs": ["ve"], "output": "r1"},
                      {"op": "reshape", "inputs": ["r1"], "output": "rstd", "attrs": {"shape": ["M"]}},
                      {"op": "mul", "inputs": ["x", "r1"], "output": "xn"},
                      {"op": "relu", "inputs": ["xn"], "output": "xr"},
                      {"op": "mul", "inputs": ["xr", "w"], "output": "y"}], "outputs": ["y", "rstd"]}
        return (js, {"M": m, "N": n},
                lambda r: {"x": r.standard_normal((m, n), dtype=np.float32), "w": r.uniform(0.5, 1.5, n).astype(np.float32)},
                2 * m * n * 4 + n * 4 + m * 4, 0, "rms-norm with a ReLU inside, f32 [8192,4096]: no dedicated kernel, one fused row program")
    if name == "rope":
        sq, b, h, d = 8192, 2, 16, 128
        t = lambda sh: {"dtype": "f32", "shape": sh, "layout": "row_major"}  # noqa: E731
        js = {"name": "rope", "tensors": {"x": t(["S", "B", "H", "D"]), "cos": t(["S", "D2"]), "sin": t(["S", "D2"]), "y": t(["S", "B", "H", "D"])},
              "ops": [{"op": "rope", "inputs": ["x", "cos", "sin"], "output": "y"}], "outputs": ["y"]}

        def gen(r):
            ang = r.uniform(-np.pi, np.pi, (sq, d // 2))
            return {"x": r.standard_normal((sq, b, h, d), dtype=np.float32), "cos": np.cos(ang).astype(np.float32), "sin": np.sin(ang).astype(np.float32)}
        return (js, {"S": sq, "B": b, "H": h, "D": d, "D2": d // 2}, gen, 2 * sq * b * h * d * 4 + 2 * sq * (d // 2) * 4, 0,
                "rope f32 [8192,2,16,128] (verify/interpreter.py:455-477), bit-exact")
    if name == "dropout":
        m, n = 8192, 4096
        t = lambda sh, dt="f32": {"dtype": dt, "shape": sh, "layout": "row_major"}  # noqa: E731
        js = {"name": "dropout", "tensors": {"x": t(["M", "N"]), "p": t([]), "seed": t([], "i64"), "y": t(["M", "N"])},
              "ops": [{"op": "dropout", "inputs": ["x", "p", "seed"], "output": "y"}], "outputs": ["y"]}
        return (js, {"M": m, "N": n},
                lambda r: {"x": r.standard_normal((m, n), dtype=np.float32), "p": np.array(0.1, np.float32), "seed": np.array(1234, np.int64)},
                2 * m * n * 4, 0, "dropout f32 [8192,4096], p = 0.1, 10 Philox rounds (verify/interpreter.py:697-742), bit-exact mask")
    if name in ("reduce_sum_all", "column_sum"):
        m, n = (8192, 8192) if name == "reduce_sum_all" else (65536, 1024)
        t = lambda sh: {"dtype": "f32", "shape": sh, "layout": "row_major"}  # noqa: E731
        whole = name == "reduce_sum_all"
        js = {"name": name, "tensors": {"x": t(["M", "N"]), "y": t([] if whole else ["N"])},
              "ops": [{"op": "reduce_sum", "inputs": ["x"], "output": "y", "attrs": {"dims": [0, 1] if whole else [0]}}], "outputs": ["y"]}
        return (js, {"M": m, "N": n}, lambda r: {"x": r.standard_normal((m, n), dtype=np.float32)}, m * n * 4 + (4 if whole else n * 4), 0,
                "sum of a whole f32 [8192,8192] tensor: one row, split over the GPU" if whole
                else "sum over the leading axis of f32 [65536,1024]: the reduced axis split over the GPU")
    raise SystemExit(f"unknown workload {name}")


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


def time_plan(lowered, sets, steps, warmup, barrier=None):
    """CUDA-event time of `steps` launches, rotating through buffer sets whose combined
    footprint exceeds L2.  Returns milliseconds."""
    import torch

    from intent_ir_b200.runtime import bind_lowered, check_plan_status

    bound = [bind_lowered(lowered, ins, outs)[0] for ins, outs in sets]  # validated once per buffer set
    for i in range(warmup):
        bound[i % len(bound)]()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        bound[i % len(bound)]()
    end.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    check_plan_status(lowered)
    return start.elapsed_time(end)


def sets_needed(bytes_per_set):
    return max(2, min(16, int(np.ceil(4 * L2_BYTES / max(bytes_per_set, 1)))))


def measure_op(name, steps, warmup, peaks):
    from intent_ir_b200.lowering import lower_intent_to_b200_kernel

    js, bind, gen, nbytes, flops, label = workload(name)
    lowered = lower_intent_to_b200_kernel(js, shape_bindings=bind)
    sets = device_sets(lowered, gen, sets_needed(nbytes), seed=11)
    ms = time_plan(lowered, sets, steps, warmup)
    per = ms / steps
    out = {"workload": label, "us_per_launch": round(per * 1e3, 3), "launches_per_step": lowered.n_launches,
           "kernels": [s["kernel"] for s in lowered.steps]}
    if nbytes < (1 << 20):  # launch-latency bound: the same plan replayed from a CUDA graph
        import torch

        from intent_ir_b200.runtime import graph_lowered

        replay, _ = graph_lowered(lowered, sets[0][0], sets[0][1])
        for _ in range(warmup):
            replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            replay()
        e1.record()
        torch.cuda.synchronize()
        out["us_per_graph_replay"] = round(e0.elapsed_time(e1) / steps * 1e3, 3)
    if flops:
        tf = flops / (per * 1e-3) / 1e12
        out.update({"tflops": round(tf, 1), "frac_of_bf16_peak": round(tf / peaks["bf16_tflops"], 4),
                    "frac_of_bf16_sustained": round(tf / peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]), 4)})
    else:
        gbs = nbytes / (per * 1e-3) / 1e9
        out.update({"gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4)})
    return out


# ---------------------------------------------------------------- CPU side ---------------------

def cpu_oracle_rate(js, bind_full, gen, row_key, rows_sample, nbytes_full, rows_full, threads, repeats=3):
    """GB/s of the CPU oracle on a row-sample of the workload, rows split over `threads`."""
    from concurrent.futures import ThreadPoolExecutor

    from intent_ir_b200.ir import IntentFunction
    from oracle import execute_intent

    intent = IntentFunction.from_json_dict(js)
    rng = np.random.default_rng(11)
    full = gen(rng)
    assert full[row_key].shape[0] == rows_full
    chunks = np.array_split(np.arange(rows_sample), threads)
    chunks = [c for c in chunks if len(c)]

    def work(idx):
        # every input whose leading extent is the row count is row-sharded with x
        ins = {k: (v[idx[0]: idx[-1] + 1] if v.ndim and v.shape[0] == rows_full else v) for k, v in full.items()}
        b = dict(bind_full)
        b["M"] = len(idx)
        with np.errstate(all="ignore"):
            return execute_intent(intent, ins, b)

    best = None
    with ThreadPoolExecutor(max_workers=len(chunks)) as pool:
        for _ in range(repeats):
            t0 = time.perf_counter()
            list(pool.map(work, chunks))
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
    nbytes = nbytes_full * rows_sample / rows_full
    return nbytes / best / 1e9, best, len(chunks)


# ---------------------------------------------------------------- sweep ------------------------

def bench_sweep(args, rank, world, local):
    """A bounded sample of the seeded verification sweep: `--sweep-cases` cases per rank (weak
    scaling), case i -> rank i % world, every case lowered, run on the GPU and diffed against
    the CPU oracle (the checker); rank 0 gathers the records on the host and reports verified
    cases per second of wall time (the sweep is bound by the CPU checker, not by the GPU)."""
    import torch

    from intent_ir_b200.sweep import generate_sweep_cases, merge_records, run_sweep
    from oracle import TestCase, infer_tolerances, run_diff

    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("cpu:gloo,cuda:nccl", device_id=torch.device("cuda", local))
    checker = dict(diff_fn=run_diff, tolerances_fn=infer_tolerances, case_type=TestCase)
    run_sweep(generate_sweep_cases(8, base_seed=10, max_elements=1 << 18), rank=0, world=1, **checker)  # warm-up, untimed
    cases = generate_sweep_cases(args.sweep_cases * world, base_seed=1000, max_elements=1 << 22, canonical_groupnorm_every=0)
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    t0 = time.perf_counter()
    records = run_sweep(cases, rank=rank, world=world, **checker)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    gathered = [records]
    if dist:
        t = torch.tensor([dt], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t[0])
        gathered = [None] * world if rank == 0 else None
        dist.gather_object(records, gathered, dst=0)
    if rank == 0:
        summary = merge_records(gathered)
        gpu_s = sum((r.get("t_gpu") or 0.0) for part in gathered for r in part)
        emit(({
            "metric": "verified_cases_per_s", "value": round(summary["ok"] / dt, 3), "unit": "cases/s", "n_gpus": world,
            "steps": len(cases), "warmup": 8, "ms_per_step": round(dt / max(len(cases), 1) * 1e3, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32/bf16", "data": "synthetic",
            "config": {"workload": f"verification sweep sample: {args.sweep_cases} seeded cases per rank (base seed 1000), "
                                   "mixed reduce/softmax/layernorm/groupnorm/matmul/chain, dims in [1,4096], f32/bf16, <= 4 Mi elements per case",
                       "checker": "CPU oracle run_diff, one thread per rank", "timing": "wall clock, max over ranks"},
            "sweep": {**summary, "gpu_busy_fraction": round(gpu_s / (dt * world), 4)},
        }))
    if dist:
        dist.destroy_process_group()


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


def main():
    reserve_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="softmax")
    ap.add_argument("--no-ops", action="store_true", help="skip the per-op table (other BASELINE configs)")
    ap.add_argument("--profile", action="store_true", help="timed launches only (for ncu captures): no clock probe, e2e, CPU arm or per-op table")
    ap.add_argument("--sweep-cases", type=int, default=96, help="cases per rank for --workload sweep")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    peaks, peak_kind = load_peaks()

    if args.workload == "sweep":
        return bench_sweep(args, rank, world, local)

    js, bind, gen, nbytes, flops, label = workload(args.workload)
    row_key = {"softmax": "input_ptr", "layernorm": "in_ptr", "chain": "x", "reduce_any": "inp", "reduce_any_large": "inp"}.get(args.workload)
    rows_full = bind.get("M", 1)

    if args.impl == "reference":
        if rank != 0:
            return
        threads = os.cpu_count() or 1
        if row_key is None:
            emit(({"impl": "reference", "unavailable": f"no row-sharded CPU arm for workload {args.workload}"}))
            return
        rows_sample = min(rows_full, 512)
        vals = []
        t_all = time.perf_counter()
        for _ in range(min(args.warmup, 3)):
            cpu_oracle_rate(js, bind, gen, row_key, rows_sample, nbytes, rows_full, threads, repeats=1)
        step_times = []
        for _ in range(args.steps):
            gbs, dt, used = cpu_oracle_rate(js, bind, gen, row_key, rows_sample, nbytes, rows_full, threads, repeats=1)
            vals.append(gbs)
            step_times.append(dt)
            if time.perf_counter() - t_all > 150:
                break
        value = float(np.median(vals))
        sample = f"{rows_sample} of {rows_full} rows per step, rows split over {used} threads, median of {len(vals)} steps"
        emit(({
            "impl": "reference", "metric": "hbm_gbs", "value": round(value, 3), "unit": "GB/s", "n_gpus": args.gpus,
            "steps": len(vals), "warmup": min(args.warmup, 3), "ms_per_step": round(float(np.median(step_times)) * 1e3, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": label, "arm": "CPU oracle port of verify/interpreter.py (numpy); the reference is Python and absent from the GPU box"},
            "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": used, "kind": "port", "sample": sample},
            "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    # NCCL announces its version on stdout at the first collective unless told otherwise; stdout is for the JSON line
    if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
        os.environ["NCCL_DEBUG"] = "WARN"
    import torch

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local)
    barrier = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        barrier = lambda: (dist.barrier(), torch.cuda.synchronize())  # noqa: E731

    from intent_ir_b200.lowering import lower_intent_to_b200_kernel
    from intent_ir_b200.runtime import run_lowered_pinned

    lowered = lower_intent_to_b200_kernel(js, shape_bindings=bind)
    sets = device_sets(lowered, gen, sets_needed(nbytes), seed=11 + rank)

    sampler = ClockSampler(local)
    sampler.start()
    ms = time_plan(lowered, sets, args.steps, args.warmup, barrier)
    # keep the clocks record meaningful for short runs: the same launches, untimed, for ~0.3 s
    t0 = time.perf_counter()
    while not args.profile and time.perf_counter() - t0 < 0.3:
        time_plan(lowered, sets, 50, 0)
    clocks = sampler.stop()
    if args.profile:
        emit(({"profile_run": True, "workload": label, "ms_per_step": ms / args.steps, "kernels": [s["kernel"] for s in lowered.steps]}))
        return

    # ---- end to end: pinned host buffers, H2D + plan + D2H per step ------------------------
    from intent_ir_b200.ops import TORCH_OF_DTYPE

    specs = lowered.io_spec["tensors"]
    host_in = {k: v.cpu().pin_memory() for k, v in sets[0][0].items()}
    host_out = {k: torch.empty([int(d) for d in specs[k]["shape"]], dtype=TORCH_OF_DTYPE[specs[k]["dtype"]]).pin_memory()
                for k in lowered.output_names}
    e2e_steps = max(3, min(args.steps, 20))
    from intent_ir_b200.runtime import HostPipeline

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

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])

    per_ms = ms / args.steps
    if flops:
        metric, unit = "tflops", "TFLOP/s"
        value = world * flops / (per_ms * 1e-3) / 1e12
        e2e_value = world * flops / (e2e_ms / e2e_steps * 1e-3) / 1e12
        per_gpu = value / world
        roof = {"bound": "tensor", "achieved": round(per_gpu, 2), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": round(per_gpu / peaks["bf16_tflops"], 4), "traffic": None}
    else:
        metric, unit = "hbm_gbs", "GB/s"
        value = world * nbytes / (per_ms * 1e-3) / 1e9
        e2e_value = world * nbytes / (e2e_ms / e2e_steps * 1e-3) / 1e9
        per_gpu = value / world
        roof = {"bound": "hbm", "achieved": round(per_gpu, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(per_gpu / peaks["hbm_gbs"], 4), "traffic": NCU_TRAFFIC.get(args.workload)}
    roof["peak_kind"] = f"of {peak_kind}"
    roof["kernel"] = lowered.steps[0]["kernel"]
    roof["algorithmic_bytes_per_launch"] = nbytes

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    line = {
        "metric": metric, "value": round(value, 2), "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(per_ms, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if flops else "f32", "data": "synthetic",
        "config": {"workload": label, "per_gpu": "one full batch per rank per step (rows sharded, no collective)",
                   "l2": f"{len(sets)} rotating buffer sets, {len(sets) * nbytes >> 20} MiB > {L2_BYTES >> 20} MiB L2"},
        "e2e": {"value": round(e2e_value, 2), "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps},
        "gpu_launches": args.steps * lowered.n_launches * world,
        "clocks": clocks,
        "roofline": roof,
    }
    if world == 1:
        if row_key is not None:
            threads = 1
            rows_sample = min(rows_full, 1024)
            gbs, dt, used = cpu_oracle_rate(js, bind, gen, row_key, rows_sample, nbytes, rows_full, threads)
            line["cpu_baseline"] = {"value": round(gbs, 3), "unit": "GB/s", "cores": used, "kind": "port",
                                    "sample": f"{rows_sample} of {rows_full} rows, best of 3, numpy {np.__version__}, host has {os.cpu_count()} cores"}
        if not args.no_ops:
            ops = {}
            for name in ("layernorm", "groupnorm", "matmul", "chain", "dag", "rmsnorm", "layernorm_residual", "masked_softmax", "rowprog", "rope", "dropout", "reduce_sum_all", "column_sum",
                         "reduce_any_large", "reduce_any"):
                if name == args.workload:
                    continue
                ops[name] = measure_op(name, max(20, min(args.steps, 100)), max(3, min(args.warmup, 10)), peaks)
            line["ops"] = ops
    emit((line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
