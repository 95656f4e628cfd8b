"""The sweep driver without a GPU: deterministic case generation, row splitting, and the
world_size-2 path (gloo ranks on CPU) with a numpy stand-in for the GPU runner — the same
fake the reference's own tests use for run_ref_fn (tests/test_diff_runner.py:58-64)."""

import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

from intent_ir_b200.ir import IntentFunction
from intent_ir_b200.sweep import KINDS, case_inputs, generate_sweep_cases, merge_records, run_sweep, split_rows
from oracle import TestCase, execute_intent, infer_tolerances, run_diff
from oracle.diff import derive_bindings

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def numpy_runner(intent, input_gen):
    """Stands in for the GPU: outputs come from the interpreter itself."""
    def run(case):
        ins = input_gen(case)
        with np.errstate(all="ignore"):
            outs = execute_intent(intent, ins, derive_bindings(case.shapes))
        return {**ins, **outs}
    return run


CHECKER = dict(diff_fn=run_diff, tolerances_fn=infer_tolerances, case_type=TestCase)


def test_cases_are_deterministic_and_in_range():
    a = generate_sweep_cases(200, base_seed=1000, max_elements=1 << 20)
    b = generate_sweep_cases(200, base_seed=1000, max_elements=1 << 20)
    assert [(c.kind, c.dtype, c.shapes, c.seed) for c in a] == [(c.kind, c.dtype, c.shapes, c.seed) for c in b]
    assert {c.kind for c in a} == set(KINDS) and {c.dtype for c in a} == {"f32", "bf16"}
    for c in a:
        assert c.elements <= 1 << 20 or c.kind == "matmul_bias_relu"
        assert all(1 <= v <= 4096 for k, v in c.shapes.items())
        IntentFunction.from_json_dict(c.intent)  # every template is a valid graph
    # case i depends on base_seed + i only
    assert generate_sweep_cases(5, base_seed=1003, max_elements=1 << 20)[0].shapes == a[3].shapes


def test_split_rows_preserves_total_rows():
    c = generate_sweep_cases(50, base_seed=7, max_elements=1 << 16)
    big = max((x for x in c if x.kind == "softmax"), key=lambda x: x.shapes["M"])
    subs = split_rows(big, 4)
    assert sum(s.shapes["M"] for s in subs) == big.shapes["M"] and len({s.case_id for s in subs}) == len(subs)
    assert split_rows(big, 1) == [big]


def test_single_rank_sweep_with_resume(tmp_path):
    cases = generate_sweep_cases(24, base_seed=1000, max_elements=1 << 12)
    recs = run_sweep(cases, out_dir=str(tmp_path), make_runner=numpy_runner, **CHECKER)
    assert len(recs) == 24 and all(r["ok"] for r in recs), [r["summary"] for r in recs if not r["ok"]]
    again = run_sweep(cases, out_dir=str(tmp_path), make_runner=numpy_runner, **CHECKER)
    # every id was already in the shard file: nothing runs again, and the restart still reports every case
    assert [r["case_id"] for r in again] == [r["case_id"] for r in recs] and all(r["resumed"] and r["ok"] for r in again)
    assert sum(1 for _ in open(tmp_path / "sweep.rank0.jsonl")) == 24
    s = merge_records([recs])
    assert s["cases"] == s["ok"] == 24 and not s["failed"]


def test_failures_are_isolated():
    cases = generate_sweep_cases(6, base_seed=1000, max_elements=1 << 10)

    def flaky(intent, input_gen):
        inner = numpy_runner(intent, input_gen)

        def run(case):
            if case.seed % 2:
                raise RuntimeError("worker lost its device")
            io = inner(case)
            return io

        return run

    recs = run_sweep(cases, make_runner=flaky, **CHECKER)
    assert len(recs) == 6
    assert [r["ok"] for r in recs] == [c.seed % 2 == 0 for c in cases]
    assert all("ref runner error" in r["summary"] for r in recs if not r["ok"])


_WORKER = r"""
import json, os, sys
sys.path.insert(0, {root!r})
import torch.distributed as dist
from tests.test_sweep_cpu import CHECKER, numpy_runner
from intent_ir_b200.sweep import generate_sweep_cases, merge_records, run_sweep
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
cases = generate_sweep_cases(20, base_seed=1000, max_elements=1 << 10)
recs = run_sweep(cases, rank=rank, world=world, out_dir={out!r}, make_runner=numpy_runner, **CHECKER)
gathered = [None] * world if rank == 0 else None
dist.gather_object(recs, gathered, dst=0)
if rank == 0:
    s = merge_records(gathered)
    s["per_rank"] = [len(g) for g in gathered]
    json.dump(s, open(os.path.join({out!r}, "summary.json"), "w"))
dist.destroy_process_group()
"""


def test_two_rank_sweep_over_gloo(tmp_path):
    pytest.importorskip("torch")
    script = tmp_path / "worker.py"
    script.write_text(_WORKER.format(root=ROOT, out=str(tmp_path)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29631", str(script)], env=env, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    s = json.load(open(tmp_path / "summary.json"))
    assert s["cases"] == s["ok"] == 20 and s["per_rank"] == [10, 10]
    shards = sorted(p.name for p in tmp_path.iterdir() if p.name.startswith("sweep.rank"))
    assert shards == ["sweep.rank0.jsonl", "sweep.rank1.jsonl"]


def test_extra_graph_families_are_valid_and_plannable(tmp_path):
    """The graphs either side of the headline path (rms-norm, residual layernorm, masked softmax, rope, dropout,
    the int8 image chain): valid IntentIR, executable by the oracle, accepted by the planner."""
    from intent_ir_b200.lowering import plan_json
    from intent_ir_b200.sweep import ALL_KINDS, EXTRA_KINDS

    cases = generate_sweep_cases(120, base_seed=77, max_elements=1 << 12, kinds=ALL_KINDS)
    assert {c.kind for c in cases} == set(ALL_KINDS)
    extra = [c for c in cases if c.kind in EXTRA_KINDS]
    recs = run_sweep(extra, out_dir=str(tmp_path), make_runner=numpy_runner, **CHECKER)
    assert len(recs) == len(extra) and all(r["ok"] for r in recs), [(r["kind"], r["summary"]) for r in recs if not r["ok"]]
    expected_last = {"rmsnorm": "rmsnorm", "layernorm_residual": "layernorm", "rope": "rope", "dropout": "dropout", "image": "warp"}
    for c in extra:
        kernels = [s["kernel"] for s in plan_json(c.intent, c.shapes)["steps"]]
        if c.kind in expected_last:
            assert kernels[-1].endswith(expected_last[c.kind]), (c.kind, c.shapes, kernels)
        else:
            assert kernels[-1] in ("softmax", "softmax+mask") or kernels[-1].startswith("rowfused"), (c.kind, kernels)


# ---- checker processes (the pipelined form) ---------------------------------------------------------------

def _exiting_from_json(js):
    """An ``intent_from_json`` that takes its whole process down for one graph family: a host-side
    stand-in for a checker process that dies in the middle of a sweep."""
    if js.get("name") == "sweep_reduce_max":
        os._exit(7)
    return IntentFunction.from_json_dict(js)


def test_pool_sweep_matches_the_serial_sweep(tmp_path):
    cases = generate_sweep_cases(40, base_seed=1000, max_elements=1 << 14)
    serial = run_sweep(cases, make_runner=numpy_runner, **CHECKER)
    pooled = run_sweep(cases, make_runner=numpy_runner, workers=2, out_dir=str(tmp_path), **CHECKER)
    assert [r["case_id"] for r in pooled] == [r["case_id"] for r in serial]  # records come back in case order
    assert all(r["ok"] for r in pooled), [(r["kind"], r["summary"]) for r in pooled if not r["ok"]]
    for a, b in zip(serial, pooled):  # same verdicts; the errors may differ in the last bits (BLAS blocking differs between processes)
        assert a["ok"] == b["ok"] and abs((a["max_abs"] or 0.0) - (b["max_abs"] or 0.0)) < 1e-4, (a, b)
    assert sum(1 for _ in open(tmp_path / "sweep.rank0.jsonl")) == 40


def test_pool_reports_a_wrong_device_result():
    cases = [c for c in generate_sweep_cases(40, base_seed=1000, max_elements=1 << 12) if c.kind in ("softmax", "reduce_sum")][:6]

    def off_by_a_bit(intent, input_gen):
        inner = numpy_runner(intent, input_gen)

        def run(case):
            io = inner(case)
            for k in intent.outputs:
                io[k] = io[k] + np.float32(0.25)
            return io

        return run

    recs = run_sweep(cases, make_runner=off_by_a_bit, workers=2, **CHECKER)
    assert len(recs) == len(cases) and not any(r["ok"] for r in recs)


def test_a_dead_checker_process_fails_its_case_only():
    cases = generate_sweep_cases(60, base_seed=1000, max_elements=1 << 10)
    victims = [c for c in cases if c.kind == "reduce_max"][:1]
    others = [c for c in cases if c.kind != "reduce_max"][:12]
    recs = run_sweep(others[:6] + victims + others[6:], make_runner=numpy_runner, workers=2, intent_from_json=_exiting_from_json, **CHECKER)
    assert len(recs) == 13
    bad = [r for r in recs if not r["ok"]]
    assert [r["case_id"] for r in bad] == [victims[0].case_id] and bad[0]["summary"] == "checker process died"


def test_lpt_partition_is_deterministic_and_balanced():
    from intent_ir_b200.sweep import estimate_cost, partition_cases

    cases = generate_sweep_cases(512, base_seed=1000, max_elements=1 << 22)
    parts = partition_cases(cases, 8, "lpt")
    assert sorted(i for p in parts for i in p) == list(range(512)) and parts == partition_cases(cases, 8, "lpt")
    loads = [sum(estimate_cost(cases[i]) for i in p) for p in parts]
    assert max(loads) / min(loads) < 1.02
    assert partition_cases(cases, 4, "mod")[1][:3] == [1, 5, 9]
    # the deal: every rank gets an equal share of every family's load
    deal = partition_cases(cases, 8, "deal")
    assert sorted(i for p in deal for i in p) == list(range(512)) and deal == partition_cases(cases, 8, "deal")
    for kind in {c.kind for c in cases}:  # every family's load is balanced by itself
        per_rank = [sum(estimate_cost(cases[i]) for i in p if cases[i].kind == kind) for p in deal]
        assert max(per_rank) / min(per_rank) < 1.25, (kind, per_rank)
    loads = [sum(estimate_cost(cases[i]) for i in p) for p in deal]
    assert max(loads) / min(loads) < 1.05


def test_host_allocator_settings_reach_this_process_and_its_children():
    """No huge-page advice for numpy's large blocks and glibc's thresholds, set for the calling process and
    inherited through the environment by the checker processes started afterwards."""
    import subprocess
    import sys

    from intent_ir_b200.sweep import host_allocator_settings

    host_allocator_settings()
    assert os.environ["NUMPY_MADVISE_HUGEPAGE"] == "0" and int(os.environ["MALLOC_MMAP_THRESHOLD_"]) == 32 << 20
    from numpy._core.multiarray import _set_madvise_hugepage

    assert _set_madvise_hugepage(False) is False  # (returns the previous setting: already off in this process)
    child = subprocess.run([sys.executable, "-c", "import numpy._core.multiarray as m; print(m._set_madvise_hugepage(False))"],
                           capture_output=True, text=True, check=True)
    assert child.stdout.strip() == "False"


def test_large_cases_are_checked_block_by_block():
    """A large case runs whole on the device and is verified in blocks of rows (products with more than a million
    results included: a block of rows of A against all of B); a wrong value in one block fails the case and the
    record names the rows."""
    from intent_ir_b200.sweep import _row_blocks

    pool = generate_sweep_cases(400, base_seed=1000, max_elements=1 << 21)
    big = [c for c in pool if c.kind in ("layernorm", "softmax", "chain", "groupnorm") and c.elements >= 1 << 19][:4]
    big += [c for c in pool if c.kind == "matmul_bias_relu" and c.shapes["M"] * c.shapes["N"] >= 1 << 20][:1]
    assert len(big) == 5 and all(len(_row_blocks(c)) > 1 for c in big)
    assert all(b > a and (b - a >= 64 or c.kind != "matmul_bias_relu") for c in big for a, b in _row_blocks(c)[:-1])
    assert [blk[0] for blk in _row_blocks(big[-1])][0] == 0 and _row_blocks(big[-1])[-1][1] == big[-1].shapes["M"]
    assert not _row_blocks([c for c in generate_sweep_cases(64, base_seed=1000, max_elements=1 << 12)][0])
    recs = run_sweep(big, make_runner=numpy_runner, **CHECKER)
    assert all(r["ok"] for r in recs), [(r["kind"], r["summary"]) for r in recs if not r["ok"]]

    def one_bad_row(intent, input_gen):
        inner = numpy_runner(intent, input_gen)

        def run(case):
            io = inner(case)
            k = intent.outputs[0]
            out = np.array(io[k], copy=True)
            out[out.shape[0] - 1] += np.float32(0.5)  # the last row (the last batch entry for groupnorm)
            io[k] = out
            return io

        return run

    recs = run_sweep(big, make_runner=one_bad_row, **CHECKER)
    assert not any(r["ok"] for r in recs) and all("rows" in r["summary"] for r in recs), [r["summary"] for r in recs]


def test_a_ranks_cpu_share_is_made_of_whole_cores(tmp_path):
    """Sixteen logical CPUs on eight two-thread cores, numbered the way Linux does (cpu k and cpu k + 8 share core
    k): each of eight ranks gets both threads of one core, the same ones whatever else runs; without topology
    files the CPU numbers decide; a restricted affinity is shared out among eight all the same."""
    from intent_ir_b200.sweep import rank_cpu_share

    for cpu in range(16):
        d = tmp_path / f"cpu{cpu}" / "topology"
        d.mkdir(parents=True)
        (d / "physical_package_id").write_text("0\n")
        (d / "core_id").write_text(f"{cpu % 8}\n")
    shares = [rank_cpu_share(range(16), r, sysfs=str(tmp_path)) for r in range(8)]
    assert [s[0] for s in shares] == [[k, k + 8] for k in range(8)]
    assert {s[1] for s in shares} == {2}
    assert sorted(c for s in shares for c in s[0]) == list(range(16))
    plain = [rank_cpu_share(range(16), r, sysfs=str(tmp_path / "absent")) for r in range(8)]
    assert [s[0] for s in plain] == [[2 * k, 2 * k + 1] for k in range(8)] and plain[0][1] == 1
    assert rank_cpu_share([3, 5, 7], 2, sysfs=str(tmp_path)) == ([7], 1)
    assert rank_cpu_share([3], 5, sysfs=str(tmp_path))[0] == [3]


def test_primed_arenas_are_in_place_before_the_cases():
    """`prime` brings every checker's arena to the asked size (mapped by the serving process too); the cases that
    follow run in it, a case that needs more still grows its own."""
    from intent_ir_b200.sweep import CheckerPool, _Shapes

    def DEVICE_STAND_IN(intent_json, shapes, ins, outs):
        intent = IntentFunction.from_json_dict(intent_json)
        return {k: v for k, v in numpy_runner(intent, lambda c: ins)(_Shapes(shapes)).items() if k in outs}

    pool = CheckerPool(2, (run_diff, infer_tolerances, TestCase), IntentFunction.from_json_dict)
    try:
        pool.prime(3 << 20)
        primed = dict(pool.served.blocks)
        assert len(primed) == 2 and all(b.size >= 3 << 20 for b in primed.values())
        cases = generate_sweep_cases(12, base_seed=1000, max_elements=1 << 16)
        recs = pool.run(cases, DEVICE_STAND_IN)
        assert all(r["ok"] for r in recs), [r["summary"] for r in recs if not r["ok"]]
        assert set(pool.served.blocks) == set(primed)  # nothing grew: the cases ran in the primed arenas
        big = [c for c in generate_sweep_cases(40, base_seed=1000, max_elements=1 << 21) if c.elements >= 1 << 20][:2]
        assert all(r["ok"] for r in pool.run(big, DEVICE_STAND_IN))
    finally:
        pool.close()
