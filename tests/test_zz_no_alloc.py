"""ib200_plan_launch_noalloc — the plan launcher for hosts that may not allocate device memory
(their memory is owned by someone else's pool, or their loop must stay clear of cudaMalloc).

The workspace that multi-kernel plans need comes from a fixed 32 MiB array inside the library
instead of from the caller.  This test drives the entry point through the C ABI (ctypes), twice
in a row on the same shared array, on an f32 graph (the FMA GEMM) and on a bf16 graph (the
tensor-core GEMM, whose status word lives in the shared array), and requires the outputs to equal
those of the ordinary ib200_plan_launch with a caller-provided workspace and to agree with the CPU
oracle at the verifier's tolerance; it shows that a status word left behind in the array is
readable through ib200_plan_check_status_noalloc and cleared by the next launch; it records what
the first call does to free device memory; and it checks that a plan too large for the built-in
array is refused with a clear message and without launching anything.

Collected last on purpose (file name), so that a run stopping at the first failure has already
run every other test.  It does not depend on them: it passes in a fresh process as well."""

import ctypes as C
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "intents.json")


def _plan(lib, graph, shapes):
    from intent_ir_b200.bindings import derive_bindings, normalise_bindings

    handle = C.c_void_p()
    rc = lib.ib200_plan_create(json.dumps(graph).encode(), json.dumps(derive_bindings(normalise_bindings(shapes))).encode(), C.byref(handle))
    assert rc == 0, lib.ib200_last_error()
    return handle


def _describe(lib, handle):
    buf = C.create_string_buffer(1 << 18)
    assert lib.ib200_plan_describe(handle, buf, len(buf)) == 0
    return json.loads(buf.value.decode())


def _mlp_graph(graphs, dtype):
    graph = json.loads(json.dumps(graphs["mlp2d"]["intent"]))
    if dtype != "f32":  # every tensor 16-bit: both GEMMs take the tensor-core kernel
        for t in graph["tensors"].values():
            if t["dtype"] == "f32":
                t["dtype"] = dtype
    return graph


def _oracle_outputs(graph, shapes, inputs):
    from intent_ir_b200.bindings import derive_bindings, normalise_bindings
    from intent_ir_b200.ir import IntentFunction
    from oracle import execute_intent, infer_tolerances

    intent = IntentFunction.from_json_dict(graph)
    with np.errstate(all="ignore"):
        want = execute_intent(intent, {k: v.float().cpu().numpy() for k, v in inputs.items()}, derive_bindings(normalise_bindings(shapes)))
    return want, infer_tolerances(intent).to_dict()


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_noalloc_launch_matches_the_caller_workspace_launch_twice(dtype):
    from intent_ir_b200 import _lib
    from intent_ir_b200.ops import TORCH_OF_DTYPE
    from oracle.diff import compare_outputs

    lib = _lib.load()
    with open(GOLDEN) as f:
        graphs = json.load(f)
    # a plan of several kernels with intermediates in scratch and a GEMM status word; the 16-bit graph's
    # extents are multiples of 8, so its GEMMs are the tensor-core kernel with its bounded waits
    graph, shapes = _mlp_graph(graphs, dtype), {"M": 96, "N": 64, "K": 72, "H": 80}
    handle = _plan(lib, graph, shapes)
    try:
        d = _describe(lib, handle)
        need = lib.ib200_plan_workspace_bytes(handle)
        assert len(d["steps"]) > 1 and 0 < need <= lib.ib200_noalloc_workspace_limit()
        assert d["status_offset"] >= 0
        if dtype == "bf16":
            assert any("gemm" in s["kernel"] and "fma" not in s["kernel"] for s in d["steps"]), d["steps"]
        stream = torch.cuda.current_stream().cuda_stream
        rng = np.random.default_rng(21)
        specs, outs = d["io_spec"]["tensors"], set(d["output_names"])

        def fresh_inputs():
            return {n: torch.from_numpy(rng.standard_normal([int(x) for x in specs[n]["shape"]]).astype(np.float32)).cuda().to(TORCH_OF_DTYPE[specs[n]["dtype"]])
                    for n in d["io_spec"]["arg_names"] if n not in outs}

        def launch(inputs, noalloc):
            res = {n: torch.full([int(x) for x in specs[n]["shape"]], float("nan"), dtype=TORCH_OF_DTYPE[specs[n]["dtype"]], device="cuda")
                   for n in outs}
            tensors = [inputs[n] if n in inputs else res[n] for n in d["io_spec"]["arg_names"]]
            args = (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
            if noalloc:
                rc = lib.ib200_plan_launch_noalloc(handle, args, len(tensors), stream)
            else:
                ws = torch.zeros(need + 256, dtype=torch.uint8, device="cuda")
                rc = lib.ib200_plan_launch(handle, args, len(tensors), (ws.data_ptr() + 255) & ~255, need, stream)
            assert rc == 0, lib.ib200_last_error()
            if noalloc:  # the status word in the built-in array says no bounded wait ran out
                assert lib.ib200_plan_check_status_noalloc(handle, stream) == 0, lib.ib200_last_error()
            torch.cuda.synchronize()
            return {n: t.float().cpu().numpy() for n, t in res.items()}

        for round_ in range(2):  # two calls in a row share the built-in array; inputs differ per round
            inputs = fresh_inputs()
            want = launch(inputs, noalloc=False)
            got = launch(inputs, noalloc=True)
            oracle, tol = _oracle_outputs(graph, shapes, inputs)
            for n in outs:
                assert np.isfinite(got[n]).all(), (round_, n)
                # the same kernels on the same inputs: the tolerance the matmul tests use, 2e-2, is far
                # looser than what is observed (bit-identical results)
                np.testing.assert_allclose(got[n], want[n], rtol=2e-2, atol=2e-2, err_msg=f"round {round_}, {n}")
                assert np.array_equal(got[n], want[n]), (round_, n)
                # and against the CPU oracle, at the tolerance the verifier infers for this graph
                verdict = compare_outputs({n: oracle[n]}, {n: got[n]}, [n], tol)
                assert verdict.ok, (round_, n, verdict.summary, verdict.max_abs_err)
    finally:
        lib.ib200_plan_destroy(handle)


def test_noalloc_status_word_is_readable_and_cleared_by_the_next_launch():
    """A bounded wait that ran out leaves a code in the plan's status word.  Under the no-allocation entry the
    word lives in the built-in array, which the caller cannot address: ib200_plan_check_status_noalloc reads it.
    The failure is injected from the host (a plan whose first argument IS its status word's neighbourhood cannot
    be built, so a tiny elementwise plan is pointed at the array through the ordinary launcher)."""
    from intent_ir_b200 import _lib

    lib = _lib.load()
    with open(GOLDEN) as f:
        graphs = json.load(f)
    graph, shapes = _mlp_graph(graphs, "bf16"), {"M": 96, "N": 64, "K": 72, "H": 80}
    handle = _plan(lib, graph, shapes)
    try:
        d = _describe(lib, handle)
        stream = torch.cuda.current_stream().cuda_stream
        specs, outs = d["io_spec"]["tensors"], set(d["output_names"])
        tensors = [torch.zeros([int(x) for x in specs[n]["shape"]], dtype=torch.bfloat16, device="cuda") for n in d["io_spec"]["arg_names"]]
        args = (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
        assert lib.ib200_plan_launch_noalloc(handle, args, len(tensors), stream) == 0
        assert lib.ib200_plan_check_status_noalloc(handle, stream) == 0
        # host injection: write code 3 ("MMA issuer waiting for a TMA stage") where a kernel would have written it
        assert lib.ib200_noalloc_debug_poke_status(handle, 3, stream) == 0
        assert lib.ib200_plan_check_status_noalloc(handle, stream) == _lib.ERR_DEVICE_WAIT
        assert b"TMA stage" in lib.ib200_last_error()
        # the next launch clears the word before its kernels run
        assert lib.ib200_plan_launch_noalloc(handle, args, len(tensors), stream) == 0
        assert lib.ib200_plan_check_status_noalloc(handle, stream) == 0
    finally:
        lib.ib200_plan_destroy(handle)


_MEMORY_PROBE = r"""
import ctypes as C, json, sys
sys.path.insert(0, {root!r})
import torch
torch.zeros(1, device="cuda"); torch.cuda.synchronize()
free = [torch.cuda.mem_get_info()[0]]                      # context up, library not loaded yet
from intent_ir_b200 import _lib
from intent_ir_b200.bindings import derive_bindings, normalise_bindings
lib = _lib.load(); torch.cuda.synchronize()
free.append(torch.cuda.mem_get_info()[0])                  # after loading the library
graph = json.load(open({golden!r}))["mlp2d"]["intent"]
h = C.c_void_p()
assert lib.ib200_plan_create(json.dumps(graph).encode(), json.dumps(derive_bindings(normalise_bindings({{"M": 96, "N": 64, "K": 72, "H": 80}}))).encode(), C.byref(h)) == 0
buf = C.create_string_buffer(1 << 18); assert lib.ib200_plan_describe(h, buf, len(buf)) == 0
d = json.loads(buf.value.decode()); specs = d["io_spec"]["tensors"]
ts = [torch.zeros([int(x) for x in specs[n]["shape"]], device="cuda") for n in d["io_spec"]["arg_names"]]
args = (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
torch.cuda.synchronize(); free.append(torch.cuda.mem_get_info()[0])   # the caller's own tensors allocated
for _ in range(3):
    assert lib.ib200_plan_launch_noalloc(h, args, len(ts), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize(); free.append(torch.cuda.mem_get_info()[0])
print(json.dumps(free))
"""


def test_noalloc_first_call_and_device_memory():
    """What the entry point costs in device memory, measured in a fresh process (the header states the outcome):
    free memory after context creation, after loading the library, after the caller's own allocations, and after
    each of three calls.  The library allocates nothing; whatever the first call costs is the CUDA runtime
    materialising the built-in array (and the kernels' code) the first time they are used."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", _MEMORY_PROBE.format(root=root, golden=GOLDEN)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    free = json.loads(r.stdout.strip().splitlines()[-1])
    steps = ["load library", "caller's tensors", "call 1", "call 2", "call 3"]
    drops = {k: free[i] - free[i + 1] for i, k in enumerate(steps)}
    print("free device memory consumed (bytes):", drops)
    assert drops["call 2"] == 0 and drops["call 3"] == 0  # nothing is allocated per call
    assert 0 <= drops["call 1"] <= 96 << 20  # at most the 32 MiB array and the kernels' code, once


def test_noalloc_refuses_plans_beyond_the_built_in_workspace():
    from intent_ir_b200 import _lib

    lib = _lib.load()
    with open(GOLDEN) as f:
        graphs = json.load(f)
    handle = _plan(lib, graphs["mlp2d"]["intent"], {"M": 8192, "N": 64, "K": 64, "H": 4096})  # 128 MiB of intermediates
    try:
        assert lib.ib200_plan_workspace_bytes(handle) > lib.ib200_noalloc_workspace_limit() == 32 << 20
        args = (C.c_void_p * 6)()
        rc = lib.ib200_plan_launch_noalloc(handle, args, 6, None)
        assert rc == _lib.ERR_BUFFER
        msg = lib.ib200_last_error().decode()
        assert "built-in workspace" in msg and "ib200_plan_launch" in msg
    finally:
        lib.ib200_plan_destroy(handle)
