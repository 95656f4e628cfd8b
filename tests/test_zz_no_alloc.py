"""ib200_plan_launch_noalloc — the plan launcher for hosts that may not allocate device memory
(their memory is owned by someone else's pool, or their loop must stay clear of cudaMalloc).

The workspace that multi-kernel plans need comes from a fixed 32 MiB array inside the library
instead of from the caller.  This test drives the entry point through the C ABI (ctypes), twice
in a row on the same shared array, and requires the outputs to equal those of the ordinary
ib200_plan_launch with a caller-provided workspace; it also checks that a plan too large for the
built-in array is refused with a clear message and without launching anything.

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


def test_noalloc_launch_matches_the_caller_workspace_launch_twice():
    from intent_ir_b200 import _lib
    from intent_ir_b200.ops import TORCH_OF_DTYPE

    lib = _lib.load()
    with open(GOLDEN) as f:
        graphs = json.load(f)
    # a plan of several kernels with intermediates in scratch and a tensor-core-GEMM status word
    graph, shapes = graphs["mlp2d"]["intent"], {"M": 96, "N": 64, "K": 72, "H": 80}
    handle = _plan(lib, graph, shapes)
    try:
        d = _describe(lib, handle)
        need = lib.ib200_plan_workspace_bytes(handle)
        assert len(d["steps"]) > 1 and 0 < need <= lib.ib200_noalloc_workspace_limit()
        stream = torch.cuda.current_stream().cuda_stream
        rng = np.random.default_rng(21)
        specs, outs = d["io_spec"]["tensors"], set(d["output_names"])

        def fresh_inputs():
            return {n: torch.from_numpy(rng.standard_normal([int(x) for x in specs[n]["shape"]]).astype(np.float32)).cuda()
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
            torch.cuda.synchronize()
            return {n: t.cpu().numpy() for n, t in res.items()}

        for round_ in range(2):  # two calls in a row share the built-in array; inputs differ per round
            inputs = fresh_inputs()
            want = launch(inputs, noalloc=False)
            got = launch(inputs, noalloc=True)
            for n in outs:
                assert np.isfinite(got[n]).all(), (round_, n)
                # the same kernels on the same inputs: the tolerance the matmul tests use, 2e-2, is far
                # looser than what is observed (bit-identical results)
                np.testing.assert_allclose(got[n], want[n], rtol=2e-2, atol=2e-2, err_msg=f"round {round_}, {n}")
                assert np.array_equal(got[n], want[n]), (round_, n)
    finally:
        lib.ib200_plan_destroy(handle)


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
