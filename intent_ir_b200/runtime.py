"""Running a lowered plan.

``run_b200_kernel`` mirrors the reference runner
``run_cuda_kernel(*, kernel_name, cuda_src, io_spec, launch, bindings, inputs_np, output_names,
extra_cuda_cflags=None) -> Dict[str, np.ndarray]`` (backends/cuda/runtime.py:22-45, body
frontends/cuda/runtime.py:926-1031): numpy arrays in, host->device copies, one launch of the
lowered kernel on torch's current stream, synchronise, device->host copies, and the returned
dict holds the inputs AND the outputs.  Scalar (rank-0) inputs missing from ``inputs_np`` are
materialised from ``bindings`` as the reference does (:984-992).

``launch_lowered`` is the device-resident variant used for timing: torch CUDA tensors in and
out, no copies, no synchronisation.

There is no fallback: without a CUDA device, or without the compiled library, these raise.
"""

from __future__ import annotations

import ctypes as C
from typing import Any, Dict, Iterable, Mapping, Optional

import numpy as np
import torch

from . import _lib
from .errors import B200LoweringError, B200RuntimeError
from .lowering import B200LoweredKernel, lookup_plan
from .ops import TORCH_OF_DTYPE

__all__ = ["run_b200_kernel", "run_lowered", "run_lowered_pinned", "HostPipeline", "launch_lowered", "bind_lowered", "graph_lowered", "check_plan_status"]

_WORKSPACES: Dict[Any, torch.Tensor] = {}


def _require_cuda() -> None:
    if not torch.cuda.is_available():
        raise B200RuntimeError("torch.cuda is not available; the B200 backend has no CPU path")


def _shape_of(spec: Mapping[str, Any], bindings: Mapping[str, Any]):
    return tuple(int(bindings[str(d)]) if isinstance(d, str) else int(d) for d in spec.get("shape", []))


def _workspace(lowered: B200LoweredKernel, device) -> Optional[torch.Tensor]:
    if lowered.workspace_bytes == 0:
        return None
    key = (lowered.io_spec["plan_id"], str(device))
    ws = _WORKSPACES.get(key)
    if ws is not None and ws.numel() < lowered.workspace_bytes + 256:
        ws = None  # never hand a plan less scratch than it asked for
    if ws is None:
        # zero-filled once: the tensor-core GEMM's status word lives in it and is only ever
        # written when a bounded wait expires
        ws = torch.zeros(lowered.workspace_bytes + 256, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
        # oldest first out: at most 256 plans and 8 GiB of scratch stay cached (bound launchers
        # keep their own reference, so eviction never frees memory that is still in use)
        while len(_WORKSPACES) > 1 and (len(_WORKSPACES) > 256 or sum(t.numel() for t in _WORKSPACES.values()) > (8 << 30)):
            _WORKSPACES.pop(next(iter(_WORKSPACES)))
    return ws


def _aligned_ptr(ws: Optional[torch.Tensor]) -> Optional[int]:
    if ws is None:
        return None
    return (ws.data_ptr() + 255) & ~255


def launch_lowered(lowered: B200LoweredKernel, tensors: Mapping[str, torch.Tensor],
                   outputs: Optional[Mapping[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    """Enqueue the plan on the current stream.  ``tensors`` maps input names to contiguous
    CUDA tensors of the declared dtype and shape; output tensors are allocated unless given.
    Returns the outputs.  Does not synchronise."""
    _require_cuda()
    specs = lowered.io_spec["tensors"]
    out_set = set(lowered.output_names)
    args, outs = [], {}
    device = None
    for name in lowered.io_spec["arg_names"]:
        spec = specs[name]
        dtype = TORCH_OF_DTYPE[spec["dtype"]]
        shape = tuple(int(d) for d in spec["shape"])
        if name in out_set:
            t = outputs.get(name) if outputs else None
            if t is None:
                if device is None:
                    device = torch.device("cuda", torch.cuda.current_device())
                t = torch.empty(shape, dtype=dtype, device=device)
            outs[name] = t
        else:
            if name not in tensors:
                raise B200RuntimeError(f"missing input {name} for B200 plan; have keys={sorted(tensors)}")
            t = tensors[name]
            device = t.device
        if not t.is_cuda:
            raise B200RuntimeError(f"{name} must be a CUDA tensor")
        if not t.is_contiguous():
            raise B200RuntimeError(f"{name} must be contiguous")
        if t.dtype != dtype:
            raise B200RuntimeError(f"{name} must have dtype {dtype}, got {t.dtype}")
        if tuple(t.shape) != shape:
            raise B200RuntimeError(f"{name} must have shape {shape}, got {tuple(t.shape)}")
        args.append(t)
    arr = (C.c_void_p * len(args))(*[t.data_ptr() or None for t in args])
    ws = _workspace(lowered, device)
    rc = _lib.load().ib200_plan_launch(lowered.plan.ptr, arr, len(args), _aligned_ptr(ws), lowered.workspace_bytes,
                                       torch.cuda.current_stream().cuda_stream)
    if rc != _lib.OK:
        raise B200RuntimeError(f"B200 plan launch failed: {_lib.last_error()} (status {rc})")
    return outs


def bind_lowered(lowered: B200LoweredKernel, tensors: Mapping[str, torch.Tensor],
                 outputs: Optional[Mapping[str, torch.Tensor]] = None):
    """Validate once, launch many times: returns ``(launch, outputs)`` where ``launch()``
    enqueues the plan on the current stream with the tensors bound here (one C call, no
    per-launch checks or allocations).  For latency-bound plans such as a [16,256]
    reduce_any, where argument checking would cost more than the kernel.  The bound tensors
    must stay alive and keep their storage while ``launch`` is in use."""
    outs = launch_lowered(lowered, tensors, outputs)  # full validation, allocates missing outputs
    out_set = set(lowered.output_names)
    order = [outs[n] if n in out_set else tensors[n] for n in lowered.io_spec["arg_names"]]
    arr = (C.c_void_p * len(order))(*[t.data_ptr() or None for t in order])
    ws = _workspace(lowered, order[0].device if order else None)
    ws_ptr, ws_bytes, plan_ptr, n = _aligned_ptr(ws), lowered.workspace_bytes, lowered.plan.ptr, len(order)
    fn = _lib.load().ib200_plan_launch
    keep = (order, ws, lowered)

    def launch(_keep=keep):
        rc = fn(plan_ptr, arr, n, ws_ptr, ws_bytes, torch.cuda.current_stream().cuda_stream)
        if rc != _lib.OK:
            raise B200RuntimeError(f"B200 plan launch failed: {_lib.last_error()} (status {rc})")

    return launch, outs


def graph_lowered(lowered: B200LoweredKernel, tensors: Mapping[str, torch.Tensor],
                  outputs: Optional[Mapping[str, torch.Tensor]] = None):
    """Capture the plan's launches into a CUDA graph: returns ``(replay, outputs)``.  For plans
    whose kernels are shorter than the cost of launching them (the reference's harness offers
    the same replay mode, scripts/experiments/triton_gpu_vs_intentir_cuda.py:106-145).  The
    bound tensors are baked into the graph; write new inputs into them before ``replay()``."""
    launch, outs = bind_lowered(lowered, tensors, outputs)
    launch()  # first use outside capture: module load, function attributes, workspace zero-fill
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launch()

    def replay(_keep=(launch, outs, tensors)):
        graph.replay()

    return replay, outs


def check_plan_status(lowered: B200LoweredKernel) -> None:
    """Synchronise the current stream and raise if a bounded device-side wait expired during the plan
    (``ib200_plan_check_status``); the status word is cleared so that the workspace can be used again.
    Raises as well when the plan's scratch has left the cache since it ran: its status can then no longer
    be read, and saying nothing would hide a failure."""
    if lowered.status_offset < 0:
        return
    found = False
    for key, ws in list(_WORKSPACES.items()):
        if key[0] != lowered.io_spec["plan_id"]:
            continue
        found = True
        with torch.cuda.device(ws.device):
            rc = _lib.load().ib200_plan_check_status(lowered.plan.ptr, _aligned_ptr(ws), torch.cuda.current_stream().cuda_stream)
        if rc != _lib.OK:
            msg = _lib.last_error()
            base = _aligned_ptr(ws) - ws.data_ptr() + lowered.status_offset
            ws[base: base + 4].zero_()
            raise B200RuntimeError(f"B200 kernel gave up on a bounded device-side wait: {msg} (status {rc})")
    if not found:
        raise B200RuntimeError("the status of this plan can no longer be read: its scratch buffer was released "
                               "(more than 256 other plans ran since); check a plan before running that many others")


def _to_device(name: str, arr: np.ndarray, dtype: torch.dtype, device) -> torch.Tensor:
    a = np.asarray(arr, order="C")  # (ascontiguousarray would turn a 0-d array into shape (1,))
    if a.dtype == np.float64 and dtype != torch.float64:
        a = a.astype(np.float32)
    t = torch.from_numpy(a).to(device=device)
    if t.dtype != dtype:
        t = t.to(dtype=dtype)
    return t.contiguous()


def run_lowered(lowered: B200LoweredKernel, inputs_np: Mapping[str, np.ndarray], device: str = "cuda",
                out: Optional[Mapping[str, np.ndarray]] = None) -> Dict[str, np.ndarray]:
    """Host arrays in, host arrays out (inputs and outputs in one dict), synchronous.  A result whose name
    is in ``out`` with the declared shape (16-bit floats widened to float32) is copied from the device
    straight into that array, which is then the one returned."""
    _require_cuda()
    specs = lowered.io_spec["tensors"]
    out_set = set(lowered.output_names)
    dev_in: Dict[str, torch.Tensor] = {}
    try:
        for name in lowered.io_spec["arg_names"]:
            if name in out_set:
                continue
            spec = specs[name]
            dtype = TORCH_OF_DTYPE[spec["dtype"]]
            shape = tuple(int(d) for d in spec["shape"])
            if name in inputs_np:
                arr = np.asarray(inputs_np[name])
                if tuple(arr.shape) != shape:
                    if arr.size == int(np.prod(shape, dtype=np.int64)) and arr.size <= 1:
                        arr = arr.reshape(shape)
                    else:
                        raise B200RuntimeError(f"input {name} has shape {tuple(arr.shape)}, the plan was lowered for {shape}")
                dev_in[name] = _to_device(name, arr, dtype, device)
            elif shape == () and name in lowered.bindings:
                val = lowered.bindings[name]
                dev_in[name] = torch.tensor(float(val) if dtype.is_floating_point else int(val), device=device, dtype=dtype)
            else:
                raise B200RuntimeError(f"missing input {name} for B200 plan; have keys={sorted(inputs_np.keys())}")
        outs = launch_lowered(lowered, dev_in)
        torch.cuda.synchronize()
    except RuntimeError as e:
        if isinstance(e, (B200RuntimeError, B200LoweringError)):
            raise
        if "out of memory" in str(e).lower():
            raise B200RuntimeError(f"CUDA OOM during input/output allocation: {e}") from e
        raise B200RuntimeError(f"B200 plan launch failed: {type(e).__name__}: {e}") from e
    check_plan_status(lowered)
    result: Dict[str, np.ndarray] = {k: np.asarray(v) for k, v in inputs_np.items()}
    for name, t in outs.items():
        if t.dtype in (torch.bfloat16, torch.float16):
            t = t.float()  # numpy has no bfloat16; values are exactly representable in float32
        dst = out.get(name) if out else None
        if dst is not None and dst.flags.c_contiguous and dst.flags.writeable and tuple(dst.shape) == tuple(t.shape) \
                and torch.from_numpy(dst).dtype == t.dtype:
            torch.from_numpy(dst).copy_(t)
            result[name] = dst
        else:
            result[name] = t.detach().cpu().numpy()
    return result


def run_lowered_pinned(lowered: B200LoweredKernel, host_inputs: Mapping[str, torch.Tensor],
                       host_outputs: Mapping[str, torch.Tensor], device: str = "cuda") -> Dict[str, torch.Tensor]:
    """Host buffers in, host buffers out, without numpy conversions: ``host_inputs`` are
    (ideally pinned) CPU tensors of the declared dtypes, ``host_outputs`` are CPU tensors that
    receive the results.  One call = host->device copies, the plan, device->host copies and a
    stream synchronise; this is the end-to-end path the benchmark times."""
    _require_cuda()
    out_set = set(lowered.output_names)
    dev_in = {n: host_inputs[n].to(device, non_blocking=True) for n in lowered.io_spec["arg_names"] if n not in out_set}
    outs = launch_lowered(lowered, dev_in)
    for name, t in outs.items():
        host_outputs[name].copy_(t, non_blocking=True)
    torch.cuda.current_stream().synchronize()
    check_plan_status(lowered)
    return dict(host_outputs)


class HostPipeline:
    """Host buffers in, host buffers out, with the copies of consecutive calls overlapped.

    ``submit(host_inputs, host_outputs)`` enqueues one run of the plan: host->device copies and
    the kernels on one stream, the device->host copies on a second stream that waits for the
    kernels.  With ``depth`` device buffer sets in rotation, the upload of call i+1 travels
    while the download of call i is still on the wire (PCIe is full duplex).  ``wait()`` blocks
    until everything submitted has landed in its host buffers and checks the plan's status word.
    Host tensors should be pinned; a host output buffer must not be reused before ``wait()``.
    """

    def __init__(self, lowered: B200LoweredKernel, depth: int = 2, device: str = "cuda"):
        _require_cuda()
        self.lowered, self.depth = lowered, max(1, int(depth))
        specs, outs = lowered.io_spec["tensors"], set(lowered.output_names)
        self._in_names = [n for n in lowered.io_spec["arg_names"] if n not in outs]
        mk = lambda n: torch.empty([int(d) for d in specs[n]["shape"]], dtype=TORCH_OF_DTYPE[specs[n]["dtype"]], device=device)  # noqa: E731
        self._slots = []
        for _ in range(self.depth):
            ins = {n: mk(n) for n in self._in_names}
            res = {n: mk(n) for n in lowered.output_names}
            launch, _ = bind_lowered(lowered, ins, res)
            self._slots.append((ins, res, launch, torch.cuda.Event(), torch.cuda.Event()))
        self._compute, self._download = torch.cuda.Stream(), torch.cuda.Stream()
        self._i = 0

    def submit(self, host_inputs: Mapping[str, torch.Tensor], host_outputs: Mapping[str, torch.Tensor]) -> None:
        ins, res, launch, computed, drained = self._slots[self._i % self.depth]
        self._i += 1
        with torch.cuda.stream(self._compute):
            self._compute.wait_event(drained)  # this slot's previous download has finished
            for n in self._in_names:
                ins[n].copy_(host_inputs[n], non_blocking=True)
            launch()
            computed.record(self._compute)
        with torch.cuda.stream(self._download):
            self._download.wait_event(computed)
            for n, t in res.items():
                host_outputs[n].copy_(t, non_blocking=True)
            drained.record(self._download)

    def wait(self) -> None:
        self._compute.synchronize()
        self._download.synchronize()
        check_plan_status(self.lowered)


def run_b200_kernel(*, kernel_name: str = "", cuda_src: str = "", io_spec: Mapping[str, Any], launch: Any = None,
                    bindings: Optional[Mapping[str, Any]] = None, inputs_np: Mapping[str, np.ndarray],
                    output_names: Optional[Iterable[str]] = None, extra_cuda_cflags: Optional[Iterable[str]] = None,
                    device: str = "cuda") -> Dict[str, np.ndarray]:
    """Keyword-compatible with the reference's ``run_cuda_kernel``.  ``io_spec`` must be the
    one returned by :func:`lower_intent_to_b200_kernel` (it names the plan); ``cuda_src``,
    ``launch`` and ``extra_cuda_cflags`` are accepted and unused (nothing is compiled)."""
    lowered = lookup_plan(io_spec)
    return run_lowered(lowered, inputs_np, device=device)
