"""Exception types of the backend, mirroring the reference's pair
``CudaLoweringError`` (backends/cuda/codegen/intentir_to_cuda.py:23-24) and
``CudaRuntimeError`` (frontends/cuda/runtime.py:23-24)."""


class B200LoweringError(RuntimeError):
    """The graph (or its shapes / dtypes) cannot be lowered to the B200 kernels."""


class B200RuntimeError(RuntimeError):
    """Launching or running a lowered plan failed."""
