"""ferrum_cuda for B200: the quantised-weight inference hot path of ferrum-gpu as hand-written
sm_100a CUDA kernels behind a C ABI (include/ferrum_cuda.h), with the host-side mirror of the
reference's operator, resident-model and engine interfaces."""
from . import _ffi  # noqa: F401
from .device import CudaError, Device  # noqa: F401
from .quant import Mode, QKind, QWeight, linear_q, upload_quantised, upload_qweight  # noqa: F401
from .resident import CudaGpt2, CudaLlama, plan_bytes  # noqa: F401
from .engine import CudaBackend, GenOpts, generate_with  # noqa: F401
