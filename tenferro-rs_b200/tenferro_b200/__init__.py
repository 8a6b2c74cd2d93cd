"""tenferro_b200: the host-side mirror of tenferro-rs' hot-path API over libtenferro_b200.so.

Layout follows the reference crates: `device` (tenferro-device), `tensor`
(tenferro-tensor), `prims` (tenferro-prims), `einsum` (tenferro-einsum).
"""
from .device import (  # noqa: F401
    ComputeDevice,
    CompletionEvent,
    Context,
    CrossMemorySpaceOperation,
    DeviceError,
    Error,
    InvalidArgument,
    LogicalMemorySpace,
    NoCompatibleComputeDevice,
    OpKind,
    RankMismatch,
    ShapeMismatch,
    Strided,
    preferred_compute_devices,
)
from .einsum import (  # noqa: F401
    ContractionTree,
    PreparedEinsum,
    Subscripts,
    einsum,
    einsum_into,
    einsum_owned,
    einsum_with_plan,
    einsum_with_plan_into,
    einsum_with_plan_owned,
    einsum_with_subscripts,
    einsum_with_subscripts_into,
    einsum_with_subscripts_owned,
)
from .prims import (  # noqa: F401
    Algebra, ContractKernel, CudaBackend, CudaPlan, Extension, PreparedGroupedGemm, PrimDescriptor, ReduceOp, grouped_gemm,
)
from .tensor import MemoryOrder, Tensor  # noqa: F401
