"""Front-end core: dtypes, devices, shapes (static, dynamic and named axes), slicing, policies, descriptors."""
from .dtype import DTypeId, Q8_0_BLOCK, Q8_0_BLOCK_BYTES, size_bytes, to_torch, from_torch  # noqa: F401
from .device import Cpu, Cuda, DeviceId, DeviceKind, DevicePreference, DeviceSet, detect_device  # noqa: F401
from .shapes import (Dim, DynDim, NamedDim, Shape, ShapeError, OperationKind, broadcast_shapes, dim, idx,  # noqa: F401
                     reshape_infer, s)
