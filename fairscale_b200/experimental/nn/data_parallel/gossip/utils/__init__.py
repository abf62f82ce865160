from .cuda_metering import CudaEventRecorder, DummyCudaEventRecorder, EventRecorder, create_event_recorder  # noqa: F401
from .helpers import MultiProcessAdapter, communicate, create_process_group, flatten_tensors, group_by_dtype, make_logger, unflatten_tensors  # noqa: F401
