"""Debug helpers: memory reports, tensor-distribution metrics, background tensor dumps (reference: ``verl/utils/debug/__init__.py``)."""
from verl_b200.utils.memory_utils import log_memory_usage as log_gpu_memory_usage  # noqa: F401
from verl_b200.utils.debug.trajectory_tracker import dump_data, get_trajectory_tracker  # noqa: F401
