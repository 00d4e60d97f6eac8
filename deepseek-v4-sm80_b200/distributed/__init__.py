"""Public names of the reference's ``minisgl.distributed`` package."""
from ..parallel.info import DistributedInfo, get_tp_info, set_tp_info, try_get_tp_info  # noqa: F401
from .launch import launch_tensor_parallel  # noqa: F401
