from .logger import init_logger  # noqa: F401
from .misc import UNSET, align_ceil, align_down, call_if_main, div_ceil, div_even  # noqa: F401
