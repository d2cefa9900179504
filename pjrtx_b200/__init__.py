"""B200-native execution backend for PjRTx: plan builder + ctypes facade over libpjrtx_b200.so."""
from . import plan  # noqa: F401
from .backend import Backend, BackendError, DeviceBuffer, Executable, load_library  # noqa: F401
from .plan import PlanBuilder  # noqa: F401
