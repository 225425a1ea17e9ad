"""B200 (sm_100a) sequential scan: drop-in for ``sequential_scan.scan_cu`` / ``scan_cu_single``
(reference: sequential_scan/__init__.py:1-2).  The Triton entry point ``scan_tr`` has no
counterpart here."""
from . import _lib

_lib.lib()   # fail at import time, loudly, when the native library has not been built

from .scan_cuda import scan as scan_cu  # noqa: E402
from .scan_cuda import scan_single as scan_cu_single  # noqa: E402
from .scan_cuda import scan_gated, set_backward_mode  # noqa: E402
from .sequential_scan_cuda import set_deterministic  # noqa: E402
from .workspace import check_status  # noqa: E402

__all__ = ["scan_cu", "scan_cu_single", "scan_gated", "set_backward_mode", "set_deterministic", "check_status"]
