"""ctypes binding of ``libfss_b200.so`` (declarations in ``include/fss_b200.h``).

There is no fallback: if the library is missing the import of the package fails with a clear
message, and nothing in the package computes a scan any other way.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libfss_b200.so"

DTYPE_BF16, DTYPE_F32 = 0, 1
ALGO_AUTO, ALGO_CHUNKED, ALGO_LOOKBACK = 0, 1, 2
FLAG_CONTINUATION = 1
FLAG_DETERMINISTIC = 2
FLAG_HOLD_DEPENDENTS = 4
E_LAYOUT = -5      # FSS_E_LAYOUT
FLAG_TEST_SHORT_WAITS, FLAG_TEST_MUTE_FIRST_BLOCK = 0x100, 0x200

ALGO_BY_NAME = {"auto": ALGO_AUTO, "chunked": ALGO_CHUNKED, "lookback": ALGO_LOOKBACK}

STATUS_TEXT = {
    1: "a tile gave up waiting for its predecessor's carry (look-back timeout)",
    2: "a tile gave up waiting for its own TMA loads",
    3: "a rank gave up waiting for another rank's carry (peer exchange timeout)",
}


class View(Structure):
    _fields_ = [("ptr", c_void_p), ("stride_b", c_int64), ("stride_t", c_int64)]


class ScanCtx(Structure):
    _fields_ = [("struct_bytes", c_uint32), ("device", c_int32), ("stream", c_void_p),
                ("workspace", c_void_p), ("workspace_bytes", c_size_t), ("status", c_void_p),
                ("algo", c_int32), ("flags", c_int32)]


class ForwardState(Structure):
    _fields_ = [("h_in", c_void_p), ("h_last", c_void_p), ("prod", c_void_p), ("block_prod", c_void_p),
                ("block_state", c_void_p)]


class BackwardState(Structure):
    _fields_ = [("u_in", c_void_p), ("h_prev", c_void_p), ("u_out", c_void_p), ("block_prod", c_void_p),
                ("block_state", c_void_p)]


class CarrySource(Structure):
    _fields_ = [("world", c_int32), ("rank", c_int32), ("table", c_void_p), ("peer_tables", POINTER(c_void_p)),
                ("peer_words", POINTER(c_void_p)), ("epoch", c_uint32), ("carry_out", c_void_p),
                ("push_state", c_void_p), ("push_prod", c_void_p), ("push_prod_out", c_void_p)]


_P = POINTER

# name -> (restype, argtypes); every symbol include/fss_b200.h declares
SIGNATURES = {
    "fss_abi_version": (c_int, []),
    "fss_strerror": (c_char_p, [c_int]),
    "fss_last_cuda_error": (c_char_p, []),
    "fss_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int]),
    "fss_workspace_init": (c_int, [c_void_p, c_size_t, c_void_p]),
    "fss_scan_forward": (c_int, [_P(ScanCtx), c_int64, c_int64, c_int64, _P(View), _P(View), _P(View)]),
    "fss_scan_backward": (c_int, [_P(ScanCtx), c_int64, c_int64, c_int64] + [_P(View)] * 5),
    "fss_scan_forward_half": (c_int, [_P(ScanCtx), c_int64, c_int64, c_int64, _P(View), _P(View), _P(View)]),
    "fss_scan_backward_half": (c_int, [_P(ScanCtx), c_int64, c_int64, c_int64] + [_P(View)] * 5),
    "fss_scan_forward_ex": (c_int, [_P(ScanCtx), c_int, c_int64, c_int64, c_int64, _P(View), _P(View), _P(View),
                                    _P(ForwardState)]),
    "fss_scan_backward_ex": (c_int, [_P(ScanCtx), c_int, c_int64, c_int64, c_int64] + [_P(View)] * 5
                             + [_P(BackwardState)]),
    "fss_scan_forward_gated": (c_int, [_P(ScanCtx), c_int, c_int64, c_int64, c_int64, _P(View), _P(View), _P(View),
                                       c_void_p, _P(View), _P(ForwardState)]),
    "fss_gates_forward": (c_int, [_P(ScanCtx), c_int, c_int64, c_int64, c_int64, _P(View), _P(View), _P(View),
                                  c_void_p, _P(View), _P(View)]),
    "fss_gates_backward": (c_int, [_P(ScanCtx), c_int, c_int64, c_int64, c_int64, _P(View), _P(View), _P(View),
                                   c_void_p] + [_P(View)] * 5 + [c_void_p]),
    "fss_block_rows": (c_int64, [c_int, c_int64, c_int64, c_int64, c_int]),
    "fss_seqpar_compose": (c_int, [_P(ScanCtx), c_int, c_int, c_int, c_int64, c_void_p, c_void_p]),
    "fss_seqpar_push": (c_int, [_P(ScanCtx), c_int, c_int, c_int, c_int64, c_void_p, c_void_p, _P(c_void_p), _P(c_void_p),
                                c_uint32]),
    "fss_seqpar_push_blocks": (c_int, [_P(ScanCtx), c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                       _P(c_void_p), _P(c_void_p), c_uint32]),
    "fss_seqpar_compose_peer": (c_int, [_P(ScanCtx), c_int, c_int, c_int, c_int64, _P(c_void_p), _P(c_void_p), c_uint32,
                                        c_void_p]),
    "fss_seqpar_fixup_forward": (c_int, [_P(ScanCtx), c_int, c_int64, c_int64, c_int64, _P(View), _P(View), _P(View),
                                         c_void_p, c_void_p, c_void_p, c_int64]),
    "fss_seqpar_fixup_backward": (c_int, [_P(ScanCtx), c_int, c_int64, c_int64, c_int64] + [_P(View)] * 5
                                  + [c_void_p, c_void_p, c_void_p, c_void_p, c_int64]),
    "fss_seqpar_fixup_forward_from": (c_int, [_P(ScanCtx), c_int, c_int64, c_int64, c_int64, _P(View), _P(View), _P(View),
                                              _P(CarrySource), c_void_p, c_void_p, c_int64]),
    "fss_seqpar_fixup_backward_from": (c_int, [_P(ScanCtx), c_int, c_int64, c_int64, c_int64] + [_P(View)] * 5
                                       + [_P(CarrySource), c_void_p, c_void_p, c_void_p, c_int64]),
    "fss_scan_forward_noalloc": (c_int, [c_int, c_int, c_void_p, c_int64, c_int64, c_int64, _P(View), _P(View), _P(View)]),
}

_lib = None


class FssError(RuntimeError):
    """A non-zero return code of the native library."""

    def __init__(self, code: int, where: str, detail: str = ""):
        self.code = code
        text = lib().fss_strerror(code).decode()
        super().__init__(f"{where}: {text} (code {code})" + (f": {detail}" if detail else ""))


def lib() -> ctypes.CDLL:
    """Load the native library once; raise ImportError when it has not been built."""
    global _lib
    if _lib is None:
        path = Path(os.environ.get("FSS_B200_LIB", LIB_PATH))
        if not path.is_file():
            raise ImportError(
                f"{path} is missing: build it with `python fast_sequential_scan_b200/build.py` "
                "(needs nvcc); this package has no CPU or PyTorch fallback")
        L = ctypes.CDLL(str(path))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)          # AttributeError here = header/library skew
            fn.restype, fn.argtypes = res, args
        if L.fss_abi_version() != 1:
            raise ImportError(f"{path}: ABI version {L.fss_abi_version()} != 1")
        _lib = L
    return _lib


def check(code: int, where: str) -> None:
    if code != 0:
        detail = lib().fss_last_cuda_error().decode() if code in (-6, -8, -9) else ""
        raise FssError(code, where, detail)
