"""Python face of the CPU checker (TEST INFRASTRUCTURE ONLY).

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference`` legs
of ``bench.py`` import this module; the product package never does.

It wraps two native libraries built by ``oracle/build_oracle.py``:

* ``libfss_oracle.so`` -- the C restatement in ``scan_oracle.c`` of the reference's sequential
  scan (sequential_scan/common.py:46-59) and of its backward
  (csrc/include/sequential_scan_cpu.hpp:36-115);
* ``_ref/libfss_ref.so`` -- the reference's own C++ loop compiled from its header (optional);
* ``_ref/libfss_refgpu.so`` -- the reference's own CUDA kernels compiled from its headers behind a
  C ABI (optional; :class:`RefGpu`).

and adds :func:`torch_loop_scan`, the same recurrence written with torch ops so that autograd
can differentiate it (the way the reference's tests obtain their gradients,
sequential_scan/test_scan_cuda.py:47-72).
"""
from __future__ import annotations

import ctypes
import math
from pathlib import Path

import numpy as np

from . import build_oracle as _build

_F = ctypes.POINTER(ctypes.c_float)
_H = ctypes.POINTER(ctypes.c_uint16)
_I = ctypes.c_int64

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.build_oracle()
        L = ctypes.CDLL(str(path))
        L.fss_oracle_scan_forward_f32.argtypes = [_F, _F, _F, _I, _I, _I]
        L.fss_oracle_scan_backward_f32.argtypes = [_F, _F, _F, _F, _F, _I, _I, _I]
        L.fss_oracle_scan_forward_bf16.argtypes = [_H, _H, _H, _I, _I, _I, ctypes.c_int]
        L.fss_oracle_scan_backward_bf16.argtypes = [_H, _H, _H, _H, _H, _I, _I, _I, ctypes.c_int]
        L.fss_oracle_round_bf16.argtypes = [_F, _H, _I]
        L.fss_oracle_widen_bf16.argtypes = [_H, _F, _I]
        L.fss_oracle_chunk_summary_f32.argtypes = [_F, _F, _F, _F, _I, _I, _I, _I]
        for f in ("fss_oracle_scan_forward_f32", "fss_oracle_scan_backward_f32",
                  "fss_oracle_scan_forward_bf16", "fss_oracle_scan_backward_bf16",
                  "fss_oracle_round_bf16", "fss_oracle_widen_bf16",
                  "fss_oracle_chunk_summary_f32"):
            getattr(L, f).restype = None
        _lib = L
    return _lib


def _f32(x) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32)


def _u16(x) -> np.ndarray:
    x = np.ascontiguousarray(x)
    assert x.dtype == np.uint16, x.dtype
    return x


def _pf(a: np.ndarray):
    return a.ctypes.data_as(_F)


def _ph(a: np.ndarray):
    return a.ctypes.data_as(_H)


# ------------------------------------------------------------------ bf16 <-> fp32 on numpy

def round_bf16(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round to nearest even."""
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().fss_oracle_round_bf16(_pf(x), _ph(out), x.size)
    return out


def widen_bf16(x: np.ndarray) -> np.ndarray:
    x = _u16(x)
    out = np.empty(x.shape, dtype=np.float32)
    lib().fss_oracle_widen_bf16(_ph(x), _pf(out), x.size)
    return out


# ------------------------------------------------------------------ the scans

def scan_forward_f32(alpha, beta) -> np.ndarray:
    a, b = _f32(alpha), _f32(beta)
    assert a.shape == b.shape and a.ndim == 3
    h = np.empty_like(a)
    if a.size:
        lib().fss_oracle_scan_forward_f32(_pf(a), _pf(b), _pf(h), *a.shape)
    return h


def scan_backward_f32(alpha, h, grad):
    a, hh, g = _f32(alpha), _f32(h), _f32(grad)
    assert a.shape == hh.shape == g.shape and a.ndim == 3
    da, db = np.empty_like(a), np.empty_like(a)
    if a.size:
        lib().fss_oracle_scan_backward_f32(_pf(a), _pf(hh), _pf(g), _pf(da), _pf(db), *a.shape)
    return da, db


def scan_forward_bf16(alpha_u16, beta_u16, fused: bool = True) -> np.ndarray:
    a, b = _u16(alpha_u16), _u16(beta_u16)
    h = np.empty_like(a)
    if a.size:
        lib().fss_oracle_scan_forward_bf16(_ph(a), _ph(b), _ph(h), *a.shape, int(fused))
    return h


def scan_backward_bf16(alpha_u16, h_u16, grad_u16, fused: bool = True):
    a, hh, g = _u16(alpha_u16), _u16(h_u16), _u16(grad_u16)
    da, db = np.empty_like(a), np.empty_like(a)
    if a.size:
        lib().fss_oracle_scan_backward_bf16(_ph(a), _ph(hh), _ph(g), _ph(da), _ph(db),
                                            *a.shape, int(fused))
    return da, db


def chunk_summary_f32(alpha2d, beta2d, row0: int, row1: int):
    """(prod, carry) of rows [row0,row1) of one [T, D] column block."""
    a, b = _f32(alpha2d), _f32(beta2d)
    T, D = a.shape
    p, c = np.empty(D, np.float32), np.empty(D, np.float32)
    lib().fss_oracle_chunk_summary_f32(_pf(a), _pf(b), _pf(p), _pf(c), T, D, row0, row1)
    return p, c


# ------------------------------------------------------------------ torch conveniences

def _np_of(t):
    """torch tensor -> (numpy array, is_bf16).  bf16 tensors become their uint16 bit patterns."""
    import torch
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16), True
    return t.float().numpy(), False


def reference_values(alpha, beta, grad=None):
    """fp32 oracle on torch inputs of either I/O dtype (bf16 inputs are widened exactly).

    Returns fp32 torch tensors ``(h, dalpha, dbeta)``; the gradients use the fp32 ``h`` and are
    ``None`` when ``grad`` is None.  This is the reference's ``torch_ref`` + autograd evaluated in
    fp32 on the same seeded, already-rounded inputs.
    """
    import torch
    a, a16 = _np_of(alpha)
    b, b16 = _np_of(beta)
    a = widen_bf16(a) if a16 else a
    b = widen_bf16(b) if b16 else b
    h = scan_forward_f32(a, b)
    if grad is None:
        return torch.from_numpy(h), None, None
    g, g16 = _np_of(grad)
    g = widen_bf16(g) if g16 else g
    da, db = scan_backward_f32(a, h, g)
    return torch.from_numpy(h), torch.from_numpy(da), torch.from_numpy(db)


def reference_values_with_state(alpha, beta, grad=None, h0=None, grad_last=None, h_saved=None):
    """The fp32 oracle for a scan that starts from the state ``h0`` ([B, D], fp32) instead of from
    nothing, i.e. the reference's sequential loop (sequential_scan/common.py:51-57) with its carry
    initialised to ``h0``: ``h_0 = alpha_0*h0 + beta_0``.  Evaluated with the unchanged C oracle on
    the sequence extended by one leading row ``(alpha=1, beta=h0)``, whose row 0 is ``h0`` itself.

    ``grad_last`` ([B, D]) is an extra gradient for the state after the last row; ``h_saved`` is the
    stored (possibly rounded) output the gradients should be formed from, as the kernels do
    (``dalpha_t = dh_t * h_{t-1}`` uses the saved ``h``); default: the oracle's own fp32 ``h``.

    Returns fp32 torch tensors ``(h, h_last, dalpha, dbeta, dh0)``; entries that do not apply are None.
    """
    import torch
    widen = lambda t: (lambda x, is16: widen_bf16(x) if is16 else x)(*_np_of(t))
    a, b = widen(alpha), widen(beta)
    B, T, D = a.shape
    s0 = None if h0 is None else _f32(h0.detach().cpu().float().numpy()).reshape(B, 1, D)
    if s0 is None:
        h = scan_forward_f32(a, b)
    else:
        a2 = np.concatenate([np.ones((B, 1, D), np.float32), a], axis=1)
        b2 = np.concatenate([s0, b], axis=1)
        h = scan_forward_f32(a2, b2)[:, 1:]
    h = np.ascontiguousarray(h)
    to_t = lambda x: None if x is None else torch.from_numpy(np.ascontiguousarray(x))
    if grad is None:
        return to_t(h), to_t(h[:, -1]), None, None, None
    g = widen(grad).copy()
    if grad_last is not None:
        g[:, -1] += _f32(grad_last.detach().cpu().float().numpy())
    hs = h if h_saved is None else widen(h_saved)
    if s0 is None:
        da, db = scan_backward_f32(a, hs, g)
        return to_t(h), to_t(h[:, -1]), to_t(da), to_t(db), None
    hs2 = np.concatenate([s0, hs], axis=1)
    g2 = np.concatenate([np.zeros((B, 1, D), np.float32), g], axis=1)
    da2, db2 = scan_backward_f32(a2, hs2, g2)
    return to_t(h), to_t(h[:, -1]), to_t(da2[:, 1:]), to_t(db2[:, 1:]), to_t(db2[:, 0])


def bf16_storage_values(alpha, beta, grad=None, fused: bool = True):
    """What an exact kernel with bf16 storage / fp32 state returns, as bf16 torch tensors."""
    import torch
    a, _ = _np_of(alpha)
    b, _ = _np_of(beta)
    h = scan_forward_bf16(a, b, fused)
    to_t = lambda x: torch.from_numpy(x.view(np.int16)).view(torch.bfloat16)
    if grad is None:
        return to_t(h), None, None
    g, _ = _np_of(grad)
    da, db = scan_backward_bf16(a, h, g, fused)
    return to_t(h), to_t(da), to_t(db)


def gated_alpha_beta(r, i, x, lam):
    """alpha, beta of the gated recurrence, evaluated in float64 with numpy and rounded ONCE to the
    I/O dtype of ``r`` (torch tensors in, torch tensors out):
        alpha = exp(-8 softplus(lam) sigmoid(r)),   beta = sqrt(1 - alpha^2) sigmoid(i) x
    The formula is the Hawk / Griffin RG-LRU the reference's README.md:3 names as its use case; the
    reference itself has no code for it (its callers pass alpha and beta)."""
    import torch
    rf, jf, xf = (t.detach().cpu().to(torch.float64).numpy() for t in (r, i, x))
    lf = lam.detach().cpu().to(torch.float64).numpy()
    sig = lambda z: 1.0 / (1.0 + np.exp(-z))
    a = np.exp(-8.0 * np.log1p(np.exp(lf)) * sig(rf))
    b = np.sqrt(1.0 - a * a) * sig(jf) * xf
    return torch.from_numpy(a).to(r.dtype), torch.from_numpy(b).to(r.dtype)


def torch_loop_scan(alpha, beta):
    """The recurrence as differentiable torch ops (step-by-step, like common.py:46-59)."""
    import torch
    state = beta[:, 0, :]
    rows = [state]
    for t in range(1, alpha.shape[1]):
        state = state * alpha[:, t, :] + beta[:, t, :]
        rows.append(state)
    return torch.stack(rows, dim=1)


def torch_slice_scan(alpha, beta):
    """The recurrence with the operation sequence of the reference's sequential PyTorch scan
    (sequential_scan/common.py:46-59): a preallocated output, and per row one multiply-add on the
    running state followed by a slice assignment into the output.  Autograd differentiates through
    the slice assignments, which is what makes the reference's CPU backward slow; this variant exists
    so that the timed CPU baseline pays the same cost.  Values are identical to torch_loop_scan."""
    import torch
    out = torch.empty_like(alpha)
    state = beta[:, 0, :]
    out[:, 0, :] = state
    for t in range(1, alpha.shape[1]):
        state = state * alpha[:, t, :] + beta[:, t, :]
        out[:, t, :] = state
    return out


# ------------------------------------------------------------------ error metrics

def mixed_error_ratio(x, ref, tol: float) -> float:
    """max |x-ref| / (tol + tol*|ref|); parity holds when the ratio is <= 1."""
    import torch
    x, ref = x.detach().float().cpu(), ref.detach().float().cpu()
    if x.numel() == 0:
        return 0.0
    if not bool(torch.isfinite(x).all()):
        return math.inf
    return float(((x - ref).abs() / (tol + tol * ref.abs())).max())


def relative_l2(x, ref) -> float:
    """||x-ref|| / ||ref||: the reference tests' metric (sequential_scan/common.py:10-11)."""
    import torch
    x, ref = x.detach().double().cpu(), ref.detach().double().cpu()
    den = float(torch.linalg.norm(ref))
    return float(torch.linalg.norm(x - ref)) / den if den else 0.0


def digits(err: float) -> float:
    """Matching digits as the reference counts them (sequential_scan/common.py:14-17)."""
    return math.inf if err == 0.0 else math.ceil(-math.log10(err))


# ------------------------------------------------------------------ the compiled reference

class RefLib:
    """The reference's own C++ CPU loop (``oracle/_ref/libfss_ref.so``), when it was built."""

    def __init__(self):
        path = _build.build_ref()
        if path is None or not Path(path).is_file():
            raise FileNotFoundError("oracle/_ref/libfss_ref.so has not been built")
        L = ctypes.CDLL(str(path))
        L.fss_ref_create.argtypes = [_I, _I, _I]
        L.fss_ref_create.restype = ctypes.c_void_p
        L.fss_ref_destroy.argtypes = [ctypes.c_void_p]
        L.fss_ref_set.argtypes = [ctypes.c_void_p, ctypes.c_int, _F]
        L.fss_ref_get.argtypes = [ctypes.c_void_p, ctypes.c_int, _F]
        L.fss_ref_forward.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.fss_ref_backward.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.fss_ref_forward.restype = None
        L.fss_ref_backward.restype = None
        L.fss_ref_destroy.restype = None
        self.L = L

    @staticmethod
    def available() -> bool:
        try:
            p = _build.build_ref()
        except Exception:
            return False
        return p is not None and Path(p).is_file()

    def job(self, B: int, T: int, D: int):
        h = self.L.fss_ref_create(B, T, D)
        return _RefJob(self.L, h, (B, T, D)) if h else None


class _RefJob:
    ALPHA, BETA, H, G, DALPHA, DBETA = range(6)

    def __init__(self, L, handle, shape):
        self.L, self.handle, self.shape = L, handle, shape

    def set(self, which: int, arr) -> None:
        a = _f32(arr)
        assert a.shape == self.shape
        self.L.fss_ref_set(self.handle, which, _pf(a))

    def get(self, which: int) -> np.ndarray:
        out = np.empty(self.shape, np.float32)
        self.L.fss_ref_get(self.handle, which, _pf(out))
        return out

    def forward(self, threads: int = 1) -> None:
        self.L.fss_ref_forward(self.handle, threads)

    def backward(self, threads: int = 1) -> None:
        self.L.fss_ref_backward(self.handle, threads)

    def close(self) -> None:
        if self.handle:
            self.L.fss_ref_destroy(self.handle)
            self.handle = None

    def __del__(self):
        self.close()


class RefGpu:
    """The reference's own CUDA kernels (``oracle/_ref/libfss_refgpu.so``; launch geometry of
    csrc/sequential_scan_kernel.cu:7-268) on torch CUDA tensors.  fp32 or bf16, contiguous
    ``[batch, seq, d_model]`` with d_model in {512, 768, 1024, 1536, 2048}, seq >= 3."""

    WIDTHS = (512, 768, 1024, 1536, 2048)

    def __init__(self):
        path = _build.build_ref_gpu()
        if path is None or not Path(path).is_file():
            raise FileNotFoundError("oracle/_ref/libfss_refgpu.so has not been built")
        L = ctypes.CDLL(str(path))
        P = ctypes.c_void_p
        for name, n in (("fss_refgpu_forward", 3), ("fss_refgpu_backward", 5),
                        ("fss_refgpu_forward_half", 3), ("fss_refgpu_backward_half", 5)):
            fn = getattr(L, name)
            fn.argtypes = [P] * n + [_I, _I, _I, P]
            fn.restype = ctypes.c_int
        self.L = L

    @staticmethod
    def available() -> bool:
        try:
            p = _build.build_ref_gpu()
        except Exception:
            return False
        return p is not None and Path(p).is_file()

    @staticmethod
    def _stream(t):
        import torch
        return torch.cuda.current_stream(t.device).cuda_stream

    def forward(self, alpha, beta, out=None):
        import torch
        assert alpha.is_cuda and alpha.is_contiguous() and beta.is_contiguous() and alpha.shape == beta.shape
        out = torch.empty_like(alpha) if out is None else out
        fn = self.L.fss_refgpu_forward_half if alpha.dtype == torch.bfloat16 else self.L.fss_refgpu_forward
        rc = fn(alpha.data_ptr(), beta.data_ptr(), out.data_ptr(), *alpha.shape, self._stream(alpha))
        if rc:
            raise RuntimeError(f"reference forward kernel refused the call (code {rc}) for shape {tuple(alpha.shape)}")
        return out

    def backward(self, alpha, h, grad, dalpha=None, dbeta=None):
        """``(dalpha, dbeta)``; pass ``dbeta=h`` for the reference's own aliasing
        (csrc/sequential_scan_kernel.cu:197)."""
        import torch
        assert alpha.is_cuda and all(t.is_contiguous() and t.shape == alpha.shape for t in (alpha, h, grad))
        dalpha = torch.empty_like(alpha) if dalpha is None else dalpha
        dbeta = torch.empty_like(alpha) if dbeta is None else dbeta
        fn = self.L.fss_refgpu_backward_half if alpha.dtype == torch.bfloat16 else self.L.fss_refgpu_backward
        rc = fn(alpha.data_ptr(), h.data_ptr(), grad.data_ptr(), dalpha.data_ptr(), dbeta.data_ptr(), *alpha.shape,
                self._stream(alpha))
        if rc:
            raise RuntimeError(f"reference backward kernel refused the call (code {rc}) for shape {tuple(alpha.shape)}")
        return dalpha, dbeta
