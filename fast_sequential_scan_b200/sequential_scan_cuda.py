"""Tensor-level face of the native library: the four functions of the reference's extension
module ``sequential_scan_cuda`` (csrc/sequential_scan.cpp:13-22), same names, same arguments,
same returns -- ``scan_forward(alpha, beta) -> h`` and
``scan_backward(alpha_saved, h_saved, grad_out) -> [grad_alpha, grad_beta]`` in fp32, and the
``*_half`` pair in bf16 -- implemented over the C ABI in ``include/fss_b200.h``.

Behaviour kept from the reference: outputs are freshly allocated with the inputs' shape and
dtype; a wrong dtype raises (the reference's ``data_ptr<T>()`` throws).  Behaviour changed on
purpose: any ``d_model`` and any ``seq`` are accepted (the reference raises ``RuntimeError`` outside
five widths, csrc/sequential_scan_kernel.cu:54); ``grad_beta`` is its own tensor (the reference's
bf16 backward returns the saved ``h`` storage, csrc/sequential_scan_kernel.cu:197); launches go to
torch's current stream; shapes, devices and layouts are validated.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch

from . import _lib, workspace

_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float32: _lib.DTYPE_F32}


def default_algo() -> int:
    """Kernel family: ``FSS_B200_ALGO`` = auto | chunked | lookback (default auto)."""
    name = os.environ.get("FSS_B200_ALGO", "auto").lower()
    if name not in _lib.ALGO_BY_NAME:
        raise ValueError(f"FSS_B200_ALGO={name!r}: expected one of {sorted(_lib.ALGO_BY_NAME)}")
    return _lib.ALGO_BY_NAME[name]


_deterministic = os.environ.get("FSS_B200_DETERMINISTIC", "0") not in ("", "0")


def set_deterministic(on: bool) -> bool:
    """Ask the single-pass kernels for run-to-run identical results (``FSS_FLAG_DETERMINISTIC``: every
    tile waits for its predecessor's final state instead of taking whichever summary is published
    first).  Slower on long sequences.  Returns the previous setting; the environment variable
    ``FSS_B200_DETERMINISTIC=1`` sets the initial one."""
    global _deterministic
    previous, _deterministic = _deterministic, bool(on)
    return previous


def _check_tensor(name: str, t: torch.Tensor, like: Optional[torch.Tensor], dtype: torch.dtype) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if t.dtype != dtype:
        raise RuntimeError(f"{name}: expected dtype {dtype}, got {t.dtype}")
    if t.dim() != 3:
        raise RuntimeError(f"{name}: expected a [batch, seq, d_model] tensor, got {tuple(t.shape)}")
    if like is not None:
        if t.shape != like.shape:
            raise RuntimeError(f"{name}: shape {tuple(t.shape)} differs from {tuple(like.shape)}")
        if t.device != like.device:
            raise RuntimeError(f"{name}: on {t.device}, expected {like.device}")


def _rowwise(t: torch.Tensor) -> torch.Tensor:
    """A tensor the kernels can address: unit channel stride, rows and batches not overlapping."""
    if t.is_contiguous():
        return t
    B, T, D = t.shape
    if t.numel() == 0:
        return t
    ok = (D == 1 or t.stride(2) == 1) and (T == 1 or t.stride(1) >= D) and \
         (B == 1 or t.stride(0) >= (T - 1) * t.stride(1) + D)
    return t if ok else t.contiguous()


def _view(t: torch.Tensor) -> _lib.View:
    B, T, D = t.shape
    if t.is_contiguous():
        return _lib.View(t.data_ptr(), max(T * D, 1), D)
    st = t.stride(1) if T > 1 else D
    sb = t.stride(0) if B > 1 else max(st * T, 1)
    return _lib.View(t.data_ptr(), sb, st)


_ws_bytes_cache: dict = {}


def _workspace_for(t: torch.Tensor, dtype_id: int) -> workspace.Workspace:
    """The calling stream's workspace on ``t``'s device, large enough for a scan of ``t``'s shape.
    The size query is a native call; its answers are remembered per shape."""
    key = (t.shape, dtype_id)
    need = _ws_bytes_cache.get(key)
    if need is None:
        B, T, D = t.shape
        need = _ws_bytes_cache[key] = _lib.lib().fss_workspace_bytes(B, T, D, dtype_id)
    return workspace.get(t.device, need)


def _ctx(device: torch.device, ws: workspace.Workspace, algo: Optional[int], flags: int = 0) -> _lib.ScanCtx:
    """The per-call context; the struct lives with the workspace and only algo / flags change per call.
    ``device`` goes to the library, which makes it current for the launch, so no torch device
    context is entered here."""
    ctx = ws.ctx
    if ctx is None or ctx.workspace != ws.buf.data_ptr():
        ctx = ws.ctx = _lib.ScanCtx(ctypes.sizeof(_lib.ScanCtx), device.index if device.index is not None else -1,
                                    ws.stream_handle, ws.buf.data_ptr(), ws.buf.numel(), ws.status.data_ptr(), 0, 0)
    ctx.algo = default_algo() if algo is None else algo
    ctx.flags = flags | (_lib.FLAG_DETERMINISTIC if _deterministic else 0)
    return ctx


def _vec(t: Optional[torch.Tensor], B: int, D: int, name: str) -> Optional[int]:
    if t is None:
        return None
    if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous() or t.numel() != B * D:
        raise RuntimeError(f"{name}: expected a contiguous fp32 CUDA tensor of {B}x{D} elements")
    return t.data_ptr()


def _blocks(t: Optional[torch.Tensor], name: str) -> Optional[int]:
    if t is None:
        return None
    if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
        raise RuntimeError(f"{name}: expected a contiguous fp32 CUDA tensor [B, nblocks, D]")
    return t.data_ptr()


def _launch_forward(a, b, h, dtype_id: int, algo, flags: int, state) -> None:
    """One checked call of ``fss_scan_forward_ex`` on tensors that were validated by the caller."""
    B, T, D = a.shape
    ws = _workspace_for(a, dtype_id)
    ctx = _ctx(a.device, ws, algo, flags)
    va, vb, vh = _view(a), _view(b), _view(h)
    rc = _lib.lib().fss_scan_forward_ex(ctypes.byref(ctx), dtype_id, B, T, D, ctypes.byref(va), ctypes.byref(vb),
                                        ctypes.byref(vh), ctypes.byref(state) if state is not None else None)
    workspace.launched(ws)
    if rc:
        _lib.check(rc, "fss_scan_forward_ex")


def _launch_backward(a, hh, g, grad_alpha, grad_beta, dtype_id: int, algo, flags: int, state) -> None:
    B, T, D = a.shape
    ws = _workspace_for(a, dtype_id)
    ctx = _ctx(a.device, ws, algo, flags)
    v0, v1, v2, v3, v4 = _view(a), _view(hh), _view(g), _view(grad_alpha), _view(grad_beta)
    rc = _lib.lib().fss_scan_backward_ex(ctypes.byref(ctx), dtype_id, B, T, D, ctypes.byref(v0), ctypes.byref(v1),
                                         ctypes.byref(v2), ctypes.byref(v3), ctypes.byref(v4),
                                         ctypes.byref(state) if state is not None else None)
    workspace.launched(ws)
    if rc:
        _lib.check(rc, "fss_scan_backward_ex")


def forward_into(alpha, beta, h, *, algo=None, continuation=False, h_in=None, h_last=None,
                 prod=None, block_prod=None, block_state=None, hold_dependents: bool = False,
                 _extra_flags: int = 0) -> None:
    """h <- scan(alpha, beta) into a caller-owned tensor, with the optional boundary state.
    ``hold_dependents`` = ``FSS_FLAG_HOLD_DEPENDENTS``: the next launch on the stream is placed only when this
    scan has finished."""
    dtype = alpha.dtype
    if dtype not in _DTYPES:
        raise RuntimeError(f"alpha: unsupported dtype {dtype} (bf16 or fp32)")
    _check_tensor("alpha", alpha, None, dtype)
    _check_tensor("beta", beta, alpha, dtype)
    _check_tensor("h", h, alpha, dtype)
    B, T, D = alpha.shape
    if alpha.numel() == 0:
        return
    a, b = _rowwise(alpha), _rowwise(beta)
    if _rowwise(h) is not h:
        raise RuntimeError("h: output must have unit channel stride and non-overlapping rows")
    state = None
    if not (h_in is None and h_last is None and prod is None and block_prod is None and block_state is None):
        state = _lib.ForwardState(_vec(h_in, B, D, "h_in"), _vec(h_last, B, D, "h_last"),
                                  _vec(prod, B, D, "prod"), _blocks(block_prod, "block_prod"),
                                  _blocks(block_state, "block_state"))
    flags = (_lib.FLAG_CONTINUATION if continuation else 0) | (_lib.FLAG_HOLD_DEPENDENTS if hold_dependents else 0)
    _launch_forward(a, b, h, _DTYPES[dtype], algo, flags | _extra_flags, state)


def gates_reference(r, i, x, lam):
    """alpha, beta of the gated recurrence with plain torch operations, in the dtype of ``r``:
    ``alpha = exp(-8 softplus(lam) sigmoid(r))``, ``beta = sqrt(1 - alpha^2) sigmoid(i) x`` (evaluated in
    fp32, rounded once).  Used where the fused kernel cannot run and by the backward of the gated scan."""
    rf, jf, xf = r.float(), i.float(), x.float()
    a = torch.exp(-8.0 * torch.nn.functional.softplus(lam.float()) * torch.sigmoid(rf))
    b = torch.sqrt(1.0 - a * a) * torch.sigmoid(jf) * xf
    return a.to(r.dtype), b.to(r.dtype)


def forward_gated_into(r, i, x, lam, h, *, continuation=False, h_in=None, h_last=None) -> None:
    """h <- scan(alpha, beta) with alpha, beta computed from the gates inside the kernel
    (``fss_scan_forward_gated``).  Raises :class:`FssError` with ``E_LAYOUT`` for layouts the
    single-pass kernel cannot take."""
    dtype = r.dtype
    if dtype not in _DTYPES:
        raise RuntimeError(f"r: unsupported dtype {dtype} (bf16 or fp32)")
    _check_tensor("r", r, None, dtype)
    _check_tensor("i", i, r, dtype)
    _check_tensor("x", x, r, dtype)
    _check_tensor("h", h, r, dtype)
    B, T, D = r.shape
    if lam.dtype != torch.float32 or lam.shape != (D,) or lam.device != r.device or not lam.is_contiguous():
        raise RuntimeError("lam: expected a contiguous fp32 vector of d_model values on the inputs' device")
    if r.numel() == 0:
        return
    rr, ii, xx = _rowwise(r), _rowwise(i), _rowwise(x)
    if _rowwise(h) is not h:
        raise RuntimeError("h: output must have unit channel stride and non-overlapping rows")
    ws = _workspace_for(r, _DTYPES[dtype])
    ctx = _ctx(r.device, ws, None, _lib.FLAG_CONTINUATION if continuation else 0)
    state = None
    if h_in is not None or h_last is not None:
        state = _lib.ForwardState(_vec(h_in, B, D, "h_in"), _vec(h_last, B, D, "h_last"), None, None, None)
    views = [_view(t) for t in (rr, ii, xx, h)]
    rc = _lib.lib().fss_scan_forward_gated(ctypes.byref(ctx), _DTYPES[dtype], B, T, D, ctypes.byref(views[0]),
                                           ctypes.byref(views[1]), ctypes.byref(views[2]), lam.data_ptr(),
                                           ctypes.byref(views[3]), ctypes.byref(state) if state is not None else None)
    workspace.launched(ws)
    _lib.check(rc, "fss_scan_forward_gated")


def _check_gate_inputs(r, i, x, lam):
    dtype = r.dtype
    if dtype not in _DTYPES:
        raise RuntimeError(f"r: unsupported dtype {dtype} (bf16 or fp32)")
    _check_tensor("r", r, None, dtype)
    if i is not None:
        _check_tensor("i", i, r, dtype)
        _check_tensor("x", x, r, dtype)
    D = r.shape[2]
    if lam.dtype != torch.float32 or lam.shape != (D,) or lam.device != r.device or not lam.is_contiguous():
        raise RuntimeError("lam: expected a contiguous fp32 vector of d_model values on the inputs' device")
    return dtype


def gates_forward(r, i, x, lam, want_beta: bool = True):
    """``(alpha, beta)`` of the gated recurrence as the fused forward forms them internally (same
    approximations, rounded to the I/O type); ``beta`` is None (and ``i``, ``x`` may be None) when
    ``want_beta`` is False.  One elementwise kernel (``fss_gates_forward``)."""
    dtype = _check_gate_inputs(r, i if want_beta else None, x if want_beta else None, lam)
    B, T, D = r.shape
    alpha = torch.empty(r.shape, dtype=dtype, device=r.device)
    beta = torch.empty(r.shape, dtype=dtype, device=r.device) if want_beta else None
    if r.numel() == 0:
        return alpha, beta
    rr = _rowwise(r)
    ii, xx = (_rowwise(i), _rowwise(x)) if want_beta else (None, None)
    ws = workspace.get(r.device, 1 << 16)
    ctx = _ctx(r.device, ws, None)
    vr, va = _view(rr), _view(alpha)
    vi, vx, vb = (_view(ii), _view(xx), _view(beta)) if want_beta else (None, None, None)
    ref = lambda v: ctypes.byref(v) if v is not None else None
    rc = _lib.lib().fss_gates_forward(ctypes.byref(ctx), _DTYPES[dtype], B, T, D, ref(vr), ref(vi), ref(vx),
                                      lam.data_ptr(), ref(va), ref(vb))
    _lib.check(rc, "fss_gates_forward")
    return alpha, beta


def gates_backward(r, i, x, lam, grad_alpha, grad_beta):
    """``(grad_r, grad_i, grad_x, grad_lam)`` from the scan's gradients with respect to alpha and beta
    (``fss_gates_backward``: one elementwise kernel, per-channel atomic sums for ``grad_lam``)."""
    dtype = _check_gate_inputs(r, i, x, lam)
    _check_tensor("grad_alpha", grad_alpha, r, dtype)
    _check_tensor("grad_beta", grad_beta, r, dtype)
    B, T, D = r.shape
    dr, di, dx = (torch.empty(r.shape, dtype=dtype, device=r.device) for _ in range(3))
    dlam = torch.zeros(D, dtype=torch.float32, device=r.device)
    if r.numel() == 0:
        return dr, di, dx, dlam
    tensors = [_rowwise(t) for t in (r, i, x, grad_alpha, grad_beta)] + [dr, di, dx]
    views = [_view(t) for t in tensors]
    ws = workspace.get(r.device, 1 << 16)
    ctx = _ctx(r.device, ws, None)
    rc = _lib.lib().fss_gates_backward(ctypes.byref(ctx), _DTYPES[dtype], B, T, D,
                                       ctypes.byref(views[0]), ctypes.byref(views[1]), ctypes.byref(views[2]),
                                       lam.data_ptr(), *[ctypes.byref(v) for v in views[3:]], dlam.data_ptr())
    _lib.check(rc, "fss_gates_backward")
    return dr, di, dx, dlam


def scan_forward_gated(r, i, x, lam) -> torch.Tensor:
    """Gated forward scan; on layouts the fused kernel cannot take, the gate kernel followed by the
    plain scan (the same gate arithmetic, two more tensor round trips)."""
    h = torch.empty(r.shape, dtype=r.dtype, device=r.device)
    try:
        forward_gated_into(r, i, x, lam, h)
    except _lib.FssError as e:
        if e.code != _lib.E_LAYOUT:
            raise
        a, b = gates_forward(r, i, x, lam)
        forward_into(a, b, h)
    return h


def backward_into(alpha, h, grad_out, grad_alpha, grad_beta, *, algo=None, continuation=False,
                  u_in=None, h_prev=None, u_out=None, block_prod=None, block_state=None,
                  hold_dependents: bool = False) -> None:
    """Reverse scan into caller-owned gradient tensors, with the optional boundary state (``hold_dependents``:
    see :func:`forward_into`)."""
    dtype = alpha.dtype
    if dtype not in _DTYPES:
        raise RuntimeError(f"alpha_saved: unsupported dtype {dtype} (bf16 or fp32)")
    _check_tensor("alpha_saved", alpha, None, dtype)
    _check_tensor("h_saved", h, alpha, dtype)
    _check_tensor("grad_out", grad_out, alpha, dtype)
    _check_tensor("grad_alpha", grad_alpha, alpha, dtype)
    _check_tensor("grad_beta", grad_beta, alpha, dtype)
    B, T, D = alpha.shape
    if alpha.numel() == 0:
        return
    a, hh, g = _rowwise(alpha), _rowwise(h), _rowwise(grad_out)
    for name, t in (("grad_alpha", grad_alpha), ("grad_beta", grad_beta)):
        if _rowwise(t) is not t:
            raise RuntimeError(f"{name}: output must have unit channel stride and non-overlapping rows")
    state = None
    if not (u_in is None and h_prev is None and u_out is None and block_prod is None and block_state is None):
        state = _lib.BackwardState(_vec(u_in, B, D, "u_in"), _vec(h_prev, B, D, "h_prev"),
                                   _vec(u_out, B, D, "u_out"), _blocks(block_prod, "block_prod"),
                                   _blocks(block_state, "block_state"))
    _launch_backward(a, hh, g, grad_alpha, grad_beta, _DTYPES[dtype], algo,
                     (_lib.FLAG_CONTINUATION if continuation else 0)
                     | (_lib.FLAG_HOLD_DEPENDENTS if hold_dependents else 0), state)


def _forward(alpha: torch.Tensor, beta: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _check_tensor("alpha", alpha, None, dtype)
    _check_tensor("beta", beta, alpha, dtype)
    h = torch.empty(alpha.shape, dtype=dtype, device=alpha.device)
    if h.numel():
        _launch_forward(_rowwise(alpha), _rowwise(beta), h, _DTYPES[dtype], None, 0, None)
    return h


def _backward(alpha_saved, h_saved, grad_out, dtype, inplace_grad_beta: bool = False) -> List[torch.Tensor]:
    _check_tensor("alpha_saved", alpha_saved, None, dtype)
    _check_tensor("h_saved", h_saved, alpha_saved, dtype)
    _check_tensor("grad_out", grad_out, alpha_saved, dtype)
    grad_alpha = torch.empty(alpha_saved.shape, dtype=dtype, device=alpha_saved.device)
    if grad_alpha.numel() == 0:
        return [grad_alpha, torch.empty_like(grad_alpha)]
    a, g = _rowwise(alpha_saved), _rowwise(grad_out)
    if inplace_grad_beta and h_saved.is_contiguous():
        # grad_beta overwrites h_saved (reference: csrc/sequential_scan_kernel.cu:197 does this
        # unconditionally for bf16).  Only the single-pass kernel can; if the layout sends the
        # call to the chunked kernels the library refuses and a separate buffer is used instead.
        try:
            _launch_backward(a, h_saved, g, grad_alpha, h_saved, _DTYPES[dtype], None, 0, None)
            return [grad_alpha, h_saved]
        except _lib.FssError as e:
            if e.code != _lib.E_LAYOUT:
                raise
    grad_beta = torch.empty(alpha_saved.shape, dtype=dtype, device=alpha_saved.device)
    _launch_backward(a, _rowwise(h_saved), g, grad_alpha, grad_beta, _DTYPES[dtype], None, 0, None)
    return [grad_alpha, grad_beta]


def scan_forward(alpha: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """fp32 forward scan (reference: csrc/sequential_scan_kernel.cu:7-58)."""
    return _forward(alpha, beta, torch.float32)


def scan_backward(alpha_saved, h_saved, grad_out, inplace_grad_beta: bool = False) -> List[torch.Tensor]:
    """fp32 backward, ``[grad_alpha, grad_beta]`` (reference: csrc/sequential_scan_kernel.cu:60-124).
    With ``inplace_grad_beta`` the second result is ``h_saved`` itself, overwritten."""
    return _backward(alpha_saved, h_saved, grad_out, torch.float32, inplace_grad_beta)


def scan_forward_half(alpha: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """bf16 forward scan, fp32 state (reference: csrc/sequential_scan_kernel.cu:126-187)."""
    return _forward(alpha, beta, torch.bfloat16)


def scan_backward_half(alpha_saved, h_saved, grad_out, inplace_grad_beta: bool = False) -> List[torch.Tensor]:
    """bf16 backward (reference: csrc/sequential_scan_kernel.cu:189-268).  ``grad_beta`` is a fresh
    tensor unless ``inplace_grad_beta`` asks for the reference's aliasing (csrc/sequential_scan_kernel.cu:197)."""
    return _backward(alpha_saved, h_saved, grad_out, torch.bfloat16, inplace_grad_beta)


# ---------------------------------------------------------------------------------------------
# Sequence-parallel pieces (no counterpart in the reference, which never splits the sequence)

def tma_eligible(*tensors: torch.Tensor) -> bool:
    """True when the single-pass kernels can take these [B, T, D] tensors (16-byte aligned bases,
    row and batch strides that are multiples of 16 bytes); otherwise ``auto`` uses the chunked kernels."""
    for t in tensors:
        per16 = 16 // t.element_size()
        B, T, D = t.shape
        if D % per16 or t.data_ptr() % 16 or (D > 1 and t.stride(2) != 1):
            return False
        if (T > 1 and t.stride(1) % per16) or (B > 1 and t.stride(0) % per16):
            return False
    return True


def block_rows(dtype: torch.dtype, B: int, T: int, D: int, algo: Optional[int] = None) -> int:
    """Rows per block of the ``block_prod`` outputs for this problem."""
    a = default_algo() if algo is None else algo
    return int(_lib.lib().fss_block_rows(_DTYPES[dtype], B, T, D, a))


def _plain_ctx(device: torch.device, algo: Optional[int] = None):
    ws = workspace.get(device, 1 << 16)
    return _ctx(device, ws, algo)


def seqpar_compose(pc: torch.Tensor, rank: int, backward: bool) -> torch.Tensor:
    """Fold the gathered ``[world, 2, n]`` (product, state) vectors into what enters ``rank``."""
    if pc.dtype != torch.float32 or not pc.is_cuda or not pc.is_contiguous() or pc.dim() != 3 or pc.shape[1] != 2:
        raise RuntimeError("pc: expected a contiguous fp32 CUDA tensor [world, 2, n]")
    world, _, n = pc.shape
    out = torch.empty(n, dtype=torch.float32, device=pc.device)
    with torch.cuda.device(pc.device):
        ctx = _plain_ctx(pc.device)
        rc = _lib.lib().fss_seqpar_compose(ctypes.byref(ctx), int(backward), world, rank, n,
                                           pc.data_ptr(), out.data_ptr())
    _lib.check(rc, "fss_seqpar_compose")
    return out


def seqpar_push(prod: torch.Tensor, state: torch.Tensor, rank: int, backward: bool, peer_tables, peer_words, epoch: int,
                short_waits: bool = False) -> None:
    """Write this rank's (product, state) pair -- two fp32 vectors of n values -- into slot ``rank`` of every
    rank's table and publish the epoch (``fss_seqpar_push``).  ``peer_tables`` / ``peer_words``: ctypes arrays of
    device pointers, one per rank."""
    for name, t in (("prod", prod), ("state", state)):
        if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous() or t.numel() != prod.numel():
            raise RuntimeError(f"{name}: expected a contiguous fp32 CUDA vector of {prod.numel()} values")
    ws = workspace.get(prod.device, 1 << 16)
    ctx = _ctx(prod.device, ws, None, _lib.FLAG_TEST_SHORT_WAITS if short_waits else 0)
    rc = _lib.lib().fss_seqpar_push(ctypes.byref(ctx), int(backward), len(peer_tables), rank, prod.numel(),
                                    prod.data_ptr(), state.data_ptr(), peer_tables, peer_words, epoch)
    _lib.check(rc, "fss_seqpar_push")


def seqpar_push_blocks(block_prod: torch.Tensor, state: torch.Tensor, prod_out: torch.Tensor, rank: int, peer_tables,
                       peer_words, epoch: int) -> None:
    """Forward push fused with the fold of the per-block products (``fss_seqpar_push_blocks``): ``block_prod``
    ``[B, nblocks, D]``, ``state`` and ``prod_out`` ``[B*D]`` fp32; raises ``FssError(E_LAYOUT)`` when D is not a
    multiple of 4."""
    B, nb, D = block_prod.shape
    ws = workspace.get(state.device, 1 << 16)
    ctx = _ctx(state.device, ws, None)
    rc = _lib.lib().fss_seqpar_push_blocks(ctypes.byref(ctx), len(peer_tables), rank, B, nb, D, _blocks(block_prod, "block_prod"),
                                           state.data_ptr(), prod_out.data_ptr(), peer_tables, peer_words, epoch)
    _lib.check(rc, "fss_seqpar_push_blocks")


def seqpar_compose_peer(n: int, device: torch.device, rank: int, backward: bool, peer_tables, peer_words, epoch: int,
                        short_waits: bool = False) -> torch.Tensor:
    """``fss_seqpar_compose_peer``: wait (bounded) for the pairs this rank folds, compose them, acknowledge."""
    out = torch.empty(n, dtype=torch.float32, device=device)
    ws = workspace.get(device, 1 << 16)
    ctx = _ctx(device, ws, None, _lib.FLAG_TEST_SHORT_WAITS if short_waits else 0)
    rc = _lib.lib().fss_seqpar_compose_peer(ctypes.byref(ctx), int(backward), len(peer_tables), rank, n,
                                            peer_tables, peer_words, epoch, out.data_ptr())
    _lib.check(rc, "fss_seqpar_compose_peer")
    return out


def seqpar_fixup_forward(alpha, beta, h, carry_in, block_prod, block_state, rows_per_block: int) -> None:
    """In place: re-scan the blocks of a zero-state forward scan that ``carry_in`` still reaches."""
    dtype = alpha.dtype
    _check_tensor("alpha", alpha, None, dtype)
    _check_tensor("beta", beta, alpha, dtype)
    _check_tensor("h", h, alpha, dtype)
    B, T, D = alpha.shape
    a, b = _rowwise(alpha), _rowwise(beta)
    va, vb, vh = _view(a), _view(b), _view(h)
    with torch.cuda.device(alpha.device):
        ws = workspace.get(alpha.device, 1 << 16)
        ctx = _ctx(alpha.device, ws, None, _lib.FLAG_CONTINUATION)
        rc = _lib.lib().fss_seqpar_fixup_forward(ctypes.byref(ctx), _DTYPES[dtype], B, T, D, ctypes.byref(va),
                                                 ctypes.byref(vb), ctypes.byref(vh), _vec(carry_in, B, D, "carry_in"),
                                                 _blocks(block_prod, "block_prod"), _blocks(block_state, "block_state"),
                                                 rows_per_block)
    _lib.check(rc, "fss_seqpar_fixup_forward")


def seqpar_fixup_backward(alpha, h, grad_out, grad_alpha, grad_beta, u_in, h_prev, block_prod, block_state,
                          rows_per_block: int, continuation: bool) -> None:
    """In place: re-scan the blocks of a zero-state backward scan that ``u_in`` still reaches."""
    dtype = alpha.dtype
    B, T, D = alpha.shape
    a, hh, g = _rowwise(alpha), _rowwise(h), _rowwise(grad_out)
    views = [_view(t) for t in (a, hh, g, grad_alpha, grad_beta)]
    with torch.cuda.device(alpha.device):
        ws = workspace.get(alpha.device, 1 << 16)
        ctx = _ctx(alpha.device, ws, None, _lib.FLAG_CONTINUATION if continuation else 0)
        rc = _lib.lib().fss_seqpar_fixup_backward(ctypes.byref(ctx), _DTYPES[dtype], B, T, D,
                                                  *[ctypes.byref(v) for v in views], _vec(u_in, B, D, "u_in"),
                                                  _vec(h_prev, B, D, "h_prev") if h_prev is not None else None,
                                                  _blocks(block_prod, "block_prod"),
                                                  _blocks(block_state, "block_state"), rows_per_block)
    _lib.check(rc, "fss_seqpar_fixup_backward")


def _carry_source(table: Optional[torch.Tensor], rank: int, peer_tables, peer_words, epoch: int, carry_out: torch.Tensor,
                  push=None):
    """``push``: ``(state, prod or None, prod_out or None)`` -- this rank's own pair, published by the fix-up kernel."""
    if epoch:                      # cells of a peer exchange: the table lives behind peer_tables[rank]
        src = _lib.CarrySource(len(peer_tables), rank, None, peer_tables, peer_words, epoch, carry_out.data_ptr())
        if push is not None:
            n = carry_out.numel()
            for name, t in zip(("push state", "push prod", "push prod_out"), push):
                if t is not None and (t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous() or t.numel() != n):
                    raise RuntimeError(f"{name}: expected a contiguous fp32 CUDA vector of {n} values")
            src.push_state, src.push_prod, src.push_prod_out = (t.data_ptr() if t is not None else None for t in push)
        return src
    if push is not None:
        raise RuntimeError("a fix-up can publish this rank's pair only with a peer exchange (epoch != 0)")
    if table.dtype != torch.float32 or not table.is_cuda or not table.is_contiguous() or table.dim() != 3 or table.shape[1] != 2:
        raise RuntimeError("table: expected a contiguous fp32 CUDA tensor [world, 2, n]")
    return _lib.CarrySource(table.shape[0], rank, table.data_ptr(), None, None, 0, carry_out.data_ptr())


def seqpar_fixup_forward_from(alpha, beta, h, table, rank: int, block_prod, block_state, rows_per_block: int, *,
                              peer_tables=None, peer_words=None, epoch: int = 0, push=None) -> torch.Tensor:
    """Forward fix-up that folds the gathered ``[world, 2, B*D]`` table itself (``fss_seqpar_fixup_forward_from``);
    with ``epoch`` it first waits for that peer exchange and acknowledges it.  Returns the folded carry ``[B, D]``.

    ``push = (state, prod or None, prod_out or None)`` (peer exchange only): the kernel also publishes this rank's own
    pair for exchange ``epoch`` -- no ``seqpar_push`` for it then; without ``prod`` it folds ``block_prod``."""
    dtype = alpha.dtype
    _check_tensor("alpha", alpha, None, dtype)
    _check_tensor("beta", beta, alpha, dtype)
    _check_tensor("h", h, alpha, dtype)
    B, T, D = alpha.shape
    a, b = _rowwise(alpha), _rowwise(beta)
    carry = torch.empty(B, D, dtype=torch.float32, device=alpha.device)
    src = _carry_source(table, rank, peer_tables, peer_words, epoch, carry, push)
    va, vb, vh = _view(a), _view(b), _view(h)
    ws = workspace.get(alpha.device, 1 << 16)
    ctx = _ctx(alpha.device, ws, None, _lib.FLAG_CONTINUATION)
    rc = _lib.lib().fss_seqpar_fixup_forward_from(ctypes.byref(ctx), _DTYPES[dtype], B, T, D, ctypes.byref(va), ctypes.byref(vb),
                                                  ctypes.byref(vh), ctypes.byref(src), _blocks(block_prod, "block_prod"),
                                                  _blocks(block_state, "block_state"), rows_per_block)
    _lib.check(rc, "fss_seqpar_fixup_forward_from")
    return carry


def seqpar_fixup_backward_from(alpha, h, grad_out, grad_alpha, grad_beta, table, rank: int, h_prev, block_prod, block_state,
                               rows_per_block: int, continuation: bool, *, peer_tables=None, peer_words=None,
                               epoch: int = 0, push=None) -> torch.Tensor:
    """Backward counterpart of :func:`seqpar_fixup_forward_from` (``push`` needs the product); returns the folded
    ``u`` ``[B, D]``."""
    dtype = alpha.dtype
    B, T, D = alpha.shape
    a, hh, g = _rowwise(alpha), _rowwise(h), _rowwise(grad_out)
    views = [_view(t) for t in (a, hh, g, grad_alpha, grad_beta)]
    u_in = torch.empty(B, D, dtype=torch.float32, device=alpha.device)
    src = _carry_source(table, rank, peer_tables, peer_words, epoch, u_in, push)
    ws = workspace.get(alpha.device, 1 << 16)
    ctx = _ctx(alpha.device, ws, None, _lib.FLAG_CONTINUATION if continuation else 0)
    rc = _lib.lib().fss_seqpar_fixup_backward_from(ctypes.byref(ctx), _DTYPES[dtype], B, T, D,
                                                   *[ctypes.byref(v) for v in views], ctypes.byref(src),
                                                   _vec(h_prev, B, D, "h_prev") if h_prev is not None else None,
                                                   _blocks(block_prod, "block_prod"), _blocks(block_state, "block_state"),
                                                   rows_per_block)
    _lib.check(rc, "fss_seqpar_fixup_backward_from")
    return u_in
