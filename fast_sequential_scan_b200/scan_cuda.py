"""``torch.autograd`` face of the scan: the classes and functions of the reference's
``sequential_scan/scan_cuda.py`` under the same names.

* :class:`SequentialScan` / :func:`scan` -- bf16 I/O; under ``torch.autocast("cuda")`` the inputs
  are cast to bf16 first (reference: scan_cuda.py:13-33, ``custom_fwd(cast_inputs=bfloat16)``).
* :class:`SequentialScanSingle` / :func:`scan_single` -- fp32, no autocast handling
  (reference: scan_cuda.py:36-54).

Both compute the gradients with the reverse scan ``dh_t = g_t + alpha_{t+1} dh_{t+1}``,
``dbeta = dh``, ``dalpha_t = dh_t h_{t-1}``.  What they keep for it is chosen by ``backward_mode``:

``"saved"`` (default)
    save ``(alpha, h)``; ``grad_beta`` is a fresh tensor, ``h`` stays valid after ``backward``.
``"inplace"``
    save ``(alpha, h)``; ``grad_beta`` is written over ``h``'s storage, so the backward allocates one
    tensor instead of two and ``h`` must not be read after ``backward``.  This is what the reference's
    bf16 backward always does (csrc/sequential_scan_kernel.cu:197, ``grad_beta = h_saved``).
``"recompute"``
    save ``(alpha, beta)`` only; the backward first scans them again into a temporary ``h`` (6 more
    bytes of traffic per element in bf16) and then overwrites that temporary with ``grad_beta``.
    The forward output is not kept alive by the graph, which matters when the caller drops it.

Boundary state (no counterpart in the reference, whose kernels always start from ``h_0 = beta_0``,
csrc/include/sequential_scan_kernel_bf16.cuh:91-100; the carry semantics are those of its
sequential loop, sequential_scan/common.py:51-57, started from ``h0`` instead of from nothing):

``h0``
    fp32 ``[batch, d_model]`` state before row 0: ``h_0 = alpha_0 * h0 + beta_0`` (``alpha_0`` IS
    used then).  Differentiable: ``dL/dh0 = alpha_0 * dh_0``.
``return_final_state``
    also return the unrounded fp32 state after the last row, ``[batch, d_model]``; a gradient that
    arrives for it is added to ``dh_{T-1}``.  Feeding it to the next call as ``h0`` continues the
    sequence exactly (chunked prefill, streaming).
``reverse``
    scan from the last row to the first (``h_t = alpha_t * h_{t+1} + beta_t``); done by flipping the
    tensors around an ordinary scan, so it costs five extra tensor passes.
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
from torch.autograd import Function

from .sequential_scan_cuda import (backward_into, forward_into, gates_backward, gates_forward, scan_backward,
                                   scan_backward_half, scan_forward, scan_forward_gated, scan_forward_half)

BACKWARD_MODES = ("saved", "inplace", "recompute")
_default_mode = "saved"


def set_backward_mode(mode: str) -> str:
    """Set the process-wide default ``backward_mode``; returns the previous one."""
    global _default_mode
    if mode not in BACKWARD_MODES:
        raise ValueError(f"backward_mode must be one of {BACKWARD_MODES}, got {mode!r}")
    previous, _default_mode = _default_mode, mode
    return previous


def _resolve(mode: Optional[str]) -> str:
    mode = _default_mode if mode is None else mode
    if mode not in BACKWARD_MODES:
        raise ValueError(f"backward_mode must be one of {BACKWARD_MODES}, got {mode!r}")
    return mode


def _forward(ctx: Any, fwd, alpha: torch.Tensor, beta: torch.Tensor, mode: Optional[str]) -> torch.Tensor:
    ctx.backward_mode = _resolve(mode)
    h = fwd(alpha, beta)
    if ctx.backward_mode == "recompute":
        ctx.save_for_backward(alpha, beta)
    else:
        ctx.save_for_backward(alpha, h)
    return h


def _backward(ctx: Any, fwd, bwd, grad_output: torch.Tensor):
    if ctx.backward_mode == "recompute":
        alpha, beta = ctx.saved_tensors
        h = fwd(alpha, beta)                       # a temporary nobody else sees: reuse it for grad_beta
        alpha_grad, beta_grad = bwd(alpha, h, grad_output, True)
    else:
        alpha, h = ctx.saved_tensors
        alpha_grad, beta_grad = bwd(alpha, h, grad_output, ctx.backward_mode == "inplace")
    return alpha_grad, beta_grad, None             # trailing None as in the reference (scan_cuda.py:33)


class SequentialScan(Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx: Any, input_alpha: torch.Tensor, input_beta: torch.Tensor,
                backward_mode: Optional[str] = None) -> torch.Tensor:
        return _forward(ctx, scan_forward_half, input_alpha, input_beta, backward_mode)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx: Any, grad_output: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, None]:
        return _backward(ctx, scan_forward_half, scan_backward_half, grad_output)


class SequentialScanSingle(Function):
    @staticmethod
    def forward(ctx: Any, input_alpha: torch.Tensor, input_beta: torch.Tensor,
                backward_mode: Optional[str] = None) -> torch.Tensor:
        return _forward(ctx, scan_forward, input_alpha, input_beta, backward_mode)

    @staticmethod
    def backward(ctx: Any, grad_output: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, None]:
        return _backward(ctx, scan_forward, scan_backward, grad_output)


class _StatefulScan(Function):
    """The scan with a state entering row 0 and / or the final state returned (and the reversed
    direction).  Inputs: alpha, beta, h0 (or None), flags.  Outputs: h[, h_last]."""

    @staticmethod
    def forward(ctx: Any, alpha: torch.Tensor, beta: torch.Tensor, h0: Optional[torch.Tensor],
                want_final: bool, reverse: bool):
        if alpha.dtype not in (torch.bfloat16, torch.float32):
            raise RuntimeError(f"alpha: unsupported dtype {alpha.dtype} (bf16 or fp32)")
        if alpha.dim() != 3:
            raise RuntimeError(f"alpha: expected a [batch, seq, d_model] tensor, got {tuple(alpha.shape)}")
        B, T, D = alpha.shape
        if T == 0:
            raise RuntimeError("a scan with boundary state needs at least one row")
        a = alpha.flip(1) if reverse else alpha
        b = beta.flip(1) if reverse else beta
        state = None
        if h0 is not None:
            if h0.shape != (B, D) or h0.device != alpha.device:
                raise RuntimeError(f"h0: expected a [{B}, {D}] tensor on {alpha.device}, got {tuple(h0.shape)}")
            state = h0.detach().float().contiguous()
        h = torch.empty(a.shape, dtype=a.dtype, device=a.device)
        h_last = torch.empty(B, D, dtype=torch.float32, device=a.device) if want_final else None
        forward_into(a, b, h, continuation=state is not None, h_in=state, h_last=h_last)
        ctx.reverse, ctx.has_state, ctx.want_final = reverse, state is not None, want_final
        ctx.h0_dtype = h0.dtype if h0 is not None else None
        ctx.save_for_backward(a, h, state)
        out = h.flip(1) if reverse else h
        return (out, h_last) if want_final else out

    @staticmethod
    def backward(ctx: Any, grad_h: torch.Tensor, grad_last: Optional[torch.Tensor] = None):
        a, h, state = ctx.saved_tensors
        B, T, D = a.shape
        g = grad_h.flip(1) if ctx.reverse else grad_h
        g = g.to(a.dtype).contiguous()
        u_in = grad_last.float().contiguous() if grad_last is not None else None
        da, db = torch.empty_like(a), torch.empty_like(a)
        u_out = torch.empty(B, D, dtype=torch.float32, device=a.device) if ctx.has_state else None
        backward_into(a, h, g, da, db, continuation=ctx.has_state, u_in=u_in, h_prev=state, u_out=u_out)
        if ctx.reverse:
            da, db = da.flip(1), db.flip(1)
        dh0 = u_out.to(ctx.h0_dtype) if ctx.has_state and ctx.needs_input_grad[2] else None
        return da, db, dh0, None, None


def _scan_any(plain_cls, dtype: torch.dtype, alpha, beta, backward_mode, h0, return_final_state, reverse):
    if h0 is None and not return_final_state and not reverse:
        return plain_cls.apply(alpha, beta, backward_mode)
    if backward_mode not in (None, "saved"):
        raise ValueError("backward_mode other than 'saved' is not available together with boundary state")
    if dtype == torch.bfloat16 and torch.is_autocast_enabled("cuda"):
        alpha, beta = alpha.to(torch.bfloat16), beta.to(torch.bfloat16)      # what custom_fwd does for scan()
    if alpha.dtype != dtype or beta.dtype != dtype:
        raise RuntimeError(f"expected {dtype} tensors, got {alpha.dtype} and {beta.dtype}")
    return _StatefulScan.apply(alpha, beta, h0, bool(return_final_state), bool(reverse))


def scan(alpha: torch.Tensor, beta: torch.Tensor, *, backward_mode: Optional[str] = None,
         h0: Optional[torch.Tensor] = None, return_final_state: bool = False, reverse: bool = False):
    """bf16 scan ``h_0 = beta_0; h_t = alpha_t * h_{t-1} + beta_t`` over ``[batch, seq, d_model]``.
    With ``return_final_state`` the result is ``(h, h_last)``; see the module docstring for ``h0``
    and ``reverse``."""
    return _scan_any(SequentialScan, torch.bfloat16, alpha, beta, backward_mode, h0, return_final_state, reverse)


def scan_single(alpha: torch.Tensor, beta: torch.Tensor, *, backward_mode: Optional[str] = None,
                h0: Optional[torch.Tensor] = None, return_final_state: bool = False, reverse: bool = False):
    """fp32 variant of :func:`scan`."""
    return _scan_any(SequentialScanSingle, torch.float32, alpha, beta, backward_mode, h0, return_final_state, reverse)


class GatedSequentialScan(Function):
    """``h = scan(alpha, beta)`` with ``alpha = exp(-8 softplus(lam) sigmoid(r))`` and
    ``beta = sqrt(1 - alpha^2) sigmoid(i) x`` (the RG-LRU of Hawk / Griffin, the use case the reference's
    README.md:3 names; the reference has no such entry point).  The forward computes the gates inside
    the scan kernel, so alpha and beta never reach memory.  The backward is three launches: the gate
    kernel re-creates alpha with the forward's own arithmetic (so the reverse scan multiplies with
    exactly the alpha that produced the saved ``h``), the reverse scan gives the gradients with
    respect to alpha and beta, and the gate-backward kernel chains them to ``r, i, x, lam``."""

    @staticmethod
    def forward(ctx: Any, r: torch.Tensor, i: torch.Tensor, x: torch.Tensor, lam: torch.Tensor) -> torch.Tensor:
        h = scan_forward_gated(r, i, x, lam)
        ctx.save_for_backward(r, i, x, lam, h)
        return h

    @staticmethod
    def backward(ctx: Any, grad_output: torch.Tensor):
        r, i, x, lam, h = ctx.saved_tensors
        alpha, _ = gates_forward(r, None, None, lam, want_beta=False)
        bwd = scan_backward_half if h.dtype == torch.bfloat16 else scan_backward
        # grad_beta may take h's place only if nobody else can see h; autograd hands out the saved tensor
        alpha_grad, beta_grad = bwd(alpha, h, grad_output.contiguous())
        dr, di, dx, dlam = gates_backward(r, i, x, lam, alpha_grad, beta_grad)
        need = ctx.needs_input_grad
        return (dr if need[0] else None, di if need[1] else None, dx if need[2] else None,
                dlam.to(lam.dtype) if need[3] else None)


def scan_gated(r: torch.Tensor, i: torch.Tensor, x: torch.Tensor, lam: torch.Tensor) -> torch.Tensor:
    """Gated scan over ``[batch, seq, d_model]`` tensors ``r, i, x`` (bf16 or fp32) and the fp32
    per-channel parameter ``lam`` of ``d_model`` values; see :class:`GatedSequentialScan`."""
    return GatedSequentialScan.apply(r, i, x, lam)
