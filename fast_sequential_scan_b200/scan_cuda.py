"""``torch.autograd`` face of the scan: the classes and functions of the reference's
``sequential_scan/scan_cuda.py`` under the same names.

* :class:`SequentialScan` / :func:`scan` -- bf16 I/O; under ``torch.autocast("cuda")`` the inputs
  are cast to bf16 first (reference: scan_cuda.py:13-33, ``custom_fwd(cast_inputs=bfloat16)``).
* :class:`SequentialScanSingle` / :func:`scan_single` -- fp32, no autocast handling
  (reference: scan_cuda.py:36-54).

Both save ``(alpha, h)`` and compute the gradients with the reverse scan
``dh_t = g_t + alpha_{t+1} dh_{t+1}``, ``dbeta = dh``, ``dalpha_t = dh_t h_{t-1}``.
"""
from __future__ import annotations

from typing import Any, Tuple

import torch
from torch.autograd import Function

from .sequential_scan_cuda import scan_backward, scan_backward_half, scan_forward, scan_forward_half


class SequentialScan(Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx: Any, input_alpha: torch.Tensor, input_beta: torch.Tensor) -> torch.Tensor:
        h = scan_forward_half(input_alpha, input_beta)
        ctx.save_for_backward(input_alpha, h)
        return h

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx: Any, grad_output: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        input_alpha, h = ctx.saved_tensors
        alpha_grad, beta_grad = scan_backward_half(input_alpha, h, grad_output)
        return alpha_grad, beta_grad


class SequentialScanSingle(Function):
    @staticmethod
    def forward(ctx: Any, input_alpha: torch.Tensor, input_beta: torch.Tensor) -> torch.Tensor:
        h = scan_forward(input_alpha, input_beta)
        ctx.save_for_backward(input_alpha, h)
        return h

    @staticmethod
    def backward(ctx: Any, grad_output: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        input_alpha, h = ctx.saved_tensors
        alpha_grad, beta_grad = scan_backward(input_alpha, h, grad_output)
        return alpha_grad, beta_grad


def scan(alpha: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """bf16 scan ``h_0 = beta_0; h_t = alpha_t * h_{t-1} + beta_t`` over ``[batch, seq, d_model]``."""
    return SequentialScan.apply(alpha, beta)


def scan_single(alpha: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """fp32 variant of :func:`scan`."""
    return SequentialScanSingle.apply(alpha, beta)
