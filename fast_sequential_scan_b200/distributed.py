"""The scan across the GPUs of one box (one process per GPU over ``torch.distributed``).

Two partitionings, neither of which exists in the reference (it is a single-GPU operator):

* **channel / batch shards** -- every ``(batch, channel)`` pair is its own recurrence, so a rank
  simply scans its slice; :func:`shard_channels` returns the slice as a view and nothing is
  exchanged.
* **sequence-parallel** -- rank ``r`` holds rows ``[r*T/G, (r+1)*T/G)``.  :func:`seqpar_scan`
  1. scans the local rows from a zero state, keeping the running product of ``alpha``;
  2. all-gathers the per-rank ``(product, last state)`` vectors (``2*B*D`` fp32 per rank);
  3. folds the maps of the ranks before it into the state entering its rows;
  4. re-scans, from its corrected entering state, every block of rows that the carry still
     reaches -- a block whose entering product times the carry is exactly zero already holds the
     exact result and is skipped (for decaying gates: all but the first few thousand rows).
  The backward mirrors this with ``u_t = alpha_t * dh_t`` flowing from the later ranks.

The numeric work is done by an ``ops`` object; :class:`NativeOps` (the product) calls the CUDA
library.  The orchestration is independent of it, which is what the CPU multi-process tests use.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def shard_channels(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """View of this rank's contiguous channel slice of a ``[B, T, D]`` tensor (no copy)."""
    D = t.shape[-1]
    if D % world:
        raise ValueError(f"d_model {D} is not divisible by {world} ranks")
    w = D // world
    return t[..., rank * w:(rank + 1) * w]


class NativeOps:
    """Local pieces on the GPU through the C ABI."""

    def __init__(self, algo: Optional[int] = None):
        self.algo = algo

    def _algo_for(self, *tensors):
        """The kernel family that will really run: block sizes of the two families differ, so a
        layout the single-pass kernels cannot take is sent to the chunked ones explicitly."""
        from . import _lib, sequential_scan_cuda as native
        if self.algo is not None:
            return self.algo
        algo = native.default_algo()
        if algo == _lib.ALGO_AUTO and not native.tma_eligible(*tensors):
            return _lib.ALGO_CHUNKED
        return algo

    def local_forward(self, alpha, beta, continuation: bool):
        from . import sequential_scan_cuda as native
        B, T, D = alpha.shape
        algo = self._algo_for(alpha, beta)
        R = native.block_rows(alpha.dtype, B, T, D, algo)
        nb = -(-T // R)
        f32 = dict(dtype=torch.float32, device=alpha.device)
        h = torch.empty_like(alpha)
        h_last, prod = torch.empty(B, D, **f32), torch.empty(B, D, **f32)
        blocks = (torch.empty(B, nb, D, **f32), torch.empty(B, nb, D, **f32), R)     # products, states, rows
        native.forward_into(alpha, beta, h, algo=algo, continuation=continuation, h_last=h_last, prod=prod,
                            block_prod=blocks[0], block_state=blocks[1])
        return h, h_last, prod, blocks

    def local_backward(self, alpha, h, grad, continuation: bool, h_prev):
        from . import sequential_scan_cuda as native
        B, T, D = alpha.shape
        algo = self._algo_for(alpha, h, grad)
        R = native.block_rows(alpha.dtype, B, T, D, algo)
        nb = -(-T // R)
        f32 = dict(dtype=torch.float32, device=alpha.device)
        da, db = torch.empty_like(alpha), torch.empty_like(alpha)
        u_out = torch.empty(B, D, **f32)
        blocks = (torch.empty(B, nb, D, **f32), torch.empty(B, nb, D, **f32), R)
        native.backward_into(alpha, h, grad, da, db, algo=algo, continuation=continuation, h_prev=h_prev,
                             u_out=u_out, block_prod=blocks[0], block_state=blocks[1])
        return da, db, u_out, blocks

    def compose(self, pc, rank: int, backward: bool):
        from . import sequential_scan_cuda as native
        return native.seqpar_compose(pc, rank, backward)

    def fixup_forward(self, alpha, beta, h, carry_in, blocks):
        from . import sequential_scan_cuda as native
        native.seqpar_fixup_forward(alpha, beta, h, carry_in, blocks[0], blocks[1], blocks[2])

    def fixup_backward(self, alpha, h, grad, da, db, u_in, h_prev, blocks, continuation: bool):
        from . import sequential_scan_cuda as native
        native.seqpar_fixup_backward(alpha, h, grad, da, db, u_in, h_prev, blocks[0], blocks[1], blocks[2],
                                     continuation)


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _gather(vec_a: torch.Tensor, vec_b: torch.Tensor, group) -> torch.Tensor:
    """All-gather of this rank's two [B, D] fp32 vectors -> [world, 2, B*D]."""
    mine = torch.stack([vec_a.reshape(-1), vec_b.reshape(-1)]).contiguous()
    world = _world(group)
    if world == 1:
        return mine.view(1, 2, mine.shape[1])
    out = torch.empty((world * 2, mine.shape[1]), dtype=mine.dtype, device=mine.device)   # ranks concatenated
    dist.all_gather_into_tensor(out, mine, group=group)
    return out.view(world, 2, mine.shape[1])


def seqpar_forward(alpha, beta, group=None, ops=None):
    """Forward of the sequence-parallel scan on this rank's rows.  Returns ``(h, saved)`` where
    ``saved`` carries what the backward needs (state entering the rows, local product)."""
    ops = ops or NativeOps()
    rank, world = _rank(group), _world(group)
    B, T, D = alpha.shape
    h, h_last, prod, blocks = ops.local_forward(alpha, beta, continuation=rank > 0)
    pc = _gather(prod, h_last, group)
    carry_in = None
    if rank > 0:
        carry_in = ops.compose(pc, rank, backward=False).reshape(B, D)
        ops.fixup_forward(alpha, beta, h, carry_in, blocks)
    return h, dict(carry_in=carry_in, prod=prod)


def seqpar_backward(alpha, h, grad, saved, group=None, ops=None):
    """Backward on this rank's rows: ``(dalpha, dbeta)`` for the local slices."""
    ops = ops or NativeOps()
    rank, world = _rank(group), _world(group)
    B, T, D = alpha.shape
    h_prev = saved["carry_in"]
    da, db, u_out, blocks = ops.local_backward(alpha, h, grad, continuation=rank > 0, h_prev=h_prev)
    pc = _gather(saved["prod"], u_out, group)
    if rank < world - 1:
        u_in = ops.compose(pc, rank, backward=True).reshape(B, D)
        ops.fixup_backward(alpha, h, grad, da, db, u_in, h_prev, blocks, continuation=rank > 0)
    return da, db


class _SeqParScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, alpha, beta, group, ops):
        h, saved = seqpar_forward(alpha, beta, group, ops)
        ctx.group, ctx.ops, ctx.extra = group, ops, saved
        ctx.save_for_backward(alpha, h)
        return h

    @staticmethod
    def backward(ctx, grad_output):
        alpha, h = ctx.saved_tensors
        da, db = seqpar_backward(alpha, h, grad_output.contiguous(), ctx.extra, ctx.group, ctx.ops)
        return da, db, None, None


def seqpar_scan(alpha: torch.Tensor, beta: torch.Tensor, group=None, ops=None) -> torch.Tensor:
    """``scan_cu`` for a sequence split across the ranks of ``group`` (this rank's rows in, this
    rank's rows of ``h`` out; differentiable)."""
    return _SeqParScan.apply(alpha, beta, group, ops)
