"""The scan across the GPUs of one box (one process per GPU over ``torch.distributed``).

Two partitionings, neither of which exists in the reference (it is a single-GPU operator):

* **channel / batch shards** -- every ``(batch, channel)`` pair is its own recurrence, so a rank
  simply scans its slice; :func:`shard_channels` returns the slice as a view and nothing is
  exchanged.
* **sequence-parallel** -- rank ``r`` holds rows ``[r*T/G, (r+1)*T/G)``.  :func:`seqpar_scan`
  1. scans the local rows from a zero state; the kernel also leaves, per block of rows, the block's
     product of ``alpha`` and the state leaving it, and a small kernel folds the block products into
     the product over all local rows;
  2. all-gathers the per-rank ``(product, last state)`` vectors (``2*B*D`` fp32 per rank);
  3. folds the maps of the ranks before it into the state entering its rows;
  4. re-scans, from its corrected entering state, the blocks of rows that the carry still reaches:
     block after block until (product of the blocks so far) x carry is exactly zero -- from there
     on the zero-state result is already exact (for decaying gates: after a few thousand rows).
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
    """Local pieces on the GPU through the C ABI.  The small fp32 vectors and block tables of a step
    live in buffers that are kept between calls (one set per shape): a training loop calls this
    with the same shapes every step, and the kernels write the (product, state) pair straight into
    the buffer that is handed to the all-gather."""

    def __init__(self, algo: Optional[int] = None):
        self.algo = algo
        self._bufs: dict = {}

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

    def _buffers(self, which: str, alpha, algo):
        """(send [2, B*D], block_prod [B, nb, D], block_state [B, nb, D], rows per block) for one direction."""
        from . import sequential_scan_cuda as native
        B, T, D = alpha.shape
        key = (which, alpha.device, alpha.dtype, B, T, D, algo)
        got = self._bufs.get(key)
        if got is None:
            R = native.block_rows(alpha.dtype, B, T, D, algo)
            nb = -(-T // R)
            f32 = dict(dtype=torch.float32, device=alpha.device)
            got = self._bufs[key] = (torch.empty(2, B * D, **f32), torch.empty(B, nb, D, **f32),
                                     torch.empty(B, nb, D, **f32), R)
        return got

    def local_forward(self, alpha, beta, continuation: bool):
        """Zero-state scan of this rank's rows.  Returns ``(h, send, blocks)``: ``send[0]`` is the product
        of alpha over the rows, ``send[1]`` the state after the last row; ``blocks`` = per-block products,
        per-block leaving states, rows per block."""
        from . import sequential_scan_cuda as native
        B, T, D = alpha.shape
        algo = self._algo_for(alpha, beta)
        send, bp, bs, R = self._buffers("fwd", alpha, algo)
        h = torch.empty_like(alpha)
        native.forward_into(alpha, beta, h, algo=algo, continuation=continuation, h_last=send[1].view(B, D),
                            prod=send[0].view(B, D), block_prod=bp, block_state=bs)
        return h, send, (bp, bs, R)

    def local_backward(self, alpha, h, grad, continuation: bool, h_prev, prod):
        """Zero-state reverse scan.  Returns ``(dalpha, dbeta, send, blocks)`` with ``send[0]`` the product of
        alpha over the rows (the forward's, copied) and ``send[1]`` what row 0 hands to the rows before it."""
        from . import sequential_scan_cuda as native
        B, T, D = alpha.shape
        algo = self._algo_for(alpha, h, grad)
        send, bp, bs, R = self._buffers("bwd", alpha, algo)
        da, db = torch.empty_like(alpha), torch.empty_like(alpha)
        send[0].copy_(prod.reshape(-1))
        native.backward_into(alpha, h, grad, da, db, algo=algo, continuation=continuation, h_prev=h_prev,
                             u_out=send[1].view(B, D), block_prod=bp, block_state=bs)
        return da, db, send, (bp, bs, R)

    def gather_buffer(self, which: str, send, world: int):
        key = ("gather", which, send.device, send.shape, world)
        got = self._bufs.get(key)
        if got is None:
            got = self._bufs[key] = torch.empty(world, 2, send.shape[1], dtype=send.dtype, device=send.device)
        return got

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


def _gather(send: torch.Tensor, group, ops, which: str) -> torch.Tensor:
    """All-gather of this rank's [2, B*D] fp32 (product, state) pair -> [world, 2, B*D]."""
    world = _world(group)
    if world == 1:
        return send.view(1, 2, send.shape[1])
    make = getattr(ops, "gather_buffer", None)
    out = make(which, send, world) if make else torch.empty((world, 2, send.shape[1]), dtype=send.dtype,
                                                            device=send.device)
    dist.all_gather_into_tensor(out.view(world * 2, send.shape[1]), send, group=group)
    return out


def _no_mark(_name: str) -> None:
    pass


def seqpar_forward(alpha, beta, group=None, ops=None, mark=_no_mark):
    """Forward of the sequence-parallel scan on this rank's rows.  Returns ``(h, saved)`` where
    ``saved`` carries what the backward needs (state entering the rows, local product).  ``mark``
    is called with a phase name after each phase has been enqueued (for timing with events)."""
    ops = ops or NativeOps()
    rank, world = _rank(group), _world(group)
    B, T, D = alpha.shape
    h, send, blocks = ops.local_forward(alpha, beta, continuation=rank > 0)
    mark("fwd_local")
    pc = _gather(send, group, ops, "fwd")
    mark("fwd_gather")
    carry_in = None
    if rank > 0:
        carry_in = ops.compose(pc, rank, backward=False).reshape(B, D)
        ops.fixup_forward(alpha, beta, h, carry_in, blocks)
    mark("fwd_fixup")
    return h, dict(carry_in=carry_in, prod=send[0].clone())


def seqpar_backward(alpha, h, grad, saved, group=None, ops=None, mark=_no_mark):
    """Backward on this rank's rows: ``(dalpha, dbeta)`` for the local slices."""
    ops = ops or NativeOps()
    rank, world = _rank(group), _world(group)
    B, T, D = alpha.shape
    h_prev = saved["carry_in"]
    da, db, send, blocks = ops.local_backward(alpha, h, grad, continuation=rank > 0, h_prev=h_prev, prod=saved["prod"])
    mark("bwd_local")
    pc = _gather(send, group, ops, "bwd")
    mark("bwd_gather")
    if rank < world - 1:
        u_in = ops.compose(pc, rank, backward=True).reshape(B, D)
        ops.fixup_backward(alpha, h, grad, da, db, u_in, h_prev, blocks, continuation=rank > 0)
    mark("bwd_fixup")
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
