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


class PeerExchange:
    """Carry exchange through peer memory: every rank's gather table and control words are allocated
    in torch's symmetric memory, so that each process holds device pointers to the tables of all GPUs
    of the box; a push kernel writes this rank's pair into every table with plain stores over NVLink,
    as 8-byte cells that carry the exchange number, and the consumer polls (bounded) the cells it needs
    and acknowledges them.  One instance serves one direction of one shape; exchanges are numbered
    from 1."""

    def __init__(self, n: int, device: torch.device, backward: bool, group=None):
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 16:
            raise RuntimeError("peer exchange serves at most 16 ranks")
        self.n, self.device, self.backward = n, device, backward
        cell_floats = self.world * 2 * n * 2          # 8-byte cells {value, exchange number}
        # one allocation: the cells, then the control words (exchange numbers start at 1, so zero = nothing yet)
        self.buf = symm_mem.empty(cell_floats + 64, dtype=torch.float32, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group.group_name)
        ptrs = list(self.handle.buffer_ptrs)
        self.tables = (ctypes.c_void_p * self.world)(*ptrs)
        self.words = (ctypes.c_void_p * self.world)(*[p + cell_floats * 4 for p in ptrs])
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group)                 # every table is zeroed before anyone pushes

    def push(self, prod: torch.Tensor, state: torch.Tensor) -> int:
        from . import sequential_scan_cuda as native
        self.epoch += 1
        native.seqpar_push(prod, state, self.rank, self.backward, self.tables, self.words, self.epoch)
        return self.epoch

    def compose(self, epoch: int) -> torch.Tensor:
        from . import sequential_scan_cuda as native
        return native.seqpar_compose_peer(self.n, self.device, self.rank, self.backward, self.tables, self.words, epoch)


class NativeOps:
    """Local pieces on the GPU through the C ABI.  The small fp32 vectors and block tables of a step
    live in buffers that are kept between calls (one set per shape): a training loop calls this
    with the same shapes every step, and the kernels write the (product, state) pair straight into
    the buffer that is handed to the all-gather."""

    def __init__(self, algo: Optional[int] = None, exchange: str = "collective"):
        """``exchange``: "collective" = ``all_gather_into_tensor`` of the process group (NCCL);
        "peer" = :class:`PeerExchange` (GPUs of one box with peer access)."""
        if exchange not in ("collective", "peer"):
            raise ValueError("exchange must be 'collective' or 'peer'")
        self.algo = algo
        self.exchange = exchange
        self._bufs: dict = {}

    def peer(self, which: str, send, group) -> PeerExchange:
        key = ("peer", which, send.device, send.shape[1])
        got = self._bufs.get(key)
        if got is None:
            got = self._bufs[key] = PeerExchange(send.shape[1], send.device, which == "bwd", group)
        return got

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
        # with the peer exchange the product over the rows is folded from the block products by the kernel that
        # publishes the pair (the fix-up, or the push launch of the rank without one): one launch less
        self._prod_pending = self.exchange == "peer" and D % 4 == 0
        native.forward_into(alpha, beta, h, algo=algo, continuation=continuation, h_last=send[1].view(B, D),
                            prod=None if self._prod_pending else send[0].view(B, D), block_prod=bp, block_state=bs,
                            hold_dependents=self.exchange == "peer" and continuation)      # a fix-up follows directly
        return h, send, (bp, bs, R)

    def local_backward(self, alpha, h, grad, continuation: bool, h_prev, prod):
        """Zero-state reverse scan.  Returns ``(dalpha, dbeta, send, blocks)`` with ``send[0]`` the product of
        alpha over the rows (the forward's, copied) and ``send[1]`` what row 0 hands to the rows before it."""
        from . import sequential_scan_cuda as native
        B, T, D = alpha.shape
        algo = self._algo_for(alpha, h, grad)
        send, bp, bs, R = self._buffers("bwd", alpha, algo)
        da, db = torch.empty_like(alpha), torch.empty_like(alpha)
        if self.exchange == "collective":          # the all-gather sends one contiguous [2, n] pair
            send[0].copy_(prod.reshape(-1))
        native.backward_into(alpha, h, grad, da, db, algo=algo, continuation=continuation, h_prev=h_prev,
                             u_out=send[1].view(B, D), block_prod=bp, block_state=bs,
                             hold_dependents=self.exchange == "peer")
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

    # The fix-up kernels can fold the exchanged table themselves (one launch less per direction): these two
    # are what seqpar_forward / seqpar_backward use when the ops object has them.
    def exchange_and_fixup_forward(self, alpha, beta, h, send, prod, blocks, rank: int, world: int, group, mark):
        """Returns ``(carry_in or None, prod)``: the state entering this rank's rows and the product of alpha
        over them, in a tensor of its own (the backward needs it after ``send`` has been reused)."""
        from . import sequential_scan_cuda as native
        if self.exchange == "peer":
            peer = self.peer("fwd", send, group)
            pending = getattr(self, "_prod_pending", False)      # the product is still to be folded from the blocks
            kept = torch.empty_like(send[0]) if pending else None
            peer.epoch += 1
            if rank == 0:                                        # no fix-up here: a push launch of its own
                if pending:
                    native.seqpar_push_blocks(blocks[0], send[1], kept, rank, peer.tables, peer.words, peer.epoch)
                else:
                    native.seqpar_push(send[0], send[1], rank, False, peer.tables, peer.words, peer.epoch)
                mark("fwd_gather")
                return None, kept if pending else send[0].clone()
            # the fix-up kernel publishes this rank's pair itself, right after the local scan
            mark("fwd_gather")
            push = (send[1], None, kept) if pending else (send[1], send[0], None)
            carry = native.seqpar_fixup_forward_from(alpha, beta, h, None, rank, blocks[0], blocks[1], blocks[2],
                                                     peer_tables=peer.tables, peer_words=peer.words, epoch=peer.epoch,
                                                     push=push)
            return carry, kept if pending else send[0].clone()
        pc = _gather(send, group, self, "fwd")
        mark("fwd_gather")
        kept = send[0].clone()
        if rank == 0:
            return None, kept
        return native.seqpar_fixup_forward_from(alpha, beta, h, pc, rank, blocks[0], blocks[1], blocks[2]), kept

    def exchange_and_fixup_backward(self, alpha, h, grad, da, db, send, prod, h_prev, blocks, rank: int, world: int,
                                    continuation: bool, group, mark):
        from . import sequential_scan_cuda as native
        if self.exchange == "peer":
            peer = self.peer("bwd", send, group)
            if rank == world - 1:
                peer.push(prod.reshape(-1), send[1])
                mark("bwd_gather")
                return None
            peer.epoch += 1
            mark("bwd_gather")
            return native.seqpar_fixup_backward_from(alpha, h, grad, da, db, None, rank, h_prev, blocks[0], blocks[1],
                                                     blocks[2], continuation, peer_tables=peer.tables,
                                                     peer_words=peer.words, epoch=peer.epoch,
                                                     push=(send[1], prod.reshape(-1), None))
        pc = _gather(send, group, self, "bwd")
        mark("bwd_gather")
        if rank == world - 1:
            return None
        return native.seqpar_fixup_backward_from(alpha, h, grad, da, db, pc, rank, h_prev, blocks[0], blocks[1], blocks[2],
                                                 continuation)

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


def _exchange_and_compose(ops, which: str, send, prod, rank: int, world: int, backward: bool, needed: bool, group, mark):
    """Hand this rank's pair (prod, send[1]) to the others and fold what this rank needs; returns the carry
    ([n]) or None."""
    if world > 1 and getattr(ops, "exchange", "collective") == "peer":
        peer = ops.peer(which, send, group)
        epoch = peer.push(prod.reshape(-1), send[1])
        mark(which + "_gather")
        return peer.compose(epoch) if needed else None
    pc = _gather(send, group, ops, which)
    mark(which + "_gather")
    return ops.compose(pc, rank, backward=backward) if needed else None


def seqpar_forward(alpha, beta, group=None, ops=None, mark=_no_mark):
    """Forward of the sequence-parallel scan on this rank's rows.  Returns ``(h, saved)`` where
    ``saved`` carries what the backward needs (state entering the rows, local product).  ``mark``
    is called with a phase name after each phase has been enqueued (for timing with events)."""
    ops = ops or NativeOps()
    rank, world = _rank(group), _world(group)
    B, T, D = alpha.shape
    fused = world > 1 and hasattr(ops, "exchange_and_fixup_forward")
    h, send, blocks = ops.local_forward(alpha, beta, continuation=rank > 0)
    mark("fwd_local")
    if fused:
        carry_in, prod = ops.exchange_and_fixup_forward(alpha, beta, h, send, send[0], blocks, rank, world, group, mark)
    else:
        carry_in = _exchange_and_compose(ops, "fwd", send, send[0], rank, world, False, rank > 0, group, mark)
        if carry_in is not None:
            carry_in = carry_in.reshape(B, D)
            ops.fixup_forward(alpha, beta, h, carry_in, blocks)
        prod = send[0].clone()
    mark("fwd_fixup")
    return h, dict(carry_in=carry_in, prod=prod)


def seqpar_backward(alpha, h, grad, saved, group=None, ops=None, mark=_no_mark):
    """Backward on this rank's rows: ``(dalpha, dbeta)`` for the local slices."""
    ops = ops or NativeOps()
    rank, world = _rank(group), _world(group)
    B, T, D = alpha.shape
    h_prev = saved["carry_in"]
    fused = world > 1 and hasattr(ops, "exchange_and_fixup_backward")
    da, db, send, blocks = ops.local_backward(alpha, h, grad, continuation=rank > 0, h_prev=h_prev, prod=saved["prod"])
    mark("bwd_local")
    if fused:
        ops.exchange_and_fixup_backward(alpha, h, grad, da, db, send, saved["prod"], h_prev, blocks, rank, world,
                                        rank > 0, group, mark)
    else:
        u_in = _exchange_and_compose(ops, "bwd", send, saved["prod"], rank, world, True, rank < world - 1, group, mark)
        if u_in is not None:
            ops.fixup_backward(alpha, h, grad, da, db, u_in.reshape(B, D), h_prev, blocks, continuation=rank > 0)
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
    rank's rows of ``h`` out; differentiable).  Pass one ``NativeOps`` object for all calls of a
    training loop: it keeps the exchange buffers (and, with ``exchange="peer"``, the peer mappings)."""
    return _SeqParScan.apply(alpha, beta, group, ops)
