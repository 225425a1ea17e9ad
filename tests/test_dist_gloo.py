"""Multi-process (gloo, CPU, world size 2 and 3) tests of the host-side multi-GPU logic.

The orchestration in ``fast_sequential_scan_b200.distributed`` is independent of who does the
local numeric work; here the local pieces are a NumPy stand-in built on the CPU checker, so the
test pins the protocol -- what is gathered, how the carries are folded, which rank fixes what --
against the single-process sequential scan.  (On a GPU the same functions run with ``NativeOps``;
``tests/test_gpu_parity.py`` covers those kernels.)
"""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


class OracleOps:
    """CPU stand-in for the CUDA pieces (same contracts as NativeOps), fp32."""
    R = 16

    def local_forward(self, alpha, beta, continuation):
        a, b = alpha.numpy().copy(), beta.numpy()
        B, T, D = a.shape
        if not continuation:
            a[:, 0] = 0.0
        h = np.zeros_like(a)
        state = np.zeros((B, D), np.float32)
        total = np.ones((B, D), np.float32)
        nb = -(-T // self.R)
        bp, bs = np.ones((B, nb, D), np.float32), np.zeros((B, nb, D), np.float32)
        for t in range(T):
            state = a[:, t] * state + b[:, t]
            total = total * a[:, t]
            bp[:, t // self.R] *= a[:, t]              # the block's own product
            h[:, t] = state
            bs[:, t // self.R] = state                 # ends as the state leaving the block
        blocks = (torch.from_numpy(bp), torch.from_numpy(bs), self.R)
        send = torch.from_numpy(np.stack([total.reshape(-1), state.reshape(-1)]))
        return torch.from_numpy(h), send, blocks

    @staticmethod
    def _backward_rows(a, hh, g, da, db, u, rows, continuation, h_prev):
        for t in rows:
            dh = g[:, t] + u
            db[:, t] = dh
            hp = hh[:, t - 1] if t > 0 else (h_prev.numpy() if (continuation and h_prev is not None) else 0.0)
            da[:, t] = dh * hp if (t > 0 or continuation) else 0.0
            u = (a[:, t] if (t > 0 or continuation) else 0.0) * dh
        return u

    def local_backward(self, alpha, h, grad, continuation, h_prev, prod):
        a, hh, g = alpha.numpy(), h.numpy(), grad.numpy()
        B, T, D = a.shape
        da, db = np.zeros_like(a), np.zeros_like(a)
        u = np.zeros((B, D), np.float32)
        nb = -(-T // self.R)
        bp, bs = np.ones((B, nb, D), np.float32), np.zeros((B, nb, D), np.float32)
        for j in range(nb - 1, -1, -1):
            rows = range(min(T, (j + 1) * self.R) - 1, j * self.R - 1, -1)
            u = self._backward_rows(a, hh, g, da, db, u, rows, continuation, h_prev)
            for t in rows:
                bp[:, j] *= (a[:, t] if (t > 0 or continuation) else 0.0)
            bs[:, j] = u
        blocks = (torch.from_numpy(bp), torch.from_numpy(bs), self.R)
        send = torch.stack([prod.reshape(-1), torch.from_numpy(u.reshape(-1).copy())])
        return torch.from_numpy(da), torch.from_numpy(db), send, blocks

    def compose(self, pc, rank, backward):
        pc = pc.numpy()
        world = pc.shape[0]
        carry = np.zeros(pc.shape[2], np.float32)
        order = range(rank) if not backward else range(world - 1, rank, -1)
        for r in order:
            carry = pc[r, 0] * carry + pc[r, 1]
        return torch.from_numpy(carry)

    def fixup_forward(self, alpha, beta, h, carry_in, blocks):
        bp, bs, R = blocks
        a, b, hh = alpha.numpy(), beta.numpy(), h.numpy()        # hh shares memory with h: in place
        T = a.shape[1]
        run = np.ones_like(carry_in.numpy())
        for j in range(-(-T // R)):
            w = run * carry_in.numpy()                 # (product of the blocks before j) * carry
            if not np.any(w):
                break
            state = (bs[:, j - 1].numpy() if j else 0.0) + w
            for t in range(j * R, min(T, (j + 1) * R)):
                state = a[:, t] * state + b[:, t]
                hh[:, t] = state
            run = run * bp[:, j].numpy()

    def fixup_backward(self, alpha, h, grad, da, db, u_in, h_prev, blocks, continuation):
        bp, bs, R = blocks
        a, hh, g = alpha.numpy(), h.numpy(), grad.numpy()
        T = a.shape[1]
        nb = -(-T // R)
        dan, dbn = da.numpy(), db.numpy()
        run = np.ones_like(u_in.numpy())
        for j in range(nb - 1, -1, -1):
            w = run * u_in.numpy()                     # (product of the blocks after j) * u_in
            if not np.any(w):
                break
            u = (0.0 if j == nb - 1 else bs[:, j + 1].numpy()) + w
            rows = range(min(T, (j + 1) * R) - 1, j * R - 1, -1)
            self._backward_rows(a, hh, g, dan, dbn, u, rows, continuation, h_prev)
            run = run * bp[:, j].numpy()


class FusedOracleOps(OracleOps):
    """The same stand-in behind the interface of the ops that fold the exchanged table inside the fix-up
    (``exchange_and_fixup_forward / _backward``, what ``NativeOps`` offers on a GPU): exercises that branch of
    ``seqpar_forward`` / ``seqpar_backward`` -- argument order, the ``(carry, product)`` return, which rank
    skips which fix-up -- on CPU ranks."""
    calls = None

    def exchange_and_fixup_forward(self, alpha, beta, h, send, prod, blocks, rank, world, group, mark):
        from fast_sequential_scan_b200 import distributed as fd
        self.calls = (self.calls or []) + ["fwd"]
        pc = fd._gather(send, group, self, "fwd")
        mark("fwd_gather")
        kept = send[0].clone()
        if rank == 0:
            return None, kept
        carry = self.compose(pc, rank, backward=False).reshape(alpha.shape[0], alpha.shape[2])
        self.fixup_forward(alpha, beta, h, carry, blocks)
        return carry, kept

    def exchange_and_fixup_backward(self, alpha, h, grad, da, db, send, prod, h_prev, blocks, rank, world, continuation,
                                    group, mark):
        from fast_sequential_scan_b200 import distributed as fd
        self.calls = (self.calls or []) + ["bwd"]
        assert continuation == (rank > 0)
        pc = fd._gather(send, group, self, "bwd")
        mark("bwd_gather")
        if rank == world - 1:
            return None
        u_in = self.compose(pc, rank, backward=True).reshape(alpha.shape[0], alpha.shape[2])
        self.fixup_backward(alpha, h, grad, da, db, u_in, h_prev, blocks, continuation)
        return u_in


def _worker(rank, world, port, mode, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fast_sequential_scan_b200 import distributed as fd
        from oracle import oracle
        gen = torch.Generator().manual_seed(123)
        B, T, D = 2, 96 * world, 24
        a = 0.6 + 0.39 * torch.rand(B, T, D, generator=gen)
        b = torch.randn(B, T, D, generator=gen)
        g = torch.randn(B, T, D, generator=gen)
        h_ref = torch.from_numpy(oracle.scan_forward_f32(a.numpy(), b.numpy()))
        da_ref, db_ref = (torch.from_numpy(x) for x in oracle.scan_backward_f32(a.numpy(), h_ref.numpy(), g.numpy()))
        if mode in ("seqpar", "seqpar_fused"):
            rows = slice(rank * T // world, (rank + 1) * T // world)
            al = a[:, rows].clone().requires_grad_(True)
            bl = b[:, rows].clone().requires_grad_(True)
            ops = FusedOracleOps() if mode == "seqpar_fused" else OracleOps()
            h = fd.seqpar_scan(al, bl, None, ops)
            h.backward(g[:, rows].clone())
            ok = (torch.allclose(h.detach(), h_ref[:, rows], rtol=1e-4, atol=1e-5)
                  and torch.allclose(bl.grad, db_ref[:, rows], rtol=1e-4, atol=1e-5)
                  and torch.allclose(al.grad, da_ref[:, rows], rtol=1e-4, atol=1e-5))
            if mode == "seqpar_fused":
                ok = ok and ops.calls == ["fwd", "bwd"]      # the fused branch ran, once per direction
        else:   # channel shards: no communication, each rank's slice equals the slice of the full result
            al, bl = fd.shard_channels(a, rank, world), fd.shard_channels(b, rank, world)
            assert al.data_ptr() == a[..., rank * (D // world):].data_ptr()      # a view, not a copy
            h = torch.from_numpy(oracle.scan_forward_f32(al.contiguous().numpy(), bl.contiguous().numpy()))
            ok = torch.equal(h, fd.shard_channels(h_ref, rank, world))
            parts = [torch.empty_like(h) for _ in range(world)]
            dist.all_gather(parts, h)          # only to check the re-assembled result, not part of the path
            ok = ok and torch.equal(torch.cat(parts, dim=-1), h_ref)
        Path(out_dir, f"rank{rank}.ok" if ok else f"rank{rank}.bad").write_text("x")
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("mode", ["seqpar", "seqpar_fused", "shards"])
def test_multi_rank_scan_matches_single_process(tmp_path, mode, world):
    if mode == "shards" and world == 3:
        world = 4      # 24 channels split evenly
    mp.spawn(_worker, args=(world, _free_port(), mode, str(tmp_path)), nprocs=world, join=True)
    assert sorted(p.name for p in tmp_path.iterdir()) == [f"rank{r}.ok" for r in range(world)]


def _absent_rank_worker(rank, world, port, out_dir):
    """Rank 1 leaves before the exchange (a host-side failure: it raises between steps, with nothing in
    flight); rank 0 must learn of it through the short process-group timeout of its all-gather instead
    of waiting forever."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    from fast_sequential_scan_b200 import distributed as fd
    gen = torch.Generator().manual_seed(5)
    a = 0.6 + 0.39 * torch.rand(1, 64, 8, generator=gen)
    b = torch.randn(1, 64, 8, generator=gen)
    try:
        if rank == 1:
            Path(out_dir, "rank1.left").write_text("x")
            return                                   # never joins the gather
        try:
            fd.seqpar_forward(a, b, None, OracleOps())
            Path(out_dir, "rank0.unnoticed").write_text("x")
        except Exception as e:                       # gloo reports the missing peer as a RuntimeError
            Path(out_dir, "rank0.detected").write_text(type(e).__name__)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_a_rank_that_skips_the_exchange_is_detected(tmp_path):
    mp.spawn(_absent_rank_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    names = sorted(p.name for p in tmp_path.iterdir())
    assert names == ["rank0.detected", "rank1.left"], names


def test_compose_rejects_a_rank_outside_the_world():
    """Argument checks of the carry composition need no device: a rank index outside the gathered
    table, or an empty world, is refused before anything is launched."""
    import ctypes
    from fast_sequential_scan_b200 import _lib
    L = _lib.lib()
    ctx = _lib.ScanCtx(ctypes.sizeof(_lib.ScanCtx), -1, None, None, 0, None, 0, 0)
    buf = (ctypes.c_float * 64)()
    ptr = ctypes.addressof(buf)
    assert L.fss_seqpar_compose(ctypes.byref(ctx), 0, 4, 4, 8, ptr, ptr) == -2      # rank == world
    assert L.fss_seqpar_compose(ctypes.byref(ctx), 0, 0, 0, 8, ptr, ptr) == -2      # empty world
    assert L.fss_seqpar_compose(ctypes.byref(ctx), 1, 4, -1, 8, ptr, ptr) == -2     # negative rank
    assert L.fss_seqpar_compose(ctypes.byref(ctx), 0, 4, 1, 8, None, ptr) == -1     # missing table
    assert L.fss_seqpar_compose(ctypes.byref(ctx), 0, 4, 1, 0, ptr, ptr) == 0       # nothing to do


def test_shard_channels_rejects_uneven_split():
    from fast_sequential_scan_b200 import distributed as fd
    with pytest.raises(ValueError):
        fd.shard_channels(torch.zeros(1, 4, 10), 0, 3)
