"""Two-GPU (NCCL) run of the sequence-parallel scan; skipped on boxes with fewer than 2 GPUs.

Each rank holds its share of the rows and runs ``seqpar_scan`` (local zero-state scan, all-gather
of the carries over NCCL, re-scan of the blocks the carry reaches) forward and backward.  Every
rank then checks its rows of h, dalpha and dbeta against the CPU checker's undivided scan of the
whole sequence at the bf16 parity bound |x - ref| <= 1e-2 + 1e-2*|ref| (gradients formed from the
h the ranks stored, as the kernels do).
"""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_dir, exchange):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import fast_sequential_scan_b200 as pkg
        from fast_sequential_scan_b200 import distributed as fd
        gen = torch.Generator().manual_seed(77)                # same full problem on every rank
        B, T, D = 2, 4096 * world, 512
        a = (0.9 + 0.0999 * torch.rand(B, T, D, generator=gen)).bfloat16()
        b = torch.randn(B, T, D, generator=gen).bfloat16()
        g = torch.randn(B, T, D, generator=gen).bfloat16()
        rows = slice(rank * T // world, (rank + 1) * T // world)
        al = a[:, rows].cuda().requires_grad_(True)
        bl = b[:, rows].cuda().requires_grad_(True)
        ops = fd.NativeOps(exchange=exchange)
        for _ in range(2):                     # twice: the second step reuses buffers, slots and epochs
            al.grad = bl.grad = None
            h = fd.seqpar_scan(al, bl, None, ops)
            h.backward(g[:, rows].cuda())
        pkg.check_status()
        # the CPU checker on the whole, undivided sequence (every rank computes it for itself)
        from oracle import oracle
        h_ref, _, _ = oracle.reference_values(a, b, None)
        h_all = [torch.empty_like(h) for _ in range(world)]
        dist.all_gather(h_all, h.detach().contiguous())
        h_saved = torch.cat(h_all, dim=1).cpu()
        da_ref, db_ref = (torch.from_numpy(x) for x in oracle.scan_backward_f32(
            a.float().numpy(), h_saved.float().numpy(), g.float().numpy()))
        ok = True
        for got, ref in ((h, h_ref[:, rows]), (al.grad, da_ref[:, rows]), (bl.grad, db_ref[:, rows])):
            ok = ok and oracle.mixed_error_ratio(got, ref, 1e-2) <= 1.0
        Path(out_dir, f"rank{rank}.{'ok' if ok else 'bad'}").write_text("x")
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("exchange", ["collective", "peer"])
def test_sequence_parallel_scan_over_nccl(tmp_path, exchange):
    """``exchange``: the carries travel by NCCL all-gather, or through peer memory (plain stores into
    every GPU's table, bounded waits; NVLS is off in both)."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), exchange), nprocs=world, join=True)
    assert sorted(p.name for p in tmp_path.iterdir()) == [f"rank{r}.ok" for r in range(world)]
