"""Two-GPU (NCCL) run of the sequence-parallel scan; skipped on boxes with fewer than 2 GPUs.

Each rank holds half of the rows, runs ``seqpar_scan`` (local zero-state scan, all-gather of the
carries over NCCL, re-scan of the blocks the carry reaches) forward and backward; rank 0 also
computes the undivided scan on its own GPU, and both are compared with the bf16 parity bound.
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


def _worker(rank, world, port, out_dir):
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
        h = fd.seqpar_scan(al, bl)
        h.backward(g[:, rows].cuda())
        pkg.check_status()
        # the undivided scan on this rank's own GPU
        af = a.cuda().requires_grad_(True)
        bf = b.cuda().requires_grad_(True)
        hf = pkg.scan_cu(af, bf)
        hf.backward(g.cuda())
        ok = True
        for got, ref in ((h, hf[:, rows]), (al.grad, af.grad[:, rows]), (bl.grad, bf.grad[:, rows])):
            err = (got.float() - ref.float()).abs()
            ok = ok and bool((err <= 2e-2 + 2e-2 * ref.float().abs()).all())   # two bf16 results compared
        Path(out_dir, f"rank{rank}.{'ok' if ok else 'bad'}").write_text("x")
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_sequence_parallel_scan_over_nccl(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(p.name for p in tmp_path.iterdir()) == [f"rank{r}.ok" for r in range(world)]
