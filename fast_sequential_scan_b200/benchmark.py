"""Sequence-length sweep of ``scan_cu``: the harness of the reference's ``benchmark.py`` for this
package (same flags, same shapes, same statistic).

    python -m fast_sequential_scan_b200.benchmark --d_model 1024 --bs 8 --plot_name bs_8_dmodel_1024 [--fwd_only]

Reference behaviour kept (benchmark.py:20-110): ``randn`` bf16 alpha/beta with ``requires_grad``,
upstream gradient ``0.1*randn``, sequence lengths 128 ... 32768, forward+backward timed unless
``--fwd_only`` is given, median of repeated runs in milliseconds.  Dropped: the Triton and
``accelerated_scan`` providers (not part of this package) and the matplotlib plot -- the table is
printed and written as ``<plot_name>.csv``.
"""
from __future__ import annotations

import argparse
import statistics

import torch

from . import scan_cu

SEQ_LENS = [128, 256, 1024, 2048, 4096, 8192, 16384, 32768]      # benchmark.py:43


def create_tensor(bs: int, sq: int, d_model: int) -> torch.Tensor:
    return torch.randn((bs, sq, d_model), device="cuda:0", dtype=torch.bfloat16, requires_grad=True)


def do_bench(fn, rep_ms: float = 100.0, warmup_ms: float = 25.0) -> float:
    """Median run time in ms: repeat ``fn`` for about ``rep_ms`` of device time, one CUDA-event pair
    per run, an L2-sized buffer cleared between runs."""
    flush = torch.empty(256 << 20, dtype=torch.int8, device="cuda:0")
    fn(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        fn()
    e1.record(); torch.cuda.synchronize()
    est = max(e0.elapsed_time(e1) / 5, 1e-3)
    for _ in range(max(1, int(warmup_ms / est))):
        fn()
    times = []
    for _ in range(max(5, min(1000, int(rep_ms / est)))):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return statistics.median(times)


def main() -> None:
    ap = argparse.ArgumentParser(description="Run the scan benchmark.")
    ap.add_argument("--d_model", type=int, required=True, help="Model dimension")
    ap.add_argument("--bs", type=int, required=True, help="Batch size")
    ap.add_argument("--plot_name", type=str, required=True, help="Name for the output table")
    ap.add_argument("--fwd_only", action="store_true", help="Time the forward pass only")
    args = ap.parse_args()

    rows = []
    for sq in SEQ_LENS:
        alpha, beta = create_tensor(args.bs, sq, args.d_model), create_tensor(args.bs, sq, args.d_model)
        dy = 0.1 * torch.randn_like(alpha)

        def y_fwd():
            return scan_cu(alpha, beta)

        def y_fwd_bwd():
            alpha.grad = beta.grad = None
            y_fwd().backward(dy)

        ms = do_bench(y_fwd if args.fwd_only else y_fwd_bwd)
        elems = args.bs * sq * args.d_model
        gbs = elems * (6 if args.fwd_only else 16) / (ms * 1e-3) / 1e9
        rows.append((sq, ms, gbs))
        print(f"sq={sq:6d}  cuda-bf16 {ms:9.4f} ms   {gbs:8.1f} GB/s algorithmic")
    with open(f"{args.plot_name}.csv", "w") as f:
        f.write("sq,cuda-bf16_ms,algorithmic_GBps\n")
        for sq, ms, gbs in rows:
            f.write(f"{sq},{ms:.6f},{gbs:.2f}\n")


if __name__ == "__main__":
    main()
