"""Generate the golden vectors in this directory from the reference implementation itself.

Imports the reference's ``sequential_scan/common.py`` *by file path* (its package ``__init__``
needs the compiled CUDA module) and runs ``torch_ref`` (common.py:46-59) on CPU, forward and --
through PyTorch autograd, as the reference's tests do (test_scan_cuda.py:47-72) -- backward.
Needs the reference checkout (``$FSS_REFERENCE_DIR`` or ``../reference`` beside the repository);
the committed ``*.npz`` files are what the test-suite reads, so this script only has to be run
again when cases are added:

    python tests/golden/make_golden.py
"""
from __future__ import annotations

import importlib.util
import os
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load_reference_common():
    root = Path(os.environ.get("FSS_REFERENCE_DIR", HERE.parent.parent.parent / "reference"))
    path = root / "sequential_scan" / "common.py"
    spec = importlib.util.spec_from_file_location("reference_common", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def gates(kind: str, shape, gen):
    """Input distributions of the benchmark configurations plus the reference tests' randn."""
    n = lambda: torch.randn(shape, generator=gen)
    if kind == "sigmoid":          # a = sigmoid(N(0,1))
        return torch.sigmoid(n()), n(), n()
    if kind == "randn":            # reference tests: alpha, beta ~ N(0,1), unbounded
        return n(), n(), n()
    if kind == "uniform":          # a ~ U(0.5, 0.999)
        return 0.5 + 0.499 * torch.rand(shape, generator=gen), n(), n()
    if kind == "hawk":             # RG-LRU shaped gates
        lam = -4.3 + 3.8 * torch.rand(shape[-1], generator=gen)
        a = torch.exp(-8.0 * torch.nn.functional.softplus(lam) * torch.sigmoid(n()))
        b = torch.sqrt(1 - a * a) * torch.sigmoid(n()) * n()
        return a, b, n()
    raise ValueError(kind)


CASES = [
    # name, B, T, D, gates, io dtype
    ("f32_tiny", 2, 16, 8, "sigmoid", "f32"),
    ("f32_t1", 3, 1, 8, "randn", "f32"),
    ("f32_t2", 2, 2, 8, "randn", "f32"),
    ("f32_t3", 2, 3, 8, "randn", "f32"),
    ("f32_odd", 3, 37, 24, "randn", "f32"),
    ("f32_uniform", 2, 300, 16, "uniform", "f32"),
    ("f32_hawk", 2, 257, 16, "hawk", "f32"),
    ("f32_ref_seq128", 2, 128, 32, "randn", "f32"),
    ("bf16_tiny", 2, 16, 8, "sigmoid", "bf16"),
    ("bf16_odd", 3, 37, 24, "randn", "bf16"),
    ("bf16_uniform", 2, 1000, 16, "uniform", "bf16"),
    ("bf16_hawk", 2, 513, 16, "hawk", "bf16"),
    # configuration 1 (B2 T1024 D768), first 8 channels only: channels are independent
    ("bf16_cfg1_ch8", 2, 1024, 8, "sigmoid", "bf16"),
    ("f32_cfg1_ch8", 2, 1024, 8, "sigmoid", "f32"),
]


def main() -> None:
    ref = load_reference_common()
    for idx, (name, B, T, D, kind, io) in enumerate(CASES):
        gen = torch.Generator().manual_seed(1000 + idx)
        a, b, g = gates(kind, (B, T, D), gen)
        if io == "bf16":   # inputs as the kernel sees them: rounded to bf16, then exact in fp32
            a, b, g = (x.bfloat16().float() for x in (a, b, g))
        a.requires_grad_(True)
        b.requires_grad_(True)
        h = ref.torch_ref(a, b)
        h.backward(g)
        # with a single row alpha is never read, so autograd leaves its gradient unset (= zero)
        da = a.grad if a.grad is not None else torch.zeros_like(a)
        out = dict(alpha=a.detach().numpy(), beta=b.detach().numpy(), grad=g.numpy(),
                   h=h.detach().numpy(), dalpha=da.numpy(), dbeta=b.grad.numpy())
        if io == "bf16":
            # the reference's own test oracle for bf16: torch_ref evaluated IN bf16
            # (test_scan_cuda.py:83-94); kept as a side metric
            hb = ref.torch_ref(a.detach().bfloat16(), b.detach().bfloat16())
            out["h_bf16_loop"] = hb.float().numpy()
        np.savez_compressed(HERE / f"{name}.npz", io=np.array(io), gates=np.array(kind), **out)
        print(f"{name}: B{B} T{T} D{D} {kind} {io}")


if __name__ == "__main__":
    main()
