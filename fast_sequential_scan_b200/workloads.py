"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (the reference's own benchmark draws ``randn`` alpha/beta and ``0.1*randn``
upstream gradients, benchmark.py:10-14,63; its tests draw ``randn`` for both,
sequential_scan/common.py:20-43).  No dataset is involved: every tensor is generated.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    batch: int
    seq: int
    d_model: int
    gates: str            # sigmoid | uniform_0.5 | uniform_0.9 | hawk | randn
    dtype: str = "bf16"   # bf16 | f32

    @property
    def elems(self) -> int:
        return self.batch * self.seq * self.d_model

    @property
    def torch_dtype(self) -> torch.dtype:
        return torch.bfloat16 if self.dtype == "bf16" else torch.float32

    def bytes_per_elem(self, backward: bool = True, forward: bool = True) -> int:
        """Algorithmic bytes: forward reads alpha, beta and writes h (3 tensors); backward reads
        alpha, h, grad and writes dalpha, dbeta (5 tensors)."""
        w = 2 if self.dtype == "bf16" else 4
        return w * ((3 if forward else 0) + (5 if backward else 0))


CONFIGS = {
    "c1": Workload("c1", 2, 1024, 768, "sigmoid"),
    "c2": Workload("c2", 8, 2048, 1024, "sigmoid"),
    "c3_512": Workload("c3_512", 4, 512, 2048, "uniform_0.5"),
    "c3_1000": Workload("c3_1000", 4, 1000, 2048, "uniform_0.5"),
    "c3_3000": Workload("c3_3000", 4, 3000, 2048, "uniform_0.5"),
    "c3_4096": Workload("c3_4096", 4, 4096, 2048, "uniform_0.5"),
    "c3_8192": Workload("c3_8192", 4, 8192, 2048, "uniform_0.5"),
    "c4_bf16": Workload("c4_bf16", 16, 4096, 2560, "hawk"),
    "c4_f32": Workload("c4_f32", 16, 4096, 2560, "hawk", "f32"),
    # one rank's share (65,536 rows) of the 524,288-row sequence-parallel configuration
    "c5_rank": Workload("c5_rank", 1, 65536, 4096, "uniform_0.9"),
}


def make_inputs(w: Workload, device="cpu", seed: int = 0, shape=None
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(alpha, beta, grad) of the workload's I/O dtype, generated in fp32 on ``device``."""
    shape = tuple(shape) if shape is not None else (w.batch, w.seq, w.d_model)
    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed)
    n = lambda s=shape: torch.randn(s, generator=gen, device=dev)
    u = lambda s=shape: torch.rand(s, generator=gen, device=dev)
    if w.gates == "sigmoid":
        a = torch.sigmoid(n()); b = n()
    elif w.gates == "uniform_0.5":
        a = 0.5 + 0.499 * u(); b = n()
    elif w.gates == "uniform_0.9":
        a = 0.9 + 0.0999 * u(); b = n()
    elif w.gates == "hawk":
        lam = -4.3 + 3.8 * u((shape[-1],))
        a = torch.exp(-8.0 * torch.nn.functional.softplus(lam) * torch.sigmoid(n()))
        b = torch.sqrt(1 - a * a) * torch.sigmoid(n()) * n()
    elif w.gates == "randn":
        a = n(); b = n()
    else:
        raise ValueError(w.gates)
    g = n()
    dt = w.torch_dtype
    return a.to(dt), b.to(dt), g.to(dt)


def make_gate_inputs(w: Workload, device="cpu", seed: int = 0, shape=None):
    """(r, i, x, lam) for the gated forward of a workload's shape: the raw quantities the "hawk"
    gates of :func:`make_inputs` are computed from (lam ~ U(-4.3, -0.5) per channel, r, i, x ~ N(0, 1))."""
    shape = tuple(shape) if shape is not None else (w.batch, w.seq, w.d_model)
    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed)
    lam = -4.3 + 3.8 * torch.rand((shape[-1],), generator=gen, device=dev)
    r, i, x = (torch.randn(shape, generator=gen, device=dev).to(w.torch_dtype) for _ in range(3))
    return r, i, x, lam
