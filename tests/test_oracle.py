"""Pins the CPU checker: the C restatement must reproduce, bit for bit, what the reference's
own ``torch_ref`` + autograd produced for the golden vectors (tests/golden/make_golden.py), and
must agree with the reference's C++ loop when that was compiled (oracle/_ref)."""
import numpy as np
import pytest
import torch

from conftest import golden_cases, load_golden
from oracle import oracle


@pytest.mark.parametrize("name", golden_cases())
def test_c_restatement_matches_reference_golden_bitwise(name):
    z = load_golden(name)
    h = oracle.scan_forward_f32(z["alpha"], z["beta"])
    assert np.array_equal(h.view(np.uint32), z["h"].view(np.uint32))
    da, db = oracle.scan_backward_f32(z["alpha"], z["h"], z["grad"])
    assert np.array_equal(db.view(np.uint32), z["dbeta"].view(np.uint32))
    assert np.array_equal(da.view(np.uint32), z["dalpha"].view(np.uint32))
    assert not da[:, 0].any()          # dalpha_0 = 0 exactly


@pytest.mark.parametrize("name", golden_cases("f32_"))
def test_torch_loop_autograd_matches_golden(name):
    z = load_golden(name)
    a = torch.from_numpy(z["alpha"]).requires_grad_(True)
    b = torch.from_numpy(z["beta"]).requires_grad_(True)
    h = oracle.torch_loop_scan(a, b)
    h.backward(torch.from_numpy(z["grad"]))
    assert torch.equal(h.detach(), torch.from_numpy(z["h"]))
    assert torch.equal(b.grad, torch.from_numpy(z["dbeta"]))
    da = a.grad if a.grad is not None else torch.zeros_like(a)
    assert torch.equal(da, torch.from_numpy(z["dalpha"]))


@pytest.mark.parametrize("name", golden_cases("bf16_"))
def test_bf16_storage_model_within_tolerance_of_golden(name):
    """fp32 state + one rounding per stored value stays inside the bf16 parity bound."""
    z = load_golden(name)
    a, b, g = (oracle.round_bf16(z[k]) for k in ("alpha", "beta", "grad"))
    assert np.array_equal(oracle.widen_bf16(a), z["alpha"])     # fixtures hold bf16-exact inputs
    for fused in (False, True):
        h = oracle.scan_forward_bf16(a, b, fused)
        da, db = oracle.scan_backward_bf16(a, h, g, fused)
        for got, key in ((h, "h"), (da, "dalpha"), (db, "dbeta")):
            r = oracle.mixed_error_ratio(torch.from_numpy(oracle.widen_bf16(got)),
                                         torch.from_numpy(z[key]), 1e-2)
            assert r <= 1.0, (key, fused, r)


def test_bf16_rounding_is_nearest_even():
    x = torch.randn(4096, generator=torch.Generator().manual_seed(3)) * 37.0
    x = torch.cat([x, torch.tensor([0.0, -0.0, 1.0, 1.00390625, 1.01171875, float("inf"), 3.3895e38])])
    got = oracle.round_bf16(x.numpy())
    want = x.bfloat16().view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got, want)
    assert np.array_equal(oracle.widen_bf16(got), x.bfloat16().float().numpy())


def test_empty_and_single_row():
    e = np.zeros((0, 5, 8), np.float32)
    assert oracle.scan_forward_f32(e, e).shape == (0, 5, 8)
    a = np.full((1, 1, 4), np.nan, np.float32)     # alpha_0 is never read
    b = np.arange(4, dtype=np.float32).reshape(1, 1, 4)
    assert np.array_equal(oracle.scan_forward_f32(a, b), b)


def test_chunk_summaries_compose_to_the_sequential_scan():
    gen = torch.Generator().manual_seed(11)
    T, D = 200, 12
    a = torch.rand(T, D, generator=gen).numpy() * 0.5 + 0.5
    b = torch.randn(T, D, generator=gen).numpy()
    h = oracle.scan_forward_f32(a[None], b[None])[0]
    state = np.zeros(D, np.float32)
    for r0 in range(0, T, 37):
        p, c = oracle.chunk_summary_f32(a, b, r0, min(T, r0 + 37))
        state = p * state + c
        assert np.allclose(state, h[min(T, r0 + 37) - 1], rtol=1e-5, atol=1e-6)


@pytest.mark.skipif(not oracle.RefLib.available(), reason="reference C++ loop not built")
@pytest.mark.parametrize("shape", [(2, 16, 8), (3, 37, 24), (2, 3, 8), (2, 128, 512)])
def test_restatement_matches_compiled_reference_loop(shape):
    gen = torch.Generator().manual_seed(5)
    a, b, g = (torch.randn(shape, generator=gen).numpy() for _ in range(3))
    job = oracle.RefLib().job(*shape)
    assert job is not None
    job.set(job.ALPHA, a); job.set(job.BETA, b); job.set(job.G, g)
    job.forward(threads=2)
    h = job.get(job.H)
    assert np.array_equal(h.view(np.uint32), oracle.scan_forward_f32(a, b).view(np.uint32))
    job.backward(threads=2)
    da, db = oracle.scan_backward_f32(a, h, g)
    assert np.array_equal(job.get(job.DBETA).view(np.uint32), db.view(np.uint32))
    assert np.array_equal(job.get(job.DALPHA).view(np.uint32), da.view(np.uint32))
    job.close()


def test_gate_formulas_of_the_oracle_against_torch():
    """float64 numpy gates == torch float64 gates, and the package's fp32 torch gates round to the
    same I/O values except where fp32 evaluation flips a rounding (rare, one unit in the last place)."""
    import torch
    from oracle import oracle
    gen = torch.Generator().manual_seed(2)
    r, i, x = (torch.randn(3, 50, 16, generator=gen) for _ in range(3))
    lam = -4.3 + 3.8 * torch.rand(16, generator=gen)
    a, b = oracle.gated_alpha_beta(r, i, x, lam)
    r64, i64, x64, l64 = (t.double() for t in (r, i, x, lam))
    a64 = torch.exp(-8.0 * torch.nn.functional.softplus(l64) * torch.sigmoid(r64))
    b64 = torch.sqrt(1 - a64 * a64) * torch.sigmoid(i64) * x64
    assert torch.equal(a, a64.float()) and torch.equal(b, b64.float())
    assert float(a.min()) > 0.0 and float(a.max()) < 1.0
    rb, ib, xb = (t.to(torch.bfloat16) for t in (r, i, x))
    ab, bb = oracle.gated_alpha_beta(rb, ib, xb, lam)
    assert ab.dtype == torch.bfloat16 and bb.dtype == torch.bfloat16


@pytest.mark.parametrize("name", golden_cases("f32_"))
def test_slice_assignment_loop_matches_golden(name):
    """The restatement with the reference's own operation sequence (a slice assignment per row,
    sequential_scan/common.py:46-59), which the bench times on the host cores, gives the golden
    values bit for bit."""
    z = load_golden(name)
    a = torch.from_numpy(z["alpha"]).requires_grad_(True)
    b = torch.from_numpy(z["beta"]).requires_grad_(True)
    h = oracle.torch_slice_scan(a, b)
    h.backward(torch.from_numpy(z["grad"]))
    assert torch.equal(h.detach(), torch.from_numpy(z["h"]))
    assert torch.equal(b.grad, torch.from_numpy(z["dbeta"]))
    da = a.grad if a.grad is not None else torch.zeros_like(a)
    assert torch.equal(da, torch.from_numpy(z["dalpha"]))


def test_state_carrying_oracle_against_autograd_of_the_loop():
    """reference_values_with_state (the C oracle on a sequence extended by one row) against autograd
    of the sequential loop started from h0, with a gradient for the final state."""
    gen = torch.Generator().manual_seed(0)
    B, T, D = 2, 50, 8
    a, b, g = torch.rand(B, T, D, generator=gen), torch.randn(B, T, D, generator=gen), torch.randn(B, T, D, generator=gen)
    h0, g_last = torch.randn(B, D, generator=gen), torch.randn(B, D, generator=gen)
    ar, br, h0r = (t.clone().requires_grad_() for t in (a, b, h0))
    state, rows = h0r, []
    for t in range(T):
        state = state * ar[:, t] + br[:, t]
        rows.append(state)
    h = torch.stack(rows, 1)
    torch.autograd.backward((h, h[:, -1]), (g, g_last))
    got = oracle.reference_values_with_state(a, b, g, h0, g_last)
    for x, y, what in zip(got, (h.detach(), h[:, -1].detach(), ar.grad, br.grad, h0r.grad),
                          ("h", "h_last", "dalpha", "dbeta", "dh0")):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6), what
    # without h0 it is the plain scan
    plain = oracle.reference_values_with_state(a, b, g)
    h_ref, da_ref, db_ref = oracle.reference_values(a, b, g)
    assert torch.equal(plain[0], h_ref) and torch.equal(plain[2], da_ref) and torch.equal(plain[3], db_ref)
    assert plain[4] is None
