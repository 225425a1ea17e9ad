"""The allocation-free forward scan, ``fss_scan_forward_noalloc``.

Some users of this library cannot hand it scratch memory: a plugin inside a host application
that owns all device memory, a loop that must stay clear of cudaMalloc's device-wide
synchronisation, a process whose memory budget is frozen.  For them the library keeps a fixed
scratch array inside its own image.  This test calls that entry point through the C ABI, twice
in a row on different data (the array is shared and keeps the previous call's contents), and
checks every element against the ordinary entry point that takes a caller-provided workspace
and against the CPU checker.
Tolerance: the library's bf16 parity bound |x - ref| <= 1e-2 + 1e-2*|ref| (fp32: 1e-5); both
entry points run the same chunked algorithm, so in practice they agree bit for bit.

The file name sorts last on purpose: if this test fails, a run that stops at the first failure
has already executed every other test.
"""
import ctypes

import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def _call_noalloc(a, b, h, dtype_id, device=None):
    from fast_sequential_scan_b200 import _lib, sequential_scan_cuda as native
    L = _lib.lib()
    B, T, D = a.shape
    va, vb, vh = native._view(a), native._view(b), native._view(h)
    stream = torch.cuda.current_stream(a.device).cuda_stream
    return L.fss_scan_forward_noalloc(dtype_id, a.device.index if device is None else device, stream, B, T, D,
                                      ctypes.byref(va), ctypes.byref(vb), ctypes.byref(vh))


def _within(got, want, tol):
    err = (got.float() - want.float()).abs()
    return bool((err <= tol + tol * want.float().abs()).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_matches_workspace_entry_point_on_two_consecutive_calls(dtype):
    from fast_sequential_scan_b200 import _lib, sequential_scan_cuda as native
    import fast_sequential_scan_b200 as pkg
    dtype_id = _lib.DTYPE_BF16 if dtype == torch.bfloat16 else _lib.DTYPE_F32
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    gen = torch.Generator(device="cuda").manual_seed(21)
    shape = (3, 700, 264)                      # not a multiple of the chunk length, 3 batches
    for call in range(2):                      # second call: new data, same shared scratch
        a = torch.sigmoid(torch.randn(shape, generator=gen, device="cuda")).to(dtype)
        b = (torch.randn(shape, generator=gen, device="cuda") * (call + 1)).to(dtype)
        want = torch.empty_like(a)
        native.forward_into(a, b, want, algo=_lib.ALGO_CHUNKED)
        got = torch.full_like(a, float("nan"))
        rc = _call_noalloc(a, b, got, dtype_id)
        assert rc == 0, _lib.lib().fss_strerror(rc)
        torch.cuda.synchronize()
        assert _within(got, want, tol), f"call {call}: differs from the workspace entry point"
        ref, _, _ = oracle.reference_values(a, b, None)
        assert _within(got.cpu(), ref, tol), f"call {call}: differs from the CPU checker"
    pkg.check_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_on_layouts_that_need_the_element_wise_path(dtype):
    """Odd d_model (no 16-byte vectors), a channel-sliced strided view, and device = -1 (the calling
    thread's current device): the paths the contiguous, vector-friendly shape above never takes."""
    from fast_sequential_scan_b200 import _lib
    dtype_id = _lib.DTYPE_BF16 if dtype == torch.bfloat16 else _lib.DTYPE_F32
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    gen = torch.Generator(device="cuda").manual_seed(22)
    # (2, 50, 7): one element per thread
    a = torch.sigmoid(torch.randn(2, 50, 7, generator=gen, device="cuda")).to(dtype)
    b = torch.randn(2, 50, 7, generator=gen, device="cuda").to(dtype)
    got = torch.full_like(a, float("nan"))
    assert _call_noalloc(a, b, got, dtype_id, device=-1) == 0
    torch.cuda.synchronize()
    assert _within(got.cpu(), oracle.reference_values(a, b, None)[0], tol)
    # channel slice [.., 8:136] of a wider tensor, output into a slice as well
    wide_a = torch.sigmoid(torch.randn(3, 300, 160, generator=gen, device="cuda")).to(dtype)
    wide_b = torch.randn(3, 300, 160, generator=gen, device="cuda").to(dtype)
    wide_h = torch.full_like(wide_a, -7.0)
    a, b, h = wide_a[..., 8:136], wide_b[..., 8:136], wide_h[..., 8:136]
    assert _call_noalloc(a, b, h, dtype_id) == 0
    torch.cuda.synchronize()
    assert _within(h.cpu(), oracle.reference_values(a.contiguous(), b.contiguous(), None)[0], tol)
    assert bool((wide_h[..., :8] == -7.0).all()) and bool((wide_h[..., 136:] == -7.0).all())


def test_noalloc_rejects_problems_beyond_its_fixed_scratch():
    from fast_sequential_scan_b200 import _lib
    a = torch.zeros(1, 16, 8, dtype=torch.bfloat16, device="cuda")
    L = _lib.lib()
    v = _lib.View(a.data_ptr(), 8192 * 4096, 4096)     # strides of the large shape; never dereferenced
    # 64 x 8192 x 4096 needs far more than the 8 MiB array: refused before anything is launched
    rc = L.fss_scan_forward_noalloc(_lib.DTYPE_BF16, 0, None, 64, 8192, 4096,
                                    ctypes.byref(v), ctypes.byref(v), ctypes.byref(v))
    assert rc == -11 and b"fixed capacity" in L.fss_strerror(rc)


def test_noalloc_capacity_boundary():
    """The largest problem the fixed array serves is accepted and correct; one chunk more is refused.
    With 16-row chunks (short sequences) the scratch holds 8*B*D*ceil(T/16) bytes."""
    from fast_sequential_scan_b200 import _lib
    L = _lib.lib()
    cap = 8 << 20
    B, D = 64, 1024
    chunk = int(L.fss_block_rows(_lib.DTYPE_F32, B, 32, D, _lib.ALGO_CHUNKED))
    assert chunk == 16
    chunks = cap // (8 * B * D)                       # 16 chunks fill the array exactly
    T_fit = chunks * chunk
    assert int(L.fss_block_rows(_lib.DTYPE_F32, B, T_fit, D, _lib.ALGO_CHUNKED)) == chunk
    gen = torch.Generator(device="cuda").manual_seed(23)
    a = torch.sigmoid(torch.randn(B, T_fit + chunk, D, generator=gen, device="cuda"))
    b = torch.randn(B, T_fit + chunk, D, generator=gen, device="cuda")
    fit_a, fit_b = a[:, :T_fit].contiguous(), b[:, :T_fit].contiguous()
    got = torch.full_like(fit_a, float("nan"))
    assert _call_noalloc(fit_a, fit_b, got, _lib.DTYPE_F32) == 0
    torch.cuda.synchronize()
    assert _within(got.cpu(), oracle.reference_values(fit_a, fit_b, None)[0], 1e-5)
    too = torch.empty_like(a)
    assert _call_noalloc(a, b, too, _lib.DTYPE_F32) == -11
