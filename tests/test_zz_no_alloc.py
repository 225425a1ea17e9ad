"""The allocation-free forward scan, ``fss_scan_forward_noalloc``.

Some users of this library cannot hand it scratch memory: a plugin inside a host application
that owns all device memory, a loop that must stay clear of cudaMalloc's device-wide
synchronisation, a process whose memory budget is frozen.  For them the library keeps a fixed
scratch array inside its own image.  This test calls that entry point through the C ABI, twice
in a row on different data (the array is shared and keeps the previous call's contents), and
checks every element against the ordinary entry point that takes a caller-provided workspace.
Tolerance: the library's bf16 parity bound |x - ref| <= 1e-2 + 1e-2*|ref| (fp32: 1e-5); both
paths run the same chunked algorithm, so in practice they agree bit for bit.

The file name sorts last on purpose: if this test fails, a run that stops at the first failure
has already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(a, b, h, dtype_id):
    from fast_sequential_scan_b200 import _lib, sequential_scan_cuda as native
    L = _lib.lib()
    B, T, D = a.shape
    va, vb, vh = native._view(a), native._view(b), native._view(h)
    stream = torch.cuda.current_stream(a.device).cuda_stream
    return L.fss_scan_forward_noalloc(dtype_id, a.device.index, stream, B, T, D,
                                      ctypes.byref(va), ctypes.byref(vb), ctypes.byref(vh))


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
        err = (got.float() - want.float()).abs()
        bound = tol + tol * want.float().abs()
        assert bool((err <= bound).all()), f"call {call}: max excess {(err - bound).max().item()}"
    pkg.check_status()


def test_noalloc_rejects_problems_beyond_its_fixed_scratch():
    from fast_sequential_scan_b200 import _lib
    a = torch.zeros(1, 16, 8, dtype=torch.bfloat16, device="cuda")
    L = _lib.lib()
    v = _lib.View(a.data_ptr(), 8192 * 4096, 4096)     # strides of the large shape; never dereferenced
    # 64 x 8192 x 4096 needs far more than the 8 MiB array: refused before anything is launched
    rc = L.fss_scan_forward_noalloc(_lib.DTYPE_BF16, 0, None, 64, 8192, 4096,
                                    ctypes.byref(v), ctypes.byref(v), ctypes.byref(v))
    assert rc == -11 and b"fixed capacity" in L.fss_strerror(rc)
