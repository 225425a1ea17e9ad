"""The product kernels against the reference project's own CUDA kernels, run on the same GPU.

``oracle/_ref/libfss_refgpu.so`` holds the reference's kernel templates
(csrc/include/sequential_scan_kernel.cuh, sequential_scan_kernel_bf16.cuh) compiled for sm_100a
behind a C ABI with the reference's launch geometry (csrc/sequential_scan_kernel.cu:7-268); it is
built by ``oracle/build_oracle.py`` where the reference checkout is present and travels with the
tree.  Shapes are the reference's own test grid (sequential_scan/test_scan_cuda.py:27-29, 80-82)
plus its benchmark shape.

fp32: the two implementations differ only in summation order and contraction, so they are held to
the fp32 parity bound against each other on gate-like inputs, and to the reference's own 7-digit
relative-L2 metric on its randn inputs.
bf16: the forward kernels both keep an fp32 state and round once per stored value -> bf16 parity
bound.  The reference's bf16 backward re-rounds its carry to bf16 at every step
(csrc/include/sequential_scan_kernel_bf16.cuh:286), the product keeps it in fp32, so gradients are
compared with the reference's own metric for that kernel, 2 digits of relative L2
(sequential_scan/test_scan_cuda.py:19), and both are compared with the CPU checker.
"""
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def refgpu():
    if not oracle.RefGpu.available():
        pytest.skip("oracle/_ref/libfss_refgpu.so was not built (needs the reference checkout and nvcc)")
    return oracle.RefGpu()


def _inputs(shape, dtype, gates):
    gen = torch.Generator(device="cuda").manual_seed(sum(shape))
    a = torch.randn(shape, generator=gen, device="cuda")
    a = torch.sigmoid(a) if gates else a
    b = torch.randn(shape, generator=gen, device="cuda")
    g = torch.randn(shape, generator=gen, device="cuda")
    return a.to(dtype), b.to(dtype), g.to(dtype)


@pytest.mark.parametrize("bs", [2, 9, 12])
@pytest.mark.parametrize("sq", [128, 512, 1024])
@pytest.mark.parametrize("d", [512, 768, 1024, 1536, 2048])
def test_fp32_kernels_agree_with_the_reference_kernels(refgpu, bs, sq, d):
    import fast_sequential_scan_b200 as pkg
    from fast_sequential_scan_b200 import sequential_scan_cuda as native
    a, b, g = _inputs((bs, sq, d), torch.float32, gates=True)
    h_ref = refgpu.forward(a, b)
    da_ref, db_ref = refgpu.backward(a, h_ref, g)
    h = native.scan_forward(a, b)
    da, db = native.scan_backward(a, h_ref, g)              # same saved h for both backward kernels
    pkg.check_status()
    for got, ref, what in ((h, h_ref, "h"), (da, da_ref, "dalpha"), (db, db_ref, "dbeta")):
        r = oracle.mixed_error_ratio(got, ref, 1e-5)
        assert r <= 1.0, f"{what}: ratio {r:.3f} against the reference's fp32 kernel"
    # the reference's own input distribution (randn alpha) and metric
    a, b, g = _inputs((bs, sq, d), torch.float32, gates=False)
    h_ref = refgpu.forward(a, b)
    h = native.scan_forward(a, b)
    assert oracle.digits(oracle.relative_l2(h, h_ref)) >= 7 or not bool(torch.isfinite(h_ref).all())


@pytest.mark.parametrize("bs", [1, 7, 15])
@pytest.mark.parametrize("sq", [128, 512, 1024])
@pytest.mark.parametrize("d", [512, 768, 1024, 1536, 2048])
def test_bf16_kernels_agree_with_the_reference_kernels(refgpu, bs, sq, d):
    import fast_sequential_scan_b200 as pkg
    from fast_sequential_scan_b200 import sequential_scan_cuda as native
    a, b, g = _inputs((bs, sq, d), torch.bfloat16, gates=True)
    h_ref = refgpu.forward(a, b)
    h = native.scan_forward_half(a, b)
    r = oracle.mixed_error_ratio(h, h_ref.float(), 1e-2)
    assert r <= 1.0, f"h: ratio {r:.3f} against the reference's bf16 kernel"
    da_ref, db_ref = refgpu.backward(a, h_ref, g)           # separate grad_beta buffer: h_ref stays intact
    da, db = native.scan_backward_half(a, h_ref, g)
    pkg.check_status()
    o_da, o_db = (torch.from_numpy(x) for x in oracle.scan_backward_f32(
        a.float().cpu().numpy(), h_ref.float().cpu().numpy(), g.float().cpu().numpy()))
    for got, ref, what in ((da, da_ref, "dalpha"), (db, db_ref, "dbeta")):
        assert oracle.digits(oracle.relative_l2(got, ref.float())) >= 2, what
    # against the CPU checker the product (fp32 carry) must be inside the parity bound, and it must
    # be at least as close as the reference's kernel (bf16 carry)
    for got, refk, orc, what in ((da, da_ref, o_da, "dalpha"), (db, db_ref, o_db, "dbeta")):
        assert oracle.mixed_error_ratio(got, orc, 1e-2) <= 1.0, what
        assert oracle.relative_l2(got, orc) <= oracle.relative_l2(refk, orc) * 1.05 + 1e-6, what


def test_benchmark_shape_and_the_reference_aliasing(refgpu):
    """bs 8, seq 2048, d_model 1024 (the shape of the reference's own benchmark, benchmark.py:43,93-98):
    forward parity, and the reference launcher's habit of writing grad_beta over the saved h
    (csrc/sequential_scan_kernel.cu:197) reproduced on both sides."""
    from fast_sequential_scan_b200 import sequential_scan_cuda as native
    a, b, g = _inputs((8, 2048, 1024), torch.bfloat16, gates=True)
    h_ref = refgpu.forward(a, b)
    h = native.scan_forward_half(a, b)
    assert oracle.mixed_error_ratio(h, h_ref.float(), 1e-2) <= 1.0
    keep = h_ref.clone()
    da_ref, db_ref = refgpu.backward(a, h_ref, g, dbeta=h_ref)          # aliased, like the reference
    assert db_ref.data_ptr() == h_ref.data_ptr()
    da, db = native.scan_backward_half(a, keep.clone(), g, inplace_grad_beta=True)
    assert oracle.digits(oracle.relative_l2(db, db_ref.float())) >= 2
    assert oracle.digits(oracle.relative_l2(da, da_ref.float())) >= 2
