// TEST INFRASTRUCTURE ONLY.  A C-ABI driver around the reference project's own CUDA kernels
// (csrc/include/sequential_scan_kernel.cuh and sequential_scan_kernel_bf16.cuh: the templates
// sequential_scan_forward[_half] / sequential_scan_backward[_half]).  Those headers are NOT
// copied here: the build recipe (oracle/build_oracle.py) passes -I<reference>/csrc/include and
// the result goes to oracle/_ref/libfss_refgpu.so.  Nothing in the product path loads it.  It
// serves two purposes: parity of the product kernels against what the reference itself computes
// on a GPU, and a like-for-like GPU timing of the reference beside the product's.
//
// The reference's launchers (csrc/sequential_scan_kernel.cu:7-268) are torch code; this file
// repeats only their launch geometry -- one CTA per batch row, d_model/4 (fp32) or d_model/8
// (bf16) threads, the five supported widths -- with raw pointers and a caller-chosen stream.
// Like the reference, the kernels need seq >= 2 (forward) / seq >= 3 (backward), contiguous
// [batch, seq, d_model] tensors and 32-bit element offsets.
#include <cstdint>

#include "sequential_scan_kernel.cuh"
#include "sequential_scan_kernel_bf16.cuh"

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {

enum { kOk = 0, kBadWidth = -1, kBadLength = -2, kTooLarge = -3, kLaunch = -4 };

int check(int64_t B, int64_t T, int64_t D, int64_t min_T) {
    if (D != 512 && D != 768 && D != 1024 && D != 1536 && D != 2048) return kBadWidth;
    if (T < min_T) return kBadLength;
    if (B < 1 || B * T * D > 0xffffffffLL) return kTooLarge;      // the kernels index with u_int
    return kOk;
}

int finish() { return cudaGetLastError() == cudaSuccess ? kOk : kLaunch; }

// expands to one case per width the reference launches (csrc/sequential_scan_kernel.cu:17-50)
#define REF_WIDTHS(X, PER) X(512, 512 / PER) X(768, 768 / PER) X(1024, 1024 / PER) X(1536, 1536 / PER) X(2048, 2048 / PER)

}  // namespace

REF_API int fss_refgpu_forward(float *alpha, float *beta, float *out, int64_t B, int64_t T, int64_t D, void *stream) {
    if (int rc = check(B, T, D, 2)) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    switch (D) {
#define X(DD, NT) case DD: sequential_scan_forward<DD, NT><<<(unsigned)B, NT, 0, s>>>(alpha, beta, out, (int)T); break;
        REF_WIDTHS(X, 4)
#undef X
    }
    return finish();
}

REF_API int fss_refgpu_backward(float *alpha, float *h, float *grad, float *dalpha, float *dbeta, int64_t B, int64_t T,
                                int64_t D, void *stream) {
    if (int rc = check(B, T, D, 3)) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    switch (D) {
#define X(DD, NT) case DD: sequential_scan_backward<DD, NT><<<(unsigned)B, NT, 0, s>>>(alpha, h, grad, dalpha, dbeta, (int)T); break;
        REF_WIDTHS(X, 4)
#undef X
    }
    return finish();
}

REF_API int fss_refgpu_forward_half(void *alpha, void *beta, void *out, int64_t B, int64_t T, int64_t D, void *stream) {
    if (int rc = check(B, T, D, 2)) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    switch (D) {
#define X(DD, NT) case DD: sequential_scan_forward_half<DD, NT><<<(unsigned)B, NT, 0, s>>>((bf16 *)alpha, (bf16 *)beta, (bf16 *)out, (int)T); break;
        REF_WIDTHS(X, 8)
#undef X
    }
    return finish();
}

// dbeta may be the same buffer as h: that is what the reference's launcher always does
// (csrc/sequential_scan_kernel.cu:197).
REF_API int fss_refgpu_backward_half(void *alpha, void *h, void *grad, void *dalpha, void *dbeta, int64_t B, int64_t T,
                                     int64_t D, void *stream) {
    if (int rc = check(B, T, D, 3)) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    switch (D) {
#define X(DD, NT) case DD: sequential_scan_backward_half<DD, NT><<<(unsigned)B, NT, 0, s>>>((bf16 *)alpha, (bf16 *)h, (bf16 *)grad, (bf16 *)dalpha, (bf16 *)dbeta, (int)T); break;
        REF_WIDTHS(X, 8)
#undef X
    }
    return finish();
}
