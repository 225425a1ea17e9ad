/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement of the reference's sequential scan, used as the
 * parity checker by tests/, by the smoke check and by the bench's cpu_baseline leg.  The product
 * path (the CUDA library) never links, loads or calls anything in this file.
 *
 * Algorithm restated (reference project paths):
 *   forward   sequential_scan/common.py:46-59 (torch_ref): out[:,0]=beta[:,0]; for t>=1
 *             h = h*alpha[:,t] + beta[:,t]           -- alpha[:,0] is never read
 *   backward  PyTorch autograd through that loop; the closed form is the one the reference's
 *             own C++ loop states in csrc/include/sequential_scan_cpu.hpp:36-115:
 *               dh_{T-1} = g_{T-1};  dh_t = g_t + alpha_{t+1} * dh_{t+1}
 *               dbeta_t  = dh_t;     dalpha_t = dh_t * h_{t-1} (t>=1);  dalpha_0 = 0
 *
 * Parity pins: tests/test_oracle.py checks these functions bit-for-bit against the golden
 * vectors in tests/golden/ (produced by importing the reference's torch_ref, see
 * tests/golden/make_golden.py) and against oracle/_ref (the reference's C++ loop compiled from
 * its own header) when that library has been built.
 *
 * Compile with -ffp-contract=off: torch evaluates h*alpha+beta as a rounded multiply followed
 * by a rounded add, and the fp32 functions below must reproduce those bits.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#if defined(__GNUC__)
#define FSS_EXPORT __attribute__((visibility("default")))
#else
#define FSS_EXPORT
#endif

/* ---------------------------------------------------------------- bf16 helpers */

static inline float bf16_to_f32(uint16_t v) {
    uint32_t u = ((uint32_t)v) << 16;
    float f;
    memcpy(&f, &u, sizeof f);
    return f;
}

/* round-to-nearest-even, NaN kept quiet: the rounding torch and __float2bfloat16_rn use */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, sizeof u);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t bias = 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)((u + bias) >> 16);
}

FSS_EXPORT void fss_oracle_round_bf16(const float *src, uint16_t *dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16(src[i]);
}

FSS_EXPORT void fss_oracle_widen_bf16(const uint16_t *src, float *dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]);
}

/* ---------------------------------------------------------------- fp32 path */

/* common.py:46-59.  Tensors are contiguous [B, T, D], D fastest. */
FSS_EXPORT void fss_oracle_scan_forward_f32(const float *alpha, const float *beta, float *h,
                                            int64_t B, int64_t T, int64_t D) {
    for (int64_t b = 0; b < B; ++b) {
        const float *ab = alpha + b * T * D;
        const float *bb = beta + b * T * D;
        float *hb = h + b * T * D;
        for (int64_t d = 0; d < D; ++d) hb[d] = bb[d];            /* common.py:51 */
        for (int64_t t = 1; t < T; ++t) {                         /* common.py:55-57 */
            const float *hp = hb + (t - 1) * D;
            float *hc = hb + t * D;
            const float *ar = ab + t * D;
            const float *br = bb + t * D;
            for (int64_t d = 0; d < D; ++d) {
                float m = hp[d] * ar[d];
                hc[d] = m + br[d];
            }
        }
    }
}

/* sequential_scan_cpu.hpp:36-115 (same values as autograd through common.py:46-59). */
FSS_EXPORT void fss_oracle_scan_backward_f32(const float *alpha, const float *h, const float *g,
                                             float *dalpha, float *dbeta,
                                             int64_t B, int64_t T, int64_t D) {
    for (int64_t b = 0; b < B; ++b) {
        const int64_t base = b * T * D;
        for (int64_t d = 0; d < D; ++d) {
            float dh = 0.0f;
            for (int64_t t = T - 1; t >= 0; --t) {
                const int64_t i = base + t * D + d;
                if (t == T - 1) {
                    dh = g[i];
                } else {
                    float m = dh * alpha[i + D];
                    dh = m + g[i];
                }
                dbeta[i] = dh;
                dalpha[i] = (t >= 1) ? dh * h[i - D] : 0.0f;
            }
        }
    }
}

/* ---------------------------------------------------------------- bf16 I/O path
 * What a kernel with bf16 storage and fp32 state computes (the reference kernels'
 * arithmetic model, csrc/include/sequential_scan_kernel_bf16.cuh:84,139-144): inputs are
 * widened exactly, the recurrence state stays fp32, every stored value is rounded to bf16
 * once.  dalpha uses the *stored* (rounded) h, as the reference's saved tensor is the bf16
 * output (sequential_scan/scan_cuda.py:20).  fused != 0 evaluates a*h+b with a single
 * rounding (fmaf), which is what a GPU FMA does; fused == 0 rounds twice like torch on CPU.
 */
#include <math.h>

FSS_EXPORT void fss_oracle_scan_forward_bf16(const uint16_t *alpha, const uint16_t *beta,
                                             uint16_t *h, int64_t B, int64_t T, int64_t D,
                                             int fused) {
    for (int64_t b = 0; b < B; ++b) {
        const int64_t base = b * T * D;
        for (int64_t d = 0; d < D; ++d) {
            float s = 0.0f;
            for (int64_t t = 0; t < T; ++t) {
                const int64_t i = base + t * D + d;
                const float bv = bf16_to_f32(beta[i]);
                if (t == 0) {
                    s = bv;
                } else {
                    const float av = bf16_to_f32(alpha[i]);
                    if (fused) {
                        s = fmaf(av, s, bv);
                    } else {
                        float m = s * av;
                        s = m + bv;
                    }
                }
                h[i] = f32_to_bf16(s);
            }
        }
    }
}

FSS_EXPORT void fss_oracle_scan_backward_bf16(const uint16_t *alpha, const uint16_t *h,
                                              const uint16_t *g, uint16_t *dalpha,
                                              uint16_t *dbeta, int64_t B, int64_t T, int64_t D,
                                              int fused) {
    for (int64_t b = 0; b < B; ++b) {
        const int64_t base = b * T * D;
        for (int64_t d = 0; d < D; ++d) {
            float dh = 0.0f;
            for (int64_t t = T - 1; t >= 0; --t) {
                const int64_t i = base + t * D + d;
                const float gv = bf16_to_f32(g[i]);
                if (t == T - 1) {
                    dh = gv;
                } else {
                    const float av = bf16_to_f32(alpha[i + D]);
                    if (fused) {
                        dh = fmaf(av, dh, gv);
                    } else {
                        float m = dh * av;
                        dh = m + gv;
                    }
                }
                dbeta[i] = f32_to_bf16(dh);
                dalpha[i] = (t >= 1) ? f32_to_bf16(dh * bf16_to_f32(h[i - D])) : (uint16_t)0;
            }
        }
    }
}

/* ---------------------------------------------------------------- chunk algebra
 * The associative form the GPU path and the sequence-parallel mode rely on: rows [s,e) of a
 * column act on the incoming state as  h_{e-1} = P*h_{s-1} + C  with  P = prod a_t  and C the
 * rows scanned from a zero state; a row-0 chunk has P = 0 because alpha_0 is never read.
 * Used only by CPU tests of the host-side carry composition.
 */
FSS_EXPORT void fss_oracle_chunk_summary_f32(const float *alpha, const float *beta,
                                             float *prod, float *carry, int64_t T, int64_t D,
                                             int64_t row0, int64_t row1) {
    for (int64_t d = 0; d < D; ++d) {
        float p = 1.0f, c = 0.0f;
        for (int64_t t = row0; t < row1 && t < T; ++t) {
            const float av = (t == 0) ? 0.0f : alpha[t * D + d];
            p = p * av;
            float m = c * av;
            c = m + beta[t * D + d];
        }
        prod[d] = p;
        carry[d] = c;
    }
}
