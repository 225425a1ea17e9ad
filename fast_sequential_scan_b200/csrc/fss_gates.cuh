// Gates of a real-gated linear recurrent unit (the RG-LRU of Hawk / Griffin, the use case the
// reference's README.md:3 names; the reference itself has no code for it -- its callers pass
// alpha and beta):
//     alpha = exp(c * sigmoid(r)),  c = -8 * softplus(lambda) per channel,
//     beta  = sqrt(1 - alpha^2) * sigmoid(i) * x.
// Gate<T> holds the arithmetic that the fused forward scan and the stand-alone gate kernels share,
// so that the alpha the backward multiplies with is bit for bit the alpha the forward scanned with.
#pragma once

#include "fss_common.cuh"

namespace fss {

// bf16 I/O rounds alpha and beta to 8 mantissa bits anyway, so it takes the one-instruction forms of
// the special-function unit (tanh.approx, ex2.approx, sqrt.approx: 4 per element); fp32 I/O uses the
// fp32 ex2 / rcp / sqrt approximations (5 per element), each within about 2^-22 relative.
template <typename T> struct Gate;
template <> struct Gate<bf16> {
    static __device__ __forceinline__ float sigmoid(float z) {
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * z));
        return fmaf(0.5f, t, 0.5f);
    }
    static __device__ __forceinline__ float prescale(float c) { return c * 1.4426950408889634f; }   // exp(z) = 2^(z log2 e)
    static __device__ __forceinline__ float exp_scaled(float z) {
        float r;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(z));
        return r;
    }
    static __device__ __forceinline__ float root(float z) {
        float r;
        asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(z));
        return r;
    }
};
template <> struct Gate<float> {
    // (tanh.approx, good to 2^-11, is not accurate enough for fp32 I/O)
    static __device__ __forceinline__ float sigmoid(float z) {
        float e, r;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * z));
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
        return r;
    }
    static __device__ __forceinline__ float prescale(float c) { return c * 1.4426950408889634f; }
    static __device__ __forceinline__ float exp_scaled(float z) {
        float r;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(z));
        return r;
    }
    static __device__ __forceinline__ float root(float z) {
        float r;
        asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(z));
        return r;
    }
};
__device__ __forceinline__ float gate_scale(float lambda) {      // -8 * softplus(lambda)
    return -8.0f * (lambda > 20.0f ? lambda : log1pf(expf(lambda)));
}
__device__ __forceinline__ float gate_scale_slope(float lambda) {      // d/dlambda of gate_scale: -8 * sigmoid(lambda)
    return -8.0f / (1.0f + expf(-lambda));
}

namespace gates {

constexpr int kThreads = 256;
constexpr int kRowsPerCta = 32;      // rows one CTA walks (bounds the partial sums it adds to dlambda)

// scales[d] = -8 * softplus(lambda[d]) * log2(e): the per-channel factor of the exponent, computed once
// per launch of the fused forward instead of once per tile
template <typename T>
__global__ void prescale(const float *__restrict__ lambda, float *__restrict__ scales, int64_t D) {
    const int64_t d = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (d < D) scales[d] = Gate<T>::prescale(gate_scale(lambda[d]));
}

// alpha (and beta when asked) as the fused forward scan computes them, rounded to T.
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
materialize(int64_t B, int64_t Tn, int64_t D, View<const T> r, View<const T> gi, View<const T> x,
            const float *__restrict__ lambda, View<T> alpha, View<T> beta, bool want_beta) {
    const int64_t nvec = D / V;
    const int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (v >= nvec) return;
    const int64_t d0 = v * V, b = blockIdx.z;
    float gsc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) gsc[k] = Gate<T>::prescale(gate_scale(lambda[d0 + k]));
    const int64_t t0 = (int64_t)blockIdx.y * kRowsPerCta, t1 = min(Tn, t0 + kRowsPerCta);
#pragma unroll 2
    for (int64_t t = t0; t < t1; ++t) {
        float rr[V], a[V];
        Frag<T, V>::load(r.row(b, t) + d0, rr);
#pragma unroll
        for (int k = 0; k < V; ++k) a[k] = Gate<T>::exp_scaled(gsc[k] * Gate<T>::sigmoid(rr[k]));
        Frag<T, V>::store(alpha.row(b, t) + d0, a);
        if (want_beta) {
            float ii[V], xx[V], bb[V];
            Frag<T, V>::load(gi.row(b, t) + d0, ii);
            Frag<T, V>::load(x.row(b, t) + d0, xx);
#pragma unroll
            for (int k = 0; k < V; ++k)
                bb[k] = Gate<T>::root(fmaf(-a[k], a[k], 1.0f)) * Gate<T>::sigmoid(ii[k]) * xx[k];
            Frag<T, V>::store(beta.row(b, t) + d0, bb);
        }
    }
}

// Chain rule through the gate formulas.  Inputs: the gradients of the scan with respect to alpha and
// beta.  Outputs: dr, di, dx (type T) and dlambda[D] (fp32, ACCUMULATED with atomic adds: the caller
// zeroes it).  The derivatives use the unrounded fp32 gate values.
//   ga = dalpha - dbeta * sigmoid(i) * x * alpha / sqrt(1 - alpha^2)      (beta depends on alpha too)
//   dr = ga * alpha * c * s(1 - s),  s = sigmoid(r);    dlambda += ga * alpha * s * dc/dlambda
//   di = dbeta * sqrt(1 - alpha^2) * x * u(1 - u),  u = sigmoid(i);   dx = dbeta * sqrt(1 - alpha^2) * u
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
backward(int64_t B, int64_t Tn, int64_t D, View<const T> r, View<const T> gi, View<const T> x,
         const float *__restrict__ lambda, View<const T> dalpha, View<const T> dbeta, View<T> dr, View<T> di,
         View<T> dx, float *__restrict__ dlambda) {
    const int64_t nvec = D / V;
    const int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (v >= nvec) return;
    const int64_t d0 = v * V, b = blockIdx.z;
    float c[V], gsc[V], slope[V], acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
        c[k] = gate_scale(lambda[d0 + k]);
        gsc[k] = Gate<T>::prescale(c[k]);
        slope[k] = gate_scale_slope(lambda[d0 + k]);
        acc[k] = 0.0f;
    }
    const int64_t t0 = (int64_t)blockIdx.y * kRowsPerCta, t1 = min(Tn, t0 + kRowsPerCta);
#pragma unroll 2
    for (int64_t t = t0; t < t1; ++t) {
        float rr[V], ii[V], xx[V], da[V], db[V], o_r[V], o_i[V], o_x[V];
        Frag<T, V>::load(r.row(b, t) + d0, rr);
        Frag<T, V>::load(gi.row(b, t) + d0, ii);
        Frag<T, V>::load(x.row(b, t) + d0, xx);
        Frag<T, V>::load(dalpha.row(b, t) + d0, da);
        Frag<T, V>::load(dbeta.row(b, t) + d0, db);
#pragma unroll
        for (int k = 0; k < V; ++k) {
            const float s = Gate<T>::sigmoid(rr[k]);
            const float a = Gate<T>::exp_scaled(gsc[k] * s);
            const float q = Gate<T>::root(fmaf(-a, a, 1.0f));
            const float u = Gate<T>::sigmoid(ii[k]);
            const float ga = da[k] - (q > 0.0f ? db[k] * u * xx[k] * a / q : 0.0f);
            const float gaa = ga * a;
            o_r[k] = gaa * c[k] * s * (1.0f - s);
            acc[k] = fmaf(gaa * s, slope[k], acc[k]);
            o_i[k] = db[k] * q * xx[k] * u * (1.0f - u);
            o_x[k] = db[k] * q * u;
        }
        Frag<T, V>::store(dr.row(b, t) + d0, o_r);
        Frag<T, V>::store(di.row(b, t) + d0, o_i);
        Frag<T, V>::store(dx.row(b, t) + d0, o_x);
    }
#pragma unroll
    for (int k = 0; k < V; ++k) atomicAdd(dlambda + d0 + k, acc[k]);
}

}  // namespace gates
}  // namespace fss
