// FSS_ALGO_CHUNKED: the any-layout path.  Three plain launches, no inter-CTA waiting:
//   1. chunk_summary  -- every chunk of L rows, scanned from a zero state, reduced to the affine
//                        map (P, C): state_out = P*state_in + C            (reads 2 tensors)
//   2. chunk_compose  -- one thread per column folds the maps in order; leaves the state that
//                        enters each chunk, and the running product, in the workspace
//   3. chunk_scan     -- every chunk re-scanned from its true entering state, results stored
// The forward state is h; the backward state is u_t = a_t*dh_t, the quantity row t hands to row
// t-1, so both directions use the same maps and the backward needs no shifted alpha row.
// One thread owns V consecutive channels (16 bytes when the layout allows, else 1 element).
#pragma once

#include "fss_common.cuh"

namespace fss {
namespace chunked {

constexpr int kThreads = 128;

struct Geometry {
    int64_t B, T, D;
    int64_t L;      // rows per chunk
    int64_t S;      // chunks per column
    int64_t nvec;   // channel groups per row
    int64_t vblocks;  // CTAs along the channel axis
};

// linear block id -> (channel block, chunk, batch)
__device__ __forceinline__ void decode_block(const Geometry &g, int64_t &vb, int64_t &s, int64_t &b) {
    int64_t id = blockIdx.x;
    vb = id % g.vblocks; id /= g.vblocks;
    s = id % g.S;
    b = id / g.S;
}

// ---------------------------------------------------------------- 1. summaries
template <typename T, int V, bool kBackward>
__global__ void __launch_bounds__(kThreads)
chunk_summary(Geometry g, View<const T> alpha, View<const T> other /* beta | grad */,
              float *__restrict__ wsP, float *__restrict__ wsC, bool continuation) {
    int64_t vb, s, b;
    decode_block(g, vb, s, b);
    const int64_t v = vb * kThreads + threadIdx.x;
    if (v >= g.nvec) return;
    const int64_t d0 = v * V;
    const int64_t r0 = s * g.L;
    const int64_t r1 = min(g.T, r0 + g.L);

    float P[V], C[V];
#pragma unroll
    for (int i = 0; i < V; ++i) { P[i] = 1.0f; C[i] = 0.0f; }

    if (!kBackward) {
#pragma unroll 4
        for (int64_t t = r0; t < r1; ++t) {
            float a[V], x[V];
            Frag<T, V>::load(alpha.row(b, t) + d0, a);
            Frag<T, V>::load(other.row(b, t) + d0, x);
            const bool head = (t == 0) && !continuation;   // alpha_0 is never read
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const float av = head ? 0.0f : a[i];
                P[i] *= av;
                C[i] = fmaf(av, C[i], x[i]);
            }
        }
    } else {
#pragma unroll 4
        for (int64_t t = r1 - 1; t >= r0; --t) {
            float a[V], x[V];
            Frag<T, V>::load(alpha.row(b, t) + d0, a);
            Frag<T, V>::load(other.row(b, t) + d0, x);
            const bool head = (t == 0) && !continuation;
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const float av = head ? 0.0f : a[i];
                P[i] *= av;
                C[i] = av * (x[i] + C[i]);                 // u_t = a_t * (g_t + u_{t+1})
            }
        }
    }
    const int64_t o = (b * g.S + s) * g.D + d0;
#pragma unroll
    for (int i = 0; i < V; ++i) { wsP[o + i] = P[i]; wsC[o + i] = C[i]; }
}

// ---------------------------------------------------------------- 2. composition
// In place: wsC[chunk] becomes the state entering that chunk, wsP[chunk] the product of alpha
// from the scan's starting end through that chunk.  block_prod receives each chunk's own product,
// block_state the state leaving it.
template <bool kBackward>
__global__ void chunk_compose(Geometry g, float *__restrict__ wsP, float *__restrict__ wsC,
                              const float *__restrict__ state_in, float *__restrict__ state_out,
                              float *__restrict__ prod_out, float *__restrict__ block_prod,
                              float *__restrict__ block_state) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= g.B * g.D) return;
    const int64_t b = idx / g.D, d = idx % g.D;
    float carry = state_in ? state_in[idx] : 0.0f;
    float run = 1.0f;
#pragma unroll 4
    for (int64_t k = 0; k < g.S; ++k) {
        const int64_t s = kBackward ? g.S - 1 - k : k;
        const int64_t o = (b * g.S + s) * g.D + d;
        const float p = wsP[o], c = wsC[o];
        wsC[o] = carry;
        carry = (carry == 0.0f) ? c : fmaf(p, carry, c);   // 0 absorbs an overflowed product
        run *= p;
        wsP[o] = run;
        if (block_prod) block_prod[o] = p;
        if (block_state) block_state[o] = carry;
    }
    if (state_out) state_out[idx] = carry;
    if (prod_out) prod_out[idx] = run;
}

// ---------------------------------------------------------------- 3. re-scan
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
chunk_scan_forward(Geometry g, View<const T> alpha, View<const T> beta, View<T> h,
                   const float *__restrict__ wsC, bool continuation) {
    int64_t vb, s, b;
    decode_block(g, vb, s, b);
    const int64_t v = vb * kThreads + threadIdx.x;
    if (v >= g.nvec) return;
    const int64_t d0 = v * V;
    const int64_t r0 = s * g.L;
    const int64_t r1 = min(g.T, r0 + g.L);

    float st[V];
    const int64_t o = (b * g.S + s) * g.D + d0;
#pragma unroll
    for (int i = 0; i < V; ++i) st[i] = wsC[o + i];

#pragma unroll 4
    for (int64_t t = r0; t < r1; ++t) {
        float a[V], x[V];
        Frag<T, V>::load(alpha.row(b, t) + d0, a);
        Frag<T, V>::load(beta.row(b, t) + d0, x);
        const bool head = (t == 0) && !continuation;
#pragma unroll
        for (int i = 0; i < V; ++i) st[i] = fmaf(head ? 0.0f : a[i], st[i], x[i]);
        Frag<T, V>::store(h.row(b, t) + d0, st);
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
chunk_scan_backward(Geometry g, View<const T> alpha, View<const T> h, View<const T> grad,
                    View<T> dalpha, View<T> dbeta, const float *__restrict__ wsC,
                    const float *__restrict__ h_prev, bool continuation) {
    int64_t vb, s, b;
    decode_block(g, vb, s, b);
    const int64_t v = vb * kThreads + threadIdx.x;
    if (v >= g.nvec) return;
    const int64_t d0 = v * V;
    const int64_t r0 = s * g.L;
    const int64_t r1 = min(g.T, r0 + g.L);

    float u[V];   // a_{t+1} * dh_{t+1}
    const int64_t o = (b * g.S + s) * g.D + d0;
#pragma unroll
    for (int i = 0; i < V; ++i) u[i] = wsC[o + i];

#pragma unroll 4
    for (int64_t t = r1 - 1; t >= r0; --t) {
        float a[V], gr[V], hp[V], da[V], dh[V];
        Frag<T, V>::load(alpha.row(b, t) + d0, a);
        Frag<T, V>::load(grad.row(b, t) + d0, gr);
        if (t > 0) {
            Frag<T, V>::load(h.row(b, t - 1) + d0, hp);
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i)
                hp[i] = (continuation && h_prev) ? h_prev[b * g.D + d0 + i] : 0.0f;
        }
        const bool head = (t == 0) && !continuation;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            dh[i] = gr[i] + u[i];
            da[i] = head ? 0.0f : dh[i] * hp[i];
            u[i] = (head ? 0.0f : a[i]) * dh[i];
        }
        Frag<T, V>::store(dbeta.row(b, t) + d0, dh);
        Frag<T, V>::store(dalpha.row(b, t) + d0, da);
    }
}

// ---------------------------------------------------------------- host side
// Chunk length: enough chunks to put a few resident threads on every SM slot, but never so short
// that the summaries' extra pass dominates.
inline int64_t pick_chunk_rows(int64_t B, int64_t T, int64_t nvec) {
    const int64_t target_threads = 148LL * 2048;
    int64_t S = ceil_div(target_threads, B * nvec > 0 ? B * nvec : 1);
    if (S < 1) S = 1;
    int64_t L = ceil_div(T, S);
    if (L < 16) L = 16;
    if (L > 256) L = 256;
    return L;
}

template <typename T> inline bool vector_ok(int64_t D, std::initializer_list<const fss_view *> views) {
    constexpr int V = VecWidth<T>::value;
    if (D % V) return false;
    for (const fss_view *v : views) {
        if (!v) continue;
        if (!aligned16(v->ptr) || (v->stride_b % V) || (v->stride_t % V)) return false;
    }
    return true;
}

inline Geometry make_geometry(int64_t B, int64_t T, int64_t D, int V) {
    Geometry g;
    g.B = B; g.T = T; g.D = D;
    g.nvec = D / V;
    g.L = pick_chunk_rows(B, T, ceil_div(D, 8));   // same L for both vector widths: block_prod layout
    g.S = ceil_div(T, g.L);
    g.vblocks = ceil_div(g.nvec, kThreads);
    return g;
}

// The kernels run on a linear grid of (channel blocks x chunks x batch rows) CTAs, which has to
// fit the 31 bits of gridDim.x; launchers refuse larger problems with FSS_E_SHAPE.
inline bool grid_fits(const Geometry &g) {
    if (g.vblocks <= 0 || g.S <= 0 || g.B <= 0) return false;
    const int64_t lim = 0x7fffffffLL;
    if (g.vblocks > lim || g.S > lim / g.vblocks) return false;
    return g.B <= lim / (g.vblocks * g.S);
}

inline size_t workspace_bytes(int64_t B, int64_t T, int64_t D) {
    Geometry g = make_geometry(B, T, D, 1);
    return 2 * align_up((size_t)(B * g.S * D) * sizeof(float), 256);
}

}  // namespace chunked
}  // namespace fss
