// Sequence-parallel pieces: every rank scans its rows from a zero state, the per-rank
// (product, state) vectors are gathered by the host (NCCL), and these kernels fold them and add
// the missing term to the rows already written.  The reference never splits the sequence; this
// follows the chunk algebra of fss_chunked.cuh one level up.
#pragma once

#include "fss_common.cuh"

namespace fss {
namespace seqpar {

constexpr int kThreads = 128;

// state' = P*state + C, with 0 absorbing an overflowed P (inf*0 would poison the chain)
__device__ __forceinline__ float fold(float P, float state, float C) {
    return state == 0.0f ? C : fmaf(P, state, C);
}

// pc: [world][2][n]  (row 0 of each rank: product, row 1: state handed on)
__global__ void compose(int backward, int world, int rank, int64_t n,
                        const float *__restrict__ pc, float *__restrict__ carry_in) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float carry = 0.0f;
    if (!backward) {
        for (int r = 0; r < rank; ++r)
            carry = fold(pc[((int64_t)r * 2 + 0) * n + i], carry, pc[((int64_t)r * 2 + 1) * n + i]);
    } else {
        for (int r = world - 1; r > rank; --r)
            carry = fold(pc[((int64_t)r * 2 + 0) * n + i], carry, pc[((int64_t)r * 2 + 1) * n + i]);
    }
    carry_in[i] = carry;
}

struct Geometry {
    int64_t B, T, D;
    int64_t R;        // rows per block (the block_prod granularity)
    int64_t NB;       // blocks per column
    int64_t nvec, vblocks;
};

__device__ __forceinline__ void decode_block(const Geometry &g, int64_t &vb, int64_t &j, int64_t &b) {
    int64_t id = blockIdx.x;
    vb = id % g.vblocks; id /= g.vblocks;
    j = id % g.NB;
    b = id / g.NB;
}

// Re-scan of the blocks that the entering state still reaches (forward).
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
fixup_forward(Geometry g, View<const T> alpha, View<const T> beta, View<T> h, const float *__restrict__ carry_in,
              const float *__restrict__ block_prod, const float *__restrict__ block_state) {
    int64_t vb, j, b;
    decode_block(g, vb, j, b);
    const int64_t v = vb * kThreads + threadIdx.x;
    if (v >= g.nvec) return;
    const int64_t d0 = v * V;
    float st[V];
    bool live = false;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int64_t o = (b * g.NB + j - 1) * g.D + d0 + i;
        const float w = (j == 0 ? 1.0f : block_prod[o]) * carry_in[b * g.D + d0 + i];
        st[i] = (j == 0 ? 0.0f : block_state[o]) + w;
        live |= (w != 0.0f);
    }
    if (!live) return;   // the zero-state result of this block is already exact
    const int64_t r0 = j * g.R, r1 = min(g.T, r0 + g.R);
#pragma unroll 4
    for (int64_t t = r0; t < r1; ++t) {
        float a[V], x[V];
        Frag<T, V>::load(alpha.row(b, t) + d0, a);
        Frag<T, V>::load(beta.row(b, t) + d0, x);
#pragma unroll
        for (int i = 0; i < V; ++i) st[i] = fmaf(a[i], st[i], x[i]);
        Frag<T, V>::store(h.row(b, t) + d0, st);
    }
}

// Re-scan of the blocks that the arriving u still reaches (backward).
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
fixup_backward(Geometry g, View<const T> alpha, View<const T> h, View<const T> grad, View<T> dalpha,
               View<T> dbeta, const float *__restrict__ u_in, const float *__restrict__ h_prev,
               const float *__restrict__ block_prod, const float *__restrict__ block_state, bool continuation) {
    int64_t vb, j, b;
    decode_block(g, vb, j, b);
    const int64_t v = vb * kThreads + threadIdx.x;
    if (v >= g.nvec) return;
    const int64_t d0 = v * V;
    float u[V];
    bool live = false;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int64_t o = (b * g.NB + j + 1) * g.D + d0 + i;
        const bool lastb = j == g.NB - 1;
        const float w = (lastb ? 1.0f : block_prod[o]) * u_in[b * g.D + d0 + i];
        u[i] = (lastb ? 0.0f : block_state[o]) + w;
        live |= (w != 0.0f);
    }
    if (!live) return;
    const int64_t r0 = j * g.R, r1 = min(g.T, r0 + g.R);
#pragma unroll 4
    for (int64_t t = r1 - 1; t >= r0; --t) {
        float a[V], gr[V], hp[V], da[V], dh[V];
        Frag<T, V>::load(alpha.row(b, t) + d0, a);
        Frag<T, V>::load(grad.row(b, t) + d0, gr);
        if (t > 0) {
            Frag<T, V>::load(h.row(b, t - 1) + d0, hp);
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) hp[i] = (continuation && h_prev) ? h_prev[b * g.D + d0 + i] : 0.0f;
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

}  // namespace seqpar
}  // namespace fss
