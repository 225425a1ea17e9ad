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

// Fix-up geometry: one CTA per (block of R rows, group of 32 channel vectors, batch row); its
// kWarps warps split the block's rows, lane = channel vector.
constexpr int kWarps = 8;
constexpr int kFixThreads = kWarps * 32;

struct Geometry {
    int64_t B, T, D;
    int64_t R;        // rows per block (the block_prod granularity)
    int64_t NB;       // blocks per column
    int64_t nvec, vblocks;   // channel vectors per row, CTAs along the channel axis (32 vectors each)
};

__device__ __forceinline__ void decode_block(const Geometry &g, int64_t id, int64_t &vb, int64_t &j, int64_t &b) {
    vb = id % g.vblocks; id /= g.vblocks;
    j = id % g.NB;
    b = id / g.NB;
}
// V consecutive floats, as 16-byte loads when the address allows it (one sector per 8 floats
// instead of one per float: the liveness check below is all loads)
template <int V> __device__ __forceinline__ void load_floats(const float *__restrict__ p, float (&out)[V]) {
    if (V % 4 == 0 && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
        for (int i = 0; i < V / 4; ++i) {
            const float4 q = reinterpret_cast<const float4 *>(p)[i];
            out[4 * i] = q.x; out[4 * i + 1] = q.y; out[4 * i + 2] = q.z; out[4 * i + 3] = q.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < V; ++i) out[i] = p[i];
    }
}
// The grid is at most a few CTAs per SM and every CTA walks the (block, channel group, batch row)
// candidates with a grid stride: almost all candidates are dead (their check costs one round of
// loads), and launching a CTA per candidate cost more than checking them.
inline unsigned fixup_grid(const Geometry &g, int sms) {
    const int64_t total = g.vblocks * g.NB * g.B;
    const int64_t cap = (int64_t)sms * (2048 / kFixThreads);
    return (unsigned)(total < cap ? total : cap);
}

// Re-scan of the blocks that the entering state still reaches (forward).  A block is live when
// (product of alpha before it) * carry_in is non-zero for some channel; a dead block already holds
// the exact result.  Inside a live block the warps first summarise their rows (P, C), then each
// re-scans its rows from  (map of the warps before it)(true state entering the block).
template <typename T, int V>
__global__ void __launch_bounds__(kFixThreads)
fixup_forward(Geometry g, View<const T> alpha, View<const T> beta, View<T> h, const float *__restrict__ carry_in,
              const float *__restrict__ block_prod, const float *__restrict__ block_state) {
    __shared__ float sP[kWarps][32][V], sC[kWarps][32][V];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t total = g.vblocks * g.NB * g.B;
    for (int64_t id = blockIdx.x; id < total; id += gridDim.x) {
    int64_t vb, j, b;
    decode_block(g, id, vb, j, b);
    const int64_t v = vb * 32 + lane;
    const bool has = v < g.nvec;
    const int64_t d0 = v * V;
    float st[V];         // what the entering state adds to this block: (product before it) * carry
    bool live = false;
#pragma unroll
    for (int i = 0; i < V; ++i) st[i] = 0.0f;
    const int64_t o = (b * g.NB + j - 1) * g.D + d0;
    if (has) {
        float pr[V];
        load_floats<V>(carry_in + b * g.D + d0, st);
        if (j > 0) {
            load_floats<V>(block_prod + o, pr);
#pragma unroll
            for (int i = 0; i < V; ++i) st[i] *= pr[i];
        }
#pragma unroll
        for (int i = 0; i < V; ++i) live |= (st[i] != 0.0f);
    }
    if (!__syncthreads_or(live)) continue;   // the zero-state result of this block is already exact
    if (has && j > 0) {
        float bs[V];
        load_floats<V>(block_state + o, bs);
#pragma unroll
        for (int i = 0; i < V; ++i) st[i] += bs[i];
    }
    const int64_t r0 = j * g.R, r1 = min(g.T, r0 + g.R);
    const int64_t per = (g.R + kWarps - 1) / kWarps;
    const int64_t w0 = min(r1, r0 + warp * per), w1 = min(r1, w0 + per);
    float P[V], C[V];
#pragma unroll
    for (int i = 0; i < V; ++i) { P[i] = 1.0f; C[i] = 0.0f; }
    if (has) {
#pragma unroll 4
        for (int64_t t = w0; t < w1; ++t) {
            float a[V], x[V];
            Frag<T, V>::load(alpha.row(b, t) + d0, a);
            Frag<T, V>::load(beta.row(b, t) + d0, x);
#pragma unroll
            for (int i = 0; i < V; ++i) { C[i] = fmaf(a[i], C[i], x[i]); P[i] *= a[i]; }
        }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) { sP[warp][lane][i] = P[i]; sC[warp][lane][i] = C[i]; }
    __syncthreads();
    if (has) {
        for (int w = 0; w < warp; ++w) {
#pragma unroll
            for (int i = 0; i < V; ++i) st[i] = fmaf(sP[w][lane][i], st[i], sC[w][lane][i]);
        }
#pragma unroll 4
        for (int64_t t = w0; t < w1; ++t) {
            float a[V], x[V];
            Frag<T, V>::load(alpha.row(b, t) + d0, a);
            Frag<T, V>::load(beta.row(b, t) + d0, x);
#pragma unroll
            for (int i = 0; i < V; ++i) st[i] = fmaf(a[i], st[i], x[i]);
            Frag<T, V>::store(h.row(b, t) + d0, st);
        }
    }
    __syncthreads();      // the summaries are read above; the next candidate may overwrite them
    }
}

// Re-scan of the blocks that the arriving u still reaches (backward); same structure, rows taken
// from the end of the block.
template <typename T, int V>
__global__ void __launch_bounds__(kFixThreads)
fixup_backward(Geometry g, View<const T> alpha, View<const T> h, View<const T> grad, View<T> dalpha,
               View<T> dbeta, const float *__restrict__ u_in, const float *__restrict__ h_prev,
               const float *__restrict__ block_prod, const float *__restrict__ block_state, bool continuation) {
    __shared__ float sP[kWarps][32][V], sC[kWarps][32][V];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t total = g.vblocks * g.NB * g.B;
    for (int64_t id = blockIdx.x; id < total; id += gridDim.x) {
    int64_t vb, j, b;
    decode_block(g, id, vb, j, b);
    const int64_t v = vb * 32 + lane;
    const bool has = v < g.nvec;
    const int64_t d0 = v * V;
    float u[V];
    bool live = false;
#pragma unroll
    for (int i = 0; i < V; ++i) u[i] = 0.0f;
    const bool lastb = j == g.NB - 1;
    const int64_t o = (b * g.NB + j + 1) * g.D + d0;
    if (has) {
        float pr[V];
        load_floats<V>(u_in + b * g.D + d0, u);
        if (!lastb) {
            load_floats<V>(block_prod + o, pr);
#pragma unroll
            for (int i = 0; i < V; ++i) u[i] *= pr[i];
        }
#pragma unroll
        for (int i = 0; i < V; ++i) live |= (u[i] != 0.0f);
    }
    if (!__syncthreads_or(live)) continue;
    if (has && !lastb) {
        float bs[V];
        load_floats<V>(block_state + o, bs);
#pragma unroll
        for (int i = 0; i < V; ++i) u[i] += bs[i];
    }
    const int64_t r0 = j * g.R, r1 = min(g.T, r0 + g.R);
    const int64_t per = (g.R + kWarps - 1) / kWarps;
    // warp 0 takes the last rows of the block, warp 1 the rows before them, ...
    const int64_t w1 = max(r0, r1 - warp * per), w0 = max(r0, w1 - per);
    float P[V], C[V];
#pragma unroll
    for (int i = 0; i < V; ++i) { P[i] = 1.0f; C[i] = 0.0f; }
    if (has) {
#pragma unroll 4
        for (int64_t t = w1 - 1; t >= w0; --t) {
            float a[V], x[V];
            Frag<T, V>::load(alpha.row(b, t) + d0, a);
            Frag<T, V>::load(grad.row(b, t) + d0, x);
            const bool head = (t == 0) && !continuation;
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const float av = head ? 0.0f : a[i];
                C[i] = av * (x[i] + C[i]);
                P[i] *= av;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) { sP[warp][lane][i] = P[i]; sC[warp][lane][i] = C[i]; }
    __syncthreads();
    if (has) {
    for (int w = 0; w < warp; ++w) {
#pragma unroll
        for (int i = 0; i < V; ++i) u[i] = fmaf(sP[w][lane][i], u[i], sC[w][lane][i]);
    }
#pragma unroll 4
    for (int64_t t = w1 - 1; t >= w0; --t) {
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
    __syncthreads();      // the summaries are read above; the next candidate may overwrite them
    }
}

}  // namespace seqpar
}  // namespace fss
