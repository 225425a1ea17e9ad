// Sequence-parallel pieces: every rank scans its rows from a zero state, the per-rank
// (product, state) vectors are gathered by the host (NCCL), and these kernels fold them and
// re-scan the rows that the state arriving from the neighbouring rank still reaches.  The
// reference never splits the sequence; this follows the chunk algebra of fss_chunked.cuh one
// level up.
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

// ------------------------------------------------------------------ carry exchange through peer memory
// Instead of a library all-gather, every rank can write its (product, state) pair straight into the
// gather tables of all ranks of the box with plain stores to peer-mapped memory (NVLink /
// NVSwitch).  The values travel as 8-byte cells {fp32 value, 32-bit epoch}: an aligned 64-bit store
// arrives whole, so a cell that carries the epoch of the current exchange holds the value written
// with it -- no flag word, no fence, no second round trip; the consumer simply polls (bounded) the
// cells it needs.  For the 32 KB pairs of a long-context run the exchange then costs a small launch
// on the producer's side where the library collective costs 20-50 microseconds.
//
// Rank q owns  table[q] = [world][2][n] cells  and  words[q] = world + 1 32-bit words:
//   words[q][r]      epoch of the last exchange whose pair from rank q rank r has finished reading
//   words[q][world]  counter of the acknowledging kernel (local use)
// Exchange number `epoch` (1, 2, ...; never 0, so nothing is ever cleared).  Before rank r
// overwrites its slot it waits until every reader of that slot (forward: the ranks after r;
// backward: the ranks before r) has acknowledged exchange epoch - 1; in a training loop that is
// always already the case, in a forward-only loop it keeps a fast rank from running more than one
// exchange ahead of a slow reader.
constexpr int kMaxPeers = 16;
struct PeerTables {
    unsigned long long *table[kMaxPeers];
    uint32_t *words[kMaxPeers];
};
constexpr int kPushThreads = 256;

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_cell(unsigned long long *p, float x, uint32_t epoch) {
    const unsigned long long c = (unsigned long long)__float_as_uint(x) | ((unsigned long long)epoch << 32);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(c) : "memory");
}
__device__ __forceinline__ unsigned long long ld_cell(const unsigned long long *p) {
    unsigned long long c;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(c) : "l"(p) : "memory");
    return c;
}
// the value of a cell once it carries `epoch` (bounded poll); false = it never did
__device__ __forceinline__ bool wait_cell(const unsigned long long *p, uint32_t epoch, uint32_t max_spins, float *out) {
    uint32_t spins = 0;
    for (;;) {
        const unsigned long long c = ld_cell(p);
        if ((uint32_t)(c >> 32) == epoch) { *out = __uint_as_float((uint32_t)c); return true; }
        if (++spins >= max_spins) return false;
        __nanosleep(32);
    }
}
// true when *p has reached `want` (epochs only grow) within max_spins polls
__device__ __forceinline__ bool wait_epoch(const uint32_t *p, uint32_t want, uint32_t max_spins) {
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(p) - want) < 0) {
        if (++spins >= max_spins) return false;
        __nanosleep(64);
    }
    return true;
}

// prod, state: this rank's two [n] vectors (local).  Writes them as cells into slot `rank` of every table.
__global__ void __launch_bounds__(kPushThreads)
peer_push(PeerTables peers, int backward, int world, int rank, int64_t n, const float *__restrict__ prod,
          const float *__restrict__ state, uint32_t epoch, int32_t *status, uint32_t max_spins) {
    // placed early (programmatic dependent launch): let the successor do the same, then wait for
    // everything before this kernel on the stream
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ int ok;
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    // readers of this rank's slot must be done with the previous exchange
    const int lo = backward ? 0 : rank + 1, hi = backward ? rank : world;
    if ((int)threadIdx.x >= lo && (int)threadIdx.x < hi && epoch > 1) {
        if (!wait_epoch(peers.words[rank] + threadIdx.x, epoch - 1, max_spins)) ok = 0;
    }
    __syncthreads();
    if (!ok) {
        if (threadIdx.x == 0 && blockIdx.x == 0) report_status(status, FSS_STATUS_EXCHANGE_TIMEOUT);
        return;
    }
    const int64_t base = (int64_t)rank * 2 * n;
    for (int64_t i = (int64_t)blockIdx.x * kPushThreads + threadIdx.x; i < 2 * n; i += (int64_t)gridDim.x * kPushThreads) {
        const float v = i < n ? prod[i] : state[i - n];
        for (int q = 0; q < world; ++q) st_cell(peers.table[q] + base + i, v, epoch);
    }
}

// The forward's push fused with the fold of the per-block products: prod[b, d] = product over the
// row blocks of block_prod[b, :, d] is computed here (a CTA owns 8 channel vectors of one batch row,
// its 64 thread rows split the blocks and combine through shared memory), written to prod_out for
// the caller to keep, and sent to every table together with the state -- one launch instead of two
// between the local scan and the exchange.
constexpr int kPushSlices = 64, kPushVecs = 8;
__global__ void __launch_bounds__(kPushSlices * kPushVecs)
peer_push_blocks(PeerTables peers, int world, int rank, int64_t S, int64_t D, const float *__restrict__ block_prod,
                 const float *__restrict__ state, float *__restrict__ prod_out, uint32_t epoch, int32_t *status,
                 uint32_t max_spins) {
    // placed early (programmatic dependent launch): let the successor do the same, then wait for
    // everything before this kernel on the stream
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float4 part[kPushSlices][kPushVecs];
    __shared__ int ok;
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    if ((int)threadIdx.x > rank && (int)threadIdx.x < world && epoch > 1) {      // forward: the later ranks read this slot
        if (!wait_epoch(peers.words[rank] + threadIdx.x, epoch - 1, max_spins)) ok = 0;
    }
    const int vec = threadIdx.x % kPushVecs, slice = threadIdx.x / kPushVecs;
    const int64_t b = blockIdx.y, B = gridDim.y;
    const int64_t d0 = ((int64_t)blockIdx.x * kPushVecs + vec) * 4;
    const int64_t n = B * D;
    float4 acc = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    if (d0 < D) {      // D is a multiple of 4 here (checked by the launcher)
        const float *base = block_prod + b * S * D + d0;
#pragma unroll 4
        for (int64_t s = slice; s < S; s += kPushSlices) {
            const float4 v = *reinterpret_cast<const float4 *>(base + s * D);
            acc.x *= v.x; acc.y *= v.y; acc.z *= v.z; acc.w *= v.w;
        }
    }
    part[slice][vec] = acc;
    __syncthreads();
    for (int half = kPushSlices / 2; half > 0; half /= 2) {
        if (slice < half) {
            const float4 o = part[slice + half][vec];
            float4 m = part[slice][vec];
            m.x *= o.x; m.y *= o.y; m.z *= o.z; m.w *= o.w;
            part[slice][vec] = m;
        }
        __syncthreads();
    }
    if (!ok) {
        if (threadIdx.x == 0 && blockIdx.x + blockIdx.y == 0) report_status(status, FSS_STATUS_EXCHANGE_TIMEOUT);
        return;
    }
    if (slice < 2 && d0 < D) {      // thread row 0 sends the products, thread row 1 the states
        const int64_t i = b * D + d0;
        float4 v;
        if (slice == 0) {
            v = part[0][vec];
            *reinterpret_cast<float4 *>(prod_out + i) = v;
        } else {
            v = *reinterpret_cast<const float4 *>(state + i);
        }
        const int64_t off = (int64_t)rank * 2 * n + (int64_t)slice * n + i;
        for (int q = 0; q < world; ++q) {
            unsigned long long *t = peers.table[q] + off;
            st_cell(t, v.x, epoch); st_cell(t + 1, v.y, epoch); st_cell(t + 2, v.z, epoch); st_cell(t + 3, v.w, epoch);
        }
    }
}

// A reader's acknowledgement: after ALL CTAs of the consuming kernel have read the pairs, its last
// CTA tells the writers (ranks lo .. hi-1) that their slots may be reused.
__device__ __forceinline__ void acknowledge(const PeerTables &peers, int world, int rank, int lo, int hi, uint32_t epoch) {
    __shared__ bool last;
    __syncthreads();
    uint32_t *counter = peers.words[rank] + world;
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t done = atomicAdd(counter, 1u);
        last = (done + 1 == gridDim.x * gridDim.y * gridDim.z);
        if (last) *counter = 0;
    }
    __syncthreads();
    if (last && (int)threadIdx.x >= lo && (int)threadIdx.x < hi) {
        __threadfence_system();
        st_release_sys(peers.words[threadIdx.x] + rank, epoch);
    }
}

// Folds the cells of the ranks this rank depends on (forward: ranks before it; backward: ranks after
// it) for V consecutive channels starting at idx; false = a cell never arrived.
template <int V>
__device__ __forceinline__ bool fold_cells(const unsigned long long *table, int64_t n, int64_t idx, int lo, int hi,
                                           bool backward, uint32_t epoch, uint32_t max_spins, float (&carry)[V]) {
    bool ok = true;
    for (int k = 0; k < hi - lo && ok; ++k) {
        const int r = backward ? hi - 1 - k : lo + k;
        const unsigned long long *p = table + ((int64_t)r * 2) * n + idx;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            float P, C;
            ok = ok && wait_cell(p + i, epoch, max_spins, &P) && wait_cell(p + n + i, epoch, max_spins, &C);
            if (ok) carry[i] = fold(P, carry[i], C);
        }
    }
    return ok;
}

// The stand-alone consumer: waits for the pairs, composes them like `compose`, acknowledges.  Every
// wait is bounded: when one runs out the status word is set to FSS_STATUS_EXCHANGE_TIMEOUT
// (carry_in is then undefined).
__global__ void __launch_bounds__(256)
peer_compose(PeerTables peers, int backward, int world, int rank, int64_t n, uint32_t epoch,
             float *__restrict__ carry_in, int32_t *status, uint32_t max_spins) {
    const int lo = backward ? rank + 1 : 0, hi = backward ? world : rank;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    bool ok = true;
    if (i < n) {
        float carry[1] = {0.0f};
        ok = fold_cells<1>(peers.table[rank], n, i, lo, hi, backward != 0, epoch, max_spins, carry);
        carry_in[i] = carry[0];
    }
    if (__syncthreads_or(!ok)) {
        if (threadIdx.x == 0) report_status(status, FSS_STATUS_EXCHANGE_TIMEOUT);
        return;      // no acknowledgement: the writers must not reuse what was not read
    }
    acknowledge(peers, world, rank, lo, hi, epoch);
}

// V consecutive floats, as 16-byte loads when the address allows it
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

// ------------------------------------------------------------------ where a fix-up gets its carry from
// Either a ready-made vector (world == 0), or the gathered table of pairs, which the fix-up kernel
// then folds itself -- plain floats filled by a collective (epoch == 0), or the cells of a peer
// exchange, polled until they carry `epoch` and acknowledged afterwards -- so that no separate
// composition launch sits between the exchange and the fix-up.
struct CarrySource {
    const float *carry;      // [B*D], used when world == 0
    const float *table;      // [world][2][n] floats in local memory (epoch == 0)
    PeerTables peers;        // cells and control words (epoch != 0)
    float *carry_out;        // optional [n]: the folded carry, for the caller to keep
    int64_t n;
    int32_t world, rank;
    uint32_t epoch, max_spins;
};

// Every thread of the CTA calls this; false = a wait ran out (reported; the caller returns).
template <int V>
__device__ __forceinline__ bool obtain_carry(const CarrySource &src, bool backward, int64_t idx, bool has, bool writer,
                                             float (&carry)[V], int32_t *status) {
#pragma unroll
    for (int i = 0; i < V; ++i) carry[i] = 0.0f;
    if (src.world == 0) {
        if (has) load_floats<V>(src.carry + idx, carry);
        return true;
    }
    const int lo = backward ? src.rank + 1 : 0, hi = backward ? src.world : src.rank;
    bool ok = true;
    if (has) {
        if (src.epoch) {
            ok = fold_cells<V>(src.peers.table[src.rank], src.n, idx, lo, hi, backward, src.epoch, src.max_spins, carry);
        } else {
            for (int k = 0; k < hi - lo; ++k) {
                const int r = backward ? hi - 1 - k : lo + k;      // forward: ranks 0..rank-1; backward: world-1 down to rank+1
                const float *p = src.table + ((int64_t)r * 2) * src.n + idx;
#pragma unroll
                for (int i = 0; i < V; ++i) carry[i] = fold(__ldcg(p + i), carry[i], __ldcg(p + src.n + i));
            }
        }
        if (ok && writer && src.carry_out) {
#pragma unroll
            for (int i = 0; i < V; ++i) src.carry_out[idx + i] = carry[i];
        }
    }
    if (src.epoch) {
        if (__syncthreads_or(!ok)) {
            if (threadIdx.x == 0 && blockIdx.x + blockIdx.y + blockIdx.z == 0) report_status(status, FSS_STATUS_EXCHANGE_TIMEOUT);
            return false;
        }
        acknowledge(src.peers, src.world, src.rank, lo, hi, src.epoch);
    }
    return true;
}

// ------------------------------------------------------------------ fix-up
// The zero-state scan left, per block of R rows, the block's own product of alpha (block_prod) and
// the state leaving the block (block_state).  With the state `carry` that really enters the rows,
// block j starts from   block_state[j-1] + (product of the blocks before j) * carry   (forward;
// the backward mirrors it from the last block down).  A block whose correction term is exactly
// zero for all its channels already holds the exact result; because the running product only
// shrinks for gates in [0, 1] -- and, once it has underflowed, stays zero in the sequential scan
// too -- the first such block ends the work of its column.
//
// Grid: (slots, channel blocks, batch rows).  The CTA in slot k handles blocks k, k + slots, ... of
// its column until it meets a dead one, so the cost follows the rows that are still reached, plus
// one cheap look per CTA.  Inside a live block the CTA's warps split the rows: each first reduces
// its rows to (P, C), then re-scans them from (map of the warps before it)(entering state).
constexpr int kFixWarps = 16;
constexpr int kFixThreads = kFixWarps * 32;
constexpr int kFixRowBatch = 4;      // rows whose loads are in flight together (two tensors)
constexpr int kFixRowBatch3 = 4;     // the same where three tensors are read per row

struct Geometry {
    int64_t B, T, D;
    int64_t R;        // rows per block (the block_prod granularity)
    int64_t NB;       // blocks per column
    int64_t nvec, vblocks;   // channel vectors per row, CTAs along the channel axis (32 vectors each)
    int slots;        // CTAs along the block axis
};

inline int choose_slots(int64_t NB, int64_t vblocks, int64_t B, int sms) {
    // one CTA per SM in total (a CTA takes a whole SM's registers); a column whose carry reaches
    // further than the slots is walked in strides
    int64_t s = (int64_t)sms / (vblocks * B > 0 ? vblocks * B : 1);
    if (s < 1) s = 1;
    if (s > NB) s = NB;
    return (int)s;
}

// Product over blocks [lo, hi) of block_prod for this lane's channels, all warps of the CTA
// together; every thread returns the full product.  `scratch` is [kFixWarps][32][V] floats.
template <int V>
__device__ __forceinline__ void block_range_product(const float *__restrict__ bp_col, int64_t D, int64_t lo, int64_t hi,
                                                    bool has, float *scratch, float (&out)[V]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 1.0f;
    if (has) {
        for (int64_t s = lo + warp; s < hi; s += kFixWarps) {
            float v[V];
            load_floats<V>(bp_col + s * D, v);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] *= v[i];
        }
    }
    __syncthreads();      // the scratch may still be read from the previous use
#pragma unroll
    for (int i = 0; i < V; ++i) scratch[(warp * 32 + lane) * V + i] = acc[i];
    __syncthreads();
#pragma unroll
    for (int i = 0; i < V; ++i) out[i] = 1.0f;
    for (int w = 0; w < kFixWarps; ++w) {
#pragma unroll
        for (int i = 0; i < V; ++i) out[i] *= scratch[(w * 32 + lane) * V + i];
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kFixThreads)
fixup_forward(Geometry g, View<const T> alpha, View<const T> beta, View<T> h, const CarrySource src,
              const float *__restrict__ block_prod, const float *__restrict__ block_state, int32_t *status) {
    // placed early (programmatic dependent launch): let the successor do the same, then wait for
    // everything before this kernel on the stream
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float sP[kFixWarps * 32 * V], sC[kFixWarps * 32 * V];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t b = blockIdx.z;
    const int64_t v = (int64_t)blockIdx.y * 32 + lane;
    const bool has = v < g.nvec;
    const int64_t d0 = v * V;
    const float *bp_col = block_prod + b * g.NB * g.D + d0;
    const float *bs_col = block_state + b * g.NB * g.D + d0;
    float carry[V], run[V];
#pragma unroll
    for (int i = 0; i < V; ++i) run[i] = 1.0f;
    if (!obtain_carry<V>(src, false, b * g.D + d0, has, blockIdx.x == 0, carry, status)) return;

    int64_t done = 0;      // blocks whose product is already in `run`
    for (int64_t j = blockIdx.x; j < g.NB; j += g.slots) {
        // running product of the blocks before j
        float more[V];
        block_range_product<V>(bp_col, g.D, done, j, has, sP, more);
        done = j;
        float st[V];
        bool live = false;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            run[i] *= more[i];
            st[i] = run[i] * carry[i];
            live |= has && (st[i] != 0.0f);
        }
        if (!__syncthreads_or(live)) break;      // this block and all later ones already hold the exact result
        if (has && j > 0) {
            float bs[V];
            load_floats<V>(bs_col + (j - 1) * g.D, bs);
#pragma unroll
            for (int i = 0; i < V; ++i) st[i] += bs[i];
        }
        const int64_t r0 = j * g.R, r1 = min(g.T, r0 + g.R);
        const int64_t per = (g.R + kFixWarps - 1) / kFixWarps;
        const int64_t w0 = min(r1, r0 + warp * per), w1 = min(r1, w0 + per);
        float P[V], C[V];
#pragma unroll
        for (int i = 0; i < V; ++i) { P[i] = 1.0f; C[i] = 0.0f; }
        if (has) {
#pragma unroll 1
            for (int64_t t0 = w0; t0 < w1; t0 += kFixRowBatch) {
                typename Frag<T, V>::Raw ra[kFixRowBatch], rx[kFixRowBatch];
#pragma unroll
                for (int r = 0; r < kFixRowBatch; ++r) {
                    if (t0 + r < w1) {
                        ra[r] = Frag<T, V>::load_raw(alpha.row(b, t0 + r) + d0);
                        rx[r] = Frag<T, V>::load_raw(beta.row(b, t0 + r) + d0);
                    }
                }
#pragma unroll
                for (int r = 0; r < kFixRowBatch; ++r) {
                    if (t0 + r < w1) {
                        float a[V], x[V];
                        Frag<T, V>::unpack(ra[r], a);
                        Frag<T, V>::unpack(rx[r], x);
#pragma unroll
                        for (int i = 0; i < V; ++i) { C[i] = fmaf(a[i], C[i], x[i]); P[i] *= a[i]; }
                    }
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < V; ++i) { sP[(warp * 32 + lane) * V + i] = P[i]; sC[(warp * 32 + lane) * V + i] = C[i]; }
        __syncthreads();
        if (has) {
            for (int w = 0; w < warp; ++w) {
#pragma unroll
                for (int i = 0; i < V; ++i) st[i] = fmaf(sP[(w * 32 + lane) * V + i], st[i], sC[(w * 32 + lane) * V + i]);
            }
#pragma unroll 1
            for (int64_t t0 = w0; t0 < w1; t0 += kFixRowBatch) {
                typename Frag<T, V>::Raw ra[kFixRowBatch], rx[kFixRowBatch];
#pragma unroll
                for (int r = 0; r < kFixRowBatch; ++r) {
                    if (t0 + r < w1) {
                        ra[r] = Frag<T, V>::load_raw(alpha.row(b, t0 + r) + d0);
                        rx[r] = Frag<T, V>::load_raw(beta.row(b, t0 + r) + d0);
                    }
                }
#pragma unroll
                for (int r = 0; r < kFixRowBatch; ++r) {
                    if (t0 + r < w1) {
                        float a[V], x[V];
                        Frag<T, V>::unpack(ra[r], a);
                        Frag<T, V>::unpack(rx[r], x);
#pragma unroll
                        for (int i = 0; i < V; ++i) st[i] = fmaf(a[i], st[i], x[i]);
                        Frag<T, V>::store(h.row(b, t0 + r) + d0, st);
                    }
                }
            }
        }
    }
}

// The same for the backward scan: u arrives after the last row, blocks are walked from the end.
template <typename T, int V>
__global__ void __launch_bounds__(kFixThreads)
fixup_backward(Geometry g, View<const T> alpha, View<const T> h, View<const T> grad, View<T> dalpha,
               View<T> dbeta, const CarrySource src, const float *__restrict__ h_prev,
               const float *__restrict__ block_prod, const float *__restrict__ block_state, bool continuation,
               int32_t *status) {
    // placed early (programmatic dependent launch): let the successor do the same, then wait for
    // everything before this kernel on the stream
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float sP[kFixWarps * 32 * V], sC[kFixWarps * 32 * V];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t b = blockIdx.z;
    const int64_t v = (int64_t)blockIdx.y * 32 + lane;
    const bool has = v < g.nvec;
    const int64_t d0 = v * V;
    const float *bp_col = block_prod + b * g.NB * g.D + d0;
    const float *bs_col = block_state + b * g.NB * g.D + d0;
    float carry[V], run[V];
#pragma unroll
    for (int i = 0; i < V; ++i) run[i] = 1.0f;
    if (!obtain_carry<V>(src, true, b * g.D + d0, has, blockIdx.x == 0, carry, status)) return;

    int64_t done = g.NB;      // blocks [done, NB) are already in `run`
    for (int64_t k = blockIdx.x; k < g.NB; k += g.slots) {
        const int64_t j = g.NB - 1 - k;
        float more[V];
        block_range_product<V>(bp_col, g.D, j + 1, done, has, sP, more);
        done = j + 1;
        float u[V];
        bool live = false;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            run[i] *= more[i];
            u[i] = run[i] * carry[i];
            live |= has && (u[i] != 0.0f);
        }
        if (!__syncthreads_or(live)) break;
        if (has && j + 1 < g.NB) {
            float bs[V];
            load_floats<V>(bs_col + (j + 1) * g.D, bs);
#pragma unroll
            for (int i = 0; i < V; ++i) u[i] += bs[i];
        }
        const int64_t r0 = j * g.R, r1 = min(g.T, r0 + g.R);
        const int64_t per = (g.R + kFixWarps - 1) / kFixWarps;
        // warp 0 takes the last rows of the block, warp 1 the rows before them, ...
        const int64_t w1 = max(r0, r1 - warp * per), w0 = max(r0, w1 - per);
        float P[V], C[V];
#pragma unroll
        for (int i = 0; i < V; ++i) { P[i] = 1.0f; C[i] = 0.0f; }
        if (has) {
#pragma unroll 1
            for (int64_t t1 = w1; t1 > w0; t1 -= kFixRowBatch) {
                typename Frag<T, V>::Raw ra[kFixRowBatch], rx[kFixRowBatch];
#pragma unroll
                for (int r = 0; r < kFixRowBatch; ++r) {
                    const int64_t t = t1 - 1 - r;
                    if (t >= w0) {
                        ra[r] = Frag<T, V>::load_raw(alpha.row(b, t) + d0);
                        rx[r] = Frag<T, V>::load_raw(grad.row(b, t) + d0);
                    }
                }
#pragma unroll
                for (int r = 0; r < kFixRowBatch; ++r) {
                    const int64_t t = t1 - 1 - r;
                    if (t >= w0) {
                        const bool head = (t == 0) && !continuation;
                        float a[V], x[V];
                        Frag<T, V>::unpack(ra[r], a);
                        Frag<T, V>::unpack(rx[r], x);
#pragma unroll
                        for (int i = 0; i < V; ++i) {
                            const float av = head ? 0.0f : a[i];
                            C[i] = av * (x[i] + C[i]);
                            P[i] *= av;
                        }
                    }
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < V; ++i) { sP[(warp * 32 + lane) * V + i] = P[i]; sC[(warp * 32 + lane) * V + i] = C[i]; }
        __syncthreads();
        if (has) {
            for (int w = 0; w < warp; ++w) {
#pragma unroll
                for (int i = 0; i < V; ++i) u[i] = fmaf(sP[(w * 32 + lane) * V + i], u[i], sC[(w * 32 + lane) * V + i]);
            }
#pragma unroll 1
            for (int64_t t1 = w1; t1 > w0; t1 -= kFixRowBatch3) {
                typename Frag<T, V>::Raw ra[kFixRowBatch3], rg[kFixRowBatch3], rh[kFixRowBatch3];
#pragma unroll
                for (int r = 0; r < kFixRowBatch3; ++r) {
                    const int64_t t = t1 - 1 - r;
                    if (t >= w0) {
                        ra[r] = Frag<T, V>::load_raw(alpha.row(b, t) + d0);
                        rg[r] = Frag<T, V>::load_raw(grad.row(b, t) + d0);
                        if (t > 0) rh[r] = Frag<T, V>::load_raw(h.row(b, t - 1) + d0);
                    }
                }
#pragma unroll
                for (int r = 0; r < kFixRowBatch3; ++r) {
                    const int64_t t = t1 - 1 - r;
                    if (t >= w0) {
                        const bool head = (t == 0) && !continuation;
                        float a[V], gr[V], hp[V], da[V], dh[V];
                        Frag<T, V>::unpack(ra[r], a);
                        Frag<T, V>::unpack(rg[r], gr);
                        if (t > 0) {
                            Frag<T, V>::unpack(rh[r], hp);
                        } else {
#pragma unroll
                            for (int i = 0; i < V; ++i)
                                hp[i] = (continuation && h_prev) ? h_prev[b * g.D + d0 + i] : 0.0f;
                        }
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
            }
        }
    }
}

}  // namespace seqpar
}  // namespace fss
