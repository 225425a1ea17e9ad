// Sequence-parallel pieces: every rank scans its rows from a zero state, the per-rank
// (product, state) pairs are exchanged -- by a collective of the host's choice, or through
// peer-mapped tables that the kernels below write and poll themselves -- and the fix-up kernels
// fold them and re-scan the rows that the state arriving from the neighbouring rank still reaches.
// The reference never splits the sequence; this follows the chunk algebra of fss_chunked.cuh one
// level up.
#pragma once

#include "fss_common.cuh"

namespace fss {
namespace seqpar {

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
// gather tables of the ranks that need it with plain stores to peer-mapped memory (NVLink /
// NVSwitch).  The values travel as 8-byte cells {fp32 value, 32-bit epoch}: an aligned 64-bit store
// arrives whole, so a cell that carries the epoch of the current exchange holds the value written
// with it -- no flag word, no fence, no second round trip; the consumer simply polls (bounded) the
// cells it needs.  For the 32 KB pairs of a long-context run the exchange then costs a few
// microseconds inside kernels that run anyway (the fix-up kernels publish their own rank's pair,
// see publish_pair) where the library collective costs 20-50 microseconds.
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
__device__ __forceinline__ void st_relaxed_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
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
// true when *p has reached `want` (epochs only grow) within max_spins polls
__device__ __forceinline__ bool wait_epoch(const uint32_t *p, uint32_t want, uint32_t max_spins) {
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(p) - want) < 0) {
        if (++spins >= max_spins) return false;
        __nanosleep(64);
    }
    return true;
}

// prod, state: this rank's two [n] vectors (local).  Writes them as cells into slot `rank` of its readers' tables.
__global__ void __launch_bounds__(kPushThreads)
peer_push(PeerTables peers, int backward, int world, int rank, int64_t n, const float *__restrict__ prod,
          const float *__restrict__ state, uint32_t epoch, int32_t *status, uint32_t max_spins) {
    // placed early (programmatic dependent launch): wait for everything before this kernel on the
    // stream, and only then let the successor be placed -- whatever the successor reads before its
    // own wait is then at least as old as this kernel's predecessor
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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
        for (int q = lo; q < hi; ++q) st_cell(peers.table[q] + base + i, v, epoch);      // only its readers poll the slot
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
    // placed early (programmatic dependent launch): wait for everything before this kernel on the
    // stream, and only then let the successor be placed -- whatever the successor reads before its
    // own wait is then at least as old as this kernel's predecessor
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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
        for (int q = rank + 1; q < world; ++q) {      // forward: only the later ranks read this slot
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

// The 2V cells {product_i, state_i} of one rank for V consecutive channels starting at idx, polled
// TOGETHER (2V independent loads per round, not 2V round trips) until all carry `epoch`; false = some
// cell never did.
template <int V>
__device__ __forceinline__ bool wait_cells(const unsigned long long *p, int64_t n, uint32_t epoch, uint32_t max_spins,
                                           float (&P)[V], float (&C)[V]) {
    uint32_t spins = 0;
    for (;;) {
        unsigned long long cp[V], cc[V];
#pragma unroll
        for (int i = 0; i < V; ++i) { cp[i] = ld_cell(p + i); cc[i] = ld_cell(p + n + i); }
        bool all = true;
#pragma unroll
        for (int i = 0; i < V; ++i) all = all && (uint32_t)(cp[i] >> 32) == epoch && (uint32_t)(cc[i] >> 32) == epoch;
        if (all) {
#pragma unroll
            for (int i = 0; i < V; ++i) { P[i] = __uint_as_float((uint32_t)cp[i]); C[i] = __uint_as_float((uint32_t)cc[i]); }
            return true;
        }
        if (++spins >= max_spins) return false;
        __nanosleep(32);
    }
}

// Folds the cells of the ranks this rank depends on (forward: ranks before it; backward: ranks after
// it) for V consecutive channels starting at idx; false = a cell never arrived.
template <int V>
__device__ __forceinline__ bool fold_cells(const unsigned long long *table, int64_t n, int64_t idx, int lo, int hi,
                                           bool backward, uint32_t epoch, uint32_t max_spins, float (&carry)[V]) {
    for (int k = 0; k < hi - lo; ++k) {
        const int r = backward ? hi - 1 - k : lo + k;
        float P[V], C[V];
        if (!wait_cells<V>(table + ((int64_t)r * 2) * n + idx, n, epoch, max_spins, P, C)) return false;
#pragma unroll
        for (int i = 0; i < V; ++i) carry[i] = fold(P[i], carry[i], C[i]);
    }
    return true;
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
    // This rank's own pair for the same exchange, published by the fix-up kernel itself (peer
    // exchange only) instead of by a push launch before it:
    const float *push_state; // [n] the state this rank hands on; NULL = nothing to publish
    const float *push_prod;  // [n] its product; NULL = fold block_prod over all blocks (forward)
    float *push_prod_out;    // optional [n]: the product, for the caller to keep
    int64_t n;
    int32_t world, rank;
    uint32_t epoch, max_spins;
};

constexpr int kCarryWarps = 16;

// Every thread of the CTA calls this; false = a wait ran out (reported; the caller returns).  The
// pairs of the ranks this one depends on are fetched by different warps at the same time -- warp k
// takes the k-th rank of the fold order and parks its (product, state) in the scratch arrays
// ([kCarryWarps][32][V] floats each) -- and then folded by every thread from shared memory: one
// round trip to the table for every kCarryWarps ranks.  The CTA has kCarryWarps warps.  After
// a peer exchange the caller acknowledges (acknowledge_begin / acknowledge_finish).
template <int V>
__device__ __forceinline__ bool obtain_carry(const CarrySource &src, bool backward, int64_t idx, bool has, bool writer,
                                             float *sP, float *sC, float (&carry)[V], int32_t *status) {
#pragma unroll
    for (int i = 0; i < V; ++i) carry[i] = 0.0f;
    if (src.world == 0) {
        if (has) load_floats<V>(src.carry + idx, carry);
        return true;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lo = backward ? src.rank + 1 : 0, hi = backward ? src.world : src.rank;
    const int count = hi - lo;      // ranks to fold, in the order k = 0 .. count-1
    __syncthreads();      // the scratch may still be read from its previous use
    for (int k0 = 0; k0 < count; k0 += kCarryWarps) {
        const int k = k0 + warp;
        bool ok = true;
        if (has && k < count) {
            const int r = backward ? hi - 1 - k : lo + k;      // forward: ranks 0..rank-1; backward: world-1 down to rank+1
            float P[V], C[V];
            if (src.epoch) {
                ok = wait_cells<V>(src.peers.table[src.rank] + ((int64_t)r * 2) * src.n + idx, src.n, src.epoch,
                                   src.max_spins, P, C);
            } else {
                const float *p = src.table + ((int64_t)r * 2) * src.n + idx;
#pragma unroll
                for (int i = 0; i < V; ++i) { P[i] = __ldcg(p + i); C[i] = __ldcg(p + src.n + i); }
            }
            if (ok) {
#pragma unroll
                for (int i = 0; i < V; ++i) { sP[(warp * 32 + lane) * V + i] = P[i]; sC[(warp * 32 + lane) * V + i] = C[i]; }
            }
        }
        if (__syncthreads_or(!ok)) {
            if (threadIdx.x == 0 && blockIdx.x + blockIdx.y + blockIdx.z == 0) report_status(status, FSS_STATUS_EXCHANGE_TIMEOUT);
            return false;      // no acknowledgement: the writers must not reuse what was not read
        }
        if (has) {
            for (int w = 0; w < kCarryWarps && k0 + w < count; ++w) {
#pragma unroll
                for (int i = 0; i < V; ++i) carry[i] = fold(sP[(w * 32 + lane) * V + i], carry[i], sC[(w * 32 + lane) * V + i]);
            }
        }
        __syncthreads();      // the scratch is free again
    }
    if (has && writer && warp == 0 && src.carry_out) {
#pragma unroll
        for (int i = 0; i < V; ++i) src.carry_out[idx + i] = carry[i];
    }
    return true;
}

// After a peer exchange every CTA of the consuming kernel calls acknowledge_begin once its reads of
// the table are done (obtain_carry has returned) and acknowledge_finish a little later: the CTA whose
// count completes the grid tells the writers (forward: the ranks before this one; backward: the ranks
// after it) that their slots may be reused.  Split in two so that the round trip of the count hides
// behind other work, and kept away from the end of the kernel, where the remote stores would delay
// the kernel's completion by an NVLink round trip.  Thread 0 of the CTA does the work.
__device__ __forceinline__ uint32_t acknowledge_begin(const CarrySource &src) {
    if (src.world == 0 || !src.epoch || threadIdx.x != 0) return 0;
    __threadfence();
    return atomicAdd(src.peers.words[src.rank] + src.world, 1u) + 1;
}
__device__ __forceinline__ void acknowledge_finish(const CarrySource &src, bool backward, uint32_t count) {
    if (src.world == 0 || !src.epoch || threadIdx.x != 0) return;
    if (count != gridDim.x * gridDim.y * gridDim.z) return;
    src.peers.words[src.rank][src.world] = 0;      // next used by the next consuming kernel on this stream
    const int lo = backward ? src.rank + 1 : 0, hi = backward ? src.world : src.rank;
    // one system-wide fence orders this GPU's reads of the table before all the words that follow; a
    // release per word would pay for the same fence once per writer (seven times on eight GPUs)
    __threadfence_system();
    for (int r = lo; r < hi; ++r) st_relaxed_sys(src.peers.words[r] + src.rank, src.epoch);
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
constexpr int kFixWarps = kCarryWarps;
constexpr int kFixThreads = kFixWarps * 32;
constexpr int kFixRowBatch = 4;      // rows whose loads are in flight together (two tensors)
constexpr int kFixStagedBatch = 4;   // rows per round of the second pass when alpha waits in shared memory (forward)
constexpr int kFixStagedBatch3 = 2;  // ... and backward
constexpr int kFixRowBatch3 = 2;     // the same where three tensors are read per row (more rows would spill registers)

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

// Memory-level parallelism without registers: a request for the line into L2, nothing comes back.
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Product over blocks [lo, hi) of block_prod for this lane's channels, all warps of the CTA
// together; every thread returns the full product.  `scratch` is [kFixWarps][32][V] floats.
template <int V, int kRound = 1>
__device__ __forceinline__ void block_range_product(const float *__restrict__ bp_col, int64_t D, int64_t lo, int64_t hi,
                                                    bool has, float *scratch, float (&out)[V]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 1.0f;
    if (has) {
        // kRound blocks per round: the loads of a round are in flight together
        for (int64_t s = lo + warp; s < hi; s += kRound * kFixWarps) {
            float v[kRound][V];
#pragma unroll
            for (int r = 0; r < kRound; ++r) {
                if (s + r * kFixWarps < hi) load_floats<V>(bp_col + (s + r * kFixWarps) * D, v[r]);
            }
#pragma unroll
            for (int r = 0; r < kRound; ++r) {
                if (s + r * kFixWarps < hi) {
#pragma unroll
                    for (int i = 0; i < V; ++i) acc[i] *= v[r][i];
                }
            }
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

// The fix-up kernel publishing this rank's own pair (src.push_state != NULL): the CTAs of the last
// slot do it, each for its channels, as soon as the local scan before the kernel is complete -- what
// a push launch between the scan and the fix-up would do, without that launch's place on the
// stream: the readers get the pair a kernel boundary earlier, and this kernel does not have to wait
// for a push kernel's remote stores to be confirmed.  Every thread of the CTA calls it; false = a
// reader never acknowledged the previous exchange (reported).
template <int V>
__device__ __forceinline__ bool publish_pair(const CarrySource &src, bool backward, const float *bp_col, int64_t D,
                                             int64_t NB, int64_t idx, bool has, float *scratch, int32_t *status) {
    const int warp = threadIdx.x >> 5;
    const int lo = backward ? 0 : src.rank + 1, hi = backward ? src.rank : src.world;      // the readers of this rank's slot
    float prod[V], state[V];
#pragma unroll
    for (int i = 0; i < V; ++i) { prod[i] = 1.0f; state[i] = 0.0f; }
    if (has) load_floats<V>(src.push_state + idx, state);
    // the readers must be done with the previous exchange before the slot is overwritten (a few
    // threads look; in a training loop the word is there already, and the look hides behind the
    // loads of the other warps below)
    bool ok = true;
    if ((int)threadIdx.x >= lo && (int)threadIdx.x < hi && src.epoch > 1)
        ok = wait_epoch(src.peers.words[src.rank] + threadIdx.x, src.epoch - 1, src.max_spins);
    if (src.push_prod) {
        if (has) load_floats<V>(src.push_prod + idx, prod);
    } else {
        block_range_product<V, 8>(bp_col, D, 0, NB, has, scratch, prod);
    }
    if (__syncthreads_or(!ok)) {
        if (threadIdx.x == 0) report_status(status, FSS_STATUS_EXCHANGE_TIMEOUT);
        return false;
    }
    if (has) {
        if (warp == 0 && src.push_prod_out) {
#pragma unroll
            for (int i = 0; i < V; ++i) src.push_prod_out[idx + i] = prod[i];
        }
        for (int q = lo + warp; q < hi; q += kCarryWarps) {
            unsigned long long *t = src.peers.table[q] + (int64_t)src.rank * 2 * src.n + idx;
#pragma unroll
            for (int i = 0; i < V; ++i) { st_cell(t + i, prod[i], src.epoch); st_cell(t + src.n + i, state[i], src.epoch); }
        }
    }
    return true;
}

// Pass 1 of a live block, forward: the map (P, C) of rows [w0, w1) of one warp, h_out = P*h_in + C.
// Reads alpha and beta only.
template <typename T, int V>
__device__ __forceinline__ void reduce_rows_forward(const View<const T> &alpha, const View<const T> &beta, int64_t b,
                                                    int64_t d0, int64_t w0, int64_t w1, typename Frag<T, V>::Raw *stage,
                                                    float (&P)[V], float (&C)[V]) {
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
                if (stage) stage[(t0 + r - w0) * 32] = ra[r];
                float a[V], x[V];
                Frag<T, V>::unpack(ra[r], a);
                Frag<T, V>::unpack(rx[r], x);
#pragma unroll
                for (int i = 0; i < V; ++i) { C[i] = fmaf(a[i], C[i], x[i]); P[i] *= a[i]; }
            }
        }
    }
}

// The same for the backward scan, rows (w0, w1] walked downwards: u_out = P*u_in + C with
// u_t = a_t * (g_t + u_{t+1}).  Reads alpha and the incoming gradient only.
template <typename T, int V>
__device__ __forceinline__ void reduce_rows_backward(const View<const T> &alpha, const View<const T> &grad, int64_t b,
                                                     int64_t d0, int64_t w0, int64_t w1, bool continuation,
                                                     typename Frag<T, V>::Raw *stage, float (&P)[V], float (&C)[V]) {
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
                if (stage) stage[(t - w0) * 32] = ra[r];
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

// The CTA's warps have each reduced their rows to (P, C); this leaves in (P, C) the map of all the
// rows of the block that come BEFORE this warp's rows in scan order (warps 0 .. warp-1, the identity
// for warp 0), so that the state entering the warp's rows is  P * (state entering the block) + C.
// Every thread of the CTA calls it.
template <int V>
__device__ __forceinline__ void prefix_of_warps(float *sP, float *sC, float (&P)[V], float (&C)[V]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();      // the scratch may still be read from its previous use
#pragma unroll
    for (int i = 0; i < V; ++i) { sP[(warp * 32 + lane) * V + i] = P[i]; sC[(warp * 32 + lane) * V + i] = C[i]; }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < V; ++i) { P[i] = 1.0f; C[i] = 0.0f; }
    for (int w = 0; w < warp; ++w) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const float p = sP[(w * 32 + lane) * V + i];
            C[i] = fmaf(p, C[i], sC[(w * 32 + lane) * V + i]);
            P[i] *= p;
        }
    }
}

// Pass 2 of a live block, forward: rows [w0, w1) re-scanned from the state `st` that enters them.
// kStaged: alpha comes from the thread's entries in shared memory (taken when used, so that only
// beta occupies registers while loads are in flight -- twice the rows per round).  The pending
// acknowledgement of a peer exchange is finished once, behind the first round's loads.
template <typename T, int V, int kBatch, bool kStaged>
__device__ __forceinline__ void rescan_rows_forward(const View<const T> &alpha, const View<const T> &beta, const View<T> &h,
                                                    int64_t b, int64_t d0, int64_t w0, int64_t w1,
                                                    const typename Frag<T, V>::Raw *stage, float (&st)[V],
                                                    const CarrySource &src, uint32_t ack, bool &acked) {
    using Raw = typename Frag<T, V>::Raw;
#pragma unroll 1
    for (int64_t t0 = w0; t0 < w1; t0 += kBatch) {
        Raw ra[kStaged ? 1 : kBatch], rx[kBatch];
#pragma unroll
        for (int r = 0; r < kBatch; ++r) {
            if (t0 + r < w1) {
                if (!kStaged) ra[r] = Frag<T, V>::load_raw(alpha.row(b, t0 + r) + d0);
                rx[r] = Frag<T, V>::load_raw(beta.row(b, t0 + r) + d0);
            }
        }
        if (!acked) { acknowledge_finish(src, false, ack); acked = true; }      // behind the loads just issued
#pragma unroll
        for (int r = 0; r < kBatch; ++r) {
            if (t0 + r < w1) {
                float a[V], x[V];
                Frag<T, V>::unpack(kStaged ? stage[(t0 + r - w0) * 32] : ra[kStaged ? 0 : r], a);
                Frag<T, V>::unpack(rx[r], x);
#pragma unroll
                for (int i = 0; i < V; ++i) st[i] = fmaf(a[i], st[i], x[i]);
                Frag<T, V>::store(h.row(b, t0 + r) + d0, st);
            }
        }
    }
}

// Pass 2, backward: rows (w0, w1] walked downwards from the u that arrives after them; writes
// dbeta = dh and dalpha = dh * h_{t-1}.  hp0: h before row 0 of the tensors (NULL = 0).
template <typename T, int V, int kBatch, bool kStaged>
__device__ __forceinline__ void rescan_rows_backward(const View<const T> &alpha, const View<const T> &h,
                                                     const View<const T> &grad, const View<T> &dalpha, const View<T> &dbeta,
                                                     int64_t b, int64_t d0, int64_t w0, int64_t w1, bool continuation,
                                                     const float *hp0, const typename Frag<T, V>::Raw *stage, float (&u)[V],
                                                     const CarrySource &src, uint32_t ack, bool &acked) {
    using Raw = typename Frag<T, V>::Raw;
#pragma unroll 1
    for (int64_t t1 = w1; t1 > w0; t1 -= kBatch) {
        Raw ra[kStaged ? 1 : kBatch], rg[kBatch], rh[kBatch];
#pragma unroll
        for (int r = 0; r < kBatch; ++r) {
            const int64_t t = t1 - 1 - r;
            if (t >= w0) {
                if (!kStaged) ra[r] = Frag<T, V>::load_raw(alpha.row(b, t) + d0);
                rg[r] = Frag<T, V>::load_raw(grad.row(b, t) + d0);
                if (t > 0) rh[r] = Frag<T, V>::load_raw(h.row(b, t - 1) + d0);
            }
        }
        if (!acked) { acknowledge_finish(src, true, ack); acked = true; }
#pragma unroll
        for (int r = 0; r < kBatch; ++r) {
            const int64_t t = t1 - 1 - r;
            if (t >= w0) {
                const bool head = (t == 0) && !continuation;
                float a[V], gr[V], hp[V], da[V], dh[V];
                Frag<T, V>::unpack(kStaged ? stage[(t - w0) * 32] : ra[kStaged ? 0 : r], a);
                Frag<T, V>::unpack(rg[r], gr);
                if (t > 0) {
                    Frag<T, V>::unpack(rh[r], hp);
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i) hp[i] = hp0 ? hp0[i] : 0.0f;
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

// Everything that does not depend on the carry -- the reduction of the CTA's first block (pass 1)
// and the block tables of the local scan -- is done before the carry is polled, i.e. while the pairs
// are still travelling; after their arrival only one pass over the rows is left.
template <typename T, int V, bool kStaged>
__global__ void __launch_bounds__(kFixThreads, 1)
fixup_forward(Geometry g, View<const T> alpha, View<const T> beta, View<T> h, const CarrySource src,
              const float *__restrict__ block_prod, const float *__restrict__ block_state, int32_t *status) {
    __shared__ float sP[kFixWarps * 32 * V], sC[kFixWarps * 32 * V];
    // kStaged: the launch comes with room for the alpha rows of one block in (dynamic) shared memory;
    // each thread parks there what it loads in the reduction pass and takes it back in the second
    // pass, which then reads one tensor less through L2.  A thread only ever reads its own entries.
    extern __shared__ __align__(16) unsigned char fix_stage[];
    using Raw = typename Frag<T, V>::Raw;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t b = blockIdx.z;
    const int64_t v = (int64_t)blockIdx.y * 32 + lane;
    const bool has = v < g.nvec;
    const int64_t d0 = v * V;
    const int64_t per = (g.R + kFixWarps - 1) / kFixWarps;
    Raw *stage = kStaged ? reinterpret_cast<Raw *>(fix_stage) + (int64_t)warp * per * 32 + lane : nullptr;
    const int64_t j0 = blockIdx.x;
    float Pp[V], Cp[V];
    // the map of the rows before this warp's rows in block j
    auto prefix_of_block = [&](int64_t j) {
#pragma unroll
        for (int i = 0; i < V; ++i) { Pp[i] = 1.0f; Cp[i] = 0.0f; }
        const int64_t r0 = j * g.R, r1 = min(g.T, r0 + g.R);
        const int64_t w0 = min(r1, r0 + warp * per), w1 = min(r1, w0 + per);
        if (has) reduce_rows_forward<T, V>(alpha, beta, b, d0, w0, w1, stage, Pp, Cp);
        prefix_of_warps<V>(sP, sC, Pp, Cp);
    };
    // Launched as a programmatic dependent: everything before this kernel on the stream is complete
    // once the wait returns.  The successor is NOT released early: the scan that follows fills the GPU,
    // and it measured 6 microseconds faster per step when placed on the empty GPU than when its CTAs
    // were parked one by one behind this kernel's last blocks.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float *bp_col = block_prod + b * g.NB * g.D + d0;
    const float *bs_col = block_state + b * g.NB * g.D + d0;
    // the CTAs of the last slot publish this rank's own pair first thing
    const bool publisher = src.push_state != nullptr && (int)blockIdx.x == g.slots - 1;
    if (publisher && !publish_pair<V>(src, false, bp_col, g.D, g.NB, b * g.D + d0, has, sP, status)) return;
    // the carry and the running product of the blocks are the same in all warps and are needed again
    // only if the CTA goes on to another block: they wait in shared memory, not in registers
    __shared__ float sCarry[32 * V], sRun[32 * V];
    float more[V], bs[V];
#pragma unroll
    for (int i = 0; i < V; ++i) { more[i] = 1.0f; bs[i] = 0.0f; }
    // The first block's share of the work that needs no carry.  The small table reads come first: the
    // reduction pass floods the memory system, and the publishing CTAs -- whose few dependent loads
    // everything else waits for -- get through faster while it has not started.
    if (j0 < g.NB) {
        if (has && j0 > 0) load_floats<V>(bs_col + (j0 - 1) * g.D, bs);
        block_range_product<V>(bp_col, g.D, 0, j0, has, sP, more);
        prefix_of_block(j0);
    }
    {
        float carry[V];
        if (!obtain_carry<V>(src, false, b * g.D + d0, has, blockIdx.x == 0, sP, sC, carry, status)) return;
        if (warp == 0) {
#pragma unroll
            for (int i = 0; i < V; ++i) { sCarry[lane * V + i] = carry[i]; sRun[lane * V + i] = 1.0f; }
        }
        __syncthreads();
    }
    const uint32_t ack = acknowledge_begin(src);
    bool acked = false;

    for (int64_t j = j0; j < g.NB; j += g.slots) {
        if (j != j0) {
            block_range_product<V>(bp_col, g.D, j - g.slots, j, has, sP, more);
            if (has) load_floats<V>(bs_col + (j - 1) * g.D, bs);
        }
        float st[V];
        bool live = false;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            more[i] *= sRun[lane * V + i];      // product of the blocks before j
            st[i] = more[i] * sCarry[lane * V + i];
            live |= has && (st[i] != 0.0f);
        }
        if (!__syncthreads_or(live)) break;      // this block and all later ones already hold the exact result
        if (warp == 0) {      // after the barrier: every warp has read the old value
#pragma unroll
            for (int i = 0; i < V; ++i) sRun[lane * V + i] = more[i];
        }
        if (j != j0) prefix_of_block(j);
#pragma unroll
        for (int i = 0; i < V; ++i) st[i] = fmaf(Pp[i], st[i] + bs[i], Cp[i]);
        const int64_t r0 = j * g.R, r1 = min(g.T, r0 + g.R);
        const int64_t w0 = min(r1, r0 + warp * per), w1 = min(r1, w0 + per);
        if (has) {
            rescan_rows_forward<T, V, kStaged ? kFixStagedBatch : kFixRowBatch, kStaged>(alpha, beta, h, b, d0, w0, w1, stage, st,
                                                                                         src, ack, acked);
        }
    }
    if (!acked) acknowledge_finish(src, false, ack);      // a CTA that met no live block
}

// The same for the backward scan: u arrives after the last row, blocks are walked from the end.
template <typename T, int V, bool kStaged>
__global__ void __launch_bounds__(kFixThreads, 1)
fixup_backward(Geometry g, View<const T> alpha, View<const T> h, View<const T> grad, View<T> dalpha,
               View<T> dbeta, const CarrySource src, const float *__restrict__ h_prev,
               const float *__restrict__ block_prod, const float *__restrict__ block_state, bool continuation,
               int32_t *status) {
    __shared__ float sP[kFixWarps * 32 * V], sC[kFixWarps * 32 * V];
    extern __shared__ __align__(16) unsigned char fix_stage[];      // see fixup_forward
    using Raw = typename Frag<T, V>::Raw;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t b = blockIdx.z;
    const int64_t v = (int64_t)blockIdx.y * 32 + lane;
    const bool has = v < g.nvec;
    const int64_t d0 = v * V;
    const int64_t per = (g.R + kFixWarps - 1) / kFixWarps;
    Raw *stage = kStaged ? reinterpret_cast<Raw *>(fix_stage) + (int64_t)warp * per * 32 + lane : nullptr;
    const int64_t k0 = blockIdx.x;      // block NB-1-k0 is this CTA's first
    float Pp[V], Cp[V];
    // the map of the rows after this warp's rows in block j (warp 0 takes the last rows of the block,
    // warp 1 the rows before them, ...)
    auto prefix_of_block = [&](int64_t j) {
#pragma unroll
        for (int i = 0; i < V; ++i) { Pp[i] = 1.0f; Cp[i] = 0.0f; }
        const int64_t r0 = j * g.R, r1 = min(g.T, r0 + g.R);
        const int64_t w1 = max(r0, r1 - warp * per), w0 = max(r0, w1 - per);
        if (has) {
            // the rows of h that the second pass reads: requested now, found in L2 then
            for (int64_t t = w1 - 1; t >= w0; --t) {
                if (t > 0) prefetch_l2(h.row(b, t - 1) + d0);
            }
            reduce_rows_backward<T, V>(alpha, grad, b, d0, w0, w1, continuation, stage, Pp, Cp);
        }
        prefix_of_warps<V>(sP, sC, Pp, Cp);
    };
    // see fixup_forward
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float *bp_col = block_prod + b * g.NB * g.D + d0;
    const float *bs_col = block_state + b * g.NB * g.D + d0;
    const bool publisher = src.push_state != nullptr && (int)blockIdx.x == g.slots - 1;
    if (publisher && !publish_pair<V>(src, true, bp_col, g.D, g.NB, b * g.D + d0, has, sP, status)) return;
    __shared__ float sCarry[32 * V], sRun[32 * V];
    float more[V], bs[V];
#pragma unroll
    for (int i = 0; i < V; ++i) { more[i] = 1.0f; bs[i] = 0.0f; }
    if (k0 < g.NB) {
        const int64_t j = g.NB - 1 - k0;
        if (has && j + 1 < g.NB) load_floats<V>(bs_col + (j + 1) * g.D, bs);
        block_range_product<V>(bp_col, g.D, j + 1, g.NB, has, sP, more);      // light reads first, see fixup_forward
        prefix_of_block(j);
    }
    {
        float carry[V];
        if (!obtain_carry<V>(src, true, b * g.D + d0, has, blockIdx.x == 0, sP, sC, carry, status)) return;
        if (warp == 0) {
#pragma unroll
            for (int i = 0; i < V; ++i) { sCarry[lane * V + i] = carry[i]; sRun[lane * V + i] = 1.0f; }
        }
        __syncthreads();
    }
    const uint32_t ack = acknowledge_begin(src);
    bool acked = false;

    for (int64_t k = k0; k < g.NB; k += g.slots) {
        const int64_t j = g.NB - 1 - k;
        if (k != k0) {
            block_range_product<V>(bp_col, g.D, j + 1, j + 1 + g.slots, has, sP, more);
            if (has) load_floats<V>(bs_col + (j + 1) * g.D, bs);
        }
        float u[V];
        bool live = false;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            more[i] *= sRun[lane * V + i];      // product of the blocks after j
            u[i] = more[i] * sCarry[lane * V + i];
            live |= has && (u[i] != 0.0f);
        }
        if (!__syncthreads_or(live)) break;
        if (warp == 0) {
#pragma unroll
            for (int i = 0; i < V; ++i) sRun[lane * V + i] = more[i];
        }
        if (k != k0) prefix_of_block(j);
#pragma unroll
        for (int i = 0; i < V; ++i) u[i] = fmaf(Pp[i], u[i] + bs[i], Cp[i]);
        const int64_t r0 = j * g.R, r1 = min(g.T, r0 + g.R);
        const int64_t w1 = max(r0, r1 - warp * per), w0 = max(r0, w1 - per);
        if (has) {
            const float *hp0 = (continuation && h_prev) ? h_prev + b * g.D + d0 : nullptr;      // h before row 0
            rescan_rows_backward<T, V, kStaged ? kFixStagedBatch3 : kFixRowBatch3, kStaged>(
                alpha, h, grad, dalpha, dbeta, b, d0, w0, w1, continuation, hp0, stage, u, src, ack, acked);
        }
    }
    if (!acked) acknowledge_finish(src, true, ack);      // a CTA that met no live block
}

}  // namespace seqpar
}  // namespace fss
