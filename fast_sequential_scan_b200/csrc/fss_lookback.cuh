// FSS_ALGO_LOOKBACK: the single-pass path.  One persistent launch per direction; every tensor
// byte crosses HBM once (forward 3 tensors, backward 5).
//
// Work unit: a 16 KiB tile per tensor of one batch row: 64 rows x 256 bytes of channels, or
// 128 x 128 / 256 x 64 when the problem has too few columns to fill the GPU otherwise (kSp = 2 / 4).
// Tiles are numbered row-block-major (all columns of the first row block, then the next ...; the
// backward numbers row blocks from the end), CTA c of G takes tiles c, c+G, c+2G... so a tile only
// ever depends on tiles with smaller numbers, which are always resident or done.
//
// A CTA (12 warps, one per SM) runs five roles, coupled only by shared-memory mbarriers:
//   producer warp (1 thread)  TMA-loads the tiles of upcoming work units into a ring of stages
//                             (cp.async.bulk.tensor, complete_tx on full[stage]); when pass 2 has
//                             finished a unit it TMA-stores the results from the same stage and
//                             refills it.
//   4 pass-1 warps            a tile has 4 * kSp row groups of 16 rows; lane (q, cl) of warp w owns
//                             group q*4 + w and 8 bytes of channels.  Scans its rows from a zero
//                             state as soon as the tile has landed and leaves (P, C) in shared memory.
//   summary warp              folds the row-group summaries of a unit into per-group exclusive
//                             prefixes and the tile summary, and publishes the latter at once, so
//                             that successors never wait for this tile's own carry resolution.
//   2 look-back warps         take units alternately: resolve the state entering the tile by
//                             decoupled look-back over the global descriptors of its predecessors,
//                             hand it to pass 2, publish the tile's inclusive descriptor.
//                             A descriptor is a set of 8-byte cells {fp32 value, tag}, each moved
//                             with relaxed gpu-scope 64-bit accesses: a cell whose tag carries this
//                             launch's epoch is complete by itself -- no flag word, no fence, one L2
//                             round trip per look-back step, several predecessors read at once.
//   4 pass-2 warps            re-scan the rows from the true entering state and overwrite the
//                             stage in place (beta -> h; grad -> dbeta, h -> dalpha).
// The roles' loops are kept small on purpose (32-bit unit counters, no division, no unrolling
// across units): the kernel is sensitive to instruction-cache misses.
// Every wait is bounded; a wait that runs out records a status, raises the abort flag that all
// other waits poll, and the CTA drains its copies and leaves.
#pragma once

#include <cuda.h>

#include <initializer_list>
#include <mutex>
#include <string>

#include "fss_common.cuh"
#include "fss_gates.cuh"

namespace fss {
namespace lookback {

constexpr int kW = 4;                         // warps per pass (pass-1 group and pass-2 group)
constexpr int kR = 16;                        // rows per warp and tile
constexpr int kRh = 8;                        // rows handled per register batch
constexpr int kTc = kW * kR;                  // rows per tile
constexpr int kRowBytes = 256;                // bytes of one tile row
constexpr int kLaneBytes = 8;
constexpr int kTileBytes = kTc * kRowBytes;   // 16 KiB per tensor and stage
constexpr int kPass2Warp0 = kW;               // warps [0,kW) run pass 1, [kW,2kW) run pass 2
constexpr int kProducerWarp = 2 * kW;
constexpr int kSummaryWarp = 2 * kW + 1;
constexpr int kLookbackWarp0 = 2 * kW + 2;    // first of the look-back warps
constexpr int kLookbackWarps = 2;             // three were measured slower on every workload
constexpr int kGens = 4;                      // generations of summary buffers: pass 1 may run this far ahead of pass 2
constexpr int kThreads = (2 * kW + 2 + kLookbackWarps) * 32;
constexpr int kGateWarp0 = 2 * kW + 2 + kLookbackWarps;      // gated forward only: kW more warps that evaluate the gates
constexpr int kThreadsGated = kThreads + kW * 32;
template <bool kGate> constexpr int threads_of() { return kGate ? kThreadsGated : kThreads; }
constexpr int kStagesFwd = 6;                 // 6 x 32 KiB
constexpr int kStagesBwd = 4;                 // 4 x 48 KiB
constexpr uint32_t kMaxSpins = 1u << 21;      // per wait; ~a second before giving up

constexpr uint32_t kStateAggregate = 1, kStateInclusive = 2;
constexpr int kWindow = 2;                    // predecessors inspected per look-back round trip

template <typename T> struct Cfg {
    static constexpr int V = kLaneBytes / (int)sizeof(T);   // channels per lane
    static constexpr int Dc = 32 * V;                       // channels per tile
};

struct Header {      // first bytes of the workspace
    uint32_t epoch;  // number of look-back launches that have completed on this workspace
    uint32_t done;   // CTAs of the running launch that have finished
    uint32_t abort;  // raised by the first wait that gives up
    uint32_t ticket; // tiles handed out beyond the first kStages per CTA (reset by the last CTA)
};

struct Params {
    int64_t B, T, D;
    int64_t ncg;      // channel groups per row
    int64_t ncols;    // B * ncg
    int64_t S;        // row blocks per column
    int64_t ntiles;
    uint4 *packets;   // [ntiles][packets per tile][32 lanes]
    Header *hdr;
    int32_t *status;
    const float *state_in;   // forward h_in / backward u_in, [B, D] or null
    float *state_out;        // forward h_last / backward u_out
    float *block_prod;       // [B, S, D]: product of alpha over the rows of each row block
    float *block_state;      // [B, S, D]: state leaving each row block
    const float *h_prev;     // backward only
    const float *lambda;     // gated forward only: [D] exponent scales -8*softplus(lambda)*log2(e), made by gates::prescale
    int continuation;
    int32_t tile_rows;       // rows per tile: 64 * split
    uint32_t max_spins;      // iterations a wait may take before it gives up
    int mute_first_block;    // test hook: row block 0 publishes no descriptors (its successors' waits run out)
    int deterministic;       // a tile only ever starts from its predecessor's inclusive state
    int hold_dependents;     // no early release of the next launch on the stream
    int64_t grid;            // CTAs of the launch
    // fixed tile order (CTA x takes tiles x, x+G, ...): ntiles = units_q * grid + units_r, so CTA x
    // owns units_q + (x < units_r) tiles; one grid stride = grid_q row blocks + grid_b batch rows +
    // grid_cg channel groups
    int32_t units_q, units_r;
    int32_t grid_q, grid_b, grid_cg;
    // ticket order: the first n_fixed units of every CTA are the fixed ones (tiles x, x+G, ...),
    // all tiles from n_fixed * G on are handed out by the counter
    int32_t n_fixed;
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// non-blocking probe of a phase (try_wait may park the warp until the phase completes)
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int32_t c0, int32_t c1, int32_t c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src,
                                             int32_t c0, int32_t c1, int32_t c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
        ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ uint32_t ld_volatile(const uint32_t *p) {
    return *reinterpret_cast<const volatile uint32_t *>(p);
}

// Descriptor cells.  A cell is 8 bytes: one fp32 value and a 32-bit tag.  An aligned 64-bit access
// is single-copy atomic, so a cell whose tag carries this launch's epoch holds the value that was
// written with it -- no separate flag, no fence.  Cells travel two at a time in 16-byte vector
// accesses (each element keeps its own tag, so nothing relies on 128-bit atomicity).  The accesses
// use the .cg cache operator: they are served by L2, the point of coherence between SMs, and --
// unlike gpu-scope "strong" accesses, which were measured to issue one after the other -- they
// pipeline, so a whole look-back window costs one round trip.
__device__ __forceinline__ unsigned long long make_cell(float x, uint32_t tag) {
    return (unsigned long long)__float_as_uint(x) | ((unsigned long long)tag << 32);
}
// N floats as N/2 cell pairs; pair j of a tile's group sits at p[j*kStride] (one uint4 per channel lane)
template <int N, int kStride = 32> struct PacketGroup {
    static_assert(N % 2 == 0, "cells are moved in pairs");
    static constexpr int kPackets = N / 2;
    static __device__ __forceinline__ void store(uint4 *p, const float (&v)[N], uint32_t tag) {
#pragma unroll
        for (int j = 0; j < kPackets; ++j)
            asm volatile("st.global.cg.v2.b64 [%0], {%1, %2};"
                         ::"l"(p + j * kStride), "l"(make_cell(v[2 * j], tag)), "l"(make_cell(v[2 * j + 1], tag)) : "memory");
    }
    // Issue the loads only: nothing here depends on the returned data, so the caller can keep
    // working (or wait on a barrier) while they are in flight, and decode() later.
    struct Raw { unsigned long long c[N]; };
    static __device__ __forceinline__ void load_raw(const uint4 *p, Raw &r) {
#pragma unroll
        for (int j = 0; j < kPackets; ++j)
            asm volatile("ld.global.cg.v2.b64 {%0, %1}, [%2];"
                         : "=l"(r.c[2 * j]), "=l"(r.c[2 * j + 1]) : "l"(p + j * kStride) : "memory");
    }
    // true when every cell of the group carries `tag`
    static __device__ __forceinline__ bool decode(const Raw &r, float (&v)[N], uint32_t tag) {
        bool ok = true;
#pragma unroll
        for (int j = 0; j < N; ++j) {
            v[j] = __uint_as_float((uint32_t)r.c[j]);
            ok &= ((uint32_t)(r.c[j] >> 32) == tag);
        }
        return ok;
    }
    static __device__ __forceinline__ bool load(const uint4 *p, float (&v)[N], uint32_t tag) {
        Raw r;
        load_raw(p, r);
        return decode(r, v, tag);
    }
};

// ------------------------------------------------------------------ 8-byte lane fragments
// What one lane owns of a tile row: 8 bytes = 4 bf16 or 2 fp32 channels.
__device__ __forceinline__ float vec_get(const float4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
__device__ __forceinline__ float vec_get(const float2 &v, int i) { return i == 0 ? v.x : v.y; }
__device__ __forceinline__ void vec_set(float4 &v, int i, float f) { if (i == 0) v.x = f; else if (i == 1) v.y = f; else if (i == 2) v.z = f; else v.w = f; }
__device__ __forceinline__ void vec_set(float2 &v, int i, float f) { if (i == 0) v.x = f; else v.y = f; }

template <typename T> struct Lane;
template <> struct Lane<bf16> {
    static constexpr int V = 4;
    using Raw = uint2;
    using VecF = float4;
    static __device__ __forceinline__ Raw zero() { return make_uint2(0u, 0u); }
    static __device__ __forceinline__ Raw one() { return make_uint2(0x3f803f80u, 0x3f803f80u); }
    static __device__ __forceinline__ void unpack(const Raw &r, float (&x)[4]) {
        x[0] = __uint_as_float(r.x << 16); x[1] = __uint_as_float(r.x & 0xffff0000u);
        x[2] = __uint_as_float(r.y << 16); x[3] = __uint_as_float(r.y & 0xffff0000u);
    }
    static __device__ __forceinline__ Raw pack(const float (&x)[4]) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]);
        __nv_bfloat162 hi = __floats2bfloat162_rn(x[2], x[3]);
        return make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
    }
};
template <> struct Lane<float> {
    static constexpr int V = 2;
    using Raw = float2;
    using VecF = float2;
    static __device__ __forceinline__ Raw zero() { return make_float2(0.0f, 0.0f); }
    static __device__ __forceinline__ Raw one() { return make_float2(1.0f, 1.0f); }
    static __device__ __forceinline__ void unpack(const Raw &r, float (&x)[2]) { x[0] = r.x; x[1] = r.y; }
    static __device__ __forceinline__ Raw pack(const float (&x)[2]) { return make_float2(x[0], x[1]); }
};

// With 64-byte tile rows the two row groups that share a half-warp read the same 16 banks when
// both are at row r.  The odd group therefore touches row r^1 in the instruction slot of row r
// (pair_slot) and swaps each register pair afterwards (pair_fix), before stores likewise.
template <int kRowStride, typename R>
__device__ __forceinline__ R &pair_slot(R *tile, int row, int dsw) {
    return tile[row * kRowStride + ((row & 1) ? -dsw : dsw)];
}
template <bool kOn, int N, typename R>
__device__ __forceinline__ void pair_fix(R (&x)[N], bool odd) {
    if (kOn) {
#pragma unroll
        for (int m = 0; m + 1 < N; m += 2) {
            // field by field, so that each becomes one select and not a divergent branch
            const auto lox = odd ? x[m + 1].x : x[m].x, loy = odd ? x[m + 1].y : x[m].y;
            const auto hix = odd ? x[m].x : x[m + 1].x, hiy = odd ? x[m].y : x[m + 1].y;
            x[m].x = lox; x[m].y = loy; x[m + 1].x = hix; x[m + 1].y = hiy;
        }
    }
}

// ------------------------------------------------------------------ bounded waits
struct Ctl {
    Header *hdr;
    int32_t *status;
    volatile int *cta_abort;   // shared-memory copy of the abort flag
    uint32_t max_spins;

    __device__ __forceinline__ bool aborted() const {
        return *cta_abort != 0 || ld_volatile(&hdr->abort) != 0;
    }
    __device__ __forceinline__ void give_up(int32_t code) const {
        *cta_abort = 1;
        atomicExch(&hdr->abort, 1u);
        report_status(status, code);
    }
    // false = the wait was abandoned (timeout here, or abort raised elsewhere).  The common case
    // is one successful try.  (An out-of-line slow path was measured: the call costs more than it saves.)
    __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, int32_t code) const {
        if (mbar_try_wait(bar, parity)) return true;
        return wait_slow(bar, parity, code);
    }
    __device__ __forceinline__ bool wait_slow(uint32_t bar, uint32_t parity, int32_t code) const {
        for (uint32_t it = 0; it < max_spins; ++it) {
            if (mbar_try_wait(bar, parity)) return *cta_abort == 0;
            if ((it & 63u) == 63u && aborted()) { *cta_abort = 1; return false; }
        }
        give_up(code);
        return false;
    }
};

// ------------------------------------------------------------------ shared-memory plan
template <int kTensors, int kStages> struct Smem {
    static constexpr int kStageBytes = kTensors * kTileBytes;
    // summaries: [generation][warp][P|C][lane] as 8-byte (fp32 x2) or 16-byte (fp32 x4) entries
    static constexpr int kAggBytes = kGens * kW * 2 * 32 * 16;
    static constexpr int kSumBytes = kGens * 3 * 32 * 16;      // [generation][tile P | tile C | entering state][lane]
    static constexpr int kBarriers = 4 * kStages + 3 * kGens;      // full, done, info, gate per stage; agg, carry, sum per generation
    static constexpr int kBytes = 128 /* alignment slack */ + kStages * kStageBytes + kAggBytes + kSumBytes +
                                  kBarriers * 8 + 16 + kStages * 16 /* unit descriptors */;
};

// A work unit as the producer describes it to the other roles (one 16-byte shared-memory slot per
// stage): tile number, row block in processing order, batch row, channel group.  k < 0 ends the CTA.
struct Unit {
    int32_t k, s, b, cg;
    template <bool kBackward> __device__ __forceinline__ int32_t row0(const Params &p) const {
        return (kBackward ? ((int32_t)p.S - 1 - s) : s) * p.tile_rows;
    }
};
__device__ __forceinline__ Unit unit_of_tile(const Params &p, int64_t tile) {
    Unit u;
    u.k = (int32_t)tile;
    u.s = (int32_t)((uint32_t)tile / (uint32_t)p.ncols);
    const uint32_t col = (uint32_t)tile - (uint32_t)u.s * (uint32_t)p.ncols;
    u.b = (int32_t)(col / (uint32_t)p.ncg);
    u.cg = (int32_t)(col - (uint32_t)u.b * (uint32_t)p.ncg);
    return u;
}

// How a role learns which tile its next unit is.
//   fixed order (kTickets = false): arithmetic only -- CTA x works on tiles x, x+G, x+2G, ...
//   tickets (kTickets = true): the first p.n_fixed units of a CTA are still the fixed ones; every
//     later unit is described by the producer in a shared-memory slot per stage (see the producer),
//     which then arrives on info[stage]; a role reads the descriptor of its next unit while it still
//     waits for the data of the current one, and only blocks if that was too early.
template <bool kTickets, int kStages> struct UnitCursor {
    const Params &p;
    const Ctl &ctl;
    const Unit *units;
    uint32_t bar_info0;
    int stride;          // units between two of this role's units (look-back warps: their number)
    Unit cur, nxt;       // unit i / i + stride; nxt valid when `have`
    bool have;
    int n_arith;         // units of this CTA that follow from arithmetic

    __device__ __forceinline__ UnitCursor(const Params &p_, const Ctl &ctl_, const Unit *units_, uint32_t bar_info0_)
        : p(p_), ctl(ctl_), units(units_), bar_info0(bar_info0_) {}

    __device__ __forceinline__ void step(Unit &u, int n) const {      // fixed order: n grid strides on
        for (int j = 0; j < n; ++j) {
            u.k += (int32_t)p.grid;
            u.s += p.grid_q;
            u.cg += p.grid_cg;
            u.b += p.grid_b;
            if (u.cg >= (int32_t)p.ncg) { u.cg -= (int32_t)p.ncg; u.b += 1; }
            if (u.b >= (int32_t)p.B) { u.b -= (int32_t)p.B; u.s += 1; }
        }
    }
    // phase of info[j % kStages] that unit j >= n_fixed completes: units n_fixed, n_fixed + 1, ... arrive in turn
    __device__ __forceinline__ uint32_t info_parity(int j) const {
        return (uint32_t)(((j - p.n_fixed) / kStages) & 1);
    }
    __device__ __forceinline__ bool try_read(int j, Unit &out) const {   // warp-uniform
        const int sj = j % kStages;
        if (!__all_sync(0xffffffffu, mbar_test_wait(bar_info0 + 8u * sj, info_parity(j)))) return false;
        out = units[sj];
        return true;
    }
    // start at unit `first_unit` of the CTA
    // u0: the CTA's first unit (tile blockIdx.x), worked out once per thread before the roles part
    __device__ __forceinline__ void init(const Unit &u0, int first_unit, int stride_) {
        stride = stride_;
        n_arith = kTickets ? p.n_fixed : p.units_q + ((int32_t)blockIdx.x < p.units_r ? 1 : 0);
        nxt = u0;
        have = first_unit < n_arith;
        if (have) step(nxt, first_unit);
        else if (kTickets) have = try_read(first_unit, nxt);
    }
    // Unit i into `cur`; false = no more units (or the wait was abandoned).  Then looks ahead to unit
    // i + stride: next_known() says whether `nxt` already describes a real unit.
    __device__ __forceinline__ bool advance(int i) {
        if (i < n_arith) {
            cur = nxt;
            if (i + stride < n_arith) step(nxt, stride);      // have stays true
            else have = kTickets ? try_read(i + stride, nxt) : false;
            return true;
        }
        if (!kTickets) return false;
        if (have) {
            cur = nxt;
        } else {
            const int si = i % kStages;
            if (!ctl.wait(bar_info0 + 8u * si, info_parity(i), FSS_STATUS_TMA_TIMEOUT)) return false;
            cur = units[si];
        }
        if (cur.k < 0) return false;
        have = try_read(i + stride, nxt);
        return true;
    }
    __device__ __forceinline__ bool next_known() const { return have && nxt.k >= 0; }
};

// Gated forward: turns kRh rows (from row `base` of this lane's group) of a stage from (r, x, i) into
// (alpha, beta) in place, rounded to the I/O type as if they had come from memory.  The odd row
// group of a 64-byte-row tile reads row r^1 in the slot of row r (see pair_slot); every value goes
// back to the slot it came from, so nothing has to be swapped here.
template <typename T, int kRowStride>
__device__ __forceinline__ void gate_rows(typename Lane<T>::Raw *a_t, typename Lane<T>::Raw *x_t,
                                          const typename Lane<T>::Raw *i_t, int base, int dsw, bool odd_grp,
                                          const float (&gsc)[Lane<T>::V], bool head, int nvalid, bool edge_rows) {
    constexpr int V = Lane<T>::V;
    using Raw = typename Lane<T>::Raw;
    Raw ra[kRh], rx[kRh], rg[kRh];
#pragma unroll
    for (int r = 0; r < kRh; ++r) {
        ra[r] = pair_slot<kRowStride>(a_t, base + r, dsw);
        rx[r] = pair_slot<kRowStride>(x_t, base + r, dsw);
        rg[r] = pair_slot<kRowStride>(i_t, base + r, dsw);
    }
#pragma unroll
    for (int r = 0; r < kRh; ++r) {
        float rr[V], ii[V], xx[V], a[V], b[V];
        Lane<T>::unpack(ra[r], rr);
        Lane<T>::unpack(rg[r], ii);
        Lane<T>::unpack(rx[r], xx);
#pragma unroll
        for (int v = 0; v < V; ++v) {
            a[v] = Gate<T>::exp_scaled(gsc[v] * Gate<T>::sigmoid(rr[v]));
            b[v] = Gate<T>::root(fmaf(-a[v], a[v], 1.0f)) * Gate<T>::sigmoid(ii[v]) * xx[v];
        }
        if (edge_rows) {       // warp-uniform and rare: first row of the sequence, rows after its end
            const int row = base + (odd_grp ? (r ^ 1) : r);      // the row this register holds
            const bool first_row = head && row == 0;             // alpha_0 is not part of the recurrence
            const bool past_end = row >= nvalid;                 // identity rows after the sequence
#pragma unroll
            for (int v = 0; v < V; ++v) {
                if (first_row) a[v] = 0.0f;
                if (past_end) { a[v] = 1.0f; b[v] = 0.0f; }
            }
        }
        ra[r] = Lane<T>::pack(a);
        rx[r] = Lane<T>::pack(b);
    }
#pragma unroll
    for (int r = 0; r < kRh; ++r) {
        pair_slot<kRowStride>(a_t, base + r, dsw) = ra[r];
        pair_slot<kRowStride>(x_t, base + r, dsw) = rx[r];
    }
}

// ------------------------------------------------------------------ the kernel
// Forward: tiles of (alpha, beta) are loaded, h is stored from beta's stage slot.
// Backward: (alpha, grad, h shifted one row down) are loaded; dbeta is stored from grad's slot,
// dalpha from h's slot.  Results are written in place in shared memory and leave through TMA
// stores issued by the producer, so the consumer warps never stall on the global write path.
template <typename T, bool kBackward, int kSp, bool kTickets, bool kGate = false>
__global__ void __launch_bounds__(threads_of<kGate>(), 1)
scan_kernel(const __grid_constant__ CUtensorMap map_alpha, const __grid_constant__ CUtensorMap map_x,
            const __grid_constant__ CUtensorMap map_h, const __grid_constant__ CUtensorMap map_out0,
            const __grid_constant__ CUtensorMap map_out1, const Params p) {
    static_assert(!(kGate && (kBackward || kTickets)), "the gate front-end exists for the plain forward only");
    constexpr bool kThree = kBackward || kGate;      // tensors loaded per unit: 3, else 2
    constexpr int kTensors = kThree ? 3 : 2;
    constexpr int kStages = kThree ? kStagesBwd : kStagesFwd;
    using SM = Smem<kTensors, kStages>;
    constexpr int V = Cfg<T>::V;
    // Tile shape: kSp = 1: 64 rows x 256 bytes; 2: 128 x 128; 4: 256 x 64 (same 16 KiB).  A warp then
    // covers kSp row groups of kR rows at once: lane = (row group q, channel lane cl).
    constexpr int LPG = 32 / kSp;                 // lanes per row group
    constexpr int Dc = Cfg<T>::Dc / kSp;          // channels per tile
    constexpr int kRowB = kRowBytes / kSp;        // bytes of a tile row
    using VecF = typename Lane<T>::VecF;          // V floats as one shared-memory word group

    // TMA tiles want 128-byte aligned shared addresses: align the dynamic window by hand
    extern __shared__ unsigned char smem_dyn[];
    unsigned char *smem_raw = smem_dyn + ((128u - (smem_u32(smem_dyn) & 127u)) & 127u);
    const uint32_t smem_base = smem_u32(smem_raw);
    VecF *agg = reinterpret_cast<VecF *>(smem_raw + kStages * SM::kStageBytes);
    VecF *sums = reinterpret_cast<VecF *>(smem_raw + kStages * SM::kStageBytes + SM::kAggBytes);
    const uint32_t bars = smem_base + kStages * SM::kStageBytes + SM::kAggBytes + SM::kSumBytes;
    volatile int *cta_abort = reinterpret_cast<volatile int *>(smem_raw + kStages * SM::kStageBytes +
                                                               SM::kAggBytes + SM::kSumBytes + SM::kBarriers * 8);
    Unit *units = reinterpret_cast<Unit *>(smem_raw + kStages * SM::kStageBytes + SM::kAggBytes + SM::kSumBytes +
                                           SM::kBarriers * 8 + 16);
    auto bar_info = [&](int s) { return bars + 8u * (2 * kStages + 3 * kGens + s); };
    auto bar_gate = [&](int s) { return bars + 8u * (3 * kStages + 3 * kGens + s); };
    auto bar_full = [&](int s) { return bars + 8u * s; };
    auto bar_done = [&](int s) { return bars + 8u * (kStages + s); };
    auto bar_agg = [&](int g) { return bars + 8u * (2 * kStages + g); };
    auto bar_carry = [&](int g) { return bars + 8u * (2 * kStages + kGens + g); };
    auto bar_sum = [&](int g) { return bars + 8u * (2 * kStages + 2 * kGens + g); };
    auto sum_at = [&](int g, int which, int ln) -> VecF & { return sums[(g * 3 + which) * 32 + ln]; };
    // agg[(g, w, P|C)][lane]
    auto agg_at = [&](int g, int w, int which, int ln) -> VecF & { return agg[((g * kW + w) * 2 + which) * 32 + ln]; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q = lane / LPG, cl = lane % LPG;
    const uint32_t first = blockIdx.x;
    const Unit u0 = unit_of_tile(p, first);
    // Programmatic dependent launch: let the next launch on the stream start its own set-up as SMs
    // become free, and do everything that touches no global memory before waiting for the previous
    // launch to finish (both instructions do nothing for an ordinary launch).  With hold_dependents
    // the next launch is not released early and starts when this one has finished
    // (FSS_FLAG_HOLD_DEPENDENTS).
    if (!p.hold_dependents) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == kProducerWarp * 32) {
        // the descriptors are kernel parameters, not data of the previous launch: fetch them now
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_alpha) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        if (kThree) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_h) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_out0) : "memory");
        if (kBackward) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_out1) : "memory");
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full(s), 1); mbar_init(bar_done(s), kW); mbar_init(bar_info(s), 1); mbar_init(bar_gate(s), kW);
        }
        for (int g = 0; g < kGens; ++g) { mbar_init(bar_agg(g), kW); mbar_init(bar_carry(g), 1); mbar_init(bar_sum(g), 1); }
        *cta_abort = 0;
        asm volatile("griddepcontrol.wait;" ::: "memory");      // the previous launch and its writes are complete
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    __syncthreads();
    const Ctl ctl{p.hdr, p.status, cta_abort, p.max_spins};
    using Cursor = UnitCursor<kTickets, kStages>;
    // This launch's epoch (tags of its descriptors) is only needed by the summary and look-back
    // warps, which read it themselves: the producer's first loads do not wait for this round trip.
    // (The header's epoch changes only after every CTA of the launch has finished.)
    uint32_t epoch = 0;
    if (warp == kSummaryWarp || warp >= kLookbackWarp0) epoch = ld_volatile(&p.hdr->epoch) + 1u;

    if (warp == kProducerWarp) {
        // ============================================================ producer
        if (lane == 0) {
            // Which tile a unit is.  Fixed order: CTA x takes tiles x, x+G, x+2G, ...  Tickets: the same
            // for the first n_fixed units, after that every refill takes the next tile from a global
            // counter, so an SM that the memory system serves faster takes more tiles and all CTAs
            // finish together.  Tickets are handed out in increasing order and each CTA works through
            // its own in order, so a tile still only depends on tiles some resident CTA has taken.
            const int64_t G = p.grid;
            uint32_t hand = 0;            // ticket requested one refill ahead (hides the atomic's latency)
            int issued = 0;               // real units whose loads were started
            int next = 0;                 // slots described so far: the units, then end markers
            bool ended = false;
            Unit nu;
            // prepare() works out what slot `next` will hold: the next unit, or, once the tiles have
            // run out, an end marker.  post() publishes it and starts the unit's loads.  With tickets,
            // markers keep being posted as stages free up, because the look-back warps take units
            // alternately and each has to meet one.  prepare() runs while the stage is still busy, so
            // its arithmetic and the ticket's round trip stay off the refill path.
            // (this thread runs alone: it only uses the cursor's arithmetic, never its warp-wide reads)
            const Cursor arith(p, ctl, units, bar_info(0));
            const int n_arith = kTickets ? p.n_fixed : p.units_q + ((int32_t)first < p.units_r ? 1 : 0);
            Unit walk = u0;               // the unit slot `next` holds while next < n_arith
            auto prepare = [&]() {
                if (next < n_arith) {
                    nu = walk;
                    arith.step(walk, 1);
                    if (kTickets && next == n_arith - 1) hand = atomicAdd(&p.hdr->ticket, 1u);
                    return;
                }
                if (!kTickets) { ended = true; nu.k = -1; return; }
                if (!ended) {
                    const int64_t tile = (int64_t)p.n_fixed * G + hand;
                    ended = tile >= p.ntiles;
                    if (!ended) {
                        hand = atomicAdd(&p.hdr->ticket, 1u);
                        nu = unit_of_tile(p, tile);
                    }
                }
                if (ended) { nu.k = -1; nu.s = nu.b = nu.cg = 0; }
            };
            auto post = [&]() {
                const int st = next % kStages;
                ++next;
                units[st] = nu;           // the producer itself reads it back when it stores the unit
                if (kTickets && next > p.n_fixed) mbar_arrive(bar_info(st));   // the other roles compute the first n_fixed
                if (nu.k < 0) return;
                const uint32_t base = smem_base + st * SM::kStageBytes;
                const int32_t c0 = nu.cg * Dc, c1 = nu.template row0<kBackward>(p), c2 = nu.b;
                mbar_arrive_expect_tx(bar_full(st), SM::kStageBytes);
                tma_load_3d(base, &map_alpha, bar_full(st), c0, c1, c2);
                tma_load_3d(base + kTileBytes, &map_x, bar_full(st), c0, c1, c2);
                if (kBackward) tma_load_3d(base + 2 * kTileBytes, &map_h, bar_full(st), c0, c1 - 1, c2);
                if (kGate) tma_load_3d(base + 2 * kTileBytes, &map_h, bar_full(st), c0, c1, c2);      // input gate
                ++issued;
            };
            // One loop for both the initial fill (slots 0 .. kStages-1) and the steady state, in which
            // slot i + kStages is described when unit i leaves its stage.
            int i = -kStages;
#pragma unroll 1
            for (; i < issued; ++i) {
                const int st = (i + kStages) % kStages;
                const uint32_t base = smem_base + st * SM::kStageBytes;
                prepare();                            // for slot i + kStages, which lives in this stage
                if (i >= 0) {
                    const Unit u = units[st];
                    const int32_t c0 = u.cg * Dc, c1 = u.template row0<kBackward>(p), c2 = u.b;
                    if (!ctl.wait(bar_done(st), (uint32_t)((i / kStages) & 1), FSS_STATUS_TMA_TIMEOUT)) break;
                    if (!kBackward) {
                        tma_store_3d(&map_out0, base + kTileBytes, c0, c1, c2);          // h
                    } else {
                        tma_store_3d(&map_out0, base + 2 * kTileBytes, c0, c1, c2);      // dalpha
                        tma_store_3d(&map_out1, base + kTileBytes, c0, c1, c2);          // dbeta
                    }
                    tma_commit();
                    if (nu.k >= 0) tma_wait_read_all();   // the stage may be overwritten once the store has read it
                }
                post();
            }
            // leave nothing in flight: loads that were issued but never consumed, and all stores
            if (i < issued) {
                for (int j = i < 0 ? 0 : i; j < issued; ++j) {
                    const uint32_t bar = bar_full(j % kStages);
                    const uint32_t par = (uint32_t)((j / kStages) & 1);
                    for (uint32_t it = 0; it < p.max_spins && !mbar_try_wait(bar, par); ++it) {}
                }
            }
            // the stores only have to be done READING shared memory before the CTA may leave; the
            // writes themselves are complete when the grid is
            tma_wait_read_all();
        }
    } else if (warp == kSummaryWarp) {
        // ============================================================ summary
        // Folds the eight warp summaries of every unit into the tile summary as soon as pass 1
        // has produced them, leaves it in shared memory for the look-back warps and publishes it
        // at once: successors of this tile can then fold it without waiting for the tile's own
        // carry resolution.  This warp never waits on anything outside its CTA.
        using AggPk = PacketGroup<2 * V, LPG>;
        constexpr int kTilePackets = (AggPk::kPackets + PacketGroup<V>::kPackets) * LPG;
        const uint32_t tag_agg = (epoch << 2) | kStateAggregate;
        Cursor cursor(p, ctl, units, bar_info(0));
        cursor.init(u0, 0, 1);
#pragma unroll 1
        for (int i = 0;; ++i) {
            const int g = i % kGens;
            if (!cursor.advance(i)) break;
            const Unit u = cursor.cur;
            const int64_t k = u.k;
            const bool last_block = u.s + 1 == (int32_t)p.S;
            const int32_t it_s = u.s;
            if (!ctl.wait(bar_agg(g), (uint32_t)((i / kGens) & 1), FSS_STATUS_LOOKBACK_TIMEOUT)) break;
            // Lane (q, cl) owns the kW consecutive row groups q*kW .. q*kW+kW-1 (one per pass-1 warp):
            // it folds them in scan order, the kSp lane groups are combined with one shuffle scan,
            // and every slot then receives the map of all groups BEFORE it (its exclusive prefix).
            // pc ends as the tile's own summary.
            VecF own_p[kW], own_c[kW];
#pragma unroll
            for (int w = 0; w < kW; ++w) { own_p[w] = agg_at(g, w, 0, lane); own_c[w] = agg_at(g, w, 1, lane); }
            float iP[V], iC[V];                           // own groups, then inclusive over the lane groups
#pragma unroll
            for (int v = 0; v < V; ++v) { iP[v] = 1.0f; iC[v] = 0.0f; }
#pragma unroll
            for (int ww = 0; ww < kW; ++ww) {
                const int w = kBackward ? kW - 1 - ww : ww;
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    iC[v] = fmaf(vec_get(own_p[w], v), iC[v], vec_get(own_c[w], v));
                    iP[v] *= vec_get(own_p[w], v);
                }
            }
#pragma unroll
            for (int d = 1; d < kSp; d <<= 1) {
                const bool valid = kBackward ? (q + d < kSp) : (q >= d);
                const int src = (kBackward ? lane + d * LPG : lane - d * LPG) & 31;
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    const float oP = __shfl_sync(0xffffffffu, iP[v], src);
                    const float oC = __shfl_sync(0xffffffffu, iC[v], src);
                    if (valid) { iC[v] = fmaf(iP[v], oC, iC[v]); iP[v] *= oP; }       // earlier groups first, then these
                }
            }
            float pc[2 * V], run[2 * V];                  // tile summary; map of the groups before this lane's
            {
                const bool has_prev = kBackward ? (q + 1 < kSp) : (q >= 1);
                const int prev = (kBackward ? lane + LPG : lane - LPG) & 31;
                const int last = (kBackward ? 0 : kSp - 1) * LPG + cl;      // lane group that ends the tile
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    const float eP = kSp > 1 ? __shfl_sync(0xffffffffu, iP[v], prev) : 1.0f;
                    const float eC = kSp > 1 ? __shfl_sync(0xffffffffu, iC[v], prev) : 0.0f;
                    run[v] = has_prev ? eP : 1.0f;
                    run[V + v] = has_prev ? eC : 0.0f;
                    pc[v] = kSp > 1 ? __shfl_sync(0xffffffffu, iP[v], last) : iP[v];
                    pc[V + v] = kSp > 1 ? __shfl_sync(0xffffffffu, iC[v], last) : iC[v];
                }
            }
#pragma unroll
            for (int ww = 0; ww < kW; ++ww) {
                const int w = kBackward ? kW - 1 - ww : ww;
                VecF ep, ec;
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    vec_set(ep, v, run[v]);
                    vec_set(ec, v, run[V + v]);
                    run[V + v] = fmaf(vec_get(own_p[w], v), run[V + v], vec_get(own_c[w], v));
                    run[v] *= vec_get(own_p[w], v);
                }
                agg_at(g, w, 0, lane) = ep;
                agg_at(g, w, 1, lane) = ec;
            }
            VecF sp, sc;
#pragma unroll
            for (int v = 0; v < V; ++v) { vec_set(sp, v, pc[v]); vec_set(sc, v, pc[V + v]); }
            sum_at(g, 0, lane) = sp;
            sum_at(g, 1, lane) = sc;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sum(g));
            if (!last_block && q == 0 && !(p.mute_first_block && it_s == 0))
                AggPk::store(p.packets + k * kTilePackets + cl, pc, tag_agg);
            // the row block's own product of alpha, for callers that stitch scans together
            if (p.block_prod && q == 0) {
                const int64_t dch = (int64_t)u.cg * Dc + cl * V;
                if (dch < p.D) {
                    const int64_t blk = kBackward ? (p.S - 1 - it_s) : it_s;
                    *reinterpret_cast<VecF *>(p.block_prod + ((int64_t)u.b * p.S + blk) * p.D + dch) = sp;
                }
            }
        }
    } else if (kGate && warp >= kGateWarp0) {
        // ============================================================ gates (gated forward only)
        // The alpha slot of a stage arrives holding r, the third slot i, the beta slot x.  These
        // warps turn them into alpha and beta in place as soon as the tile has landed, one warp per
        // row-group mapping of the pass-1 warps, so that the special-function work runs beside the
        // scan instead of inside it.  (Measured on the c4 shape, bf16: gates inside pass 1 0.44 ms,
        // here 0.40 ms; giving half of the rows back to the pass-1 warps 0.61 ms.)
        using Raw = typename Lane<T>::Raw;
        constexpr int kRowStride = kRowB / (int)sizeof(Raw);
        const int gw = warp - kGateWarp0;
        const int grp = q * kW + gw;
        constexpr bool kPairSwap = kRowB == 64;
        const bool odd_grp = kPairSwap && (q & 1);
        const int dsw = odd_grp ? kRowStride : 0;
        const uint32_t lane_off = (uint32_t)(grp * kR) * kRowB + (uint32_t)cl * kLaneBytes;
        Cursor cursor(p, ctl, units, bar_info(0));
        cursor.init(u0, 0, 1);
        // this lane's channel scales (a table made once per launch), always fetched one unit ahead so
        // that the load's latency never sits between a landed tile and its gates
        auto load_scales = [&](const Unit &un, float (&out)[V]) {
            const int64_t dch = (int64_t)un.cg * Dc + cl * V;
#pragma unroll
            for (int v = 0; v < V; ++v) out[v] = dch + v < p.D ? __ldg(p.lambda + dch + v) : 0.0f;
        };
        float gsc_next[V];
        load_scales(u0, gsc_next);
#pragma unroll 1
        for (int i = 0;; ++i) {
            const int st = i % kStages;
            if (!cursor.advance(i)) break;
            const Unit u = cursor.cur;
            const int32_t row0 = u.template row0<kBackward>(p);
            const bool head = (row0 == 0) && (grp == 0) && !p.continuation;
            const int64_t left = p.T - row0 - (int64_t)grp * kR;
            const int nvalid = left >= kR ? kR : (left > 0 ? (int)left : 0);
            float gsc[V];
#pragma unroll
            for (int v = 0; v < V; ++v) gsc[v] = gsc_next[v];
            if (cursor.next_known()) load_scales(cursor.nxt, gsc_next);
            if (!ctl.wait(bar_full(st), (uint32_t)((i / kStages) & 1), FSS_STATUS_TMA_TIMEOUT)) break;
            Raw *a_t = reinterpret_cast<Raw *>(smem_raw + st * SM::kStageBytes + lane_off);
            Raw *x_t = reinterpret_cast<Raw *>(smem_raw + st * SM::kStageBytes + kTileBytes + lane_off);
            const Raw *i_t = reinterpret_cast<const Raw *>(smem_raw + st * SM::kStageBytes + 2 * kTileBytes + lane_off);
            const bool edge_rows = __any_sync(0xffffffffu, head || nvalid < kR);
#pragma unroll 1
            for (int hb = 0; hb < kR / kRh; ++hb)
                gate_rows<T, kRowStride>(a_t, x_t, i_t, kRh * hb, dsw, odd_grp, gsc, head, nvalid, edge_rows);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_gate(st));
        }
    } else if (warp >= kLookbackWarp0) {
        // ============================================================ look-back
        // kLookbackWarps warps share the work units round-robin, so several carry resolutions
        // (each a few L2 round trips) are in flight per CTA.
        constexpr int NI = V;                          // floats of an inclusive descriptor
        constexpr int kWin = kWindow;
        using AggPk = PacketGroup<2 * V, LPG>;         // (P, C) of the tile scanned from zero
        using IncPk = PacketGroup<NI, LPG>;                 // state after the tile (and product up to it)
        constexpr int kTilePackets = (AggPk::kPackets + IncPk::kPackets) * LPG;
        const uint32_t tag_agg = (epoch << 2) | kStateAggregate;
        const uint32_t tag_inc = (epoch << 2) | kStateInclusive;
        const int lb = warp - kLookbackWarp0;
        const int ch = cl * V;      // first channel of this lane inside the tile
        auto agg_packets = [&](int64_t k) { return p.packets + k * kTilePackets + cl; };
        auto inc_packets = [&](int64_t k) { return p.packets + k * kTilePackets + AggPk::kPackets * LPG + cl; };

        // The predecessor's inclusive descriptor is fetched one of this warp's units ahead of its use
        // (as soon as the producer has described that unit) and, if it was not there yet, once more
        // when the unit starts.
        typename IncPk::Raw pre;
        bool have_pre = false;
        Cursor cursor(p, ctl, units, bar_info(0));
        cursor.init(u0, lb, kLookbackWarps);
        auto first_look = [&]() {         // start reading the inclusive state before this warp's next unit
            have_pre = cursor.next_known() && cursor.nxt.s > 0;
            if (have_pre) IncPk::load_raw(inc_packets((int64_t)cursor.nxt.k - p.ncols), pre);
        };
        first_look();

#pragma unroll 1
        for (int i = lb;; i += kLookbackWarps) {
            const int g = i % kGens;
            const bool had_pre = have_pre;
            if (!cursor.advance(i)) break;
            const Unit u = cursor.cur;
            const int64_t k = u.k;
            const int32_t s = u.s, b = u.b;
            const int64_t dch = (int64_t)u.cg * Dc + ch;     // channel in the tensor
            const bool ch_ok = dch < p.D;
            float cur[NI];
            bool hit = false;
            if (had_pre) hit = __all_sync(0xffffffffu, IncPk::decode(pre, cur, tag_inc));
            first_look();                  // for this warp's next unit (decoded when that unit starts)
            // While pass 1 and the summary warp are still working on this unit, keep asking for the
            // predecessor's inclusive state: this warp has nothing else to do, and in the common case
            // the answer is there before the summary is, so the carry costs no extra round trip.
            if (s > 0) {
                uint32_t polls = 0;
                while (!hit) {      // every exit below is decided by a warp vote
                    const bool summary_in = mbar_test_wait(bar_sum(g), (uint32_t)((i / kGens) & 1));
                    if (__all_sync(0xffffffffu, summary_in)) break;
                    typename IncPk::Raw again;
                    IncPk::load_raw(inc_packets(k - p.ncols), again);
                    hit = __all_sync(0xffffffffu, IncPk::decode(again, cur, tag_inc));
                    if (!hit && (++polls & 31u) == 0u && (polls >= p.max_spins || __any_sync(0xffffffffu, ctl.aborted()))) break;
                }
            }
            if (!ctl.wait(bar_sum(g), (uint32_t)((i / kGens) & 1), FSS_STATUS_LOOKBACK_TIMEOUT)) break;
            if (s > 0 && !hit) {       // one more look now that the summary is in
                typename IncPk::Raw again;
                IncPk::load_raw(inc_packets(k - p.ncols), again);
                hit = __all_sync(0xffffffffu, IncPk::decode(again, cur, tag_inc));
            }

            // the tile's summary, folded by the summary warp
            float Pt[V], Ct[V];
            {
                const VecF sp = sum_at(g, 0, lane), sc = sum_at(g, 1, lane);
#pragma unroll
                for (int v = 0; v < V; ++v) { Pt[v] = vec_get(sp, v); Ct[v] = vec_get(sc, v); }
            }

            // ---- the state entering this tile
            float cin[V];
            bool ok = true;
            auto state0 = [&](int v) {
                return (p.state_in && ch_ok) ? p.state_in[(int64_t)b * p.D + dch + v] : 0.0f;
            };
            if (s == 0) {
#pragma unroll
                for (int v = 0; v < V; ++v) cin[v] = state0(v);
            } else if (hit) {
#pragma unroll
                for (int v = 0; v < V; ++v) cin[v] = cur[v];
            } else {
                float Pa[V], Ca[V];          // map of the tiles between the predecessor at q and this one
#pragma unroll
                for (int v = 0; v < V; ++v) { Pa[v] = 1.0f; Ca[v] = 0.0f; }
                int64_t q = k - p.ncols;
                uint32_t spins = 0;
                bool found = false;
                while (!found) {
                    // read up to kWin predecessors in one round trip
                    float inc[kWin][NI], ag[kWin][2 * V];
                    bool inc_ok[kWin], ag_ok[kWin];
#pragma unroll
                    for (int j = 0; j < kWin; ++j) {
                        const int64_t qj = q - j * p.ncols;
                        inc_ok[j] = false; ag_ok[j] = false;
                        if (qj >= 0) {
                            inc_ok[j] = IncPk::load(inc_packets(qj), inc[j], tag_inc);
                            ag_ok[j] = AggPk::load(agg_packets(qj), ag[j], tag_agg);
                        }
                    }
                    int adv = 0;          // predecessors folded in this round
                    bool stop = false;
#pragma unroll
                    for (int j = 0; j < kWin; ++j) {
                        const int64_t qj = q - j * p.ncols;     // warp-uniform
                        if (found || stop) {
                            // nothing more to do in this round
                        } else if (qj < 0) {
                            stop = true;
                        } else if (__all_sync(0xffffffffu, inc_ok[j])) {
#pragma unroll
                            for (int v = 0; v < V; ++v) cin[v] = fmaf(Pa[v], inc[j][v], Ca[v]);
                            found = true;
                        } else if (!p.deterministic && __all_sync(0xffffffffu, ag_ok[j])) {
#pragma unroll
                            for (int v = 0; v < V; ++v) {
                                Ca[v] = fmaf(Pa[v], ag[j][V + v], Ca[v]);
                                Pa[v] *= ag[j][v];
                            }
                            adv = j + 1;
                            if (qj - p.ncols < 0) {      // folded everything down to row block 0
#pragma unroll
                                for (int v = 0; v < V; ++v) cin[v] = fmaf(Pa[v], state0(v), Ca[v]);
                                found = true;
                            }
                        } else {
                            stop = true;                 // not published yet: poll again from here
                        }
                    }
                    if (found) break;
                    q -= (int64_t)adv * p.ncols;
                    if (adv == 0) {
                        ++spins;
                        if ((spins & 15u) == 0u && __any_sync(0xffffffffu, ctl.aborted())) { ok = false; break; }
                        if (spins >= p.max_spins) {
                            if (lane == 0) ctl.give_up(FSS_STATUS_LOOKBACK_TIMEOUT);
                            ok = false;
                            break;
                        }
                        __nanosleep(32);
                    }
                }
                if (!ok) break;
            }
            // ---- hand the entering state to the consumers: each warp applies the exclusive prefix
            // the summary warp left in its slot
            {
                VecF vin;
#pragma unroll
                for (int v = 0; v < V; ++v) vec_set(vin, v, cin[v]);
                sum_at(g, 2, lane) = vin;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_carry(g));

            // ---- publish the inclusive descriptor: the state after this tile
            float out[NI];
#pragma unroll
            for (int v = 0; v < V; ++v) out[v] = fmaf(Pt[v], cin[v], Ct[v]);
            if (s + 1 < (int32_t)p.S && q == 0 && !(p.mute_first_block && s == 0)) IncPk::store(inc_packets(k), out, tag_inc);

            if (ch_ok && q == 0) {
                VecF vo;
#pragma unroll
                for (int v = 0; v < V; ++v) vec_set(vo, v, out[v]);
                if (p.block_state) {
                    const int64_t blk = kBackward ? (p.S - 1 - s) : s;
                    *reinterpret_cast<VecF *>(p.block_state + ((int64_t)b * p.S + blk) * p.D + dch) = vo;
                }
                if (s + 1 == (int32_t)p.S && p.state_out)
                    *reinterpret_cast<VecF *>(p.state_out + (int64_t)b * p.D + dch) = vo;
            }
        }
    } else if (warp < kPass2Warp0) {
        // ============================================================ pass 1
        // Scans this warp's rows of every unit from a zero state as soon as the tile has landed
        // and leaves (P, C); never waits for a carry, only for the summary buffers to be free.
        using Raw = typename Lane<T>::Raw;
        constexpr int kRowStride = kRowB / (int)sizeof(Raw);
        const int grp = q * kW + warp;             // this lane's row group inside the tile
        constexpr bool kPairSwap = kRowB == 64;
        const bool odd_grp = kPairSwap && (q & 1);
        const int dsw = odd_grp ? kRowStride : 0;
        const uint32_t lane_off = (uint32_t)(grp * kR) * kRowB + (uint32_t)cl * kLaneBytes;
        Cursor cursor(p, ctl, units, bar_info(0));
        cursor.init(u0, 0, 1);
#pragma unroll 1
        for (int i = 0;; ++i) {
            const int st = i % kStages, g = i % kGens;
            if (!cursor.advance(i)) break;
            const Unit u = cursor.cur;
            const int32_t row0 = u.template row0<kBackward>(p);
            const bool head = (row0 == 0) && (grp == 0) && !p.continuation;
            // rows of this group that exist in the sequence (fewer than kR only in the last row block)
            const int64_t left = p.T - row0 - (int64_t)grp * kR;
            const int nvalid = left >= kR ? kR : (left > 0 ? (int)left : 0);
            if (i >= kGens) {      // the summary buffers of this generation are free once pass 2 of unit i-kGens is done
                const int o = i - kGens;
                if (!ctl.wait(bar_done((int)(o % kStages)), (uint32_t)((o / kStages) & 1), FSS_STATUS_LOOKBACK_TIMEOUT)) break;
            }
            if (!ctl.wait(bar_full(st), (uint32_t)((i / kStages) & 1), FSS_STATUS_TMA_TIMEOUT)) break;
            Raw *a_t = reinterpret_cast<Raw *>(smem_raw + st * SM::kStageBytes + lane_off);
            Raw *x_t = reinterpret_cast<Raw *>(smem_raw + st * SM::kStageBytes + kTileBytes + lane_off);
            // gated forward: the gate warps turn the stage into (alpha, beta), edge rows included
            if (kGate && !ctl.wait(bar_gate(st), (uint32_t)((i / kStages) & 1), FSS_STATUS_TMA_TIMEOUT)) break;
            // row 0 of the whole sequence: alpha_0 is not part of the recurrence
            if (!kGate && head) a_t[0] = Lane<T>::zero();
            // rows past the end of the sequence arrive zero-filled; alpha = 1 (beta, grad = 0) makes
            // them the identity for both passes, so the state after the tile is the state after
            // the last real row
            if (!kGate && nvalid < kR) {
                for (int r = nvalid; r < kR; ++r) a_t[r * kRowStride] = Lane<T>::one();
            }
            float P[V], C[V];
#pragma unroll
            for (int v = 0; v < V; ++v) { P[v] = 1.0f; C[v] = 0.0f; }
#pragma unroll 1
            for (int hb = 0; hb < kR / kRh; ++hb) {
                const int base = kBackward ? kR - kRh * (hb + 1) : kRh * hb;     // rows of this batch
                Raw ra[kRh], rx[kRh];
#pragma unroll
                for (int r = 0; r < kRh; ++r) {
                    ra[r] = pair_slot<kRowStride>(a_t, base + r, dsw);
                    rx[r] = pair_slot<kRowStride>(x_t, base + r, dsw);
                }
                pair_fix<kPairSwap>(ra, odd_grp);
                pair_fix<kPairSwap>(rx, odd_grp);
#pragma unroll
                for (int j = 0; j < kRh; ++j) {
                    const int r = kBackward ? kRh - 1 - j : j;
                    float a[V], x[V];
                    Lane<T>::unpack(ra[r], a);
                    Lane<T>::unpack(rx[r], x);
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        if (!kBackward) C[v] = fmaf(a[v], C[v], x[v]);
                        else C[v] = a[v] * (x[v] + C[v]);
                        P[v] *= a[v];
                    }
                }
            }
            VecF vp, vc;
#pragma unroll
            for (int v = 0; v < V; ++v) { vec_set(vp, v, P[v]); vec_set(vc, v, C[v]); }
            agg_at(g, warp, 0, lane) = vp;
            agg_at(g, warp, 1, lane) = vc;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_agg(g));
        }
    } else {
        // ============================================================ pass 2
        // Re-scans this warp's rows from the true entering state and writes the results in place.
        using Raw = typename Lane<T>::Raw;
        constexpr int kRowStride = kRowB / (int)sizeof(Raw);
        const int w2 = warp - kPass2Warp0;
        const int grp = q * kW + w2;
        constexpr bool kPairSwap = kRowB == 64;
        const bool odd_grp = kPairSwap && (q & 1);
        const int dsw = odd_grp ? kRowStride : 0;
        const uint32_t lane_off = (uint32_t)(grp * kR) * kRowB + (uint32_t)cl * kLaneBytes;
        const int ch = cl * V;
        Cursor cursor(p, ctl, units, bar_info(0));
        cursor.init(u0, 0, 1);
#pragma unroll 1
        for (int i = 0;; ++i) {
            const int st = i % kStages, g = i % kGens;
            if (!cursor.advance(i)) break;
            const Unit u = cursor.cur;
            const bool head = (u.template row0<kBackward>(p) == 0) && (grp == 0);
            const int32_t b = u.b;
            const int64_t dch = (int64_t)u.cg * Dc + ch;
            const Raw *a_t = reinterpret_cast<const Raw *>(smem_raw + st * SM::kStageBytes + lane_off);
            Raw *x_t = reinterpret_cast<Raw *>(smem_raw + st * SM::kStageBytes + kTileBytes + lane_off);
            Raw *h_t = reinterpret_cast<Raw *>(smem_raw + st * SM::kStageBytes + 2 * kTileBytes + lane_off);
            // the carry barrier is reached through pass 1 of this unit, so the tile is resident
            if (!ctl.wait(bar_carry(g), (uint32_t)((i / kGens) & 1), FSS_STATUS_LOOKBACK_TIMEOUT)) break;
            // state entering this warp's rows = (map of the warps before it)(state entering the tile)
            float stv[V];
            {
                const VecF ep = agg_at(g, w2, 0, lane), ec = agg_at(g, w2, 1, lane), vin = sum_at(g, 2, lane);
#pragma unroll
                for (int v = 0; v < V; ++v) stv[v] = fmaf(vec_get(ep, v), vec_get(vin, v), vec_get(ec, v));
            }
#pragma unroll 1
            for (int hb = 0; hb < kR / kRh; ++hb) {
                const int base = kBackward ? kR - kRh * (hb + 1) : kRh * hb;
                Raw ra[kRh], rx[kRh];
#pragma unroll
                for (int r = 0; r < kRh; ++r) {
                    ra[r] = pair_slot<kRowStride>(a_t, base + r, dsw);
                    rx[r] = pair_slot<kRowStride>(x_t, base + r, dsw);
                }
                pair_fix<kPairSwap>(ra, odd_grp);
                pair_fix<kPairSwap>(rx, odd_grp);
                if (!kBackward) {
#pragma unroll
                    for (int r = 0; r < kRh; ++r) {
                        float a[V], x[V];
                        Lane<T>::unpack(ra[r], a);
                        Lane<T>::unpack(rx[r], x);
#pragma unroll
                        for (int v = 0; v < V; ++v) stv[v] = fmaf(a[v], stv[v], x[v]);
                        if (kPairSwap) rx[r] = Lane<T>::pack(stv);
                        else x_t[(base + r) * kRowStride] = Lane<T>::pack(stv);
                    }
                    if (kPairSwap) {
                        pair_fix<kPairSwap>(rx, odd_grp);
#pragma unroll
                        for (int r = 0; r < kRh; ++r) pair_slot<kRowStride>(x_t, base + r, dsw) = rx[r];
                    }
                } else {
                    Raw rh[kRh];
#pragma unroll
                    for (int r = 0; r < kRh; ++r) rh[r] = pair_slot<kRowStride>(h_t, base + r, dsw);
                    pair_fix<kPairSwap>(rh, odd_grp);
                    if (base == 0 && head && p.continuation && p.h_prev) {    // h_{-1} of a continued sequence
                        float hp[V];
#pragma unroll
                        for (int v = 0; v < V; ++v) hp[v] = (dch < p.D) ? p.h_prev[(int64_t)b * p.D + dch + v] : 0.0f;
                        rh[0] = Lane<T>::pack(hp);
                    }
#pragma unroll
                    for (int j = 0; j < kRh; ++j) {
                        const int r = kRh - 1 - j;
                        float a[V], x[V], hp[V], da[V], dh[V];
                        Lane<T>::unpack(ra[r], a);
                        Lane<T>::unpack(rx[r], x);
                        Lane<T>::unpack(rh[r], hp);
#pragma unroll
                        for (int v = 0; v < V; ++v) {
                            dh[v] = x[v] + stv[v];
                            da[v] = dh[v] * hp[v];
                            stv[v] = a[v] * dh[v];
                        }
                        if (base + r == 0 && head && !p.continuation) {
#pragma unroll
                            for (int v = 0; v < V; ++v) da[v] = 0.0f;
                        }
                        if (kPairSwap) { rx[r] = Lane<T>::pack(dh); rh[r] = Lane<T>::pack(da); }
                        else {
                            x_t[(base + r) * kRowStride] = Lane<T>::pack(dh);
                            h_t[(base + r) * kRowStride] = Lane<T>::pack(da);
                        }
                    }
                    if (kPairSwap) {
                        pair_fix<kPairSwap>(rx, odd_grp);
                        pair_fix<kPairSwap>(rh, odd_grp);
#pragma unroll
                        for (int r = 0; r < kRh; ++r) {
                            pair_slot<kRowStride>(x_t, base + r, dsw) = rx[r];
                            pair_slot<kRowStride>(h_t, base + r, dsw) = rh[r];
                        }
                    }
                }
            }
            fence_proxy_async();      // make the in-place results visible to the TMA store
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_done(st));
        }
    }

    // ---- leave: the last CTA advances the epoch, which invalidates every descriptor of this launch
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t prev = atomicAdd(&p.hdr->done, 1u);
        if (prev + 1 == gridDim.x) {
            p.hdr->done = 0;
            p.hdr->ticket = 0;
            p.hdr->abort = 0;
            __threadfence();
            p.hdr->epoch = ld_volatile(&p.hdr->epoch) + 1u;
        }
    }
}

// ------------------------------------------------------------------ host side
// Tile shape for a problem: split s gives tiles of 64*s rows x 256/s bytes.  Narrow, tall tiles
// multiply the number of columns; with fewer columns than about two per SM several row blocks of
// one column are in flight at once and the carry chain between them limits the speed.
inline int choose_split(int dtype, int64_t B, int64_t T, int64_t D) {
    static const int env = [] { const char *e = getenv("FSS_B200_SPLIT"); return e ? atoi(e) : 0; }();
    if (env == 1 || env == 2 || env == 4) return env;
    const int64_t row_bytes = D * (dtype == FSS_DTYPE_BF16 ? 2 : 4);
    const int64_t cols = B * ceil_div(row_bytes, kRowBytes);
    int s = 1;
    while (s < 4 && cols * s < 2 * 148 && row_bytes >= kRowBytes / s && T >= 2 * kTc * s * 2) s *= 2;
    return s;
}
// Tile order.  Returns how many units at the END of a CTA's share are handed out by the global
// counter instead of by arithmetic (see the producer): 0 = fixed order throughout, a large value =
// everything after the first ring of stages.  Measured on B200: SMs are not served equally by the
// memory system, so with a fixed order the first CTA finishes several microseconds before the
// last; tiles taken by ticket let the fast SMs take more.  The descriptors that ticketed units
// travel in cost a little per unit, which is why short launches only ticket their tail.
// The forward kernel (six stages in flight) lost 2-15 % with any number of ticketed units on every
// workload measured, so it keeps the fixed order.  FSS_B200_TAIL=<n> forces n for both directions
// (0 = fixed order); FSS_B200_TICKETS=0 / 1 forces none / all for the backward kernel.
constexpr int kAllTickets = 1 << 30;
inline int choose_tail(int dtype, bool backward, int64_t B, int64_t T, int64_t D) {
    static const int env_tail = [] { const char *e = getenv("FSS_B200_TAIL"); return e ? atoi(e) : -1; }();
    static const int env_all = [] { const char *e = getenv("FSS_B200_TICKETS"); return !e ? -1 : (e[0] == '1' ? 1 : 0); }();
    if (env_tail >= 0) return env_tail;
    if (!backward) return 0;
    if (env_all >= 0) return env_all ? kAllTickets : 0;
    const int64_t bytes = B * T * D * (dtype == FSS_DTYPE_BF16 ? 2 : 4);
    return bytes >= ((int64_t)96 << 20) ? kAllTickets : 0;
}
inline int64_t block_rows(int dtype, int64_t B, int64_t T, int64_t D) { return (int64_t)kTc * choose_split(dtype, B, T, D); }

template <typename T> inline int64_t channel_groups(int64_t D) { return ceil_div(D, Cfg<T>::Dc); }

// descriptor packets per tile: the aggregate (P, C) and the inclusive state
template <typename T> constexpr int packets_per_tile() {
    return (PacketGroup<2 * Cfg<T>::V>::kPackets + PacketGroup<Cfg<T>::V>::kPackets) * 32;
}
inline size_t workspace_bytes(int64_t B, int64_t T, int64_t D, int dtype) {
    const int Dc = dtype == FSS_DTYPE_BF16 ? Cfg<bf16>::Dc : Cfg<float>::Dc;
    const int per_tile = dtype == FSS_DTYPE_BF16 ? packets_per_tile<bf16>() : packets_per_tile<float>();
    size_t worst = 0;
    for (int s = 1; s <= 4; s *= 2) {       // any tile shape the launcher may pick
        const int64_t ntiles = B * ceil_div(D, Dc / s) * ceil_div(T, (int64_t)kTc * s);
        const size_t need = (size_t)ntiles * (per_tile / s) * 16;
        if (need > worst) worst = need;
    }
    return worst;
}
// float scratch a launch may use: per-block products when the caller asks for the total product
// without providing a block array
inline size_t float_scratch_bytes(int64_t B, int64_t T, int64_t D) {
    return (size_t)(B * ceil_div(T, (int64_t)kTc) * D) * sizeof(float);
}

// What TMA needs: 16-byte aligned bases and strides, extents that fit its 32-bit coordinates.
template <typename T>
inline bool layout_ok(int64_t B, int64_t Tn, int64_t D, std::initializer_list<const fss_view *> views) {
    constexpr int64_t per16 = 16 / (int64_t)sizeof(T);
    if (D % per16) return false;
    if (Tn > (1LL << 30) || D > (1LL << 30) || B > (1LL << 30)) return false;
    for (const fss_view *v : views) {
        if (!v || !aligned16(v->ptr)) return false;
        if (v->stride_t % per16 || (B > 1 && v->stride_b % per16)) return false;
        if ((v->stride_t * (int64_t)sizeof(T)) >= (1LL << 40)) return false;
        if (B > 1 && (v->stride_b * (int64_t)sizeof(T)) >= (1LL << 40)) return false;
    }
    return true;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// 3-D map (channels, rows, batch) with a (Dc, kTc, 1) box; out-of-range elements read as zero
// and are dropped on store.
template <typename T>
inline bool make_map(CUtensorMap *map, const fss_view *v, int64_t B, int64_t Tn, int64_t D, int split, std::string *err) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { *err = "cuTensorMapEncodeTiled entry point not found"; return false; }
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)Tn, (cuuint64_t)B};
    const int64_t sb = B > 1 ? v->stride_b : v->stride_t * Tn;
    const cuuint64_t strides[2] = {(cuuint64_t)(v->stride_t * (int64_t)sizeof(T)),
                                   (cuuint64_t)(sb * (int64_t)sizeof(T))};
    const cuuint32_t box[3] = {(cuuint32_t)(Cfg<T>::Dc / split), (cuuint32_t)(kTc * split), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapDataType dt = sizeof(T) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const CUresult r = fn(map, dt, 3, v->ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        *err = "cuTensorMapEncodeTiled returned " + std::to_string((int)r) + " for ptr " +
               std::to_string((unsigned long long)(uintptr_t)v->ptr) + " dims " + std::to_string(D) + "x" +
               std::to_string(Tn) + "x" + std::to_string(B) + " strides " + std::to_string(strides[0]) + "," +
               std::to_string(strides[1]);
        return false;
    }
    return true;
}

// Encoding a descriptor is a driver call; a training loop presents the same few tensors (same
// address, shape and strides) launch after launch, so each host thread keeps the descriptors it
// built last: 16 sets x 4 ways, keyed by everything the encoding depends on.  A descriptor holds
// no reference to the memory it describes, so an entry stays valid when the buffer is freed and
// the address is reused for a tensor of the same geometry.
struct MapKey {
    const void *ptr;
    int64_t B, T, D, sb, st;
    int32_t split, esize;
    bool operator==(const MapKey &o) const {
        return ptr == o.ptr && B == o.B && T == o.T && D == o.D && sb == o.sb && st == o.st && split == o.split &&
               esize == o.esize;
    }
};
struct MapCache {
    static constexpr int kSets = 16, kWays = 4;
    struct Slot { MapKey key; CUtensorMap map; bool valid; };
    Slot slots[kSets][kWays] = {};
    uint8_t next[kSets] = {};
};
template <typename T>
inline const CUtensorMap *cached_map(const fss_view *v, int64_t B, int64_t Tn, int64_t D, int split, std::string *err) {
    static thread_local MapCache cache;
    const MapKey key{v->ptr, B, Tn, D, v->stride_b, v->stride_t, split, (int32_t)sizeof(T)};
    const uintptr_t a = reinterpret_cast<uintptr_t>(v->ptr);
    const int set = (int)(((a >> 9) ^ (a >> 21) ^ (uintptr_t)split) % MapCache::kSets);
    for (auto &slot : cache.slots[set])
        if (slot.valid && slot.key == key) return &slot.map;
    auto &slot = cache.slots[set][cache.next[set]];
    cache.next[set] = (uint8_t)((cache.next[set] + 1) % MapCache::kWays);
    slot.valid = false;
    if (!make_map<T>(&slot.map, v, B, Tn, D, split, err)) return nullptr;
    slot.key = key;
    slot.valid = true;
    return &slot.map;
}

// CTAs that fit the device at once (one per SM with these shared-memory sizes), per device.
template <typename T, bool kBackward, int kSp, bool kTickets, bool kGate> inline int resident_ctas(int device, int smem_bytes, cudaError_t *err) {
    static std::mutex mu;
    static int cached[64];
    static bool have[64];
    std::lock_guard<std::mutex> lock(mu);
    if (device < 0 || device >= 64) { *err = cudaErrorInvalidDevice; return 0; }
    if (!have[device]) {
        auto kern = scan_kernel<T, kBackward, kSp, kTickets, kGate>;
        *err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (*err != cudaSuccess) return 0;
        int per_sm = 0, sms = 0;
        *err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads_of<kGate>(), smem_bytes);
        if (*err != cudaSuccess) return 0;
        *err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (*err != cudaSuccess) return 0;
        cached[device] = per_sm * sms;
        have[device] = true;
    }
    *err = cudaSuccess;
    return cached[device];
}

template <typename T, bool kBackward, int kSp, bool kTickets, bool kGate = false>
inline int launch_split(const fss_scan_ctx *ctx, const WsPlan &ws, int64_t B, int64_t Tn, int64_t D,
                  const fss_view *alpha, const fss_view *x, const fss_view *h, const fss_view *out0,
                  const fss_view *out1, Params p, int tail, std::string *err_text) {
    constexpr int kTensors = (kBackward || kGate) ? 3 : 2;
    constexpr int kStages = (kBackward || kGate) ? kStagesBwd : kStagesFwd;
    constexpr int smem_bytes = Smem<kTensors, kStages>::kBytes;
    constexpr int Dc = Cfg<T>::Dc / kSp;

    // copies: a later look-up may evict the slot an earlier pointer refers to
    CUtensorMap m_alpha, m_x, m_h, m_o0, m_o1;
    auto fetch = [&](CUtensorMap *dst, const fss_view *v) {
        const CUtensorMap *m = cached_map<T>(v, B, Tn, D, kSp, err_text);
        if (m) *dst = *m;
        return m != nullptr;
    };
    if (!fetch(&m_alpha, alpha) || !fetch(&m_x, x) || !fetch(&m_o0, out0)) return FSS_E_TENSORMAP;
    if (kBackward) {
        if (!fetch(&m_h, h) || !fetch(&m_o1, out1)) return FSS_E_TENSORMAP;
    } else if (kGate) {
        if (!fetch(&m_h, h)) return FSS_E_TENSORMAP;      // the input gate
        m_o1 = m_o0;
    } else {
        m_h = m_alpha; m_o1 = m_o0;
    }

    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) { *err_text = cudaGetErrorString(e); return FSS_E_DEVICE; }
    const int resident = resident_ctas<T, kBackward, kSp, kTickets, kGate>(device, smem_bytes, &e);
    if (e != cudaSuccess || resident < 1) { *err_text = cudaGetErrorString(e); return FSS_E_LAUNCH; }

    p.B = B; p.T = Tn; p.D = D;
    p.ncg = ceil_div(D, Dc);
    p.ncols = B * p.ncg;
    p.S = ceil_div(Tn, (int64_t)kTc * kSp);
    p.tile_rows = kTc * kSp;
    p.ntiles = p.ncols * p.S;
    if (p.ntiles > 0x7fffffffLL) return FSS_E_SHAPE;      // tile numbers travel as 32-bit values
    if ((size_t)p.ntiles * (packets_per_tile<T>() / kSp) * 16 > ws.packet_bytes) return FSS_E_WORKSPACE;
    p.hdr = reinterpret_cast<Header *>(ws.hdr);
    p.packets = reinterpret_cast<uint4 *>(ws.packets);
    p.status = ctx->status;
    p.continuation = (ctx->flags & FSS_FLAG_CONTINUATION) ? 1 : 0;
    p.max_spins = (ctx->flags & FSS_FLAG_TEST_SHORT_WAITS) ? 4096u : kMaxSpins;
    p.mute_first_block = (ctx->flags & FSS_FLAG_TEST_MUTE_FIRST_BLOCK) ? 1 : 0;
    p.deterministic = (ctx->flags & FSS_FLAG_DETERMINISTIC) ? 1 : 0;
    p.hold_dependents = (ctx->flags & FSS_FLAG_HOLD_DEPENDENTS) ? 1 : 0;

    const unsigned grid = (unsigned)(p.ntiles < resident ? p.ntiles : resident);
    p.grid = grid;
    p.units_q = (int32_t)(p.ntiles / grid);
    p.units_r = (int32_t)(p.ntiles % grid);
    p.grid_q = (int32_t)(grid / p.ncols);
    p.grid_b = (int32_t)((grid % p.ncols) / p.ncg);
    p.grid_cg = (int32_t)((grid % p.ncols) % p.ncg);
    // every CTA owns at least units_q tiles in the fixed order; the last `tail` of those, and
    // everything after them, go by ticket (at least the first ring stays fixed: its loads start
    // before anything else is known)
    {
        const int32_t ring = p.units_q < kStages ? p.units_q : kStages;
        const int64_t keep = (int64_t)p.units_q - tail;
        p.n_fixed = kTickets ? (int32_t)(keep > ring ? keep : ring) : p.units_q + 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads_of<kGate>());
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = (cudaStream_t)ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    // Programmatic dependent launch: a launch with this attribute may start its set-up while the
    // launch before it on the stream drains (it still waits for that launch's completion before it
    // touches global memory).  Measured on B200: forward launches always gain (1-2 % on c2 / c3);
    // backward launches gain only when they are short (up to 14 % at one or two tiles per CTA) and
    // lose about 3 % when they are long, so those keep the ordinary launch.  FSS_B200_PDL=0 / 1
    // forces it off / on for both directions.
    constexpr int64_t kPdlMaxUnits = 8;
    static const int pdl_env = [] { const char *e = getenv("FSS_B200_PDL"); return !e ? -1 : (e[0] == '1' ? 1 : 0); }();
    const bool use_pdl = pdl_env >= 0 ? pdl_env == 1 : (!kBackward || p.ntiles <= kPdlMaxUnits * (int64_t)grid);
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, scan_kernel<T, kBackward, kSp, kTickets, kGate>, m_alpha, m_x, m_h, m_o0, m_o1, p);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) { *err_text = std::string("look-back launch: ") + cudaGetErrorString(e); return FSS_E_LAUNCH; }
    return FSS_OK;
}

template <typename T, bool kBackward>
inline int launch(const fss_scan_ctx *ctx, const WsPlan &ws, int64_t B, int64_t Tn, int64_t D,
                  const fss_view *alpha, const fss_view *x, const fss_view *h, const fss_view *out0,
                  const fss_view *out1, Params p, std::string *err_text) {
    const int dtype = sizeof(T) == 2 ? FSS_DTYPE_BF16 : FSS_DTYPE_F32;
    const int tail = choose_tail(dtype, kBackward, B, Tn, D);
#define FSS_LAUNCH_SPLIT(SP)                                                                                       \
    return tail > 0 ? launch_split<T, kBackward, SP, true>(ctx, ws, B, Tn, D, alpha, x, h, out0, out1, p, tail, err_text) \
                    : launch_split<T, kBackward, SP, false>(ctx, ws, B, Tn, D, alpha, x, h, out0, out1, p, 0, err_text)
    switch (choose_split(dtype, B, Tn, D)) {
    case 4: FSS_LAUNCH_SPLIT(4);
    case 2: FSS_LAUNCH_SPLIT(2);
    default: FSS_LAUNCH_SPLIT(1);
    }
#undef FSS_LAUNCH_SPLIT
}

// prod[b, d] = product over the row blocks of block_prod[b, :, d].  A CTA owns 8 channel vectors
// (float4) of one batch row; its 64 thread rows split the blocks, so that every thread has only a
// handful of independent loads, and combine through shared memory.
constexpr int kProdSlices = 64, kProdVecs = 8;
__global__ void __launch_bounds__(kProdSlices * kProdVecs)
column_product(const float *__restrict__ block_prod, float *__restrict__ prod, int64_t S, int64_t D) {
    __shared__ float4 part[kProdSlices][kProdVecs];
    const int vec = threadIdx.x % kProdVecs, slice = threadIdx.x / kProdVecs;
    const int64_t b = blockIdx.y;
    const int64_t d0 = ((int64_t)blockIdx.x * kProdVecs + vec) * 4;
    float4 acc = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    if (d0 < D) {
        const float *base = block_prod + b * S * D + d0;
        const bool vec_ok = d0 + 4 <= D && (D % 4 == 0) && (reinterpret_cast<uintptr_t>(base) & 15u) == 0;
#pragma unroll 4
        for (int64_t s = slice; s < S; s += kProdSlices) {
            float4 v;
            if (vec_ok) {
                v = *reinterpret_cast<const float4 *>(base + s * D);
            } else {
                v.x = base[s * D];
                v.y = d0 + 1 < D ? base[s * D + 1] : 1.0f;
                v.z = d0 + 2 < D ? base[s * D + 2] : 1.0f;
                v.w = d0 + 3 < D ? base[s * D + 3] : 1.0f;
            }
            acc.x *= v.x; acc.y *= v.y; acc.z *= v.z; acc.w *= v.w;
        }
    }
    part[slice][vec] = acc;
    __syncthreads();
    // tree over the slices (the order of the factors is fixed, so the result is reproducible)
    for (int half = kProdSlices / 2; half > 0; half /= 2) {
        if (slice < half) {
            const float4 o = part[slice + half][vec];
            float4 m = part[slice][vec];
            m.x *= o.x; m.y *= o.y; m.z *= o.z; m.w *= o.w;
            part[slice][vec] = m;
        }
        __syncthreads();
    }
    if (slice == 0 && d0 < D) {
        const float4 r = part[0][vec];
        float *out = prod + b * D + d0;
        out[0] = r.x;
        if (d0 + 1 < D) out[1] = r.y;
        if (d0 + 2 < D) out[2] = r.z;
        if (d0 + 3 < D) out[3] = r.w;
    }
}
inline int launch_column_product(const float *block_prod, float *prod, int64_t B, int64_t S, int64_t D, cudaStream_t stream,
                                 std::string *err_text) {
    if (B > 65535) { *err_text = "product of alpha: more than 65535 batch rows"; return FSS_E_SHAPE; }
    const dim3 grid((unsigned)ceil_div(D, 4 * kProdVecs), (unsigned)B);
    column_product<<<grid, kProdSlices * kProdVecs, 0, stream>>>(block_prod, prod, S, D);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { *err_text = std::string("product launch: ") + cudaGetErrorString(e); return FSS_E_LAUNCH; }
    return FSS_OK;
}

template <typename T>
inline int forward(const fss_scan_ctx *ctx, const WsPlan &ws, int64_t B, int64_t Tn, int64_t D,
                   const fss_view *alpha, const fss_view *beta, const fss_view *h,
                   const fss_forward_state *st, std::string *err_text) {
    Params p{};
    const bool cont = ctx->flags & FSS_FLAG_CONTINUATION;
    float *prod = nullptr;
    if (st) {
        p.state_in = cont ? st->h_in : nullptr;
        p.state_out = st->h_last;
        p.block_prod = st->block_prod;
        p.block_state = st->block_state;
        prod = st->prod;
    }
    if (prod && !p.block_prod) {      // the total product is folded from the per-block products: keep them in scratch
        if (float_scratch_bytes(B, Tn, D) > ws.float_bytes) return FSS_E_WORKSPACE;
        p.block_prod = reinterpret_cast<float *>(ws.floats);
    }
    const int rc = launch<T, false>(ctx, ws, B, Tn, D, alpha, beta, nullptr, h, nullptr, p, err_text);
    if (rc != FSS_OK || !prod) return rc;
    const int dtype = sizeof(T) == 2 ? FSS_DTYPE_BF16 : FSS_DTYPE_F32;
    const int64_t S = ceil_div(Tn, block_rows(dtype, B, Tn, D));
    return launch_column_product(p.block_prod, prod, B, S, D, (cudaStream_t)ctx->stream, err_text);
}

// Forward scan whose alpha and beta are computed in the kernel from the recurrence gate r, the input
// gate i, the input x and the per-channel parameter lambda (see Gate).
template <typename T>
inline int forward_gated(const fss_scan_ctx *ctx, const WsPlan &ws, int64_t B, int64_t Tn, int64_t D,
                         const fss_view *r, const fss_view *i, const fss_view *x, const float *lambda,
                         const fss_view *h, const fss_forward_state *st, std::string *err_text) {
    Params p{};
    const bool cont = ctx->flags & FSS_FLAG_CONTINUATION;
    if (st) {
        p.state_in = cont ? st->h_in : nullptr;
        p.state_out = st->h_last;
    }
    // the per-channel exponent scales, once per launch, into the float scratch of the workspace
    if ((size_t)D * sizeof(float) > ws.float_bytes) return FSS_E_WORKSPACE;
    float *scales = reinterpret_cast<float *>(ws.floats);
    gates::prescale<T><<<(unsigned)ceil_div(D, 256), 256, 0, (cudaStream_t)ctx->stream>>>(lambda, scales, D);
    {
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) { *err_text = std::string("gate scale launch: ") + cudaGetErrorString(e); return FSS_E_LAUNCH; }
    }
    p.lambda = scales;
    const int dtype = sizeof(T) == 2 ? FSS_DTYPE_BF16 : FSS_DTYPE_F32;
    switch (choose_split(dtype, B, Tn, D)) {
    case 4: return launch_split<T, false, 4, false, true>(ctx, ws, B, Tn, D, r, x, i, h, nullptr, p, 0, err_text);
    case 2: return launch_split<T, false, 2, false, true>(ctx, ws, B, Tn, D, r, x, i, h, nullptr, p, 0, err_text);
    default: return launch_split<T, false, 1, false, true>(ctx, ws, B, Tn, D, r, x, i, h, nullptr, p, 0, err_text);
    }
}

template <typename T>
inline int backward(const fss_scan_ctx *ctx, const WsPlan &ws, int64_t B, int64_t Tn, int64_t D,
                    const fss_view *alpha, const fss_view *h, const fss_view *grad, const fss_view *dalpha,
                    const fss_view *dbeta, const fss_backward_state *st, std::string *err_text) {
    Params p{};
    const bool cont = ctx->flags & FSS_FLAG_CONTINUATION;
    if (st) {
        p.state_in = st->u_in;
        p.state_out = st->u_out;
        p.block_prod = st->block_prod;
        p.block_state = st->block_state;
        p.h_prev = cont ? st->h_prev : nullptr;
    }
    return launch<T, true>(ctx, ws, B, Tn, D, alpha, grad, h, dalpha, dbeta, p, err_text);
}

// fp32 state vectors are moved as 8- or 16-byte words by the single-pass kernels
inline bool state_aligned(std::initializer_list<const void *> ptrs) {
    for (const void *q : ptrs)
        if (q && !aligned16(q)) return false;
    return true;
}

}  // namespace lookback
}  // namespace fss
