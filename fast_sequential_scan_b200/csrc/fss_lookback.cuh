// FSS_ALGO_LOOKBACK: the single-pass path.  One persistent launch per direction; every tensor
// byte crosses HBM once (forward 3 tensors, backward 5).
//
// Work unit: a tile of kTc = 64 rows x 256 bytes of channels (128 bf16 / 64 fp32 channels) of one
// batch row.  Tiles are numbered row-block-major (all columns of the first row block, then the
// next ...; the backward numbers row blocks from the end), CTA c of G takes tiles c, c+G, c+2G...
// so a tile only ever depends on tiles with smaller numbers, which are always resident or done.
//
// A CTA runs three roles, coupled only by shared-memory mbarriers:
//   producer warp (1 thread)  TMA-loads the tiles of upcoming work units into a ring of stages
//                             (cp.async.bulk.tensor, complete_tx on full[stage]); when a unit is
//                             finished it TMA-stores the results that were written in place and
//                             refills the stage.
//   8 consumer warps          each owns 8 rows of the tile, each lane 8 bytes of channels.
//                             pass 1: scan own rows from a zero state -> (P, C) to shared memory;
//                             pass 2: re-scan from the true entering state, results in place.
//                             Software-pipelined: pass 1 of unit i+1 runs before pass 2 of unit i,
//                             so the carry resolution below is off the critical path.
//   look-back warp            folds the 8 warp summaries into the tile summary, resolves the
//                             state entering the tile by decoupled look-back over the global
//                             tile descriptors of its predecessors (aggregate / inclusive flags,
//                             release/acquire at gpu scope), publishes its own, and hands every
//                             consumer warp its entering state.
// Every wait is bounded; a wait that runs out records a status, raises the abort flag that all
// other waits poll, and the CTA drains its copies and leaves.
#pragma once

#include <cuda.h>

#include <initializer_list>
#include <mutex>
#include <string>

#include "fss_common.cuh"

namespace fss {
namespace lookback {

constexpr int kW = 8;                         // consumer warps
constexpr int kR = 8;                         // rows per consumer warp and tile
constexpr int kTc = kW * kR;                  // rows per tile
constexpr int kRowBytes = 256;                // bytes of one tile row
constexpr int kLaneBytes = 8;
constexpr int kTileBytes = kTc * kRowBytes;   // 16 KiB per tensor and stage
constexpr int kProducerWarp = kW;
constexpr int kLookbackWarp = kW + 1;
constexpr int kThreads = (kW + 2) * 32;
constexpr int kStagesFwd = 6;                 // 6 x 32 KiB
constexpr int kStagesBwd = 4;                 // 4 x 48 KiB
constexpr uint32_t kMaxSpins = 1u << 21;      // per wait; ~a second before giving up

constexpr uint32_t kStateAggregate = 1, kStateInclusive = 2;

template <typename T> struct Cfg {
    static constexpr int V = kLaneBytes / (int)sizeof(T);   // channels per lane
    static constexpr int Dc = 32 * V;                       // channels per tile
};

struct Header {      // first bytes of the workspace
    uint32_t epoch;  // number of look-back launches that have completed on this workspace
    uint32_t done;   // CTAs of the running launch that have finished
    uint32_t abort;  // raised by the first wait that gives up
    uint32_t pad;
};

struct Params {
    int64_t B, T, D;
    int64_t ncg;      // channel groups per row
    int64_t ncols;    // B * ncg
    int64_t S;        // row blocks per column
    int64_t ntiles;
    uint32_t *flags;  // [ntiles]
    float *desc;      // [ntiles][4][Dc]: aggregate P, aggregate C, inclusive C, inclusive P
    Header *hdr;
    int32_t *status;
    const float *state_in;   // forward h_in / backward u_in, [B, D] or null
    float *state_out;        // forward h_last / backward u_out
    float *prod_out;         // forward prod
    float *block_prod;       // [B, S, D]
    const float *h_prev;     // backward only
    int continuation;
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

__device__ __forceinline__ uint32_t ld_acquire(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release(uint32_t *p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_volatile(const uint32_t *p) {
    return *reinterpret_cast<const volatile uint32_t *>(p);
}

// ------------------------------------------------------------------ 8-byte lane fragments
template <typename T> struct Lane;
template <> struct Lane<bf16> {
    static constexpr int V = 4;
    static __device__ __forceinline__ void load(uint32_t addr, float (&x)[4]) {
        uint32_t w0, w1;
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(w0), "=r"(w1) : "r"(addr));
        x[0] = __uint_as_float(w0 << 16); x[1] = __uint_as_float(w0 & 0xffff0000u);
        x[2] = __uint_as_float(w1 << 16); x[3] = __uint_as_float(w1 & 0xffff0000u);
    }
    static __device__ __forceinline__ void store(uint32_t addr, const float (&x)[4]) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]);
        __nv_bfloat162 hi = __floats2bfloat162_rn(x[2], x[3]);
        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(*reinterpret_cast<uint32_t *>(&lo)),
                     "r"(*reinterpret_cast<uint32_t *>(&hi)) : "memory");
    }
};
template <> struct Lane<float> {
    static constexpr int V = 2;
    static __device__ __forceinline__ void load(uint32_t addr, float (&x)[2]) {
        asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(x[0]), "=f"(x[1]) : "r"(addr));
    }
    static __device__ __forceinline__ void store(uint32_t addr, const float (&x)[2]) {
        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(x[0]), "f"(x[1]) : "memory");
    }
};

// V consecutive floats of a global fp32 vector (descriptor / state arrays), L2-coherent
template <int V> __device__ __forceinline__ void ldg_vec(const float *p, float (&x)[V]) {
    if constexpr (V == 4) {
        const float4 r = __ldcg(reinterpret_cast<const float4 *>(p));
        x[0] = r.x; x[1] = r.y; x[2] = r.z; x[3] = r.w;
    } else {
        const float2 r = __ldcg(reinterpret_cast<const float2 *>(p));
        x[0] = r.x; x[1] = r.y;
    }
}
template <int V> __device__ __forceinline__ void stg_vec(float *p, const float (&x)[V]) {
    if constexpr (V == 4) {
        __stcg(reinterpret_cast<float4 *>(p), make_float4(x[0], x[1], x[2], x[3]));
    } else {
        __stcg(reinterpret_cast<float2 *>(p), make_float2(x[0], x[1]));
    }
}

// ------------------------------------------------------------------ bounded waits
struct Ctl {
    Header *hdr;
    int32_t *status;
    volatile int *cta_abort;   // shared-memory copy of the abort flag

    __device__ __forceinline__ bool aborted() const {
        return *cta_abort != 0 || ld_volatile(&hdr->abort) != 0;
    }
    __device__ __forceinline__ void give_up(int32_t code) const {
        *cta_abort = 1;
        atomicExch(&hdr->abort, 1u);
        report_status(status, code);
    }
    // false = the wait was abandoned (timeout here, or abort raised elsewhere)
    __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, int32_t code) const {
        for (uint32_t it = 0; it < kMaxSpins; ++it) {
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
    static constexpr int kAggFloats = 2 * kW * 2 * 128;    // [2 generations][warp][P|C][<=128 channels]
    static constexpr int kBarriers = 2 * kStages + 4;
    static constexpr int kBytes = 128 /* alignment slack */ + kStages * kStageBytes + kAggFloats * 4 + kBarriers * 8 + 16;
};

struct Tile { int64_t k, s, col, b, cg, row0; };

template <bool kBackward>
__device__ __forceinline__ Tile decode_tile(const Params &p, int64_t k) {
    Tile t;
    t.k = k;
    t.s = k / p.ncols;
    t.col = k - t.s * p.ncols;
    t.b = t.col / p.ncg;
    t.cg = t.col - t.b * p.ncg;
    t.row0 = (kBackward ? (p.S - 1 - t.s) : t.s) * (int64_t)kTc;
    return t;
}

// ------------------------------------------------------------------ the kernel
// Forward: tensors (alpha, beta) are loaded, h is stored from beta's stage slot.
// Backward: (alpha, grad, h shifted one row down) are loaded; dbeta is stored from grad's slot,
// dalpha from h's slot.
template <typename T, bool kBackward>
__global__ void __launch_bounds__(kThreads, 1)
scan_kernel(const __grid_constant__ CUtensorMap map_alpha, const __grid_constant__ CUtensorMap map_x,
            const __grid_constant__ CUtensorMap map_h, const __grid_constant__ CUtensorMap map_out0,
            const __grid_constant__ CUtensorMap map_out1, const Params p) {
    constexpr int kTensors = kBackward ? 3 : 2;
    constexpr int kStages = kBackward ? kStagesBwd : kStagesFwd;
    using SM = Smem<kTensors, kStages>;
    constexpr int V = Cfg<T>::V;
    constexpr int Dc = Cfg<T>::Dc;

    // TMA tiles want 128-byte aligned shared addresses: align the dynamic window by hand
    extern __shared__ unsigned char smem_dyn[];
    unsigned char *smem_raw = smem_dyn + ((128u - (smem_u32(smem_dyn) & 127u)) & 127u);
    const uint32_t smem_base = smem_u32(smem_raw);
    float *agg = reinterpret_cast<float *>(smem_raw + kStages * SM::kStageBytes);
    const uint32_t agg_u32 = smem_base + kStages * SM::kStageBytes;
    const uint32_t bars = agg_u32 + SM::kAggFloats * 4;
    volatile int *cta_abort = reinterpret_cast<volatile int *>(smem_raw + kStages * SM::kStageBytes +
                                                               SM::kAggFloats * 4 + SM::kBarriers * 8);
    volatile uint32_t *epoch_s = reinterpret_cast<volatile uint32_t *>(const_cast<int *>(cta_abort) + 1);
    auto bar_full = [&](int s) { return bars + 8u * s; };
    auto bar_done = [&](int s) { return bars + 8u * (kStages + s); };
    auto bar_agg = [&](int g) { return bars + 8u * (2 * kStages + g); };
    auto bar_carry = [&](int g) { return bars + 8u * (2 * kStages + 2 + g); };
    // agg[g][w][0|1][channel]
    auto agg_off = [&](int g, int w, int which) { return ((g * kW + w) * 2 + which) * 128; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t G = gridDim.x;
    const int64_t first = blockIdx.x;
    const int64_t n_my = first < p.ntiles ? (p.ntiles - first + G - 1) / G : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_done(s), kW); }
        for (int g = 0; g < 2; ++g) { mbar_init(bar_agg(g), kW); mbar_init(bar_carry(g), 1); }
        *cta_abort = 0;
        *epoch_s = ld_volatile(&p.hdr->epoch) + 1u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    __syncthreads();
    const uint32_t epoch = *epoch_s;
    const Ctl ctl{p.hdr, p.status, cta_abort};

    if (warp == kProducerWarp) {
        // ============================================================ producer
        if (lane == 0) {
            auto issue = [&](int64_t i) {
                const Tile t = decode_tile<kBackward>(p, first + i * G);
                const int st = (int)(i % kStages);
                const uint32_t base = smem_base + st * SM::kStageBytes;
                const int32_t c0 = (int32_t)(t.cg * Dc), c1 = (int32_t)t.row0, c2 = (int32_t)t.b;
                mbar_arrive_expect_tx(bar_full(st), SM::kStageBytes);
                tma_load_3d(base, &map_alpha, bar_full(st), c0, c1, c2);
                tma_load_3d(base + kTileBytes, &map_x, bar_full(st), c0, c1, c2);
                if (kBackward) tma_load_3d(base + 2 * kTileBytes, &map_h, bar_full(st), c0, c1 - 1, c2);
            };
            int64_t issued = 0;
            for (; issued < n_my && issued < kStages; ++issued) issue(issued);
            int64_t i = 0;
            for (; i < n_my; ++i) {
                const int st = (int)(i % kStages);
                if (!ctl.wait(bar_done(st), (uint32_t)((i / kStages) & 1), FSS_STATUS_TMA_TIMEOUT)) break;
                const Tile t = decode_tile<kBackward>(p, first + i * G);
                const uint32_t base = smem_base + st * SM::kStageBytes;
                const int32_t c0 = (int32_t)(t.cg * Dc), c1 = (int32_t)t.row0, c2 = (int32_t)t.b;
                if (!kBackward) {
                    tma_store_3d(&map_out0, base + kTileBytes, c0, c1, c2);          // h
                } else {
                    tma_store_3d(&map_out0, base + 2 * kTileBytes, c0, c1, c2);      // dalpha
                    tma_store_3d(&map_out1, base + kTileBytes, c0, c1, c2);          // dbeta
                }
                tma_commit();
                if (issued < n_my) {
                    tma_wait_read_all();      // the stage may be overwritten once the store has read it
                    issue(issued);
                    ++issued;
                }
            }
            // leave nothing in flight: loads that were issued but never consumed, and all stores
            if (i < n_my) {
                for (int64_t j = i; j < issued; ++j) {
                    const uint32_t bar = bar_full((int)(j % kStages));
                    const uint32_t par = (uint32_t)((j / kStages) & 1);
                    for (uint32_t it = 0; it < kMaxSpins && !mbar_try_wait(bar, par); ++it) {}
                }
            }
            tma_wait_all();
        }
    } else if (warp == kLookbackWarp) {
        // ============================================================ look-back
        const int ch = lane * V;    // first channel of this lane inside the tile
        for (int64_t i = 0; i < n_my; ++i) {
            const Tile t = decode_tile<kBackward>(p, first + i * G);
            const int g = (int)(i & 1);
            const int64_t dch = t.cg * Dc + ch;          // channel in the tensor
            const bool ch_ok = dch < p.D;
            float *my_desc = p.desc + t.k * (4 * Dc) + ch;

            // early, non-blocking peek at the predecessor (overlaps the consumers' pass 1)
            // (every lane issues its own acquire load; the decision is taken by vote so that the
            // warp stays converged even if lanes were to observe the flag at different moments)
            uint32_t peek = 0;
            if (t.s > 0) peek = ld_acquire(p.flags + (t.k - p.ncols));
            float pre_c[V], pre_p[V];
            const bool peek_hit = __all_sync(0xffffffffu, (t.s > 0) && (peek == ((epoch << 2) | kStateInclusive)));
            if (peek_hit) {
                const float *pd = p.desc + (t.k - p.ncols) * (4 * Dc) + ch;
                ldg_vec<V>(pd + 2 * Dc, pre_c);
                ldg_vec<V>(pd + 3 * Dc, pre_p);
            }

            if (!ctl.wait(bar_agg(g), (uint32_t)((i >> 1) & 1), FSS_STATUS_LOOKBACK_TIMEOUT)) break;

            // fold the warp summaries in scan order; keep the exclusive prefixes for hand-out
            float Pex[kW][V], Cex[kW][V], Pt[V], Ct[V];
#pragma unroll
            for (int v = 0; v < V; ++v) { Pt[v] = 1.0f; Ct[v] = 0.0f; }
#pragma unroll
            for (int j = 0; j < kW; ++j) {
                const int w = kBackward ? kW - 1 - j : j;
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    Pex[w][v] = Pt[v]; Cex[w][v] = Ct[v];
                    const float pw = agg[agg_off(g, w, 0) + ch + v];
                    const float cw = agg[agg_off(g, w, 1) + ch + v];
                    Ct[v] = fmaf(pw, Ct[v], cw);
                    Pt[v] *= pw;
                }
            }

            // ---- the state entering this tile, and the product of alpha before it
            float cin[V], pin[V];
            bool ok = true;
            if (t.s == 0) {
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    cin[v] = (p.state_in && ch_ok) ? p.state_in[t.b * p.D + dch + v] : 0.0f;
                    pin[v] = 1.0f;
                }
            } else if (peek_hit) {
#pragma unroll
                for (int v = 0; v < V; ++v) { cin[v] = pre_c[v]; pin[v] = pre_p[v]; }
            } else {
                // publish the aggregate so successors need not wait for this tile's own look-back
                stg_vec<V>(my_desc, Pt);
                stg_vec<V>(my_desc + Dc, Ct);
                __syncwarp();
                if (lane == 0) st_release(p.flags + t.k, (epoch << 2) | kStateAggregate);
                float Pa[V], Ca[V];
#pragma unroll
                for (int v = 0; v < V; ++v) { Pa[v] = 1.0f; Ca[v] = 0.0f; }
                int64_t q = t.k - p.ncols;
                while (true) {
                    uint32_t f = 0;
                    uint32_t it = 0;
                    for (; it < kMaxSpins; ++it) {
                        f = ld_acquire(p.flags + q);
                        if (__all_sync(0xffffffffu, (f >> 2) == epoch && (f & 3u) != 0)) break;
                        if ((it & 15u) == 15u && __any_sync(0xffffffffu, ctl.aborted())) { ok = false; break; }
                        __nanosleep(40);
                    }
                    if (ok && it == kMaxSpins) { if (lane == 0) ctl.give_up(FSS_STATUS_LOOKBACK_TIMEOUT); ok = false; }
                    if (!ok) break;
                    const float *qd = p.desc + q * (4 * Dc) + ch;
                    float x0[V], x1[V];
                    // a tile that has ever shown "aggregate" keeps valid aggregate data, so a mixed
                    // observation is handled as aggregate
                    if (__all_sync(0xffffffffu, (f & 3u) == kStateInclusive)) {
                        ldg_vec<V>(qd + 2 * Dc, x0);
                        ldg_vec<V>(qd + 3 * Dc, x1);
#pragma unroll
                        for (int v = 0; v < V; ++v) { cin[v] = fmaf(Pa[v], x0[v], Ca[v]); pin[v] = Pa[v] * x1[v]; }
                        break;
                    }
                    ldg_vec<V>(qd, x0);          // aggregate P
                    ldg_vec<V>(qd + Dc, x1);     // aggregate C
#pragma unroll
                    for (int v = 0; v < V; ++v) { Ca[v] = fmaf(Pa[v], x1[v], Ca[v]); Pa[v] *= x0[v]; }
                    q -= p.ncols;
                    if (q < 0) {
#pragma unroll
                        for (int v = 0; v < V; ++v) {
                            const float s0 = (p.state_in && ch_ok) ? p.state_in[t.b * p.D + dch + v] : 0.0f;
                            cin[v] = fmaf(Pa[v], s0, Ca[v]);
                            pin[v] = Pa[v];
                        }
                        break;
                    }
                }
                if (!ok) break;
            }

            // ---- publish the inclusive state, then hand the consumers their entering states
            float cinc[V], pinc[V];
#pragma unroll
            for (int v = 0; v < V; ++v) { cinc[v] = fmaf(Pt[v], cin[v], Ct[v]); pinc[v] = Pt[v] * pin[v]; }
            if (t.s + 1 < p.S) {
                stg_vec<V>(my_desc + 2 * Dc, cinc);
                stg_vec<V>(my_desc + 3 * Dc, pinc);
                __syncwarp();
                if (lane == 0) st_release(p.flags + t.k, (epoch << 2) | kStateInclusive);
            }
#pragma unroll
            for (int w = 0; w < kW; ++w) {
#pragma unroll
                for (int v = 0; v < V; ++v) agg[agg_off(g, w, 0) + ch + v] = fmaf(Pex[w][v], cin[v], Cex[w][v]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_carry(g));

            if (ch_ok) {
                if (p.block_prod) {
                    const int64_t blk = kBackward ? (p.S - 1 - t.s) : t.s;
                    float *bp = p.block_prod + (t.b * p.S + blk) * p.D + dch;
#pragma unroll
                    for (int v = 0; v < V; ++v) bp[v] = pinc[v];
                }
                if (t.s + 1 == p.S) {
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        if (p.state_out) p.state_out[t.b * p.D + dch + v] = cinc[v];
                        if (p.prod_out) p.prod_out[t.b * p.D + dch + v] = pinc[v];
                    }
                }
            }
        }
    } else {
        // ============================================================ consumers
        const uint32_t lane_off = (uint32_t)(warp * kR) * kRowBytes + (uint32_t)lane * kLaneBytes;
        const int ch = lane * V;

        auto pass1 = [&](int64_t i) -> bool {
            const Tile t = decode_tile<kBackward>(p, first + i * G);
            const int st = (int)(i % kStages), g = (int)(i & 1);
            if (!ctl.wait(bar_full(st), (uint32_t)((i / kStages) & 1), FSS_STATUS_TMA_TIMEOUT)) return false;
            const uint32_t a_t = smem_base + st * SM::kStageBytes + lane_off;
            const uint32_t x_t = a_t + kTileBytes;
            // row 0 of the whole sequence: alpha_0 is not part of the recurrence
            if (t.row0 == 0 && warp == 0 && !p.continuation) {
                float z[V];
#pragma unroll
                for (int v = 0; v < V; ++v) z[v] = 0.0f;
                Lane<T>::store(a_t, z);
            }
            float P[V], C[V];
#pragma unroll
            for (int v = 0; v < V; ++v) { P[v] = 1.0f; C[v] = 0.0f; }
#pragma unroll
            for (int j = 0; j < kR; ++j) {
                const int r = kBackward ? kR - 1 - j : j;
                float a[V], x[V];
                Lane<T>::load(a_t + r * kRowBytes, a);
                Lane<T>::load(x_t + r * kRowBytes, x);
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    if (!kBackward) C[v] = fmaf(a[v], C[v], x[v]);
                    else C[v] = a[v] * (x[v] + C[v]);
                    P[v] *= a[v];
                }
            }
#pragma unroll
            for (int v = 0; v < V; ++v) {
                agg[agg_off(g, warp, 0) + ch + v] = P[v];
                agg[agg_off(g, warp, 1) + ch + v] = C[v];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_agg(g));
            return true;
        };

        auto pass2 = [&](int64_t i) -> bool {
            const Tile t = decode_tile<kBackward>(p, first + i * G);
            const int st = (int)(i % kStages), g = (int)(i & 1);
            if (!ctl.wait(bar_carry(g), (uint32_t)((i >> 1) & 1), FSS_STATUS_LOOKBACK_TIMEOUT)) return false;
            const uint32_t a_t = smem_base + st * SM::kStageBytes + lane_off;
            const uint32_t x_t = a_t + kTileBytes;
            float stv[V];
#pragma unroll
            for (int v = 0; v < V; ++v) stv[v] = agg[agg_off(g, warp, 0) + ch + v];
            if (!kBackward) {
#pragma unroll
                for (int r = 0; r < kR; ++r) {
                    float a[V], x[V];
                    Lane<T>::load(a_t + r * kRowBytes, a);
                    Lane<T>::load(x_t + r * kRowBytes, x);
#pragma unroll
                    for (int v = 0; v < V; ++v) stv[v] = fmaf(a[v], stv[v], x[v]);
                    Lane<T>::store(x_t + r * kRowBytes, stv);
                }
            } else {
                const uint32_t h_t = x_t + kTileBytes;
                const bool head = (t.row0 == 0) && (warp == 0);
                if (head && p.continuation && p.h_prev) {    // h_{-1} of a continued sequence
                    float hp[V];
                    const int64_t dch = t.cg * Dc + ch;
#pragma unroll
                    for (int v = 0; v < V; ++v) hp[v] = (dch < p.D) ? p.h_prev[t.b * p.D + dch + v] : 0.0f;
                    Lane<T>::store(h_t, hp);
                }
#pragma unroll
                for (int j = 0; j < kR; ++j) {
                    const int r = kR - 1 - j;
                    float a[V], x[V], hp[V], da[V], dh[V];
                    Lane<T>::load(a_t + r * kRowBytes, a);
                    Lane<T>::load(x_t + r * kRowBytes, x);
                    Lane<T>::load(h_t + r * kRowBytes, hp);
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        dh[v] = x[v] + stv[v];
                        da[v] = dh[v] * hp[v];
                        stv[v] = a[v] * dh[v];
                    }
                    if (r == 0 && head && !p.continuation) {
#pragma unroll
                        for (int v = 0; v < V; ++v) da[v] = 0.0f;
                    }
                    Lane<T>::store(x_t + r * kRowBytes, dh);
                    Lane<T>::store(h_t + r * kRowBytes, da);
                }
            }
            fence_proxy_async();      // make the in-place results visible to the TMA store
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_done(st));
            return true;
        };

        bool alive = n_my > 0 && pass1(0);
        for (int64_t i = 0; alive && i < n_my; ++i) {
            if (i + 1 < n_my) alive = pass1(i + 1);
            if (alive) alive = pass2(i);
        }
    }

    // ---- leave: the last CTA advances the epoch, which invalidates every flag of this launch
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t prev = atomicAdd(&p.hdr->done, 1u);
        if (prev + 1 == gridDim.x) {
            p.hdr->done = 0;
            p.hdr->abort = 0;
            __threadfence();
            p.hdr->epoch = epoch;
        }
    }
}

// ------------------------------------------------------------------ host side
inline int64_t block_rows(int, int64_t, int64_t, int64_t) { return kTc; }

template <typename T> inline int64_t channel_groups(int64_t D) { return ceil_div(D, Cfg<T>::Dc); }

// float scratch (tile descriptors); the flag words live in the workspace's flag area
inline size_t workspace_bytes(int64_t B, int64_t T, int64_t D, int dtype) {
    const int Dc = dtype == FSS_DTYPE_BF16 ? Cfg<bf16>::Dc : Cfg<float>::Dc;
    const int64_t ntiles = B * ceil_div(D, Dc) * ceil_div(T, kTc);
    return (size_t)ntiles * 4 * Dc * sizeof(float);
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
inline bool make_map(CUtensorMap *map, const fss_view *v, int64_t B, int64_t Tn, int64_t D) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)Tn, (cuuint64_t)B};
    const int64_t sb = B > 1 ? v->stride_b : v->stride_t * Tn;
    const cuuint64_t strides[2] = {(cuuint64_t)(v->stride_t * (int64_t)sizeof(T)),
                                   (cuuint64_t)(sb * (int64_t)sizeof(T))};
    const cuuint32_t box[3] = {(cuuint32_t)Cfg<T>::Dc, (cuuint32_t)kTc, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapDataType dt = sizeof(T) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    return fn(map, dt, 3, v->ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// CTAs that fit the device at once (one per SM with these shared-memory sizes), per device.
template <typename T, bool kBackward> inline int resident_ctas(int device, int smem_bytes, cudaError_t *err) {
    static std::mutex mu;
    static int cached[64];
    static bool have[64];
    std::lock_guard<std::mutex> lock(mu);
    if (device < 0 || device >= 64) { *err = cudaErrorInvalidDevice; return 0; }
    if (!have[device]) {
        auto kern = scan_kernel<T, kBackward>;
        *err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (*err != cudaSuccess) return 0;
        int per_sm = 0, sms = 0;
        *err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem_bytes);
        if (*err != cudaSuccess) return 0;
        *err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (*err != cudaSuccess) return 0;
        cached[device] = per_sm * sms;
        have[device] = true;
    }
    *err = cudaSuccess;
    return cached[device];
}

template <typename T, bool kBackward>
inline int launch(const fss_scan_ctx *ctx, const WsPlan &ws, int64_t B, int64_t Tn, int64_t D,
                  const fss_view *alpha, const fss_view *x, const fss_view *h, const fss_view *out0,
                  const fss_view *out1, Params p, std::string *err_text) {
    constexpr int kTensors = kBackward ? 3 : 2;
    constexpr int kStages = kBackward ? kStagesBwd : kStagesFwd;
    constexpr int smem_bytes = Smem<kTensors, kStages>::kBytes;
    constexpr int Dc = Cfg<T>::Dc;

    CUtensorMap m_alpha, m_x, m_h, m_o0, m_o1;
    if (!make_map<T>(&m_alpha, alpha, B, Tn, D) || !make_map<T>(&m_x, x, B, Tn, D) ||
        !make_map<T>(&m_o0, out0, B, Tn, D))
        return FSS_E_TENSORMAP;
    if (kBackward) {
        if (!make_map<T>(&m_h, h, B, Tn, D) || !make_map<T>(&m_o1, out1, B, Tn, D)) return FSS_E_TENSORMAP;
    } else {
        m_h = m_alpha; m_o1 = m_o0;
    }

    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) { *err_text = cudaGetErrorString(e); return FSS_E_DEVICE; }
    const int resident = resident_ctas<T, kBackward>(device, smem_bytes, &e);
    if (e != cudaSuccess || resident < 1) { *err_text = cudaGetErrorString(e); return FSS_E_LAUNCH; }

    p.B = B; p.T = Tn; p.D = D;
    p.ncg = ceil_div(D, Dc);
    p.ncols = B * p.ncg;
    p.S = ceil_div(Tn, kTc);
    p.ntiles = p.ncols * p.S;
    if ((size_t)p.ntiles * 4 > ws.flag_bytes || (size_t)p.ntiles * 4 * Dc * sizeof(float) > ws.float_bytes)
        return FSS_E_WORKSPACE;
    p.hdr = reinterpret_cast<Header *>(ws.hdr);
    p.flags = reinterpret_cast<uint32_t *>(ws.flags);
    p.desc = reinterpret_cast<float *>(ws.floats);
    p.status = ctx->status;
    p.continuation = (ctx->flags & FSS_FLAG_CONTINUATION) ? 1 : 0;

    const unsigned grid = (unsigned)(p.ntiles < resident ? p.ntiles : resident);
    scan_kernel<T, kBackward><<<grid, kThreads, smem_bytes, (cudaStream_t)ctx->stream>>>(
        m_alpha, m_x, m_h, m_o0, m_o1, p);
    e = cudaGetLastError();
    if (e != cudaSuccess) { *err_text = std::string("look-back launch: ") + cudaGetErrorString(e); return FSS_E_LAUNCH; }
    return FSS_OK;
}

template <typename T>
inline int forward(const fss_scan_ctx *ctx, const WsPlan &ws, int64_t B, int64_t Tn, int64_t D,
                   const fss_view *alpha, const fss_view *beta, const fss_view *h,
                   const fss_forward_state *st, std::string *err_text) {
    Params p{};
    const bool cont = ctx->flags & FSS_FLAG_CONTINUATION;
    if (st) {
        p.state_in = cont ? st->h_in : nullptr;
        p.state_out = st->h_last;
        p.prod_out = st->prod;
        p.block_prod = st->block_prod;
    }
    return launch<T, false>(ctx, ws, B, Tn, D, alpha, beta, nullptr, h, nullptr, p, err_text);
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
        p.h_prev = cont ? st->h_prev : nullptr;
    }
    return launch<T, true>(ctx, ws, B, Tn, D, alpha, grad, h, dalpha, dbeta, p, err_text);
}

}  // namespace lookback
}  // namespace fss
