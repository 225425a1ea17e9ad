// Shared device/host helpers of the sm_100a sequential-scan library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fss_b200.h"

namespace fss {

using bf16 = __nv_bfloat16;

// ------------------------------------------------------------------ tensor view (device side)
template <typename T> struct View {
    T *ptr;
    int64_t sb, st;  // batch / row stride in elements
    __host__ __device__ __forceinline__ T *row(int64_t b, int64_t t) const { return ptr + b * sb + t * st; }
};

template <typename T> inline View<T> make_view(const fss_view *v) {
    return View<T>{reinterpret_cast<T *>(v->ptr), v->stride_b, v->stride_t};
}

// ------------------------------------------------------------------ 16-byte row fragments
// A fragment is V consecutive channels of one row held as fp32 in registers.  V = 8 (bf16) or
// 4 (fp32) moves 16 bytes per access; V = 1 is the any-alignment path.
template <typename T, int V> struct Frag;

template <> struct Frag<bf16, 8> {
    using Raw = uint4;      // the fragment as it travels: unpacked only when used, to keep loads in flight cheap
    static __device__ __forceinline__ Raw load_raw(const bf16 *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }
    static __device__ __forceinline__ void unpack(const Raw &r, float (&x)[8]) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[2 * i] = __uint_as_float(w[i] << 16);
            x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void load(const bf16 *p, float (&x)[8]) { unpack(load_raw(p), x); }
    static __device__ __forceinline__ void store(bf16 *p, const float (&x)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 v = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&v);
        }
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

template <> struct Frag<bf16, 1> {
    using Raw = bf16;
    static __device__ __forceinline__ Raw load_raw(const bf16 *p) { return *p; }
    static __device__ __forceinline__ void unpack(const Raw &r, float (&x)[1]) { x[0] = __bfloat162float(r); }
    static __device__ __forceinline__ void load(const bf16 *p, float (&x)[1]) {
        x[0] = __bfloat162float(*p);
    }
    static __device__ __forceinline__ void store(bf16 *p, const float (&x)[1]) {
        *p = __float2bfloat16_rn(x[0]);
    }
};

template <> struct Frag<float, 4> {
    using Raw = float4;
    static __device__ __forceinline__ Raw load_raw(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
    static __device__ __forceinline__ void unpack(const Raw &r, float (&x)[4]) { x[0] = r.x; x[1] = r.y; x[2] = r.z; x[3] = r.w; }
    static __device__ __forceinline__ void load(const float *p, float (&x)[4]) { unpack(load_raw(p), x); }
    static __device__ __forceinline__ void store(float *p, const float (&x)[4]) {
        *reinterpret_cast<float4 *>(p) = make_float4(x[0], x[1], x[2], x[3]);
    }
};

template <> struct Frag<float, 1> {
    using Raw = float;
    static __device__ __forceinline__ Raw load_raw(const float *p) { return __ldg(p); }
    static __device__ __forceinline__ void unpack(const Raw &r, float (&x)[1]) { x[0] = r; }
    static __device__ __forceinline__ void load(const float *p, float (&x)[1]) { x[0] = __ldg(p); }
    static __device__ __forceinline__ void store(float *p, const float (&x)[1]) { *p = x[0]; }
};

// Read-modify-write flavour for the fix-up kernels (the value was produced by an earlier kernel
// on the same stream, so the plain, coherent load path is used).
template <typename T, int V> struct FragRW;
template <> struct FragRW<bf16, 8> {
    static __device__ __forceinline__ void load(const bf16 *p, float (&x)[8]) {
        const uint4 r = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[2 * i] = __uint_as_float(w[i] << 16);
            x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};
template <> struct FragRW<bf16, 1> {
    static __device__ __forceinline__ void load(const bf16 *p, float (&x)[1]) { x[0] = __bfloat162float(*p); }
};
template <> struct FragRW<float, 4> {
    static __device__ __forceinline__ void load(const float *p, float (&x)[4]) {
        const float4 r = *reinterpret_cast<const float4 *>(p);
        x[0] = r.x; x[1] = r.y; x[2] = r.z; x[3] = r.w;
    }
};
template <> struct FragRW<float, 1> {
    static __device__ __forceinline__ void load(const float *p, float (&x)[1]) { x[0] = *p; }
};

template <typename T> struct VecWidth;
template <> struct VecWidth<bf16> { static constexpr int value = 8; };
template <> struct VecWidth<float> { static constexpr int value = 4; };

// ------------------------------------------------------------------ status word
// Written only when a bounded wait gives up; works for device memory and for pinned host memory.
__device__ __forceinline__ void report_status(int32_t *status, int32_t code) {
    if (status != nullptr) {
        atomicCAS_system(reinterpret_cast<int *>(status), 0, code);
        __threadfence_system();
    }
}

// ------------------------------------------------------------------ host helpers
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Records the text fss_last_cuda_error() returns for the calling thread and hands back `code`
// (defined once, in fss_api.cu).
int cuda_fail(cudaError_t e, const char *what, int code);

// A view must span its extents without rows or batches overlapping, and its last element's
// offset must be representable (the kernels index with 64-bit element offsets).
inline int check_view_extents(const fss_view *v, int64_t B, int64_t T, int64_t D) {
    if (!v || !v->ptr) return FSS_E_NULL;
    if (v->stride_t < D) return FSS_E_SHAPE;
    if (T > 1 && v->stride_t > (INT64_MAX / 8) / T) return FSS_E_SHAPE;
    if (B > 1) {
        if (v->stride_b < (T - 1) * v->stride_t + D) return FSS_E_SHAPE;
        if (v->stride_b > (INT64_MAX / 8) / B) return FSS_E_SHAPE;
    }
    return FSS_OK;
}
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Workspace plan: [256-byte header | descriptor packets | float scratch].  The split depends only
// on the workspace's total size, so for one allocation the packet area always sits at the same
// place and only ever holds 16-byte packets whose fourth word is a tag: a stale float can never
// pass for a tag of the current launch.
constexpr size_t kWsHeaderBytes = 256;
struct WsPlan {
    char *hdr, *packets, *floats;
    size_t packet_bytes, float_bytes;
};
inline WsPlan plan_workspace(void *ws, size_t bytes) {
    WsPlan w{};
    if (bytes < kWsHeaderBytes + 1024) return w;
    w.hdr = static_cast<char *>(ws);
    w.packet_bytes = (bytes - kWsHeaderBytes) / 2 / 256 * 256;
    w.packets = w.hdr + kWsHeaderBytes;
    w.floats = w.packets + w.packet_bytes;
    w.float_bytes = bytes - kWsHeaderBytes - w.packet_bytes;
    return w;
}
// total size whose plan leaves at least `need` bytes in each of the two areas
inline size_t workspace_total(size_t need) { return kWsHeaderBytes + 2 * align_up(need + 256, 256) + 1024; }

}  // namespace fss
