// fss_scan_forward_noalloc: the chunked forward scan for callers that may not allocate.
//
// Every other entry point of this library takes its scratch from the caller, who normally gets
// it from cudaMalloc or a framework allocator.  Some callers cannot do that at the moment they
// need a scan: a plugin living inside a host application that has already handed all device
// memory to its own pool, a service loop that must not hit cudaMalloc's implicit device-wide
// synchronisation, code that runs after the memory budget of the process has been frozen.  For
// them this file carries its own scratch: one fixed array in device memory that is part of the
// library image.  Every GPU that loads the library holds these FSS_NOALLOC_SCRATCH_BYTES until the
// process exits, which is why the size is modest and the shapes it serves are bounded.
//
// The array is shared by all calls.  Nothing in it has to start at zero (each call writes every
// word it later reads: chunk summaries first, then their composition, then the re-scan), and it
// keeps whatever the last call left.  Two calls whose kernels overlap on the GPU (different
// streams, or different host threads without ordering) would trample each other's summaries:
// callers have to serialise them.
//
// Host code cannot use the array's name as a pointer -- on the host that name is only a handle
// for the runtime.  The device address is looked up with cudaGetSymbolAddress, once per device,
// with that device current, on the first call that targets the device; that first call should
// therefore be made before any stream capture begins.
#include <mutex>

#include "fss_chunked.cuh"
#include "fss_common.cuh"

namespace {

// the scratch itself: lives in the library image, one copy per device that loads it
static __device__ __align__(256) unsigned char g_noalloc_scratch[FSS_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void *g_scratch_addr[kMaxDevices];      // device address of g_noalloc_scratch, per device ordinal
bool g_scratch_known[kMaxDevices];

// Device address of the scratch on `device` (which must be current); looked up once per device.
int scratch_address(int device, void **out) {
    if (device < 0 || device >= kMaxDevices) return FSS_E_DEVICE;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_known[device]) {
        void *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess) return fss::cuda_fail(e, "cudaGetSymbolAddress(no-alloc scratch)", FSS_E_DEVICE);
        if (ptr == nullptr) return FSS_E_DEVICE;
        g_scratch_addr[device] = ptr;
        g_scratch_known[device] = true;
    }
    *out = g_scratch_addr[device];
    return FSS_OK;
}

template <typename T, int V>
int run(cudaStream_t stream, float *scratch, int64_t B, int64_t Tn, int64_t D, const fss_view *alpha,
        const fss_view *beta, const fss_view *h) {
    using namespace fss;
    using namespace fss::chunked;
    const Geometry g = make_geometry(B, Tn, D, V);
    const size_t half = align_up((size_t)(B * g.S * D) * sizeof(float), 256);
    float *wsP = scratch;
    float *wsC = reinterpret_cast<float *>(reinterpret_cast<char *>(scratch) + half);
    if (!grid_fits(g)) return FSS_E_SHAPE;
    const unsigned blocks = (unsigned)(g.vblocks * g.S * B);
    auto a = make_view<const T>(alpha);
    auto b = make_view<const T>(beta);
    chunk_summary<T, V, false><<<blocks, kThreads, 0, stream>>>(g, a, b, wsP, wsC, false);
    chunk_compose<false><<<(unsigned)ceil_div(B * D, 128), 128, 0, stream>>>(g, wsP, wsC, nullptr, nullptr,
                                                                           nullptr, nullptr, nullptr);
    chunk_scan_forward<T, V><<<blocks, kThreads, 0, stream>>>(g, a, b, make_view<T>(h), wsC, false);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FSS_OK : cuda_fail(e, "no-alloc forward launch", FSS_E_LAUNCH);
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int fss_scan_forward_noalloc(int dtype, int device, void *stream, int64_t B, int64_t T, int64_t D,
                             const fss_view *alpha, const fss_view *beta, const fss_view *h) {
    using namespace fss;
    if (dtype != FSS_DTYPE_BF16 && dtype != FSS_DTYPE_F32) return FSS_E_DTYPE;
    if (B < 0 || T < 0 || D < 0) return FSS_E_SHAPE;
    if (B == 0 || T == 0 || D == 0) return FSS_OK;
    int rc;
    if ((rc = check_view_extents(alpha, B, T, D)) || (rc = check_view_extents(beta, B, T, D)) ||
        (rc = check_view_extents(h, B, T, D)))
        return rc;
    // the fixed scratch bounds the problem: two fp32 values per (batch, chunk, channel)
    if (chunked::workspace_bytes(B, T, D) > (size_t)FSS_NOALLOC_SCRATCH_BYTES) return FSS_E_TOO_LARGE;

    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice", FSS_E_DEVICE);
    const int dev = device >= 0 ? device : prev;
    e = cudaSetDevice(dev);                                          // the lookup needs `dev` current
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice", FSS_E_DEVICE);
    void *scratch = nullptr;
    rc = scratch_address(dev, &scratch);
    if (rc == FSS_OK) {
        cudaStream_t s = (cudaStream_t)stream;
        float *ws = static_cast<float *>(scratch);
        if (dtype == FSS_DTYPE_BF16) {
            rc = chunked::vector_ok<bf16>(D, {alpha, beta, h}) ? run<bf16, 8>(s, ws, B, T, D, alpha, beta, h)
                                                               : run<bf16, 1>(s, ws, B, T, D, alpha, beta, h);
        } else {
            rc = chunked::vector_ok<float>(D, {alpha, beta, h}) ? run<float, 4>(s, ws, B, T, D, alpha, beta, h)
                                                                : run<float, 1>(s, ws, B, T, D, alpha, beta, h);
        }
    }
    if (dev != prev) cudaSetDevice(prev);
    return rc;
}
