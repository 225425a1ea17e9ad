// C ABI of the library (see include/fss_b200.h): argument checks, algorithm choice, launches.
// Nothing here allocates or frees device memory, and nothing synchronises the device.
#include <cstdio>
#include <cstring>
#include <initializer_list>
#include <string>

#include "fss_chunked.cuh"
#include "fss_common.cuh"
#include "fss_gates.cuh"
#include "fss_lookback.cuh"
#include "fss_seqpar.cuh"

#define FSS_API extern "C" __attribute__((visibility("default")))

namespace fss {

thread_local std::string g_cuda_error;

// shared with the other translation units of the library (declared in fss_common.cuh)
int cuda_fail(cudaError_t e, const char *what, int code) {
    g_cuda_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
    return code;
}

#define FSS_CUDA(call, what)                                      \
    do {                                                          \
        cudaError_t e_ = (call);                                  \
        if (e_ != cudaSuccess) return cuda_fail(e_, what, FSS_E_LAUNCH); \
    } while (0)

// Makes ctx->device current for the duration of a call and puts the previous one back.  The
// first call of a thread always binds the device, so that driver entry points used later (TMA
// descriptor encoding) find a current context even on threads that never touched CUDA through
// this library (autograd worker threads, for instance).
struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    int error = FSS_OK;
    int device = -1;
    explicit DeviceGuard(int want) {
        static thread_local int bound = -1;
        cudaError_t e = cudaGetDevice(&prev);
        if (e != cudaSuccess) { error = cuda_fail(e, "cudaGetDevice", FSS_E_DEVICE); return; }
        device = want >= 0 ? want : prev;
        if (device != prev || bound != device) {
            e = cudaSetDevice(device);
            if (e != cudaSuccess) { error = cuda_fail(e, "cudaSetDevice", FSS_E_DEVICE); return; }
            bound = device;
            switched = device != prev;
        }
    }
    ~DeviceGuard() { if (switched) cudaSetDevice(prev); }
};

static int check_ctx(const fss_scan_ctx *ctx) {
    if (!ctx) return FSS_E_NULL;
    if (ctx->struct_bytes != sizeof(fss_scan_ctx)) return FSS_E_ARGS;
    if (ctx->algo < FSS_ALGO_AUTO || ctx->algo > FSS_ALGO_LOOKBACK) return FSS_E_ALGO;
    return FSS_OK;
}

static int check_view(const fss_view *v, int64_t B, int64_t T, int64_t D) {
    return check_view_extents(v, B, T, D);
}

// Two views are "the same tensor" when they start at the same address.  Outputs that start where
// an input starts are refused (the one sanctioned case, grad_beta over h, is handled by the
// caller); partial overlaps of differently placed views are the caller's responsibility.
static bool same_start(const fss_view *a, const fss_view *b) { return a->ptr == b->ptr; }

static int check_shape(int dtype, int64_t B, int64_t T, int64_t D) {
    if (dtype != FSS_DTYPE_BF16 && dtype != FSS_DTYPE_F32) return FSS_E_DTYPE;
    if (B < 0 || T < 0 || D < 0) return FSS_E_SHAPE;
    return FSS_OK;
}

// A call that may end in the chunked kernels must fit their linear grid (checked for the
// one-element-per-thread geometry, the largest grid the family launches).
static int check_chunked_grid(const fss_scan_ctx *ctx, int64_t B, int64_t T, int64_t D) {
    if (ctx->algo == FSS_ALGO_LOOKBACK) return FSS_OK;
    return chunked::grid_fits(chunked::make_geometry(B, T, D, 1)) ? FSS_OK : FSS_E_SHAPE;
}

static int need_workspace(const fss_scan_ctx *ctx, int64_t B, int64_t T, int64_t D, int dtype) {
    if (!ctx->workspace || ctx->workspace_bytes < fss_workspace_bytes(B, T, D, dtype)) return FSS_E_WORKSPACE;
    if (!aligned16(ctx->workspace)) return FSS_E_WORKSPACE;
    return FSS_OK;
}

// Launch with the programmatic-dependent-launch attribute: the kernel may be placed while its
// predecessor on the stream drains; it must execute griddepcontrol.wait before it touches anything
// the predecessor wrote (the kernels launched this way do so first thing).
template <typename... Params, typename... Args>
static cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, Params(args)...);
}

static int launch_check(const char *what) {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FSS_OK : cuda_fail(e, what, FSS_E_LAUNCH);
}

// ------------------------------------------------------------------ chunked path
template <typename T, int V>
static int chunked_forward(const fss_scan_ctx *ctx, int64_t B, int64_t Tn, int64_t D,
                           const fss_view *alpha, const fss_view *beta, const fss_view *h,
                           const fss_forward_state *st) {
    using namespace chunked;
    cudaStream_t stream = (cudaStream_t)ctx->stream;
    const Geometry g = make_geometry(B, Tn, D, V);
    float *wsP = reinterpret_cast<float *>(plan_workspace(ctx->workspace, ctx->workspace_bytes).floats);
    float *wsC = reinterpret_cast<float *>((char *)wsP + align_up((size_t)(B * g.S * D) * sizeof(float), 256));
    const bool cont = ctx->flags & FSS_FLAG_CONTINUATION;
    if (!chunked::grid_fits(g)) return FSS_E_SHAPE;
    const unsigned blocks = (unsigned)(g.vblocks * g.S * B);
    auto a = make_view<const T>(alpha);
    auto b = make_view<const T>(beta);
    auto out = make_view<T>(h);
    chunk_summary<T, V, false><<<blocks, kThreads, 0, stream>>>(g, a, b, wsP, wsC, cont);
    const int64_t cols = B * D;
    chunk_compose<false><<<(unsigned)ceil_div(cols, 128), 128, 0, stream>>>(
        g, wsP, wsC, (st && cont) ? st->h_in : nullptr, st ? st->h_last : nullptr,
        st ? st->prod : nullptr, st ? st->block_prod : nullptr, st ? st->block_state : nullptr);
    chunk_scan_forward<T, V><<<blocks, kThreads, 0, stream>>>(g, a, b, out, wsC, cont);
    return launch_check("chunked forward launch");
}

template <typename T, int V>
static int chunked_backward(const fss_scan_ctx *ctx, int64_t B, int64_t Tn, int64_t D,
                            const fss_view *alpha, const fss_view *h, const fss_view *grad,
                            const fss_view *dalpha, const fss_view *dbeta,
                            const fss_backward_state *st) {
    using namespace chunked;
    cudaStream_t stream = (cudaStream_t)ctx->stream;
    const Geometry g = make_geometry(B, Tn, D, V);
    float *wsP = reinterpret_cast<float *>(plan_workspace(ctx->workspace, ctx->workspace_bytes).floats);
    float *wsC = reinterpret_cast<float *>((char *)wsP + align_up((size_t)(B * g.S * D) * sizeof(float), 256));
    const bool cont = ctx->flags & FSS_FLAG_CONTINUATION;
    if (!chunked::grid_fits(g)) return FSS_E_SHAPE;
    const unsigned blocks = (unsigned)(g.vblocks * g.S * B);
    auto a = make_view<const T>(alpha);
    auto hh = make_view<const T>(h);
    auto gr = make_view<const T>(grad);
    chunk_summary<T, V, true><<<blocks, kThreads, 0, stream>>>(g, a, gr, wsP, wsC, cont);
    const int64_t cols = B * D;
    chunk_compose<true><<<(unsigned)ceil_div(cols, 128), 128, 0, stream>>>(
        g, wsP, wsC, st ? st->u_in : nullptr, st ? st->u_out : nullptr, nullptr,
        st ? st->block_prod : nullptr, st ? st->block_state : nullptr);
    chunk_scan_backward<T, V><<<blocks, kThreads, 0, stream>>>(
        g, a, hh, gr, make_view<T>(dalpha), make_view<T>(dbeta), wsC,
        (st && cont) ? st->h_prev : nullptr, cont);
    return launch_check("chunked backward launch");
}

template <typename T>
static int forward_typed(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t Tn, int64_t D,
                         const fss_view *alpha, const fss_view *beta, const fss_view *h,
                         const fss_forward_state *st) {
    int algo = ctx->algo;
    if (algo != FSS_ALGO_CHUNKED) {
        const bool ok = lookback::layout_ok<T>(B, Tn, D, {alpha, beta, h}) &&
                        (!st || lookback::state_aligned({st->h_in, st->h_last, st->prod, st->block_prod, st->block_state}));
        if (!ok && algo == FSS_ALGO_LOOKBACK) return FSS_E_LAYOUT;
        algo = ok ? FSS_ALGO_LOOKBACK : FSS_ALGO_CHUNKED;
    }
    if (algo == FSS_ALGO_LOOKBACK)
        return lookback::forward<T>(ctx, plan_workspace(ctx->workspace, ctx->workspace_bytes), B, Tn, D, alpha, beta, h, st, &g_cuda_error);
    constexpr int V = VecWidth<T>::value;
    if (chunked::vector_ok<T>(D, {alpha, beta, h}))
        return chunked_forward<T, V>(ctx, B, Tn, D, alpha, beta, h, st);
    return chunked_forward<T, 1>(ctx, B, Tn, D, alpha, beta, h, st);
}

template <typename T>
static int backward_typed(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t Tn, int64_t D,
                          const fss_view *alpha, const fss_view *h, const fss_view *grad,
                          const fss_view *dalpha, const fss_view *dbeta,
                          const fss_backward_state *st) {
    int algo = ctx->algo;
    // grad_beta written over h (what the reference's bf16 backward always does,
    // csrc/sequential_scan_kernel.cu:197).  Safe in the look-back kernel: row t of h is read by
    // the tile that holds row t and, as h_{t-1}, by the tile that holds row t+1; the latter is
    // earlier in the backward tile order, and this tile's results leave only after its carry
    // arrived, i.e. after that earlier tile's loads.  The chunked kernels give no such order.
    const bool inplace = dbeta->ptr == h->ptr;
    if (inplace && (dbeta->stride_b != h->stride_b || dbeta->stride_t != h->stride_t)) return FSS_E_LAYOUT;
    if (algo != FSS_ALGO_CHUNKED) {
        const bool ok = lookback::layout_ok<T>(B, Tn, D, {alpha, h, grad, dalpha, dbeta}) &&
                        (!st || lookback::state_aligned({st->u_in, st->h_prev, st->u_out, st->block_prod, st->block_state}));
        if (!ok && algo == FSS_ALGO_LOOKBACK) return FSS_E_LAYOUT;
        algo = ok ? FSS_ALGO_LOOKBACK : FSS_ALGO_CHUNKED;
    }
    if (inplace && algo == FSS_ALGO_CHUNKED) return FSS_E_LAYOUT;
    if (algo == FSS_ALGO_LOOKBACK)
        return lookback::backward<T>(ctx, plan_workspace(ctx->workspace, ctx->workspace_bytes), B, Tn, D, alpha, h, grad,
                                     dalpha, dbeta, st, &g_cuda_error);
    constexpr int V = VecWidth<T>::value;
    if (chunked::vector_ok<T>(D, {alpha, h, grad, dalpha, dbeta}))
        return chunked_backward<T, V>(ctx, B, Tn, D, alpha, h, grad, dalpha, dbeta, st);
    return chunked_backward<T, 1>(ctx, B, Tn, D, alpha, h, grad, dalpha, dbeta, st);
}

}  // namespace fss

using namespace fss;

// ====================================================================== exported functions

FSS_API int fss_abi_version(void) { return FSS_ABI_VERSION; }

FSS_API const char *fss_strerror(int code) {
    switch (code) {
    case FSS_OK: return "ok";
    case FSS_E_NULL: return "a required pointer is NULL";
    case FSS_E_SHAPE: return "bad shape or stride";
    case FSS_E_DTYPE: return "unknown dtype";
    case FSS_E_WORKSPACE: return "workspace missing, misaligned or too small";
    case FSS_E_LAYOUT: return "layout not usable by the look-back (TMA) kernels";
    case FSS_E_LAUNCH: return "CUDA launch failed";
    case FSS_E_ALGO: return "unknown algorithm";
    case FSS_E_DEVICE: return "CUDA device selection failed";
    case FSS_E_TENSORMAP: return "TMA descriptor rejected by the driver";
    case FSS_E_ARGS: return "struct_bytes does not match this library";
    case FSS_E_TOO_LARGE: return "problem larger than this entry point's fixed capacity";
    case FSS_E_ALIAS: return "an output tensor starts at the address of an input (or of the other output)";
    }
    return "unknown error code";
}

FSS_API const char *fss_last_cuda_error(void) { return g_cuda_error.c_str(); }

FSS_API size_t fss_workspace_bytes(int64_t B, int64_t T, int64_t D, int dtype) {
    if (B <= 0 || T <= 0 || D <= 0) return workspace_total(0);
    size_t a = chunked::workspace_bytes(B, T, D);
    size_t b = lookback::workspace_bytes(B, T, D, dtype);
    size_t c = lookback::float_scratch_bytes(B, T, D);
    if (b > a) a = b;
    return workspace_total(a > c ? a : c);
}

FSS_API int fss_workspace_init(void *workspace, size_t bytes, void *stream) {
    if (!workspace) return FSS_E_NULL;
    FSS_CUDA(cudaMemsetAsync(workspace, 0, bytes, (cudaStream_t)stream), "cudaMemsetAsync(workspace)");
    return FSS_OK;
}

FSS_API int64_t fss_block_rows(int dtype, int64_t B, int64_t T, int64_t D, int algo) {
    if (B <= 0 || T <= 0 || D <= 0) return 1;
    if (algo == FSS_ALGO_CHUNKED) return chunked::make_geometry(B, T, D, 1).L;
    return lookback::block_rows(dtype, B, T, D);
}

FSS_API int fss_scan_forward_ex(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                                const fss_view *alpha, const fss_view *beta, const fss_view *h,
                                const fss_forward_state *state) {
    int rc;
    if ((rc = check_ctx(ctx))) return rc;
    if ((rc = check_shape(dtype, B, T, D))) return rc;
    if (B == 0 || T == 0 || D == 0) return FSS_OK;
    if ((rc = check_view(alpha, B, T, D)) || (rc = check_view(beta, B, T, D)) || (rc = check_view(h, B, T, D)))
        return rc;
    if (same_start(h, alpha) || same_start(h, beta)) return FSS_E_ALIAS;
    if ((rc = check_chunked_grid(ctx, B, T, D))) return rc;
    if ((rc = need_workspace(ctx, B, T, D, dtype))) return rc;
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
    return dtype == FSS_DTYPE_BF16
               ? forward_typed<bf16>(ctx, dtype, B, T, D, alpha, beta, h, state)
               : forward_typed<float>(ctx, dtype, B, T, D, alpha, beta, h, state);
}

FSS_API int fss_scan_forward_gated(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                                   const fss_view *r, const fss_view *i, const fss_view *x,
                                   const float *lambda, const fss_view *h, const fss_forward_state *state) {
    int rc;
    if ((rc = check_ctx(ctx))) return rc;
    if ((rc = check_shape(dtype, B, T, D))) return rc;
    if (B == 0 || T == 0 || D == 0) return FSS_OK;
    if (!lambda) return FSS_E_NULL;
    for (const fss_view *v : {r, i, x, h})
        if ((rc = check_view(v, B, T, D))) return rc;
    if (same_start(h, r) || same_start(h, i) || same_start(h, x)) return FSS_E_ALIAS;
    if (state && (state->prod || state->block_prod || state->block_state)) return FSS_E_ARGS;
    if (ctx->algo == FSS_ALGO_CHUNKED) return FSS_E_LAYOUT;       // single-pass kernel only
    if (state && !lookback::state_aligned({state->h_in, state->h_last})) return FSS_E_LAYOUT;
    if ((rc = need_workspace(ctx, B, T, D, dtype))) return rc;
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
    const WsPlan ws = plan_workspace(ctx->workspace, ctx->workspace_bytes);
    if (dtype == FSS_DTYPE_BF16) {
        if (!lookback::layout_ok<bf16>(B, T, D, {r, i, x, h})) return FSS_E_LAYOUT;
        return lookback::forward_gated<bf16>(ctx, ws, B, T, D, r, i, x, lambda, h, state, &g_cuda_error);
    }
    if (!lookback::layout_ok<float>(B, T, D, {r, i, x, h})) return FSS_E_LAYOUT;
    return lookback::forward_gated<float>(ctx, ws, B, T, D, r, i, x, lambda, h, state, &g_cuda_error);
}

FSS_API int fss_scan_backward_ex(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                                 const fss_view *alpha, const fss_view *h, const fss_view *grad_out,
                                 const fss_view *grad_alpha, const fss_view *grad_beta,
                                 const fss_backward_state *state) {
    int rc;
    if ((rc = check_ctx(ctx))) return rc;
    if ((rc = check_shape(dtype, B, T, D))) return rc;
    if (B == 0 || T == 0 || D == 0) return FSS_OK;
    for (const fss_view *v : {alpha, h, grad_out, grad_alpha, grad_beta})
        if ((rc = check_view(v, B, T, D))) return rc;
    // grad_beta may be h itself (checked in backward_typed); every other coincidence is refused
    if (same_start(grad_alpha, alpha) || same_start(grad_alpha, h) || same_start(grad_alpha, grad_out) ||
        same_start(grad_alpha, grad_beta) || same_start(grad_beta, alpha) || same_start(grad_beta, grad_out))
        return FSS_E_ALIAS;
    if ((rc = check_chunked_grid(ctx, B, T, D))) return rc;
    if ((rc = need_workspace(ctx, B, T, D, dtype))) return rc;
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
    return dtype == FSS_DTYPE_BF16
               ? backward_typed<bf16>(ctx, dtype, B, T, D, alpha, h, grad_out, grad_alpha, grad_beta, state)
               : backward_typed<float>(ctx, dtype, B, T, D, alpha, h, grad_out, grad_alpha, grad_beta, state);
}

FSS_API int fss_scan_forward(const fss_scan_ctx *ctx, int64_t B, int64_t T, int64_t D,
                             const fss_view *alpha, const fss_view *beta, const fss_view *h) {
    return fss_scan_forward_ex(ctx, FSS_DTYPE_F32, B, T, D, alpha, beta, h, nullptr);
}

FSS_API int fss_scan_backward(const fss_scan_ctx *ctx, int64_t B, int64_t T, int64_t D,
                              const fss_view *alpha, const fss_view *h, const fss_view *grad_out,
                              const fss_view *grad_alpha, const fss_view *grad_beta) {
    return fss_scan_backward_ex(ctx, FSS_DTYPE_F32, B, T, D, alpha, h, grad_out, grad_alpha, grad_beta, nullptr);
}

FSS_API int fss_scan_forward_half(const fss_scan_ctx *ctx, int64_t B, int64_t T, int64_t D,
                                  const fss_view *alpha, const fss_view *beta, const fss_view *h) {
    return fss_scan_forward_ex(ctx, FSS_DTYPE_BF16, B, T, D, alpha, beta, h, nullptr);
}

FSS_API int fss_scan_backward_half(const fss_scan_ctx *ctx, int64_t B, int64_t T, int64_t D,
                                   const fss_view *alpha, const fss_view *h, const fss_view *grad_out,
                                   const fss_view *grad_alpha, const fss_view *grad_beta) {
    return fss_scan_backward_ex(ctx, FSS_DTYPE_BF16, B, T, D, alpha, h, grad_out, grad_alpha, grad_beta, nullptr);
}

// ---------------------------------------------------------------------- sequence-parallel
FSS_API int fss_seqpar_compose(const fss_scan_ctx *ctx, int backward, int world, int rank, int64_t n,
                               const float *pc, float *carry_in) {
    int rc;
    if ((rc = check_ctx(ctx))) return rc;
    if (!pc || !carry_in) return FSS_E_NULL;
    if (world < 1 || rank < 0 || rank >= world || n < 0) return FSS_E_SHAPE;
    if (n == 0) return FSS_OK;
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
    seqpar::compose<<<(unsigned)ceil_div(n, 256), 256, 0, (cudaStream_t)ctx->stream>>>(
        backward, world, rank, n, pc, carry_in);
    return launch_check("seqpar compose launch");
}

namespace fss {
static int fill_peers(seqpar::PeerTables *peers, int world, void *const *tables, void *const *words) {
    if (!tables || !words) return FSS_E_NULL;
    for (int q = 0; q < world; ++q) {
        if (!tables[q] || !words[q]) return FSS_E_NULL;
        peers->table[q] = static_cast<unsigned long long *>(tables[q]);
        peers->words[q] = static_cast<uint32_t *>(words[q]);
    }
    return FSS_OK;
}
static int check_exchange(const fss_scan_ctx *ctx, int world, int rank, int64_t n, uint32_t epoch) {
    if (int rc = check_ctx(ctx)) return rc;
    if (world < 1 || world > seqpar::kMaxPeers || rank < 0 || rank >= world || n < 0 || epoch == 0) return FSS_E_SHAPE;
    return FSS_OK;
}
static uint32_t exchange_spins(const fss_scan_ctx *ctx) {
    return (ctx->flags & FSS_FLAG_TEST_SHORT_WAITS) ? 4096u : (1u << 22);
}
}  // namespace fss

FSS_API int fss_seqpar_push(const fss_scan_ctx *ctx, int backward, int world, int rank, int64_t n, const float *prod,
                            const float *state, void *const *peer_tables, void *const *peer_words, uint32_t epoch) {
    int rc;
    if ((rc = check_exchange(ctx, world, rank, n, epoch))) return rc;
    if (!prod || !state) return FSS_E_NULL;
    seqpar::PeerTables peers{};
    if ((rc = fill_peers(&peers, world, peer_tables, peer_words))) return rc;
    if (n == 0) return FSS_OK;
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
    int64_t blocks = ceil_div(2 * n, (int64_t)seqpar::kPushThreads);
    if (blocks > 148) blocks = 148;
    FSS_CUDA(launch_dependent(seqpar::peer_push, dim3((unsigned)blocks), dim3(seqpar::kPushThreads), 0,
                              (cudaStream_t)ctx->stream, peers, backward, world, rank, n, prod, state, epoch, ctx->status,
                              exchange_spins(ctx)),
             "carry push launch");
    return launch_check("carry push launch");
}

FSS_API int fss_seqpar_push_blocks(const fss_scan_ctx *ctx, int world, int rank, int64_t B, int64_t nblocks, int64_t D,
                                   const float *block_prod, const float *state, float *prod_out,
                                   void *const *peer_tables, void *const *peer_words, uint32_t epoch) {
    int rc;
    if ((rc = check_exchange(ctx, world, rank, B * D, epoch))) return rc;
    if (!block_prod || !state || !prod_out) return FSS_E_NULL;
    if (B < 0 || nblocks < 1 || D < 0 || B > 65535) return FSS_E_SHAPE;
    if (D % 4 || !aligned16(block_prod) || !aligned16(state) || !aligned16(prod_out)) return FSS_E_LAYOUT;
    seqpar::PeerTables peers{};
    if ((rc = fill_peers(&peers, world, peer_tables, peer_words))) return rc;
    if (B == 0 || D == 0) return FSS_OK;
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
    const dim3 grid((unsigned)ceil_div(D, 4 * seqpar::kPushVecs), (unsigned)B);
    FSS_CUDA(launch_dependent(seqpar::peer_push_blocks, grid, dim3(seqpar::kPushSlices * seqpar::kPushVecs), 0,
                              (cudaStream_t)ctx->stream, peers, world, rank, nblocks, D, block_prod, state, prod_out, epoch,
                              ctx->status, exchange_spins(ctx)),
             "carry push launch");
    return launch_check("carry push launch");
}

FSS_API int fss_seqpar_compose_peer(const fss_scan_ctx *ctx, int backward, int world, int rank, int64_t n,
                                    void *const *peer_tables, void *const *peer_words, uint32_t epoch,
                                    float *carry_in) {
    int rc;
    if ((rc = check_exchange(ctx, world, rank, n, epoch))) return rc;
    if (!carry_in) return FSS_E_NULL;
    seqpar::PeerTables peers{};
    if ((rc = fill_peers(&peers, world, peer_tables, peer_words))) return rc;
    if (n == 0) return FSS_OK;
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
    seqpar::peer_compose<<<(unsigned)ceil_div(n, 256), 256, 0, (cudaStream_t)ctx->stream>>>(
        peers, backward, world, rank, n, epoch, carry_in, ctx->status, exchange_spins(ctx));
    return launch_check("carry compose launch");
}

namespace fss {
// multiprocessors of the current device (cached per device; 148 if the query fails)
static int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        cached[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
    }
    return cached[dev];
}

static seqpar::Geometry fixup_geometry(int64_t B, int64_t T, int64_t D, int64_t R, int V) {
    seqpar::Geometry g;
    g.B = B; g.T = T; g.D = D; g.R = R;
    g.NB = ceil_div(T, R);
    g.nvec = D / V;
    g.vblocks = ceil_div(g.nvec, 32);
    g.slots = seqpar::choose_slots(g.NB, g.vblocks, B, sm_count());
    return g;
}
static bool fixup_grid_ok(const seqpar::Geometry &g) { return g.vblocks <= 65535 && g.B <= 65535; }

// A fix-up kernel publishes this rank's own pair itself only when all its CTAs are on the GPU at
// the same time: they wait for pairs that the same kernel publishes on the other ranks, so a grid
// that runs in waves could wait for a CTA that has not started.  For such a grid the pair is sent
// by a push launch placed before the fix-up, as a caller without `push_state` would do.
static int publish_before(const fss_scan_ctx *ctx, const seqpar::Geometry &g, int backward, seqpar::CarrySource *src,
                          const float *bp) {
    if (!src->push_state) return FSS_OK;
    if ((int64_t)g.slots * g.vblocks * g.B <= sm_count()) return FSS_OK;
    const int64_t n = g.B * g.D;
    if (src->push_prod) {
        int64_t blocks = ceil_div(2 * n, (int64_t)seqpar::kPushThreads);
        if (blocks > 148) blocks = 148;
        FSS_CUDA(launch_dependent(seqpar::peer_push, dim3((unsigned)blocks), dim3(seqpar::kPushThreads), 0,
                                  (cudaStream_t)ctx->stream, src->peers, backward, (int)src->world, (int)src->rank, n,
                                  src->push_prod, src->push_state, src->epoch, ctx->status, src->max_spins),
                 "carry push launch");
    } else {
        if (g.D % 4 || !src->push_prod_out || !aligned16(bp) || !aligned16(src->push_state) || !aligned16(src->push_prod_out))
            return FSS_E_LAYOUT;
        const dim3 grid((unsigned)ceil_div(g.D, 4 * seqpar::kPushVecs), (unsigned)g.B);
        FSS_CUDA(launch_dependent(seqpar::peer_push_blocks, grid, dim3(seqpar::kPushSlices * seqpar::kPushVecs), 0,
                                  (cudaStream_t)ctx->stream, src->peers, (int)src->world, (int)src->rank, g.NB, g.D, bp,
                                  src->push_state, src->push_prod_out, src->epoch, ctx->status, src->max_spins),
                 "carry push launch");
    }
    if (int rc = launch_check("carry push launch")) return rc;
    src->push_state = nullptr;
    src->push_prod = nullptr;
    src->push_prod_out = nullptr;
    return FSS_OK;
}

// Room for the alpha rows of one block in shared memory (see the fix-up kernels): 16 warps x `per`
// rows x 32 lanes of the packed fragment; 0 = the block is too tall, the kernels then read alpha twice.
template <typename T, int V, typename Kernel>
static size_t fixup_stage_bytes(const seqpar::Geometry &g, Kernel kernel) {
    const int64_t per = (g.R + seqpar::kFixWarps - 1) / seqpar::kFixWarps;
    const size_t bytes = (size_t)seqpar::kFixWarps * per * 32 * sizeof(typename Frag<T, V>::Raw);
    constexpr size_t kMost = 160 * 1024;
    if (bytes == 0 || bytes > kMost) return 0;
    // the limit is raised once per device and kernel instantiation (the template parameters make this function unique)
    static bool raised[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (!raised[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMost) != cudaSuccess) {
            (void)cudaGetLastError();
            return 0;
        }
        raised[dev] = true;
    }
    return bytes;
}

template <typename T, int V>
static int fixup_forward_launch(const fss_scan_ctx *ctx, int64_t B, int64_t Tn, int64_t D, const fss_view *alpha,
                                const fss_view *beta, const fss_view *h, const seqpar::CarrySource &carry_from, const float *bp,
                                const float *bs, int64_t R) {
    const seqpar::Geometry g = fixup_geometry(B, Tn, D, R, V);
    if (!fixup_grid_ok(g)) return FSS_E_SHAPE;
    seqpar::CarrySource carry_in = carry_from;
    if (int rc = publish_before(ctx, g, 0, &carry_in, bp)) return rc;
    const dim3 grid((unsigned)g.slots, (unsigned)g.vblocks, (unsigned)B);
    const size_t stage = fixup_stage_bytes<T, V>(g, seqpar::fixup_forward<T, V, true>);
    if (stage) {
        FSS_CUDA(launch_dependent(seqpar::fixup_forward<T, V, true>, grid, dim3(seqpar::kFixThreads), stage,
                                  (cudaStream_t)ctx->stream, g, make_view<const T>(alpha), make_view<const T>(beta),
                                  make_view<T>(h), carry_in, bp, bs, ctx->status),
                 "seqpar forward fix-up launch");
    } else {
        FSS_CUDA(launch_dependent(seqpar::fixup_forward<T, V, false>, grid, dim3(seqpar::kFixThreads), 0,
                                  (cudaStream_t)ctx->stream, g, make_view<const T>(alpha), make_view<const T>(beta),
                                  make_view<T>(h), carry_in, bp, bs, ctx->status),
                 "seqpar forward fix-up launch");
    }
    return launch_check("seqpar forward fix-up launch");
}

template <typename T, int V>
static int fixup_backward_launch(const fss_scan_ctx *ctx, int64_t B, int64_t Tn, int64_t D, const fss_view *alpha,
                                 const fss_view *h, const fss_view *grad, const fss_view *da, const fss_view *db,
                                 const seqpar::CarrySource &u_from, const float *h_prev, const float *bp, const float *bs,
                                 int64_t R) {
    const seqpar::Geometry g = fixup_geometry(B, Tn, D, R, V);
    if (!fixup_grid_ok(g)) return FSS_E_SHAPE;
    seqpar::CarrySource u_in = u_from;
    if (int rc = publish_before(ctx, g, 1, &u_in, bp)) return rc;
    const dim3 grid((unsigned)g.slots, (unsigned)g.vblocks, (unsigned)B);
    const size_t stage = fixup_stage_bytes<T, V>(g, seqpar::fixup_backward<T, V, true>);
    const bool cont = (ctx->flags & FSS_FLAG_CONTINUATION) != 0;
    if (stage) {
        FSS_CUDA(launch_dependent(seqpar::fixup_backward<T, V, true>, grid, dim3(seqpar::kFixThreads), stage,
                                  (cudaStream_t)ctx->stream, g, make_view<const T>(alpha), make_view<const T>(h),
                                  make_view<const T>(grad), make_view<T>(da), make_view<T>(db), u_in, h_prev, bp, bs, cont,
                                  ctx->status),
                 "seqpar backward fix-up launch");
    } else {
        FSS_CUDA(launch_dependent(seqpar::fixup_backward<T, V, false>, grid, dim3(seqpar::kFixThreads), 0,
                                  (cudaStream_t)ctx->stream, g, make_view<const T>(alpha), make_view<const T>(h),
                                  make_view<const T>(grad), make_view<T>(da), make_view<T>(db), u_in, h_prev, bp, bs, cont,
                                  ctx->status),
                 "seqpar backward fix-up launch");
    }
    return launch_check("seqpar backward fix-up launch");
}

static int fixup_forward_dispatch(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D, const fss_view *alpha,
                                  const fss_view *beta, const fss_view *h, const seqpar::CarrySource &src, const float *bp,
                                  const float *bs, int64_t R) {
    if (dtype == FSS_DTYPE_BF16) {
        if (chunked::vector_ok<bf16>(D, {alpha, beta, h}))
            return fixup_forward_launch<bf16, 8>(ctx, B, T, D, alpha, beta, h, src, bp, bs, R);
        return fixup_forward_launch<bf16, 1>(ctx, B, T, D, alpha, beta, h, src, bp, bs, R);
    }
    if (chunked::vector_ok<float>(D, {alpha, beta, h}))
        return fixup_forward_launch<float, 4>(ctx, B, T, D, alpha, beta, h, src, bp, bs, R);
    return fixup_forward_launch<float, 1>(ctx, B, T, D, alpha, beta, h, src, bp, bs, R);
}
static int fixup_backward_dispatch(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D, const fss_view *alpha,
                                   const fss_view *h, const fss_view *grad, const fss_view *da, const fss_view *db,
                                   const seqpar::CarrySource &src, const float *h_prev, const float *bp, const float *bs,
                                   int64_t R) {
#define FSS_FIXB(TT, VV) fixup_backward_launch<TT, VV>(ctx, B, T, D, alpha, h, grad, da, db, src, h_prev, bp, bs, R)
    if (dtype == FSS_DTYPE_BF16)
        return chunked::vector_ok<bf16>(D, {alpha, h, grad, da, db}) ? FSS_FIXB(bf16, 8) : FSS_FIXB(bf16, 1);
    return chunked::vector_ok<float>(D, {alpha, h, grad, da, db}) ? FSS_FIXB(float, 4) : FSS_FIXB(float, 1);
#undef FSS_FIXB
}
static seqpar::CarrySource ready_carry(const float *carry) {
    seqpar::CarrySource s{};
    s.carry = carry;
    return s;
}
// From the caller's description of a gathered table; FSS_OK or an error code.
static int table_carry(const fss_scan_ctx *ctx, const fss_carry_source *src, int64_t n, seqpar::CarrySource *out) {
    if (!src || (!src->table && !src->epoch)) return FSS_E_NULL;
    if (src->world < 1 || src->world > seqpar::kMaxPeers || src->rank < 0 || src->rank >= src->world) return FSS_E_SHAPE;
    seqpar::CarrySource s{};
    s.table = src->table;
    s.carry_out = src->carry_out;
    s.n = n;
    s.world = src->world;
    s.rank = src->rank;
    s.epoch = src->epoch;
    s.max_spins = exchange_spins(ctx);
    if (src->epoch) {
        if (int rc = fill_peers(&s.peers, src->world, src->peer_tables, src->peer_words)) return rc;
    }
    if (src->push_state) {
        if (!src->epoch) return FSS_E_NULL;      // only a peer exchange can be published from inside the kernel
        s.push_state = src->push_state;
        s.push_prod = src->push_prod;
        s.push_prod_out = src->push_prod_out;
    }
    *out = s;
    return FSS_OK;
}
}  // namespace fss

FSS_API int fss_seqpar_fixup_forward(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                                     const fss_view *alpha, const fss_view *beta, const fss_view *h,
                                     const float *carry_in, const float *block_prod, const float *block_state,
                                     int64_t block_rows) {
    int rc;
    if ((rc = check_ctx(ctx))) return rc;
    if ((rc = check_shape(dtype, B, T, D))) return rc;
    if (B == 0 || T == 0 || D == 0) return FSS_OK;
    for (const fss_view *v : {alpha, beta, h})
        if ((rc = check_view(v, B, T, D))) return rc;
    if (!carry_in || !block_prod || !block_state) return FSS_E_NULL;
    if (block_rows < 1) return FSS_E_SHAPE;
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
    return fixup_forward_dispatch(ctx, dtype, B, T, D, alpha, beta, h, ready_carry(carry_in), block_prod, block_state, block_rows);
}

FSS_API int fss_seqpar_fixup_forward_from(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                                          const fss_view *alpha, const fss_view *beta, const fss_view *h,
                                          const fss_carry_source *source, const float *block_prod,
                                          const float *block_state, int64_t block_rows) {
    int rc;
    if ((rc = check_ctx(ctx))) return rc;
    if ((rc = check_shape(dtype, B, T, D))) return rc;
    if (B == 0 || T == 0 || D == 0) return FSS_OK;
    for (const fss_view *v : {alpha, beta, h})
        if ((rc = check_view(v, B, T, D))) return rc;
    if (!block_prod || !block_state) return FSS_E_NULL;
    if (block_rows < 1) return FSS_E_SHAPE;
    seqpar::CarrySource src;
    if ((rc = table_carry(ctx, source, B * D, &src))) return rc;
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
    return fixup_forward_dispatch(ctx, dtype, B, T, D, alpha, beta, h, src, block_prod, block_state, block_rows);
}

FSS_API int fss_seqpar_fixup_backward(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                                      const fss_view *alpha, const fss_view *h, const fss_view *grad_out,
                                      const fss_view *grad_alpha, const fss_view *grad_beta, const float *u_in,
                                      const float *h_prev, const float *block_prod, const float *block_state,
                                      int64_t block_rows) {
    int rc;
    if ((rc = check_ctx(ctx))) return rc;
    if ((rc = check_shape(dtype, B, T, D))) return rc;
    if (B == 0 || T == 0 || D == 0) return FSS_OK;
    for (const fss_view *v : {alpha, h, grad_out, grad_alpha, grad_beta})
        if ((rc = check_view(v, B, T, D))) return rc;
    if (!u_in || !block_prod || !block_state) return FSS_E_NULL;
    if (block_rows < 1) return FSS_E_SHAPE;
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
    return fixup_backward_dispatch(ctx, dtype, B, T, D, alpha, h, grad_out, grad_alpha, grad_beta, ready_carry(u_in), h_prev,
                                   block_prod, block_state, block_rows);
}

FSS_API int fss_seqpar_fixup_backward_from(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                                           const fss_view *alpha, const fss_view *h, const fss_view *grad_out,
                                           const fss_view *grad_alpha, const fss_view *grad_beta,
                                           const fss_carry_source *source, const float *h_prev, const float *block_prod,
                                           const float *block_state, int64_t block_rows) {
    int rc;
    if ((rc = check_ctx(ctx))) return rc;
    if ((rc = check_shape(dtype, B, T, D))) return rc;
    if (B == 0 || T == 0 || D == 0) return FSS_OK;
    for (const fss_view *v : {alpha, h, grad_out, grad_alpha, grad_beta})
        if ((rc = check_view(v, B, T, D))) return rc;
    if (!block_prod || !block_state) return FSS_E_NULL;
    if (block_rows < 1) return FSS_E_SHAPE;
    seqpar::CarrySource src;
    if ((rc = table_carry(ctx, source, B * D, &src))) return rc;
    if (src.push_state && !src.push_prod) return FSS_E_NULL;      // the backward has no block products of alpha to fold
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
    return fixup_backward_dispatch(ctx, dtype, B, T, D, alpha, h, grad_out, grad_alpha, grad_beta, src, h_prev, block_prod,
                                   block_state, block_rows);
}

// ---------------------------------------------------------------------- gates outside the scan
namespace fss {
template <typename T, int V>
static int gates_forward_launch(const fss_scan_ctx *ctx, int64_t B, int64_t Tn, int64_t D, const fss_view *r,
                                const fss_view *i, const fss_view *x, const float *lambda, const fss_view *alpha,
                                const fss_view *beta) {
    const dim3 grid((unsigned)ceil_div(D / V, gates::kThreads), (unsigned)ceil_div(Tn, gates::kRowsPerCta), (unsigned)B);
    const fss_view *bv = beta ? beta : alpha;
    gates::materialize<T, V><<<grid, gates::kThreads, 0, (cudaStream_t)ctx->stream>>>(
        B, Tn, D, make_view<const T>(r), make_view<const T>(i ? i : r), make_view<const T>(x ? x : r), lambda,
        make_view<T>(alpha), make_view<T>(bv), beta != nullptr);
    return launch_check("gate launch");
}
template <typename T, int V>
static int gates_backward_launch(const fss_scan_ctx *ctx, int64_t B, int64_t Tn, int64_t D, const fss_view *r,
                                 const fss_view *i, const fss_view *x, const float *lambda, const fss_view *da,
                                 const fss_view *db, const fss_view *dr, const fss_view *di, const fss_view *dx,
                                 float *dlambda) {
    const dim3 grid((unsigned)ceil_div(D / V, gates::kThreads), (unsigned)ceil_div(Tn, gates::kRowsPerCta), (unsigned)B);
    gates::backward<T, V><<<grid, gates::kThreads, 0, (cudaStream_t)ctx->stream>>>(
        B, Tn, D, make_view<const T>(r), make_view<const T>(i), make_view<const T>(x), lambda, make_view<const T>(da),
        make_view<const T>(db), make_view<T>(dr), make_view<T>(di), make_view<T>(dx), dlambda);
    return launch_check("gate backward launch");
}
static bool gate_grid_ok(int64_t B, int64_t Tn) { return B <= 65535 && ceil_div(Tn, gates::kRowsPerCta) <= 65535; }
}  // namespace fss

FSS_API int fss_gates_forward(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                              const fss_view *r, const fss_view *i, const fss_view *x, const float *lambda,
                              const fss_view *alpha, const fss_view *beta) {
    int rc;
    if ((rc = check_ctx(ctx))) return rc;
    if ((rc = check_shape(dtype, B, T, D))) return rc;
    if (B == 0 || T == 0 || D == 0) return FSS_OK;
    if (!lambda) return FSS_E_NULL;
    if ((rc = check_view(r, B, T, D)) || (rc = check_view(alpha, B, T, D))) return rc;
    if (beta && ((rc = check_view(i, B, T, D)) || (rc = check_view(x, B, T, D)) || (rc = check_view(beta, B, T, D))))
        return rc;
    if (!gate_grid_ok(B, T)) return FSS_E_SHAPE;
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
#define FSS_GF(TT, VV) gates_forward_launch<TT, VV>(ctx, B, T, D, r, i, x, lambda, alpha, beta)
    if (dtype == FSS_DTYPE_BF16)
        return chunked::vector_ok<bf16>(D, {r, beta ? i : r, beta ? x : r, alpha, beta}) ? FSS_GF(bf16, 8) : FSS_GF(bf16, 1);
    return chunked::vector_ok<float>(D, {r, beta ? i : r, beta ? x : r, alpha, beta}) ? FSS_GF(float, 4) : FSS_GF(float, 1);
#undef FSS_GF
}

FSS_API int fss_gates_backward(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                               const fss_view *r, const fss_view *i, const fss_view *x, const float *lambda,
                               const fss_view *grad_alpha, const fss_view *grad_beta, const fss_view *grad_r,
                               const fss_view *grad_i, const fss_view *grad_x, float *grad_lambda) {
    int rc;
    if ((rc = check_ctx(ctx))) return rc;
    if ((rc = check_shape(dtype, B, T, D))) return rc;
    if (B == 0 || T == 0 || D == 0) return FSS_OK;
    if (!lambda || !grad_lambda) return FSS_E_NULL;
    for (const fss_view *v : {r, i, x, grad_alpha, grad_beta, grad_r, grad_i, grad_x})
        if ((rc = check_view(v, B, T, D))) return rc;
    if (!gate_grid_ok(B, T)) return FSS_E_SHAPE;
    DeviceGuard guard(ctx->device);
    if (guard.error) return guard.error;
#define FSS_GB(TT, VV) gates_backward_launch<TT, VV>(ctx, B, T, D, r, i, x, lambda, grad_alpha, grad_beta, grad_r, grad_i, grad_x, grad_lambda)
    if (dtype == FSS_DTYPE_BF16)
        return chunked::vector_ok<bf16>(D, {r, i, x, grad_alpha, grad_beta, grad_r, grad_i, grad_x}) ? FSS_GB(bf16, 8) : FSS_GB(bf16, 1);
    return chunked::vector_ok<float>(D, {r, i, x, grad_alpha, grad_beta, grad_r, grad_i, grad_x}) ? FSS_GB(float, 4) : FSS_GB(float, 1);
#undef FSS_GB
}
