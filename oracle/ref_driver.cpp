// TEST INFRASTRUCTURE ONLY.  A C-ABI driver around the reference project's own CPU loop
// (csrc/include/sequential_scan_cpu.hpp, templates reference_scan_fwd / reference_scan_bwd).
// That header is NOT copied here: the build recipe (oracle/build_oracle.py) passes
// -I<reference>/csrc/include and the result goes to oracle/_ref/libfss_ref.so.  Nothing in the
// product path loads this library; it validates the C restatement in scan_oracle.c and serves
// as the timed CPU baseline.
//
// The reference templates take compile-time <batch, seq, d_model>, so only the shapes listed
// in FSS_REF_SHAPES exist.  The header's "#pragma omp parallel for" shares one carry array
// between threads and is wrong when enabled, so this file is compiled WITHOUT -fopenmp and each
// batch element is run as its own <1, T, D> call; those calls are independent, which lets this
// driver spread them over host threads without touching the reference's code.
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "sequential_scan_cpu.hpp"

namespace {

struct Job {
    int64_t B, T, D;
    std::vector<std::vector<float>> alpha, beta, h, g, dalpha, dbeta;  // one vector per batch row
    void (*fwd)(std::vector<float> *, std::vector<float> *, std::vector<float> *);
    void (*bwd)(std::vector<float> *, std::vector<float> *, std::vector<float> *,
                std::vector<float> *, std::vector<float> *);
};

template <int T, int D> void bind(Job *j) {
    j->fwd = &reference_scan_fwd<1, T, D>;
    j->bwd = &reference_scan_bwd<1, T, D>;
}

// (seq, d_model) pairs that exist in this build.
#define FSS_REF_SHAPES(X) \
    X(16, 8) X(37, 24) X(3, 8) X(128, 512) X(256, 512) X(1024, 768) X(2048, 1024)

bool bind_shape(Job *j) {
#define X(TT, DD) \
    if (j->T == TT && j->D == DD) { bind<TT, DD>(j); return true; }
    FSS_REF_SHAPES(X)
#undef X
    return false;
}

template <class F> void for_each_batch(Job *j, int threads, F f) {
    if (threads < 1) threads = 1;
    if (threads > j->B) threads = (int)j->B;
    if (threads == 1) {
        for (int64_t b = 0; b < j->B; ++b) f(b);
        return;
    }
    std::vector<std::thread> pool;
    for (int w = 0; w < threads; ++w)
        pool.emplace_back([=] { for (int64_t b = w; b < j->B; b += threads) f(b); });
    for (auto &t : pool) t.join();
}

}  // namespace

extern "C" {

// Returns nullptr when (T, D) is not one of the instantiated shapes.
__attribute__((visibility("default"))) void *fss_ref_create(int64_t B, int64_t T, int64_t D) {
    Job *j = new Job();
    j->B = B; j->T = T; j->D = D;
    if (!bind_shape(j)) { delete j; return nullptr; }
    const size_t n = (size_t)T * (size_t)D;
    for (auto *v : {&j->alpha, &j->beta, &j->h, &j->g, &j->dalpha, &j->dbeta})
        v->assign((size_t)B, std::vector<float>(n, 0.0f));
    return j;
}

__attribute__((visibility("default"))) void fss_ref_destroy(void *p) { delete (Job *)p; }

// which: 0 alpha, 1 beta, 2 h, 3 g, 4 dalpha, 5 dbeta.  Buffers are contiguous [B, T, D] fp32.
static std::vector<std::vector<float>> *pick(Job *j, int which) {
    switch (which) {
    case 0: return &j->alpha; case 1: return &j->beta; case 2: return &j->h;
    case 3: return &j->g; case 4: return &j->dalpha; case 5: return &j->dbeta;
    }
    return nullptr;
}

__attribute__((visibility("default"))) int fss_ref_set(void *p, int which, const float *src) {
    Job *j = (Job *)p; auto *v = pick(j, which); if (!v) return -1;
    const size_t n = (size_t)j->T * (size_t)j->D;
    for (int64_t b = 0; b < j->B; ++b) std::memcpy((*v)[b].data(), src + b * n, n * sizeof(float));
    return 0;
}

__attribute__((visibility("default"))) int fss_ref_get(void *p, int which, float *dst) {
    Job *j = (Job *)p; auto *v = pick(j, which); if (!v) return -1;
    const size_t n = (size_t)j->T * (size_t)j->D;
    for (int64_t b = 0; b < j->B; ++b) std::memcpy(dst + b * n, (*v)[b].data(), n * sizeof(float));
    return 0;
}

// h = scan(alpha, beta): reference_scan_fwd<1,T,D> once per batch row.
__attribute__((visibility("default"))) void fss_ref_forward(void *p, int threads) {
    Job *j = (Job *)p;
    for_each_batch(j, threads, [j](int64_t b) { j->fwd(&j->alpha[b], &j->beta[b], &j->h[b]); });
}

// (dalpha, dbeta) from (alpha, h, g): reference_scan_bwd<1,T,D> once per batch row.
__attribute__((visibility("default"))) void fss_ref_backward(void *p, int threads) {
    Job *j = (Job *)p;
    for_each_batch(j, threads, [j](int64_t b) {
        j->bwd(&j->alpha[b], &j->h[b], &j->g[b], &j->dalpha[b], &j->dbeta[b]);
    });
}

}  // extern "C"
