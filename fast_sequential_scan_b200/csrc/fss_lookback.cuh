// placeholder until the single-pass kernels land: reports "layout not usable" for every input
#pragma once
#include <initializer_list>
#include "fss_common.cuh"
namespace fss { namespace lookback {
template <typename T> inline bool layout_ok(int64_t, int64_t, int64_t, std::initializer_list<const fss_view *>) { return false; }
inline size_t workspace_bytes(int64_t, int64_t, int64_t, int) { return 0; }
inline int64_t block_rows(int, int64_t, int64_t, int64_t) { return 64; }
template <typename T> inline int forward(const fss_scan_ctx *, char *, size_t, int64_t, int64_t, int64_t, const fss_view *, const fss_view *, const fss_view *, const fss_forward_state *) { return FSS_E_LAYOUT; }
template <typename T> inline int backward(const fss_scan_ctx *, char *, size_t, int64_t, int64_t, int64_t, const fss_view *, const fss_view *, const fss_view *, const fss_view *, const fss_view *, const fss_backward_state *) { return FSS_E_LAYOUT; }
}}
