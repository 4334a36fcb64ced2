// capi_checks.cuh -- argument checks shared by the extern "C" entry points (capi.cu, seqops.cu, moe.cu).
#pragma once
#include "common.cuh"

// ---- strider helpers (tensor/strider.rs) ------------------------------------------------------------------
[[maybe_unused]] static int64_t view_len(const cc_view* v) {
    int64_t n = 1;
    for (int i = 0; i < v->ndim; i++) n *= v->shape[i];
    return n;
}
[[maybe_unused]] static bool view_contiguous(const cc_view* v) {                      // strider.rs:182-206
    if (v->ndim == 0) return true;
    if (v->strides[v->ndim - 1] != 1) return false;
    int64_t last = 1;
    for (int i = v->ndim - 1; i >= 0; i--) {
        if (last != v->strides[i]) return false;
        last *= v->shape[i];
    }
    return true;
}
[[maybe_unused]] static bool view_ok(const cc_view* v) { return v && v->buf && v->ndim >= 1 && v->ndim <= CC_MAX_DIMS; }
// highest element offset the view addresses (-1 for an empty view); negative strides / shapes are rejected by the caller
[[maybe_unused]] static int64_t view_max_offset(const cc_view* v) {
    int64_t off = 0;
    for (int i = 0; i < v->ndim; i++) {
        if (v->shape[i] <= 0) return -1;
        off += (v->shape[i] - 1) * v->strides[i];
    }
    return off;
}
[[maybe_unused]] static bool view_in_bounds(const cc_view* v) {
    for (int i = 0; i < v->ndim; i++) if (v->shape[i] < 0 || v->strides[i] < 0) return false;
    return view_max_offset(v) < v->buf->nelems;
}

// argument checks shared by every op: a usable view whose highest addressed element lies inside its buffer (the strider lives on
// the host side of the ABI, so a stale or mismatched shape must become a TensorError here, not an out-of-bounds device read)
#define CHECK_VIEW(dev, v, what)                                                         \
    if (!(dev)) return CC_ERR_ARG;                                                       \
    CC_ENTER(dev);                                                                       \
    if (!view_ok(v)) return cc_fail((dev), CC_ERR_ARG, "%s: bad tensor view", what);     \
    if (!view_in_bounds(v)) return cc_fail((dev), CC_ERR_TENSOR, "%s: view addresses element %lld of a buffer of %lld", what, \
                                           (long long)view_max_offset(v), (long long)(v)->buf->nelems)
// a quantized weight matrix is laid out in planes that depend on its row length: the view must be the matrix itself (or a prefix
// of its rows), never a reshape
#define CHECK_QUANT_MATRIX(dev, v, what)                                                                                       \
    if (cc_is_quant((v)->buf->dtype))                                                                                          \
        CC_REQUIRE(dev, (v)->ndim == 2 && (v)->shape[1] == (v)->buf->cols && (v)->shape[0] <= (v)->buf->rows,                  \
                   "%s: view [%lld, %lld] does not match the quantized matrix [%lld, %lld]", what, (long long)(v)->shape[0],   \
                   (long long)((v)->ndim == 2 ? (v)->shape[1] : 0), (long long)(v)->buf->rows, (long long)(v)->buf->cols)
// lazy mode (lazy.cu): after the same argument checks as eager mode the op is queued instead of launched
enum { L_COPY_ROWS, L_DUP, L_RMS_NORM, L_MUL, L_ADD, L_SCALE, L_MATVEC, L_ROPE, L_CONCAT, L_CONTIGUOUS, L_BMM, L_SOFTMAX, L_SILU, L_GELU, L_ALLREDUCE, L_ALLGATHER, L_ARGMAX };
int cc_lazy_record(cc_device* dev, int kind, const cc_view* a, const cc_view* b, cc_buf* out, float f, int64_t i0, int64_t i1, int64_t i2,
                   const int64_t* rows, int n_rows);
#define LAZY(dev) ((dev)->lz != nullptr && !(dev)->exact)
#define FLUSH(dev)                                  \
    do {                                            \
        if (LAZY(dev)) { int _rc = cc_lazy_flush(dev); if (_rc) return _rc; } \
    } while (0)

#define REQUIRE_F32(dev, v, what) CC_REQUIRE(dev, (v)->buf->dtype == CC_F32, "%s: not f32, but got type %d", what, (v)->buf->dtype)

