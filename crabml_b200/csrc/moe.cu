// moe.cu -- routed feed-forward of include/crabml_seqops.h: the router (32-bit softmax scores, correction for the choice only,
// group-limited top-k) and the chosen experts' gated feed-forward.
//
// Expert execution is per (token, chosen slot): the hidden row act(W_gate x) * (W_up x) of slot s lands in hid[t][s][:], and the
// down projection sums the slots IN SLOT ORDER.  A token's result therefore depends only on the token, never on which other
// tokens share the call (no atomics, no order that depends on the batch).  BF16 expert weights round the operand row to bfloat16
// (x for gate / up, the hidden row for down) and accumulate in f32, exactly like cc_matmul_vec does for BF16 matrices.
#include <cuda_bf16.h>
#include <stdlib.h>

#include "../../include/crabml_seqops.h"
#include "capi_checks.cuh"

#define MOE_ENTER(dev, what)                                                                                          \
    if (!(dev)) return CC_ERR_ARG;                                                                                    \
    CC_ENTER(dev);                                                                                                    \
    if (LAZY(dev)) return cc_fail((dev), CC_ERR_UNSUPPORTED, "%s: not available on a lazy (graph / megakernel) device", what)
#define MOE_VIEW(dev, v, what)                                                                                        \
    do {                                                                                                              \
        if (!view_ok(v)) return cc_fail((dev), CC_ERR_ARG, "%s: bad tensor view", what);                              \
        if (!view_in_bounds(v)) return cc_fail((dev), CC_ERR_TENSOR, "%s: view out of bounds", what);                 \
        CC_REQUIRE(dev, view_contiguous(v), "%s: not contiguous", what);                                              \
    } while (0)

// ---- router ---------------------------------------------------------------------------------------------------------------------------
// Shared memory per token: s[E] (softmax scores), c[E] (choice scores, -inf once taken or masked), gs[n_groups].
// Ties go to the lowest index.
__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
}
#define RT_WARPS 8
// one CTA per token: its warps share the experts' logits (a warp per expert, lanes striding D), then warp 0 does the softmax and the choice
__global__ void __launch_bounds__(RT_WARPS * 32) moe_route_kernel(const float* __restrict__ x, const float* __restrict__ wr, const float* __restrict__ corr,
                                                                  int* __restrict__ ids, float* __restrict__ wts, int T, int D, int E, int top, int n_groups, int keep,
                                                                  int renorm, int score_fn, int group_top, float renorm_eps) {
    extern __shared__ float rt_sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    float* s = rt_sm;
    float* c = s + E;
    float* gs = c + E;
    const float* xr = x + (int64_t)t * D;
    for (int e = warp; e < E; e += RT_WARPS) {
        const float* w = wr + (int64_t)e * D;
        float acc = 0.0f;
        for (int d = lane; d < D; d += 32) acc = fmaf(w[d], xr[d], acc);
        acc = warp_sum(acc);
        if (lane == 0) s[e] = acc;
    }
    __syncthreads();
    if (warp != 0) return;
    if (score_fn == CC_ROUTE_SIGMOID) {
        for (int e = lane; e < E; e += 32) { const float v = 1.0f / (1.0f + expf(-s[e])); s[e] = v; c[e] = corr ? v + corr[e] : v; }
    } else {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
        mx = warp_max(mx);
        __syncwarp();
        float sum = 0.0f;
        for (int e = lane; e < E; e += 32) { const float v = expf(s[e] - mx); s[e] = v; sum += v; }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < E; e += 32) { const float v = s[e] * inv; s[e] = v; c[e] = corr ? v + corr[e] : v; }
    }
    __syncwarp();
    if (n_groups > 1) {
        const int per = E / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            // the group's score: the sum of its group_top largest choice scores, largest first (picked in order: below the last
            // pick, or equal to it at a higher index)
            float m = 0.0f, lv = INFINITY; int li = -1;
            for (int n = 0; n < group_top; n++) {
                float bv = -INFINITY; int bi = -1;
                for (int e = 0; e < per; e++) {
                    const float v = c[g * per + e];
                    if ((v < lv || (v == lv && e > li)) && (bi < 0 || v > bv)) { bv = v; bi = e; }
                }
                if (bi < 0) break;
                m = n == 0 ? bv : m + bv; lv = bv; li = bi;
            }
            gs[g] = m;
        }
        __syncwarp();
        // take the `keep` best groups (marking a taken group +inf), then mask every expert of a group that was not taken
        for (int r = 0; r < keep; r++) {
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) { const float v = gs[g]; if (v != INFINITY && v > bv) { bv = v; bi = g; } }
            warp_argmax(bv, bi);
            if (lane == 0 && bi != 0x7fffffff) gs[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32) if (gs[e / per] != INFINITY) c[e] = -INFINITY;
        __syncwarp();
    }
    float wsum = 0.0f;
    for (int r = 0; r < top; r++) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) { const float v = c[e]; if (v > bv) { bv = v; bi = e; } }
        warp_argmax(bv, bi);
        if (bi == 0x7fffffff) bi = 0;                       // unreachable with finite scores (keep * group size >= top); never index out of range
        if (lane == 0) {
            ids[(int64_t)t * top + r] = bi;
            wts[(int64_t)t * top + r] = s[bi];
            c[bi] = -INFINITY;
        }
        wsum += s[bi];
        __syncwarp();
    }
    if (renorm && lane == 0) for (int r = 0; r < top; r++) wts[(int64_t)t * top + r] /= wsum + renorm_eps;
}
extern "C" CC_API int cc_moe_route_ex(cc_device* dev, const cc_view* x, const cc_view* router_w, const cc_view* correction, const cc_route_params* rp, cc_buf** ids_out,
                                      cc_buf** weights_out) {
    MOE_ENTER(dev, "moe_route");
    if (!rp) return cc_fail(dev, CC_ERR_ARG, "moe_route: no parameters");
    int32_t top = rp->top, n_groups = rp->n_groups, keep_groups = rp->keep_groups;
    const int32_t renormalise = rp->renormalise, group_top = rp->group_top < 1 ? 1 : rp->group_top;
    CC_REQUIRE(dev, rp->score == CC_ROUTE_SOFTMAX || rp->score == CC_ROUTE_SIGMOID, "moe_route: unknown score function %d", rp->score);
    if (!ids_out || !weights_out) return cc_fail(dev, CC_ERR_ARG, "moe_route: out is NULL");
    MOE_VIEW(dev, x, "moe_route x"); MOE_VIEW(dev, router_w, "moe_route router_w");
    REQUIRE_F32(dev, x, "moe_route x"); REQUIRE_F32(dev, router_w, "moe_route router_w");
    CC_REQUIRE(dev, x->ndim == 2 && router_w->ndim == 2 && router_w->shape[1] == x->shape[1], "moe_route: x must be [T, D] and router_w [E, D]");
    const int64_t T = x->shape[0], D = x->shape[1], E = router_w->shape[0];
    if (correction) { MOE_VIEW(dev, correction, "moe_route correction"); REQUIRE_F32(dev, correction, "moe_route correction"); CC_REQUIRE(dev, view_len(correction) == E, "moe_route: correction must have one number per expert"); }
    if (n_groups <= 1) { n_groups = 1; keep_groups = 1; }
    CC_REQUIRE(dev, top >= 1 && top <= E && E % n_groups == 0 && keep_groups >= 1 && keep_groups <= n_groups && (int64_t)keep_groups * (E / n_groups) >= top,
               "moe_route: experts=%lld top=%d groups=%d keep=%d do not fit", (long long)E, top, n_groups, keep_groups);
    cc_buf *ids = nullptr, *wts = nullptr;
    int rc = cc_new_activation(dev, T * top, CC_I32, false, &ids);
    if (rc) return rc;
    rc = cc_new_activation(dev, T * top, CC_F32, false, &wts);
    if (rc) { cc_tensor_release(ids); return rc; }
    *ids_out = ids; *weights_out = wts;
    if (T == 0) return CC_OK;
    const size_t smem = (size_t)(2 * E + (n_groups > 1 ? n_groups : 0)) * 4;
    if (smem > 200 * 1024) return cc_fail(dev, CC_ERR_UNSUPPORTED, "moe_route: %lld experts need %zu bytes of shared memory", (long long)E, smem);
    if (smem > 48 * 1024) CC_CUDA(dev, cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    moe_route_kernel<<<(unsigned)T, RT_WARPS * 32, smem, dev->stream>>>((const float*)x->buf->plane[0], (const float*)router_w->buf->plane[0],
                                                                                                     correction ? (const float*)correction->buf->plane[0] : nullptr,
                                                                                                     (int*)ids->base, (float*)wts->base, (int)T, (int)D, (int)E, top, n_groups,
                                                                                                     keep_groups, renormalise, rp->score, group_top, rp->renorm_eps);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}
extern "C" CC_API int cc_moe_route(cc_device* dev, const cc_view* x, const cc_view* router_w, const cc_view* correction, int32_t top, int32_t n_groups,
                                   int32_t keep_groups, int32_t renormalise, cc_buf** ids_out, cc_buf** weights_out) {
    const cc_route_params rp = {CC_ROUTE_SOFTMAX, top, n_groups, keep_groups, 1, renormalise, 0.0f};
    return cc_moe_route_ex(dev, x, router_w, correction, &rp, ids_out, weights_out);
}

// ---- experts ---------------------------------------------------------------------------------------------------------------------------
// an id outside [0, E) (only possible with a caller-made table) is clamped, never used as an address
__device__ __forceinline__ int moe_clamp(int e, int E) { return e < 0 ? 0 : e >= E ? E - 1 : e; }
__device__ __forceinline__ float moe_w(const float* w, int64_t i) { return w[i]; }
__device__ __forceinline__ float moe_w(const uint16_t* w, int64_t i) { return __uint_as_float((unsigned)w[i] << 16); }
template <class WT> __device__ __forceinline__ float moe_round(float v);
template <> __device__ __forceinline__ float moe_round<float>(float v) { return v; }
template <> __device__ __forceinline__ float moe_round<uint16_t>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float moe_act(float z, int act, float alpha) {
    return act == CC_ACT_SILU ? z / (1.0f + expf(-z)) : act == CC_ACT_GELU_TANH ? 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)))
         : act == CC_ACT_SWISH ? z / (1.0f + expf(-(alpha * z))) : z;
}
// the gated unit: act(min(g, limit)) * (clamp(u, -limit, limit) + up_shift); limit <= 0 clamps nothing
__device__ __forceinline__ float moe_glu(float g, float u, const cc_glu_params P) {
    if (P.limit > 0.0f) { g = fminf(g, P.limit); u = fminf(fmaxf(u, -P.limit), P.limit); }
    return moe_act(g, P.act, P.alpha) * (u + P.up_shift);
}

// grid (T * top, ceil(ff / 8)), 256 threads: the CTA stages x[t] (rounded for BF16 weights); a warp owns one hidden row of the slot's expert
template <class WT>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(const float* __restrict__ x, const int* __restrict__ ids, const WT* __restrict__ wg, const WT* __restrict__ wu,
                                                          float* __restrict__ hid, int D, int ff, int top, cc_glu_params act, int E) {
    extern __shared__ float mg_sm[];
    const int ts = blockIdx.x, t = ts / top;
    const int e = moe_clamp(ids[ts], E);
    for (int d = threadIdx.x; d < D; d += 256) mg_sm[d] = moe_round<WT>(x[(int64_t)t * D + d]);
    __syncthreads();
    const int r = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= ff) return;
    const int64_t base = ((int64_t)e * ff + r) * D;
    float g = 0.0f, u = 0.0f;
    for (int d = lane; d < D; d += 32) { const float xv = mg_sm[d]; g = fmaf(moe_w(wg, base + d), xv, g); u = fmaf(moe_w(wu, base + d), xv, u); }
    g = warp_sum(g); u = warp_sum(u);
    if (lane == 0) hid[(int64_t)ts * ff + r] = moe_glu(g, u, act);
}
// grid (T, ceil(D / 8)), 256 threads: the CTA stages the token's top hidden rows; a warp owns one output coordinate and adds the slots in order
template <class WT>
__global__ void __launch_bounds__(256) moe_down_kernel(const float* __restrict__ hid, const int* __restrict__ ids, const float* __restrict__ wts, const WT* __restrict__ wd,
                                                       float* __restrict__ out, int D, int ff, int top, int E) {
    extern __shared__ float md_sm[];
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < top * ff; i += 256) md_sm[i] = moe_round<WT>(hid[(int64_t)t * top * ff + i]);
    __syncthreads();
    const int d = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (d >= D) return;
    float acc = 0.0f;
    for (int s = 0; s < top; s++) {
        const int e = moe_clamp(ids[(int64_t)t * top + s], E);
        const int64_t base = ((int64_t)e * D + d) * ff;
        float p = 0.0f;
        for (int f = lane; f < ff; f += 32) p = fmaf(moe_w(wd, base + f), md_sm[s * ff + f], p);
        p = warp_sum(p);
        acc = fmaf(wts[(int64_t)t * top + s], p, acc);
    }
    if (lane == 0) out[(int64_t)t * D + d] = acc;
}

template <class WT>
static int moe_launch(cc_device* dev, const float* x, const int* ids, const float* wts, const void* wg, const void* wu, const void* wd, float* hid, float* out, int64_t T,
                      int D, int ff, int top, cc_glu_params act, int E) {
    const size_t s1 = (size_t)D * 4, s2 = (size_t)top * ff * 4;
    if (s1 > 200 * 1024 || s2 > 200 * 1024) return cc_fail(dev, CC_ERR_UNSUPPORTED, "moe_experts: row does not fit shared memory");
    if (s1 > 48 * 1024) CC_CUDA(dev, cudaFuncSetAttribute(moe_gate_up_kernel<WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s1));
    if (s2 > 48 * 1024) CC_CUDA(dev, cudaFuncSetAttribute(moe_down_kernel<WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s2));
    moe_gate_up_kernel<WT><<<dim3((unsigned)(T * top), (unsigned)((ff + 7) / 8)), 256, s1, dev->stream>>>(x, ids, (const WT*)wg, (const WT*)wu, hid, D, ff, top, act, E);
    CC_LAUNCH_CHECK(dev);
    moe_down_kernel<WT><<<dim3((unsigned)T, (unsigned)((D + 7) / 8)), 256, s2, dev->stream>>>(hid, ids, wts, (const WT*)wd, out, D, ff, top, E);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}

// ---- grouped path (BF16 weights, many rows): the (token, slot) rows are sorted by expert and every expert's rows run through the
// tensor-core pipeline of prefill_gemm.cu in ONE grouped launch per projection.  A row's products and the order of its k sum do not
// depend on its neighbours in the tile, and the slots are combined in slot order, so a token's result is still independent of the batch.
bool cc_grouped_bf16_supported(int64_t m, int64_t k);
int cc_launch_grouped_bf16(cc_device* dev, const cc_buf* w_stack, int64_t n_groups, int64_t m, int64_t k, const void* x_bf16, int64_t n_rows, const int* groups_dev,
                           int max_tiles, int block_n, float* out);

// one CTA: counts per expert (shared-memory atomics), exclusive offsets, the tile table {n_tiles | expert, first row, rows, 0 ...}, and
// pos[i] = sorted row of entry i = (token, slot).  The order of the rows INSIDE an expert is arbitrary; no value depends on it.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ ids, int n, int E, int block_n, int* __restrict__ pos, int* __restrict__ table) {
    extern __shared__ int ms_sm[];            // counts[E], offsets[E]
    int* cnt = ms_sm;
    int* off = ms_sm + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) pos[i] = atomicAdd(&cnt[moe_clamp(ids[i], E)], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, nt = 0;
        for (int e = 0; e < E; e++) {
            off[e] = o;
            for (int r = 0; r < cnt[e]; r += block_n) {
                int* t = table + 4 + 4 * nt++;
                t[0] = e; t[1] = o + r; t[2] = min(block_n, cnt[e] - r); t[3] = 0;
            }
            o += cnt[e];
        }
        table[0] = nt;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) pos[i] += off[moe_clamp(ids[i], E)];
}
// xs[pos[i]][:] = bf16(x[i / top][:]) ; one warp per entry
__global__ void moe_gather_bf16_kernel(const float* __restrict__ x, const int* __restrict__ pos, __nv_bfloat16* __restrict__ xs, int n, int top, int D) {
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= n) return;
    const float* src = x + (int64_t)(i / top) * D;
    __nv_bfloat16* dst = xs + (int64_t)pos[i] * D;
    for (int d = lane * 2; d < D; d += 64) *(__nv_bfloat162*)(dst + d) = __floats2bfloat162_rn(src[d], src[d + 1]);
}
__global__ void moe_glu_bf16_kernel(const float* __restrict__ g, const float* __restrict__ u, __nv_bfloat16* __restrict__ h, int64_t n, cc_glu_params act) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i >= n) return;
    *(__nv_bfloat162*)(h + i) = __floats2bfloat162_rn(moe_glu(g[i], u[i], act), moe_glu(g[i + 1], u[i + 1], act));
}
// out[t][d] = sum over the slots, in slot order, of weights[t][s] * y[pos[t * top + s]][d]
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos, const float* __restrict__ wts, float* __restrict__ out, int64_t T, int top, int D) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * D) return;
    const int64_t t = i / D; const int d = (int)(i % D);
    float acc = 0.0f;
    for (int s = 0; s < top; s++) acc = fmaf(wts[t * top + s], y[(int64_t)pos[t * top + s] * D + d], acc);
    out[i] = acc;
}

static int moe_grouped(cc_device* dev, const float* x, const int* ids, const float* wts, const cc_buf* wg, const cc_buf* wu, const cc_buf* wd, float* out, int64_t T, int D,
                       int ff, int top, int E, cc_glu_params act) {
    const int64_t n = T * top;
    const int block_n = n / E >= 96 ? 128 : 64;
    const int max_tiles = (int)((n + block_n - 1) / block_n) + E;
    // one pool block: pos[n] | table[4 + 4 * max_tiles] | xs bf16 [n][D] | g f32 [n][ff] | u f32 [n][ff] | h bf16 [n][ff] | y f32 [n][D]
    auto al = [](size_t v) { return (v + 255) & ~(size_t)255; };
    const size_t o_pos = 0, o_tab = al((size_t)n * 4), o_xs = o_tab + al((size_t)(4 + 4 * max_tiles) * 4), o_g = o_xs + al((size_t)n * D * 2), o_u = o_g + al((size_t)n * ff * 4),
                 o_h = o_u + al((size_t)n * ff * 4), o_y = o_h + al((size_t)n * ff * 2), total = o_y + al((size_t)n * D * 4);
    uint8_t* base = nullptr; size_t cls = 0;
    int rc = cc_pool_alloc(dev, total, (void**)&base, &cls);
    if (rc) return rc;
    int* pos = (int*)(base + o_pos); int* table = (int*)(base + o_tab);
    __nv_bfloat16* xs = (__nv_bfloat16*)(base + o_xs); float* g = (float*)(base + o_g); float* u = (float*)(base + o_u);
    __nv_bfloat16* h = (__nv_bfloat16*)(base + o_h); float* y = (float*)(base + o_y);
    moe_sort_kernel<<<1, 1024, (size_t)2 * E * 4, dev->stream>>>(ids, (int)n, E, block_n, pos, table);
    dev->launches++;
    moe_gather_bf16_kernel<<<(unsigned)((n + 7) / 8), 256, 0, dev->stream>>>(x, pos, xs, (int)n, top, D);
    dev->launches++;
    rc = cc_launch_grouped_bf16(dev, wg, E, ff, D, xs, n, table, max_tiles, block_n, g);
    if (!rc) rc = cc_launch_grouped_bf16(dev, wu, E, ff, D, xs, n, table, max_tiles, block_n, u);
    if (!rc) {
        moe_glu_bf16_kernel<<<(unsigned)((n * ff / 2 + 255) / 256), 256, 0, dev->stream>>>(g, u, h, n * ff, act);
        dev->launches++;
        rc = cc_launch_grouped_bf16(dev, wd, E, D, ff, h, n, table, max_tiles, block_n, y);
    }
    if (!rc) {
        moe_combine_kernel<<<(unsigned)((T * D + 255) / 256), 256, 0, dev->stream>>>(y, pos, wts, out, T, top, D);
        CC_LAUNCH_CHECK(dev);
    }
    cc_pool_free(dev, base, cls);
    return rc;
}

extern "C" CC_API int cc_moe_experts_glu(cc_device* dev, const cc_view* x, const cc_view* ids, const cc_view* weights, const cc_view* w_gate, const cc_view* w_up,
                                         const cc_view* w_down, int32_t n_experts, int32_t ff, const cc_glu_params* glu, cc_buf** out) {
    MOE_ENTER(dev, "moe_experts");
    if (!glu) return cc_fail(dev, CC_ERR_ARG, "moe_experts: no gated-unit parameters");
    const cc_glu_params act = *glu;
    if (!out) return cc_fail(dev, CC_ERR_ARG, "moe_experts: out is NULL");
    MOE_VIEW(dev, x, "moe_experts x"); MOE_VIEW(dev, ids, "moe_experts ids"); MOE_VIEW(dev, weights, "moe_experts weights");
    MOE_VIEW(dev, w_gate, "moe_experts w_gate"); MOE_VIEW(dev, w_up, "moe_experts w_up"); MOE_VIEW(dev, w_down, "moe_experts w_down");
    REQUIRE_F32(dev, x, "moe_experts x"); REQUIRE_F32(dev, weights, "moe_experts weights");
    CC_REQUIRE(dev, ids->buf->dtype == CC_I32, "moe_experts: ids must be I32");
    CC_REQUIRE(dev, x->ndim == 2 && ids->ndim == 2 && ids->shape[0] == x->shape[0] && view_len(weights) == view_len(ids), "moe_experts: x must be [T, D], ids and weights [T, top]");
    const int64_t T = x->shape[0], D = x->shape[1], top = ids->shape[1];
    const int wt = w_gate->buf->dtype;
    CC_REQUIRE(dev, (wt == CC_F32 || wt == CC_BF16) && w_up->buf->dtype == wt && w_down->buf->dtype == wt, "moe_experts: expert weights must all be F32 or all BF16");
    CC_REQUIRE(dev, n_experts > 0 && ff > 0 && view_len(w_gate) == (int64_t)n_experts * ff * D && view_len(w_up) == (int64_t)n_experts * ff * D &&
                        view_len(w_down) == (int64_t)n_experts * D * ff,
               "moe_experts: weight stacks do not fit experts=%d ff=%d D=%lld", n_experts, ff, (long long)D);
    cc_buf* o = nullptr;
    int rc = cc_new_activation(dev, T * D, CC_F32, false, &o);
    if (rc) return rc;
    *out = o;
    if (T == 0) return CC_OK;
    static const int grouped_min_rows = getenv("CRABML_MOE_GROUPED_MIN") ? atoi(getenv("CRABML_MOE_GROUPED_MIN")) : 128;
    if (wt == CC_BF16 && T * top >= grouped_min_rows && n_experts <= 4096 && D % 2 == 0 && ff % 2 == 0 && cc_grouped_bf16_supported(ff, D) && cc_grouped_bf16_supported(D, ff) &&
        ((uintptr_t)w_gate->buf->plane[0] & 15) == 0 && ((uintptr_t)w_up->buf->plane[0] & 15) == 0 && ((uintptr_t)w_down->buf->plane[0] & 15) == 0)
        return moe_grouped(dev, (const float*)x->buf->plane[0], (const int*)ids->buf->plane[0], (const float*)weights->buf->plane[0], w_gate->buf, w_up->buf, w_down->buf,
                           (float*)o->base, T, (int)D, ff, (int)top, n_experts, act);
    void* hid = nullptr; size_t cls = 0;
    rc = cc_pool_alloc(dev, (size_t)T * top * ff * 4, &hid, &cls);
    if (rc) return rc;
    const float* xp = (const float*)x->buf->plane[0];
    const int* ip = (const int*)ids->buf->plane[0];
    const float* wp = (const float*)weights->buf->plane[0];
    if (wt == CC_F32) rc = moe_launch<float>(dev, xp, ip, wp, w_gate->buf->plane[0], w_up->buf->plane[0], w_down->buf->plane[0], (float*)hid, (float*)o->base, T, (int)D, ff, (int)top, act, n_experts);
    else rc = moe_launch<uint16_t>(dev, xp, ip, wp, w_gate->buf->plane[0], w_up->buf->plane[0], w_down->buf->plane[0], (float*)hid, (float*)o->base, T, (int)D, ff, (int)top, act, n_experts);
    cc_pool_free(dev, hid, cls);
    return rc;
}
extern "C" CC_API int cc_moe_experts(cc_device* dev, const cc_view* x, const cc_view* ids, const cc_view* weights, const cc_view* w_gate, const cc_view* w_up,
                                     const cc_view* w_down, int32_t n_experts, int32_t ff, int32_t act, cc_buf** out) {
    const cc_glu_params glu = {act, 1.0f, 0.0f, 0.0f};
    return cc_moe_experts_glu(dev, x, ids, weights, w_gate, w_up, w_down, n_experts, ff, &glu, out);
}
