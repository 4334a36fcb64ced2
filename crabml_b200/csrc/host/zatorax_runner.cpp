// zatorax_runner.cpp -- host driver of the Zatorax decoder family over the C ABI (crabml_cuda.h + crabml_seqops.h).
// Like llama2_runner.cpp this file contains no arithmetic: it owns the weights' handles, the per-sequence state slots, and the
// order of the tensor ops.
//
//   layer:   x += norm1(mixer(x)) ;  x += norm2(ff(x))          (norm on the sublayer OUTPUT, one-number gain, 32-bit residual)
//   delta:   q,k,v = silu(conv(W x)) ; q,k unit vectors per head (q also * dk^-1/2) ; gated delta rule ; per-head RMS norm * weight
//            * silu(W_g x) ; W_o
//   attention: q,k RMS-normed per head ; keys/values into the layer's ring (or read from the ring of layer kv_from) ; windowed
//            softmax with the logarithmic distance penalty ; W_o
//   ff:      router -> top experts (+ shared expert), weighted sum
#include <algorithm>
#include <cmath>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "../../../include/crabml_zatorax.h"
#include "seq_runner.hpp"

using crabml::CudaTensor;
using crabml::TensorError;

namespace {

struct Layer {
    czr_layer_config c{};
    CudaTensor norm1, norm2, q, k, v, o, q_conv, k_conv, v_conv, b, a, a_log, dt_bias, out_norm, g, q_norm, k_norm, r1, r2, router, correction, e_gate, e_up, e_down,
        s_gate, s_up, s_down;
    int64_t ring = 0;            // attention layers with keys of their own: rows of the key/value rings
};

// per-sequence, per-layer state.  attention (own keys): kring / vring.  delta: S and the three convolution tails.
struct LayerState {
    CudaTensor kring, vring, S, tq, tk, tv;
};
struct State : crabml::SeqState {
    std::vector<LayerState> layers;
};

cc_view view_of(const CudaTensor& t) { return t.view(); }
const cc_view* opt(const CudaTensor& t, cc_view& store) {
    if (!t.valid()) return nullptr;
    store = t.view();
    return &store;
}

}  // namespace

// the sequence slots, the step function and greedy generation are the shared ones of seq_runner.hpp
struct czr_runner_impl : csr_runner {
    czr_config conf{};
    std::vector<Layer> layers;
    CudaTensor embed, final_norm, head;

    std::unique_ptr<crabml::SeqState> make_state() override;
    void reset_state(crabml::SeqState& s) override;
    CudaTensor forward_chunk(crabml::SeqState& s, int64_t pos0, const int64_t* tokens, int64_t n, int device_slot) override;
    CudaTensor logits_of(const CudaTensor& x, const std::vector<int64_t>& rows) override;
    CudaTensor delta_mixer(const Layer& L, LayerState& st, const CudaTensor& x);
    CudaTensor attention_mixer(int li, State& s, const CudaTensor& x, int64_t pos0);
    CudaTensor feed_forward(const Layer& L, const CudaTensor& x);
};

std::unique_ptr<crabml::SeqState> czr_runner_impl::make_state() {
    auto sp = std::make_unique<State>();
    State& s = *sp;
    s.layers.resize(layers.size());
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer& L = layers[i];
        LayerState& st = s.layers[i];
        const auto& c = L.c;
        if (c.mixer == CZR_MIXER_ATTENTION) {
            if (c.kv_from < 0) {
                st.kring = CudaTensor::alloc({L.ring, (int64_t)c.kv_heads * c.dim}, CC_F32, dev);
                st.vring = CudaTensor::alloc({L.ring, (int64_t)c.kv_heads * c.vdim}, CC_F32, dev);
            }
        } else {
            st.S = CudaTensor::alloc({c.heads, c.dim, c.vdim}, CC_F32, dev);
            if (c.conv > 1) {
                st.tq = CudaTensor::alloc({c.conv - 1, (int64_t)c.kv_heads * c.dim}, CC_F32, dev);
                st.tk = CudaTensor::alloc({c.conv - 1, (int64_t)c.kv_heads * c.dim}, CC_F32, dev);
                st.tv = CudaTensor::alloc({c.conv - 1, (int64_t)c.heads * c.vdim}, CC_F32, dev);
            }
        }
    }
    return sp;
}

// a reused slot starts like a new one: the recurrence and the convolutions see zeros before position 0.  The rings need no reset:
// a query at position i only reads rows of positions 0..i of ITS sequence, all written since the slot was opened.
void czr_runner_impl::reset_state(crabml::SeqState& base) {
    for (auto& st : static_cast<State&>(base).layers)
        for (CudaTensor* t : {&st.S, &st.tq, &st.tk, &st.tv})
            if (t->valid()) { cc_view v = t->view(); check(cc_tensor_zero(dev, &v)); }
}

CudaTensor czr_runner_impl::delta_mixer(const Layer& L, LayerState& st, const CudaTensor& x) {
    const auto& c = L.c;
    const int64_t n = x.shape()[0];
    auto conv = [&](const CudaTensor& w, const CudaTensor& cw, CudaTensor& tail, int hs, bool unit, float scale) {
        CudaTensor p = w.matmul_vec(x);
        cc_view pv = p.view(), wv = cw.view(), tv{};
        const cc_view* tp = opt(tail, tv);
        cc_buf* out = nullptr;
        check(cc_short_conv(dev, &pv, &wv, tp, CC_ACT_SILU, hs, unit ? 1 : 0, 1e-6f, scale, &out));
        return adopt(out, {n, p.shape()[1]});
    };
    CudaTensor q = conv(L.q, L.q_conv, st.tq, c.dim, true, 1.0f / std::sqrt((float)c.dim));
    CudaTensor k = conv(L.k, L.k_conv, st.tk, c.dim, true, 1.0f);
    CudaTensor v = conv(L.v, L.v_conv, st.tv, c.vdim, false, 1.0f);
    CudaTensor a = L.a.matmul_vec(x), b = L.b.matmul_vec(x), gate = L.g.matmul_vec(x);
    cc_view qv = q.view(), kv = k.view(), vv = v.view(), av = a.view(), bv = b.view(), alv = L.a_log.view(), dtv = L.dt_bias.view(), sv = st.S.view();
    cc_buf* ob = nullptr;
    check(cc_gated_delta_rule(dev, &qv, &kv, &vv, &av, &bv, &alv, &dtv, &sv, c.heads, c.kv_heads, c.dim, c.vdim, &ob));
    CudaTensor o = adopt(ob, {n, (int64_t)c.heads * c.vdim});
    cc_view ov = o.view(), gv = gate.view(), nv = L.out_norm.view();
    check(cc_gated_head_rms_norm(dev, &ov, &gv, &nv, c.vdim, conf.norm_eps, CC_ACT_SILU));
    return L.o.matmul_vec(o);
}

CudaTensor czr_runner_impl::attention_mixer(int li, State& s, const CudaTensor& x, int64_t pos0) {
    const Layer& L = layers[li];
    const auto& c = L.c;
    const int64_t n = x.shape()[0];
    const int src = c.kv_from >= 0 ? c.kv_from : li;
    LayerState& kvst = s.layers[src];
    if (c.kv_from < 0) {
        CudaTensor k = L.k.matmul_vec(x), v = L.v.matmul_vec(x);
        cc_view kr = kvst.kring.view(), vr = kvst.vring.view(), kv = k.view(), vv = v.view(), nw{};
        check(cc_kv_ring_append(dev, &kr, &vr, &kv, &vv, opt(L.k_norm, nw), conf.norm_eps, pos0, c.kv_heads, c.dim, c.vdim));
    }
    CudaTensor q = L.q.matmul_vec(x);
    cc_view qv = q.view(), kr = kvst.kring.view(), vr = kvst.vring.view(), qn{}, r1{}, r2{};
    cc_buf* ob = nullptr;
    check(cc_window_attention(dev, &qv, opt(L.q_norm, qn), conf.norm_eps, &kr, &vr, pos0, c.heads, c.kv_heads, c.dim, c.vdim, c.window, c.scale, opt(L.r1, r1),
                              opt(L.r2, r2), &ob));
    CudaTensor o = adopt(ob, {n, (int64_t)c.heads * c.vdim});
    return L.o.matmul_vec(o);
}

CudaTensor czr_runner_impl::feed_forward(const Layer& L, const CudaTensor& x) {
    const auto& c = L.c;
    const int64_t n = x.shape()[0];
    cc_view xv = x.view(), rw = L.router.view(), cv{};
    cc_buf *ids = nullptr, *wts = nullptr, *ob = nullptr;
    check(cc_moe_route(dev, &xv, &rw, opt(L.correction, cv), c.top, c.groups, c.keep_groups, 0, &ids, &wts));
    CudaTensor tid = adopt(ids, {n, c.top}), tw = adopt(wts, {n, c.top});
    cc_view iv = tid.view(), wv = tw.view(), g = L.e_gate.view(), u = L.e_up.view(), d = L.e_down.view();
    check(cc_moe_experts(dev, &xv, &iv, &wv, &g, &u, &d, c.experts, c.expert_ff, CC_ACT_SILU, &ob));
    CudaTensor y = adopt(ob, {n, conf.width});
    if (c.shared_ff > 0) {
        CudaTensor h1 = L.s_gate.matmul_vec(x), h2 = L.s_up.matmul_vec(x);
        cc_view h1v = h1.view(), h2v = h2.view();
        check(cc_glu_inplace(dev, &h1v, &h2v, CC_ACT_SILU));
        CudaTensor sh = L.s_down.matmul_vec(h1);
        cc_view yv = y.view(), sv = sh.view();      // (not add_inplace: like the reference's CPU code it skips a tail of len % 4 elements)
        check(cc_gated_sum(dev, &yv, 1, &sv, nullptr, nullptr, nullptr, nullptr, nullptr));
    }
    return y;
}

// one pass over n <= chunk tokens at positions s.len .. ; returns the residual stream [n, width] after the last layer
CudaTensor czr_runner_impl::forward_chunk(crabml::SeqState& base, int64_t pos0, const int64_t* tokens, int64_t n, int device_slot) {
    State& s = static_cast<State&>(base);
    CudaTensor x = CudaTensor::alloc({n, conf.width}, CC_F32, dev);
    if (device_slot >= 0) x.copy_rows_from_slot(embed, device_slot);
    else x.copy_rows_from(embed, std::vector<int64_t>(tokens, tokens + n));
    for (size_t li = 0; li < layers.size(); li++) {
        const Layer& L = layers[li];
        {
            CudaTensor y = L.c.mixer == CZR_MIXER_DELTA ? delta_mixer(L, s.layers[li], x) : attention_mixer((int)li, s, x, pos0);
            cc_view xv = x.view(), yv = y.view(), gv = L.norm1.view();
            check(cc_rms_norm_gain(dev, &xv, &yv, &gv, conf.norm_eps, 1));
        }
        if (L.c.has_mlp) {
            CudaTensor y = feed_forward(L, x);
            cc_view xv = x.view(), yv = y.view(), gv = L.norm2.view();
            check(cc_rms_norm_gain(dev, &xv, &yv, &gv, conf.norm_eps, 1));
        }
        x = std::move(x).with_name("layer:" + std::to_string(li) + ":" + std::to_string(pos0));
    }
    return x;
}

CudaTensor czr_runner_impl::logits_of(const CudaTensor& x, const std::vector<int64_t>& rows) {
    const int64_t nw = (int64_t)rows.size();
    CudaTensor xs = CudaTensor::alloc({nw, conf.width}, CC_F32, dev);
    xs.copy_rows_from(x, rows);
    CudaTensor xn = CudaTensor::alloc({nw, conf.width}, CC_F32, dev);
    cc_view dv = xn.view(), sv = xs.view(), gv = final_norm.view();
    check(cc_rms_norm_gain(dev, &dv, &sv, &gv, conf.norm_eps, 0));
    return head.matmul_vec(xn);
}

extern "C" CC_API int czr_runner_create(cc_device* dev, const czr_config* conf, const czr_layer_config* lc, const czr_layer_weights* lw, cc_buf* embed, cc_buf* final_norm,
                                        cc_buf* head, czr_runner** out) {
    if (!dev || !conf || !lc || !lw || !embed || !final_norm || !head || !out) return CC_ERR_ARG;
    czr_runner_impl* r = new czr_runner_impl();
    r->dev = dev;
    r->conf = *conf;
    if (r->conf.chunk <= 0) r->conf.chunk = 256;
    r->width = conf->width; r->vocab = conf->vocab; r->chunk = r->conf.chunk;
    std::string err;
    int rc = crabml::seq_guarded(r, &err, [&] {
        const int64_t D = conf->width;
        if (conf->n_layers < 1 || D < 1 || conf->vocab < 1) throw TensorError("bad model sizes");
        r->embed = CudaTensor::wrap(dev, embed, {conf->vocab, D});
        r->final_norm = CudaTensor::wrap(dev, final_norm, {1});
        r->head = CudaTensor::wrap(dev, head, {conf->vocab, D});
        r->layers.resize(conf->n_layers);
        for (int i = 0; i < conf->n_layers; i++) {
            Layer& L = r->layers[i];
            const czr_layer_config& c = L.c = lc[i];
            const czr_layer_weights& w = lw[i];
            const std::string at = "layer " + std::to_string(i) + ": ";
            if (c.heads < 1 || c.kv_heads < 1 || c.heads % c.kv_heads || c.dim < 1 || c.vdim < 1) throw TensorError(at + "bad head counts / sizes");
            auto need = [&](cc_buf* b, const char* name, std::vector<int64_t> shape) {
                if (!b) throw TensorError(at + "tensor '" + name + "' is missing");
                return CudaTensor::wrap(dev, b, shape);
            };
            L.norm1 = need(w.norm1, "norm1", {1});
            const int64_t qk = (int64_t)c.kv_heads * c.dim, hv = (int64_t)c.heads * c.vdim;
            if (c.mixer == CZR_MIXER_DELTA) {
                if (c.conv < 1) throw TensorError(at + "the convolution needs at least one tap");
                L.q = need(w.q, "mix.q", {qk, D}); L.k = need(w.k, "mix.k", {qk, D}); L.v = need(w.v, "mix.v", {hv, D});
                L.q_conv = need(w.q_conv, "mix.q.conv", {qk, c.conv}); L.k_conv = need(w.k_conv, "mix.k.conv", {qk, c.conv}); L.v_conv = need(w.v_conv, "mix.v.conv", {hv, c.conv});
                L.b = need(w.b, "mix.b", {c.heads, D}); L.a = need(w.a, "mix.a", {c.heads, D});
                L.a_log = need(w.a_log, "mix.A_log", {c.heads}); L.dt_bias = need(w.dt_bias, "mix.dt_bias", {c.heads});
                L.out_norm = need(w.out_norm, "mix.norm", {c.vdim}); L.g = need(w.g, "mix.g", {hv, D}); L.o = need(w.o, "mix.o", {D, hv});
            } else if (c.mixer == CZR_MIXER_ATTENTION) {
                L.q = need(w.q, "mix.q", {(int64_t)c.heads * c.dim, D});
                L.q_norm = need(w.q_norm, "mix.q.norm", {c.dim});
                L.r1 = need(w.r1, "mix.r1", {c.heads}); L.r2 = need(w.r2, "mix.r2", {c.heads});
                L.o = need(w.o, "mix.o", {D, hv});
                if (c.kv_from < 0) {
                    L.k = need(w.k, "mix.k", {qk, D}); L.v = need(w.v, "mix.v", {(int64_t)c.kv_heads * c.vdim, D});
                    L.k_norm = need(w.k_norm, "mix.k.norm", {c.dim});
                } else {
                    if (c.kv_from >= i) throw TensorError(at + "kv_from must name an earlier layer");
                    const czr_layer_config& s = lc[c.kv_from];
                    if (s.mixer != CZR_MIXER_ATTENTION || s.kv_from >= 0) throw TensorError(at + "kv_from must name an attention layer with keys of its own");
                    if (s.kv_heads != c.kv_heads || s.dim != c.dim || s.vdim != c.vdim) throw TensorError(at + "kv_from: key/value head counts and sizes differ");
                }
                if (c.window < 1) throw TensorError(at + "the window must be at least 1");
            } else throw TensorError(at + "unknown mixer");
            if (c.has_mlp) {
                L.norm2 = need(w.norm2, "norm2", {1});
                if (c.experts < 1 || c.top < 1 || c.top > c.experts || c.expert_ff < 1) throw TensorError(at + "bad router sizes");
                L.router = need(w.router, "mlp.router", {c.experts, D});
                if (w.correction) L.correction = CudaTensor::wrap(dev, w.correction, {c.experts});
                L.e_gate = need(w.e_gate, "mlp.e*.gate", {(int64_t)c.experts * c.expert_ff, D});
                L.e_up = need(w.e_up, "mlp.e*.up", {(int64_t)c.experts * c.expert_ff, D});
                L.e_down = need(w.e_down, "mlp.e*.down", {(int64_t)c.experts * D, c.expert_ff});
                if (c.shared_ff > 0) {
                    L.s_gate = need(w.s_gate, "mlp.shared.gate", {c.shared_ff, D}); L.s_up = need(w.s_up, "mlp.shared.up", {c.shared_ff, D});
                    L.s_down = need(w.s_down, "mlp.shared.down", {D, c.shared_ff});
                }
            }
        }
        // a ring must hold the widest window of any layer that reads it, plus the longest pass
        for (int i = 0; i < conf->n_layers; i++) {
            const czr_layer_config& c = r->layers[i].c;
            if (c.mixer != CZR_MIXER_ATTENTION) continue;
            Layer& src = r->layers[c.kv_from >= 0 ? c.kv_from : i];
            src.ring = std::max<int64_t>(src.ring, (int64_t)c.window - 1 + r->conf.chunk);
        }
        for (auto& L : r->layers) {
            const auto& c = L.c;
            if (c.mixer == CZR_MIXER_ATTENTION) r->state_bytes_per_slot += c.kv_from < 0 ? L.ring * c.kv_heads * (int64_t)(c.dim + c.vdim) * 4 : 0;
            else r->state_bytes_per_slot += ((int64_t)c.heads * c.dim * c.vdim + (int64_t)(c.conv - 1) * (2 * c.kv_heads * c.dim + c.heads * c.vdim)) * 4;
        }
    });
    if (rc != CC_OK) {
        crabml::seq_set_create_error(err);       // readable after the half-built runner is gone (csr_last_create_error)
        delete r;
        return rc;
    }
    *out = r;
    return CC_OK;
}

// the family's older names of the shared entry points
extern "C" CC_API const char* czr_last_create_error(void) { return csr_last_create_error(); }
extern "C" CC_API void czr_runner_destroy(czr_runner* r) { csr_runner_destroy(r); }
extern "C" CC_API const char* czr_runner_last_error(czr_runner* r) { return csr_runner_last_error(r); }
extern "C" CC_API int czr_seq_open(czr_runner* r, int32_t* slot_out) { return csr_seq_open(r, slot_out); }
extern "C" CC_API int czr_seq_close(czr_runner* r, int32_t slot) { return csr_seq_close(r, slot); }
extern "C" CC_API int64_t czr_seq_len(czr_runner* r, int32_t slot) { return csr_seq_len(r, slot); }
extern "C" CC_API int czr_runner_stats(czr_runner* r, int64_t* out3) { return csr_runner_stats(r, out3); }
extern "C" CC_API int czr_runner_step(czr_runner* r, int32_t slot, const int64_t* tokens, int32_t n_tokens, const int32_t* want, int32_t n_want, float* logits_out) {
    return csr_runner_step(r, slot, tokens, n_tokens, want, n_want, logits_out);
}
extern "C" CC_API int czr_runner_generate_greedy(czr_runner* r, int32_t slot, const int64_t* prompt, int32_t n_prompt, int32_t steps, int64_t eos, int64_t* out_tokens,
                                                 int32_t* n_out) {
    return csr_runner_generate_greedy(r, slot, prompt, n_prompt, steps, eos, out_tokens, n_out);
}
