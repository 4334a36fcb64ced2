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
#include "cuda_tensor.hpp"

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
struct Slot {
    std::vector<LayerState> layers;
    int64_t len = 0;
    bool live = false;
};

cc_view view_of(const CudaTensor& t) { return t.view(); }
const cc_view* opt(const CudaTensor& t, cc_view& store) {
    if (!t.valid()) return nullptr;
    store = t.view();
    return &store;
}

}  // namespace

struct czr_runner {
    cc_device* dev = nullptr;
    czr_config conf{};
    std::vector<Layer> layers;
    CudaTensor embed, final_norm, head;
    std::vector<Slot> slots;
    int64_t state_bytes_per_slot = 0;
    std::string last_error;

    void check(int rc) { CudaTensor::check(dev, rc); }
    CudaTensor adopt(cc_buf* b, std::vector<int64_t> shape) { return CudaTensor(dev, b, crabml::TensorStrider(std::move(shape))); }

    void make_slot(Slot& s);
    void reset_slot(Slot& s);
    CudaTensor delta_mixer(const Layer& L, LayerState& st, const CudaTensor& x);
    CudaTensor attention_mixer(int li, Slot& s, const CudaTensor& x, int64_t pos0);
    CudaTensor feed_forward(const Layer& L, const CudaTensor& x);
    CudaTensor forward_chunk(Slot& s, const int64_t* tokens, int64_t n, int device_slot);
    CudaTensor logits_of(const CudaTensor& x, const std::vector<int64_t>& rows);
    void step(int32_t slot, const int64_t* tokens, int32_t n, const int32_t* want, int32_t n_want, float* out);
    Slot& slot_ref(int32_t slot) {
        if (slot < 0 || slot >= (int32_t)slots.size() || !slots[slot].live) throw TensorError("sequence slot " + std::to_string(slot) + " is not open");
        return slots[slot];
    }
};

void czr_runner::make_slot(Slot& s) {
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
}

// a reused slot starts like a new one: the recurrence and the convolutions see zeros before position 0.  The rings need no reset:
// a query at position i only reads rows of positions 0..i of ITS sequence, all written since the slot was opened.
void czr_runner::reset_slot(Slot& s) {
    for (auto& st : s.layers)
        for (CudaTensor* t : {&st.S, &st.tq, &st.tk, &st.tv})
            if (t->valid()) { cc_view v = t->view(); check(cc_tensor_zero(dev, &v)); }
    s.len = 0;
}

CudaTensor czr_runner::delta_mixer(const Layer& L, LayerState& st, const CudaTensor& x) {
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

CudaTensor czr_runner::attention_mixer(int li, Slot& s, const CudaTensor& x, int64_t pos0) {
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

CudaTensor czr_runner::feed_forward(const Layer& L, const CudaTensor& x) {
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
        y = std::move(y).add_inplace(sh);
    }
    return y;
}

// one pass over n <= chunk tokens at positions s.len .. ; returns the residual stream [n, width] after the last layer
CudaTensor czr_runner::forward_chunk(Slot& s, const int64_t* tokens, int64_t n, int device_slot) {
    const int64_t pos0 = s.len;
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
    s.len += n;
    return x;
}

CudaTensor czr_runner::logits_of(const CudaTensor& x, const std::vector<int64_t>& rows) {
    const int64_t nw = (int64_t)rows.size();
    CudaTensor xs = CudaTensor::alloc({nw, conf.width}, CC_F32, dev);
    xs.copy_rows_from(x, rows);
    CudaTensor xn = CudaTensor::alloc({nw, conf.width}, CC_F32, dev);
    cc_view dv = xn.view(), sv = xs.view(), gv = final_norm.view();
    check(cc_rms_norm_gain(dev, &dv, &sv, &gv, conf.norm_eps, 0));
    return head.matmul_vec(xn);
}

void czr_runner::step(int32_t slot, const int64_t* tokens, int32_t n, const int32_t* want, int32_t n_want, float* out) {
    Slot& s = slot_ref(slot);
    for (int i = 0; i < n; i++)
        if (tokens[i] < 0 || tokens[i] >= conf.vocab) throw TensorError("token id " + std::to_string(tokens[i]) + " is outside the vocabulary");
    for (int i = 0; i < n_want; i++)
        if (want[i] < 0 || want[i] >= n || (i > 0 && want[i] <= want[i - 1])) throw TensorError("wanted positions must be ascending indices into the step's tokens");
    int wi = 0;
    for (int64_t c0 = 0; c0 < n; c0 += conf.chunk) {
        const int64_t cn = std::min<int64_t>(conf.chunk, n - c0);
        CudaTensor x = forward_chunk(s, tokens + c0, cn, -1);
        std::vector<int64_t> rows;
        while (wi + (int)rows.size() < n_want && want[wi + rows.size()] < c0 + cn) rows.push_back(want[wi + rows.size()] - c0);
        if (!rows.empty()) {
            CudaTensor lg = logits_of(x, rows);
            lg.export_to(out + (size_t)wi * conf.vocab, rows.size() * (size_t)conf.vocab);
            wi += (int)rows.size();
        }
    }
}

static thread_local std::string g_create_error;

template <class F>
static int guarded(czr_runner* r, F&& f) {
    try {
        f();
        return CC_OK;
    } catch (const TensorError& e) {
        if (r) r->last_error = e.what();
        return CC_ERR_TENSOR;
    } catch (const std::exception& e) {
        if (r) r->last_error = e.what();
        return CC_ERR_ARG;
    }
}

extern "C" CC_API int czr_runner_create(cc_device* dev, const czr_config* conf, const czr_layer_config* lc, const czr_layer_weights* lw, cc_buf* embed, cc_buf* final_norm,
                                        cc_buf* head, czr_runner** out) {
    if (!dev || !conf || !lc || !lw || !embed || !final_norm || !head || !out) return CC_ERR_ARG;
    czr_runner* r = new czr_runner();
    r->dev = dev;
    r->conf = *conf;
    if (r->conf.chunk <= 0) r->conf.chunk = 256;
    int rc = guarded(r, [&] {
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
        g_create_error = r->last_error;          // readable after the half-built runner is gone (czr_last_create_error)
        delete r;
        return rc;
    }
    *out = r;
    return CC_OK;
}

extern "C" CC_API const char* czr_last_create_error(void) { return g_create_error.c_str(); }
extern "C" CC_API void czr_runner_destroy(czr_runner* r) { delete r; }
extern "C" CC_API const char* czr_runner_last_error(czr_runner* r) { return r ? r->last_error.c_str() : ""; }

extern "C" CC_API int czr_seq_open(czr_runner* r, int32_t* slot_out) {
    if (!r || !slot_out) return CC_ERR_ARG;
    return guarded(r, [&] {
        int found = -1;
        for (size_t i = 0; i < r->slots.size(); i++)
            if (!r->slots[i].live) { found = (int)i; break; }            // lowest free slot first: closed slots are reused before new ones are made
        if (found < 0) {
            r->slots.emplace_back();
            found = (int)r->slots.size() - 1;
            r->make_slot(r->slots[found]);
        }
        r->reset_slot(r->slots[found]);
        r->slots[found].live = true;
        *slot_out = found;
    });
}
extern "C" CC_API int czr_seq_close(czr_runner* r, int32_t slot) {
    if (!r) return CC_ERR_ARG;
    return guarded(r, [&] { r->slot_ref(slot).live = false; });
}
extern "C" CC_API int64_t czr_seq_len(czr_runner* r, int32_t slot) {
    if (!r || slot < 0 || slot >= (int32_t)r->slots.size() || !r->slots[slot].live) return -1;
    return r->slots[slot].len;
}
extern "C" CC_API int czr_runner_stats(czr_runner* r, int64_t* out3) {
    if (!r || !out3) return CC_ERR_ARG;
    out3[0] = (int64_t)r->slots.size();
    out3[1] = 0;
    for (auto& s : r->slots) out3[1] += s.live;
    out3[2] = r->state_bytes_per_slot;
    return CC_OK;
}

extern "C" CC_API int czr_runner_step(czr_runner* r, int32_t slot, const int64_t* tokens, int32_t n_tokens, const int32_t* want, int32_t n_want, float* logits_out) {
    if (!r || !tokens || n_tokens < 1 || n_want < 0 || (n_want > 0 && (!want || !logits_out))) return CC_ERR_ARG;
    return guarded(r, [&] { r->step(slot, tokens, n_tokens, want, n_want, logits_out); });
}

extern "C" CC_API int czr_runner_generate_greedy(czr_runner* r, int32_t slot, const int64_t* prompt, int32_t n_prompt, int32_t steps, int64_t eos, int64_t* out_tokens,
                                                 int32_t* n_out) {
    if (!r || !prompt || n_prompt < 1 || steps < 1 || !out_tokens || !n_out) return CC_ERR_ARG;
    *n_out = 0;
    return guarded(r, [&] {
        Slot& s = r->slot_ref(slot);
        for (int i = 0; i < n_prompt; i++)
            if (prompt[i] < 0 || prompt[i] >= r->conf.vocab) throw TensorError("token id outside the vocabulary");
        CudaTensor x;
        int64_t last_n = 0;
        for (int64_t c0 = 0; c0 < n_prompt; c0 += r->conf.chunk) {
            last_n = std::min<int64_t>(r->conf.chunk, n_prompt - c0);
            x = r->forward_chunk(s, prompt + c0, last_n, -1);
        }
        r->logits_of(x, {last_n - 1}).reshape({r->conf.vocab}).argmax_to_slot(0, 0);
        int64_t done = 1;
        if (eos >= 0) r->check(cc_read_history(r->dev, 0, 1, out_tokens));
        for (; done < steps; done++) {
            if (eos >= 0 && out_tokens[done - 1] == eos) break;
            x = r->forward_chunk(s, nullptr, 1, 0);
            r->logits_of(x, {0}).reshape({r->conf.vocab}).argmax_to_slot(0, done);
            if (eos >= 0) r->check(cc_read_history(r->dev, done, 1, out_tokens + done));
        }
        if (eos < 0) r->check(cc_read_history(r->dev, 0, done, out_tokens));
        *n_out = (int32_t)done;
    });
}
