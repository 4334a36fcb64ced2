// meresun_runner.cpp -- host driver of the Meresun decoder family over the C ABI (crabml_cuda.h + crabml_seqops.h).  Like the other
// runners it contains no arithmetic: it owns the weights' handles, says what a sequence holds (one latent cache per layer RUN) and
// in which order the tensor ops run.  Slots, step and greedy generation are the shared ones of seq_runner.hpp.
//
//   run:     h = group_norm(x) ; x += mixer(h) * sigmoid(W_g1 h + b1) + ff(h) * sigmoid(W_g2 h + b2) ; x += token_side(x, token)
//            (W_dkv, W_dq, W_g1, W_g2 and a dense W_up all multiply h: they are one stacked matrix and one product, cut afterwards)
//   mixer:   c_q = norm(W_dq h) ; q = W_uq c_q, rotated part turned ; row [norm(c) | turned r] of W_dkv h into the run's ring ; then
//            few rows (decoding): q folded through W_uk ; windowed softmax with a sink over the ring's rows ; result through W_uv per head
//            many rows (prompts): keys [W_uk c | r] and values W_uv c of the ring's rows as dense products ; the same attention per head
//            ; W_o
//   ff:      W_down PolyNorm(W_up h)   or   router -> top experts, weighted sum
#include <cmath>
#include <string>
#include <vector>

#include "../../../include/crabml_meresun.h"
#include "seq_runner.hpp"

using crabml::CudaTensor;
using crabml::TensorError;

namespace {

struct Layer {
    cmr_layer_config c{};
    CudaTensor norm1, h_stack, dq_norm, uq, dkv_norm, uk, uv, uk_t, uv_f32, sink, rot_freq, o, rg1_b, rg2_b, down, act, router, correction, e_gate, e_up, e_down, side_table,
        side_gate, side_proj, side_norm;
    std::vector<int32_t> widths;                         // column blocks of h_stack's product, in order
    int i_g1 = -1, i_g2 = -1, i_up = -1;                 // which block is which (blocks 0 and 1: the cache row, the query latent); -1: absent
    int64_t ring = 0;            // rows of the latent cache of one run of this layer
};
// a run of a layer: looped layers run several times with the same weights, each time on a cache of its own
struct Run {
    int layer;
    bool add_embedding;          // the first layer of a repeated pass: the embedding output joins x before it
};
struct State : crabml::SeqState {
    std::vector<CudaTensor> ring;          // per run: [rows, kv_rank + rot_dim]
};
const cc_view* opt(const CudaTensor& t, cc_view& store) {
    if (!t.valid()) return nullptr;
    store = t.view();
    return &store;
}

struct Runner : csr_runner {
    cmr_config conf{};
    std::vector<Layer> layers;
    std::vector<Run> runs;
    CudaTensor embed, final_norm, head;

    std::unique_ptr<crabml::SeqState> make_state() override {
        auto s = std::make_unique<State>();
        for (const Run& r : runs) {
            const Layer& L = layers[r.layer];
            s->ring.push_back(CudaTensor::alloc({L.ring, (int64_t)L.c.kv_rank + L.c.rot_dim}, CC_F32, dev));
        }
        return s;
    }
    // nothing to clear: a query at position i only reads rows of positions <= i of ITS sequence, all written since the slot was opened
    void reset_state(crabml::SeqState&) override {}

    CudaTensor norm(const CudaTensor& x, const CudaTensor& w, int groups) {
        CudaTensor h = CudaTensor::alloc(x.shape(), CC_F32, dev);
        cc_view hv = h.view(), xv = x.view(), wv = w.view();
        check(cc_group_rms_norm(dev, &hv, &xv, &wv, groups, conf.norm_eps));
        return h;
    }

    // ckv: the new tokens' raw cache rows W_dkv h; cq: their raw query latents W_dq h
    CudaTensor mixer(const Layer& L, CudaTensor& ring, const CudaTensor& ckv, CudaTensor cq, int64_t pos0) {
        const auto& c = L.c;
        const int64_t n = ckv.shape()[0];
        if (c.window <= 0 && pos0 + n > L.ring) throw TensorError("a sequence of " + std::to_string(pos0 + n) + " tokens does not fit the cache of " + std::to_string(L.ring));
        cc_view fq{};
        const cc_view* freq = opt(L.rot_freq, fq);
        // the cache row of every new token
        {
            cc_view rv = ring.view(), cv = ckv.view(), nw{};
            check(cc_latent_ring_append(dev, &rv, &cv, opt(L.dkv_norm, nw), conf.norm_eps, c.kv_rank, freq, c.rot_mag, pos0));
        }
        // queries through their latent
        cq = norm(cq, L.dq_norm, 1);
        CudaTensor q = L.uq.matmul_vec(cq);
        cc_view qv = q.view();
        cc_buf* b = nullptr;
        cc_view rv = ring.view(), sk{};
        CudaTensor o;
        if (n * c.heads > 64) {
            if (freq) check(cc_rope_pairs(dev, &qv, c.heads, c.dim + c.rot_dim, c.dim, freq, c.rot_mag, pos0));
            // many rows: expand the cached rows once for all queries of the pass.  The expansion keeps the ring's row order (position p in
            // row p % ring), so the attention reads it like the ring itself; rows no token has written yet are never visible.
            const int64_t rows = std::min<int64_t>(L.ring, pos0 + n);
            const int64_t cols = (int64_t)c.kv_rank + c.rot_dim;
            CudaTensor lat = CudaTensor(ring).with_strider(crabml::TensorStrider({rows, c.kv_rank}, {cols, 1})).contiguous();
            CudaTensor kp = L.uk.matmul_vec(lat), v = L.uv.matmul_vec(lat);
            cc_view kpv = kp.view(), vv = v.view();
            check(cc_head_concat_shared(dev, &kpv, &rv, c.heads, c.kv_rank, c.rot_dim, &b));
            CudaTensor keys = adopt(b, {rows, (int64_t)c.heads * (c.dim + c.rot_dim)});
            cc_view kv = keys.view();
            b = nullptr;
            check(cc_window_attention_sink(dev, &qv, nullptr, 0.0f, &kv, &vv, pos0, c.heads, c.heads, c.dim + c.rot_dim, c.vdim, c.window, c.scale, nullptr, nullptr,
                                           opt(L.sink, sk), &b));
            o = adopt(b, {n, (int64_t)c.heads * c.vdim});
        } else {
            // few rows: all heads read the one cached row per position; keys are whole rows, values their first kv_rank columns.  The
            // query's rotated part is turned while it is carried past the fold.
            cc_view ukv = L.uk_t.view();
            check(cc_head_project(dev, &qv, &ukv, c.heads, c.rot_dim, freq, c.rot_mag, pos0, &b));
            CudaTensor ql = adopt(b, {n, (int64_t)c.heads * (c.kv_rank + c.rot_dim)});
            cc_view qlv = ql.view();
            b = nullptr;
            check(cc_window_attention_sink(dev, &qlv, nullptr, 0.0f, &rv, nullptr, pos0, c.heads, 1, c.kv_rank + c.rot_dim, c.kv_rank, c.window, c.scale, nullptr, nullptr,
                                           opt(L.sink, sk), &b));
            CudaTensor ol = adopt(b, {n, (int64_t)c.heads * c.kv_rank});
            cc_view olv = ol.view(), uvv = L.uv_f32.view();
            b = nullptr;
            check(cc_head_project(dev, &olv, &uvv, c.heads, 0, nullptr, 1.0f, 0, &b));
            o = adopt(b, {n, (int64_t)c.heads * c.vdim});
        }
        return L.o.matmul_vec(o);
    }

    // z: the dense feed-forward's W_up h (unused by a routed one)
    CudaTensor feed_forward(const Layer& L, const CudaTensor& h, CudaTensor z) {
        const auto& c = L.c;
        const int64_t n = h.shape()[0];
        if (c.ff_kind == CMR_FF_DENSE) {
            cc_view zv = z.view(), av = L.act.view();
            check(cc_poly_norm(dev, &zv, &av, conf.norm_eps));
            return L.down.matmul_vec(z);
        }
        cc_view hv = h.view(), rw = L.router.view(), cv{};
        cc_buf *ids = nullptr, *wts = nullptr, *ob = nullptr;
        const cc_route_params rp = {CC_ROUTE_SIGMOID, c.top, c.groups, c.keep_groups, 2, 1, 1e-20f};
        check(cc_moe_route_ex(dev, &hv, &rw, opt(L.correction, cv), &rp, &ids, &wts));
        CudaTensor tid = adopt(ids, {n, c.top}), tw = adopt(wts, {n, c.top});
        cc_view iv = tid.view(), wv = tw.view(), g = L.e_gate.view(), u = L.e_up.view(), d = L.e_down.view();
        const cc_glu_params glu = {CC_ACT_SWISH, 1.702f, c.limit, 1.0f};
        check(cc_moe_experts_glu(dev, &hv, &iv, &wv, &g, &u, &d, c.experts, c.ff, &glu, &ob));
        return adopt(ob, {n, conf.width});
    }

    CudaTensor forward_chunk(crabml::SeqState& base, int64_t pos0, const int64_t* tokens, int64_t n, int device_slot) override {
        State& s = static_cast<State&>(base);
        auto gather = [&](const CudaTensor& table, int64_t cols) {
            CudaTensor t = CudaTensor::alloc({n, cols}, CC_F32, dev);
            if (device_slot >= 0) t.copy_rows_from_slot(table, device_slot);
            else t.copy_rows_from(table, std::vector<int64_t>(tokens, tokens + n));
            return t;
        };
        CudaTensor x = gather(embed, conf.width);
        CudaTensor x0;
        for (const Run& r : runs)
            if (r.add_embedding) { x0 = x.dup(); break; }
        for (size_t ri = 0; ri < runs.size(); ri++) {
            const Layer& L = layers[runs[ri].layer];
            if (runs[ri].add_embedding) {            // (not add_inplace: like the reference's CPU code it skips a tail of len % 4 elements)
                cc_view xv = x.view(), ev = x0.view();
                check(cc_gated_sum(dev, &xv, 1, &ev, nullptr, nullptr, nullptr, nullptr, nullptr));
            }
            {
                CudaTensor h = norm(x, L.norm1, conf.norm_groups);
                std::vector<CudaTensor> part;
                {
                    CudaTensor all = L.h_stack.matmul_vec(h);
                    cc_view av = all.view();
                    std::vector<cc_buf*> outs(L.widths.size(), nullptr);
                    check(cc_split_cols(dev, &av, (int32_t)L.widths.size(), L.widths.data(), outs.data()));
                    for (size_t p = 0; p < outs.size(); p++) part.push_back(adopt(outs[p], {n, L.widths[p]}));
                }
                CudaTensor y = mixer(L, s.ring[ri], part[0], part[1], pos0);
                CudaTensor g1, f, g2;
                if (L.i_g1 >= 0) g1 = part[L.i_g1];
                if (L.c.ff_kind != CMR_FF_NONE) {
                    f = feed_forward(L, h, L.i_up >= 0 ? part[L.i_up] : CudaTensor());
                    if (L.i_g2 >= 0) g2 = part[L.i_g2];
                }
                cc_view xv = x.view(), yv = y.view(), g1v{}, b1v{}, fv{}, g2v{}, b2v{};
                check(cc_gated_sum(dev, &xv, 1, &yv, opt(g1, g1v), opt(L.rg1_b, b1v), opt(f, fv), opt(g2, g2v), opt(L.rg2_b, b2v)));
            }
            if (L.side_table.valid()) {
                CudaTensor g = L.side_gate.matmul_vec(x);
                CudaTensor e = gather(L.side_table, conf.side_dim);
                cc_view gv = g.view(), ev = e.view();
                check(cc_glu_inplace(dev, &gv, &ev, CC_ACT_GELU_TANH));
                CudaTensor y = L.side_proj.matmul_vec(g);
                cc_view xv = x.view(), yv = y.view(), nv = L.side_norm.view();
                check(cc_rms_norm_gain(dev, &xv, &yv, &nv, conf.norm_eps, 1));
            }
            x = std::move(x).with_name("run:" + std::to_string(ri) + ":" + std::to_string(pos0));
        }
        return x;
    }

    CudaTensor logits_of(const CudaTensor& x, const std::vector<int64_t>& rows) override {
        bool all = (int64_t)rows.size() == x.shape()[0];
        for (size_t i = 0; all && i < rows.size(); i++) all = rows[i] == (int64_t)i;
        if (all) return head.matmul_vec(norm(x, final_norm, conf.norm_groups));          // every row in order (a decoded token): no copy
        CudaTensor xs = CudaTensor::alloc({(int64_t)rows.size(), conf.width}, CC_F32, dev);
        xs.copy_rows_from(x, rows);
        return head.matmul_vec(norm(xs, final_norm, conf.norm_groups));
    }
};

}  // namespace

extern "C" CC_API int cmr_runner_create(cc_device* dev, const cmr_config* conf, const cmr_layer_config* lc, const cmr_layer_weights* lw, cc_buf* embed, cc_buf* final_norm,
                                        cc_buf* head, csr_runner** out) {
    if (!dev || !conf || !lc || !lw || !embed || !final_norm || !head || !out) return CC_ERR_ARG;
    Runner* r = new Runner();
    r->dev = dev;
    r->conf = *conf;
    if (r->conf.chunk <= 0) r->conf.chunk = 256;
    if (r->conf.max_seq <= 0) r->conf.max_seq = 4096;
    r->width = conf->width; r->vocab = conf->vocab; r->chunk = r->conf.chunk;
    std::string err;
    int rc = crabml::seq_guarded(r, &err, [&] {
        const int64_t D = conf->width;
        if (conf->n_layers < 1 || D < 1 || conf->vocab < 1) throw TensorError("bad model sizes");
        if (conf->norm_groups < 1 || D % conf->norm_groups) throw TensorError("the norm's groups do not divide the width");
        r->embed = CudaTensor::wrap(dev, embed, {conf->vocab, D});
        r->final_norm = CudaTensor::wrap(dev, final_norm, {D});
        r->head = CudaTensor::wrap(dev, head, {conf->vocab, D});
        r->layers.resize(conf->n_layers);
        for (int i = 0; i < conf->n_layers; i++) {
            Layer& L = r->layers[i];
            const cmr_layer_config& c = L.c = lc[i];
            const cmr_layer_weights& w = lw[i];
            const std::string at = "layer " + std::to_string(i) + ": ";
            if (c.heads < 1 || c.dim < 1 || c.rot_dim < 0 || c.vdim < 1 || c.q_rank < 1 || c.kv_rank < 1) throw TensorError(at + "bad head counts / sizes");
            auto need = [&](cc_buf* b, const char* name, std::vector<int64_t> shape) {
                if (!b) throw TensorError(at + "tensor '" + name + "' is missing");
                return CudaTensor::wrap(dev, b, shape);
            };
            auto maybe = [&](cc_buf* b, std::vector<int64_t> shape) { return b ? CudaTensor::wrap(dev, b, shape) : CudaTensor(); };
            const int64_t qh = c.dim + c.rot_dim, hv = (int64_t)c.heads * c.vdim;
            L.norm1 = need(w.norm1, "norm1", {D});
            L.dq_norm = need(w.dq_norm, "mix.dq.norm", {c.q_rank}); L.uq = need(w.uq, "mix.uq", {c.heads * qh, c.q_rank});
            L.dkv_norm = need(w.dkv_norm, "mix.dkv.norm", {c.kv_rank});
            L.rg1_b = maybe(w.rg1_b, {D}); L.rg2_b = maybe(w.rg2_b, {D});
            if (c.ff_kind == CMR_FF_NONE && L.rg2_b.valid()) throw TensorError(at + "a gate for a feed-forward the layer does not have");
            L.widths = {c.kv_rank + c.rot_dim, c.q_rank};
            if (L.rg1_b.valid()) { L.i_g1 = (int)L.widths.size(); L.widths.push_back((int32_t)D); }
            if (L.rg2_b.valid()) { L.i_g2 = (int)L.widths.size(); L.widths.push_back((int32_t)D); }
            if (c.ff_kind == CMR_FF_DENSE) { if (c.ff < 1) throw TensorError(at + "bad feed-forward width"); L.i_up = (int)L.widths.size(); L.widths.push_back(c.ff); }
            int64_t on_h = 0;
            for (int32_t v : L.widths) on_h += v;
            L.h_stack = need(w.h_stack, "the stack of mix.dkv, mix.dq, rg1, rg2, mlp.up", {on_h, D});
            L.uk = need(w.uk, "mix.uk", {(int64_t)c.heads * c.dim, c.kv_rank}); L.uv = need(w.uv, "mix.uv", {hv, c.kv_rank});
            L.uk_t = need(w.uk_t, "mix.uk (per head transposed)", {(int64_t)c.heads * c.kv_rank, c.dim}); L.uv_f32 = need(w.uv_f32, "mix.uv (F32)", {hv, c.kv_rank});
            L.o = need(w.o, "mix.o", {D, hv});
            L.sink = maybe(w.sink, {c.heads});
            if (w.rot_freq) {
                const int64_t pairs = cc_tensor_capacity(w.rot_freq);
                if (2 * pairs > c.rot_dim) throw TensorError(at + "more rotated pairs than the rotated part holds");
                L.rot_freq = CudaTensor::wrap(dev, w.rot_freq, {pairs});
            }
            if (L.uk_t.dtype() != CC_F32 || L.uv_f32.dtype() != CC_F32) throw TensorError(at + "the folded forms of mix.uk / mix.uv must be F32: they enter the 32-bit scores and sums");
            if (c.ff_kind == CMR_FF_DENSE) {
                L.down = need(w.down, "mlp.down", {D, c.ff}); L.act = need(w.act, "mlp.act", {4});
            } else if (c.ff_kind == CMR_FF_ROUTED) {
                if (c.experts < 1 || c.top < 1 || c.top > c.experts || c.ff < 1) throw TensorError(at + "bad router sizes");
                L.router = need(w.router, "mlp.router", {c.experts, D});
                L.correction = maybe(w.correction, {c.experts});
                L.e_gate = need(w.e_gate, "mlp.e*.gate", {(int64_t)c.experts * c.ff, D});
                L.e_up = need(w.e_up, "mlp.e*.up", {(int64_t)c.experts * c.ff, D});
                L.e_down = need(w.e_down, "mlp.e*.down", {(int64_t)c.experts * D, c.ff});
            } else if (c.ff_kind != CMR_FF_NONE) throw TensorError(at + "unknown feed-forward kind");
            if (conf->side_dim > 0) {
                L.side_table = need(w.side_table, "side.embed", {conf->vocab, conf->side_dim});
                L.side_gate = need(w.side_gate, "side.gate", {conf->side_dim, D}); L.side_proj = need(w.side_proj, "side.proj", {D, conf->side_dim});
                L.side_norm = need(w.side_norm, "side.norm", {D});
            }
            // a ring holds the window's reach behind the first token of a pass, plus the pass
            L.ring = c.window > 0 ? (int64_t)c.window - 1 + r->conf.chunk : std::max<int64_t>(r->conf.max_seq, r->conf.chunk);
        }
        // the order of the runs
        const int n = conf->n_layers;
        int a = conf->loop_start, b = conf->loop_stop, times = conf->loop_times;
        if (times <= 1 || b <= a) { a = b = 0; times = 1; }
        if (a < 0 || b > n) throw TensorError("the loop does not lie inside the layers");
        for (int i = 0; i < a; i++) r->runs.push_back({i, false});
        for (int t = 0; t < times; t++)
            for (int i = a; i < b; i++) r->runs.push_back({i, t > 0 && i == a});
        for (int i = b; i < n; i++) r->runs.push_back({i, false});
        for (const Run& run : r->runs) {
            const Layer& L = r->layers[run.layer];
            r->state_bytes_per_slot += L.ring * ((int64_t)L.c.kv_rank + L.c.rot_dim) * 4;
        }
    });
    if (rc != CC_OK) {
        crabml::seq_set_create_error(err);
        delete r;
        return rc;
    }
    *out = r;
    return CC_OK;
}
