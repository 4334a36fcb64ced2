"""The mechanisms the Meresun family added to include/crabml_seqops.h, each alone, against its function in the plain reference
(tests/meresun_ref.py).  Where random inputs would hide a fault (a window's edge, a far key, a sink, a masked group) the inputs are
made so that it shows."""
import numpy as np
import pytest

from crabml_b200 import capi, rotary, seqops
from tests import meresun_ref as R
from tests.gpu_common import make_device
from tests.meresun_common import rot

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    d = make_device()
    yield d
    d.close()


def T32(dev, a, shape=None):
    from crabml_b200 import CudaTensor
    a = np.asarray(a, np.float32)
    return CudaTensor.new(a, list(shape if shape is not None else a.shape), dev)


def W(dev, a, dtype):
    from crabml_b200 import CudaTensor
    from crabml_b200.safetensors import f32_to_bf16
    a = np.ascontiguousarray(a, np.float32)
    if dtype == capi.BF16:
        return CudaTensor.from_cpu(f32_to_bf16(a).reshape(a.shape), list(a.shape), capi.BF16, dev)
    return CudaTensor.from_cpu(a, list(a.shape), capi.F32, dev)


def bf16(a):
    from crabml_b200.safetensors import bf16_to_f32, f32_to_bf16
    return bf16_to_f32(f32_to_bf16(np.asarray(a, np.float32))).reshape(np.shape(a))


@pytest.mark.parametrize("rows,cols,groups", [(1, 12, 1), (5, 36, 3), (9, 200, 2), (3, 7, 7), (70, 96, 4)])
def test_group_rms_norm(dev, rows, cols, groups):
    rng = np.random.default_rng(cols)
    x = rng.standard_normal((rows, cols)) * 3; w = rng.standard_normal(cols)
    got = seqops.group_rms_norm(T32(dev, x), T32(dev, w), groups, 1e-5).export().reshape(rows, cols)
    assert np.abs(got - R.group_rms_norm(x, w, groups, 1e-5)).max() < 1e-5


def test_split_cols(dev):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((13, 30)).astype(np.float32)
    for widths in ([30], [1, 29], [7, 3, 11, 9], [4, 4, 4, 4, 4, 4, 3, 3]):
        parts = seqops.split_cols(T32(dev, x), widths)
        at = 0
        for p, wd in zip(parts, widths):
            assert np.array_equal(p.export().reshape(13, wd), x[:, at:at + wd])
            at += wd
    with pytest.raises(capi.TensorError):
        seqops.split_cols(T32(dev, x), [10, 10])


@pytest.mark.parametrize("cols", [1, 7, 320, 1000])
def test_poly_norm(dev, cols):
    rng = np.random.default_rng(cols)
    z = rng.standard_normal((6, cols)) * 2; coef = np.array([0.7, -0.3, 0.2, 0.05])
    got = seqops.poly_norm(T32(dev, z), T32(dev, coef), 1e-5).export().reshape(6, cols)
    want = R.poly_norm(z.astype(np.float32).astype(np.float64), coef.astype(np.float32).astype(np.float64), 1e-5)
    assert np.abs(got - want).max() < 2e-5 * max(1.0, np.abs(want).max())


def test_gated_sum_every_combination(dev):
    rng = np.random.default_rng(3)
    x0, y1, g1, y2, g2 = (rng.standard_normal((7, 10)) for _ in range(5))
    b1, b2 = rng.standard_normal(10), rng.standard_normal(10)
    cases = [(dict(g1=g1, b1=b1, y2=y2, g2=g2, b2=b2), y1 * R.sigmoid(g1 + b1) + y2 * R.sigmoid(g2 + b2)),
             (dict(g1=g1), y1 * R.sigmoid(g1)), (dict(), y1), (dict(y2=y2), y1 + y2), (dict(g1=g1, b1=b1, y2=y2), y1 * R.sigmoid(g1 + b1) + y2)]
    for kw, want in cases:
        for acc in (True, False):
            dst = T32(dev, x0)
            seqops.gated_sum(dst, T32(dev, y1), accumulate=acc, **{k: T32(dev, v) for k, v in kw.items()})
            assert np.abs(dst.export().reshape(7, 10) - (x0 + want if acc else want)).max() < 1e-5, (sorted(kw), acc)
    with pytest.raises(capi.TensorError):
        seqops.gated_sum(T32(dev, x0), T32(dev, y1), b1=T32(dev, b1))                   # a bias without its gate


@pytest.mark.parametrize("r,pos0", [(rot(8), 0), (rot(8), 4093), (rot(6, scaling=None), 17), (rot(2, base=50.0), 300)])
def test_rope_pairs_rotates_only_its_columns(dev, r, pos0):
    rng = np.random.default_rng(pos0)
    T, H, off, tail = 9, 3, 5, 2
    hs = off + r["dims"] + tail
    x = rng.standard_normal((T, H, hs))
    f, mag = rotary.table_of(r)
    got = seqops.rope_pairs(T32(dev, x.reshape(T, -1)), H, hs, off, T32(dev, f), mag, pos0).export().reshape(T, H, hs)
    want = x.copy()
    want[..., off:off + r["dims"]] = R.rotate_pairs(x[..., off:off + r["dims"]], pos0 + np.arange(T), *R.rotary_frequencies(r))
    # the angle is a 32-bit product: its rounding grows with the position
    assert np.abs(got - want).max() < 1e-5 + 4e-7 * (pos0 + T) * np.abs(x).max()
    assert np.array_equal(got[..., :off], x[..., :off].astype(np.float32)) and np.array_equal(got[..., off + r["dims"]:], x[..., off + r["dims"]:].astype(np.float32))


def test_latent_ring_append_norms_rotates_and_wraps(dev):
    from crabml_b200 import CudaTensor
    rng = np.random.default_rng(5)
    rank, rd, ring_rows, T = 11, 6, 7, 19
    r = rot(rd)
    f, mag = rotary.table_of(r)
    ckv = rng.standard_normal((T, rank + rd)) * 2; nw = rng.standard_normal(rank)
    want = np.concatenate([R.rms_norm(ckv[:, :rank], nw, 1e-5), R.rotate_pairs(ckv[:, rank:], np.arange(T), *R.rotary_frequencies(r))], 1)
    ring = CudaTensor.alloc([ring_rows, rank + rd], capi.F32, dev)
    at = 0
    for n in (3, 1, 2, 7, 6):                        # portions that cross the ring's end
        seqops.latent_ring_append(ring, T32(dev, ckv[at:at + n]), T32(dev, nw), 1e-5, rank, T32(dev, f), mag, at)
        at += n
        got = ring.export().reshape(ring_rows, -1)
        for p in range(max(0, at - ring_rows), at):
            assert np.abs(got[p % ring_rows] - want[p]).max() < 1e-5, (at, p)
    with pytest.raises(capi.TensorError):
        seqops.latent_ring_append(ring, T32(dev, ckv[:8]), T32(dev, nw), 1e-5, rank, T32(dev, f), mag, 0)     # more rows than the ring holds


@pytest.mark.parametrize("T,H,n_in,rest,n_out", [(1, 3, 8, 4, 20), (9, 2, 12, 6, 14), (70, 4, 4, 2, 11), (17, 1, 32, 0, 64), (8, 5, 130, 2, 3), (3, 2, 600, 64, 5)])
def test_head_project(dev, T, H, n_in, rest, n_out):
    rng = np.random.default_rng(T * 10 + H)
    x = rng.standard_normal((T, H, n_in + rest)); w = rng.standard_normal((H * n_out, n_in)) / 3
    got = seqops.head_project(T32(dev, x.reshape(T, -1)), T32(dev, w), H, rest).export().reshape(T, H, n_out + rest)
    want = np.concatenate([np.einsum("thd,hnd->thn", x[..., :n_in], w.reshape(H, n_out, n_in)), x[..., n_in:]], -1)
    assert np.abs(got - want).max() < 3e-5


def test_head_project_rotates_carried_columns(dev):
    rng = np.random.default_rng(9)
    T, H, n_in, rest, n_out, pos0 = 11, 3, 6, 7, 5, 123
    r = rot(4)
    f, mag = rotary.table_of(r)
    x = rng.standard_normal((T, H, n_in + rest)); w = rng.standard_normal((H * n_out, n_in))
    got = seqops.head_project(T32(dev, x.reshape(T, -1)), T32(dev, w), H, rest, T32(dev, f), mag, pos0).export().reshape(T, H, n_out + rest)
    want = np.concatenate([np.einsum("thd,hnd->thn", x[..., :n_in], w.reshape(H, n_out, n_in)),
                           R.rotate_pairs(x[..., n_in:n_in + 4], pos0 + np.arange(T), *R.rotary_frequencies(r)), x[..., n_in + 4:]], -1)
    assert np.abs(got - want).max() < 3e-5


def test_head_concat_shared(dev):
    rng = np.random.default_rng(8)
    a = rng.standard_normal((11, 3, 5)); shared = rng.standard_normal((14, 9))
    got = seqops.head_concat_shared(T32(dev, a.reshape(11, -1)), T32(dev, shared), 3, 4, 3).export().reshape(11, 3, 8)
    want = np.concatenate([a, np.repeat(shared[:11, None, 4:7], 3, 1)], -1)
    assert np.array_equal(got, want.astype(np.float32))


# ---- the whole mixer out of the ops, against the reference's one function ----------------------------------------------------------------
def mixer_weights(rng, D, H, dn, dr, dv, qr, kr, sink_scale=1.0):
    def m(o, i):
        return bf16(rng.standard_normal((o, i)) / np.sqrt(i))
    return {"m.dq": m(qr, D), "m.dq.norm": 1 + 0.1 * rng.standard_normal(qr), "m.uq": m(H * (dn + dr), qr), "m.dkv": m(kr + dr, D), "m.dkv.norm": 1 + 0.1 * rng.standard_normal(kr),
            "m.uk": m(H * dn, kr), "m.uv": m(H * dv, kr), "m.o": m(D, H * dv), "m.sink": rng.standard_normal(H) * sink_scale}


class Mixer:
    """the op chain of one latent-attention layer on one sequence, fed in portions (what the runner's mixer does)"""

    def __init__(self, dev, w, m, ring_rows, eps=1e-5, expand_over=64):
        from crabml_b200 import CudaTensor
        self.dev, self.m, self.eps, self.at, self.expand_over, self.rows = dev, m, eps, 0, expand_over, ring_rows
        self.w = {k: T32(dev, v) for k, v in w.items()}
        uk = np.asarray(w["m.uk"], np.float32).reshape(m["heads"], m["dim"], m["kv_rank"])
        self.w["m.uk_t"] = T32(dev, np.ascontiguousarray(uk.transpose(0, 2, 1)).reshape(-1, m["dim"]))
        f, self.mag = rotary.table_of(m["rot"])
        self.f = T32(dev, f)
        self.ring = CudaTensor.alloc([ring_rows, m["kv_rank"] + m["rot_dim"]], capi.F32, dev)

    def feed(self, h):
        m, w, n = self.m, self.w, h.shape[0]
        H, dn, dr, dv, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        hd = T32(self.dev, h)
        seqops.latent_ring_append(self.ring, w["m.dkv"].matmul_vec(hd), w["m.dkv.norm"], self.eps, kr, self.f, self.mag, self.at)
        cq = seqops.group_rms_norm(w["m.dq"].matmul_vec(hd), w["m.dq.norm"], 1, self.eps)
        q = w["m.uq"].matmul_vec(cq)
        if n * H > self.expand_over:              # many rows: per-head keys and values of the ring's rows, then attention per head
            from crabml_b200 import TensorStrider
            q = seqops.rope_pairs(q, H, dn + dr, dn, self.f, self.mag, self.at)
            rows = min(self.rows, self.at + n)
            lat = self.ring.with_strider(TensorStrider([rows, kr], [kr + dr, 1])).contiguous()
            keys = seqops.head_concat_shared(w["m.uk"].matmul_vec(lat), self.ring, H, kr, dr)
            o = seqops.window_attention_sink(q, keys, w["m.uv"].matmul_vec(lat), self.at, H, H, dn + dr, dv, m["mask"]["size"], m["scale"], sink=w.get("m.sink"))
        else:                                     # few rows: the up-projections folded into the query and applied to the result
            ql = seqops.head_project(q, w["m.uk_t"], H, dr, self.f, self.mag, self.at)     # the rotated part is turned on the way
            ol = seqops.window_attention_sink(ql, self.ring, None, self.at, H, 1, kr + dr, kr, m["mask"]["size"], m["scale"], sink=w.get("m.sink"))
            o = seqops.head_project(ol, w["m.uv"], H, 0)
        out = w["m.o"].matmul_vec(o).export().reshape(n, -1)
        self.at += n
        return out


@pytest.mark.parametrize("H,dn,dr,dv,qr,kr,window", [(3, 8, 4, 10, 12, 20, 7), (1, 16, 2, 5, 6, 9, 1), (8, 24, 12, 40, 48, 80, 37), (6, 4, 8, 3, 10, 33, 200), (64, 2, 2, 2, 8, 6, 5), (16, 4, 4, 40, 8, 36, 50), (4, 6, 2, 70, 8, 12, 3)])
def test_latent_attention_whole_and_in_portions(dev, H, dn, dr, dv, qr, kr, window):
    rng = np.random.default_rng(H * 7 + window)
    D, T = 24, 61
    m = {"heads": H, "dim": dn, "rot_dim": dr, "vdim": dv, "q_rank": qr, "kv_rank": kr, "mask": {"size": window}, "scale": 1.0 / np.sqrt(dn + dr), "rot": rot(dr)}
    w = mixer_weights(rng, D, H, dn, dr, dv, qr, kr)
    h = rng.standard_normal((T, D))
    want = R.latent_attention(h.astype(np.float32).astype(np.float64), w, "m.", m, 1e-5)
    for expand_over in (64, 0, 10 ** 9):              # the runner's rule, every pass expanded, every pass folded
        for portions in ([T], [1] * T, [29] + [1] * 32, [2, 3, 30, 2, 17, 1, 1, 5], [2] * 30 + [1]):
            mx = Mixer(dev, w, m, window - 1 + max(portions), expand_over=expand_over)      # the smallest ring that holds the window behind the longest portion
            got = np.concatenate([mx.feed(h[a:a + n]) for a, n in zip(np.cumsum([0] + portions[:-1]), portions)])
            assert np.abs(got - want).max() < 3e-5 * max(1.0, np.abs(want).max()), (expand_over, portions)


def _crafted(dev, window, T, j_star, sink=-1e30, ring_rows=None, portions=None, expand_over=8):
    """One head; every query and the key at j_star point the same way in the rotation-free part, strongly, so that whoever sees
    j_star returns (nearly) its value and nobody else does.  -> output [T, dv] with value coordinate 0 = 1 only at j_star."""
    H, dn, dr, dv, qr, kr, D = 1, 4, 2, 3, 4, 4, 8
    m = {"heads": H, "dim": dn, "rot_dim": dr, "vdim": dv, "q_rank": qr, "kv_rank": kr, "mask": {"size": window}, "scale": 1.0, "rot": rot(dr, scaling=None)}
    w = {"m.dq": np.eye(qr, D), "m.dq.norm": np.ones(qr), "m.uq": np.zeros((dn + dr, qr)), "m.dkv": np.eye(kr + dr, D), "m.dkv.norm": np.ones(kr),
         "m.uk": np.zeros((dn, kr)), "m.uv": np.zeros((dv, kr)), "m.o": np.eye(D, dv), "m.sink": np.array([sink])}
    w["m.uq"][0, 0] = 30.0                    # q_plain[0] = 30 * c_q[0]
    w["m.uk"][0, 1] = 1.0                     # k_plain[0] = c[1]
    w["m.uv"][0, 1] = 1.0                     # v[0] = c[1]
    w["m.uv"][1, 0] = 1.0
    h = np.zeros((T, D)); h[:, 0] = 1.0       # c = normed (1, 0, 0, 0) = (2, 0, 0, 0): k_plain = 0, v = (0, 2, 0)
    h[j_star, :2] = (0.0, 1.0)                # at j_star c = (0, 2, 0, 0): k_plain[0] = 2 -> score 30 * 2 * 2 = 120 for every query with c_q[0] = 2
    portions = portions or [T]
    mx = Mixer(dev, w, m, ring_rows or window - 1 + max(portions), expand_over=expand_over)
    got = np.concatenate([mx.feed(h[a:a + n]) for a, n in zip(np.cumsum([0] + portions[:-1]), portions)])
    want = R.latent_attention(h, w, "m.", m, 1e-5)
    assert np.abs(got - want).max() < 1e-4
    return got[:, :dv]


@pytest.mark.parametrize("portions", [None, [20] + [1] * 30, [2] * 25, [7, 1, 19, 23]])
def test_window_edge_shows_in_and_out(dev, portions):
    window, T, j = 9, 50, 21
    out = _crafted(dev, window, T, j, portions=portions)
    for i in range(T):
        if i == j:
            continue                          # the query at j_star itself has c_q[0] = 0: all its scores are 0
        seen = 0 <= i - j < window
        assert (out[i, 0] > 1.99) == seen and (out[i, 1] < 0.01) == seen, (i, out[i])
    assert out[j + window - 1, 0] > 1.99 and out[j + window, 0] < 1e-6        # the last position that sees it, the first that does not


def test_far_key_among_hundreds_prompt_and_decoded(dev):
    window, T, j = 400, 520, 70
    for portions in (None, [440] + [1] * 80, [256, 200, 64]):
        out = _crafted(dev, window, T, j, portions=portions)
        assert out[j + 399, 0] > 1.99 and out[j + 400, 0] < 1e-6 and out[j + 1, 0] > 1.99 and out[j - 1, 0] < 1e-6


def test_sink_takes_its_share_once_and_unscaled(dev):
    # no key stands out (j_star's own query row is the only special one): every visible key scores 0; n visible keys and a sink of
    # ln(3) give each key the weight 1 / (n + 3)
    window, T = 4, 9
    H, dn, dr, dv, kr, D = 1, 2, 2, 2, 2, 4
    m = {"heads": H, "dim": dn, "rot_dim": dr, "vdim": dv, "q_rank": 2, "kv_rank": kr, "mask": {"size": window}, "scale": 57.0, "rot": rot(dr)}
    w = {"m.dq": np.eye(2, D), "m.dq.norm": np.ones(2), "m.uq": np.zeros((dn + dr, 2)), "m.dkv": np.eye(kr + dr, D), "m.dkv.norm": np.ones(kr),
         "m.uk": np.eye(dn, kr), "m.uv": np.eye(dv, kr), "m.o": np.eye(D, dv), "m.sink": np.array([np.log(3.0)])}
    h = np.zeros((T, D)); h[:, 0] = 1.0
    mx = Mixer(dev, w, m, window - 1 + T)
    out = mx.feed(h)
    c0 = 1.0 / np.sqrt(0.5 + 1e-5)                         # the normed latent's first coordinate, which is also the value's
    for i in range(T):
        n = min(i + 1, window)
        assert abs(out[i, 0] - c0 * n / (n + 3.0)) < 1e-5, i
    # a sink far below every score changes nothing; one far above takes everything
    for sink, frac in ((-1e30, 1.0), (80.0, 0.0)):
        w["m.sink"] = np.array([sink])
        out = Mixer(dev, w, m, window - 1 + T).feed(h)
        assert np.abs(out[:, 0] - c0 * frac).max() < 1e-5


# ---- routed feed-forward ----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,top,groups,keep", [(8, 2, 4, 2), (6, 2, 3, 2), (4, 4, 1, 1), (16, 5, 4, 2), (12, 1, 6, 1), (9, 3, 3, 3), (64, 6, 8, 3)])
def test_sigmoid_router_against_reference(dev, E, top, groups, keep):
    rng = np.random.default_rng(E + top)
    T, D = 40, 24
    x = rng.standard_normal((T, D)); wr = rng.standard_normal((E, D)) / 2
    corr = rng.standard_normal(E) * 0.3 - 1.5            # most choice scores are negative: a masked expert must count as -inf, not as 0
    ids, wts = seqops.moe_route_ex(T32(dev, x), T32(dev, wr), T32(dev, corr), top, groups, keep, score=capi.ROUTE_SIGMOID, group_top=2, renormalise=True, renorm_eps=1e-20)
    x32, w32, c32 = (np.asarray(a, np.float32).astype(np.float64) for a in (x, wr, corr))
    rid, rw = R.route(x32, w32, c32, top, groups, keep)
    gid = ids.export().view(np.int32).reshape(T, top)                  # I32 tensors are exported bit for bit
    got_w = wts.export().reshape(T, top)
    assert np.array_equal(gid, rid)
    assert np.abs(got_w - rw).max() < 1e-5 and np.abs(got_w.sum(-1) - 1).max() < 1e-5


@pytest.mark.parametrize("dtype", [capi.F32, capi.BF16])
@pytest.mark.parametrize("T,D,E,ff,top", [(3, 24, 4, 10, 2), (1, 64, 8, 64, 3), (200, 64, 4, 64, 2), (150, 128, 6, 128, 1)])
def test_clamped_experts_weighted_sum(dev, dtype, T, D, E, ff, top):
    from crabml_b200 import CudaTensor
    rng = np.random.default_rng(T + D)
    limit = 0.8
    x = rng.standard_normal((T, D)) * 1.5                 # wide enough that gate and up hit the clamp often
    wg, wu, wd = (bf16(rng.standard_normal(s) / np.sqrt(s[-1])) for s in ((E, ff, D), (E, ff, D), (E, D, ff)))
    ids = np.stack([rng.permutation(E)[:top] for _ in range(T)]).astype(np.int32)
    wts = rng.uniform(0.1, 1.0, (T, top))
    tid = CudaTensor.from_cpu(ids, [T, top], capi.I32, dev)
    got = seqops.moe_experts_glu(T32(dev, x), tid, T32(dev, wts), W(dev, wg.reshape(E * ff, D), dtype), W(dev, wu.reshape(E * ff, D), dtype), W(dev, wd.reshape(E * D, ff), dtype),
                                 E, ff, act=capi.ACT_SWISH, alpha=1.702, limit=limit, up_shift=1.0).export().reshape(T, D)
    xin = bf16(x) if dtype == capi.BF16 else x.astype(np.float32)
    want = np.zeros((T, D))
    for t in range(T):
        for e, a in zip(ids[t], wts[t].astype(np.float32)):
            want[t] += a * R.expert(xin[t].astype(np.float64), wg[e], wu[e], wd[e], limit)
    tol = 2e-2 if dtype == capi.BF16 else 3e-5                # bfloat16 rounds the hidden row before the down projection
    assert np.abs(got - want).max() < tol * max(1.0, np.abs(want).max())
    hit = np.mean(np.abs(np.einsum("td,efd->tef", xin, wu)) > limit)
    assert hit > 0.05                                          # the clamp was exercised
