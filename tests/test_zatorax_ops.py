"""Each mechanism of include/crabml_seqops.h alone, against its function in the plain reference (tests/zatorax_ref.py).
Where random inputs would hide a fault (a window's edge, a far key, a masked group) the inputs are made so that it shows."""
import numpy as np
import pytest

from crabml_b200 import capi, seqops
from tests import zatorax_ref as R
from tests.gpu_common import make_device

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
    """a weight matrix as the loader uploads it"""
    from crabml_b200 import CudaTensor
    from crabml_b200.zatorax import f32_to_bf16
    a = np.ascontiguousarray(a, np.float32)
    if dtype == capi.BF16:
        return CudaTensor.from_cpu(f32_to_bf16(a), list(a.shape), capi.BF16, dev)
    return CudaTensor.from_cpu(a, list(a.shape), capi.F32, dev)


def bf16(a):
    from crabml_b200.zatorax import bf16_to_f32, f32_to_bf16
    return bf16_to_f32(f32_to_bf16(np.asarray(a, np.float32))).reshape(np.shape(a))


@pytest.mark.parametrize("b", [1, 5, 8, 40, 130, 300])
@pytest.mark.parametrize("m,k", [(24, 48), (7, 100), (130, 64), (72, 192), (640, 128)])
def test_dense_products_f32_and_bf16(dev, b, m, k):
    rng = np.random.default_rng(b * 1000 + m + k)
    w = bf16(rng.standard_normal((m, k)) / np.sqrt(k))
    x = rng.standard_normal((b, k)).astype(np.float32)
    got = W(dev, w, capi.F32).matmul_vec(T32(dev, x)).export().reshape(b, m)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(got - want).max() < 2e-5
    got = W(dev, w, capi.BF16).matmul_vec(T32(dev, x)).export().reshape(b, m)
    want = bf16(x).astype(np.float64) @ w.astype(np.float64).T           # the activation is rounded, the sum is 32-bit
    assert np.abs(got - want).max() < 2e-5


@pytest.mark.parametrize("gain_n", [1, 40])
def test_rms_norm_gain_assign_and_accumulate(dev, gain_n):
    rng = np.random.default_rng(1)
    y = rng.standard_normal((9, 40)) * 3
    x0 = rng.standard_normal((9, 40))
    g = rng.standard_normal(gain_n)
    want = R.rms_unit(y, 1e-5) * g
    dst = T32(dev, x0)
    seqops.rms_norm_gain(dst, T32(dev, y), T32(dev, g), 1e-5, accumulate=True)
    assert np.abs(dst.export().reshape(9, 40) - (x0 + want)).max() < 1e-5
    seqops.rms_norm_gain(dst, T32(dev, y), T32(dev, g), 1e-5, accumulate=False)
    assert np.abs(dst.export().reshape(9, 40) - want).max() < 1e-5


def test_gated_head_rms_norm_and_glu(dev):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((5, 3 * 20)); gate = rng.standard_normal((5, 3 * 20)); w = rng.standard_normal(20)
    want = (R.rms_unit(x.reshape(5, 3, 20), 1e-6) * w * R.silu(gate.reshape(5, 3, 20))).reshape(5, 60)
    got = seqops.gated_head_rms_norm(T32(dev, x), T32(dev, gate), T32(dev, w), 20, 1e-6).export().reshape(5, 60)
    assert np.abs(got - want).max() < 1e-5
    got = seqops.glu_inplace(T32(dev, gate), T32(dev, x)).export().reshape(5, 60)
    assert np.abs(got - R.silu(gate) * x).max() < 1e-5


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_conv_whole_and_in_portions(dev, taps):
    from crabml_b200 import CudaTensor
    rng = np.random.default_rng(taps)
    T, heads, hs = 23, 3, 10
    C = heads * hs
    x = rng.standard_normal((T, C)); w = rng.standard_normal((C, taps))
    y = R.silu(R.causal_conv(x, w)).reshape(T, heads, hs)
    want_unit = (y / np.sqrt((y * y).sum(-1, keepdims=True) + 1e-6) * 0.25).reshape(T, C)
    for portions in ([T], [1] * T, [2, 3, 1, 7, 2, 8], [5, 18]):
        tail = CudaTensor.alloc([max(taps - 1, 1), C], capi.F32, dev) if taps > 1 else None
        outs, at = [], 0
        for n in portions:
            outs.append(seqops.short_conv(T32(dev, x[at:at + n]), T32(dev, w), tail, capi.ACT_SILU, hs, True, 1e-6, 0.25).export().reshape(n, C))
            at += n
        assert np.abs(np.concatenate(outs) - want_unit).max() < 2e-6, portions
    tail = CudaTensor.alloc([max(taps - 1, 1), C], capi.F32, dev) if taps > 1 else None
    got = seqops.short_conv(T32(dev, x), T32(dev, w), tail, capi.ACT_SILU).export().reshape(T, C)            # no unit norm (the value path)
    assert np.abs(got - y.reshape(T, C)).max() < 1e-5


@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 64, 48), (2, 2, 32, 72), (3, 1, 20, 12), (1, 1, 128, 8), (2, 1, 8, 130), (2, 1, 128, 128)])
def test_gated_delta_rule_whole_portions_and_state(dev, H, G, dk, dv):
    from crabml_b200 import CudaTensor
    rng = np.random.default_rng(H * 100 + dk)
    T = 37
    q = rng.standard_normal((T, G, dk)); k = rng.standard_normal((T, G, dk)); v = rng.standard_normal((T, H, dv))
    q /= np.linalg.norm(q, axis=-1, keepdims=True) * np.sqrt(dk); k /= np.linalg.norm(k, axis=-1, keepdims=True)
    a = rng.standard_normal((T, H)) * 2; b = rng.standard_normal((T, H)) * 2
    a_log = np.log(rng.uniform(0.3, 3.0, H)); dt = rng.uniform(-2, 1, H)
    beta = R.sigmoid(b); decay = np.exp(-np.exp(a_log)[None] * R.softplus(a + dt[None]))
    want, S_want = R.delta_rule(q, k, v, beta, decay)
    for portions in ([T], [1] * T, [2, 5, 1, 29], [36, 1]):
        state = CudaTensor.alloc([H, dk, dv], capi.F32, dev)
        outs, at = [], 0
        for n in portions:
            sl = slice(at, at + n)
            outs.append(seqops.gated_delta_rule(T32(dev, q[sl].reshape(n, -1)), T32(dev, k[sl].reshape(n, -1)), T32(dev, v[sl].reshape(n, -1)), T32(dev, a[sl]),
                                                T32(dev, b[sl]), T32(dev, a_log), T32(dev, dt), state, H, G, dk, dv).export().reshape(n, H, dv))
            at += n
        got = np.concatenate(outs)
        assert np.abs(got - want).max() < 2e-5 * max(1.0, np.abs(want).max()), portions
        assert np.abs(state.export().reshape(H, dk, dv) - S_want).max() < 2e-5 * max(1.0, np.abs(S_want).max())


def test_delta_state_keeps_a_far_write(dev):
    """with decay ~ 1 and orthogonal keys, what token 0 wrote is read back 300 tokens later, through portions of 1"""
    from crabml_b200 import CudaTensor
    H = G = 1; dk, dv, T = 32, 16, 301
    k = np.zeros((T, 1, dk)); k[0, 0, 0] = 1.0; k[1:, 0, 1] = 1.0
    q = np.zeros((T, 1, dk)); q[-1, 0, 0] = 1.0
    v = np.zeros((T, 1, dv)); v[0, 0] = np.arange(dv) + 1.0
    a = np.full((T, 1), -30.0); b = np.full((T, 1), 30.0)           # softplus -> 0: decay 1 ; beta 1
    state = CudaTensor.alloc([H, dk, dv], capi.F32, dev)
    out = None
    for t in range(T):
        out = seqops.gated_delta_rule(T32(dev, q[t].reshape(1, -1)), T32(dev, k[t].reshape(1, -1)), T32(dev, v[t].reshape(1, -1)), T32(dev, a[t:t + 1]), T32(dev, b[t:t + 1]),
                                      T32(dev, [0.0]), T32(dev, [0.0]), state, H, G, dk, dv)
    assert np.abs(out.export() - (np.arange(dv) + 1.0)).max() < 1e-4


def _attend(dev, q, k, v, knw, qnw, eps, H, G, dk, dv, window, scale, r1, r2, ring, portions):
    """append + attend portion by portion through a ring of `ring` rows"""
    from crabml_b200 import CudaTensor
    kring = CudaTensor.alloc([ring, G * dk], capi.F32, dev); vring = CudaTensor.alloc([ring, G * dv], capi.F32, dev)
    outs, at = [], 0
    for n in portions:
        sl = slice(at, at + n)
        seqops.kv_ring_append(kring, vring, T32(dev, k[sl].reshape(n, -1)), T32(dev, v[sl].reshape(n, -1)), T32(dev, knw) if knw is not None else None, eps, at, G, dk, dv)
        outs.append(seqops.window_attention(T32(dev, q[sl].reshape(n, -1)), T32(dev, qnw) if qnw is not None else None, eps, kring, vring, at, H, G, dk, dv, window, scale,
                                            T32(dev, r1) if r1 is not None else None, T32(dev, r2) if r2 is not None else None).export().reshape(n, H, dv))
        at += n
    return np.concatenate(outs)


@pytest.mark.parametrize("H,G,dk,dv,window", [(4, 2, 16, 24, 7), (3, 3, 40, 8, 1), (2, 1, 64, 64, 50), (6, 2, 12, 20, 13)])
def test_window_attention_random(dev, H, G, dk, dv, window):
    rng = np.random.default_rng(window)
    T = 45
    q = rng.standard_normal((T, H, dk)); k = rng.standard_normal((T, G, dk)); v = rng.standard_normal((T, G, dv))
    qnw = rng.standard_normal(dk); knw = rng.standard_normal(dk); r1 = rng.uniform(0.1, 2, H); r2 = rng.uniform(0.1, 2, H)
    want = R.windowed_softmax_attention(R.rms_unit(q, 1e-5) * qnw, R.rms_unit(k, 1e-5) * knw, v, window, 0.2, r1, r2)
    for portions, chunk in (([T], T), ([1] * T, 1), ([2, 3, 11, 1, 28], 28), ([20, 25], 25)):
        got = _attend(dev, q, k, v, knw, qnw, 1e-5, H, G, dk, dv, window, 0.2, r1, r2, window - 1 + chunk, portions)          # the smallest legal ring: rows are reused
        assert np.abs(got - want).max() < 2e-5, portions


def test_window_edge_shows_in_and_out(dev):
    """one key scores far above all others: a query sees its value exactly while 0 <= i - j < window, in prompts and decoded alone"""
    H = G = 1; dk, dv, window, T, j = 8, 4, 6, 20, 5
    k = np.zeros((T, 1, dk)); k[:, 0, 1] = 1.0; k[j, 0, 0] = 40.0; k[j, 0, 1] = 0.0
    q = np.zeros((T, 1, dk)); q[:, 0, 0] = 1.0
    v = np.zeros((T, 1, dv)); v[j, 0, 0] = 1.0; v[:, 0, 1] = 1.0; v[j, 0, 1] = 0.0
    for portions in ([T], [1] * T, [j + window - 1, 1, 1, T - j - window - 1], [2] * (T // 2)):
        got = _attend(dev, q, k, v, None, None, 0.0, H, G, dk, dv, window, 1.0, None, None, window - 1 + max(portions), portions)
        for i in range(T):
            seen = 0 <= i - j < window
            assert abs(got[i, 0, 0] - (1.0 if seen else 0.0)) < 1e-6, (portions, i)
        assert got[j + window - 1, 0, 0] > 0.999 and got[j + window, 0, 0] == 0.0


def test_far_key_among_hundreds(dev):
    """a wide window: the key 400 positions back stands out and is found, from a prompt and from a decoded token"""
    H = G = 1; dk, dv, T, window = 16, 4, 420, 512
    rng = np.random.default_rng(0)
    k = rng.standard_normal((T, 1, dk)) * 0.1; q = rng.standard_normal((T, 1, dk)) * 0.1
    v = rng.standard_normal((T, 1, dv)); k[15, 0] = 0; k[15, 0, 3] = 30.0; q[415, 0] = 0; q[415, 0, 3] = 3.0
    want = R.windowed_softmax_attention(q, k, v, window, 1.0, np.array([0.5]), np.array([0.25]))
    assert np.abs(want[415, 0] - v[15, 0]).max() < 1e-3
    for portions in ([T], [410] + [1] * 10, [100, 200, 115, 5]):
        got = _attend(dev, q, k, v, None, None, 0.0, H, G, dk, dv, window, 1.0, [0.5], [0.25], window - 1 + max(portions), portions)
        assert np.abs(got - want).max() < 2e-5


@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 4, 2), (6, 2, 1, 1), (12, 4, 3, 3), (4, 4, 2, 2), (5, 1, 5, 1), (64, 6, 8, 3)])
def test_router_against_reference(dev, E, top, groups, keep):
    rng = np.random.default_rng(E * 10 + top)
    T, D = 50, 24
    x = rng.standard_normal((T, D)); wr = rng.standard_normal((E, D)) * 0.5
    corr = rng.standard_normal(E) - 1.0                        # mostly NEGATIVE choice scores: a mask of 0 instead of -inf would win
    w = {"m.router": wr, "m.correction": corr}
    chosen, weights = R.route(x.astype(np.float32).astype(np.float64), {k: v.astype(np.float32).astype(np.float64) for k, v in w.items()}, "m",
                              {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}})
    ids, wts = seqops.moe_route(T32(dev, x), T32(dev, wr), T32(dev, corr), top, groups, keep)
    got_ids = ids.export().view(np.int32).reshape(T, top)
    got_w = wts.export().reshape(T, top)
    assert np.array_equal(got_ids, chosen)
    assert np.abs(got_w - weights).max() < 1e-6
    assert abs(got_w.sum(-1) - 1.0).min() > 1e-3 or top == E            # not renormalised


@pytest.mark.parametrize("dtype", [capi.F32, capi.BF16])
@pytest.mark.parametrize("T,D,E,ff,top", [(19, 40, 5, 28, 2), (200, 128, 6, 64, 3), (333, 64, 3, 192, 1), (70, 192, 40, 64, 4)])
def test_experts_weighted_sum(dev, dtype, T, D, E, ff, top):
    """few rows: one warp per hidden row; many rows of BF16 weights with 64-aligned sizes: rows sorted by expert through the grouped
    tensor-core product (experts with no row, with one row and with several tiles of rows all occur)"""
    from crabml_b200 import CudaTensor
    rng = np.random.default_rng(5 + T)
    x = rng.standard_normal((T, D)).astype(np.float32)
    wg = bf16(rng.standard_normal((E, ff, D)) / np.sqrt(D)); wu = bf16(rng.standard_normal((E, ff, D)) / np.sqrt(D)); wd = bf16(rng.standard_normal((E, D, ff)) / np.sqrt(ff))
    pool = np.array([e for e in range(E) if e != 1])            # expert 1 gets no row at all
    ids = np.stack([rng.permutation(pool)[:top] for _ in range(T)]).astype(np.int32)
    if top < len(pool):
        ids[ids == pool[-1]] = pool[0]
        ids[0, 0] = pool[-1]                                     # and the last one exactly one row (the others of row 0 differ from it)
        for t in range(T):                                       # keep a token's experts distinct
            seen = set()
            for s_ in range(top):
                while int(ids[t, s_]) in seen:
                    ids[t, s_] = pool[(int(np.where(pool == ids[t, s_])[0][0]) + 1) % (len(pool) - 1)]
                seen.add(int(ids[t, s_]))
    wts = rng.uniform(0.1, 0.6, (T, top)).astype(np.float32)
    want = np.zeros((T, D))
    for t in range(T):
        for s in range(top):
            e = ids[t, s]
            want[t] += wts[t, s] * (wd[e].astype(np.float64) @ (R.silu(wg[e].astype(np.float64) @ x[t]) * (wu[e].astype(np.float64) @ x[t])))
    tid = CudaTensor.from_cpu(ids, [T, top], capi.I32, dev)
    got = seqops.moe_experts(T32(dev, x), tid, T32(dev, wts), W(dev, wg.reshape(E * ff, D), dtype), W(dev, wu.reshape(E * ff, D), dtype), W(dev, wd.reshape(E * D, ff), dtype),
                             E, ff).export().reshape(T, D)
    if dtype == capi.BF16:            # the product path rounds x and the hidden row to bfloat16: do the same to the reference
        want = np.zeros((T, D))
        for t in range(T):
            for s in range(top):
                e = ids[t, s]
                xb = bf16(x[t]).astype(np.float64)
                hrow = np.float32(R.silu((wg[e].astype(np.float64) @ xb).astype(np.float32).astype(np.float64))) * (wu[e].astype(np.float64) @ xb).astype(np.float32)
                want[t] += wts[t, s] * (wd[e].astype(np.float64) @ bf16(hrow).astype(np.float64))
    assert np.abs(got - want).max() < (2e-5 if dtype == capi.F32 else 2e-2)


def test_bad_arguments_are_tensor_errors(dev):
    from crabml_b200 import CudaTensor, TensorError
    with pytest.raises(TensorError):
        seqops.moe_route(T32(dev, np.zeros((2, 8))), T32(dev, np.zeros((6, 8))), None, 4, 3, 1)           # 1 group of 2 cannot give 4 experts
    kring = CudaTensor.alloc([4, 8], capi.F32, dev); vring = CudaTensor.alloc([4, 8], capi.F32, dev)
    with pytest.raises(TensorError):                                                                      # window 6 needs more rows than the ring has
        seqops.window_attention(T32(dev, np.zeros((1, 8))), None, 0.0, kring, vring, 10, 1, 1, 8, 8, 6, 1.0)
