"""Plain, slow numpy statement of the Zatorax design, one function per mechanism, in float64.

This is the oracle of tests/test_zatorax_*.py.  It shares no code with the product path (crabml_b200/zatorax.py and the
CUDA kernels): it takes a parsed config dict and a {name: ndarray} weight dict and runs a WHOLE sequence at once --
no cache, no state object, no chunking -- so every cached / chunked / batched product path can be held against it.

Notation: T tokens, D model width, H heads, G key/value heads, dk key size, dv value size.
"""
from __future__ import annotations

import numpy as np

F = np.float64


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose gain is ONE number for all coordinates."""
    return rms_unit(x, eps) * F(g)


def linear(w, x):
    """weights are stored [out, in]; x is [T, in]."""
    return x @ np.asarray(w, F).T


def causal_conv(x, taps_w):
    """x [T, C], taps_w [C, K]; the last column multiplies the current token, zeros before the start."""
    T, C = x.shape
    K = taps_w.shape[1]
    xp = np.concatenate([np.zeros((K - 1, C), F), x], 0)
    y = np.zeros((T, C), F)
    for j in range(K):
        y += xp[j:j + T] * np.asarray(taps_w, F)[:, j][None, :]
    return y


def delta_rule(q, k, v, beta, decay, S0=None):
    """The recurrence alone.  q, k [T, G, dk] (already normalised), v [T, H, dv], beta, decay [T, H]; per head, per token, in this order:
    S <- decay S ; u = beta (v - S^T k) ; S <- S + k u^T ; o = S^T q.   -> (o [T, H, dv], final S [H, dk, dv])"""
    T, G, dk = q.shape
    H, dv = v.shape[1], v.shape[2]
    rep = H // G
    o = np.zeros((T, H, dv), F)
    Sf = np.zeros((H, dk, dv), F)
    for hd in range(H):
        S = np.zeros((dk, dv), F) if S0 is None else np.array(S0[hd], F)
        g = hd // rep
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
        Sf[hd] = S
    return o, Sf


def delta_mixer(h, w, p, m, eps):
    """Gated delta rule.  h [T, D]; w: weights; p: tensor prefix '<layer>.mix'; m: the layer's mixer config."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(linear(w[p + ".q"], h), w[p + ".q.conv"])).reshape(T, G, dk)
    k = silu(causal_conv(linear(w[p + ".k"], h), w[p + ".k.conv"])).reshape(T, G, dk)
    v = silu(causal_conv(linear(w[p + ".v"], h), w[p + ".v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt(np.sum(q * q, -1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt(np.sum(k * k, -1, keepdims=True) + 1e-6)
    beta = sigmoid(linear(w[p + ".b"], h))                                                   # [T, H]
    decay = np.exp(-np.exp(np.asarray(w[p + ".A_log"], F))[None, :] * softplus(linear(w[p + ".a"], h) + np.asarray(w[p + ".dt_bias"], F)[None, :]))
    gate = silu(linear(w[p + ".g"], h)).reshape(T, H, dv)
    o, _ = delta_rule(q, k, v, beta, decay)
    o = rms_unit(o, eps) * np.asarray(w[p + ".norm"], F)[None, None, :] * gate
    return linear(w[p + ".o"], o.reshape(T, H * dv))


def attention_keys_values(h, w, p, m, eps):
    """The keys (after their norm) and values a layer with projections of its own puts into its cache."""
    G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k = rms_unit(linear(w[p + ".k"], h).reshape(T, G, dk), eps) * np.asarray(w[p + ".k.norm"], F)[None, None, :]
    v = linear(w[p + ".v"], h).reshape(T, G, dv)
    return k, v


def windowed_softmax_attention(q, k, v, win, scale, r1, r2):
    """q [T, H, dk] and k [T, G, dk] after their norms, v [T, G, dv].  Position i sees j with 0 <= i - j < win;
    score = q.k * scale - r1[h] * ln(1 + r2[h] * (i - j)); ordinary softmax over the visible keys."""
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    rep = H // G
    out = np.zeros((T, H, dv), F)
    for i in range(T):
        lo = max(0, i - win + 1)
        dist = (i - np.arange(lo, i + 1)).astype(F)
        for hd in range(H):
            g = hd // rep
            s = (k[lo:i + 1, g] @ q[i, hd]) * scale - r1[hd] * np.log1p(r2[hd] * dist)
            e = np.exp(s - s.max())
            out[i, hd] = (e / e.sum()) @ v[lo:i + 1, g]
    return out


def attention_mixer(h, w, p, m, eps, k, v):
    """Sliding-window softmax attention with a logarithmic distance penalty.  k, v: [T, G, dk] / [T, G, dv] (own or borrowed)."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    win, scale = m["mask"]["size"], F(m["scale"])
    q = rms_unit(linear(w[p + ".q"], h).reshape(T, H, dk), eps) * np.asarray(w[p + ".q.norm"], F)[None, None, :]
    out = windowed_softmax_attention(q, k, v, win, scale, np.asarray(w[p + ".r1"], F), np.asarray(w[p + ".r2"], F))
    return linear(w[p + ".o"], out.reshape(T, H * dv))


def expert(h, w, p):
    return linear(w[p + ".down"], silu(linear(w[p + ".gate"], h)) * linear(w[p + ".up"], h))


def route(h, w, p, r):
    """-> (chosen [T, top] expert ids, weights [T, top])."""
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    z = linear(w[p + ".router"], h)
    e = np.exp(z - z.max(-1, keepdims=True))
    s = e / e.sum(-1, keepdims=True)
    choice = s + np.asarray(w[p + ".correction"], F)[None, :]
    T = h.shape[0]
    per = E // groups["count"]
    gscore = choice.reshape(T, groups["count"], per).max(-1)
    kept = np.argsort(-gscore, axis=-1, kind="stable")[:, :groups["keep"]]
    allowed = np.zeros((T, groups["count"]), bool)
    np.put_along_axis(allowed, kept, True, -1)
    masked = np.where(np.repeat(allowed, per, axis=1), choice, -np.inf)
    chosen = np.argsort(-masked, axis=-1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(s, chosen, -1)


def moe(h, w, p, mlp):
    chosen, weights = route(h, w, p, mlp["router"])
    out = np.zeros((h.shape[0], np.asarray(w[p + ".e0.down"]).shape[0]), F)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            out[t] += wt * expert(h[t:t + 1], w, f"{p}.e{int(e)}")[0]
    if mlp.get("shared"):
        out += expert(h, w, p + ".shared")
    return out


def forward(conf, w, tokens, return_layers=False):
    """-> logits [T, vocab] (and the residual stream after every layer)."""
    eps = conf["norm"]["eps"]
    w = {k: np.asarray(v, F) for k, v in w.items()}
    x = w["embed"][np.asarray(tokens)]
    kv, layers = {}, []
    for i, L in enumerate(conf["layers"]):
        p = f"l{i}.mix"
        m = L["mixer"]
        if L["type"] == "delta":
            y = delta_mixer(x, w, p, m, eps)
        elif L["type"] == "attention":
            if m.get("kv_from") is not None:
                k, v = kv[m["kv_from"]]
            else:
                k, v = kv[i] = attention_keys_values(x, w, p, m, eps)
            y = attention_mixer(x, w, p, m, eps, k, v)
        else:
            raise ValueError(L["type"])
        x = x + scalar_norm(y, w[f"l{i}.norm1"], eps)
        if L.get("mlp"):
            x = x + scalar_norm(moe(x, w, f"l{i}.mlp", L["mlp"]), w[f"l{i}.norm2"], eps)
        layers.append(x.copy())
    logits = linear(w["head"], scalar_norm(x, w["final.norm"], eps))
    return (logits, np.stack(layers)) if return_layers else logits
