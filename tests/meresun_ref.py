"""A plain, slow statement of the Meresun decoder in float64 numpy: one function per mechanism, whole sequences only, no cache, no
portions, no batches.  It shares no code with crabml_b200; the tests compare the framework with it.

Notation: x [T, D] is the residual stream of one sequence, positions 0 .. T-1; a matrix W is stored [out, in] and applied as x @ W.T.
`w` maps tensor names to float arrays, `conf` is the config.json dict as written (optional keys may be missing)."""
import numpy as np


def rms_norm(x, weight, eps):
    x = np.asarray(x, np.float64)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * weight


def group_rms_norm(x, weight, groups, eps):
    """the last axis is cut into `groups` equal consecutive parts, each divided by its own root mean square"""
    x = np.asarray(x, np.float64)
    parts = x.reshape(x.shape[:-1] + (groups, x.shape[-1] // groups))
    parts = parts / np.sqrt((parts * parts).mean(-1, keepdims=True) + eps)
    return parts.reshape(x.shape) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


# ---- rotary positions --------------------------------------------------------------------------------------------------------------
def rotary_frequencies(rot):
    """-> (frequency of pair i, i < dims / 2 ; factor on cos and sin)"""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * np.log(original / (2.0 * np.pi * turns)) / (2.0 * np.log(base))
    lo = max(np.floor(dim_of(float(sc["fast"]))), 0.0)
    hi = min(np.ceil(dim_of(float(sc["slow"]))), dims - 1.0)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * np.log(factor) + 1.0


def rotate_pairs(v, positions, freq, mag):
    """v [T, ..., dims]: coordinate 2i is paired with 2i+1; positions [T]"""
    v = np.asarray(v, np.float64)
    ang = np.asarray(positions, np.float64)[:, None] * freq[None, :]
    shape = (v.shape[0],) + (1,) * (v.ndim - 2) + (freq.size,)
    c, s = (np.cos(ang) * mag).reshape(shape), (np.sin(ang) * mag).reshape(shape)
    a, b = v[..., 0::2], v[..., 1::2]
    out = np.empty_like(v)
    out[..., 0::2] = a * c - b * s
    out[..., 1::2] = b * c + a * s
    return out


# ---- mixer ---------------------------------------------------------------------------------------------------------------------------
def latent_attention(h, w, p, m, eps):
    """h [T, D]; p: the tensor prefix '<layer>.mix.'; m: the layer's mixer sizes"""
    T = h.shape[0]
    H, dn, dr, dv, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = np.arange(T)
    freq, mag = rotary_frequencies(m["rot"])
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_pairs(q[..., dn:], pos, freq, mag)
    kv = h @ w[p + "dkv"].T
    c = rms_norm(kv[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(kv[:, rank:], pos, freq, mag)                 # [T, dr], one for all heads
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    window = int(m["mask"]["size"]) if m.get("mask") else 0
    out = np.zeros((T, H, dv))
    for i in range(T):
        lo = max(0, i - window + 1) if window > 0 else 0
        for hh in range(H):
            s = (k_plain[lo:i + 1, hh] @ q_plain[i, hh] + k_rot[lo:i + 1] @ q_rot[i, hh]) * float(m["scale"])
            sink = float(w[p + "sink"][hh]) if p + "sink" in w else -np.inf
            mx = max(s.max(), sink)
            e = np.exp(s - mx)
            out[i, hh] = (e / (e.sum() + np.exp(sink - mx))) @ v[lo:i + 1, hh]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ---- feed-forwards -----------------------------------------------------------------------------------------------------------------
def poly_norm(z, coef, eps):
    def unit(a):
        return a / np.sqrt((a * a).mean(-1, keepdims=True) + eps)
    return coef[0] * unit(z) + coef[1] * unit(z ** 2) + coef[2] * unit(z ** 3) + coef[3]


def dense_ff(h, w, p, eps):
    return poly_norm(h @ w[p + "up"].T, np.asarray(w[p + "act"], np.float64), eps) @ w[p + "down"].T


def route(h, router, correction, top, n_groups, keep):
    """-> (ids [T, top], weights [T, top]) ; ties go to the lower index"""
    s = sigmoid(h @ router.T)
    choice = s + correction
    T, E = s.shape
    if n_groups > 1:
        per = E // n_groups
        g = np.sort(choice.reshape(T, n_groups, per), -1)[..., ::-1][..., :2].sum(-1)
        for t in range(T):
            kept = np.argsort(-g[t], kind="stable")[:keep]
            mask = np.full(E, -np.inf)
            for k in kept:
                mask[k * per:(k + 1) * per] = 0.0
            choice[t] = choice[t] + mask
    ids = np.argsort(-choice, -1, kind="stable")[:, :top]
    wt = np.take_along_axis(s, ids, -1)
    return ids, wt / (wt.sum(-1, keepdims=True) + 1e-20)


def expert(h, gate, up, down, limit):
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def moe_ff(h, w, p, mlp):
    r = mlp["router"]
    grp = r.get("groups") or {"count": 1, "keep": 1}
    ids, wt = route(h, w[p + "router"], w[p + "correction"], int(r["top"]), int(grp["count"]), int(grp["keep"]))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t], wt[t]):
            out[t] += a * expert(h[t], w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"], float(mlp["expert"]["limit"]))
    return out


# ---- the stack -----------------------------------------------------------------------------------------------------------------------
def layer(conf, w, i, x, tokens):
    L, p, eps = conf["layers"][i], f"l{i}.", float(conf["norm"]["eps"])
    h = group_rms_norm(x, w[p + "norm1"], int(conf["norm"].get("groups", 1)), eps)
    assert L["type"] == "latent_attention"
    y = latent_attention(h, w, p + "mix.", L["mixer"], eps)
    if p + "rg1" in w:
        y = y * sigmoid(h @ w[p + "rg1"].T + w[p + "rg1.b"])
    mlp = L.get("mlp")
    if mlp:
        f = dense_ff(h, w, p + "mlp.", eps) if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp)
        if p + "rg2" in w:
            f = f * sigmoid(h @ w[p + "rg2"].T + w[p + "rg2.b"])
        y = y + f
    x = x + y
    if conf.get("token_side"):
        d = int(conf["token_side"]["dim"])
        e = w["side.embed"][tokens][:, i * d:(i + 1) * d]
        g = gelu_tanh(x @ w[p + "side.gate"].T) * e
        x = x + rms_norm(g @ w[p + "side.proj"].T, w[p + "side.norm"], eps)
    return x


def layer_runs(conf):
    """[(layer, first of a repeated pass?)] in the order the layers run"""
    n = len(conf["layers"])
    lp = conf.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
    runs = [(i, False) for i in range(a)]
    for r in range(times):
        runs += [(i, r > 0 and i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(conf, w, tokens, residuals=None):
    """-> logits [T, vocab]; residuals (a list) receives the stream after every layer run"""
    tokens = np.asarray(tokens)
    w = {k: np.asarray(v, np.float64) for k, v in w.items()}
    eps = float(conf["norm"]["eps"])
    x0 = w["embed"][tokens] * float((conf.get("embedding") or {}).get("scale", 1.0))
    x = x0
    for i, again in layer_runs(conf):
        if again:
            x = x + x0
        x = layer(conf, w, i, x, tokens)
        if residuals is not None:
            residuals.append(x)
    return group_rms_norm(x, w["final.norm"], int(conf["norm"].get("groups", 1)), eps) @ w["head"].T
