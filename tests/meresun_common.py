"""Small Meresun configurations for the tests and helpers that run the framework's runner the way a server would: open a slot, feed
portions, read logits."""
import numpy as np


def rot(dims, base=10000.0, scaling="default"):
    if scaling == "default":
        scaling = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = scaling
    return r


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, groups=3, keep=2, ff=12, limit=1.0):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}


def layer(heads=3, dim=8, rot_dim=4, vdim=10, q_rank=12, kv_rank=20, window=7, scale=0.3, mlp="default", rotary="default"):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "mask": {"size": window}, "scale": scale,
         "rot": rot(rot_dim) if rotary == "default" else rotary}
    return {"type": "latent_attention", "mixer": m, "mlp": dense() if mlp == "default" else mlp}


def config(layers, width=36, vocab=53, eps=1e-5, groups=3, side=5, loop=None, embed_scale=0.7):
    c = {"architecture": "Meresun", "vocab": vocab, "width": width, "embedding": {"scale": embed_scale}, "norm": {"eps": eps, "groups": groups}, "layers": layers}
    if side:
        c["token_side"] = {"dim": side}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


def mixed_config():
    """a dense layer, then a looped pair (routed, none) that runs twice, then a routed one with other sizes; windows differ per layer"""
    return config([layer(window=5), layer(heads=2, dim=12, rot_dim=6, vdim=7, q_rank=9, kv_rank=14, window=9, mlp=moe()), layer(window=4, mlp=None),
                   layer(heads=4, dim=4, rot_dim=2, vdim=16, q_rank=20, kv_rank=11, window=6, mlp=moe(experts=4, top=1, groups=0, ff=20, limit=0.6))], loop=(1, 3, 2))


def rel_err(got, want):
    """per row: RMS of the mean-free difference over the RMS of the mean-free reference"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((w ** 2).mean(-1))


def run_portions(model, tokens, portions, want_all=True):
    """feeds `tokens` cut into `portions` (a list of sizes summing to len(tokens)) through a fresh slot; -> logits of every position"""
    slot = model.open()
    out, at = [], 0
    for n in portions:
        out.append(model.step(slot, tokens[at:at + n], list(range(n)) if want_all else []))
        at += n
    assert at == len(tokens)
    model.close_seq(slot)
    return np.concatenate(out, 0)
