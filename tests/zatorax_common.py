"""Small Zatorax configurations for the tests (none of them a size combination of any shipped model) and helpers that run the
framework's runner the way a server would: open a slot, feed portions, read logits."""
import numpy as np


def moe_cfg(experts=6, top=2, groups=3, keep=2, ff=24, shared=16):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}},
            "shared": {"ff": shared} if shared else None}


def delta_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, mlp="default"):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": moe_cfg() if mlp == "default" else mlp}


def attn_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=7, scale=0.3, kv_from=None, mlp="default"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": moe_cfg() if mlp == "default" else mlp}


def config(layers, width=48, vocab=61, eps=1e-5):
    return {"architecture": "Zatorax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def mixed_config():
    """delta, attention, a borrower with a WIDER window than its source, delta with other sizes, attention without feed-forward"""
    return config([delta_layer(), attn_layer(window=5), attn_layer(window=9, kv_from=1, mlp=moe_cfg(experts=4, top=1, groups=1, keep=1, shared=0)),
                   delta_layer(heads=2, kv_heads=2, dim=8, vdim=40, conv=2, mlp=None), attn_layer(heads=3, kv_heads=1, dim=24, vdim=8, window=4, mlp=None)])


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
