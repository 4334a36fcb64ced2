"""The Meresun decoder family: configuration, weight loading and the Python handle on its C++ runner
(crabml_b200/csrc/host/meresun_runner.cpp; the stack is described in include/crabml_meresun.h).

A model folder holds config.json and model.safetensors.  config.json gives every size and every constant that can differ between
models of the family: `vocab`, `width`, `embedding.scale`, `norm` (`eps`, `groups`), `token_side.dim`, `loop` (`start`, `stop`,
`times`) and `layers`, a list whose entries name the layer's mixer (`type`: "latent_attention"), the mixer's sizes (`mixer`) and its
feed-forward (`mlp`: kind "dense" or "moe", or null).  Tensor names: `embed`, `side.embed`, `head`, `final.norm`, and per layer i
`l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`, `l<i>.rg1`, `l<i>.rg2` (+ `.b`), `l<i>.side.*`.

Precision: `dtype="bfloat16"` keeps the matrices of the dense products in bfloat16 (activations are rounded to bfloat16 at the input
of a product, sums are 32-bit); `dtype="float32"` widens them and every product is a true 32-bit one.  In both modes the residual
stream, norms, rotations, attention scores and sums (with the key / value up-projections folded into them), routers and gates are
32-bit.
"""
from __future__ import annotations

import ctypes as C
import json
import os

import numpy as np

from . import capi, rotary
from .capi import CudaError, TensorError
from .safetensors import bf16_to_f32, f32_to_bf16, read_safetensors
from .seqmodel import SeqModel, Uploader, handle_of
from .tensor import CudaTensorDevice

ARCHITECTURE = "Meresun"
FF_KINDS = {"dense": 1, "moe": 2}


# ---- configuration ----------------------------------------------------------------------------------------------------------------
def parse_config(conf: dict) -> dict:
    """Validates a config.json dict and fills the optional keys, so that the rest of the code reads one shape of dict."""
    if conf.get("architecture", ARCHITECTURE) != ARCHITECTURE:
        raise TensorError(f"not a {ARCHITECTURE} config: architecture = {conf.get('architecture')!r}")
    norm = conf["norm"]
    out = {"architecture": ARCHITECTURE, "vocab": int(conf["vocab"]), "width": int(conf["width"]),
           "embedding": {"scale": float((conf.get("embedding") or {}).get("scale", 1.0))},
           "norm": {"eps": float(norm["eps"]), "groups": int(norm.get("groups", 1))},
           "token_side": {"dim": int(conf["token_side"]["dim"])} if conf.get("token_side") else None, "layers": []}
    n = len(conf["layers"])
    lp = conf.get("loop")
    out["loop"] = {"start": int(lp["start"]), "stop": int(lp["stop"]), "times": int(lp["times"])} if lp else {"start": 0, "stop": 0, "times": 1}
    if not (0 <= out["loop"]["start"] <= out["loop"]["stop"] <= n) or out["loop"]["times"] < 1:
        raise TensorError(f"loop {out['loop']} does not fit {n} layers")
    if out["width"] % out["norm"]["groups"]:
        raise TensorError("norm.groups does not divide the width")
    for i, L in enumerate(conf["layers"]):
        if L["type"] != "latent_attention":
            raise TensorError(f"layer {i}: unknown mixer type {L['type']!r}")
        m = dict(L["mixer"])
        for key in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
            m[key] = int(m[key])
        m["scale"] = float(m["scale"])
        m["mask"] = {"size": int(m["mask"]["size"])} if m.get("mask") else None
        if m.get("rot"):
            r = m["rot"]
            sc = r.get("scaling")
            m["rot"] = {"dims": int(r["dims"]), "base": float(r["base"]),
                        "scaling": {k: float(sc[k]) for k in ("factor", "original", "fast", "slow")} if sc else None}
            if m["rot"]["dims"] > m["rot_dim"] or m["rot"]["dims"] % 2:
                raise TensorError(f"layer {i}: rot.dims must be even and at most rot_dim")
        else:
            m["rot"] = None
        mlp = L.get("mlp")
        if mlp is not None:
            kind = mlp.get("kind")
            if kind not in FF_KINDS:
                raise TensorError(f"layer {i}: unknown feed-forward kind {kind!r}")
            if kind == "dense":
                mlp = {"kind": "dense", "ff": int(mlp["ff"])}
            else:
                r = mlp["router"]
                g = r.get("groups") or {"count": 1, "keep": 1}
                mlp = {"kind": "moe", "expert": {"ff": int(mlp["expert"]["ff"]), "limit": float(mlp["expert"].get("limit", 0.0))},
                       "router": {"experts": int(r["experts"]), "top": int(r["top"]), "groups": {"count": int(g["count"]), "keep": int(g["keep"])}}}
        out["layers"].append({"type": "latent_attention", "mixer": m, "mlp": mlp})
    return out


def expected_tensors(conf: dict, gated: bool = True, sink: bool = True) -> dict:
    """name -> shape of every tensor a model of this config has"""
    D, V = conf["width"], conf["vocab"]
    t = {"embed": [V, D], "head": [V, D], "final.norm": [D]}
    side = conf["token_side"]["dim"] if conf.get("token_side") else 0
    if side:
        t["side.embed"] = [V, side * len(conf["layers"])]
    for i, L in enumerate(conf["layers"]):
        m, p = L["mixer"], f"l{i}."
        H, dn, dr, dv, qr, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
        t.update({p + "norm1": [D], p + "mix.dq": [qr, D], p + "mix.dq.norm": [qr], p + "mix.uq": [H * (dn + dr), qr], p + "mix.dkv": [kr + dr, D],
                  p + "mix.dkv.norm": [kr], p + "mix.uk": [H * dn, kr], p + "mix.uv": [H * dv, kr], p + "mix.o": [D, H * dv]})
        if sink:
            t[p + "mix.sink"] = [H]
        if gated:
            t.update({p + "rg1": [D, D], p + "rg1.b": [D]})
        mlp = L["mlp"]
        if mlp:
            if gated:
                t.update({p + "rg2": [D, D], p + "rg2.b": [D]})
            if mlp["kind"] == "dense":
                t.update({p + "mlp.up": [mlp["ff"], D], p + "mlp.down": [D, mlp["ff"]], p + "mlp.act": [4]})
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                t.update({p + "mlp.router": [E, D], p + "mlp.correction": [E]})
                for e in range(E):
                    t.update({f"{p}mlp.e{e}.gate": [ff, D], f"{p}mlp.e{e}.up": [ff, D], f"{p}mlp.e{e}.down": [D, ff]})
        if side:
            t.update({p + "side.gate": [side, D], p + "side.proj": [D, side], p + "side.norm": [D]})
    return t


def random_weights(conf: dict, seed: int = 0, scale: float = 1.0) -> dict:
    """Random weights of a config (float32 arrays whose values are exact in bfloat16), sized so that activations stay O(1)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in expected_tensors(conf).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm") or name == "final.norm":
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif leaf == "sink":
            a = rng.standard_normal(shape)
        elif leaf == "b":
            a = rng.standard_normal(shape) * 0.5
        elif leaf == "act":
            a = np.array([0.6, 0.3, 0.15, 0.05]) + 0.05 * rng.standard_normal(4)
        elif leaf == "correction":
            a = rng.standard_normal(shape) * 0.2
        elif name in ("embed", "side.embed"):
            a = rng.standard_normal(shape)
        else:
            a = rng.standard_normal(shape) * (scale / np.sqrt(shape[-1]))
        out[name] = bf16_to_f32(f32_to_bf16(np.asarray(a, np.float32))).reshape(shape)
    return out


# ---- the model on a device ------------------------------------------------------------------------------------------------------------
class MeresunModel(SeqModel):
    """Weights of one model on one device + its runner (sequences, steps and generation: seqmodel.SeqModel).  `weights`: {name: float32
    ndarray} or the pair read_safetensors returns.  The gates `l<i>.rg1/rg2` and the sinks are used where the tensors exist."""

    def __init__(self, device: CudaTensorDevice, conf: dict, weights, dtype: str = "bfloat16", chunk: int = 0, max_seq: int = 0):
        self.device, self.conf, self.dtype = device, parse_config(conf), dtype
        up = Uploader(device, weights, dtype)
        c = self.conf
        names = up.weights
        up.check(expected_tensors(c, gated=any(n.endswith(".rg1") for n in names), sink=any(n.endswith(".sink") for n in names)))
        nl = len(c["layers"])
        side = c["token_side"]["dim"] if c["token_side"] else 0
        # the embedding scale is folded into the (32-bit) table: one rounding, as when it is applied to the looked-up row
        embed = up.f32("embed") * np.float32(c["embedding"]["scale"])
        self.tensors = {"embed": up.table(embed), "final.norm": up.vec("final.norm"), "head": up.mat("head")}
        side_all = up.f32("side.embed") if side else None
        lcs = (capi.cmr_layer_config * nl)()
        lws = (capi.cmr_layer_weights * nl)()
        for i, L in enumerate(c["layers"]):
            m, mlp, p = L["mixer"], L["mlp"], f"l{i}."
            lc = lcs[i]
            lc.heads, lc.dim, lc.rot_dim, lc.vdim, lc.q_rank, lc.kv_rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            lc.window, lc.scale, lc.rot_mag = (m["mask"]["size"] if m["mask"] else 0), m["scale"], 1.0
            t = {"norm1": up.vec(p + "norm1"), "dq_norm": up.vec(p + "mix.dq.norm"), "uq": up.mat(p + "mix.uq"), "dkv_norm": up.vec(p + "mix.dkv.norm"),
                 "uk": up.mat(p + "mix.uk"), "uv": up.mat(p + "mix.uv"), "o": up.mat(p + "mix.o")}
            # one product for everything that multiplies the layer's normed input (the order include/crabml_meresun.h gives)
            on_h = [p + "mix.dkv", p + "mix.dq"]
            # the few-row pass folds the up-projections into the 32-bit scores and sums: F32 copies, the key one transposed head by head
            uk = up.f32(p + "mix.uk").reshape(m["heads"], m["dim"], m["kv_rank"])
            t["uk_t"] = up.table(np.ascontiguousarray(uk.transpose(0, 2, 1)).reshape(m["heads"] * m["kv_rank"], m["dim"]))
            t["uv_f32"] = t["uv"] if dtype == "float32" else up.mat32(p + "mix.uv")
            if p + "mix.sink" in names:
                t["sink"] = up.vec(p + "mix.sink")
            if m["rot"] and m["rot"]["dims"] > 0:
                freq, mag = rotary.table_of(m["rot"])
                t["rot_freq"], lc.rot_mag = up.table(freq), mag
            for g in ("rg1", "rg2"):
                if p + g in names and (g == "rg1" or mlp):
                    on_h.append(p + g)
                    t[g + "_b"] = up.vec(p + g + ".b")
            if mlp and mlp["kind"] == "dense":
                on_h.append(p + "mlp.up")
            t["h_stack"] = up.stack(on_h)
            lc.ff_kind = FF_KINDS[mlp["kind"]] if mlp else 0
            if mlp and mlp["kind"] == "dense":
                lc.ff = mlp["ff"]
                t["down"], t["act"] = up.mat(p + "mlp.down"), up.vec(p + "mlp.act")
            elif mlp:
                r = mlp["router"]
                lc.ff, lc.limit = mlp["expert"]["ff"], mlp["expert"]["limit"]
                lc.experts, lc.top, lc.groups, lc.keep_groups = r["experts"], r["top"], r["groups"]["count"], r["groups"]["keep"]
                t["router"], t["correction"] = up.mat32(p + "mlp.router"), up.vec(p + "mlp.correction")
                for part in ("gate", "up", "down"):
                    t["e_" + part] = up.stack([f"{p}mlp.e{e}.{part}" for e in range(r["experts"])])
            if side:
                t["side_table"] = up.table(side_all[:, i * side:(i + 1) * side])
                t["side_gate"], t["side_proj"], t["side_norm"] = up.mat(p + "side.gate"), up.mat(p + "side.proj"), up.vec(p + "side.norm")
            for k, v in t.items():
                setattr(lws[i], k, handle_of(v))
                self.tensors[f"{p}{k}"] = v                                  # keep alive
        lp = c["loop"]
        cc = capi.cmr_config(nl, c["width"], c["vocab"], c["norm"]["eps"], c["norm"]["groups"], lp["start"], lp["stop"], lp["times"], side, int(chunk), int(max_seq))
        h = C.c_void_p()
        rc = device.lib.cmr_runner_create(device.handle, C.byref(cc), lcs, lws, self.tensors["embed"].buf.handle, self.tensors["final.norm"].buf.handle,
                                          self.tensors["head"].buf.handle, C.byref(h))
        if rc != capi.CC_OK:
            raise (TensorError if rc == capi.CC_ERR_TENSOR else CudaError)(f"cmr_runner_create failed [{rc}]: {device.lib.csr_last_create_error().decode()}")
        self.handle = h
        self.vocab = c["vocab"]
        self._keep = (lcs, lws)


def load(path: str, device: CudaTensorDevice, dtype: str = "bfloat16", chunk: int = 0, max_seq: int = 0) -> MeresunModel:
    """path: a folder with config.json and model.safetensors"""
    with open(os.path.join(path, "config.json")) as f:
        conf = json.load(f)
    return MeresunModel(device, conf, read_safetensors(os.path.join(path, "model.safetensors")), dtype, chunk, max_seq)
