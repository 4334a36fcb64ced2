"""The Zatorax decoder family: configuration, weight loading and the Python handle on its C++ runner
(crabml_b200/csrc/host/zatorax_runner.cpp).

A model folder holds config.json and model.safetensors.  config.json gives every size and every constant that can differ between
models of the family: `vocab`, `width`, `norm.eps` and `layers`, a list whose entries name the layer's mixer (`type`: "delta" or
"attention"), the mixer's sizes (`mixer`) and its feed-forward (`mlp`, or null).  Tensor names: `embed`, `head`, `final.norm`,
and per layer i `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*` (experts `e0`, `e1`, ..., `shared`, `router`, `correction`).

Precision: `dtype="bfloat16"` keeps the matrices in bfloat16 (activations are rounded to bfloat16 at the input of a product, sums are
32-bit); `dtype="float32"` widens them to f32 and every product is a true 32-bit one.  In both modes the residual stream, norms,
softmax, routers, convolutions, gates and the recurrent state are 32-bit.
"""
from __future__ import annotations

import ctypes as C
import json
import os

import numpy as np

from . import capi
from .capi import CudaError, TensorError
from .safetensors import bf16_to_f32, f32_to_bf16, read_safetensors, write_safetensors  # noqa: F401  (also this module's names)
from .seqmodel import SeqModel, Uploader, handle_of
from .tensor import CudaTensorDevice

ARCHITECTURE = "Zatorax"
MIXERS = {"delta": 0, "attention": 1}


# ---- configuration ----------------------------------------------------------------------------------------------------------------
def parse_config(conf: dict) -> dict:
    """Validates a config.json dict and fills the optional keys, so that the rest of the code reads one shape of dict."""
    if conf.get("architecture", ARCHITECTURE) != ARCHITECTURE:
        raise TensorError(f"not a {ARCHITECTURE} config: architecture = {conf.get('architecture')!r}")
    out = {"architecture": ARCHITECTURE, "vocab": int(conf["vocab"]), "width": int(conf["width"]), "norm": {"eps": float(conf["norm"]["eps"])}, "layers": []}
    for i, L in enumerate(conf["layers"]):
        kind = L["type"]
        if kind not in MIXERS:
            raise TensorError(f"layer {i}: unknown mixer type {kind!r}")
        m = dict(L["mixer"])
        for key in ("heads", "kv_heads", "dim", "vdim"):
            m[key] = int(m[key])
        if kind == "delta":
            m["conv"] = int(m["conv"])
        else:
            m["mask"] = {"size": int(m["mask"]["size"])}
            m["scale"] = float(m["scale"])
            m["kv_from"] = None if m.get("kv_from") is None else int(m["kv_from"])
        mlp = L.get("mlp")
        if mlp is not None:
            if mlp.get("kind", "moe") != "moe":
                raise TensorError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            r = mlp["router"]
            g = r.get("groups") or {"count": 1, "keep": 1}
            mlp = {"kind": "moe", "expert": {"ff": int(mlp["expert"]["ff"])},
                   "router": {"experts": int(r["experts"]), "top": int(r["top"]), "groups": {"count": int(g["count"]), "keep": int(g["keep"])}},
                   "shared": {"ff": int(mlp["shared"]["ff"])} if mlp.get("shared") else None}
        out["layers"].append({"type": kind, "mixer": m, "mlp": mlp})
    return out


def expected_tensors(conf: dict) -> dict:
    """name -> shape of every tensor a model of this config has."""
    D, V = conf["width"], conf["vocab"]
    t = {"embed": [V, D], "head": [V, D], "final.norm": []}
    for i, L in enumerate(conf["layers"]):
        m, p = L["mixer"], f"l{i}."
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        t[p + "norm1"] = []
        if L["type"] == "delta":
            K = m["conv"]
            t.update({p + "mix.q": [G * dk, D], p + "mix.q.conv": [G * dk, K], p + "mix.k": [G * dk, D], p + "mix.k.conv": [G * dk, K],
                      p + "mix.v": [H * dv, D], p + "mix.v.conv": [H * dv, K], p + "mix.b": [H, D], p + "mix.A_log": [H], p + "mix.norm": [dv],
                      p + "mix.a": [H, D], p + "mix.dt_bias": [H], p + "mix.g": [H * dv, D], p + "mix.o": [D, H * dv]})
        else:
            t.update({p + "mix.q": [H * dk, D], p + "mix.q.norm": [dk], p + "mix.r1": [H], p + "mix.r2": [H], p + "mix.o": [D, H * dv]})
            if m.get("kv_from") is None:
                t.update({p + "mix.k": [G * dk, D], p + "mix.v": [G * dv, D], p + "mix.k.norm": [dk]})
        mlp = L["mlp"]
        if mlp:
            t[p + "norm2"] = []
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            t[p + "mlp.router"] = [E, D]
            t[p + "mlp.correction"] = [E]
            names = [f"e{e}" for e in range(E)]
            for n in names:
                t.update({f"{p}mlp.{n}.gate": [ff, D], f"{p}mlp.{n}.up": [ff, D], f"{p}mlp.{n}.down": [D, ff]})
            if mlp["shared"]:
                sf = mlp["shared"]["ff"]
                t.update({p + "mlp.shared.gate": [sf, D], p + "mlp.shared.up": [sf, D], p + "mlp.shared.down": [D, sf]})
    return t


def random_weights(conf: dict, seed: int = 0, scale: float = 1.0) -> dict:
    """Random weights of a config (float32 arrays whose values are exact in bfloat16), sized so that activations stay O(1)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in expected_tensors(conf).items():
        leaf = name.split(".")[-1]
        if name.endswith("norm1") or name.endswith("norm2") or name == "final.norm":
            a = np.asarray(1.0 + 0.1 * rng.standard_normal(), np.float32)
        elif leaf == "norm":                                       # per-head norm weights
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif leaf == "conv":
            a = rng.standard_normal(shape) * 0.5
        elif leaf == "A_log":
            a = np.log(rng.uniform(0.5, 4.0, shape))
        elif leaf == "dt_bias":
            a = rng.uniform(-3.0, 0.0, shape)
        elif leaf == "r1":
            a = rng.uniform(0.2, 1.5, shape)
        elif leaf == "r2":
            a = rng.uniform(0.05, 1.0, shape)
        elif leaf == "correction":
            a = rng.standard_normal(shape) * 0.05
        elif name == "embed":
            a = rng.standard_normal(shape)
        else:
            a = rng.standard_normal(shape) * (scale / np.sqrt(shape[-1]))
        out[name] = bf16_to_f32(f32_to_bf16(np.asarray(a, np.float32))).reshape(shape)
    return out


# ---- the model on a device ------------------------------------------------------------------------------------------------------------
class ZatoraxModel(SeqModel):
    """Weights of one model on one device + its runner (sequences, steps and generation: seqmodel.SeqModel).  `weights`: {name: float32
    ndarray} (values representable in bfloat16 when dtype == "bfloat16") or the pair read_safetensors returns."""

    def __init__(self, device: CudaTensorDevice, conf: dict, weights, dtype: str = "bfloat16", chunk: int = 0):
        self.device, self.conf, self.dtype = device, parse_config(conf), dtype
        up = Uploader(device, weights, dtype)
        up.check(expected_tensors(self.conf))
        vec, mat, stack = up.vec, up.mat, up.stack

        c = self.conf
        self.tensors = {"embed": up.mat32("embed"), "final.norm": vec("final.norm"), "head": mat("head")}
        lcs = (capi.czr_layer_config * len(c["layers"]))()
        lws = (capi.czr_layer_weights * len(c["layers"]))()
        for i, L in enumerate(c["layers"]):
            m, mlp, p = L["mixer"], L["mlp"], f"l{i}."
            lc = lcs[i]
            lc.mixer, lc.heads, lc.kv_heads, lc.dim, lc.vdim = MIXERS[L["type"]], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            lc.conv, lc.window, lc.kv_from, lc.scale = 0, 0, -1, 0.0
            t = {"norm1": vec(p + "norm1")}
            if L["type"] == "delta":
                lc.conv = m["conv"]
                for k in ("q", "k", "v", "b", "a", "g", "o"):
                    t[k] = mat(p + "mix." + k)
                for k in ("q", "k", "v"):
                    t[k + "_conv"] = up.mat32(f"{p}mix.{k}.conv")
                t["a_log"], t["dt_bias"], t["out_norm"] = vec(p + "mix.A_log"), vec(p + "mix.dt_bias"), vec(p + "mix.norm")
            else:
                lc.window, lc.scale = m["mask"]["size"], m["scale"]
                lc.kv_from = -1 if m.get("kv_from") is None else m["kv_from"]
                t["q"], t["o"] = mat(p + "mix.q"), mat(p + "mix.o")
                t["q_norm"], t["r1"], t["r2"] = vec(p + "mix.q.norm"), vec(p + "mix.r1"), vec(p + "mix.r2")
                if lc.kv_from < 0:
                    t["k"], t["v"], t["k_norm"] = mat(p + "mix.k"), mat(p + "mix.v"), vec(p + "mix.k.norm")
            lc.has_mlp = int(mlp is not None)
            if mlp:
                r = mlp["router"]
                lc.experts, lc.top, lc.groups, lc.keep_groups, lc.expert_ff = r["experts"], r["top"], r["groups"]["count"], r["groups"]["keep"], mlp["expert"]["ff"]
                lc.shared_ff = mlp["shared"]["ff"] if mlp["shared"] else 0
                t["norm2"] = vec(p + "norm2")
                t["router"] = up.mat32(p + "mlp.router")
                t["correction"] = vec(p + "mlp.correction")
                for part, key in (("gate", "e_gate"), ("up", "e_up"), ("down", "e_down")):
                    t[key] = stack([f"{p}mlp.e{e}.{part}" for e in range(r["experts"])])
                if mlp["shared"]:
                    for part in ("gate", "up", "down"):
                        t["s_" + part] = mat(f"{p}mlp.shared.{part}")
            for k, v in t.items():
                setattr(lws[i], k, handle_of(v))
                self.tensors[f"{p}{k}"] = v                                  # keep alive
        cc = capi.czr_config(len(c["layers"]), c["width"], c["vocab"], c["norm"]["eps"], int(chunk))
        h = C.c_void_p()
        rc = device.lib.czr_runner_create(device.handle, C.byref(cc), lcs, lws, self.tensors["embed"].buf.handle, self.tensors["final.norm"].buf.handle,
                                          self.tensors["head"].buf.handle, C.byref(h))
        if rc != capi.CC_OK:
            raise (TensorError if rc == capi.CC_ERR_TENSOR else CudaError)(f"czr_runner_create failed [{rc}]: {device.lib.czr_last_create_error().decode()}")
        self.handle = h
        self.vocab = c["vocab"]
        self._keep = (lcs, lws)


def load(path: str, device: CudaTensorDevice, dtype: str = "bfloat16", chunk: int = 0) -> ZatoraxModel:
    """path: a folder with config.json and model.safetensors"""
    with open(os.path.join(path, "config.json")) as f:
        conf = json.load(f)
    return ZatoraxModel(device, conf, read_safetensors(os.path.join(path, "model.safetensors")), dtype, chunk)
