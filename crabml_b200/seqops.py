"""Python handles on the sequence-mixing / routing ops of include/crabml_seqops.h (ctypes over the C ABI; used by the tests and
by anyone who builds a model out of these mechanisms in Python).  Arguments are CudaTensors; outputs are new CudaTensors."""
from __future__ import annotations

import ctypes as C

from . import capi
from .tensor import CudaTensor, TensorStrider, _Buf


def _v(t):
    return C.byref(t._view()) if t is not None else None


def _new(dev, handle, shape):
    return CudaTensor(_Buf(dev, handle), TensorStrider(shape), dev)


def tensor_zero(x):
    x.device.check(x.device.lib.cc_tensor_zero(x.device.handle, _v(x)))


def rms_norm_gain(dst, y, gain, eps, accumulate=False):
    dst.device.check(dst.device.lib.cc_rms_norm_gain(dst.device.handle, _v(dst), _v(y), _v(gain), float(eps), int(accumulate)))
    return dst


def gated_head_rms_norm(x, gate, w, head_size, eps, gate_act=capi.ACT_SILU):
    x.device.check(x.device.lib.cc_gated_head_rms_norm(x.device.handle, _v(x), _v(gate), _v(w), int(head_size), float(eps), int(gate_act)))
    return x


def glu_inplace(gate, up, act=capi.ACT_SILU):
    gate.device.check(gate.device.lib.cc_glu_inplace(gate.device.handle, _v(gate), _v(up), int(act)))
    return gate


def short_conv(x, w, tail, act=capi.ACT_SILU, head_size=0, unit_norm=False, unit_eps=1e-6, unit_scale=1.0):
    h = C.c_void_p()
    x.device.check(x.device.lib.cc_short_conv(x.device.handle, _v(x), _v(w), _v(tail), int(act), int(head_size), int(unit_norm), float(unit_eps),
                                              float(unit_scale), C.byref(h)))
    return _new(x.device, h, x.shape())


def gated_delta_rule(q, k, v, a, b, a_log, dt_bias, state, n_heads, n_kv, dk, dv):
    h = C.c_void_p()
    q.device.check(q.device.lib.cc_gated_delta_rule(q.device.handle, _v(q), _v(k), _v(v), _v(a), _v(b), _v(a_log), _v(dt_bias), _v(state), n_heads, n_kv, dk, dv,
                                                    C.byref(h)))
    return _new(q.device, h, [q.shape()[0], n_heads * dv])


def kv_ring_append(kring, vring, k, v, k_norm_w, eps, pos0, n_kv, dk, dv):
    kring.device.check(kring.device.lib.cc_kv_ring_append(kring.device.handle, _v(kring), _v(vring), _v(k), _v(v), _v(k_norm_w), float(eps), int(pos0), n_kv, dk, dv))


def window_attention(q, q_norm_w, eps, kring, vring, pos0, n_heads, n_kv, dk, dv, window, scale, r1=None, r2=None):
    h = C.c_void_p()
    q.device.check(q.device.lib.cc_window_attention(q.device.handle, _v(q), _v(q_norm_w), float(eps), _v(kring), _v(vring), int(pos0), n_heads, n_kv, dk, dv,
                                                    int(window), float(scale), _v(r1), _v(r2), C.byref(h)))
    return _new(q.device, h, [q.shape()[0], n_heads * dv])


def moe_route(x, router_w, correction, top, n_groups=1, keep_groups=1, renormalise=False):
    """-> (ids I32 [T, top] as a CudaTensor, weights F32 [T, top])"""
    hi, hw = C.c_void_p(), C.c_void_p()
    x.device.check(x.device.lib.cc_moe_route(x.device.handle, _v(x), _v(router_w), _v(correction), int(top), int(n_groups), int(keep_groups), int(renormalise),
                                             C.byref(hi), C.byref(hw)))
    T = x.shape()[0]
    return _new(x.device, hi, [T, top]), _new(x.device, hw, [T, top])


def moe_experts(x, ids, weights, w_gate, w_up, w_down, n_experts, ff, act=capi.ACT_SILU):
    h = C.c_void_p()
    x.device.check(x.device.lib.cc_moe_experts(x.device.handle, _v(x), _v(ids), _v(weights), _v(w_gate), _v(w_up), _v(w_down), int(n_experts), int(ff), int(act),
                                               C.byref(h)))
    return _new(x.device, h, list(x.shape()))
