"""The Python handle every multi-sequence model of this package shares (include/crabml_seqrunner.h): sequence slots, the step
function, greedy generation.  A family's class (zatorax.ZatoraxModel, meresun.MeresunModel) uploads its weights, creates its runner
and sets `self.handle`, `self.device`, `self.vocab`; everything a server calls afterwards is here.  `Uploader` holds the rules by
which a family's tensors reach the device."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi
from .capi import CudaError, TensorError
from .safetensors import bf16_to_f32, f32_to_bf16
from .tensor import CudaTensor


class SeqModel:
    handle = None

    def _check(self, rc):
        if rc == capi.CC_OK:
            return
        msg = self.device.lib.csr_runner_last_error(self.handle).decode()
        raise (TensorError if rc == capi.CC_ERR_TENSOR else CudaError)(msg)

    def open(self) -> int:
        s = C.c_int32(-1)
        self._check(self.device.lib.csr_seq_open(self.handle, C.byref(s)))
        return int(s.value)

    def close_seq(self, slot: int):
        self._check(self.device.lib.csr_seq_close(self.handle, int(slot)))

    def seq_len(self, slot: int) -> int:
        return int(self.device.lib.csr_seq_len(self.handle, int(slot)))

    def stats(self) -> dict:
        a = (C.c_int64 * 3)()
        self._check(self.device.lib.csr_runner_stats(self.handle, a))
        return {"slots": int(a[0]), "live": int(a[1]), "state_bytes_per_slot": int(a[2])}

    def step(self, slot: int, tokens, want=()) -> np.ndarray:
        """feeds the sequence's next tokens; -> logits [len(want), vocab] of the wanted places among them"""
        toks = (C.c_int64 * len(tokens))(*[int(t) for t in tokens])
        w = (C.c_int32 * max(1, len(want)))(*[int(i) for i in want])
        out = np.zeros((len(want), self.vocab), np.float32)
        self._check(self.device.lib.csr_runner_step(self.handle, int(slot), toks, len(tokens), w, len(want), out.ctypes.data_as(C.c_void_p) if len(want) else None))
        return out

    def generate_greedy(self, slot: int, prompt, steps: int, eos: int = -1):
        p = (C.c_int64 * len(prompt))(*[int(t) for t in prompt])
        out = (C.c_int64 * max(1, steps))()
        n = C.c_int32(0)
        self._check(self.device.lib.csr_runner_generate_greedy(self.handle, int(slot), p, len(prompt), steps, eos, out, C.byref(n)))
        return [int(out[i]) for i in range(n.value)]

    def close(self):
        if getattr(self, "handle", None):
            self.device.lib.csr_runner_destroy(self.handle)
            self.handle = None


class Uploader:
    """weights: {name: float32 ndarray}, or the pair safetensors.read_safetensors returns (bfloat16 tensors as bit patterns).
    dtype "bfloat16": the matrices of dense products stay bfloat16 on the device; "float32": they are widened.  Everything else
    (norm weights, biases, tables, anything that enters 32-bit arithmetic directly) is float32 in both modes."""

    def __init__(self, device, weights, dtype):
        if dtype not in ("bfloat16", "float32"):
            raise TensorError(f"dtype must be bfloat16 or float32, not {dtype!r}")
        self.device, self.dtype, self.bf16_names = device, dtype, set()
        if isinstance(weights, tuple):
            weights, self.bf16_names = weights
        self.weights = weights

    def check(self, want: dict):
        """want: name -> shape of every tensor the config implies; a missing or misshaped one is refused before anything is uploaded"""
        missing = [n for n in want if n not in self.weights]
        if missing:
            raise TensorError(f"model is missing {len(missing)} tensors, first: {missing[0]}")
        for n, shape in want.items():
            if list(np.asarray(self.weights[n]).shape) != list(shape):
                raise TensorError(f"tensor {n}: shape {list(np.asarray(self.weights[n]).shape)} in the file, {list(shape)} by the config")

    def f32(self, name) -> np.ndarray:
        a = self.weights[name]
        return bf16_to_f32(np.asarray(a)).reshape(np.shape(a)) if name in self.bf16_names else np.asarray(a, np.float32)

    def table(self, a32, shape=None) -> CudaTensor:
        a32 = np.ascontiguousarray(a32, np.float32)
        return CudaTensor.from_cpu(a32, list(shape if shape is not None else a32.shape), capi.F32, self.device)

    def vec(self, name) -> CudaTensor:
        a = self.f32(name).reshape(-1)
        return self.table(a, [a.size])

    def mat32(self, name) -> CudaTensor:
        return self.table(self.f32(name))

    def _mat_from(self, a32, bits16) -> CudaTensor:
        shape = list(a32.shape if a32 is not None else bits16.shape)
        if self.dtype == "float32":
            return self.table(a32 if a32 is not None else bf16_to_f32(bits16).reshape(shape), shape)
        return CudaTensor.from_cpu(np.ascontiguousarray(bits16 if bits16 is not None else f32_to_bf16(a32).reshape(shape)), shape, capi.BF16, self.device)

    def mat(self, name) -> CudaTensor:
        a = self.weights[name]
        return self._mat_from(None, np.asarray(a)) if name in self.bf16_names else self._mat_from(np.asarray(a, np.float32), None)

    def stack(self, names) -> CudaTensor:
        """the named matrices one under the other (expert-major stacks)"""
        if all(n in self.bf16_names for n in names):
            return self._mat_from(None, np.concatenate([np.asarray(self.weights[n]) for n in names], 0))
        return self._mat_from(np.concatenate([self.f32(n) for n in names], 0), None)


def handle_of(t: CudaTensor):
    h = t.buf.handle
    return h.value if hasattr(h, "value") else h
