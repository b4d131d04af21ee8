"""TEST / BASELINE INFRASTRUCTURE, NOT PRODUCT: a CPU decode harness for timing.

The reference ships no CPU GPT-2 runtime (llm/src/runtime.cu is CUDA only; the server's
`--model cpu` is a token counter, server/include/model.hpp:70-75).  What it ships for the CPU
are three FP32 OpenMP kernels -- ti_cpu_gemm / ti_cpu_layernorm / ti_cpu_softmax
(backend/runtime.cpp:6-8, kernels/src/cpu/*.cpp) -- and the host codec.  This module COMPOSES
those reference functions (from oracle/_ref, built by oracle/Makefile) into the decode sequence
of llm/src/runtime.cu:141-155,163-165 so the benchmark can print a CPU number beside the GPU one:

  * every INT8 matrix is dequantised once with the reference ti_host_dequantize_i8 -> fp32;
  * per step: embedding add (numpy), ti_cpu_layernorm, ti_cpu_gemm (M = batch) + bias,
    attention per request over its fp32 KV history (numpy dot products + ti_cpu_softmax),
    tanh-GELU and residual adds (numpy), fp32 lm_head by ti_cpu_gemm, argmax (lowest id on ties).

`kind` is "reference" when the reference kernels are used, "port" when oracle/_ref is absent
and the same sequence runs on numpy matmul / the C oracle instead.  Activations are fp32
throughout (the reference CPU kernels are fp32), so logits agree with the GPU path only to
about 1e-2; that is checked in tests/, the timing is what this module is for.
"""
from __future__ import annotations

import ctypes as C
import os
import time
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"


class CpuKernels:
    def __init__(self):
        self.kind = "port"
        self.cpu = self.codec = None
        if (REF / "libtinyinfer_cpu.so").exists() and (REF / "libtinyinfer_host_codec.so").exists():
            self.cpu = C.CDLL(str(REF / "libtinyinfer_cpu.so"))
            self.codec = C.CDLL(str(REF / "libtinyinfer_host_codec.so"))
            p, i, f, z = C.c_void_p, C.c_int, C.c_float, C.c_size_t
            self.cpu.ti_cpu_gemm.argtypes, self.cpu.ti_cpu_gemm.restype = [p, p, p, i, i, i], None      # (a, b, y, m, k, n)
            self.cpu.ti_cpu_softmax.argtypes, self.cpu.ti_cpu_softmax.restype = [p, p, i, i], None
            self.cpu.ti_cpu_layernorm.argtypes, self.cpu.ti_cpu_layernorm.restype = [p, p, p, p, i, i, f], None
            self.codec.ti_host_dequantize_i8.argtypes, self.codec.ti_host_dequantize_i8.restype = [p, z, z, p, z, p, z], C.c_int
            self.kind = "reference"

    def dequantize(self, q, scales):
        q, scales = np.ascontiguousarray(q), np.ascontiguousarray(scales)
        if self.codec is None:
            return (q.astype(np.float32) * scales).astype(np.float16).astype(np.float32)
        out = np.empty(q.shape, np.float16)
        if self.codec.ti_host_dequantize_i8(q.ctypes.data, q.size, q.shape[1], scales.ctypes.data, scales.size, out.ctypes.data, out.size):
            raise ValueError("reference codec rejected the weights")
        return out.astype(np.float32)

    def gemm(self, a, w):
        a = np.ascontiguousarray(a, np.float32)
        if self.cpu is None:
            return a @ w
        y = np.empty((a.shape[0], w.shape[1]), np.float32)
        self.cpu.ti_cpu_gemm(a.ctypes.data, w.ctypes.data, y.ctypes.data, a.shape[0], a.shape[1], w.shape[1])
        return y

    def layernorm(self, x, g, b):
        x = np.ascontiguousarray(x, np.float32)
        if self.cpu is None:
            mu = x.mean(-1, keepdims=True)
            return (x - mu) / np.sqrt(x.var(-1, keepdims=True) + 1e-5) * g + b
        y = np.empty_like(x)
        self.cpu.ti_cpu_layernorm(x.ctypes.data, g.ctypes.data, b.ctypes.data, y.ctypes.data, x.shape[0], x.shape[1], 1e-5)
        return y

    def softmax(self, x):
        x = np.ascontiguousarray(x, np.float32)
        if self.cpu is None:
            e = np.exp(x - x.max(-1, keepdims=True))
            return e / e.sum(-1, keepdims=True)
        y = np.empty_like(x)
        self.cpu.ti_cpu_softmax(x.ctypes.data, y.ctypes.data, x.shape[0], x.shape[1])
        return y


class CpuDecoder:
    """fp32 GPT-2 decode over per-request KV histories, one token per request per step."""

    def __init__(self, tensors, arch, threads=None):
        if threads:
            os.environ["OMP_NUM_THREADS"] = str(threads)
        self.k = CpuKernels()
        if threads:
            # an OpenMP runtime that is already loaded has read the environment; tell it directly as well
            try:
                C.CDLL("libgomp.so.1").omp_set_num_threads(int(threads))
            except OSError:
                pass
        self.arch = arch
        self.H, self.nh, self.L = arch["hidden"], arch["heads"], arch["layers"]
        self.d = self.H // self.nh
        f32 = lambda name: np.ascontiguousarray(tensors[name], np.float32)
        def linear(name, bias=True):
            if name + ".weight.scales" in tensors:
                w = self.k.dequantize(tensors[name + ".weight"], tensors[name + ".weight.scales"])
            else:
                w = f32(name + ".weight")
            return w, (f32(name + ".bias") if bias else None)
        self.wte, self.wpe = f32("transformer.wte.weight"), f32("transformer.wpe.weight")
        self.lnf = (f32("transformer.ln_f.weight"), f32("transformer.ln_f.bias"))
        self.blocks = []
        for layer in range(self.L):
            p = f"transformer.h.{layer}."
            self.blocks.append({"ln1": (f32(p + "ln_1.weight"), f32(p + "ln_1.bias")), "ln2": (f32(p + "ln_2.weight"), f32(p + "ln_2.bias")),
                                "qkv": linear(p + "attn.c_attn"), "proj": linear(p + "attn.c_proj"),
                                "fc": linear(p + "mlp.c_fc"), "proj2": linear(p + "mlp.c_proj")})
        self.head = linear("lm_head", bias=False)[0]
        self.kcache, self.vcache, self.lengths = [], [], []

    def start(self, lengths, capacity, rng=None, histories=None):
        """Per-request caches [layer][head][capacity][d].  Either filled with random values up to
        `lengths` (timing: the prefill is skipped) or empty (lengths 0) to be filled by step()."""
        self.lengths = list(lengths)
        b = len(lengths)
        shape = (b, self.L, self.nh, capacity, self.d)
        if rng is not None:
            self.kcache = rng.standard_normal(shape, dtype=np.float32) * 0.5
            self.vcache = rng.standard_normal(shape, dtype=np.float32)
        else:
            self.kcache, self.vcache = np.zeros(shape, np.float32), np.zeros(shape, np.float32)

    def step(self, ids):
        """Appends one token per request; returns (next ids, fp32 logits [B, vocab])."""
        k, H, nh, d = self.k, self.H, self.nh, self.d
        b = len(ids)
        pos = np.array(self.lengths)
        x = self.wte[np.asarray(ids)] + self.wpe[pos]
        for layer, blk in enumerate(self.blocks):
            qkv = k.gemm(k.layernorm(x, *blk["ln1"]), blk["qkv"][0]) + blk["qkv"][1]
            q, kk, vv = qkv[:, :H].reshape(b, nh, d), qkv[:, H:2 * H].reshape(b, nh, d), qkv[:, 2 * H:].reshape(b, nh, d)
            attn = np.empty((b, nh, d), np.float32)
            for r in range(b):
                t = self.lengths[r]
                self.kcache[r, layer, :, t], self.vcache[r, layer, :, t] = kk[r], vv[r]
                keys, vals = self.kcache[r, layer, :, :t + 1], self.vcache[r, layer, :, :t + 1]
                scores = np.einsum("hd,htd->ht", q[r], keys) * (1.0 / np.sqrt(d))
                attn[r] = np.einsum("ht,htd->hd", k.softmax(scores), vals)
            res = x + k.gemm(attn.reshape(b, H), blk["proj"][0]) + blk["proj"][1]
            h = k.gemm(k.layernorm(res, *blk["ln2"]), blk["fc"][0]) + blk["fc"][1]
            h = 0.5 * h * (1.0 + np.tanh(0.7978845608028654 * (h + 0.044715 * h * h * h)))
            x = res + k.gemm(h.astype(np.float32), blk["proj2"][0]) + blk["proj2"][1]
        logits = k.gemm(k.layernorm(x, *self.lnf), self.head)
        self.lengths = [t + 1 for t in self.lengths]
        return logits.argmax(-1).tolist(), logits


def time_decode(tensors, arch, lengths, steps, warmup=1, seed=0, threads=None):
    """Seconds per decode step of a batch whose requests hold `lengths` cached positions (random
    KV contents: the prefill is not part of the sample).  Returns a dict for the benchmark."""
    rng = np.random.default_rng(seed)
    dec = CpuDecoder(tensors, arch, threads)
    capacity = max(lengths) + warmup + steps + 1
    dec.start(lengths, capacity, rng=rng)
    ids = rng.integers(0, arch["vocab"], len(lengths)).tolist()
    for _ in range(warmup):
        ids, _ = dec.step(ids)
    t0 = time.perf_counter()
    for _ in range(steps):
        ids, _ = dec.step(ids)
    elapsed = time.perf_counter() - t0
    cores = int(os.environ.get("OMP_NUM_THREADS") or os.cpu_count() or 1)
    return {"seconds_per_step": elapsed / steps, "tokens_per_s": len(lengths) * steps / elapsed, "kind": dec.k.kind,
            "cores": cores, "steps": steps}
