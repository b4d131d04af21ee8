"""TEST INFRASTRUCTURE, NOT PRODUCT: numpy/ctypes front end of oracle/ti_oracle.c.

The C file restates the reference's operators; this module loads it and composes the
operators into the reference's GPT-2 forward sequence (llm/src/runtime.cu:135-168) so the
CUDA runtime can be checked logits-for-logits and token-for-token on a CPU.  Only tests/,
the smoke check and the benchmark's cpu_baseline leg import this module.

fp16 arrays are numpy float16 (same bits as the uint16 the C side takes).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_build" / "libti_oracle.so"


def build(force=False):
    """Compile ti_oracle.c (a second or two with gcc); returns the library path."""
    source = HERE / "ti_oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["make", "-s", "-C", str(HERE), "oracle"], check=True)
    return LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
        p, z, i, i64, f = C.c_void_p, C.c_size_t, C.c_int, C.c_int64, C.c_float
        for name, args, res in (
            ("orc_quantize_f16", [p, z, z, p, p], i), ("orc_dequantize_i8", [p, z, z, p, p], i),
            ("orc_gemm", [p, p, p, p, p, p, i, i, i, i], None),
            ("orc_layernorm_f16", [p, p, p, p, i, i, f], None), ("orc_gelu_new_f16", [p, p, i64], None),
            ("orc_softmax_f16", [p, p, i, i], None),
            ("orc_attention_f16", [p, p, p, p, p, p, p, i, i, i, i, i, i], None),
            ("orc_embed_f16", [p, p, p, p, p, i, i], None), ("orc_add_f16", [p, p, p, i64], None),
            ("orc_argmax_f32", [p, p, i, i], None), ("orc_nll_f32", [p, p, p, i, i], None),
            ("orc_h2f", [C.c_uint16], f), ("orc_f2h", [f], C.c_uint16),
        ):
            fn = getattr(_lib, name)
            fn.argtypes, fn.restype = args, res
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def quantize(w16):
    """[K,N] float16 -> (int8 [K,N], float32 [N]); raises ValueError like the reference."""
    w16 = _c(w16, np.float16)
    q = np.empty(w16.shape, np.int8)
    s = np.empty(w16.shape[1], np.float32)
    if lib().orc_quantize_f16(_ptr(w16), w16.shape[0], w16.shape[1], _ptr(q), _ptr(s)):
        raise ValueError("quantize rejected input")
    return q, s


def dequantize(q, scales):
    q, scales = _c(q, np.int8), _c(scales, np.float32)
    out = np.empty(q.shape, np.float16)
    if lib().orc_dequantize_i8(_ptr(q), q.shape[0], q.shape[1], _ptr(scales), _ptr(out)):
        raise ValueError("dequantize rejected input")
    return out


def gemm_int8(a, q, scales, bias=None, out_fp32=False):
    a, q, scales = _c(a, np.float16), _c(q, np.int8), _c(scales, np.float32)
    bias = None if bias is None else _c(bias, np.float16)
    m, k = a.shape
    n = q.shape[1]
    out = np.empty((m, n), np.float32 if out_fp32 else np.float16)
    lib().orc_gemm(_ptr(a), _ptr(q), _ptr(scales), None, _ptr(bias), _ptr(out), m, n, k, int(out_fp32))
    return out


def gemm_f16(a, w, bias=None, out_fp32=False):
    a, w = _c(a, np.float16), _c(w, np.float16)
    bias = None if bias is None else _c(bias, np.float16)
    m, k = a.shape
    n = w.shape[1]
    out = np.empty((m, n), np.float32 if out_fp32 else np.float16)
    lib().orc_gemm(_ptr(a), None, None, _ptr(w), _ptr(bias), _ptr(out), m, n, k, int(out_fp32))
    return out


def layernorm(x, g, b, eps=1e-5):
    x = _c(x, np.float16)
    out = np.empty_like(x)
    cols = x.shape[-1]
    lib().orc_layernorm_f16(_ptr(x), _ptr(_c(g, np.float16)), _ptr(_c(b, np.float16)), _ptr(out), x.size // cols, cols, eps)
    return out


def gelu_new(x):
    x = _c(x, np.float16)
    out = np.empty_like(x)
    lib().orc_gelu_new_f16(_ptr(x), _ptr(out), x.size)
    return out


def softmax(x):
    x = _c(x, np.float16)
    out = np.empty_like(x)
    lib().orc_softmax_f16(_ptr(x), _ptr(out), x.size // x.shape[-1], x.shape[-1])
    return out


def attention(q, k, v, q_lengths, kv_lengths, offsets, causal=True):
    q, k, v = _c(q, np.float16), _c(k, np.float16), _c(v, np.float16)
    b, h, nq, d = q.shape
    out = np.empty_like(q)
    ql, kl, off = (_c(x, np.int32) for x in (q_lengths, kv_lengths, offsets))
    lib().orc_attention_f16(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(ql), _ptr(kl), _ptr(off),
                            b, h, nq, k.shape[2], d, int(causal))
    return out


def add(a, b):
    a, b = _c(a, np.float16), _c(b, np.float16)
    out = np.empty_like(a)
    lib().orc_add_f16(_ptr(a), _ptr(b), _ptr(out), a.size)
    return out


def argmax(logits):
    logits = _c(logits, np.float32)
    out = np.empty(logits.shape[0], np.int32)
    lib().orc_argmax_f32(_ptr(logits), _ptr(out), logits.shape[0], logits.shape[1])
    return out


def nll(logits, targets):
    logits, targets = _c(logits, np.float32), _c(targets, np.int32)
    out = np.empty(logits.shape[0], np.float64)
    lib().orc_nll_f32(_ptr(logits), _ptr(targets), _ptr(out), logits.shape[0], logits.shape[1])
    return out


class Gpt2Oracle:
    """The reference's forward pass, one request at a time, with a per-slot KV history.

    `tensors` maps artifact tensor names to numpy arrays (see tinyinfer_b200.artifact.load):
    int8 weights [in,out] with float32 `.scales`, float16 biases, LayerNorm and embeddings.
    Sequence restated from ti_llm_model::transform / forward, llm/src/runtime.cu:135-168;
    cache semantics from llm/cache_reference.py (per-slot, absolute positions, isolated).
    Works for any (layers, heads, hidden) found in `arch`, so the medium shape runs too.
    """

    def __init__(self, tensors, arch):
        self.t, self.arch = tensors, arch
        self.layers, self.heads, self.hidden = arch["layers"], arch["heads"], arch["hidden"]
        self.d = self.hidden // self.heads
        self.cache = {}

    def reset(self, slot):
        self.cache.pop(slot, None)

    def length(self, slot):
        return 0 if slot not in self.cache else self.cache[slot][0][0].shape[1]

    def _linear(self, x, name, fp32=False, bias=True):
        t = self.t
        b = t[name + ".bias"] if bias else None
        if name + ".weight.scales" in t:
            return gemm_int8(x, t[name + ".weight"], t[name + ".weight.scales"], b, fp32)
        return gemm_f16(x, t[name + ".weight"], b, fp32)

    def forward(self, slot, tokens):
        """Append `tokens` to `slot`; returns fp32 logits [vocab] of the last position."""
        t, H, nh, d = self.t, self.hidden, self.heads, self.d
        start, n = self.length(slot), len(tokens)
        ids = np.asarray(tokens, np.int32)
        pos = np.arange(start, start + n, dtype=np.int32)
        x = np.empty((n, H), np.float16)
        lib().orc_embed_f16(_ptr(ids), _ptr(pos), _ptr(t["transformer.wte.weight"]), _ptr(t["transformer.wpe.weight"]), _ptr(x), n, H)
        if slot not in self.cache:
            self.cache[slot] = [[np.zeros((nh, 0, d), np.float16), np.zeros((nh, 0, d), np.float16)] for _ in range(self.layers)]
        for layer in range(self.layers):
            p = f"transformer.h.{layer}."
            norm = layernorm(x, t[p + "ln_1.weight"], t[p + "ln_1.bias"])
            qkv = self._linear(norm, p + "attn.c_attn")
            q, k, v = (qkv[:, i * H:(i + 1) * H].reshape(n, nh, d).transpose(1, 0, 2) for i in range(3))
            kv = self.cache[slot][layer]
            kv[0] = np.concatenate([kv[0], k], axis=1)
            kv[1] = np.concatenate([kv[1], v], axis=1)
            total = start + n
            attn = attention(q[None], kv[0][None], kv[1][None], [n], [total], [start], True)[0]
            merged = attn.transpose(1, 0, 2).reshape(n, H)
            res = add(x, self._linear(merged, p + "attn.c_proj"))
            norm = layernorm(res, t[p + "ln_2.weight"], t[p + "ln_2.bias"])
            act = gelu_new(self._linear(norm, p + "mlp.c_fc"))
            x = add(res, self._linear(act, p + "mlp.c_proj"))
        last = layernorm(x[-1:], t["transformer.ln_f.weight"], t["transformer.ln_f.bias"])
        return self._linear(last, "lm_head", fp32=True, bias=False)[0]

    def greedy(self, slot, prompt, new_tokens, margins=None):
        """Exactly `new_tokens` greedy ids; the last one is not appended (tinyinfer_llm.h:41-43).
        `margins`, if a list, receives the top-1/top-2 logit gap of every step."""
        self.reset(slot)
        out, tokens = [], list(prompt)
        for _ in range(new_tokens):
            logits = self.forward(slot, tokens)
            nxt = int(argmax(logits[None])[0])
            if margins is not None:
                top2 = np.partition(logits, -2)[-2:]
                margins.append(float(top2[1] - top2[0]))
            out.append(nxt)
            tokens = [nxt]
        return out
