"""Pins oracle/ti_oracle.c to the reference: its own known-answer tests and outputs of the
reference's quantiser/codec stored in tests/golden/quant_golden.json."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import ti_oracle as orc

GOLDEN = json.loads((Path(__file__).parent / "golden" / "quant_golden.json").read_text())


def h(values):
    return np.asarray(values, np.float16)


# Known answers of the reference's llm/tests/test_contracts.py:22-48.
def test_kat_output_axis_zero_and_signed_channels():
    q, s = orc.quantize(h([[0, 127, -254], [0, 0, 127], [0, -127, 0]]))
    assert s.tolist() == [1.0, 1.0, 2.0]
    assert q.tolist() == [[0, 127, -127], [0, 0, 64], [0, -127, 0]]
    assert orc.dequantize(q, s).astype(np.float64).tolist() == [[0, 127, -254], [0, 0, 128], [0, -127, 0]]


def test_kat_ties_to_even_and_clipping():
    q, s = orc.quantize(h([[127], [.5], [1.5], [2.5], [-.5], [-1.5], [-2.5], [-127]]))
    assert s.tolist() == [1.0]
    assert q.ravel().tolist() == [127, 0, 2, 2, 0, -2, -2, -127]


def test_kat_dequant_rounds_back_to_fp16():
    rows = h([[.00123, -1.75], [-.00345, .3]])
    q, s = orc.quantize(rows)
    back = orc.dequantize(q, s)
    assert np.abs(back.astype(np.float64) - rows.astype(np.float64)).max() < .02


# Hand matrices of the reference's fuzz/check_codec.py:21-32 (dequantised bytes).
def test_kat_codec_dequant_matrix():
    q = np.array([[-127, -3, -1, 0, 1, 3, 127], [1, 2, 3, 4, 5, 6, 7]], np.int8)
    s = np.array([2 ** -24, 0.5, 1., 1., 1., 2., np.float32(65504 / 127)], np.float32)
    want = (q.astype(np.float32) * s).astype(np.float16)   # fp32 product, one RN-even narrowing
    assert orc.dequantize(q, s).view(np.uint16).tolist() == want.view(np.uint16).tolist()


@pytest.mark.parametrize("qv,sv", [(-128, 1.), (127, 1e10), (1, 0.), (1, float("nan")), (1, float("inf"))])
def test_invalid_dequant_rejected(qv, sv):
    with pytest.raises(ValueError):
        orc.dequantize(np.array([[qv]], np.int8), np.array([sv], np.float32))


def test_nonfinite_quant_rejected():
    with pytest.raises(ValueError):
        orc.quantize(np.array([[1.0], [np.inf]], np.float16))


@pytest.mark.parametrize("case", GOLDEN["cases"], ids=lambda c: c["name"])
def test_reference_generated_vectors(case):
    w = np.array(case["w_bits"], np.uint16).view(np.float16).reshape(case["rows"], case["cols"])
    q, s = orc.quantize(w)
    assert q.ravel().tolist() == case["q"]
    assert s.view(np.uint32).tolist() == case["scale_bits"]
    assert orc.dequantize(q, s).view(np.uint16).ravel().tolist() == case["dequant_bits"]


def test_all_finite_half_sweep_digest():
    sweep = GOLDEN["all_finite_half_sweep"]
    bits = np.array([i for i in range(65536) if i & 0x7c00 != 0x7c00], np.uint16)
    w = bits.view(np.float16).reshape(-1, sweep["columns"])
    q, s = orc.quantize(w)
    assert hashlib.sha256(q.tobytes()).hexdigest() == sweep["q_sha256"]
    assert hashlib.sha256(s.tobytes()).hexdigest() == sweep["scales_sha256"]
    assert hashlib.sha256(orc.dequantize(q, s).tobytes()).hexdigest() == sweep["dequant_sha256"]


def test_half_conversion_matches_numpy_everywhere():
    lib = orc.lib()
    bits = np.arange(65536, dtype=np.uint16)
    finite = bits[(bits & 0x7c00) != 0x7c00]
    for b in finite[::7]:
        assert np.float32(lib.orc_h2f(int(b))) == np.float32(np.uint16(b).view(np.float16))
    rng = np.random.default_rng(3)
    values = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-6, 2000), rng.normal(0, 3e4, 2000),
                             [65519.9, 65520.0, -65520.0, 2 ** -25, 2 ** -24 * 1.5, 0.0]]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = values.astype(np.float16).view(np.uint16)
    got = np.array([lib.orc_f2h(float(v)) for v in values], np.uint16)
    assert (got == want).all()


def test_operator_restatements_against_float64():
    rng = np.random.default_rng(5)
    a = rng.normal(0, 1, (5, 48)).astype(np.float16)
    w = rng.normal(0, 0.05, (48, 19)).astype(np.float16)
    bias = rng.normal(0, 0.1, 19).astype(np.float16)
    q, s = orc.quantize(w)
    deq = orc.dequantize(q, s).astype(np.float64)
    want = a.astype(np.float64) @ deq + bias.astype(np.float64)
    np.testing.assert_allclose(orc.gemm_int8(a, q, s, bias, out_fp32=True), want, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(orc.gemm_int8(a, q, s, bias).astype(np.float64), want, rtol=2e-3, atol=2e-3)
    x = rng.normal(0, 1, (3, 257)).astype(np.float16)
    g, b = rng.normal(1, 0.1, 257).astype(np.float16), rng.normal(0, 0.1, 257).astype(np.float16)
    xf = x.astype(np.float64)
    ln = (xf - xf.mean(-1, keepdims=True)) / np.sqrt(xf.var(-1, keepdims=True) + 1e-5) * g + b
    np.testing.assert_allclose(orc.layernorm(x, g, b).astype(np.float64), ln, rtol=2e-3, atol=2e-3)
    gelu = 0.5 * xf * (1 + np.tanh(0.7978845608028654 * (xf + 0.044715 * xf ** 3)))
    np.testing.assert_allclose(orc.gelu_new(x).astype(np.float64), gelu, rtol=2e-3, atol=2e-3)
    e = np.exp(xf - xf.max(-1, keepdims=True))
    np.testing.assert_allclose(orc.softmax(x).astype(np.float64), e / e.sum(-1, keepdims=True), rtol=2e-3, atol=1e-4)


def test_attention_masks_and_zero_rows():
    # Ragged / masked cases of bench/v2/kernels/correctness.py:77-82, checked against float64 softmax.
    rng = np.random.default_rng(7)
    for nq, nk, ql, kl, off, causal in ((17, 33, [17, 11], [33, 0], [0, 0], True), (1, 31, [1, 1], [31, 19], [30, 18], True),
                                        (5, 19, [5, 0], [13, 19], [7, 0], True), (9, 11, [7, 9], [11, 8], [0, 0], False)):
        q = (rng.normal(0, .5, (2, 2, nq, 64))).astype(np.float16)
        k = (rng.normal(0, .5, (2, 2, nk, 64))).astype(np.float16)
        v = rng.normal(0, 1, (2, 2, nk, 64)).astype(np.float16)
        out = orc.attention(q, k, v, ql, kl, off, causal).astype(np.float64)
        qi, ki = np.arange(nq)[None, :, None], np.arange(nk)[None, None, :]
        mask = (qi < np.array(ql)[:, None, None]) & (ki < np.array(kl)[:, None, None])
        if causal:
            mask &= ki <= np.array(off)[:, None, None] + qi
        s = np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k.astype(np.float64)) / 8.0
        s = np.where(mask[:, None], s, -np.inf)
        with np.errstate(invalid="ignore"):
            p = np.exp(s - s.max(-1, keepdims=True))
            p = np.nan_to_num(p / p.sum(-1, keepdims=True))
        want = np.einsum("bhqk,bhkd->bhqd", p, v.astype(np.float64))
        np.testing.assert_allclose(out, want, rtol=2e-3, atol=2e-3)
        dead = ~mask.any(-1)
        assert not out[np.broadcast_to(dead[:, None, :, None], out.shape)].any()


def test_argmax_lowest_index_on_ties():
    logits = np.array([[1, 5, 5, 2], [7, 7, 7, 7], [0, -1, 3, 3]], np.float32)
    assert orc.argmax(logits).tolist() == [1, 0, 2]
