"""GPU quantiser (ti_b200_quantize_f16) against the reference's golden vectors and the CPU oracle: bit-exact."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
GOLDEN = json.loads((Path(__file__).parent / "golden" / "quant_golden.json").read_text())


@pytest.fixture(scope="module")
def ops():
    from tinyinfer_b200.native_ops import NativeOps
    return NativeOps()


def device_half(bits, rows, cols):
    return torch.from_numpy(np.array(bits, np.uint16).view(np.float16).reshape(rows, cols)).cuda()


@pytest.mark.parametrize("case", GOLDEN["cases"], ids=[c["name"] for c in GOLDEN["cases"]])
def test_golden_cases(ops, case):
    q, scales = ops.quantize_int8(device_half(case["w_bits"], case["rows"], case["cols"]))
    assert q.cpu().numpy().ravel().tolist() == case["q"]
    assert scales.cpu().numpy().view(np.uint32).tolist() == case["scale_bits"]
    assert int(q.min()) >= -127                                   # -128 is never produced


def test_all_finite_half_sweep_digest(ops):
    sweep = GOLDEN["all_finite_half_sweep"]
    bits = [i for i in range(65536) if i & 0x7c00 != 0x7c00]
    q, scales = ops.quantize_int8(device_half(bits, len(bits) // sweep["columns"], sweep["columns"]))
    assert hashlib.sha256(q.cpu().numpy().tobytes()).hexdigest() == sweep["q_sha256"]
    assert hashlib.sha256(scales.cpu().numpy().tobytes()).hexdigest() == sweep["scales_sha256"]


def test_model_sized_matrix_matches_oracle_and_feeds_the_gemm(ops):
    from oracle import ti_oracle as orc
    torch.manual_seed(7)
    w = (torch.randn((768, 2304), device="cuda") * 0.02).half()
    q, scales = ops.quantize_int8(w)
    want_q, want_s = orc.quantize(w.cpu().numpy())
    assert np.array_equal(q.cpu().numpy(), want_q) and np.array_equal(scales.cpu().numpy(), want_s)
    a = torch.randn((8, 768), device="cuda").half()
    out = ops.gemm_int8(a, q, scales)                             # the quantised matrix goes straight into the GEMM
    ref = a.float() @ (q.float() * scales).half().float()
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=1e-2)


def test_nonfinite_input_is_rejected(ops):
    w = torch.zeros((4, 8), device="cuda", dtype=torch.float16)
    w[2, 3] = float("inf")
    with pytest.raises(ValueError):
        ops.quantize_int8(w)
    w[2, 3] = float("nan")
    with pytest.raises(ValueError):
        ops.quantize_int8(w)
