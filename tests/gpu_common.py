"""Helpers shared by the GPU parity tests: library handles, tolerances, seeded inputs."""
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
REF_DIR = ROOT / "oracle" / "_ref"

# Operator tolerance of the reference's own gate (bench/v2/configs/kernels.json:15-16).
ATOL = RTOL = 0.02
# Model-level gates: logits within max-abs 2e-2 / rel 1e-2 of the reference runtime.
LOGIT_ATOL, LOGIT_RTOL = 2e-2, 1e-2


def our_ops():
    from tinyinfer_b200.native_ops import NativeOps
    return NativeOps()


def reference_ops():
    """The reference's own CUDA operators (compiled for sm_100a by oracle/Makefile) behind the same wrapper."""
    path = REF_DIR / "libtinyinfer_backend.so"
    if not path.exists():
        pytest.skip("reference build oracle/_ref is absent")
    from tinyinfer_b200.native_ops import NativeOps
    return NativeOps(path)


def close(actual, expected, atol=ATOL, rtol=RTOL):
    import torch
    torch.testing.assert_close(actual.float().cpu(), torch.as_tensor(np.asarray(expected, dtype=np.float32)) if not hasattr(expected, "float")
                               else expected.float().cpu(), atol=atol, rtol=rtol)


def int8_case(torch, m, n, k, seed, scale_lo=1e-3, scale_hi=2e-2):
    """Operator-sweep inputs: A ~ N(0,1) fp16, W uniform int8 in [-127,127], scales uniform in
    [scale_lo, scale_hi] rounded to fp16 and stored as fp32, bias ~ N(0,0.1) fp16."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.randn((m, k), generator=g).half().cuda()
    w = torch.randint(-127, 128, (k, n), generator=g, dtype=torch.int8).cuda()
    s = (torch.rand(n, generator=g) * (scale_hi - scale_lo) + scale_lo).half().float().cuda()
    bias = (torch.randn(n, generator=g) * 0.1).half().cuda()
    return a, w, s, bias
