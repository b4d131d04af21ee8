"""GPU parity of the operator ABI: our sm_100a kernels, called through the C ABI, against
(a) the CPU oracle and (b) the reference's own kernels compiled for sm_100a (oracle/_ref).

Cases follow the reference's operator gate (bench/v2/kernels/correctness.py:6-130) and the
operator sweep of the benchmark definition.
"""
import gc

import numpy as np
import pytest

from oracle import ti_oracle as orc
from tests.gpu_common import ATOL, RTOL, close, int8_case, our_ops, reference_ops

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ops():
    return our_ops()


@pytest.fixture(scope="module")
def ref():
    return reference_ops()


def _quantise(b):
    scale = b.float().abs().amax(dim=0).div(127).clamp_min(1e-8)
    quant = (b.float() / scale).round().clamp(-127, 127).to(torch.int8)
    return quant, scale


@pytest.mark.parametrize("config", [0, 4, 7, 11])
@pytest.mark.parametrize("m,n,k", [(1, 7, 3), (17, 33, 19), (65, 67, 63), (128, 128, 128)])
@pytest.mark.parametrize("int8", [False, True])
def test_gemm_gate_cases(ops, m, n, k, config, int8):
    # correctness.py:24-50: odd shapes, zero channel, fp32 and fp16 outputs, every config family
    torch.manual_seed(m * 1000 + n + config)
    a = (torch.randn((m, k), device="cuda") * 0.25).half()
    b = (torch.randn((k, n), device="cuda") * 0.25).half()
    bias = (torch.randn(n, device="cuda") * 0.1).half()
    if int8:
        b[:, 0] = 0
        quant, scale = _quantise(b)
        out32 = ops.gemm_int8(a, quant, scale, bias=bias, config=config, output_dtype=torch.float32)
        out16 = ops.gemm_int8(a, quant, scale, bias=bias, config=config)
        want = orc.gemm_int8(a.cpu().numpy(), quant.cpu().numpy(), scale.cpu().numpy(), bias.cpu().numpy(), out_fp32=True)
    else:
        out32 = ops.gemm(a, b, bias=bias, config=config, output_dtype=torch.float32)
        out16 = ops.gemm(a, b, bias=bias, config=config)
        want = orc.gemm_f16(a.cpu().numpy(), b.cpu().numpy(), bias.cpu().numpy(), out_fp32=True)
    close(out32, want, atol=1e-3, rtol=1e-3)          # fp32 output: only the summation order differs
    close(out16, want)
    assert out16.dtype == torch.float16 and out32.dtype == torch.float32


SWEEP_KN = [(768, 2304), (768, 768), (768, 3072), (3072, 768), (768, 50257)]


@pytest.mark.parametrize("k,n", SWEEP_KN)
@pytest.mark.parametrize("m", [1, 8, 32])
def test_operator_sweep_against_reference_kernels(ops, ref, m, k, n):
    a, w, s, bias = int8_case(torch, m, n, k, seed=1)
    got = ops.gemm_int8(a, w, s, bias=bias)
    want = ref.gemm_int8(a, w, s, bias=bias)
    got32 = ops.gemm_int8(a, w, s, bias=bias, output_dtype=torch.float32)
    want32 = ref.gemm_int8(a, w, s, bias=bias, output_dtype=torch.float32)
    torch.cuda.synchronize()
    close(got32, want32, atol=2e-3, rtol=1e-4)        # both accumulate in fp32; order differs
    # fp16 outputs: the same value up to the fp32 summation noise (bounded above) plus, where that
    # noise straddles a rounding boundary, one fp16 ulp
    diff = (got.float() - want.float()).abs()
    ulp = want.float().abs() * 2 ** -10
    assert (diff <= ulp + 2e-3).all(), f"max excess {(diff - ulp).max().item()}"
    assert (diff > 0).float().mean().item() < 0.05


@pytest.mark.parametrize("m", [1, 5, 128, 512])
def test_operator_sweep_against_oracle(ops, m):
    a, w, s, bias = int8_case(torch, m, 2304, 768, seed=1)
    want = orc.gemm_int8(a.cpu().numpy(), w.cpu().numpy(), s.cpu().numpy(), bias.cpu().numpy(), out_fp32=True)
    close(ops.gemm_int8(a, w, s, bias=bias, output_dtype=torch.float32), want, atol=2e-3, rtol=1e-4)
    close(ops.gemm_int8(a, w, s, bias=bias), want)


@pytest.mark.parametrize("k,n", [(768, 2304), (3072, 768)])
def test_a_row_does_not_depend_on_the_row_count(ops, k, n):
    """The tensor-core GEMM changes its shape with the row count -- 32-row tiles with the partial sums pushed to the
    finishing CTA, 64-row tiles, one CTA per tile walking the whole K with an accumulator per K range, scalar or
    8-column finishing -- but every form adds the same K ranges in the same order: the first rows of a large call are
    bit-identical to a call with only those rows, with and without the fused GELU / residual epilogue."""
    a, w, s, bias = int8_case(torch, 1500, n, k, seed=5)
    res = torch.randn((1500, n), device="cuda").half()
    small = ops.gemm_int8(a[:20], w, s, bias=bias)
    small_fused = ops.gemm_int8_fused(a[:20], w, s, bias=bias, gelu=True, residual=res[:20])
    for rows in (48, 200, 700, 1500):
        assert torch.equal(ops.gemm_int8(a[:rows], w, s, bias=bias)[:20], small), f"{rows} rows"
        got = ops.gemm_int8_fused(a[:rows], w, s, bias=bias, gelu=True, residual=res[:rows].contiguous())
        assert torch.equal(got[:20], small_fused), f"{rows} rows, fused epilogue"
    want = orc.gemm_int8(a.cpu().numpy(), w.cpu().numpy(), s.cpu().numpy(), bias.cpu().numpy(), out_fp32=True)
    close(ops.gemm_int8(a, w, s, bias=bias), want)


def test_ragged_shapes_through_every_form_of_the_tensor_core_gemm(ops):
    """N not a multiple of the 128-column slab, K not a multiple of the 64-row stage (so the last K ranges of the
    split are short or empty), row counts that end inside a tile: 32-row, 64-row and whole-K forms against the oracle,
    and the first rows of every call bit-identical."""
    k, n = 520, 1008            # rows of W must stay 16-byte aligned for the tensor-core path (TMA)
    a, w, s, bias = int8_case(torch, 1500, n, k, seed=9)
    want = orc.gemm_int8(a.cpu().numpy(), w.cpu().numpy(), s.cpu().numpy(), bias.cpu().numpy(), out_fp32=True)
    first = None
    for rows in (7, 33, 100, 700, 1500):
        got = ops.gemm_int8(a[:rows], w, s, bias=bias)
        close(got, want[:rows])
        close(ops.gemm_int8(a[:rows], w, s, bias=bias, output_dtype=torch.float32), want[:rows], atol=2e-3, rtol=1e-4)
        if first is None:
            first = got
        else:
            assert torch.equal(got[:7], first), f"{rows} rows"


@pytest.mark.parametrize("m,n,k", [(1, 3072, 768), (8, 768, 3072), (32, 3072, 768), (3, 100, 40)])
def test_fused_bias_gelu_residual_equals_reference_sequence(ops, ref, m, n, k):
    a, w, s, bias = int8_case(torch, m, n, k, seed=1)
    res = torch.randn((m, n), device="cuda").half()
    # reference sequence: gemm (fp16 out) -> gelu_new -> fp16 add, three kernels
    lin = ref.gemm_int8(a, w, s, bias=bias)
    act = ref.gelu_new(lin)
    summed = (act.float() + res.float()).half()
    got_act = ops.gemm_int8_fused(a, w, s, bias=bias, gelu=True)
    got_sum = ops.gemm_int8_fused(a, w, s, bias=bias, gelu=True, residual=res)
    got_res = ops.gemm_int8_fused(a, w, s, bias=bias, residual=res)
    close(got_act, act)
    close(got_sum, summed)
    close(got_res, (lin.float() + res.float()).half())
    mine = ops.gelu_new(ops.gemm_int8(a, w, s, bias=bias))
    assert torch.equal(mine, got_act)                   # fusing changes no rounding point
    with pytest.raises(ValueError):
        ops.gemm_int8_fused(a, w, s, gelu=True, output_dtype=torch.float32)


ATTN_CASES = [(17, 33, [17, 11], [33, 0], [0, 0], True), (1, 31, [1, 1], [31, 19], [30, 18], True),
              (5, 19, [5, 0], [13, 19], [7, 0], True), (9, 11, [7, 9], [11, 8], [0, 0], False),
              (40, 200, [40, 33], [200, 161], [160, 128], True)]


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("config", [0, 1])
@pytest.mark.parametrize("nq,nk,ql,kl,off,causal", ATTN_CASES)
def test_attention_gate_cases(ops, ref, d, config, nq, nk, ql, kl, off, causal):
    # correctness.py:52-84 (+ one longer ragged case)
    torch.manual_seed(nq * 100 + nk + d)
    q = (torch.randn((2, 2, nq, d), device="cuda") * 0.5).half()
    k = (torch.randn((2, 2, nk, d), device="cuda") * 0.5).half()
    v = torch.randn_like(k)
    out = ops.attention(q, k, v, q_lengths=ql, kv_lengths=kl, query_offsets=off, causal=causal, config=config)
    want = orc.attention(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), ql, kl, off, causal)
    close(out, want.astype(np.float32))
    close(out, ref.attention(q, k, v, q_lengths=ql, kv_lengths=kl, query_offsets=off, causal=causal, config=config))
    qi = torch.arange(nq, device="cuda")[None, :, None]
    ki = torch.arange(nk, device="cuda")[None, None, :]
    mask = (qi < torch.tensor(ql, device="cuda")[:, None, None]) & (ki < torch.tensor(kl, device="cuda")[:, None, None])
    if causal:
        mask = mask & (ki <= torch.tensor(off, device="cuda")[:, None, None] + qi)
    dead = ~mask.any(dim=-1)[:, None, :, None].expand_as(out)
    assert out[dead].count_nonzero().item() == 0       # all-masked rows are exact zeros


@pytest.mark.parametrize("batch,heads,nk,lengths,chunk", [(2, 2, 31, [31, 19], 32), (3, 12, 700, [700, 1, 333], 128),
                                                          (4, 12, 1024, [1024, 513, 512, 129], 128), (2, 3, 96, [0, 96], 64),
                                                          # chunk >= history: one 8-warp CTA per (request, head)
                                                          (4, 12, 1024, [1024, 257, 256, 1], 1024), (3, 12, 700, [700, 0, 333], 704)])
def test_decode_attention_in_place_equals_general_attention(ops, ref, batch, heads, nk, lengths, chunk):
    torch.manual_seed(nk)
    q = (torch.randn((batch, heads, 1, 64), device="cuda") * 0.5).half()
    k = (torch.randn((batch, heads, nk, 64), device="cuda") * 0.5).half()
    v = torch.randn_like(k)
    got = ops.attention_decode(q, k, v, lengths, chunk=chunk)
    offsets = [max(n - 1, 0) for n in lengths]
    want = ref.attention(q, k, v, q_lengths=[1] * batch, kv_lengths=lengths, query_offsets=offsets, causal=True)
    close(got, want)
    close(got, orc.attention(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), [1] * batch, lengths, offsets, True).astype(np.float32))
    for b, n in enumerate(lengths):
        if n == 0:
            assert got[b].count_nonzero().item() == 0


@pytest.mark.parametrize("cols", [1, 7, 257, 768, 1024, 3072])
def test_layernorm_gelu_softmax(ops, ref, cols):
    torch.manual_seed(cols)
    x = torch.randn((3, cols), device="cuda").half()
    g, b = torch.randn(cols, device="cuda").half(), torch.randn(cols, device="cuda").half()
    ln, ln_ref = ops.layernorm(x, g, b), ref.layernorm(x, g, b)
    # The row sums replay the reference's summation order, so LayerNorm and softmax are bit-equal.
    assert torch.equal(ln, ln_ref)
    assert torch.equal(ops.softmax(x), ref.softmax(x))
    assert torch.equal(ops.gelu_new(x), ref.gelu_new(x))
    close(ln, orc.layernorm(x.cpu().numpy(), g.cpu().numpy(), b.cpu().numpy()).astype(np.float32))
    close(ops.gelu_new(x), orc.gelu_new(x.cpu().numpy()).astype(np.float32))
    close(ops.softmax(x), orc.softmax(x.cpu().numpy()).astype(np.float32))
    odd = torch.randn((5, 2, cols), device="cuda").half()          # leading dims are flattened into rows
    assert torch.equal(ops.layernorm(odd, g, b), ref.layernorm(odd, g, b))
    assert torch.equal(ops.gelu_new(odd.flatten()[1:]), ref.gelu_new(odd.flatten()[1:]))     # 2-byte aligned only


def test_legacy_fp32_gemm_symbol(ops):
    a, b = torch.randn((33, 19), device="cuda"), torch.randn((19, 67), device="cuda")
    close(ops.legacy_gemm(a, b), a.double().cpu() @ b.double().cpu(), atol=1e-4, rtol=1e-4)


def test_non_default_stream_and_input_lifetime(ops):
    # correctness.py:96-115
    default = torch.cuda.current_stream()
    stream = torch.cuda.Stream()
    a = torch.randn((33, 19), device="cuda").half()
    b = torch.randn((19, 67), device="cuda").half()
    expected = a.float() @ b.float()
    stream.wait_stream(default)
    with torch.cuda.stream(stream):
        blocker = torch.ones((256, 256), device="cuda", dtype=torch.float16) * 0.001
        for _ in range(8):
            blocker = blocker @ blocker
        actual = ops.gemm(a, b, config=0, output_dtype=torch.float32)
    del a, b
    gc.collect()
    for _ in range(32):
        t1 = torch.empty((33, 19), device="cuda", dtype=torch.float16); t1.fill_(123)
        t2 = torch.empty((19, 67), device="cuda", dtype=torch.float16); t2.fill_(124)
    default.wait_stream(stream)
    close(actual, expected, atol=1e-2, rtol=1e-2)


def test_invalid_tensor_contracts(ops):
    # correctness.py:117-135
    a = torch.ones((2, 3), device="cuda", dtype=torch.float16)
    b = torch.ones((3, 4), device="cuda", dtype=torch.float16)
    for fn in (lambda: ops.gemm(a.cpu(), b), lambda: ops.gemm(a.float(), b), lambda: ops.gemm(a.t(), b),
               lambda: ops.gemm(a, b, config=True), lambda: ops.gemm(a, b, config=12),
               lambda: ops.gemm(a, b, bias=torch.zeros(3, device="cuda", dtype=torch.float16)),
               lambda: ops.gemm(a.clone().requires_grad_(), b)):
        with pytest.raises((ValueError, TypeError)):
            fn()
    q = torch.ones((1, 1, 1, 64), device="cuda", dtype=torch.float16)
    for fn in (lambda: ops.attention(q, q, q, q_lengths=[2]), lambda: ops.attention(q, q, q, query_offsets=[-1]),
               lambda: ops.attention(q, q, q, kv_lengths=[True]), lambda: ops.attention(q, q, q, causal=1)):
        with pytest.raises((ValueError, TypeError)):
            fn()


def test_native_status_codes(ops):
    """Direct C-ABI calls: device mismatch, unsupported config, workspace rule, null scales."""
    import ctypes
    lib = ops.lib
    a = torch.ones((2, 4), device="cuda", dtype=torch.float16)
    w = torch.ones((4, 16), device="cuda", dtype=torch.int8)
    s = torch.ones(16, device="cuda")
    y = torch.empty((2, 16), device="cuda", dtype=torch.float16)
    args = (a.data_ptr(), w.data_ptr(), s.data_ptr(), None, y.data_ptr(), None, 2, 16, 4, 0)
    assert lib.ti_v2_gemm_ex_i8(*args, 0, 0, 0) == 0
    assert lib.ti_v2_gemm_ex_i8(*args, 0, 0, 7) == 2                       # not the current device
    assert lib.ti_v2_gemm_ex_i8(*args, 12, 0, 0) == 3
    assert lib.ti_v2_gemm_ex_i8(*args, 6, 0, 0) == 1                       # config >= 6 needs a workspace
    assert b"workspace" in lib.ti_v2_last_error()
    bad = (a.data_ptr(), w.data_ptr(), None, None, y.data_ptr(), None, 2, 16, 4, 0)
    assert lib.ti_v2_gemm_ex_i8(*bad, 0, 0, 0) == 1
    assert lib.ti_v2_gemm_ex_i8(a.data_ptr(), w.data_ptr(), s.data_ptr(), None, y.data_ptr(), None, 2, 16, 4, 5, 0, 0, 0) == 1
    assert lib.ti_v2_gelu_new_f16(a.data_ptr(), a.data_ptr(), ctypes.c_int64(0), 0, 0) == 1
    torch.cuda.synchronize()
    assert torch.equal(y, torch.full_like(y, 4.0))


@pytest.mark.parametrize("d", [64, 128])
def test_attention_accepts_tensors_that_are_only_two_byte_aligned(ops, d):
    """The reference's validators ask for 2-byte alignment of q/k/v/y (backend/include/tinyinfer_host_validation.hpp);
    views that start one element into an allocation must be accepted and give the same bits as aligned copies."""
    torch.manual_seed(d)
    nq, nk, ql, kl, off = 17, 33, [17, 11], [33, 20], [16, 9]
    shapes = {"q": (2, 2, nq, d), "k": (2, 2, nk, d), "v": (2, 2, nk, d)}
    aligned = {name: (torch.randn(shape, device="cuda") * 0.5).half() for name, shape in shapes.items()}
    want = ops.attention(aligned["q"], aligned["k"], aligned["v"], q_lengths=ql, kv_lengths=kl, query_offsets=off, causal=True)
    shifted = {}
    for name, tensor in aligned.items():
        base = torch.empty(tensor.numel() + 8, device="cuda", dtype=torch.float16)
        shifted[name] = base[1:1 + tensor.numel()].view(tensor.shape)
        shifted[name].copy_(tensor)
        assert shifted[name].data_ptr() % 16 == 2
    out_base = torch.zeros(aligned["q"].numel() + 8, device="cuda", dtype=torch.float16)
    out = out_base[1:1 + aligned["q"].numel()].view(aligned["q"].shape)
    meta = [torch.tensor(values, dtype=torch.int32, device="cuda") for values in (ql, kl, off)]
    status = ops.lib.ti_v2_attention_f16(shifted["q"].data_ptr(), shifted["k"].data_ptr(), shifted["v"].data_ptr(), out.data_ptr(),
                                         meta[0].data_ptr(), meta[1].data_ptr(), meta[2].data_ptr(), 2, 2, nq, nk, d, 1, 0,
                                         torch.cuda.current_stream().cuda_stream, torch.cuda.current_device())
    assert status == 0, ops.lib.ti_v2_last_error()
    torch.cuda.synchronize()
    assert torch.equal(out, want)


TC_ATTN_CASES = [(200, 300, [200, 77], [300, 150], [100, 73], True), (1024, 1024, [1024, 1000], [1024, 1000], [0, 0], True),
                 (130, 257, [130, 64], [257, 0], [0, 0], False), (64, 64, [64, 1], [64, 64], [0, 63], True),
                 (300, 700, [300, 5], [650, 700], [350, 695], True)]


@pytest.mark.parametrize("nq,nk,ql,kl,off,causal", TC_ATTN_CASES)
def test_attention_with_many_query_rows_runs_on_tensor_cores_and_matches(ops, ref, nq, nk, ql, kl, off, causal):
    """64 or more query rows of 64-wide heads take the tcgen05 attention kernel: against the reference's kernel and the
    CPU oracle (same gate, atol = rtol = 0.02), all-masked and padding rows exact zeros, and a request's rows do not
    depend on the other request in the call."""
    torch.manual_seed(nq + nk)
    q = (torch.randn((2, 3, nq, 64), device="cuda") * 0.5).half()
    k = (torch.randn((2, 3, nk, 64), device="cuda") * 0.5).half()
    v = torch.randn_like(k)
    out = ops.attention(q, k, v, q_lengths=ql, kv_lengths=kl, query_offsets=off, causal=causal)
    close(out, ref.attention(q, k, v, q_lengths=ql, kv_lengths=kl, query_offsets=off, causal=causal))
    if nq * nk <= 300 * 700:
        want = orc.attention(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), ql, kl, off, causal)
        close(out, want.astype(np.float32))
    qi = torch.arange(nq, device="cuda")[None, :, None]
    ki = torch.arange(nk, device="cuda")[None, None, :]
    mask = (qi < torch.tensor(ql, device="cuda")[:, None, None]) & (ki < torch.tensor(kl, device="cuda")[:, None, None])
    if causal:
        mask = mask & (ki <= torch.tensor(off, device="cuda")[:, None, None] + qi)
    dead = ~mask.any(dim=-1)[:, None, :, None].expand_as(out)
    assert out[dead].count_nonzero().item() == 0
    alone = ops.attention(q[:1].contiguous(), k[:1].contiguous(), v[:1].contiguous(), q_lengths=ql[:1], kv_lengths=kl[:1],
                          query_offsets=off[:1], causal=causal)
    assert torch.equal(alone[0], out[0])


@pytest.mark.parametrize("k,n", [(768, 2304), (3072, 768), (768, 50304)])
@pytest.mark.parametrize("m", [8, 32, 100, 512, 1500])
def test_fp16_weights_run_the_tensor_core_kernel_with_the_bits_of_the_int8_path(ops, ref, m, k, n):
    """ti_v2_gemm_ex_f16 (reference backend/runtime_v2.cu:62-68) from 5 rows on takes the same tcgen05 kernel as the
    INT8 path, the weight tiles rearranged instead of dequantised: given the fp16 values an INT8 matrix dequantises to it
    returns exactly the bits of the INT8 call, and it stays inside the gate of the reference's own kernel."""
    a, w, s, bias = int8_case(torch, m, n, k, seed=7)
    w16 = (w.float() * s[None, :]).half()                       # fp16_rn(float(q) * scale): the reference's dequantisation
    got = ops.gemm(a, w16, bias=bias)
    assert torch.equal(got, ops.gemm_int8(a, w, s, bias=bias))
    got32 = ops.gemm(a, w16, bias=bias, output_dtype=torch.float32)
    assert torch.equal(got32, ops.gemm_int8(a, w, s, bias=bias, output_dtype=torch.float32))
    if n <= 4096:
        close(got32, ref.gemm(a, w16, bias=bias, output_dtype=torch.float32), atol=2e-3, rtol=1e-4)
