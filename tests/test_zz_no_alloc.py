"""The allocation-free decode attention (ti_b200_attention_decode_static_f16).

Some users of this library cannot allocate GPU memory at call time -- a token loop that fixed its
memory budget at start-up, an operator running inside a host program that owns all device memory,
a process already at its memory limit -- so this entry point keeps its scratch in a fixed array
inside the library.  It must give exactly the results of ti_b200_attention_decode_f16 (same kernels,
same order), also when called repeatedly: the array is shared and keeps the previous call's contents.

Collected last on purpose, so that a run stopping at the first failure has run everything else.
"""
import ctypes

import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _library():
    import tinyinfer_b200
    lib = ctypes.CDLL(str(tinyinfer_b200.library("backend")))
    p, i, u, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_int64
    lib.ti_v2_last_error.restype = ctypes.c_char_p
    lib.ti_b200_attention_decode_scratch_floats.argtypes, lib.ti_b200_attention_decode_scratch_floats.restype = [i, i, i, i], i64
    lib.ti_b200_attention_decode_static_capacity_floats.argtypes, lib.ti_b200_attention_decode_static_capacity_floats.restype = [], ctypes.c_longlong
    lib.ti_b200_attention_decode_f16.argtypes, lib.ti_b200_attention_decode_f16.restype = [p, p, p, p, p, i, i, i, i, i, p, i64, u, i], i
    lib.ti_b200_attention_decode_static_f16.argtypes, lib.ti_b200_attention_decode_static_f16.restype = [p, p, p, p, p, i, i, i, i, i, u, i], i
    return lib


def _case(seed, batch, heads, kv_len, lengths):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn((batch, heads, 1, 64), generator=g) * 0.5).half().cuda()
    k = (torch.randn((batch, heads, kv_len, 64), generator=g) * 0.5).half().cuda()
    v = torch.randn((batch, heads, kv_len, 64), generator=g).half().cuda()
    return q, k, v, torch.tensor(lengths, dtype=torch.int32, device="cuda")


def _both(lib, q, k, v, lengths, chunk):
    batch, heads, _, d = q.shape
    kv_len = k.shape[2]
    stream, device = torch.cuda.current_stream().cuda_stream, torch.cuda.current_device()
    floats = lib.ti_b200_attention_decode_scratch_floats(batch, heads, kv_len, chunk)
    scratch = torch.empty(floats, dtype=torch.float32, device="cuda")
    regular, fixed = torch.empty_like(q), torch.full_like(q, float("nan"))
    status = lib.ti_b200_attention_decode_f16(q.data_ptr(), k.data_ptr(), v.data_ptr(), regular.data_ptr(), lengths.data_ptr(), batch, heads,
                                              kv_len, d, chunk, scratch.data_ptr(), floats, stream, device)
    assert status == 0, lib.ti_v2_last_error()
    status = lib.ti_b200_attention_decode_static_f16(q.data_ptr(), k.data_ptr(), v.data_ptr(), fixed.data_ptr(), lengths.data_ptr(), batch, heads,
                                                     kv_len, d, chunk, stream, device)
    assert status == 0, lib.ti_v2_last_error()
    torch.cuda.synchronize()
    return regular, fixed


def test_static_scratch_matches_regular_entry_point_on_consecutive_calls():
    lib = _library()
    # first call: long ragged histories, several chunks per request
    q, k, v, lengths = _case(1, 4, 12, 900, [900, 513, 128, 1])
    regular, fixed = _both(lib, q, k, v, lengths, 128)
    assert torch.equal(regular, fixed)
    # second call right after it, different shape and shorter histories: stale partials of the first
    # call are still in the array and must not leak into the result
    q, k, v, lengths = _case(2, 3, 5, 300, [77, 300, 0])
    regular, fixed = _both(lib, q, k, v, lengths, 64)
    assert torch.equal(regular, fixed)
    assert fixed[2].count_nonzero().item() == 0           # empty history -> exact zeros
    # and against the general attention operator, within the operator tolerance used elsewhere
    from tinyinfer_b200.native_ops import NativeOps
    ops = NativeOps()
    want = ops.attention(q, k, v, q_lengths=[1, 1, 1], kv_lengths=lengths.tolist(), query_offsets=[76, 299, 0], causal=True)
    torch.testing.assert_close(fixed.float(), want.float(), atol=0.02, rtol=0.02)


def test_static_scratch_rejects_oversized_problems_with_a_clear_error():
    lib = _library()
    capacity = lib.ti_b200_attention_decode_static_capacity_floats()
    batch, heads, kv_len, chunk = 64, 64, 1024, 32             # 64*64*32*66 floats, far beyond 4 MiB
    assert lib.ti_b200_attention_decode_scratch_floats(batch, heads, kv_len, chunk) > capacity
    q = torch.zeros((batch, heads, 1, 64), device="cuda", dtype=torch.float16)
    k = torch.zeros((batch, heads, kv_len, 64), device="cuda", dtype=torch.float16)
    lengths = torch.full((batch,), kv_len, dtype=torch.int32, device="cuda")
    out = torch.full_like(q, 7.0)
    status = lib.ti_b200_attention_decode_static_f16(q.data_ptr(), k.data_ptr(), k.data_ptr(), out.data_ptr(), lengths.data_ptr(), batch, heads,
                                                     kv_len, 64, chunk, torch.cuda.current_stream().cuda_stream, torch.cuda.current_device())
    assert status == 1
    message = lib.ti_v2_last_error().decode()
    assert "scratch" in message and str(capacity) in message
    torch.cuda.synchronize()
    assert torch.equal(out, torch.full_like(out, 7.0))           # nothing was launched


def test_static_scratch_single_chunk_path_and_capacity_boundary():
    lib = _library()
    # a chunk that covers the whole history takes the kernel that merges in shared memory: the array is not touched
    q, k, v, lengths = _case(3, 2, 3, 200, [200, 131])
    regular, fixed = _both(lib, q, k, v, lengths, 256)
    assert torch.equal(regular, fixed)
    # the largest problem of this shape family that still fits the array (31 x 16 x 32 chunks x 66 floats = 1,047,552 of
    # 1,048,576), bit for bit against the caller-scratch entry ...
    capacity = lib.ti_b200_attention_decode_static_capacity_floats()
    assert lib.ti_b200_attention_decode_scratch_floats(31, 16, 1024, 32) <= capacity
    q, k, v, lengths = _case(4, 31, 16, 1024, [1024 - 7 * i for i in range(31)])
    regular, fixed = _both(lib, q, k, v, lengths, 32)
    assert torch.equal(regular, fixed)
    # ... and the next larger one (71 x 7 x 32 x 66 = 1,049,664) is refused before anything is launched
    assert lib.ti_b200_attention_decode_scratch_floats(71, 7, 1024, 32) > capacity
    q, k, v, lengths = _case(5, 71, 7, 1024, [1024] * 71)
    out = torch.full_like(q, 3.0)
    status = lib.ti_b200_attention_decode_static_f16(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lengths.data_ptr(), 71, 7, 1024, 64, 32,
                                                     torch.cuda.current_stream().cuda_stream, torch.cuda.current_device())
    assert status == 1 and "scratch" in lib.ti_v2_last_error().decode()
    torch.cuda.synchronize()
    assert torch.equal(out, torch.full_like(out, 3.0))
