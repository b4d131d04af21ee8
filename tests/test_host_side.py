"""CPU-only checks: quantiser specification, host codec library, ABI surface, wrappers' host logic."""
import ctypes
import json
import re
import sys
from pathlib import Path

import numpy as np
import pytest

import tinyinfer_b200
from oracle import ti_oracle as orc
from tinyinfer_b200 import artifact, quantization
from tinyinfer_b200.host_codec import HostCodec

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = json.loads((ROOT / "tests/golden/quant_golden.json").read_text())


@pytest.fixture(scope="module")
def built():
    from tinyinfer_b200 import build
    return build.build()


# ------------------------------------------------------------------ quantiser specification
def test_spec_known_answers():
    # reference llm/tests/test_contracts.py:22-34
    q, s = quantization.quantize([[0, 127, -254], [0, 0, 127], [0, -127, 0]])
    assert s == [1.0, 1.0, 2.0] and q == [[0, 127, -127], [0, 0, 64], [0, -127, 0]]
    assert quantization.dequantize(q, s) == [[0, 127, -254], [0, 0, 128], [0, -127, 0]]
    q, s = quantization.quantize([[127], [.5], [1.5], [2.5], [-.5], [-1.5], [-2.5], [-127]])
    assert s == [1.0] and q == [[127], [0], [2], [2], [0], [-2], [-2], [-127]]


def test_spec_rejects_what_the_reference_rejects():
    # reference llm/tests/test_contracts.py:50-57
    for rows in ([], [[]], [[1], [1, 2]], [[float("nan")]], [[True]], [[float("inf")]]):
        with pytest.raises((ValueError, OverflowError)):
            quantization.quantize(rows)
    for q, s in (([[1]], []), ([[1]], [0]), ([[1]], [-1]), ([[1]], [float("nan")]), ([[1]], [True]),
                 ([[-128]], [1]), ([[1.0]], [1]), ([[128]], [1])):
        with pytest.raises(ValueError):
            quantization.dequantize(q, s)


@pytest.mark.parametrize("case", GOLDEN["cases"], ids=lambda c: c["name"])
def test_spec_and_codec_match_reference_vectors(case, built):
    w = np.array(case["w_bits"], np.uint16).view(np.float16).reshape(case["rows"], case["cols"])
    q, s = quantization.quantize(w.astype(np.float64).tolist())
    assert [v for row in q for v in row] == case["q"]
    assert np.array(s, np.float32).view(np.uint32).tolist() == case["scale_bits"]
    deq = quantization.dequantize(q, s)
    assert np.array(deq, np.float16).view(np.uint16).ravel().tolist() == case["dequant_bits"]
    codec = HostCodec()
    qn, sn = codec.quantize_array(w)
    assert qn.ravel().tolist() == case["q"] and sn.view(np.uint32).tolist() == case["scale_bits"]
    assert codec.dequantize_array(qn, sn).view(np.uint16).ravel().tolist() == case["dequant_bits"]


def test_codec_exhaustive_half_sweep(built):
    import hashlib
    sweep = GOLDEN["all_finite_half_sweep"]
    bits = np.array([i for i in range(65536) if i & 0x7c00 != 0x7c00], np.uint16)
    codec = HostCodec()
    q, s = codec.quantize_array(bits.view(np.float16).reshape(-1, sweep["columns"]))
    assert hashlib.sha256(q.tobytes()).hexdigest() == sweep["q_sha256"]
    assert hashlib.sha256(s.tobytes()).hexdigest() == sweep["scales_sha256"]
    assert hashlib.sha256(codec.dequantize_array(q, s).tobytes()).hexdigest() == sweep["dequant_sha256"]


def test_codec_failure_atomicity(built):
    # reference fuzz/check_codec.py:33-57
    lib = HostCodec().lib
    src = (ctypes.c_uint16 * 2)(0x3c00, 0x7c00); out = (ctypes.c_int8 * 2)(17, 19); scale = (ctypes.c_float * 1)(23.)
    before = bytes(out), bytes(scale)
    assert lib.ti_host_quantize_f16(src, 2, 1, out, 2, scale, 1) == 1 and before == (bytes(out), bytes(scale))
    src = (ctypes.c_uint16 * 2)(0x3c00, 0x4000)
    assert lib.ti_host_quantize_f16(src, 2, 1, out, 1, scale, 1) == 1 and before == (bytes(out), bytes(scale))
    assert lib.ti_host_quantize_f16(src, 2, 1, ctypes.cast(src, ctypes.c_void_p), 2, scale, 1) == 1
    for qv, sv in [(-128, 1.), (127, 1e10), (1, 0.), (1, float("nan")), (1, float("inf"))]:
        qq = (ctypes.c_int8 * 1)(qv); ss = (ctypes.c_float * 1)(sv); yy = (ctypes.c_uint16 * 1)(0x1234)
        assert lib.ti_host_dequantize_i8(qq, 1, 1, ss, 1, yy, 1) == 1 and yy[0] == 0x1234
    for values, scales in [([1, -128], [1., 1.]), ([1, 127], [1., 1e10]), ([1, 1], [1., 0.]), ([1, 1], [1., float("nan")])]:
        qq = (ctypes.c_int8 * 2)(*values); ss = (ctypes.c_float * 2)(*scales); yy = (ctypes.c_uint16 * 2)(0x1234, 0x5678)
        assert lib.ti_host_dequantize_i8(qq, 2, 2, ss, 2, yy, 2) == 1 and bytes(yy) == bytes((ctypes.c_uint16 * 2)(0x1234, 0x5678))


def test_codec_random_matrices_match_oracle(built):
    rng = np.random.default_rng(11)
    codec = HostCodec()
    for shape, std in (((768, 96), 0.02), ((64, 513), 1.0), ((1, 1), 3.0)):
        w = rng.normal(0, std, shape).astype(np.float16)
        q, s = codec.quantize_array(w)
        qo, so = orc.quantize(w)
        assert (q == qo).all() and (s.view(np.uint32) == so.view(np.uint32)).all()
        assert (codec.dequantize_array(q, s).view(np.uint16) == orc.dequantize(qo, so).view(np.uint16)).all()


# ------------------------------------------------------------------ ABI surface
def _declared(header):
    text = re.sub(r"/\*.*?\*/", "", (ROOT / "include" / header).read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ti_[a-z0-9_]+)\s*\(", text)))


@pytest.mark.parametrize("header,lib", [("tinyinfer_backend_v2.h", "backend"), ("tinyinfer_host_codec.h", "host_codec"),
                                        ("tinyinfer_llm.h", "llm")])
def test_library_exports_every_declared_symbol(header, lib, built):
    handle = ctypes.CDLL(str(tinyinfer_b200.library(lib)))
    names = _declared(header)
    assert names, header
    for name in names:
        assert hasattr(handle, name), f"{lib} library lacks {name}"


def test_extension_header_symbols(built):
    backend = ctypes.CDLL(str(tinyinfer_b200.library("backend")))
    llm = ctypes.CDLL(str(tinyinfer_b200.library("llm")))
    for name in _declared("tinyinfer_b200_ext.h"):
        assert hasattr(backend, name) or hasattr(llm, name), name


def test_versions_and_catalog(built):
    from tinyinfer_b200.native_ops import GEMM_CATALOG
    backend = ctypes.CDLL(str(tinyinfer_b200.library("backend")))
    backend.ti_v2_gemm_catalog_json.restype = ctypes.c_char_p
    assert backend.ti_v2_abi_version() == 2
    catalog = json.loads(backend.ti_v2_gemm_catalog_json())
    assert catalog["schema_version"] == 1 and catalog["only_config"] == -1
    assert [{**c, "tile": tuple(c["tile"])} for c in catalog["configs"]] == list(GEMM_CATALOG)
    assert ctypes.CDLL(str(tinyinfer_b200.library("llm"))).ti_llm_abi_version() == 1
    assert ctypes.CDLL(str(tinyinfer_b200.library("host_codec"))).ti_host_codec_abi_version() == 1


def test_runtime_struct_layout_and_row_packing():
    # reference llm/tests/test_contracts.py:140-149
    from tinyinfer_b200.runtime import Options, Trace, _rows
    assert ctypes.sizeof(Options) == 28 and ctypes.sizeof(Trace) == 96
    ids, lengths, stride = _rows([[10, 11], [12]])
    assert (list(ids), list(lengths), stride) == ([10, 11, 12, 0], [2, 1], 2)
    for rows in ([], [[]], [[True]], [[-1]], [[50257]]):
        with pytest.raises(ValueError):
            _rows(rows)


def test_native_ops_reject_cpu_tensors_before_any_native_call(built):
    import torch
    from tinyinfer_b200.native_ops import NativeOps
    ops = NativeOps()
    a = torch.ones((2, 3), dtype=torch.float16)
    with pytest.raises(TypeError):
        ops.gemm(a, a.t().contiguous())
    with pytest.raises(TypeError):
        ops.layernorm(a, a[0], a[0])


# ------------------------------------------------------------------ artifact format
TINY = {**artifact.GPT2_SMALL, "layers": 1, "heads": 1, "hidden": 64, "capacity": 16}


def _check(path):
    lib = ctypes.CDLL(str(tinyinfer_b200.library("llm")))
    lib.ti_llm_last_error.restype = ctypes.c_char_p
    out = [ctypes.c_int32() for _ in range(4)]
    status = lib.ti_b200_artifact_check(str(path).encode(), *[ctypes.byref(o) for o in out])
    return status, lib.ti_llm_last_error().decode(), [o.value for o in out]


def test_artifact_round_trip_and_rejections(tmp_path, built):
    manifest_path = artifact.write_synthetic(tmp_path / "tiny", TINY, seed=5)
    status, text, shape = _check(manifest_path)
    assert status == 0 and shape == [1, 1, 64, 1], text
    manifest, tensors = artifact.load(manifest_path)
    source = artifact.synthetic_tensors(TINY, 5)
    q, s = orc.quantize(source["transformer.h.0.mlp.c_fc.weight"])
    assert (tensors["transformer.h.0.mlp.c_fc.weight"] == q).all()
    assert (tensors["transformer.h.0.mlp.c_fc.weight.scales"].view(np.uint32) == s.view(np.uint32)).all()
    qh, sh = orc.quantize(np.ascontiguousarray(source["transformer.wte.weight"].T))
    assert (tensors["lm_head.weight"] == qh).all() and (tensors["lm_head.weight.scales"] == sh).all()
    assert all(e["offset"] % 256 == 0 for e in manifest["tensors"])

    def variant(name, mutate, binary=None):
        d = tmp_path / name
        d.mkdir()
        m = json.loads(manifest_path.read_text())
        mutate(m)
        (d / "manifest.json").write_text(json.dumps(m))
        data = bytearray((manifest_path.parent / "weights.bin").read_bytes())
        if binary:
            binary(data)
        (d / "weights.bin").write_bytes(data)
        return _check(d / "manifest.json")

    assert variant("identity", lambda m: m.__setitem__("model_id", "other"))[0] == 1
    assert variant("schema", lambda m: m.__setitem__("schema_version", 2))[0] == 1
    assert variant("flip", lambda m: None, lambda b: b.__setitem__(1000, b[1000] ^ 1))[0] == 1
    assert variant("extent", lambda m: m["tensors"][0].__setitem__("nbytes", m["tensors"][0]["nbytes"] - 2))[0] == 1
    assert variant("unaligned", lambda m: m["tensors"][1].__setitem__("offset", m["tensors"][1]["offset"] + 2))[0] == 1
    assert variant("dup", lambda m: m["tensors"].append(dict(m["tensors"][0])))[0] == 1
    assert variant("heads", lambda m: m["architecture"].__setitem__("heads", 2))[0] == 1
    status, text, _ = _check(tmp_path / "missing" / "manifest.json")
    assert status == 2 and "cannot open" in text


def test_weight_byte_count_matches_published_artifact_size(tmp_path):
    # GPT-2 small int8: 123,532,032 weight + 532,804 scale + 165,888 bias + 76,800 LayerNorm bytes
    shapes = artifact.tensor_shapes(artifact.GPT2_SMALL)
    linear = sum(np.prod(s) for n, s in shapes.items() if len(s) == 2 and ".h." in n) + 768 * 50257
    assert linear == 123_532_032
    scales = 4 * (sum(s[1] for n, s in shapes.items() if len(s) == 2 and ".h." in n) + 50257)
    assert scales == 532_804
    assert 2 * sum(s[0] for n, s in shapes.items() if n.endswith(".bias") and ".ln_" not in n) == 165_888


def test_no_heavy_imports_in_runtime_wrapper():
    import subprocess
    code = "import sys; import tinyinfer_b200.runtime; print(any(m in sys.modules for m in ('torch','numpy')))"
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT)
    assert out.stdout.strip() == "False", out.stderr
