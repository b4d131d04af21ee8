"""Regenerates tests/golden/quant_golden.json from the reference itself.

Needs the reference checkout (see --reference) and the reference host codec built
by `make -C oracle ref-host`; neither is available where the GPU tests run, which is why
the outputs are committed.  Imports the reference's pure-Python quantiser spec
(llm/quantization.py), its exporter twin (llm/export_weights.py:quantized_bytes) and its
native codec wrapper (llm/host_codec.py), feeds them seeded inputs, and stores inputs as
fp16 bit patterns with the outputs all three agree on.

    python tests/golden/make_golden.py [--reference <checkout>]
"""
import argparse
import array
import hashlib
import json
import os
import struct
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default=os.environ.get("TINYINFER_REFERENCE"), required="TINYINFER_REFERENCE" not in os.environ,
                        help="the reference checkout (or the TINYINFER_REFERENCE environment variable)")
    args = parser.parse_args()
    sys.path.insert(0, args.reference)
    from llm.export_weights import quantized_bytes
    from llm.host_codec import HostCodec
    from llm.quantization import dequantize, quantize

    codec = HostCodec(ROOT / "oracle/_ref/libtinyinfer_host_codec.so")
    rng = np.random.default_rng(20261125)
    cases = []

    def add(name, matrix16):
        matrix16 = np.asarray(matrix16, np.float16)
        rows = matrix16.astype(np.float64).tolist()
        q, scales = quantize(rows)                                   # pure-Python spec
        flat = array.array("f", matrix16.astype(np.float32).ravel().tolist())
        qb, sb = quantized_bytes(flat, matrix16.shape[1])            # exporter twin
        qn, sn = codec.quantized_bytes(flat, matrix16.shape[1])      # native codec
        q_flat = [v for row in q for v in row]
        assert list(array.array("b", qb)) == q_flat and list(array.array("b", qn)) == q_flat, name
        assert sb == sn == struct.pack(f"<{len(scales)}f", *scales), name
        deq = dequantize(q, scales)
        deq_bits = [int(np.float16(v).view(np.uint16)) for row in deq for v in row]
        native = codec.dequantized_half_bytes(qn, sn, matrix16.shape[1])
        assert list(np.frombuffer(native, np.uint16)) == deq_bits, name
        cases.append({"name": name, "rows": matrix16.shape[0], "cols": matrix16.shape[1],
                      "w_bits": matrix16.view(np.uint16).ravel().tolist(), "q": q_flat,
                      "scale_bits": list(np.frombuffer(sb, np.uint32).tolist()), "dequant_bits": deq_bits})

    add("normal_0.02", rng.normal(0, 0.02, (48, 24)))
    add("normal_1", rng.normal(0, 1.0, (33, 17)))
    add("zero_column", np.concatenate([np.zeros((9, 1)), rng.normal(0, 0.3, (9, 6))], axis=1))
    add("half_steps", (rng.integers(-254, 255, (40, 8)) / 2.0))
    add("tiny_and_huge", np.array([[2.0 ** -24, 65504.0, -6.1e-5], [-(2.0 ** -24), -65504.0, 3.0e-5],
                                   [0.0, 1.0, -0.0]]))
    add("single_row", rng.normal(0, 0.5, (1, 13)))
    add("single_col", rng.normal(0, 0.5, (29, 1)))

    # Exhaustive sweep of every finite binary16 pattern, 32 columns (fuzz/check_codec.py:19-21);
    # 63,488 values are too many to store, so the reference's output is kept as a digest.
    bits = np.array([i for i in range(65536) if i & 0x7c00 != 0x7c00], np.uint16)
    flat = array.array("f", bits.view(np.float16).astype(np.float32).tolist())
    qn, sn = codec.quantized_bytes(flat, 32)
    assert (qn, sn) == quantized_bytes(flat, 32)
    deq = codec.dequantized_half_bytes(qn, sn, 32)
    sweep = {"columns": 32, "elements": len(bits), "q_sha256": hashlib.sha256(qn).hexdigest(),
             "scales_sha256": hashlib.sha256(sn).hexdigest(), "dequant_sha256": hashlib.sha256(deq).hexdigest()}

    out = {"generator": "tests/golden/make_golden.py", "source": "reference llm/quantization.py + llm/export_weights.py + backend/host_codec.cpp",
           "cases": cases, "all_finite_half_sweep": sweep}
    path = Path(__file__).with_name("quant_golden.json")
    path.write_text(json.dumps(out, separators=(",", ":")) + "\n")
    print(path, path.stat().st_size, "bytes,", len(cases), "cases")


if __name__ == "__main__":
    main()
