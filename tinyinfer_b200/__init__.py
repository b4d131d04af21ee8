"""tinyinfer_b200: the INT8-weight GPT-2 decode path of tinyinfer, rebuilt for B200 (sm_100a).

Host side mirrors the reference's Python surface for this path:
    tinyinfer_b200.native_ops.NativeOps      <-> llm/native_ops.py   (ti_v2_* operator ABI)
    tinyinfer_b200.quantization              <-> llm/quantization.py (quantiser specification)
    tinyinfer_b200.host_codec.HostCodec      <-> llm/host_codec.py   (ti_host_* codec ABI)
    tinyinfer_b200.runtime.NativeModel       <-> llm/runtime.py      (ti_llm_* model ABI)
    tinyinfer_b200.artifact                  <-> llm/export_weights.py (manifest.json + weights.bin)
The compute lives in tinyinfer_b200/lib/*.so, built in-tree by tinyinfer_b200.build from
tinyinfer_b200/csrc.  There is no CPU fallback: without the libraries, or without a CUDA
device, the operators raise.
"""
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
LIB_DIR = PACKAGE_DIR / "lib"


def library(name: str) -> Path:
    """Path of a built native library ('backend', 'llm', 'host_codec'); raises if it is missing."""
    path = LIB_DIR / f"libtinyinfer_{name}.so"
    if not path.exists():
        raise FileNotFoundError(f"{path} is not built; run `python -m tinyinfer_b200.build`")
    return path
