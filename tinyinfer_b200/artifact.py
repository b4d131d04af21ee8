"""Weight artifacts: `manifest.json` + 256-byte-aligned `weights.bin`.

The on-disk format is the reference exporter's (llm/export_weights.py:163-205) and is what both
the reference loader (llm/src/artifact.hpp:153-199) and this package's loader
(csrc/artifact.hpp) verify: schema 1, pinned identity strings, architecture block, precision,
per-tensor name/dtype/shape/offset/nbytes/sha256, whole-file sha256.  Linear weights are stored
[input, output] (GPT-2 Conv1D orientation, never transposed); in an int8 artifact each becomes
`<name>.weight` int8 plus `<name>.weight.scales` float32, quantised by the host codec; the
vocabulary projection `lm_head.weight` is the transpose of the fp16 token embedding.

The reference exporter needs the pretrained safetensors file.  This module writes the same
format from SEEDED RANDOM weights instead (N(0, 0.02) matrices, zero biases, LayerNorm gamma 1 /
beta 0), which is what the benchmark configurations are defined on.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np

from .host_codec import HostCodec

ALIGNMENT = 256
# Identity strings the loaders require (reference llm/protocol.py:7-9).
MODEL_ID = "openai-community/gpt2"
MODEL_REVISION = "607a30d783dfa663caf39e06633721c8d4cfcd7e"
MODEL_SHA256 = "248dfc3911869ec493c76e65bf2fcf7f615828b0254c12b473182f0f81d3a707"

GPT2_SMALL = {"layers": 12, "heads": 12, "hidden": 768, "vocab": 50257, "capacity": 1024,
              "gelu": "gelu_new", "layer_norm_eps": 1e-5}
GPT2_MEDIUM = {**GPT2_SMALL, "layers": 24, "heads": 16, "hidden": 1024}


def tensor_shapes(arch):
    """Ordered {name: shape} of the fp16 source tensors (reference expected_tensors, export_weights.py:33-47)."""
    h, v = arch["hidden"], arch["vocab"]
    shapes = {"transformer.wte.weight": [v, h], "transformer.wpe.weight": [arch["capacity"], h],
              "transformer.ln_f.weight": [h], "transformer.ln_f.bias": [h]}
    for layer in range(arch["layers"]):
        p = f"transformer.h.{layer}."
        for norm in ("ln_1", "ln_2"):
            shapes[p + norm + ".weight"] = [h]
            shapes[p + norm + ".bias"] = [h]
        for name, shape in (("attn.c_attn", [h, 3 * h]), ("attn.c_proj", [h, h]), ("mlp.c_fc", [h, 4 * h]), ("mlp.c_proj", [4 * h, h])):
            shapes[p + name + ".weight"] = shape
            shapes[p + name + ".bias"] = [shape[1]]
    return shapes


def synthetic_tensors(arch, seed, std=0.02, dense=False):
    """Seeded random fp16 tensors: matrices N(0, std), biases 0, LayerNorm gamma 1 / beta 0 (the benchmark
    configurations' initialisation).  dense=True also randomises the vectors (biases N(0, 0.05), gamma 1 + N(0, 0.1),
    beta N(0, 0.05)) so that a test sees every bias / LayerNorm parameter take part."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(arch).items():
        if len(shape) == 2:
            out[name] = rng.standard_normal(shape, dtype=np.float32).__mul__(np.float32(std)).astype(np.float16)
        elif ".ln_" in name and name.endswith(".weight"):
            out[name] = (1 + 0.1 * rng.standard_normal(shape, dtype=np.float32)).astype(np.float16) if dense else np.ones(shape, np.float16)
        else:
            out[name] = (0.05 * rng.standard_normal(shape, dtype=np.float32)).astype(np.float16) if dense else np.zeros(shape, np.float16)
    return out


def write_artifact(directory, tensors, arch, precision="int8", codec=None):
    """Writes manifest.json + weights.bin under `directory` (created; must not hold an artifact)."""
    if precision not in ("fp16", "int8"):
        raise ValueError("precision must be fp16/int8")
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    codec = codec or (HostCodec() if precision == "int8" else None)
    entries, whole = [], hashlib.sha256()
    with open(directory / "weights.bin", "xb") as binary:
        def put(name, dtype, array):
            raw = np.ascontiguousarray(array).tobytes()
            pad = bytes((-binary.tell()) % ALIGNMENT)
            binary.write(pad)
            whole.update(pad)
            entries.append({"name": name, "dtype": dtype, "shape": list(array.shape), "offset": binary.tell(),
                            "nbytes": len(raw), "sha256": hashlib.sha256(raw).hexdigest()})
            binary.write(raw)
            whole.update(raw)

        def put_linear(name, w16):
            if precision == "int8":
                q, scales = codec.quantize_array(w16)
                put(name, "int8", q)
                put(name + ".scales", "float32", scales)
            else:
                put(name, "float16", w16)

        for name, shape in tensor_shapes(arch).items():
            array = np.ascontiguousarray(tensors[name], np.float16)
            if list(array.shape) != shape:
                raise ValueError(f"wrong shape for {name}")
            if len(shape) == 2 and ".h." in name and name.endswith(".weight"):
                put_linear(name, array)
            else:
                put(name, "float16", array)
        put_linear("lm_head.weight", np.ascontiguousarray(tensors["transformer.wte.weight"].T, np.float16))
        size = binary.tell()
    manifest = {"schema_version": 1, "model_id": MODEL_ID, "revision": MODEL_REVISION, "source_sha256": MODEL_SHA256,
                "precision": precision, "architecture": arch, "binary": "weights.bin", "binary_bytes": size,
                "binary_sha256": whole.hexdigest(), "alignment": ALIGNMENT,
                "quantization": {"axis": "output", "range": [-127, 127], "rounding": "ties_to_even", "zero_channel_scale": 1,
                                 "reference": "fp16", "dequantize": "fp32_then_fp16"},
                "tied_head": "transpose_of_fp16_transformer.wte.weight_then_optional_quantization",
                "weights": "synthetic seeded random initialisation, not pretrained", "tensors": entries}
    (directory / "manifest.json").write_text(json.dumps(manifest, indent=1, allow_nan=False) + "\n", encoding="ascii")
    return manifest


def write_synthetic(directory, arch=None, seed=0, precision="int8", std=0.02, dense=False):
    """Seeded random model of `arch` (default GPT-2 small) -> artifact directory; returns the manifest path."""
    arch = dict(arch or GPT2_SMALL)
    directory = Path(directory)
    manifest_path = directory / "manifest.json"
    if manifest_path.exists() and (directory / "weights.bin").exists():
        existing = json.loads(manifest_path.read_text())
        if existing.get("architecture") == arch and existing.get("precision") == precision and existing.get("synthetic_seed") == seed and \
                bool(existing.get("synthetic_dense")) == dense:
            return manifest_path
        (directory / "weights.bin").unlink()
    elif (directory / "weights.bin").exists():
        (directory / "weights.bin").unlink()
    manifest = write_artifact(directory, synthetic_tensors(arch, seed, std, dense), arch, precision)
    manifest["synthetic_seed"] = seed
    manifest["synthetic_dense"] = dense
    manifest_path.write_text(json.dumps(manifest, indent=1, allow_nan=False) + "\n", encoding="ascii")
    return manifest_path


_DTYPES = {"float16": np.float16, "float32": np.float32, "int8": np.int8}


def load(manifest_path):
    """(manifest dict, {tensor name: numpy array}) with hashes checked; arrays are views of one buffer."""
    manifest_path = Path(manifest_path)
    manifest = json.loads(manifest_path.read_text(encoding="ascii"))
    blob = np.fromfile(manifest_path.parent / manifest["binary"], np.uint8)
    if blob.size != manifest["binary_bytes"] or hashlib.sha256(blob.tobytes()).hexdigest() != manifest["binary_sha256"]:
        raise ValueError("weights binary SHA256/length mismatch")
    tensors = {}
    for entry in manifest["tensors"]:
        raw = blob[entry["offset"]:entry["offset"] + entry["nbytes"]]
        tensors[entry["name"]] = raw.view(_DTYPES[entry["dtype"]]).reshape(entry["shape"])
    return manifest, tensors


def weight_bytes(manifest):
    """Bytes a decode step must read once regardless of batch: int8/fp16 linear weights, scales,
    biases and LayerNorm parameters (embedding tables are counted per token, not here)."""
    skip = ("transformer.wte.weight", "transformer.wpe.weight")
    return sum(e["nbytes"] for e in manifest["tensors"] if e["name"] not in skip)
