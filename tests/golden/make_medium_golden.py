"""Generates tests/golden/medium_prefill_golden.json: logits of the CPU oracle (oracle/ti_oracle.py, the reference's
forward sequence llm/src/runtime.cu:135-168 restated) for the GPT-2 medium shape at the size of the prefill
configuration -- 768-token prompts, seed 3 -- which the reference runtime cannot load (compile-time 12 layers / 768).

    python tests/golden/make_medium_golden.py          # CPU only, a few minutes

The artifact is the seed-3 synthetic one of tinyinfer_b200.artifact (regenerated from the seed wherever the test
runs).  For requests 0 and 5 of the eight prompts the oracle's last-position logits after the prefill, and after one
decode step on the oracle's own next token, are sampled at every 61st vocabulary index plus the 16 largest ones.
"""
import json
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import ti_oracle as orc          # noqa: E402
from tinyinfer_b200 import artifact          # noqa: E402

SAMPLED_REQUESTS = (0, 5)


def prompts():
    rng = np.random.default_rng(3)
    return [rng.integers(0, 50257, 768).tolist() for _ in range(8)]


def sample(logits):
    index = sorted(set(range(0, 50257, 61)) | set(np.argsort(logits)[-16:].tolist()))
    return {"index": index, "value": [float(logits[i]) for i in index], "argmax": int(orc.argmax(logits[None])[0])}


def main():
    with tempfile.TemporaryDirectory() as tmp:
        manifest = artifact.write_synthetic(Path(tmp) / "medium", artifact.GPT2_MEDIUM, seed=3)
        meta, tensors = artifact.load(manifest)
        oracle = orc.Gpt2Oracle(tensors, meta["architecture"])
        out = {"artifact": "tinyinfer_b200.artifact.write_synthetic(GPT2_MEDIUM, seed=3)", "prompts": "numpy default_rng(3), 8 x 768 ids uniform in [0, 50257)",
               "binary_sha256": meta["binary_sha256"], "requests": {}}
        all_prompts = prompts()
        for r in SAMPLED_REQUESTS:
            prefill = oracle.forward(r, all_prompts[r])
            first = sample(prefill)
            step = oracle.forward(r, [first["argmax"]])
            out["requests"][str(r)] = {"prefill": first, "decode": sample(step)}
            oracle.reset(r)
            print("request", r, "done", flush=True)
    path = Path(__file__).with_name("medium_prefill_golden.json")
    path.write_text(json.dumps(out) + "\n")
    print("wrote", path)


if __name__ == "__main__":
    main()
