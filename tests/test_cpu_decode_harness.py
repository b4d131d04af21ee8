"""The CPU decode harness used as the timed baseline computes the same model as the oracle."""
import numpy as np

from oracle import cpu_decode
from oracle import ti_oracle as orc
from tinyinfer_b200 import artifact

TINY = {**artifact.GPT2_SMALL, "layers": 2, "heads": 2, "hidden": 128, "capacity": 32}


def test_cpu_harness_tracks_the_oracle(tmp_path):
    manifest_path = artifact.write_synthetic(tmp_path / "tiny", TINY, seed=3, std=0.05)
    meta, tensors = artifact.load(manifest_path)
    oracle = orc.Gpt2Oracle(tensors, meta["architecture"])
    dec = cpu_decode.CpuDecoder(tensors, meta["architecture"])
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 50257, n).tolist() for n in (5, 3)]
    dec.start([0, 0], capacity=16)
    # feed the prompts token by token (request 1 is shorter: pad its tail with repeats that we ignore)
    logits = None
    for t in range(3):
        _, logits = dec.step([prompts[0][t], prompts[1][t]])
    want1 = oracle.forward(1, prompts[1])
    np.testing.assert_allclose(logits[1], want1, atol=3e-2, rtol=2e-2)
    assert int(np.argmax(logits[1])) == int(orc.argmax(want1[None])[0])
    assert dec.k.kind in ("reference", "port")


def test_time_decode_reports_throughput(tmp_path):
    manifest_path = artifact.write_synthetic(tmp_path / "tiny", TINY, seed=3)
    meta, tensors = artifact.load(manifest_path)
    out = cpu_decode.time_decode(tensors, meta["architecture"], [4, 9, 1], steps=2, warmup=1)
    assert out["tokens_per_s"] > 0 and out["steps"] == 2 and out["cores"] >= 1
