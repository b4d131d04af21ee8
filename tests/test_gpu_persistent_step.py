"""The persistent decode step (one kernel per greedy step, csrc/decode_step.cuh) against the launch-per-operation step
it replaces (reference loop llm/src/runtime.cu:135-168): same logits bit for bit, same tokens, same cache contents,
on artifacts whose biases and LayerNorm parameters are all non-trivial; and against the reference runtime itself."""
import numpy as np
import pytest

from tests.gpu_common import LOGIT_ATOL, LOGIT_RTOL, REF_DIR

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def logits_of(result):
    return torch.frombuffer(result["logits"], dtype=torch.float32).reshape(result["shape"]).clone()


def prompts_of(seed, lengths):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, 50257, int(n)).tolist() for n in lengths]


@pytest.fixture(scope="module")
def dense_manifest(tmp_path_factory):
    from tinyinfer_b200 import artifact
    return artifact.write_synthetic(tmp_path_factory.mktemp("gpt2_small_dense"), seed=5, dense=True)


@pytest.fixture(scope="module")
def model(dense_manifest):
    from tinyinfer_b200.runtime import NativeModel
    with NativeModel(None, dense_manifest, max_batch=32, cache_slots=32, capacity=1024) as m:
        yield m


def run_plan(model, plan, prompts, steps, forced=None):
    """Prefill, then `steps` single-token passes with logits; returns (list of logits per step, tokens fed)."""
    assert model.decode_plan(plan) == plan
    model.reset_all()
    slots = list(range(len(prompts)))
    out = model.forward(slots, prompts)
    ids = out["next_tokens"]
    history, fed = [], []
    for step in range(steps):
        if forced is not None:
            ids = forced[step]
        fed.append(list(ids))
        out = model.forward(slots, [[t] for t in ids])
        history.append(logits_of(out))
        assert out["next_tokens"] == history[-1].argmax(-1).tolist()
        ids = out["next_tokens"]
    return history, fed


@pytest.mark.parametrize("lengths", [(32,), (5, 140, 33, 64, 1), tuple(np.random.default_rng(2).integers(16, 513, 32))],
                         ids=["batch1", "batch5", "batch32"])
def test_logits_bit_identical_to_launch_per_operation_step(model, lengths):
    if model.decode_plan(1) != 1:
        pytest.skip("persistent step not available on this device")
    prompts = prompts_of(11, lengths)
    graph, fed = run_plan(model, 0, prompts, 6)
    fused, _ = run_plan(model, 1, prompts, 6, forced=fed)
    for step, (a, b) in enumerate(zip(fused, graph)):
        assert torch.isfinite(a).all()
        assert torch.equal(a, b), f"step {step}: max |diff| {(a - b).abs().max().item()}"
    model.reset_all()


def test_device_resident_steps_and_greedy_match_the_other_plan(model):
    if model.decode_plan(1) != 1:
        pytest.skip("persistent step not available on this device")
    prompts = prompts_of(12, (20, 75, 140, 9, 300, 31, 64))
    tokens = {}
    for plan in (0, 1):
        model.decode_plan(plan)
        model.reset_all()
        tokens[plan] = model.greedy(prompts, [40, 3, 17, 40, 8, 1, 25])["tokens"]
    assert tokens[0] == tokens[1]
    # cache contents written by the fused step serve the other plan: continue a fused prefix with the graph plan
    model.decode_plan(1)
    model.reset_all()
    first = model.forward([0, 1], prompts[:2], return_logits=False)["next_tokens"]
    mid = model.decode_steps([0, 1], first, 12)["tokens"]
    model.decode_plan(0)
    tail_graph = model.decode_steps([0, 1], mid[-1], 5)["tokens"]
    model.reset_all()
    first2 = model.forward([0, 1], prompts[:2], return_logits=False)["next_tokens"]
    assert first2 == first
    all_graph = model.decode_steps([0, 1], first2, 17)["tokens"]
    assert all_graph[:12] == mid and all_graph[12:] == tail_graph
    model.decode_plan(1)
    model.reset_all()


def test_dense_artifact_matches_reference_runtime(model, dense_manifest):
    """Every bias and LayerNorm parameter non-zero: logits of both plans against the reference's own runtime."""
    path = REF_DIR / "libtinyinfer_llm.so"
    if not path.exists():
        pytest.skip("reference build oracle/_ref is absent")
    from tinyinfer_b200.runtime import NativeModel
    prompts = prompts_of(13, (32, 7, 200, 64))
    with NativeModel(path, dense_manifest, max_batch=4, cache_slots=4, capacity=1024) as ref:
        theirs = logits_of(ref.forward([0, 1, 2, 3], prompts))
        model.decode_plan(1)
        model.reset_all()
        ours = logits_of(model.forward([0, 1, 2, 3], prompts))
        bound = LOGIT_ATOL + LOGIT_RTOL * theirs.abs()
        assert ((ours - theirs).abs() <= bound).all()
        ids = theirs.argmax(-1).tolist()
        for step in range(8):
            a = logits_of(model.forward([0, 1, 2, 3], [[t] for t in ids]))
            b = logits_of(ref.forward([0, 1, 2, 3], [[t] for t in ids]))
            diff = (a - b).abs()
            assert (diff <= LOGIT_ATOL + LOGIT_RTOL * b.abs()).all(), f"step {step}: max |diff| {diff.max().item()}"
            ids = b.argmax(-1).tolist()
    model.reset_all()


@pytest.mark.parametrize("arch_name", ["tiny", "medium"])
def test_other_shapes(tmp_path_factory, arch_name):
    """A 2-layer / 256-wide model (4 K ranges per GEMM) and the GPT-2 medium shape (24 layers, hidden 1024)."""
    from tinyinfer_b200 import artifact
    from tinyinfer_b200.runtime import NativeModel
    arch = ({**artifact.GPT2_SMALL, "layers": 2, "heads": 4, "hidden": 256, "capacity": 128} if arch_name == "tiny"
            else {**artifact.GPT2_MEDIUM, "capacity": 128})
    manifest = artifact.write_synthetic(tmp_path_factory.mktemp(f"gpt2_{arch_name}_dense"), arch, seed=6, dense=True)
    with NativeModel(None, manifest, max_batch=8, cache_slots=8, capacity=128) as m:
        if m.decode_plan(1) != 1:
            pytest.skip("persistent step not available for this shape")
        prompts = prompts_of(14, (10, 3, 40, 1, 22))
        graph, fed = run_plan(m, 0, prompts, 5)
        fused, _ = run_plan(m, 1, prompts, 5, forced=fed)
        for step, (a, b) in enumerate(zip(fused, graph)):
            assert torch.equal(a, b), f"{arch_name} step {step}: max |diff| {(a - b).abs().max().item()}"
        m.reset_all()
        assert m.decode_plan(0) == 0
        want = m.greedy(prompts, 12)["tokens"]
        m.decode_plan(1)
        m.reset_all()
        assert m.greedy(prompts, 12)["tokens"] == want
