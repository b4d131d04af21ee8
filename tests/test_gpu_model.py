"""GPU parity of the model ABI: our runtime against the reference's runtime (compiled for
sm_100a, oracle/_ref) and the CPU oracle, on the same seeded artifact and token ids, plus the
reference's own model gate (llm/gpu_correctness.py:4-91) replayed on our runtime."""
import numpy as np
import pytest

from tests.gpu_common import LOGIT_ATOL, LOGIT_RTOL, REF_DIR

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

CACHED_ATOL, CACHED_RTOL = 0.03, 0.005      # reference llm/configs/evaluation.json:13-14


@pytest.fixture(scope="module")
def manifest(tmp_path_factory):
    from tinyinfer_b200 import artifact
    return artifact.write_synthetic(tmp_path_factory.mktemp("gpt2_small_seed0"), seed=0)


@pytest.fixture(scope="module")
def model(manifest):
    from tinyinfer_b200.runtime import NativeModel
    with NativeModel(None, manifest, max_batch=32, cache_slots=32, capacity=1024) as m:
        yield m


@pytest.fixture(scope="module")
def ref_model(manifest):
    path = REF_DIR / "libtinyinfer_llm.so"
    if not path.exists():
        pytest.skip("reference build oracle/_ref is absent")
    from tinyinfer_b200.runtime import NativeModel
    with NativeModel(path, manifest, max_batch=32, cache_slots=32, capacity=1024) as m:
        yield m


def logits_of(result):
    value = torch.frombuffer(result["logits"], dtype=torch.float32).reshape(result["shape"]).clone()
    assert torch.isfinite(value).all()
    assert result["next_tokens"] == value.argmax(-1).tolist()
    return value


def assert_logits_close(ours, theirs, what):
    """The model gate: |ours - theirs| <= 2e-2 + 1e-2 * |theirs| for every logit; prints the margin used."""
    diff = (ours - theirs).abs()
    bound = LOGIT_ATOL + LOGIT_RTOL * theirs.abs()
    print(f"{what}: max |diff| {diff.max().item():.3e}, worst diff/bound {(diff / bound).max().item():.3f}, "
          f"argmax equal {(ours.argmax(-1) == theirs.argmax(-1)).float().mean().item():.3f}")
    assert (diff <= bound).all(), f"{what}: max |diff| {diff.max().item()}"


def tokens(seed, count):
    return np.random.default_rng(seed).integers(0, 50257, count).tolist()


def test_config0_logits_and_greedy_tokens_match_reference_runtime(model, ref_model):
    """Batch 1, 32-token prompt, 64 greedy tokens, seed 0."""
    prompt = tokens(0, 32)
    model.reset_all(); ref_model.reset_all()
    ours, theirs = logits_of(model.forward([0], [prompt])), logits_of(ref_model.forward([0], [prompt]))
    assert_logits_close(ours, theirs, "config0 prompt logits")
    model.reset_all(); ref_model.reset_all()
    got = model.greedy([prompt], 64)["tokens"][0]
    want = ref_model.greedy([prompt], 64)["tokens"][0]
    assert len(got) == 64 and got[:32] == want[:32]
    agree = next((i for i, (x, y) in enumerate(zip(got, want)) if x != y), 64)
    print(f"greedy agreement with the reference runtime: first {agree} of 64 tokens")


def test_decode_logits_track_reference_step_by_step(model, ref_model):
    prompt = tokens(7, 40)
    model.reset_all(); ref_model.reset_all()
    a, b = model.forward([3], [prompt]), ref_model.forward([3], [prompt])
    for step in range(24):
        la, lb = logits_of(a), logits_of(b)
        assert_logits_close(la, lb, f"decode step {step}")
        nxt = b["next_tokens"][0]                   # teacher-force the reference's token so histories stay equal
        a, b = model.forward([3], [[nxt]]), ref_model.forward([3], [[nxt]])


def test_logits_match_cpu_oracle(model, manifest):
    from oracle import ti_oracle as orc
    from tinyinfer_b200 import artifact
    meta, tensors = artifact.load(manifest)
    oracle = orc.Gpt2Oracle(tensors, meta["architecture"])
    prompt = tokens(1, 12)
    model.reset_all()
    ours = logits_of(model.forward([0], [prompt]))[0]
    want = torch.from_numpy(oracle.forward(0, prompt))
    torch.testing.assert_close(ours, want, atol=LOGIT_ATOL, rtol=LOGIT_RTOL)
    step = logits_of(model.forward([0], [[int(want.argmax())]]))[0]
    torch.testing.assert_close(step, torch.from_numpy(oracle.forward(0, [int(want.argmax())])), atol=LOGIT_ATOL, rtol=LOGIT_RTOL)


def test_reference_model_gate_on_our_runtime(model):
    """llm/gpu_correctness.py:13-72 without the HF branch."""
    ids = tokens(42, 64)
    prompts = [ids[0:33], ids[41:58]]
    model.reset_all()
    independent = []
    for prompt in prompts:
        model.reset(0)
        independent.append(logits_of(model.forward([0], [prompt]))[0])
    full = torch.stack(independent)
    model.reset_all()
    batched = logits_of(model.forward([0, 1], prompts))
    torch.testing.assert_close(batched, full, atol=CACHED_ATOL, rtol=CACHED_RTOL)
    model.reset_all()
    model.forward([0, 1], [p[:3] for p in prompts], return_logits=False, return_next=False)
    cached = logits_of(model.forward([0, 1], [p[3:] for p in prompts]))
    torch.testing.assert_close(cached, full, atol=CACHED_ATOL, rtol=CACHED_RTOL)
    model.reset(0)
    survivor = logits_of(model.forward([1], [[ids[59]]]))
    model.reset(2)
    expected = logits_of(model.forward([2], [prompts[1] + [ids[59]]]))
    torch.testing.assert_close(survivor, expected, atol=CACHED_ATOL, rtol=CACHED_RTOL)
    before = model.lengths()
    for slots, rows in (([1, 1], [[3], [4]]), ([1], [[3] * model.options.capacity])):
        with pytest.raises(RuntimeError):
            model.forward(slots, rows, return_logits=False, return_next=False)
        assert model.lengths() == before
    score = model.score(ids[:33], [0] + [1] * 32, positions=True)
    assert model.lengths() == before and score["target_count"] == 32
    assert abs(sum(score["position_nll"]) - score["sum_nll"]) <= 1e-7 * max(1., score["sum_nll"])
    subset_mask = [0] + [int(i % 3 != 0) for i in range(1, 33)]
    subset = model.score(ids[:33], subset_mask, positions=True)
    want = sum(v for v, use in zip(score["position_nll"], subset_mask) if use)
    assert subset["target_count"] == sum(subset_mask) and abs(subset["sum_nll"] - want) <= 1e-7 * max(1., want)
    assert all(v == 0 for v, use in zip(subset["position_nll"], subset_mask) if not use)
    model.reset_all()
    gen_prompts, requested = [prompts[0][:7], prompts[1][:5]], [3, 1]
    mixed = model.greedy(gen_prompts, requested, slots=[0, 1])
    assert mixed["output_lengths"] == requested and model.lengths()[:2] == [9, 5]
    for row, count, generated in zip(gen_prompts, requested, mixed["tokens"]):
        model.reset(2)
        assert model.greedy([row], count, slots=[2])["tokens"][0] == generated
    trace = model.trace()
    for key in ("embedding", "gemm_int8", "layernorm", "gelu", "attention", "residual", "kv_scatter_gather", "lm_head", "argmax", "nll"):
        assert trace[key] > 0, key
    model.reset_all()


def test_score_matches_reference_runtime(model, ref_model):
    ids = tokens(9, 48)
    mask = [0] + [1] * 47
    a, b = model.score(ids, mask, positions=True), ref_model.score(ids, mask, positions=True)
    assert a["target_count"] == b["target_count"] == 47
    assert abs(a["sum_nll"] - b["sum_nll"]) <= 2e-3 * b["sum_nll"]
    np.testing.assert_allclose(a["position_nll"], b["position_nll"], atol=3e-2, rtol=1e-2)


def test_config2_ragged_batch32_decode_matches_reference(model, ref_model):
    """Batch 32, prompt lengths uniform in [16,512], greedy continuation, seed 2 (shortened to 16 tokens)."""
    rng = np.random.default_rng(2)
    lengths = rng.integers(16, 513, 32)
    prompts = [rng.integers(0, 50257, int(n)).tolist() for n in lengths]
    model.reset_all(); ref_model.reset_all()
    ours = logits_of(model.forward(list(range(32)), prompts))
    theirs = logits_of(ref_model.forward(list(range(32)), prompts))
    assert_logits_close(ours, theirs, "config2 ragged prefill logits")
    nxt = theirs.argmax(-1).tolist()
    for _ in range(4):
        a = logits_of(model.forward(list(range(32)), [[t] for t in nxt]))
        b = logits_of(ref_model.forward(list(range(32)), [[t] for t in nxt]))
        assert_logits_close(a, b, "config2 decode step")
        nxt = b.argmax(-1).tolist()
    assert model.lengths() == ref_model.lengths()
    model.reset_all(); ref_model.reset_all()
    got = model.greedy(prompts, 16)["tokens"]
    want = ref_model.greedy(prompts, 16)["tokens"]
    same = sum(g == w for g, w in zip(got, want))
    print(f"batch-32 ragged greedy: {same}/32 requests identical over 16 tokens")
    assert same >= 28


def test_slot_reuse_and_page_recycling(model):
    prompt = tokens(5, 70)
    model.reset_all()
    first = logits_of(model.forward([5], [prompt]))
    for slot in (6, 7, 8):
        model.forward([slot], [tokens(slot, 100)], return_logits=False, return_next=False)
    model.reset(5); model.reset(7)
    again = logits_of(model.forward([7], [prompt]))
    assert torch.equal(first, again)               # same kernels, same order: bit-identical whatever pages are used
    model.reset_all()
    assert model.lengths() == [0] * 32


def test_validation_errors_and_struct_size(model, manifest):
    import ctypes as C
    from tinyinfer_b200.runtime import NativeModel, Options
    with pytest.raises(RuntimeError):
        model.greedy([[1, 2, 3]], 1022)            # prompt + new tokens exceeds capacity
    model.forward([0], [[1, 2]], return_logits=False, return_next=False)
    with pytest.raises(RuntimeError):
        model.greedy([[1]], 1, slots=[0])          # greedy needs an empty slot
    model.reset_all()
    lib = model.lib
    bad = Options(24, 0, 1, 1, 16, 0, 0)
    handle = C.c_void_p()
    assert lib.ti_llm_create(str(manifest).encode(), C.byref(bad), C.byref(handle)) == 1 and not handle
    with pytest.raises(ValueError):
        NativeModel(None, manifest, max_batch=65, cache_slots=65)


def test_logits_do_not_depend_on_batch_composition(model):
    """The reference's batched-vs-single and mixed-greedy gates hold there with difference exactly 0
    (one kernel serves every M).  Same property here: bit-equal logits alone or in a ragged batch of 9,
    at prefill and at decode, and identical greedy tokens."""
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, 50257, int(n)).tolist() for n in (3, 70, 1, 33, 128, 17, 64, 5, 200)]
    model.reset_all()
    together = logits_of(model.forward(list(range(9)), prompts))
    step = logits_of(model.forward(list(range(9)), [[int(t)] for t in together.argmax(-1)]))
    for i in (0, 2, 4, 8):
        model.reset(20)
        alone = logits_of(model.forward([20], [prompts[i]]))[0]
        assert torch.equal(alone, together[i]), f"prefill logits of request {i} depend on the batch"
        alone_step = logits_of(model.forward([20], [[int(together[i].argmax())]]))[0]
        assert torch.equal(alone_step, step[i]), f"decode logits of request {i} depend on the batch"
    model.reset_all()
    batch_tokens = model.greedy(prompts, [12, 3, 9, 1, 6, 12, 2, 7, 4])["tokens"]
    for i in (1, 2, 5, 7):
        model.reset(20)
        assert model.greedy([prompts[i]], len(batch_tokens[i]), slots=[20])["tokens"][0] == batch_tokens[i]
    model.reset_all()


def test_admissions_folded_into_a_decode_step_change_nothing(model):
    """The server appends the prompts of newly admitted requests to the decode step of the running ones (one pass).
    Running requests must get bit-identical logits whether or not prompts ride along (their attention takes the
    decode kernel in both cases), and the newcomers the same logits as in a pass of their own."""
    rng = np.random.default_rng(33)
    running = [rng.integers(0, 50257, int(n)).tolist() for n in (40, 300, 97)]
    newcomers = [rng.integers(0, 50257, int(n)).tolist() for n in (150, 1, 31)]
    model.reset_all()
    ids = [int(t) for t in logits_of(model.forward([0, 1, 2], running)).argmax(-1)]
    step_alone = logits_of(model.forward([0, 1, 2], [[t] for t in ids]))
    prefill_alone = logits_of(model.forward([3, 4, 5], newcomers))
    model.reset_all()
    model.forward([0, 1, 2], running, return_logits=False)
    order = [3, 0, 4, 1, 2, 5]
    rows = [newcomers[0], [ids[0]], newcomers[1], [ids[1]], [ids[2]], newcomers[2]]
    mixed = logits_of(model.forward(order, rows))
    assert torch.equal(mixed[[1, 3, 4]], step_alone), "a running request's logits depend on the admissions in its step"
    assert torch.equal(mixed[[0, 2, 5]], prefill_alone), "a prompt's logits depend on the decode rows it travels with"
    model.reset_all()


def test_step_by_step_decoding_with_speculative_continuation(model):
    """A caller that feeds the model's outputs back through forward() gets, after a few steps, its next step launched
    ahead of the call.  Tokens must equal greedy()'s, also when the caller stops continuing (another token, another
    slot set, a reset) while a speculative step is in flight."""
    rng = np.random.default_rng(44)
    prompts = [rng.integers(0, 50257, int(n)).tolist() for n in (20, 75, 140)]
    model.reset_all()
    want = model.greedy(prompts, 40)["tokens"]
    model.reset_all()
    ids = model.forward([0, 1, 2], prompts, return_logits=False)["next_tokens"]
    got = [[t] for t in ids]
    for _ in range(39):
        ids = model.forward([0, 1, 2], [[t] for t in ids], return_logits=False)["next_tokens"]
        for row, t in zip(got, ids):
            row.append(t)
    assert got == want
    assert model.lengths()[:3] == [len(p) + 39 for p in prompts]
    # break the pattern: request 1 continues with another token than the one predicted; compare with a fresh context
    forced = [ids[0], (ids[1] + 1) % 50257, ids[2]]
    after = logits_of(model.forward([0, 1, 2], [[t] for t in forced]))
    model.reset_all()
    model.forward([5, 6, 7], [p + g[:39] for p, g in zip(prompts, want)], return_logits=False)
    fresh = logits_of(model.forward([5, 6, 7], [[t] for t in forced]))
    # (the fresh context was prefilled in one pass, the other grew token by token: same values up to summation order)
    assert torch.allclose(after, fresh, atol=5e-3, rtol=0) and torch.equal(after.argmax(-1), fresh.argmax(-1))
    # continue long enough to arm again, then reset one slot and reuse it while a speculative step may be in flight
    ids = [int(t) for t in fresh.argmax(-1)]
    for _ in range(12):
        ids = model.forward([5, 6, 7], [[t] for t in ids], return_logits=False)["next_tokens"]
    model.reset(6)
    again = logits_of(model.forward([6], [prompts[0]]))
    model.reset_all()
    alone = logits_of(model.forward([0], [prompts[0]]))
    assert torch.equal(again, alone)
    model.reset_all()


def test_medium_shape_matches_cpu_oracle(tmp_path_factory):
    """GPT-2 medium shape (24 layers, 16 heads, hidden 1024), seed 3: the reference runtime cannot load it
    (compile-time 12/12/768), so the operator-composed CPU oracle is the reference here."""
    from oracle import ti_oracle as orc
    from tinyinfer_b200 import artifact
    from tinyinfer_b200.runtime import NativeModel
    manifest = artifact.write_synthetic(tmp_path_factory.mktemp("gpt2_medium_seed3"), artifact.GPT2_MEDIUM, seed=3)
    meta, tensors = artifact.load(manifest)
    oracle = orc.Gpt2Oracle(tensors, meta["architecture"])
    prompt = tokens(3, 10)
    with NativeModel(None, manifest, max_batch=8, cache_slots=8, capacity=64) as m:
        ours = logits_of(m.forward([0], [prompt]))[0]
        want = torch.from_numpy(oracle.forward(0, prompt))
        assert_logits_close(ours[None], want[None], "medium prompt logits vs oracle")
        nxt = int(want.argmax())
        step = logits_of(m.forward([0], [[nxt]]))[0]
        assert_logits_close(step[None], torch.from_numpy(oracle.forward(0, [nxt]))[None], "medium decode logits vs oracle")
        m.reset_all()
        batch = m.greedy([prompt, prompt[:4]], [6, 3])
        m.reset_all()
        assert m.greedy([prompt], 6)["tokens"][0] == batch["tokens"][0]


def test_two_devices_in_one_process(manifest):
    """One model context per GPU inside one process (what the server's workers do): both give the same tokens."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from tinyinfer_b200.runtime import NativeModel
    prompt = tokens(4, 20)
    with NativeModel(None, manifest, device=0, max_batch=4, cache_slots=4, capacity=128) as a, \
            NativeModel(None, manifest, device=1, max_batch=4, cache_slots=4, capacity=128) as b:
        ta = a.greedy([prompt, prompt[:5]], [10, 4])["tokens"]
        tb = b.greedy([prompt, prompt[:5]], [10, 4])["tokens"]
        assert ta == tb
        la = logits_of(a.forward([2], [prompt]))
        lb = logits_of(b.forward([2], [prompt]))
        assert torch.equal(la, lb)


def _inject(model, kind, after=0):
    import ctypes as C
    fn = model.lib.ti_b200_llm_inject_failure
    fn.argtypes, fn.restype = [C.c_void_p, C.c_int32, C.c_int32], C.c_int
    assert fn(model._model, kind, after) == 0


@pytest.mark.parametrize("kind", [0, 1], ids=["host_exception", "device_wait_runs_out"])
def test_execution_failure_poisons_the_model(manifest, kind):
    """Reference semantics (llm/src/runtime.cu:127,172-174, tinyinfer_llm.h:9-11): an execution failure returns
    TI_LLM_CUDA / INTERNAL, every later call fails until destroy, lengths stay as they were, destroy works.
    kind 0 throws on the host inside the second forward call; kind 1 lets a one-thread kernel's bounded wait run out
    (microseconds; nothing faults), which the next synchronising call finds in the device status word."""
    from tinyinfer_b200.runtime import NativeModel
    prompt = tokens(8, 12)
    with NativeModel(None, manifest, max_batch=2, cache_slots=2, capacity=64) as m:
        first = m.forward([0], [prompt], return_logits=False)["next_tokens"]
        before = m.lengths()
        _inject(m, kind, 0)
        with pytest.raises(RuntimeError) as failed:
            m.forward([0], [first], return_logits=False)
        assert "status 3" in str(failed.value)                      # TI_LLM_CUDA
        for call in (lambda: m.forward([1], [prompt]), lambda: m.lengths(), lambda: m.reset(0), lambda: m.greedy([prompt], 2, slots=[1])):
            with pytest.raises(RuntimeError) as again:
                call()
            assert "poisoned" in str(again.value)
    # a fresh context on the same device works (the status word was cleared with the failure)
    with NativeModel(None, manifest, max_batch=2, cache_slots=2, capacity=64) as m:
        assert m.forward([0], [prompt], return_logits=False)["next_tokens"] == first
        assert m.lengths() == before
