#!/usr/bin/env python
"""Benchmark of the INT8-weight GPT-2 decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the metric's batched decode configuration): GPT-2 small, INT8 weights, random-init
artifact (seed 0), batch 32 per GPU, prompt lengths uniform in [16, 512], 128 new tokens per
request, token ids uniform, seed 2.  One "step" is one decode step of the whole batch (32 tokens);
the default K + W covers the 127 decode steps of the 128-token generation.  With N > 1 every rank
holds a full replica on its own GPU and runs the same per-GPU workload (weak scaling, no
collective on the data path); the timed region is bracketed by barrier + synchronize and the
slowest rank's device time is used.

Printed JSON (one line, rank 0):
  value      tokens/s with tokens, positions and KV cache resident on the GPU between steps
             (ti_b200_llm_decode_steps; CUDA events on the model's stream)
  e2e        tokens/s through the per-step reference-facing call ti_llm_forward_batch: every step
             copies the step's ids + metadata from pinned host memory to the GPU and reads the
             step's next-token ids back to the host
  roofline   the dominant kernel -- the persistent decode step, one launch per step: algorithmic weight + KV
             bytes of a step over the mean launch duration (CUDA events over the timed region) against the
             measured copy bandwidth of this pool's B200s
  config0    the batch-1 configuration (32-token prompt, 63 decode steps) the HBM-roofline target is stated on
  cpu_baseline  the decode sequence composed from the reference's own CPU kernels, timed on the
             host cores for a bounded sample of the same workload

--impl reference times the reference's own runtime (its CUDA kernels compiled unmodified for sm_100a into
oracle/_ref) on the same workload through the same per-step call; when that build is absent it falls back to the CPU
composition.  The reference has no CPU GPT-2 runtime of its own.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

BATCH, NEW_TOKENS, PROMPT_LO, PROMPT_HI, WORKLOAD_SEED, WEIGHT_SEED = 32, 128, 16, 512, 2, 0
WORKLOAD = ("GPT-2 small INT8-weight batched decode: batch 32 per GPU, prompt lengths uniform in [16,512], "
            "128 new tokens per request, seed 2")
FALLBACK_HBM_GBS = 6650.0


def workload_prompts():
    rng = np.random.default_rng(WORKLOAD_SEED)
    lengths = rng.integers(PROMPT_LO, PROMPT_HI + 1, BATCH)
    return [rng.integers(0, 50257, int(n)).tolist() for n in lengths]


def artifact_path():
    """Seeded random GPT-2 small artifact, written once per machine."""
    from tinyinfer_b200 import artifact
    base = Path(os.environ.get("TINYINFER_B200_CACHE", Path(tempfile.gettempdir()) / "tinyinfer_b200_bench"))
    return artifact.write_synthetic(base / f"gpt2_small_int8_seed{WEIGHT_SEED}", seed=WEIGHT_SEED)


def peak_hbm():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def step_bytes(weight_bytes, cached, hidden=768, kv_per_position=36864):
    """Algorithmic bytes of one decode step: every weight byte once, plus per request one wte and
    one wpe row and its KV history read (cached positions) and extended (one position)."""
    return weight_bytes + sum(2 * hidden * 2 + kv_per_position * (t + 1) for t in cached)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.rows, self.proc = device, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.device)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *_):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()

    def summary(self):
        good = [r for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        if not good:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in good for n, v in zip(names, r[5:9]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(float(r[1]) for r in good), "sm_max_mhz": float(good[0][2]), "reasons": reasons,
                "samples": len(good), "power_w_max": max(float(r[3]) for r in good if r[3].replace(".", "").isdigit())}


# ---------------------------------------------------------------------------- CPU arm
def cpu_arm(steps, warmup, threads=None):
    from oracle import cpu_decode
    from tinyinfer_b200 import artifact
    meta, tensors = artifact.load(artifact_path())
    lengths = [len(p) + NEW_TOKENS // 2 for p in workload_prompts()]        # cache sizes mid-way through the generation
    result = cpu_decode.time_decode(tensors, meta["architecture"], lengths, steps, warmup, seed=WORKLOAD_SEED, threads=threads)
    sample = (f"{steps} decode steps (+{warmup} warm-up) of the batch-32 workload at its mid-generation cache lengths; KV histories "
              "filled with random values instead of running the prefill; harness composed from the reference's ti_cpu_gemm/"
              "ti_cpu_layernorm/ti_cpu_softmax + host codec" if result["kind"] == "reference" else
              f"{steps} decode steps of the batch-32 workload on the numpy port (oracle/_ref absent)")
    return result, sample


def config_block(world):
    return {"workload": WORKLOAD, "replicas": world, "l2": "inputs larger than L2 (about 0.5 GB of weights + KV per step)",
            "weights": f"random N(0,0.02), seed {WEIGHT_SEED}"}


def physical_cores():
    """Cores this process may use (the launcher may have set OMP_NUM_THREADS=1, which is not a property of the machine)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def setup_ranks():
    """(torch, dist or None, local rank): one process per GPU; NCCL only for the barrier and the max / sum of the timing."""
    import torch
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        # stdout carries the one JSON line: while the communicator comes up (NCCL prints a version banner on file
        # descriptor 1 when NCCL_DEBUG is set) descriptor 1 points at stderr
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    return torch, dist, local


def reference_main(args, rank, world):
    """The reference's own runtime on this box: oracle/_ref/libtinyinfer_llm.so is llm/src/runtime.cu and its WMMA
    kernels compiled unmodified for sm_100a.  Same artifact, same prompts, same per-step call (ti_llm_forward_batch with
    host ids in, host ids out), one replica per GPU like the other arm.  Without that build: the CPU composition."""
    ref_lib = ROOT / "oracle" / "_ref" / "libtinyinfer_llm.so"
    K, W = max(1, args.steps), max(3, args.warmup)
    line = {"impl": "reference", "metric": "int8_gpt2_decode_tokens_per_s", "unit": "tokens/s", "n_gpus": args.gpus, "steps": K,
            "warmup": W, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic", "config": config_block(world)}
    if not ref_lib.exists():
        if rank != 0:
            return
        result, sample = cpu_arm(min(K, 6), 1, threads=physical_cores())
        line.update({"value": result["tokens_per_s"], "ms_per_step": result["seconds_per_step"] * 1e3, "dtype": "f32", "gpu_launches": 0,
                     "reference_runs_on": "host CPU cores (oracle/_ref CUDA build absent)",
                     "cpu_baseline": {"value": result["tokens_per_s"], "unit": "tokens/s", "cores": result["cores"], "kind": result["kind"], "sample": sample},
                     "e2e": {"value": result["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        print(json.dumps(line))
        return
    torch, dist, local = setup_ranks()
    from tinyinfer_b200.runtime import NativeModel
    from tinyinfer_b200 import replicas
    if rank == 0:
        artifact_path()
    if dist:
        dist.barrier()
    prompts, slots = workload_prompts(), list(range(BATCH))
    with NativeModel(ref_lib, artifact_path(), device=local, max_batch=BATCH, cache_slots=BATCH, capacity=1024) as model:
        t0 = time.perf_counter()
        ids = model.forward(slots, prompts, return_logits=False)["next_tokens"]
        ttft_ms = (time.perf_counter() - t0) * 1e3
        for _ in range(W):
            ids = model.forward(slots, [[t] for t in ids], return_logits=False)["next_tokens"]
        steps = min(K, 1024 - max(model.lengths()[:BATCH]) - 1)
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        with ClockSampler(local) as clocks:
            t0 = time.perf_counter()
            for _ in range(steps):
                ids = model.forward(slots, [[t] for t in ids], return_logits=False)["next_tokens"]      # returns after its own stream sync
            seconds = time.perf_counter() - t0
        trace = model.trace()
    _, slowest, value = replicas.job_throughput(BATCH * steps, seconds, dist, "cuda")
    if rank == 0:
        line.update({"value": value, "ms_per_step": slowest / steps * 1e3, "steps": steps, "dtype": "f16 activations x int8 weights, f32 accumulate",
                     "reference_runs_on": "the same B200: reference CUDA runtime (WMMA kernels, about 161 launches per step) compiled for sm_100a",
                     "prefill_ttft_ms": ttft_ms, "clocks": clocks.summary(), "gpu_launches": 0,
                     "reference_trace": {k: trace[k] for k in ("forward_calls", "gemm_int8", "attention")},
                     "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 5 * BATCH * 4, "d2h_bytes_per_step": BATCH * 4,
                             "api": "ti_llm_forward_batch per step (the timed call itself)"}})
        if world == 1 and not args.no_cpu:
            result, sample = cpu_arm(steps=int(os.environ.get("TINYINFER_B200_CPU_STEPS", 4)), warmup=1, threads=physical_cores())
            line["cpu_baseline"] = {"value": result["tokens_per_s"], "unit": "tokens/s", "cores": result["cores"], "kind": result["kind"], "sample": sample}
        print(json.dumps(line))
    if dist:
        dist.barrier()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------- GPU arm
def graph_seconds(enqueue, launches, replays=10):
    """Device seconds per kernel launch: `enqueue()` issues `launches` kernels on the current stream
    through the raw C ABI; they are captured into a CUDA graph once and the graph is replayed, so no
    host work sits between launches and the CUDA events time the GPU alone."""
    import torch
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        enqueue()                                   # first call: function attributes, tensor-map driver entry
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        enqueue()
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e-3 / (replays * launches)


def kernel_rooflines(cached, peak):
    """The kernel families that carry a decode step's bytes, timed alone on the step's shapes.  Each
    round walks distinct buffers totalling more than the 126 MB L2, so every launch streams from HBM
    as it does inside a real step (where ~0.5 GB passes between two uses of the same weights)."""
    import torch
    from tinyinfer_b200.native_ops import NativeOps
    ops = NativeOps()
    lib, dev = ops.lib, torch.cuda.current_device()
    out = {}
    stream = lambda: torch.cuda.current_stream().cuda_stream

    def check(status):
        if status:
            raise RuntimeError(lib.ti_v2_last_error().decode())

    # decode attention over the ragged histories, one launch per "layer" with its own K/V
    kmax, layers = max(cached) + 1, 12
    lengths = torch.tensor([t + 1 for t in cached], dtype=torch.int32, device="cuda")
    q = torch.randn((BATCH, 12, 1, 64), device="cuda").half()
    y = torch.empty_like(q)
    kv = [(torch.randn((BATCH, 12, kmax, 64), device="cuda", dtype=torch.float16), torch.randn((BATCH, 12, kmax, 64), device="cuda", dtype=torch.float16))
          for _ in range(layers)]
    chunk = (kmax + 31) // 32 * 32          # one CTA per (request, head), as the model runtime launches it
    floats = lib.ti_b200_attention_decode_scratch_floats(BATCH, 12, kmax, chunk)
    scratch = torch.empty(floats, dtype=torch.float32, device="cuda")
    def attn():
        for k, v in kv:
            check(lib.ti_b200_attention_decode_f16(q.data_ptr(), k.data_ptr(), v.data_ptr(), y.data_ptr(), lengths.data_ptr(), BATCH, 12, kmax, 64, chunk,
                                                   scratch.data_ptr(), floats, stream(), dev))
    seconds = graph_seconds(attn, layers)
    nbytes = int(lengths.sum().item()) * 12 * 64 * 2 * 2 + BATCH * 12 * 64 * 2 * 2
    out["attention_decode (1 layer: 32 ragged requests x 12 heads)"] = {"seconds": seconds, "bytes": nbytes, "launches_per_step": 12}
    del kv

    def gemm_family(name, shapes, sets, fp32, per_step):
        groups = [[(torch.randn((BATCH, k), device="cuda").half(), torch.randint(-127, 128, (k, n), dtype=torch.int8, device="cuda"),
                    torch.rand(n, device="cuda") * 0.019 + 0.001, torch.zeros(n, device="cuda", dtype=torch.float16),
                    torch.empty((BATCH, n), device="cuda", dtype=torch.float32 if fp32 else torch.float16), k, n) for k, n in shapes]
                  for _ in range(sets)]
        def run():
            for group in groups:
                for a, w, sc, bias, yy, k, n in group:
                    check(lib.ti_v2_gemm_ex_i8(a.data_ptr(), w.data_ptr(), sc.data_ptr(), bias.data_ptr(), yy.data_ptr(), None, BATCH, n, k, int(fp32), 0,
                                               stream(), dev))
        seconds = graph_seconds(run, sets * len(shapes)) * len(shapes)
        nbytes = sum(k * n + 4 * n + 2 * n + 2 * BATCH * k + (4 if fp32 else 2) * BATCH * n for k, n in shapes)
        out[name] = {"seconds": seconds, "bytes": nbytes, "launches_per_step": per_step}

    gemm_family("gemm_int8 lm_head (M=32, 768x50304, fp32 out)", [(768, 50304)], 5, True, 1)
    for label, shape in (("qkv 768x2304", (768, 2304)), ("attn proj 768x768", (768, 768)), ("mlp fc 768x3072", (768, 3072)),
                         ("mlp proj 3072x768", (3072, 768))):
        gemm_family(f"gemm_int8 {label} (M=32)", [shape], max(24, int(260e6 // (shape[0] * shape[1])) + 1), False, 12)
    for v in out.values():
        v["gbs"] = v["bytes"] / v["seconds"] / 1e9
        v["frac"] = v["gbs"] / peak
    return out


def operator_sweep(shapes=((768, 2304), (768, 768), (768, 3072), (3072, 768), (768, 50257)), rows_of=(1, 8, 32, 128, 512), gelu_too=True):
    """Standalone INT8-weight GEMV/GEMM sweep (activations fp16 N(0,1), weights uniform int8, fp16-representable
    scales in [1e-3, 2e-2], seed 1): device time per launch from a CUDA graph, achieved GB/s on the algorithmic
    bytes 2MK + KN + 6N + 2MN (4MN for the fp32 vocabulary projection) and TFLOP/s on 2MNK."""
    import torch
    from tinyinfer_b200.native_ops import NativeOps
    ops = NativeOps()
    lib, dev = ops.lib, torch.cuda.current_device()
    peak, _ = peak_hbm()
    torch.manual_seed(1)
    rows = []
    for k, n in shapes:
        sets = max(2, int(260e6 // (k * n)) + 1)                         # distinct weights > L2 per round
        ws = [torch.randint(-127, 128, (k, n), dtype=torch.int8, device="cuda") for _ in range(sets)]
        sc = (torch.rand(n, device="cuda") * 0.019 + 0.001).half().float()
        bias = (torch.randn(n, device="cuda") * 0.1).half()
        for m in rows_of:
            a = torch.randn((m, k), device="cuda").half()
            fp32 = n == 50257
            y = torch.empty((m, n), device="cuda", dtype=torch.float32 if fp32 else torch.float16)
            for gelu in ((0,) if fp32 or not gelu_too else (0, 1)):
                def run():
                    for w in ws:
                        if gelu:
                            st = lib.ti_b200_gemm_i8_fused(a.data_ptr(), w.data_ptr(), sc.data_ptr(), bias.data_ptr(), None, y.data_ptr(), m, n, k, 0, 1,
                                                           torch.cuda.current_stream().cuda_stream, dev)
                        else:
                            st = lib.ti_v2_gemm_ex_i8(a.data_ptr(), w.data_ptr(), sc.data_ptr(), bias.data_ptr(), y.data_ptr(), None, m, n, k, int(fp32), 0,
                                                      torch.cuda.current_stream().cuda_stream, dev)
                        if st:
                            raise RuntimeError(lib.ti_v2_last_error().decode())
                seconds = graph_seconds(run, sets)
                nbytes = 2 * m * k + k * n + 6 * n + (4 if fp32 else 2) * m * n
                rows.append({"K": k, "N": n, "M": m, "epilogue": "bias+gelu" if gelu else "bias", "us": seconds * 1e6,
                             "GBps": nbytes / seconds / 1e9, "hbm_frac": nbytes / seconds / 1e9 / peak, "TFLOPs": 2.0 * m * n * k / seconds / 1e12})
        del ws
    return rows


# DRAM bytes over algorithmic bytes of one launch of the persistent decode step, from the ncu capture summarised in
# profiles/decode_step_kernel_batch32.md (dram__bytes_read.sum + dram__bytes_write.sum of one launch).
# dram__bytes_read + dram__bytes_write per launch, as captured once with ncu on the same shapes: (bytes, summary file)
KERNEL_TRAFFIC = {
    "attention_decode": (27_125_400, "profiles/attn_decode_staged_kernel_batch32.md"),
    "qkv 768x2304": (1_910_000, "profiles/gemm_tc_kernel_decode_batch32.md"),
    "attn proj 768x768": (740_000, "profiles/gemm_tc_kernel_decode_batch32.md"),
    "mlp fc 768x3072": (2_500_000, "profiles/gemm_tc_kernel_decode_batch32.md"),
    "mlp proj 3072x768": (2_660_000, "profiles/gemm_tc_kernel_decode_batch32.md"),
    "lm_head": (38_931_000, "profiles/gemm_tc_kernel_lm_head_batch32.md"),
}
STEP_TRAFFIC_SOURCE = "profiles/decode_step_kernel_batch32.md"
STEP_TRAFFIC_RATIO = 1.06


def config0_record(model, weights, peak):
    """Batch 1: 32-token prompt (seed 0), 63 decode steps with the cache at 32..94 positions."""
    prompt = np.random.default_rng(0).integers(0, 50257, 32).tolist()
    model.reset_all()
    first = model.forward([0], [prompt], return_logits=False)["next_tokens"]
    model.decode_steps([0], first, 63)                                   # warm: same steps, then again timed
    model.reset_all()
    first = model.forward([0], [prompt], return_logits=False)["next_tokens"]
    out = model.decode_steps([0], first, 63)
    nbytes = sum(step_bytes(weights, [32 + i]) for i in range(63))
    seconds = out["device_ms"] * 1e-3
    model.reset_all()
    return {"workload": "GPT-2 small INT8, batch 1, 32-token prompt, 63 greedy decode steps (cache 32..94 positions), seed 0",
            "us_per_step": seconds / 63 * 1e6, "tokens_per_s": 63 / seconds, "algorithmic_bytes_per_token": nbytes / 63,
            "achieved_GBps": nbytes / seconds / 1e9, "frac": nbytes / seconds / 1e9 / peak, "gpu_launches_per_step": 1 if model.decode_plan() == 1 else 63}


def config3_record(device):
    """GPT-2 medium shape (24 layers, hidden 1024, 16 heads; seed 3), batch 8: prefill of 8 x 768 tokens (so that 256
    generated tokens fit the 1024 learned positions), then 255 decode steps."""
    from tinyinfer_b200 import artifact
    from tinyinfer_b200.runtime import NativeModel
    base = Path(os.environ.get("TINYINFER_B200_CACHE", Path(tempfile.gettempdir()) / "tinyinfer_b200_bench"))
    manifest = artifact.write_synthetic(base / "gpt2_medium_int8_seed3", artifact.GPT2_MEDIUM, seed=3)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, 50257, 768).tolist() for _ in range(8)]
    with NativeModel(None, manifest, device=device, max_batch=8, cache_slots=8, capacity=1024) as m:
        m.forward(list(range(8)), [p[:64] for p in prompts], return_logits=False)      # warm-up pass
        m.reset_all()
        t0 = time.perf_counter()
        first = m.forward(list(range(8)), prompts, return_logits=False)["next_tokens"]
        prefill_s = time.perf_counter() - t0
        m.decode_steps(list(range(8)), first, 8)
        out = m.decode_steps(list(range(8)), first, 247)
        plan = m.decode_plan()
    linear_flops = 2.0 * 8 * 768 * (24 * (1024 * 3072 + 1024 * 1024 + 2 * 1024 * 4096))
    return {"workload": "GPT-2 medium shape INT8, batch 8, prefill 8 x 768 tokens then decode, seed 3", "prefill_ms": prefill_s * 1e3,
            "prefill_tokens_per_s": 8 * 768 / prefill_s, "prefill_linear_TFLOPs": linear_flops / prefill_s / 1e12,
            "decode_us_per_step": out["device_ms"] * 1e3 / 247, "decode_tokens_per_s": 8 * 247 / (out["device_ms"] * 1e-3),
            "decode_plan": "persistent step" if plan == 1 else "launch per operation"}


def server_record(torch, dist, rank, world, manifest_path, model_kind, requests, rate, replicas_per_gpu=2, max_batch=32):
    """The batching-server workload (`requests` requests, Poisson arrivals, prompts log-uniform in [8, 900], outputs uniform in
    [16, 256], seed 4) against ONE tinyinfer_server process that owns all `world` GPUs (`replicas_per_gpu` workers and
    model replicas per GPU with `max_batch` requests each -- by default two of 32, the configuration's 64 requests in
    flight per GPU as two overlapping decode streams -- requests routed to the worker with the fewest outstanding tokens).  Rank 0 starts the server; every rank
    plays an equal share of the request stream through its own asyncio load generator; totals are summed, latency samples
    merged.  `rate` is far above what the GPUs sustain, so the requests queue at the server: a saturating load.
    model_kind "cpu" swaps the GPU model for the protocol stand-in (a token counter) and so measures the ceiling of the
    host side alone: socket front end, router, load generators."""
    import asyncio
    import socket
    from tinyinfer_b200 import replicas
    from tinyinfer_b200.server import binary, loadgen
    box, proc = [None], None
    if rank == 0:
        with socket.socket() as probe:
            probe.bind(("127.0.0.1", 0))
            port = probe.getsockname()[1]
        devices = ",".join(str(d) for d in range(world) for _ in range(replicas_per_gpu))
        cmd = [str(binary()), "--model", model_kind, "--port", str(port), "--devices", devices,
               "--max-batch", str(max_batch), "--max-wait-us", "2000", "--max-new-tokens", "256", "--max-pending", "20000",
               "--max-connections", "19000", "--per-connection", "32"]
        if model_kind == "native":
            cmd += ["--manifest", str(manifest_path)]
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        import select
        waited, _, _ = select.select([proc.stdout], [], [], 180.0)          # model load on every GPU; never block the run on it
        ready = proc.stdout.readline() if waited else ""
        try:
            box[0] = port if ready and json.loads(ready).get("ready") else -1
        except ValueError:
            box[0] = -1
    if dist:
        dist.broadcast_object_list(box, src=0)
    port = box[0]
    result = None
    if port > 0:
        items = loadgen.workload(4, rate, requests)
        mine = replicas.shard(items, rank, world)
        if dist:
            dist.barrier()
        records, start = asyncio.run(loadgen.run_items("127.0.0.1", port, mine, outstanding=4096))
        done = [r for r in records if r.get("status") == 0]
        share = {"tokens": sum(r["tokens"] for r in done), "window": max((r["finished_at"] for r in done), default=start) - start,
                 "completed": len(done), "offered": len(mine), "batch": sum(r["batch_size"] for r in done),
                 "per_token_ms": [r["decode_s"] / (r["tokens"] - 1) * 1e3 for r in done if r["tokens"] > 1],
                 "ttft_ms": [r["ttft_s"] * 1e3 for r in done]}
        shares = [share]
        if dist:
            shares = [None] * world
            dist.all_gather_object(shares, share)
        if rank == 0:
            tokens, window = sum(x["tokens"] for x in shares), max(x["window"] for x in shares)
            completed = sum(x["completed"] for x in shares)
            per_token = [v for x in shares for v in x["per_token_ms"]]
            ttft = [v for x in shares for v in x["ttft_ms"]]
            result = {"model": model_kind, "gpus": world, "requests": requests, "completed": completed, "offered_rate_per_s": rate,
                      "generated_tokens": tokens, "tokens_per_s": tokens / window if window > 0 else 0.0, "drain_window_s": window,
                      "mean_batch_size": sum(x["batch"] for x in shares) / max(1, completed),
                      "per_output_token_ms": loadgen.summarise(per_token), "ttft_ms": loadgen.summarise(ttft),
                      "load_generators": world, "replicas_per_gpu": replicas_per_gpu, "max_batch_per_replica": max_batch,
                      "in_flight_per_gpu": replicas_per_gpu * max_batch}
    if dist:
        dist.barrier()
    if proc is not None:
        proc.terminate()
        try:
            proc.communicate(timeout=20)
        except subprocess.TimeoutExpired:
            proc.kill()
    return result


def prefill_main(args):
    """Only the prefill of the 32 prompts of the workload (8,248 rows in one pass), `--steps` times: the command the
    prefill profiles under profiles/ were captured with.  Prints the host-timed milliseconds per pass."""
    import torch
    from tinyinfer_b200.runtime import NativeModel
    torch.cuda.set_device(0)
    prompts, slots = workload_prompts(), list(range(BATCH))
    with NativeModel(None, artifact_path(), device=0, max_batch=BATCH, cache_slots=BATCH, capacity=1024) as model:
        times = []
        for _ in range(max(1, args.steps)):
            model.reset_all()
            t0 = time.perf_counter()
            model.forward(slots, prompts, return_logits=False)
            times.append((time.perf_counter() - t0) * 1e3)
    print(json.dumps({"prefill_ms": times, "rows": sum(len(p) for p in prompts)}))


def gpu_main(args, rank, world):
    torch, dist, local = setup_ranks()

    def barrier():
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(value):
        if not dist:
            return value
        t = torch.tensor([value], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    from tinyinfer_b200 import artifact, replicas
    from tinyinfer_b200.runtime import NativeModel
    if rank == 0:
        manifest_path = artifact_path()
    barrier()
    manifest_path = artifact_path()
    manifest = json.loads(Path(manifest_path).read_text())
    weights = artifact.weight_bytes(manifest)
    prompts = workload_prompts()
    slots = list(range(BATCH))
    K, W = max(1, args.steps), max(0, args.warmup)
    peak, peak_source = peak_hbm()

    with NativeModel(None, manifest_path, device=local, max_batch=BATCH, cache_slots=BATCH, capacity=1024) as model:
        if args.plan is not None:
            model.decode_plan(args.plan)
        persistent = model.decode_plan() == 1

        def prefill():
            model.reset_all()
            t0 = time.perf_counter()
            first = model.forward(slots, prompts, return_logits=False)["next_tokens"]
            return first, (time.perf_counter() - t0) * 1e3

        def timed_steps(count, warm):
            """`count` device-resident steps after `warm` untimed ones: (device ms, algorithmic bytes)."""
            ids, _ = prefill()
            if warm:
                ids = model.decode_steps(slots, ids, warm)["tokens"][-1]
            barrier()
            ms, done, nbytes = 0.0, 0, 0
            while done < count:
                lengths_now = model.lengths()[:BATCH]
                n = min(count - done, 1024 - max(lengths_now))
                if n <= 0:                                  # generation exhausted the context: start over (untimed prefill)
                    ids, _ = prefill()
                    continue
                out = model.decode_steps(slots, ids, n)
                ms += out["device_ms"]
                ids = out["tokens"][-1]
                nbytes += sum(step_bytes(weights, [t + i for t in lengths_now]) for i in range(n))
                done += n
            barrier()
            return ms, nbytes

        # ---- value: device-resident decode steps ------------------------------------------------
        _, ttft_ms = prefill()
        with ClockSampler(local) as clocks:
            device_ms, total_bytes = timed_steps(K, W)
        _, slowest_s, value = replicas.job_throughput(BATCH * K, device_ms * 1e-3, dist, "cuda")    # sum of tokens / slowest rank
        device_ms = slowest_s * 1e3
        # kernels of one decode step.  Persistent plan: one.  Launch-per-operation plan: embed, 12 x (QKV GEMM with LayerNorm
        # prologue and K/V placement, attention, projection GEMM, FC GEMM with LayerNorm prologue, projection GEMM), final
        # LayerNorm, vocabulary GEMM, argmax, advance.
        launches_per_step = 1 if persistent else 1 + 12 * 5 + (0 if BATCH <= 8 else 1) + 2   # embed, 5 per layer, final LayerNorm, lm_head with argmax, publish
        step_gbs = total_bytes / (device_ms * 1e-3) / 1e9

        if args.quick:
            if rank == 0:
                print(json.dumps({"metric": "int8_gpt2_decode_tokens_per_s", "value": value, "unit": "tokens/s", "steps": K, "warmup": W,
                                  "ms_per_step": device_ms / K, "gpu_launches": launches_per_step * K, "quick": True}))
            return
        # ---- e2e: per-step reference-facing call, host ids in, host ids out ----------------------
        first, _ = prefill()
        ids = first
        for _ in range(max(W, 3)):
            ids = model.forward(slots, [[t] for t in ids], return_logits=False)["next_tokens"]
        e2e_steps = min(K, 1024 - max(model.lengths()[:BATCH]) - 1)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            ids = model.forward(slots, [[t] for t in ids], return_logits=False)["next_tokens"]
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        barrier()
        e2e = {"value": world * BATCH * e2e_steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 5 * BATCH * 4,
               "d2h_bytes_per_step": BATCH * 4 + 4, "steps": e2e_steps, "api": "ti_llm_forward_batch per step",
               "note": "includes the ctypes marshalling of llm/runtime.py-style Python lists"}
        # the generation call a user makes (prompts in, all tokens out), reference's decode-rate definition
        model.reset_all()
        gen = model.greedy(prompts, NEW_TOKENS)
        decode_s = (max(gen["total_ms"]) - gen["ttft_ms"][0]) * 1e-3
        e2e["greedy_batch_tokens_per_s"] = world * BATCH * (NEW_TOKENS - 1) / decode_s
        e2e["greedy_batch_ttft_ms"] = gen["ttft_ms"][0]

        extras = {}
        if rank == 0 and world == 1 and not args.no_extras:
            extras["config0"] = config0_record(model, weights, peak)
            # the other decode plan on the same workloads, for the record (both produce the same bits)
            other = 0 if persistent else 1
            try:
                model.decode_plan(other)
                ms_other, _ = timed_steps(min(K, 40), 3)
                extras["other_decode_plan"] = {"plan": "persistent step kernel (1 launch per step)" if other == 1 else "launch per operation (64 launches per step)",
                                               "ms_per_step": ms_other / min(K, 40), "config0": config0_record(model, weights, peak)}
            except RuntimeError as error:                     # plan 1 is not available for every shape / device
                extras["other_decode_plan"] = {"unavailable": str(error)}
            model.decode_plan(1 if persistent else 0)

    # ---- the batching server on all N GPUs (after this process's own replica is gone), then its host side alone
    server = {}
    if not args.no_server:
        # 4096 requests per GPU keep every replica busy for several seconds; the total stays under the server's descriptor
        # limit (every request holds its own connection while it waits in the queue)
        offered = min(4096 * world, 16384)
        server["native"] = server_record(torch, dist, rank, world, manifest_path, "native", offered, 4000.0 * world)
        server["host_side_ceiling"] = server_record(torch, dist, rank, world, manifest_path, "cpu", offered, 4000.0 * world)
        if world == 1:
            # outside the configuration (more than 64 requests in flight per GPU): what one B200 sustains when four
            # replicas of 64 overlap their decode steps
            server["beyond"] = server_record(torch, dist, rank, world, manifest_path, "native", offered, 4000.0, replicas_per_gpu=4, max_batch=64)

    line = {"metric": "int8_gpt2_decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": device_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 activations x int8 weights, f32 accumulate",
            "data": "synthetic", "config": config_block(world), "prefill_ttft_ms": ttft_ms,
            "e2e": e2e, "gpu_launches": launches_per_step * K, "clocks": clocks.summary()}
    if rank == 0:
        per_gpu_gbs = step_gbs / world if world > 1 else step_gbs
        if persistent:
            traffic = None if STEP_TRAFFIC_RATIO is None else int(total_bytes / K * STEP_TRAFFIC_RATIO)
            line["roofline"] = {"kernel": "decode_step_kernel: one persistent launch per decode step (embedding .. argmax), grid = SM count",
                                "bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
                                "traffic": traffic, "traffic_source": STEP_TRAFFIC_SOURCE if traffic is not None else None,
                                "algorithmic_bytes": total_bytes / K, "launch_us": device_ms / K * 1e3, "peak_source": peak_source,
                                "share_of_step": 1.0,
                                "note": "algorithmic weight + KV bytes of a step / mean launch duration, CUDA events on the model's stream"}
        line["step_roofline"] = {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
                                 "bytes_per_step": total_bytes / K, "note": "algorithmic weight+KV bytes per step / step time, per GPU"}
        line.update(extras)
        if server:
            line["server"] = server["native"]
            line["server_host_side_ceiling"] = server["host_side_ceiling"]
            if "beyond" in server:
                line["server_256_in_flight"] = server["beyond"]
        if world == 1 and not args.no_extras:
            cached_at_start = [len(p) + W for p in prompts]
            kernels = kernel_rooflines(cached_at_start, peak)
            line["kernels"] = {k: {"us": v["seconds"] * 1e6, "GBps": v["gbs"], "frac": v["frac"], "launches_per_step": v["launches_per_step"]}
                               for k, v in kernels.items()}
            line["kernels_note"] = "operator kernels of the launch-per-operation plan, each timed alone (CUDA graph over > L2 buffers)"
            if not persistent:
                # The dominant kernel = the kernel instantiation with the largest share of the step: the two projections
                # are launches of one instantiation, as are the two GEMMs with the LayerNorm prologue.
                groups = {"gemm_tc_kernel<32,0>: attention projection 768x768 and mlp projection 3072x768 (+ residual), 24 launches per step": ("attn proj 768x768", "mlp proj 3072x768"),
                          "gemm_tc_kernel<32,2>: LayerNorm + qkv 768x2304 (K/V placement) and LayerNorm + mlp fc 768x3072 (GELU), 24 launches per step": ("qkv 768x2304", "mlp fc 768x3072"),
                          "attn_decode_staged_kernel: 32 ragged requests x 12 heads, 12 launches per step": ("attention_decode",),
                          "gemm_tc_kernel<32,0,lean>: vocabulary projection 768x50304, 1 launch per step": ("lm_head",)}
                totals = {}
                for name, parts in groups.items():
                    members = [v for k, v in kernels.items() if any(part in k for part in parts)]
                    traffic = [next((t for key, (t, _) in KERNEL_TRAFFIC.items() if key in k), None) for k in kernels if any(part in k for part in parts)]
                    source = next((src for key, (_, src) in KERNEL_TRAFFIC.items() if any(key in k for k in kernels if any(part in k for part in parts))), None)
                    launches = sum(v["launches_per_step"] for v in members)
                    totals[name] = {"seconds": sum(v["seconds"] * v["launches_per_step"] for v in members), "launches": launches,
                                    "bytes": sum(v["bytes"] * v["launches_per_step"] for v in members),
                                    "traffic": None if any(t is None for t in traffic) else sum(t * v["launches_per_step"] for t, v in zip(traffic, members)),
                                    "source": source}
                name, top = max(totals.items(), key=lambda kv: kv[1]["seconds"])
                achieved = top["bytes"] / top["seconds"] / 1e9
                line["roofline"] = {"kernel": name, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                                    "traffic": None if top["traffic"] is None else int(top["traffic"] / top["launches"]),
                                    "traffic_source": top["source"] if top["traffic"] is not None else None,
                                    "algorithmic_bytes": int(top["bytes"] / top["launches"]), "us_per_launch": top["seconds"] / top["launches"] * 1e6,
                                    "note": "bytes, traffic and time are averages per launch of this instantiation; every kernel of the step is in `kernels`",
                                    "peak_source": peak_source, "share_of_step": top["seconds"] / (device_ms * 1e-3 / K)}
            line["operator_sweep_768x3072"] = [{k: (round(v, 3) if isinstance(v, float) else v) for k, v in row.items()}
                                               for row in operator_sweep(((768, 3072),), (1, 32, 128, 512), gelu_too=False)]
            line["config3"] = config3_record(local)
        if world == 1 and not args.no_cpu:
            result, sample = cpu_arm(steps=int(os.environ.get("TINYINFER_B200_CPU_STEPS", 6)), warmup=1, threads=physical_cores())
            line["cpu_baseline"] = {"value": result["tokens_per_s"], "unit": "tokens/s", "cores": result["cores"], "kind": result["kind"], "sample": sample}
        print(json.dumps(line))
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=120)
    parser.add_argument("--warmup", type=int, default=7)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    parser.add_argument("--no-server", action="store_true", help="skip the batching-server workload")
    parser.add_argument("--no-extras", action="store_true", help="skip config 0, config 3, the operator kernels and the sweep excerpt")
    parser.add_argument("--plan", type=int, choices=[0, 1], default=None, help="decode plan: 0 launch per operation replayed as a CUDA graph (default), 1 one persistent kernel per step")
    parser.add_argument("--quick", action="store_true", help="only the device-resident timed steps (for profilers)")
    parser.add_argument("--prefill", action="store_true", help="only the prefill pass of the workload's 32 prompts, --steps times (for profilers)")
    parser.add_argument("--sweep", action="store_true", help="operator sweep of the INT8-weight GEMV/GEMM instead of the decode benchmark")
    args = parser.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.sweep:
        if rank == 0:
            import torch
            torch.cuda.set_device(0)
            for row in operator_sweep():
                print(json.dumps(row))
    elif args.prefill:
        if rank == 0:
            prefill_main(args)
    elif args.impl == "reference":
        reference_main(args, rank, world)
    else:
        gpu_main(args, rank, world)


if __name__ == "__main__":
    main()
