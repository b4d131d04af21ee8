"""Open-loop load generator for the batching server.

    python -m tinyinfer_b200.server.loadgen --port 8091 --rate 200 --requests 4096 [--seed 4]

Workload of the serving configuration: `requests` generate-requests arrive as a Poisson process of
`rate` requests/s (exponential gaps drawn up front, so slow responses never delay later arrivals);
prompt lengths are log-uniform in [8, 900], output lengths uniform in [16, 256] and clamped so that
prompt + output <= 1024; token ids uniform.  Everything derives from random.Random(f"{seed}:{rate}")
as in the reference's generator (server/loadgen.py:36-43), so a (seed, rate) pair always names the
same byte-identical request stream.  Each request uses its own TCP connection (connect time is
part of its latency), as the reference's load test does (server/README.md "Offered-load experiment").

Reported (JSON on stdout): completed / failed counts, aggregate generated tokens per second over the
whole run (first send to last final), and p50 / p99 / p99.9 of time-to-first-token, time per output
token ((final - first) / (tokens - 1)) and request latency, percentiles interpolated at
(n-1)*p/100 (server/loadgen.py:46-49).
"""
from __future__ import annotations

import argparse
import asyncio
import json
import math
import random
import time

from . import protocol

CONTEXT = 1024


def workload(seed, rate, count, prompt_range=(8, 900), output_range=(16, 256)):
    """[(due_seconds, request_id, prompt_tokens, max_new_tokens)] -- deterministic in (seed, rate)."""
    if type(seed) is not int or count < 1 or not rate > 0:
        raise ValueError("seed/rate/count")
    rng = random.Random(f"{seed}:{rate}")
    lo, hi = prompt_range
    due, items = 0.0, []
    for index in range(count):
        due += rng.expovariate(rate)
        prompt_len = min(hi, max(lo, int(round(math.exp(rng.uniform(math.log(lo), math.log(hi)))))))
        new_tokens = min(rng.randint(*output_range), CONTEXT - prompt_len)
        prompt = [rng.randrange(protocol.VOCAB) for _ in range(prompt_len)]
        items.append((due, index + 1, prompt, new_tokens))
    return items


def percentile(values, p):
    if not values or any(not math.isfinite(v) or v < 0 for v in values):
        raise ValueError("percentile needs finite nonnegative samples")
    ordered = sorted(values)
    position = (len(ordered) - 1) * p / 100.0
    low = int(math.floor(position))
    high = min(low + 1, len(ordered) - 1)
    return ordered[low] + (ordered[high] - ordered[low]) * (position - low)


def summarise(samples):
    return {f"p{str(p).replace('.', '_')}": percentile(samples, p) for p in (50, 99, 99.9)} if samples else None


async def _one(host, port, item, start, gate, records, timeout):
    due, identifier, prompt, new_tokens = item
    await asyncio.sleep(max(0.0, start + due - time.perf_counter()))
    record = {"id": identifier, "prompt": len(prompt), "requested": new_tokens, "status": "error"}
    async with gate:
        writer = None
        try:
            sent = time.perf_counter()
            reader, writer = await asyncio.wait_for(asyncio.open_connection(host, port), timeout)
            writer.write(protocol.request(identifier, prompt, new_tokens))
            await writer.drain()
            first_at = None
            while True:
                reply = await asyncio.wait_for(protocol.read_response(reader), timeout)
                now = time.perf_counter()
                if reply["kind"] == protocol.FIRST:
                    first_at = now
                    continue
                record.update(status=reply["status"], tokens=len(reply["tokens"]), batch_size=reply["batch_size"],
                              latency_s=now - (start + due), ttft_s=(first_at or now) - sent, finished_at=now,
                              decode_s=now - (first_at or now), queue_ns=reply["queue_ns"], server_ns=reply["server_ns"])
                break
        except (OSError, asyncio.TimeoutError, ValueError, asyncio.IncompleteReadError) as error:
            record["error"] = type(error).__name__
        finally:
            if writer is not None:
                writer.close()
    records.append(record)


async def run_items(host, port, items, outstanding=2048, timeout=300.0):
    """Sends `items` (a list from workload(), or a share of one) at their due times; returns the raw per-request records
    and the clock value the due times are relative to."""
    gate = asyncio.Semaphore(outstanding)
    records = []
    start = time.perf_counter() + 0.05
    await asyncio.gather(*(_one(host, port, item, start, gate, records, timeout) for item in items))
    return records, start


def report(records, start, offered, offered_window_s, rate=None, seed=None):
    done = [r for r in records if r.get("status") == 0]
    last = max((r["finished_at"] for r in done), default=start)
    tokens = sum(r["tokens"] for r in done)
    per_token = [r["decode_s"] / (r["tokens"] - 1) for r in done if r["tokens"] > 1]
    return {"rate": rate, "seed": seed, "offered": offered, "completed": len(done), "failed": offered - len(done),
            "offered_window_s": offered_window_s, "drain_window_s": last - start, "generated_tokens": tokens,
            "tokens_per_s": tokens / (last - start) if last > start else 0.0,
            "prompt_tokens": sum(r["prompt"] for r in done),
            "mean_batch_size": sum(r["batch_size"] for r in done) / len(done) if done else 0.0,
            "ttft_ms": summarise([r["ttft_s"] * 1e3 for r in done]),
            "per_output_token_ms": summarise([v * 1e3 for v in per_token]),
            "request_latency_ms": summarise([r["latency_s"] * 1e3 for r in done]),
            "statuses": {str(k): sum(1 for r in records if r.get("status") == k) for k in {r.get("status") for r in records}}}


async def run(host, port, rate, count, seed, outstanding=2048, timeout=300.0):
    items = workload(seed, rate, count)
    records, start = await run_items(host, port, items, outstanding, timeout)
    return report(records, start, count, items[-1][0], rate, seed)


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--host", default="127.0.0.1")
    parser.add_argument("--port", type=int, default=8091)
    parser.add_argument("--rate", type=float, required=True, help="Poisson arrival rate, requests per second")
    parser.add_argument("--requests", type=int, default=4096)
    parser.add_argument("--seed", type=int, default=4)
    parser.add_argument("--outstanding", type=int, default=2048)
    args = parser.parse_args()
    print(json.dumps(asyncio.run(run(args.host, args.port, args.rate, args.requests, args.seed, args.outstanding))))


if __name__ == "__main__":
    main()
