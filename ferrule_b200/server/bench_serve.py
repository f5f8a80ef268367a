"""Synthetic serving sweep against a running OpenAI-compatible server.

Workload: input lengths log-uniform over [min_in, max_in], output lengths uniform over
[min_out, max_out], token ids uniform over the vocabulary, `shared_fraction` of the requests start
with one common `shared_prefix`-token prefix (exercises prefix sharing / copy-on-write), Poisson
arrivals whose rate tracks the target concurrency.  Per concurrency level the report has p50/p99
TTFT and TPOT, committed tokens/s and failure counts.  Counterpart of
scripts/bench_vllm_serve.sh (TTFT / TPOT / ITL / E2EL percentiles with a random dataset).
"""
from __future__ import annotations

import asyncio
import json
import math
import random
import time
from typing import Dict, List


def _pct(v: List[float], p: float) -> float:
    if not v:
        return 0.0
    s = sorted(v)
    return s[min(int(p * len(s)), len(s) - 1)]


async def _one(client, url: str, model: str, prompt: List[int], max_tokens: int, out: Dict) -> None:
    body = {"prompt": prompt, "max_tokens": max_tokens, "stream": True, "ignore_eos": True, "return_token_ids": True}
    if model:
        body["model"] = model
    t0 = time.perf_counter()
    stamps = []
    try:
        async with client.stream("POST", url + "/v1/completions", json=body, timeout=None) as r:
            if r.status_code != 200:
                out["failed"] += 1
                out.setdefault("errors", []).append(f"http {r.status_code}: {(await r.aread())[:200]!r}")
                return
            async for line in r.aiter_lines():
                if line.startswith("data: ") and line != "data: [DONE]":
                    obj = json.loads(line[6:])
                    if "error" in obj:                       # engine failure reported inside a 200 stream
                        out["failed"] += 1
                        out.setdefault("errors", []).append(str(obj["error"].get("message"))[:200])
                        return
                    if obj.get("token_ids") or (obj.get("choices") and obj["choices"][0].get("text")):
                        stamps.append(time.perf_counter())
    except Exception:  # noqa: BLE001
        out["failed"] += 1
        return
    if stamps:
        out["ttft"].append(stamps[0] - t0)
        if len(stamps) > 1:
            out["tpot"].append((stamps[-1] - stamps[0]) / (len(stamps) - 1))
        out["tokens"] += len(stamps)
    out["e2e"].append(time.perf_counter() - t0)


async def _level(url, model, conc, n_req, rng, vocab, min_in, max_in, min_out, max_out, prefix, frac) -> Dict:
    import httpx
    out = {"ttft": [], "tpot": [], "e2e": [], "tokens": 0, "failed": 0}
    shared = [rng.randrange(vocab) for _ in range(prefix)]
    sem = asyncio.Semaphore(conc)
    t0 = time.perf_counter()
    async with httpx.AsyncClient() as client:
        async def guarded(p, m):
            async with sem:
                await _one(client, url, model, p, m, out)
        tasks = []
        for _ in range(n_req):
            n_in = int(math.exp(rng.uniform(math.log(min_in), math.log(max_in))))
            p = [rng.randrange(vocab) for _ in range(n_in)]
            if rng.random() < frac and n_in > len(shared):
                p[:len(shared)] = shared
            tasks.append(asyncio.create_task(guarded(p, rng.randint(min_out, max_out))))
            await asyncio.sleep(rng.expovariate(max(conc, 1) * 4.0))       # Poisson arrivals
        await asyncio.gather(*tasks)
    dt = time.perf_counter() - t0
    return {"concurrency": conc, "requests": n_req, "failed": out["failed"], "seconds": round(dt, 3),
            "committed_tokens_per_s": round(out["tokens"] / dt, 2),
            "ttft_p50_s": round(_pct(out["ttft"], 0.5), 4), "ttft_p99_s": round(_pct(out["ttft"], 0.99), 4),
            "tpot_p50_s": round(_pct(out["tpot"], 0.5), 5), "tpot_p99_s": round(_pct(out["tpot"], 0.99), 5),
            "e2e_p50_s": round(_pct(out["e2e"], 0.5), 4), "tokens": out["tokens"],
            "errors": sorted(set(out.get("errors", [])))[:3]}


def run_sweep(url, model, concurrency, n_req, seed, vocab, min_in, max_in, min_out, max_out, prefix, frac) -> Dict:
    rng = random.Random(seed)
    # a level needs at least as many requests as its concurrency to ever reach it
    levels = [asyncio.run(_level(url, model, c, max(n_req, c), rng, vocab, min_in, max_in, min_out, max_out, prefix,
                                 frac)) for c in concurrency]
    out = {"url": url, "levels": levels}
    try:        # the server's own counters: KV high-water mark, copy-on-write copies, prefix reuse, preemptions
        import httpx
        m = httpx.get(url + "/metrics", timeout=10).json()
        eng = (m.get("worker") or {}).get("engine") or {}
        out["server"] = {"kv": eng.get("kv"), "scheduler": eng.get("scheduler"),
                         "speculative": eng.get("speculative"),
                         "prefix_cache": {k: eng.get(k) for k in ("prefix_hits", "prefix_tokens_reused",
                                                                  "prefix_entries", "prefix_evictions")},
                         "decode_steps": eng.get("decode_steps"), "prefill_chunks": eng.get("prefill_chunks")}
    except Exception as exc:  # noqa: BLE001 - the sweep's own numbers stand without it
        out["server"] = {"unavailable": str(exc)[:200]}
    return out
