"""Load generator for the chat-completions server: the reference's ``client_benchmark.py`` without the
OpenAI SDK and without its prompt list.

Sends ``NUM_REQUESTS`` chat requests (sequentially or from ``CONCURRENCY`` threads), records latency
and token counts per request and writes the same JSON summary fields as the reference
(``client_benchmark.py:172-218``): avg / median / std / min / max latency and requests per second,
plus tokens per second.  Prompts are synthetic: space-separated decimal token IDs from a seeded
generator (the server's stub tokenizer reads them; a real tokenizer treats them as text).
Environment keys as in the reference: HOST, PORT, MODEL, NUM_REQUESTS, MAX_TOKENS, TEMPERATURE,
LOG_FILE, CONCURRENCY; extra: PROMPT_TOKENS (default 16), SEED.
"""

from __future__ import annotations

import json
import os
import random
import statistics
import time
import urllib.request
from concurrent.futures import ThreadPoolExecutor
from typing import Callable, Dict, List, Optional


def synthetic_prompts(n: int, tokens: int, seed: int = 0, vocab: int = 151936) -> List[str]:
    rng = random.Random(seed)
    return [" ".join(str(rng.randrange(vocab)) for _ in range(tokens)) for _ in range(n)]


def http_post(url: str, body: dict, timeout: float = 300.0) -> dict:
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def wait_for_server(base: str, timeout: float = 180.0) -> None:
    deadline = time.time() + timeout
    while time.time() < deadline:
        try:
            with urllib.request.urlopen(f"{base}/health", timeout=3):
                return
        except Exception:
            time.sleep(1.0)
    raise RuntimeError(f"server at {base} not ready after {timeout:.0f}s")


def summarise(records: List[dict], wall_s: float) -> Dict[str, float]:
    lat = [r["latency_s"] for r in records if r.get("latency_s") is not None]
    out_tok = sum(r.get("output_tokens", 0) for r in records)
    return {
        "num_requests": len(records),
        "num_failed": len(records) - len(lat),
        "avg_latency_s": round(statistics.mean(lat), 4) if lat else 0.0,
        "median_latency_s": round(statistics.median(lat), 4) if lat else 0.0,
        "std_latency_s": round(statistics.stdev(lat), 4) if len(lat) > 1 else 0.0,
        "min_latency_s": round(min(lat), 4) if lat else 0.0,
        "max_latency_s": round(max(lat), 4) if lat else 0.0,
        "throughput_req_s": round(len(lat) / wall_s, 4) if wall_s > 0 else 0.0,
        "tokens_per_s": round(out_tok / wall_s, 2) if wall_s > 0 else 0.0,
        "tokens_per_s_per_request": round(out_tok / sum(lat), 2) if lat and sum(lat) > 0 else 0.0,
    }


def run(post: Callable[[dict], dict], prompts: List[str], model: str, max_tokens: int, temperature: float = 0.0,
        concurrency: int = 1) -> dict:
    """``post(body) -> response dict``; returns {"config", "results", "summary"}."""
    def one(i_prompt):
        i, prompt = i_prompt
        body = {"model": model, "messages": [{"role": "user", "content": prompt}], "max_tokens": max_tokens,
                "temperature": temperature}
        t0 = time.perf_counter()
        try:
            resp = post(body)
            dt = time.perf_counter() - t0
            usage = resp.get("usage", {})
            return {"index": i, "latency_s": round(dt, 4), "prompt_tokens": usage.get("prompt_tokens", 0),
                    "output_tokens": usage.get("completion_tokens", 0),
                    "finish_reason": resp["choices"][0].get("finish_reason"),
                    "answer": resp["choices"][0]["message"]["content"]}
        except Exception as exc:
            return {"index": i, "latency_s": None, "prompt_tokens": 0, "output_tokens": 0, "error": str(exc)}

    t0 = time.perf_counter()
    if concurrency <= 1:
        records = [one(x) for x in enumerate(prompts)]
    else:
        with ThreadPoolExecutor(max_workers=concurrency) as pool:
            records = list(pool.map(one, enumerate(prompts)))
    wall = time.perf_counter() - t0
    return {"config": {"model": model, "max_tokens": max_tokens, "temperature": temperature,
                       "concurrency": concurrency, "num_requests": len(prompts)},
            "results": records, "summary": summarise(records, wall)}


def main(argv: Optional[List[str]] = None) -> None:
    base = os.getenv("HOST", "http://localhost") + ":" + os.getenv("PORT", "8000")
    model = os.getenv("MODEL", "Qwen/Qwen3-0.6B")
    n = int(os.getenv("NUM_REQUESTS", "100"))
    prompts = synthetic_prompts(n, int(os.getenv("PROMPT_TOKENS", "16")), seed=int(os.getenv("SEED", "0")))
    wait_for_server(base)
    report = run(lambda body: http_post(f"{base}/v1/chat/completions", body), prompts, model,
                 int(os.getenv("MAX_TOKENS", "128")), float(os.getenv("TEMPERATURE", "0.0")),
                 int(os.getenv("CONCURRENCY", "1")))
    with open(os.getenv("LOG_FILE", "latency_log_megakernel.json"), "w") as f:
        json.dump(report, f, indent=2)
    print(json.dumps(report["summary"], indent=2))


if __name__ == "__main__":
    main()
