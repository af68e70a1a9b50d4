"""Serving benchmark client: sends synthetic requests to an OpenAI-compatible endpoint and
reports throughput and latency percentiles.

    python -m omni_npu_b200.serving.bench_client --base-url http://127.0.0.1:8000 \
        --num-prompts 256 --input-len 1024 --output-len 256 --max-concurrency 128 \
        --num-processes 4 --num-warmups 8 [--request-rate 32] [--profile]

Metrics: request / input-token / output-token throughput, TTFT, TPOT, ITL and end-to-end
latency (mean, median, p99).  ``--num-processes`` forks client processes (one asyncio loop
each) so that the client does not become the bottleneck at high request rates;
``--num-warmups`` sends that many untimed requests first; ``--profile`` brackets the timed
part with the server's ``/start_profile`` / ``/stop_profile`` when it has them.  Same flags
as the ones the reference adds to ``vllm bench serve``
(omni_npu/vllm_patches/patches/common/patch_bench.py:905-1139).
"""
from __future__ import annotations

import argparse
import asyncio
import json
import multiprocessing as mp
import random
import statistics
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class RequestResult:
    ok: bool = False
    prompt_len: int = 0
    output_len: int = 0
    ttft: float = 0.0
    latency: float = 0.0
    itl: List[float] = field(default_factory=list)
    error: str = ""


def synth_prompt(rng: random.Random, n: int, vocab: int) -> List[int]:
    return [rng.randrange(10, vocab) for _ in range(n)]


async def send_one(session, url: str, model: str, prompt: List[int], output_len: int) -> RequestResult:
    res = RequestResult(prompt_len=len(prompt))
    body = {"model": model, "prompt": prompt, "max_tokens": output_len, "temperature": 0.0, "ignore_eos": True,
            "stream": True}
    t0 = time.perf_counter()
    last = t0
    try:
        async with session.post(url, json=body) as resp:
            if resp.status != 200:
                res.error = f"HTTP {resp.status}"
                return res
            async for raw in resp.content:
                line = raw.decode().strip()
                if not line.startswith("data:"):
                    continue
                data = line[5:].strip()
                if data == "[DONE]":
                    break
                toks = json.loads(data)["choices"][0].get("token_ids") or []
                if not toks:
                    continue
                now = time.perf_counter()
                if res.output_len == 0:
                    res.ttft = now - t0
                else:
                    res.itl.append((now - last) / len(toks))
                last = now
                res.output_len += len(toks)
        res.latency = time.perf_counter() - t0
        res.ok = res.output_len > 0
    except Exception as e:      # connection errors count as failed requests
        res.error = str(e)
    return res


async def run_client(args, prompts: List[List[int]], rate: float) -> List[RequestResult]:
    import aiohttp
    url = args.base_url.rstrip("/") + "/v1/completions"
    sem = asyncio.Semaphore(max(1, args.max_concurrency))
    timeout = aiohttp.ClientTimeout(total=args.request_timeout)
    async with aiohttp.ClientSession(timeout=timeout) as session:
        async def guarded(p):
            async with sem:
                return await send_one(session, url, args.model, p, args.output_len)

        tasks = []
        rng = random.Random(args.seed + 17)
        for p in prompts:
            tasks.append(asyncio.create_task(guarded(p)))
            if rate > 0:
                await asyncio.sleep(rng.expovariate(rate))
        return list(await asyncio.gather(*tasks))


def _worker(args, prompts, rate, q) -> None:
    q.put(asyncio.run(run_client(args, prompts, rate)))


def percentile(xs: List[float], p: float) -> float:
    if not xs:
        return 0.0
    xs = sorted(xs)
    k = min(len(xs) - 1, max(0, int(round(p / 100.0 * (len(xs) - 1)))))
    return xs[k]


def summarise(results: List[RequestResult], wall: float) -> Dict[str, float]:
    ok = [r for r in results if r.ok]
    out_tok = sum(r.output_len for r in ok)
    in_tok = sum(r.prompt_len for r in ok)
    tpot = [(r.latency - r.ttft) / (r.output_len - 1) for r in ok if r.output_len > 1]
    itl = [x for r in ok for x in r.itl]

    def stats(name, xs, scale=1e3):
        return {f"mean_{name}_ms": scale * statistics.fmean(xs) if xs else 0.0,
                f"median_{name}_ms": scale * percentile(xs, 50), f"p99_{name}_ms": scale * percentile(xs, 99)}

    summary = {"completed": len(ok), "failed": len(results) - len(ok), "duration_s": wall,
               "request_throughput": len(ok) / wall if wall > 0 else 0.0,
               "input_token_throughput": in_tok / wall if wall > 0 else 0.0,
               "output_token_throughput": out_tok / wall if wall > 0 else 0.0,
               "total_token_throughput": (in_tok + out_tok) / wall if wall > 0 else 0.0}
    summary.update(stats("ttft", [r.ttft for r in ok]))
    summary.update(stats("tpot", tpot))
    summary.update(stats("itl", itl))
    summary.update(stats("e2el", [r.latency for r in ok]))
    return summary


def run(args) -> Dict[str, float]:
    rng = random.Random(args.seed)
    if args.num_warmups > 0:
        warm = [synth_prompt(rng, args.input_len, args.vocab_size) for _ in range(args.num_warmups)]
        asyncio.run(run_client(args, warm, 0.0))
    prompts = [synth_prompt(rng, args.input_len, args.vocab_size) for _ in range(args.num_prompts)]
    nproc = max(1, args.num_processes)
    if args.profile:
        _post(args.base_url, "/start_profile")
    t0 = time.perf_counter()
    if nproc == 1:
        results = asyncio.run(run_client(args, prompts, args.request_rate))
    else:
        q: mp.Queue = mp.Queue()
        shards = [prompts[i::nproc] for i in range(nproc)]
        procs = [mp.Process(target=_worker, args=(args, s, args.request_rate / nproc, q)) for s in shards if s]
        for p in procs:
            p.start()
        results = [r for _ in procs for r in q.get()]
        for p in procs:
            p.join()
    wall = time.perf_counter() - t0
    if args.profile:
        _post(args.base_url, "/stop_profile")
    return summarise(results, wall)


def _post(base: str, path: str) -> None:
    import urllib.request
    try:
        urllib.request.urlopen(urllib.request.Request(base.rstrip("/") + path, data=b"{}", method="POST"), timeout=5)
    except Exception:
        pass


def make_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser("omni_npu_b200.serving.bench_client")
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="model")
    ap.add_argument("--num-prompts", type=int, default=256)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--vocab-size", type=int, default=32000)
    ap.add_argument("--request-rate", type=float, default=0.0, help="requests/s (Poisson); 0 = all at once")
    ap.add_argument("--max-concurrency", type=int, default=128)
    ap.add_argument("--num-processes", type=int, default=1)
    ap.add_argument("--num-warmups", type=int, default=0)
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--request-timeout", type=float, default=3600.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--save-result", default=None)
    return ap


def main(argv=None) -> None:
    args = make_parser().parse_args(argv)
    summary = run(args)
    print(json.dumps(summary, indent=2))
    if args.save_result:
        with open(args.save_result, "w") as f:
            json.dump(summary, f, indent=2)


if __name__ == "__main__":
    main()
