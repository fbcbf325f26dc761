#!/usr/bin/env python
"""Constant-rate load test against a running router, reading the timing response headers.

Counterpart of the reference's k6 script (`load_tests/starcoder_load.js`): N requests per second for a duration,
thresholds on p95 time-per-token and p95 queue time, zero failures.

    python deploy/load_test.py --url http://127.0.0.1:3000 --rps 10 --seconds 60 --max-new-tokens 60
"""
import argparse
import asyncio
import json
import statistics
import sys
import time

import aiohttp


async def one(session, url, body, out):
    t0 = time.perf_counter()
    try:
        async with session.post(url + "/generate", json=body) as r:
            await r.read()
            out.append(dict(status=r.status, total=time.perf_counter() - t0, tpt=float(r.headers.get("x-time-per-token", 0)),
                            queue=float(r.headers.get("x-queue-time", 0))))
    except Exception as e:  # connection errors count as failures
        out.append(dict(status=0, error=str(e)))


async def main(a):
    out, tasks = [], []
    body = {"inputs": a.prompt, "parameters": {"max_new_tokens": a.max_new_tokens, "do_sample": False}}
    if a.adapter_id:
        body["parameters"]["adapter_id"] = a.adapter_id
    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=300)) as s:
        t_end = time.perf_counter() + a.seconds
        while time.perf_counter() < t_end:
            tasks.append(asyncio.create_task(one(s, a.url, body, out)))
            await asyncio.sleep(1.0 / a.rps)
        await asyncio.gather(*tasks)
    ok = [r for r in out if r["status"] == 200]
    p95 = lambda xs: sorted(xs)[int(0.95 * (len(xs) - 1))] if xs else float("nan")
    res = dict(requests=len(out), failures=len(out) - len(ok), p95_time_per_token_ms=p95([r["tpt"] for r in ok]),
               p95_queue_time_ms=p95([r["queue"] for r in ok]), mean_total_s=statistics.mean([r["total"] for r in ok]) if ok else None)
    print(json.dumps(res))
    bad = res["failures"] > 0 or res["p95_time_per_token_ms"] > a.max_tpt_ms or res["p95_queue_time_ms"] > a.max_queue_ms
    sys.exit(1 if bad else 0)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:3000")
    ap.add_argument("--rps", type=float, default=10)
    ap.add_argument("--seconds", type=float, default=60)
    ap.add_argument("--max-new-tokens", type=int, default=60)
    ap.add_argument("--prompt", default="def print_hello")
    ap.add_argument("--adapter-id", default=None)
    ap.add_argument("--max-tpt-ms", type=float, default=90)
    ap.add_argument("--max-queue-ms", type=float, default=1500)
    asyncio.run(main(ap.parse_args()))
