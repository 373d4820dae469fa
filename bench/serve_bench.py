"""Client-side load generator for a running server: output tok/s, TTFT and TPOT percentiles.

    python bench/serve_bench.py --url http://127.0.0.1:8000 --model NAME --vocab 248320 \
        --concurrency 256 --requests 256 --prompt-len 2048 --output-len 256            # 256 simultaneous requests
    python bench/serve_bench.py ... --sessions 64 --rounds 4-8 --rate 4 --first-len 6000 \
        --grow 100-2000 --output-len 50-800                                            # multi-round sessions

Requests stream token ids (``return_token_ids``), greedy, ``ignore_eos``, exact ``max_tokens``;
every token's arrival time is recorded on the client. Definitions (same as the reference's own probe,
``tools/serve_probe.py:197-226``): TTFT = first token time - request start; TPOT = (last - first token
time) / (n - 1); output tok/s = all output tokens / wall time of the run. A session's round r+1 prompt is
round r's prompt + its output ids + new random tokens, so the server's session-tail cache is exercised;
``cached_tokens`` from the usage chunk is summed.

    python bench/serve_bench.py ... --trace bench/sample_trace.csv --concurrency 8    # recorded-trace replay

``--trace`` replays a CSV of ``session_id,round_idx,input_len,output_len,prefix_len,tool_wait_after_ms`` rows
(the column layout of the reference's recorded sample, ``.vibesys/shared/tracelab/recorded_sessions.csv``):
round r of a session sends the first ``prefix_len`` tokens of what the session has seen so far (its previous
prompt plus the ids the server generated) followed by ``input_len`` new random tokens, asks for exactly
``output_len`` tokens, then sleeps ``tool_wait_after_ms``. ``--concurrency`` is the number of session slots.

A run is ``valid`` only when every planned step ran, none failed and the output total equals the requested one
(``attempted_steps`` / ``success_steps`` / ``failed_steps`` / ``target_output_tokens`` in the JSON line, the rule
of the reference's replay harness, ``.vibesys/shared/tracelab/replay.py:37-66``); otherwise the exit code is 1.
A failed step ends its session.
"""

from __future__ import annotations

import argparse
import json
import random
import sys
import threading
import time

import requests


def _range(text: str) -> tuple[int, int]:
    if "-" in text:
        a, b = text.split("-")
        return int(a), int(b)
    return int(text), int(text)


def stream_once(url: str, model: str, prompt: list[int], max_tokens: int) -> dict:
    body = {"model": model, "prompt": prompt, "max_tokens": max_tokens, "temperature": 0, "ignore_eos": True,
            "return_token_ids": True, "stream": True, "stream_options": {"include_usage": True}}
    t0 = time.perf_counter()
    stamps, ids, usage, error = [], [], None, None
    try:
        with requests.post(url + "/v1/completions", json=body, stream=True, timeout=3600) as r:
            r.raise_for_status()
            for line in r.iter_lines():
                if not line.startswith(b"data: ") or line == b"data: [DONE]":
                    continue
                ev = json.loads(line[6:])
                if ev.get("error"):
                    error = str(ev["error"])[:200]
                if ev.get("usage"):
                    usage = ev["usage"]
                for ch in ev.get("choices", []):
                    toks = ch.get("token_ids") or []
                    if toks:
                        stamps.append(time.perf_counter())
                        ids.extend(toks)
    except (requests.RequestException, ValueError) as e:  # a failed step is counted, and ends its session's later rounds
        error = f"{type(e).__name__}: {e}"[:200]
    if error is None and len(ids) != max_tokens:
        error = f"{len(ids)} tokens for max_tokens={max_tokens} with ignore_eos"
    return {"start": t0, "stamps": stamps, "ids": ids, "usage": usage or {}, "target": max_tokens, "error": error}


def pct(vals: list[float], p: float) -> float | None:
    if not vals:
        return None
    s = sorted(vals)
    return s[min(len(s) - 1, int(p * len(s)))]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", required=True)
    ap.add_argument("--model", required=True)
    ap.add_argument("--vocab", type=int, default=248320)
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--requests", type=int, default=0, help="single-round mode: number of requests")
    ap.add_argument("--prompt-len", default="1024")
    ap.add_argument("--output-len", default="128")
    ap.add_argument("--sessions", type=int, default=0, help="multi-round mode: number of sessions")
    ap.add_argument("--rounds", default="4-8")
    ap.add_argument("--first-len", type=int, default=6000, help="median of the lognormal first-round prompt length")
    ap.add_argument("--max-first-len", type=int, default=65536)
    ap.add_argument("--grow", default="100-2000")
    ap.add_argument("--rate", type=float, default=0.0, help="Poisson arrivals per second (0 = all at once)")
    ap.add_argument("--trace", default="", help="CSV of recorded sessions to replay")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    rng = random.Random(a.seed)
    lo_v, hi_v = 3, a.vocab - 1
    out_lo, out_hi = _range(a.output_len)
    results, lock = [], threading.Lock()
    gate = threading.Semaphore(a.concurrency)

    def run_session(first_prompt: list[int], rounds: int, grow: tuple[int, int], delay: float, srng: random.Random) -> None:
        time.sleep(delay)
        prompt = first_prompt
        for r in range(rounds):
            with gate:
                res = stream_once(a.url, a.model, prompt, srng.randint(out_lo, out_hi))
            res["round"] = r
            with lock:
                results.append(res)
            if res["error"]:
                return
            prompt = prompt + res["ids"] + [srng.randint(lo_v, hi_v) for _ in range(srng.randint(*grow))]

    def run_trace(rows: list[dict], srng: random.Random) -> None:
        seen: list[int] = []
        with gate:  # a session holds its slot through tool waits, as the recorded runner does
            for row in rows:
                keep = min(int(row["prefix_len"]), len(seen))
                pad = int(row["prefix_len"]) - keep
                prompt = seen[:keep] + [srng.randint(lo_v, hi_v) for _ in range(pad + int(row["input_len"]))]
                res = stream_once(a.url, a.model, prompt, int(row["output_len"]))
                res["round"] = int(row["round_idx"])
                with lock:
                    results.append(res)
                if res["error"]:
                    return
                seen = prompt + res["ids"]
                time.sleep(int(row.get("tool_wait_after_ms") or 0) / 1e3)

    threads = []
    t_arrive = 0.0
    by_session: dict[str, list[dict]] = {}
    if a.trace:
        import csv

        with open(a.trace, newline="") as f:
            for row in csv.DictReader(f):
                by_session.setdefault(row["session_id"], []).append(row)
        for rows in by_session.values():
            rows.sort(key=lambda r: int(r["round_idx"]))
            threads.append(threading.Thread(target=run_trace, args=(rows, random.Random(rng.random()))))
    elif a.sessions:
        r_lo, r_hi = _range(a.rounds)
        for _ in range(a.sessions):
            n = int(min(a.max_first_len, max(16, rng.lognormvariate(0, 0.8) * a.first_len)))
            srng = random.Random(rng.random())
            first = [srng.randint(lo_v, hi_v) for _ in range(n)]
            if a.rate > 0:
                t_arrive += rng.expovariate(a.rate)
            threads.append(threading.Thread(target=run_session, args=(first, rng.randint(r_lo, r_hi), _range(a.grow), t_arrive, srng)))
    else:
        p_lo, p_hi = _range(a.prompt_len)
        for _ in range(a.requests or a.concurrency):
            srng = random.Random(rng.random())
            first = [srng.randint(lo_v, hi_v) for _ in range(srng.randint(p_lo, p_hi))]
            if a.rate > 0:
                t_arrive += rng.expovariate(a.rate)
            threads.append(threading.Thread(target=run_session, args=(first, 1, (0, 0), t_arrive, srng)))
    t0 = time.perf_counter()
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    ttft = [r["stamps"][0] - r["start"] for r in results if r["stamps"]]
    tpot = [(r["stamps"][-1] - r["stamps"][0]) / (len(r["stamps"]) - 1) for r in results if len(r["stamps"]) > 1]
    first_round = [r["stamps"][0] - r["start"] for r in results if r["stamps"] and r["round"] == 0]
    later = [r["stamps"][0] - r["start"] for r in results if r["stamps"] and r["round"] > 0]
    tokens = sum(len(r["ids"]) for r in results)
    failed = [r for r in results if r["error"]]
    planned = sum(len(v) for v in by_session.values()) if a.trace else None
    target = sum(int(row["output_len"]) for v in by_session.values() for row in v) if a.trace else sum(r["target"] for r in results)
    # a replay counts only when every planned step ran, none failed and the output total is exact (the rule of the
    # reference's harness, .vibesys/shared/tracelab/replay.py:37-66)
    valid = not failed and tokens == target and (planned is None or planned == len(results))
    ms = lambda v: None if v is None else round(v * 1e3, 2)  # noqa: E731
    print(json.dumps({
        "requests": len(results), "output_tokens": tokens, "wall_s": round(wall, 3),
        "attempted_steps": len(results), "success_steps": len(results) - len(failed), "failed_steps": len(failed),
        "planned_steps": planned, "target_output_tokens": target, "valid": valid, "errors": [r["error"] for r in failed][:3],
        "output_tok_s": round(tokens / wall, 1),
        "ttft_ms": {"p50": ms(pct(ttft, 0.5)), "p90": ms(pct(ttft, 0.9))},
        "ttft_first_round_ms_p50": ms(pct(first_round, 0.5)), "ttft_later_rounds_ms_p50": ms(pct(later, 0.5)),
        "tpot_ms": {"p50": ms(pct(tpot, 0.5)), "p90": ms(pct(tpot, 0.9))},
        "prompt_tokens": sum(r["usage"].get("prompt_tokens", 0) for r in results),
        "cached_tokens": sum((r["usage"].get("prompt_tokens_details") or {}).get("cached_tokens", 0) for r in results),
    }), flush=True)
    if not valid:
        sys.exit(1)


if __name__ == "__main__":
    main()
