"""Service checker: drives a RUNNING server over HTTP and decides whether a real forward pass answers.

    python bench/service_check.py --url http://127.0.0.1:8000 [--model NAME] [--gates echo,answers,determinism,stream]
                                  [--n 20] [--concurrency 8] [--seed 0]

Needs no weights and no GPU on the checking side. Four gates, each a rate against a threshold:

* ``echo`` (>= 0.90): every request carries a fresh random sentinel that the prompt asks the model to repeat; canned
  or templated output cannot contain it.
* ``answers`` (>= 0.75): factual prompts at temperature 0 with one fixed answer; a prompt echoer fails here.
* ``determinism`` (>= 0.90): the same prompt twice at temperature 0, streamed, must give the same text.
* ``stream`` (>= 0.90): a streamed and a non-streamed request of the same prompt give the same text.

``echo`` and ``answers`` need the real checkpoint; a server with random weights (tests, benches) is checked with
``--gates determinism,stream``. Prints one JSON line; exit code 0 iff no transport error happened and every chosen
gate cleared its threshold (reference: ``.vibesys/tasks/default/accuracy_checker/checker.py:119-351``)."""

from __future__ import annotations

import argparse
import json
import random
import string
import sys
from concurrent.futures import ThreadPoolExecutor

import requests

THRESHOLDS = {"echo": 0.90, "answers": 0.75, "determinism": 0.90, "stream": 0.90}

KNOWN = [
    ("What is the capital of France? Answer with one word.", ["paris"]),
    ("What is 1 + 1? Answer with the number only.", ["2", "two"]),
    ("What is the chemical symbol for water? Answer briefly.", ["h2o"]),
    ("How many days are there in a week? Answer with the number only.", ["7", "seven"]),
    ("What colour do you get when you mix blue and yellow? Answer with one word.", ["green"]),
    ("What is the opposite of hot? Answer with one word.", ["cold"]),
    ("Which planet is known as the Red Planet? Answer with one word.", ["mars"]),
    ("What is 10 divided by 2? Answer with the number only.", ["5", "five"]),
    ("What is the first letter of the English alphabet? Answer with the letter only.", ["a"]),
    ("What is the largest ocean on Earth? Answer briefly.", ["pacific"]),
]

NEUTRAL = [
    "Write one sentence about the sea.", "Name three fruits.", "Describe a quiet morning in a few words.",
    "Give a short definition of a river.", "List two uses of a hammer.", "Say something about winter.",
    "What does a librarian do?", "Explain what a bridge is for.", "Describe the colour of the sky at noon.",
    "What is a bicycle?",
]


def chat_text(url: str, model: str | None, content: str, max_tokens: int, stream: bool, timeout: float) -> tuple[str, str | None]:
    """One greedy chat request; returns ``(text, error)``. Reasoning deltas are not part of the text."""
    body = {"messages": [{"role": "user", "content": content}], "max_tokens": max_tokens, "temperature": 0, "stream": stream}
    if model:
        body["model"] = model
    try:
        if not stream:
            r = requests.post(url + "/v1/chat/completions", json=body, timeout=timeout)
            r.raise_for_status()
            return (r.json()["choices"][0]["message"].get("content") or ""), None
        parts = []
        with requests.post(url + "/v1/chat/completions", json=body, stream=True, timeout=timeout) as r:
            r.raise_for_status()
            for line in r.iter_lines():
                if not line.startswith(b"data: ") or line == b"data: [DONE]":
                    continue
                for ch in json.loads(line[6:]).get("choices", []):
                    piece = (ch.get("delta") or {}).get("content")
                    if piece:
                        parts.append(piece)
        return "".join(parts), None
    except (requests.RequestException, KeyError, IndexError, ValueError) as e:
        return "", f"{type(e).__name__}: {e}"


def run_gates(url: str, model: str | None, gates: list[str], n: int, concurrency: int, seed: int, timeout: float = 600.0) -> dict:
    rng = random.Random(seed)
    url = url.rstrip("/")
    jobs: list[tuple[str, object]] = []  # (gate, payload)
    if "echo" in gates:
        for _ in range(n):
            s = "".join(rng.choice(string.ascii_uppercase + string.digits) for _ in range(10))
            jobs.append(("echo", s))
    if "answers" in gates:
        for i in range(n):
            jobs.append(("answers", KNOWN[i % len(KNOWN)]))
    if "determinism" in gates:
        for i in range(n):
            jobs.append(("determinism", f"{NEUTRAL[i % len(NEUTRAL)]} (request {rng.randrange(10**6)})"))
    if "stream" in gates:
        for i in range(n):
            jobs.append(("stream", f"{NEUTRAL[(i + 3) % len(NEUTRAL)]} (request {rng.randrange(10**6)})"))

    def one(job) -> tuple[str, bool, str | None]:
        gate, payload = job
        if gate == "echo":
            text, err = chat_text(url, model, f"Repeat the following code exactly and say nothing else: {payload}", 32, True, timeout)
            return gate, payload in text, err
        if gate == "answers":
            q, accepted = payload
            text, err = chat_text(url, model, q, 32, True, timeout)
            low = text.lower()
            return gate, any(a in low for a in accepted), err
        if gate == "determinism":
            a, e1 = chat_text(url, model, payload, 48, True, timeout)
            b, e2 = chat_text(url, model, payload, 48, True, timeout)
            return gate, a == b and (a != "" or e1 is None), e1 or e2
        a, e1 = chat_text(url, model, payload, 48, True, timeout)
        b, e2 = chat_text(url, model, payload, 48, False, timeout)
        return gate, a == b, e1 or e2

    with ThreadPoolExecutor(max_workers=max(1, concurrency)) as pool:
        results = list(pool.map(one, jobs))
    out: dict = {"url": url, "requests": len(jobs), "errors": [e for _, _, e in results if e][:5],
                 "error_count": sum(1 for _, _, e in results if e), "gates": {}}
    ok = out["error_count"] == 0
    for gate in gates:
        mine = [good for g, good, _ in results if g == gate]
        rate = sum(mine) / len(mine) if mine else 0.0
        passed = rate >= THRESHOLDS[gate]
        out["gates"][gate] = {"rate": round(rate, 3), "threshold": THRESHOLDS[gate], "n": len(mine), "pass": passed}
        ok = ok and passed
    out["pass"] = ok
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--url", required=True)
    ap.add_argument("--model", default=None)
    ap.add_argument("--gates", default="echo,answers,determinism,stream")
    ap.add_argument("--n", type=int, default=20, help="requests per gate")
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    gates = [g for g in args.gates.split(",") if g]
    unknown = [g for g in gates if g not in THRESHOLDS]
    if unknown:
        ap.error(f"unknown gate(s) {unknown}; choose from {sorted(THRESHOLDS)}")
    out = run_gates(args.url, args.model, gates, args.n, args.concurrency, args.seed)
    print(json.dumps(out), flush=True)
    return 0 if out["pass"] else 1


if __name__ == "__main__":
    sys.exit(main())
