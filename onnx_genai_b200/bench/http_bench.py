"""HTTP benchmarks against any OpenAI-compatible server: cross-runtime comparison and multi-turn sessions.

Two tools, both black-box (they only speak ``/v1/chat/completions`` / ``/v1/completions`` with ``stream: true``), so
the same command measures this server, the reference's server, or any other runtime side by side -- what the
reference's ``compare`` and ``multiturn`` binaries do (crates/onnx-genai-bench/README.md; src/bin/compare.rs,
src/bin/multiturn.rs):

``compare``    for each target and prompt: time to first token, decode rate after the first token, total latency,
               at a chosen concurrency, medians and p90 over repeats.
``multiturn``  one growing conversation, sent turn by turn; with ``--session`` the server keeps the conversation under an
               ``X-Session-Id`` and only the new turn is prefilled, without it the whole history is sent each time.  The
               per-turn time to first token shows what the session (or the server's prefix cache) saves.

Timing is wall clock on the client, per request, from just before the request is written to the arrival of each
streamed chunk.  Stdlib only (``http.client``), so the tool runs wherever Python does.

    python -m onnx_genai_b200.bench.http_bench compare --target ours=http://127.0.0.1:8000 --target other=http://127.0.0.1:8001 \\
        --prompt "Explain paged attention." --max-tokens 128 --concurrency 4 --repeats 5
    python -m onnx_genai_b200.bench.http_bench multiturn --url http://127.0.0.1:8000 --turns 6 --session
"""
from __future__ import annotations

import argparse
import http.client
import json
import statistics
import sys
import threading
import time
from urllib.parse import urlparse


def _connect(base_url: str, timeout: float):
    u = urlparse(base_url)
    cls = http.client.HTTPSConnection if u.scheme == "https" else http.client.HTTPConnection
    return cls(u.hostname, u.port or (443 if u.scheme == "https" else 80), timeout=timeout), (u.path.rstrip("/") or "")


def request_json(base_url: str, method: str, path: str, body=None, headers=None, timeout: float = 60.0):
    conn, prefix = _connect(base_url, timeout)
    try:
        data = json.dumps(body).encode() if body is not None else None
        conn.request(method, prefix + path, body=data, headers={"Content-Type": "application/json", **(headers or {})})
        resp = conn.getresponse()
        raw = resp.read()
        if resp.status >= 400:
            raise RuntimeError(f"{method} {base_url}{path} -> {resp.status}: {raw[:300].decode(errors='replace')}")
        return json.loads(raw) if raw else None
    finally:
        conn.close()


def stream_once(base_url: str, body: dict, chat: bool = True, headers=None, timeout: float = 600.0) -> dict:
    """One streamed request.  Returns ttft_ms, total_ms, chunks (streamed pieces with content), decode_tok_s (chunks after
    the first per second after the first), text, and usage when the server reports it."""
    conn, prefix = _connect(base_url, timeout)
    path = prefix + ("/v1/chat/completions" if chat else "/v1/completions")
    payload = json.dumps({**body, "stream": True}).encode()
    pieces, first, usage = [], None, None
    t0 = time.perf_counter()
    try:
        conn.request("POST", path, body=payload, headers={"Content-Type": "application/json", "Accept": "text/event-stream", **(headers or {})})
        resp = conn.getresponse()
        if resp.status >= 400:
            raise RuntimeError(f"POST {base_url}{path} -> {resp.status}: {resp.read()[:300].decode(errors='replace')}")
        while True:
            line = resp.readline()
            if not line:
                break
            line = line.strip()
            if not line.startswith(b"data:"):
                continue
            data = line[5:].strip()
            if data == b"[DONE]":
                break
            try:
                event = json.loads(data)
            except ValueError:
                continue
            usage = event.get("usage") or usage
            for choice in event.get("choices") or []:
                piece = (choice.get("delta") or {}).get("content") if chat else choice.get("text")
                if piece:
                    if first is None:
                        first = time.perf_counter()
                    pieces.append(piece)
        t1 = time.perf_counter()
    finally:
        conn.close()
    n = len(pieces)
    tokens = (usage or {}).get("completion_tokens") or n
    decode_s = (t1 - first) if first is not None else 0.0
    return {"ttft_ms": (first - t0) * 1e3 if first is not None else None, "total_ms": (t1 - t0) * 1e3, "chunks": n,
            "completion_tokens": tokens, "decode_tok_s": (tokens - 1) / decode_s if tokens > 1 and decode_s > 0 else None,
            "text": "".join(pieces), "usage": usage}


def _summary(values):
    vals = sorted(v for v in values if v is not None)
    if not vals:
        return None
    return {"p50": statistics.median(vals), "p90": vals[min(len(vals) - 1, int(0.9 * len(vals)))], "min": vals[0], "max": vals[-1], "n": len(vals)}


def compare(targets: dict, prompts: list, model: str | None = None, max_tokens: int = 64, concurrency: int = 1, repeats: int = 3,
            warmup: int = 1, chat: bool = True, temperature: float = 0.0) -> dict:
    """``targets``: name -> base URL.  Every target sees the same prompts, ``concurrency`` requests in flight at a time."""
    report = {}
    for name, url in targets.items():
        served = model
        if served is None:
            try:
                served = request_json(url, "GET", "/v1/models")["data"][0]["id"]
            except Exception:
                served = "default"

        def body(prompt):
            core = {"model": served, "max_tokens": max_tokens, "temperature": temperature}
            return {**core, "messages": [{"role": "user", "content": prompt}]} if chat else {**core, "prompt": prompt}

        for _ in range(warmup):
            stream_once(url, body(prompts[0]), chat)
        results, errors, lock = [], [], threading.Lock()
        jobs = [p for _ in range(repeats) for p in prompts]

        def worker():
            while True:
                with lock:
                    if not jobs:
                        return
                    prompt = jobs.pop()
                try:
                    r = stream_once(url, body(prompt), chat)
                    with lock:
                        results.append(r)
                except Exception as e:     # one failed request should not hide the others' numbers
                    with lock:
                        errors.append(str(e))

        t0 = time.perf_counter()
        threads = [threading.Thread(target=worker) for _ in range(max(1, concurrency))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        wall = time.perf_counter() - t0
        total_tokens = sum(r["completion_tokens"] for r in results)
        report[name] = {"url": url, "model": served, "requests": len(results), "errors": errors[:3], "concurrency": concurrency,
                        "ttft_ms": _summary(r["ttft_ms"] for r in results), "decode_tok_s": _summary(r["decode_tok_s"] for r in results),
                        "total_ms": _summary(r["total_ms"] for r in results),
                        "aggregate_tok_s": total_tokens / wall if wall > 0 else None}
    names = list(report)
    if len(names) >= 2 and report[names[0]]["ttft_ms"] and report[names[1]]["ttft_ms"]:
        a, b = report[names[0]], report[names[1]]
        report["ratio"] = {"of": f"{names[0]} / {names[1]}",
                           "ttft": a["ttft_ms"]["p50"] / b["ttft_ms"]["p50"],
                           "aggregate_tok_s": (a["aggregate_tok_s"] / b["aggregate_tok_s"]) if a["aggregate_tok_s"] and b["aggregate_tok_s"] else None}
    return report


def multiturn(url: str, turns: int = 4, model: str | None = None, max_tokens: int = 32, use_session: bool = True,
              user_text: str = "Tell me one more fact about memory hierarchies, in a sentence.") -> dict:
    """One conversation of ``turns`` user turns.  With a session only the new turn is sent (the server holds the history);
    without, the client resends the whole history each time."""
    served = model or request_json(url, "GET", "/v1/models")["data"][0]["id"]
    headers, sid = {}, None
    if use_session:
        made = request_json(url, "POST", "/v1/sessions")
        sid = made.get("id") or made.get("session_id")
        headers = {"X-Session-Id": sid}
    history, rows = [], []
    try:
        for turn in range(turns):
            msg = {"role": "user", "content": f"[turn {turn + 1}] {user_text}"}
            history.append(msg)
            body = {"model": served, "max_tokens": max_tokens, "temperature": 0.0, "messages": [msg] if use_session else list(history)}
            r = stream_once(url, body, True, headers)
            history.append({"role": "assistant", "content": r["text"]})
            rows.append({"turn": turn + 1, "ttft_ms": r["ttft_ms"], "total_ms": r["total_ms"], "completion_tokens": r["completion_tokens"],
                         "prompt_tokens": (r["usage"] or {}).get("prompt_tokens")})
    finally:
        if sid is not None:
            try:
                request_json(url, "DELETE", f"/v1/sessions/{sid}")
            except Exception:
                pass
    return {"url": url, "model": served, "session": use_session, "turns": rows,
            "ttft_ms_first": rows[0]["ttft_ms"] if rows else None, "ttft_ms_last": rows[-1]["ttft_ms"] if rows else None}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("compare")
    c.add_argument("--target", action="append", required=True, metavar="NAME=URL")
    c.add_argument("--prompt", action="append")
    c.add_argument("--model")
    c.add_argument("--max-tokens", type=int, default=64)
    c.add_argument("--concurrency", type=int, default=1)
    c.add_argument("--repeats", type=int, default=3)
    c.add_argument("--warmup", type=int, default=1)
    c.add_argument("--completions", action="store_true", help="use /v1/completions instead of chat")
    m = sub.add_parser("multiturn")
    m.add_argument("--url", required=True)
    m.add_argument("--turns", type=int, default=4)
    m.add_argument("--model")
    m.add_argument("--max-tokens", type=int, default=32)
    m.add_argument("--session", action="store_true")
    args = ap.parse_args(argv)
    if args.cmd == "compare":
        targets = {}
        for t in args.target:
            name, sep, url = t.partition("=")
            if not sep:
                ap.error(f"--target wants NAME=URL, got {t!r}")
            targets[name] = url
        out = compare(targets, args.prompt or ["Explain what a KV cache is in two sentences."], args.model, args.max_tokens,
                      args.concurrency, args.repeats, args.warmup, not args.completions)
    else:
        out = multiturn(args.url, args.turns, args.model, args.max_tokens, args.session)
    json.dump(out, sys.stdout, indent=2)
    sys.stdout.write("\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
