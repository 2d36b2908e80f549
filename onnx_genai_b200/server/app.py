"""OpenAI-compatible HTTP server with SSE streaming.

Route surface of the reference's axum server (crates/onnx-genai-server/src/lib.rs:65-133):
``/health``, ``/v1/models``, ``/v1/status``, ``/v1/resources``, ``/v1/sessions`` (POST, DELETE),
``/v1/completions``, ``/v1/chat/completions`` (SSE when ``stream: true``), ``/v1/embeddings``
(declined with a precise error: decoder packages expose no pooled output), ``/metrics``
(Prometheus text) and opt-in ``/v1/debug/*``.  Like the reference (src/driver.rs:266-326) the
engine is owned by ONE driver thread; request handlers talk to it through queues, and the driver
runs the continuous-batching step loop so concurrent requests share every forward pass.
"""
from __future__ import annotations

import asyncio
import json
import queue
import threading
import time
import uuid

from fastapi import FastAPI, Header, HTTPException, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..engine.api import Engine, GenerateOptions
from .. import reasoning as reasoning_mod
from . import tools as tool_calls
from .metrics import Metrics


class EngineDriver:
    """Owns the engine on a dedicated thread; multiplexes requests into shared engine steps."""

    def __init__(self, engine: Engine, max_queue_depth: int = 256, admission_window_ms: float = 2.0):
        self.engine = engine
        # an idle driver that receives a request waits this long for companions before its first step, so
        # requests that arrive together prefill together (the reference's micro-batch window is 2-12 ms,
        # crates/onnx-genai-server/src/driver.rs:935-1050)
        self.admission_window_s = max(0.0, admission_window_ms) / 1e3
        self.inbox: queue.Queue = queue.Queue()
        self.max_queue_depth = max_queue_depth
        self.active: dict = {}
        self.tokens_generated = 0
        self.started = time.time()
        self._stop = False
        self.thread = threading.Thread(target=self._run, name="onnx-genai-batch-driver", daemon=True)
        self.thread.start()

    def submit(self, ids, opt: GenerateOptions, loop, out_q: asyncio.Queue):
        if self.inbox.qsize() + len(self.active) >= self.max_queue_depth:
            raise OverflowError("queue full")
        self.inbox.put(("gen", ids, opt, loop, out_q))

    def submit_embed(self, ids, loop, out_q: asyncio.Queue):
        if self.inbox.qsize() + len(self.active) >= self.max_queue_depth:
            raise OverflowError("queue full")
        self.inbox.put(("embed", ids, loop, out_q))

    def cancel(self, out_q):
        self.inbox.put(("cancel", out_q))

    def shutdown(self):
        self._stop = True
        self.inbox.put(("noop",))

    def _admit(self, item):
        kind = item[0]
        if kind == "gen":
            _, ids, opt, loop, out_q = item
            try:
                sid, state = self.engine._submit(ids, opt)
            except Exception as exc:
                loop.call_soon_threadsafe(out_q.put_nowait, ("error", str(exc)))
                return
            self.active[sid] = {"loop": loop, "q": out_q, "state": state, "out": [], "emitted": "", "opt": opt}
        elif kind == "embed":
            _, ids, loop, out_q = item
            try:
                import numpy as np

                sid = self.engine.llm.add_request(np.asarray(ids, dtype=np.int32), 1, temperature=0.0, ignore_eos=True)
            except Exception as exc:
                loop.call_soon_threadsafe(out_q.put_nowait, ("error", str(exc)))
                return
            self.engine.llm.hidden_taps[sid & 0x7FFFFFFF] = None
            self.active[sid] = {"loop": loop, "q": out_q, "embed": True}
        elif kind == "cancel":
            for sid, a in list(self.active.items()):
                if a["q"] is item[1]:
                    self.engine.llm.core.cancel(sid)
                    self.engine._finish(sid)
                    del self.active[sid]

    def _run(self):
        eng = self.engine
        while not self._stop:
            try:
                was_idle = not self.active
                item = self.inbox.get(timeout=0.25 if not self.active else 0.0)
                self._admit(item)
                if was_idle and self.admission_window_s > 0:
                    deadline = time.perf_counter() + self.admission_window_s
                    while True:
                        left = deadline - time.perf_counter()
                        if left <= 0:
                            break
                        self._admit(self.inbox.get(timeout=left))
                while True:
                    self._admit(self.inbox.get_nowait())
            except queue.Empty:
                pass
            if not self.active or not eng.llm.has_work:
                continue
            try:
                events = eng.llm.step().events
            except Exception as exc:  # fail every in-flight request with the cause, keep serving
                for sid, a in list(self.active.items()):
                    a["loop"].call_soon_threadsafe(a["q"].put_nowait, ("error", f"engine step failed: {exc}"))
                    eng._finish(sid)
                self.active.clear()
                continue
            for sid, tok, fin in events:
                a = self.active.get(sid)
                if a is None:
                    continue
                if a.get("embed"):
                    if fin is not None:
                        vec = eng.llm.hidden_taps.pop(sid & 0x7FFFFFFF, None)
                        eng.llm.core.release(sid)
                        eng.llm.stats.pop(sid, None)
                        a["loop"].call_soon_threadsafe(a["q"].put_nowait, ("embedding", vec))
                        del self.active[sid]
                    continue
                self.tokens_generated += 1
                a["out"].append(tok)
                a["state"]["ids"].append(tok)
                text = eng.detokenize(a["out"]) if eng.tokenizer is not None else ""
                delta = text[len(a["emitted"]):]
                for s in a["opt"].stop or ():
                    hit = text.find(s) if s else -1
                    if hit >= 0:
                        delta = text[len(a["emitted"]):hit] if hit > len(a["emitted"]) else ""
                        eng.llm.core.cancel(sid)
                        fin = "stop"
                        break
                if fin is None and eng.constraint_finished(a["state"]):
                    eng.llm.core.cancel(sid)
                    fin = "stop"
                if delta.endswith("�") and fin is None:
                    delta = ""  # incomplete UTF-8 sequence: wait for the next token
                a["emitted"] += delta
                a["loop"].call_soon_threadsafe(a["q"].put_nowait, ("token", tok, delta, fin))
                if fin is not None:
                    lp = list(a["state"]["logprobs"])
                    a["loop"].call_soon_threadsafe(a["q"].put_nowait, ("done", fin, len(a["out"]), lp))
                    eng._finish(sid, a["state"]["ids"])
                    del self.active[sid]


def _options_from_request(body: dict, default_max: int, max_cap: int) -> GenerateOptions:
    mt = body.get("max_completion_tokens", body.get("max_tokens", default_max))
    mt = max(0, min(int(mt if mt is not None else default_max), max_cap))
    temperature = body.get("temperature", 1.0)
    temperature = 1.0 if temperature is None else float(temperature)
    stop = body.get("stop") or ()
    if isinstance(stop, str):
        stop = (stop,)
    lp = body.get("top_logprobs") if body.get("logprobs") is True else (body.get("logprobs") if isinstance(body.get("logprobs"), int) else 0)
    if body.get("logprobs") is True and not lp:
        lp = 1
    if lp and int(lp) > 20:
        raise HTTPException(400, "top_logprobs must be <= 20")
    constraint = None
    rf = body.get("response_format") or {}
    if rf.get("type") == "json_object":
        constraint = ("json_object",)
    elif rf.get("type") == "json_schema":
        schema = (rf.get("json_schema") or {}).get("schema")
        if schema is None:
            raise HTTPException(400, "response_format.json_schema.schema is required when type is 'json_schema'")
        constraint = ("json_schema", schema)
    elif rf.get("type") not in (None, "text"):
        raise HTTPException(400, f"response_format.type {rf.get('type')!r} is not supported; use text, json_object or json_schema")
    if body.get("guided_regex"):
        constraint = ("regex", str(body["guided_regex"]))
    elif body.get("guided_choice"):
        constraint = ("choice", list(body["guided_choice"]))
    elif body.get("guided_json") is not None:
        constraint = ("json_schema", body["guided_json"])
    if constraint is not None:
        from ..engine import constraints as _cons

        try:
            _cons.make_constraint(constraint)      # reject unsupported schemas / patterns before queueing
        except ValueError as exc:
            raise HTTPException(400, str(exc)) from exc
    return GenerateOptions(
        constraint=constraint,
        max_new_tokens=mt, temperature=temperature, greedy=(temperature == 0.0), top_p=float(body.get("top_p") or 1.0),
        top_k=int(body.get("top_k") or 0), min_p=float(body.get("min_p") or 0.0), top_a=float(body.get("top_a") or 0.0),
        typical_p=float(body.get("typical_p") or 1.0), repetition_penalty=float(body.get("repetition_penalty") or 1.0),
        frequency_penalty=float(body.get("frequency_penalty") or 0.0), presence_penalty=float(body.get("presence_penalty") or 0.0),
        dry_multiplier=float(body.get("dry_multiplier") or 0.0), dry_base=float(body.get("dry_base") or 1.75),
        dry_allowed_length=int(body.get("dry_allowed_length") or 2), mirostat=bool(body.get("mirostat")),
        mirostat_tau=float(body.get("mirostat_tau") or 5.0), mirostat_eta=float(body.get("mirostat_eta") or 0.1),
        xtc_probability=float(body.get("xtc_probability") or 0.0), xtc_threshold=float(body.get("xtc_threshold") or 0.1),
        seed=int(body.get("seed") or 0), stop=tuple(stop), logprobs=int(lp or 0))


def create_app(engine: Engine, model_name: str = "model", max_output_tokens: int = 4096, max_queue_depth: int = 256,
               enable_debug_endpoints: bool = False, node_id: str = "node-0", admission_window_ms: float = 2.0,
               default_reasoning_effort: str | None = None, image_pipeline=None, speech_pipeline=None, transcriber=None,
               media_chat=None) -> FastAPI:
    app = FastAPI(title="onnx-genai-b200")
    driver = EngineDriver(engine, max_queue_depth, admission_window_ms)
    metrics = Metrics()
    app.state.driver, app.state.metrics, app.state.engine = driver, metrics, engine
    sessions: dict = {}
    # models whose chat template declares a thinking block get it returned as `reasoning_content`
    think = reasoning_mod.detect(getattr(engine, "chat_template", None))

    @app.middleware("http")
    async def trace_request(request: Request, call_next):
        t0 = time.perf_counter()
        response = await call_next(request)
        metrics.request(request.url.path, response.status_code, time.perf_counter() - t0)
        return response

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "onnx-genai-b200"}]}

    @app.get("/v1/status")
    async def status():
        snap = engine.resource_snapshot()
        up = max(1e-6, time.time() - driver.started)
        return {"node_id": node_id, "model": model_name, "kv_usage": snap["kv_usage"], "pages_total": snap["kv_pages_total"],
                "pages_free": snap["kv_pages_free"], "queue_depth": driver.inbox.qsize() + snap["waiting"],
                "active_requests": len(driver.active), "tokens_per_second": driver.tokens_generated / up,
                "batch_utilization": snap["running"] / max(1, engine.llm.cfg.max_seqs), "prefix_hashes": [],
                "sessions": len(sessions)}

    @app.get("/v1/resources")
    async def resources():
        snap = engine.resource_snapshot()
        cfg = engine.llm.cfg
        return {"limits": {"max_sessions": 256, "max_queue_depth": max_queue_depth, "max_output_tokens": max_output_tokens},
                "kv": {"pages_total": snap["kv_pages_total"], "page_tokens": 16, "dtype": cfg.kv_dtype},
                "batching": {"continuous": True, "max_batch": cfg.max_seqs, "max_tokens_per_step": cfg.max_tokens_per_step,
                             "chunked_prefill": cfg.prefill_chunk, "preemption": cfg.preempt}}

    @app.post("/v1/sessions")
    async def create_session():
        sid = "sess-" + uuid.uuid4().hex[:12]
        sessions[sid] = engine.create_session()
        return {"id": sid}

    @app.delete("/v1/sessions/{sid}")
    async def delete_session(sid: str):
        if sid not in sessions:
            raise HTTPException(404, f"session {sid!r} does not exist")
        engine.close_session(sessions.pop(sid))
        return {"id": sid, "deleted": True}

    @app.get("/metrics")
    async def prometheus():
        snap = engine.resource_snapshot()
        return PlainTextResponse(metrics.render(extra={
            "onnx_genai_active_sessions": len(sessions), "onnx_genai_pending_requests": driver.inbox.qsize(),
            "onnx_genai_batch_size": snap["running"], "onnx_genai_kv_pages_free": snap["kv_pages_free"],
            "onnx_genai_kv_pages_total": snap["kv_pages_total"], "onnx_genai_prefix_cache_hits_total": snap["prefix_cache_hits"],
            "onnx_genai_prefix_cache_lookups_total": snap["prefix_cache_lookups"], "onnx_genai_preemptions_total": snap["preemptions"],
            "onnx_genai_engine_steps_total": snap["steps"]}), media_type="text/plain; version=0.0.4")

    @app.post("/v1/embeddings")
    async def embeddings(request: Request):
        """Last-token pooling of the final-normed hidden state, L2-normalised (``encoding_format`` float only)."""
        import numpy as np

        body = await _json(request)
        inputs = body.get("input")
        if isinstance(inputs, str) or (isinstance(inputs, list) and inputs and isinstance(inputs[0], int)):
            inputs = [inputs]
        if not isinstance(inputs, list) or not inputs:
            raise HTTPException(400, "input must be a string, a list of strings, or token-id lists")
        if body.get("encoding_format", "float") != "float":
            raise HTTPException(400, "only encoding_format 'float' is supported")
        loop = asyncio.get_running_loop()
        queues, total = [], 0
        for item in inputs:
            ids = engine.tokenize(item) if isinstance(item, str) else [int(t) for t in item]
            if not ids:
                raise HTTPException(400, "an input is empty after tokenisation")
            if len(ids) >= engine.llm.cfg.max_seq_len:
                raise HTTPException(400, f"an input has {len(ids)} tokens but the model's context is {engine.llm.cfg.max_seq_len}")
            total += len(ids)
            q: asyncio.Queue = asyncio.Queue()
            try:
                driver.submit_embed(ids, loop, q)
            except OverflowError:
                metrics.rejected()
                raise HTTPException(429, f"request queue is full ({max_queue_depth} in flight); retry later")
            queues.append(q)
        data = []
        for i, q in enumerate(queues):
            ev = await q.get()
            if ev[0] == "error" or ev[1] is None:
                raise HTTPException(500, f"embedding failed: {ev[1]}")
            vec = np.asarray(ev[1], dtype=np.float32)
            vec = vec / max(float(np.linalg.norm(vec)), 1e-12)
            data.append({"object": "embedding", "index": i, "embedding": [float(v) for v in vec]})
        metrics.prompt_tokens(total)
        return {"object": "list", "model": model_name, "data": data, "usage": {"prompt_tokens": total, "total_tokens": total}}

    # Media routes of the reference server.  Image generation is served when a text-to-image workflow package is mounted
    # (``image_pipeline``, see server/images.py), speech synthesis when a speech package is (``speech_pipeline``, server/audio.py);
    # image-to-image comes with the image routes (and answers 400 when the workflow has no image input); transcription is
    # served when a transcriber is mounted (``transcriber``, server/transcribe.py); a route without its pipeline answers 501 with the reason.
    if image_pipeline is not None:
        from .images import add_image_routes

        add_image_routes(app, image_pipeline, model_name)
    if speech_pipeline is not None:
        from .audio import add_speech_routes

        add_speech_routes(app, speech_pipeline)
    if transcriber is not None:
        from .transcribe import add_transcription_routes

        add_transcription_routes(app, transcriber, model_name)
    def _not_served(kind: str):
        async def handler():
            raise HTTPException(501, f"{kind} needs a {kind.split()[0]} model pipeline; this server hosts decoder-only text models "
                                     "(chat, completions, embeddings)")
        return handler

    for _path, _kind in (("/v1/images/generations", "image generation"), ("/sdapi/v1/txt2img", "image generation"),
                         ("/sdapi/v1/img2img", "image generation"), ("/v1/audio/transcriptions", "audio transcription"),
                         ("/v1/audio/speech", "speech synthesis")):
        if image_pipeline is not None and _path in ("/v1/images/generations", "/sdapi/v1/txt2img", "/sdapi/v1/img2img"):
            continue
        if speech_pipeline is not None and _path == "/v1/audio/speech":
            continue
        if transcriber is not None and _path == "/v1/audio/transcriptions":
            continue
        app.post(_path)(_not_served(_kind))

    if enable_debug_endpoints:
        @app.get("/v1/debug/trace")
        async def debug_trace_summary():
            from ..utils import trace

            with trace.TRACER.lock:
                spans = list(trace.TRACER.spans)
            totals: dict = {}
            for name, a, b, _cat in spans:
                t = totals.setdefault(name, [0, 0.0])
                t[0] += 1
                t[1] += b - a
            return {"enabled": trace.TRACER.enabled, "spans": len(spans),
                    "stages": {k: {"calls": v[0], "total_ms": round(v[1] * 1e3, 3)} for k, v in sorted(totals.items())}}

        @app.get("/v1/debug/config")
        async def debug_config():
            from ..utils.runtime_config import runtime_config

            out = {k: (v if isinstance(v, (int, float, str, bool, type(None))) else str(v)) for k, v in engine.llm.cfg.__dict__.items()}
            out["environment"] = runtime_config().describe()       # what the ONNX_GENAI_* variables resolved to
            out["cuda_graph_declines"] = [{"bucket": list(k), "reason": why} for k, why in engine.llm.graph_declines]
            out["device_faults"] = engine.llm.device_faults
            return out

        @app.get("/v1/debug/kv")
        async def debug_kv():
            return engine.resource_snapshot()

        @app.get("/v1/debug/sessions")
        async def debug_sessions():
            return {"sessions": [{"id": k, "tokens": engine.session_len(v)} for k, v in sessions.items()],
                    "active_requests": len(driver.active), "queued": driver.inbox.qsize()}

        @app.get("/v1/debug/profile")
        async def debug_profile():
            from .. import ops

            return {"launch_counts": dict(ops.launch_counts), "engine_steps": engine.llm.steps,
                    "graph_replays": engine.llm.graph_replays, "graph_declines": [str(d) for d in engine.llm.graph_declines],
                    "h2d_bytes": engine.llm.h2d_bytes, "d2h_bytes": engine.llm.d2h_bytes}

        @app.get("/v1/debug/trace/perfetto")
        async def debug_trace():
            from ..utils import trace

            return JSONResponse(trace.chrome_trace_events())

    async def _run_generation(ids, opt, request: Request):
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        try:
            driver.submit(ids, opt, loop, q)
        except OverflowError:
            metrics.rejected()
            raise HTTPException(429, f"request queue is full ({max_queue_depth} in flight); retry later")
        return q

    def _prompt_ids(body, chat: bool, session_header):
        if chat:
            msgs = body.get("messages")
            if not isinstance(msgs, list) or not msgs:
                raise HTTPException(400, "messages must be a non-empty list of {role, content} objects")
            from . import multimodal as mm

            try:
                norm, images, audio = mm.split_content(msgs)
                if images or audio:
                    # media attachments go to the mounted media chat (a workflow package with a typed media input)
                    mm.admit_attachments(media_chat, model_name, len(images), len(audio))
                    body["_media"] = {"image": images[0] if images else None, "audio": audio[0] if audio else None}
            except mm.MediaError as exc:
                raise HTTPException(exc.status, str(exc)) from exc
            tools = body.get("tools")
            if body.get("tool_choice") == "none":
                tools = None
            if tools:
                norm = tool_calls.inject_tool_prompt(norm, tools, body.get("tool_choice"))
            if body.get("response_format", {}).get("type") in ("json_object", "json_schema"):
                norm = norm + [{"role": "system", "content": "Respond with a single valid JSON object and nothing else."}]
            # templates that take a reasoning effort (low / medium / high) read it as a variable; others ignore it
            effort = body.get("reasoning_effort") or default_reasoning_effort
            if effort is not None and effort not in ("low", "medium", "high"):
                raise HTTPException(400, f"reasoning_effort must be low, medium or high, not {effort!r}")
            text = engine.apply_chat_template(norm, add_generation_prompt=True, tools=tools,
                                              **({"reasoning_effort": effort} if effort else {}))
        else:
            text = body.get("prompt")
            if isinstance(text, list):
                text = text[0] if text and isinstance(text[0], str) else text
            if body.get("suffix") and isinstance(text, str):  # fill-in-the-middle
                try:
                    text = engine.fim_prompt(text, body["suffix"])
                except ValueError as exc:
                    raise HTTPException(400, str(exc)) from exc
        ids = engine.tokenize(text) if isinstance(text, str) else [int(t) for t in (text or [])]
        if not ids:
            raise HTTPException(400, "the prompt is empty after tokenisation")
        if session_header and session_header in sessions:
            hist = engine._session(sessions[session_header]).tokens
            ids = hist + ids
        limit = engine.llm.cfg.max_seq_len
        if len(ids) >= limit:
            raise HTTPException(400, f"prompt has {len(ids)} tokens but the model's context is {limit}; shorten the prompt")
        return ids

    async def _complete_with_media(body: dict, ids, opt, rid: str, created: int):
        """A chat request that carries an image or an audio clip: the media chat's workflow runs the whole generation
        (encoder, merge, decoder loop); the answer is returned whole, or as one content chunk when streaming."""
        media = body["_media"]
        loop = asyncio.get_running_loop()
        t0 = time.perf_counter()
        try:
            out_ids = await loop.run_in_executor(None, lambda: media_chat.generate(
                ids, image=media["image"], audio=media["audio"], max_new_tokens=opt.max_new_tokens))
        except Exception as exc:
            raise HTTPException(422, f"the media input could not be processed: {exc}") from exc
        text = engine.detokenize(list(out_ids))
        metrics.prompt_tokens(len(ids))
        metrics.completion_tokens(len(out_ids))
        metrics.ttft(time.perf_counter() - t0)
        metrics.e2e(time.perf_counter() - t0)
        usage = {"prompt_tokens": len(ids), "completion_tokens": len(out_ids), "total_tokens": len(ids) + len(out_ids)}
        fin = "length" if len(out_ids) >= opt.max_new_tokens else "stop"
        if body.get("stream"):
            async def gen():
                base = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": model_name}
                yield _sse({**base, "choices": [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]})
                if text:
                    yield _sse({**base, "choices": [{"index": 0, "delta": {"content": text}, "finish_reason": None}]})
                yield _sse({**base, "choices": [{"index": 0, "delta": {}, "finish_reason": fin}], "usage": usage})
                yield "data: [DONE]\n\n"

            return StreamingResponse(gen(), media_type="text/event-stream")
        thought, answer = reasoning_mod.split(text, think)
        msg = {"role": "assistant", "content": answer}
        if thought is not None:
            msg["reasoning_content"] = thought
        return JSONResponse({"id": rid, "object": "chat.completion", "created": created, "model": model_name,
                             "choices": [{"index": 0, "message": msg, "finish_reason": fin}], "usage": usage})

    async def _complete(body: dict, request: Request, chat: bool, session_header):
        opt = _options_from_request(body, 256, max_output_tokens)
        n_choices = body.get("n", 1)
        if not isinstance(n_choices, int) or isinstance(n_choices, bool) or not 1 <= n_choices <= 16:
            raise HTTPException(400, f"n must be an integer between 1 and 16, not {n_choices!r}")
        if n_choices > 1 and body.get("stream"):
            raise HTTPException(400, "n > 1 is not supported with stream: true; request the samples without streaming")
        ids = _prompt_ids(body, chat, session_header)
        rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]
        created = int(time.time())
        if body.get("_media"):
            return await _complete_with_media(body, ids, opt, rid, created)
        q = await _run_generation(ids, opt, request)
        t0 = time.perf_counter()
        metrics.prompt_tokens(len(ids))
        obj = "chat.completion" if chat else "text_completion"

        def finish_session(out_ids):
            if session_header and session_header in sessions:
                engine._session(sessions[session_header]).tokens = ids + list(out_ids)

        if body.get("stream"):
            async def gen():
                first = True
                out_ids = []
                splitter = reasoning_mod.StreamSplitter(think if chat else None)
                try:
                    if chat:
                        yield _sse({"id": rid, "object": obj + ".chunk", "created": created, "model": model_name,
                                    "choices": [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]})
                    while True:
                        ev = await q.get()
                        if ev[0] == "error":
                            yield _sse({"error": {"message": ev[1], "type": "engine_error"}})
                            break
                        if ev[0] == "token":
                            _, tok, delta, fin = ev
                            out_ids.append(tok)
                            if first:
                                metrics.ttft(time.perf_counter() - t0)
                                first = False
                            if delta:
                                if chat:
                                    r_d, a_d = splitter.feed(delta)
                                    payload = {}
                                    if r_d:
                                        payload["reasoning_content"] = r_d
                                    if a_d:
                                        payload["content"] = a_d
                                    if not payload:
                                        continue
                                    choice = {"index": 0, "delta": payload, "finish_reason": None}
                                else:
                                    choice = {"index": 0, "text": delta, "finish_reason": None}
                                yield _sse({"id": rid, "object": obj + ".chunk", "created": created, "model": model_name,
                                            "choices": [choice]})
                        elif ev[0] == "done":
                            _, fin, n, _lp = ev
                            metrics.completion_tokens(n)
                            metrics.e2e(time.perf_counter() - t0)
                            choice = ({"index": 0, "delta": {}, "finish_reason": fin} if chat
                                      else {"index": 0, "text": "", "finish_reason": fin})
                            yield _sse({"id": rid, "object": obj + ".chunk", "created": created, "model": model_name,
                                        "choices": [choice],
                                        "usage": {"prompt_tokens": len(ids), "completion_tokens": n, "total_tokens": len(ids) + n}})
                            finish_session(out_ids)
                            break
                    yield "data: [DONE]\n\n"
                except asyncio.CancelledError:
                    driver.cancel(q)
                    raise

            return StreamingResponse(gen(), media_type="text/event-stream")

        async def collect(queue, pending=None):
            """Drain one generation: (text, token ids, finish reason, logprobs)."""
            text, out_ids, fin, lps = "", [], None, []
            while True:
                ev = pending if pending is not None else await queue.get()
                pending = None
                if ev[0] == "error":
                    raise HTTPException(500, ev[1])
                if ev[0] == "token":
                    if not out_ids:
                        metrics.ttft(time.perf_counter() - t0)
                    out_ids.append(ev[1])
                    text += ev[2]
                elif ev[0] == "done":
                    return text, out_ids, ev[1], ev[3]

        def make_choice(index, text, out_ids, fin, lps):
            if chat:
                thought, text = reasoning_mod.split(text, think)
                msg = {"role": "assistant", "content": text}
                if thought is not None:
                    msg["reasoning_content"] = thought
                calls = tool_calls.parse_tool_calls(text) if body.get("tools") else []
                if calls:
                    msg = {"role": "assistant", "content": None, "tool_calls": calls}
                    fin = "tool_calls"
                choice = {"index": index, "message": msg, "finish_reason": fin}
                if lps:
                    choice["logprobs"] = {"content": [
                        {"token": engine.detokenize([t]), "logprob": lp, "top_logprobs": [{"token": engine.detokenize([i]), "logprob": l} for i, l in top]}
                        for t, (lp, top) in zip(out_ids, lps)]}
            else:
                choice = {"index": index, "text": text, "finish_reason": fin}
                if lps:
                    choice["logprobs"] = {"tokens": [engine.detokenize([t]) for t in out_ids], "token_logprobs": [lp for lp, _ in lps]}
            return choice

        queues, first_event = [q], None
        if n_choices > 1:
            # the other samples are submitted once the first has produced a token: by then its prompt pages are in the
            # prefix cache, so the copies prefill only the last partial page instead of the whole prompt again
            import dataclasses

            first_event = await q.get()
            for i in range(1, n_choices):
                queues.append(await _run_generation(ids, dataclasses.replace(opt, seed=(opt.seed or 0) + i), request))
        results = [await collect(q, first_event)] + [await collect(other) for other in queues[1:]]
        total_out = sum(len(r[1]) for r in results)
        metrics.completion_tokens(total_out)
        metrics.e2e(time.perf_counter() - t0)
        finish_session(results[0][1])
        usage = {"prompt_tokens": len(ids), "completion_tokens": total_out, "total_tokens": len(ids) + total_out}
        choices = [make_choice(i, *r) for i, r in enumerate(results)]
        return JSONResponse({"id": rid, "object": obj, "created": created, "model": model_name, "choices": choices, "usage": usage})

    @app.post("/v1/completions")
    async def completions(request: Request, x_session_id: str | None = Header(default=None)):
        return await _complete(await _json(request), request, False, x_session_id)

    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request, x_session_id: str | None = Header(default=None)):
        return await _complete(await _json(request), request, True, x_session_id)

    @app.on_event("shutdown")
    async def _shutdown():
        driver.shutdown()

    return app


async def _json(request: Request) -> dict:
    try:
        body = await request.json()
    except Exception:
        raise HTTPException(400, "request body is not valid JSON")
    if not isinstance(body, dict):
        raise HTTPException(400, "request body must be a JSON object")
    return body


def _sse(obj) -> str:
    return "data: " + json.dumps(obj, ensure_ascii=False) + "\n\n"
