"""Cluster router: replica-level data parallelism behind one OpenAI endpoint.

Policy and health rules of the reference's router (crates/onnx-genai-router/src/router.rs:39-135,
node_poller.rs, session_map.rs): a request goes to (1) the node its ``X-Session-Id`` is pinned to,
else (2) a node that advertises the prompt's prefix hash, else (3) the least-loaded healthy node
(kv_usage, then queue depth).  Nodes are polled on ``/v1/status``; after ``unhealthy_after_misses``
(default 3) missed polls a node is demoted and its sessions migrate (a `MigrationEvent` is
recorded); drained nodes finish their sessions but take no new ones.  ``/router/*`` exposes
nodes, sessions, migrations and Prometheus counters.
"""
from __future__ import annotations

import asyncio
import hashlib
import json
import time
from dataclasses import dataclass, field


@dataclass
class NodeState:
    url: str
    healthy: bool = True
    draining: bool = False
    misses: int = 0
    kv_usage: float = 0.0
    queue_depth: int = 0
    tokens_per_second: float = 0.0
    prefix_hashes: set = field(default_factory=set)
    last_seen: float = 0.0


@dataclass
class MigrationEvent:
    session_id: str
    from_node: str
    to_node: str
    reason: str
    at: float


def prefix_hash(text: str, chars: int = 256) -> str:
    return hashlib.sha256(text[:chars].encode("utf-8", "ignore")).hexdigest()[:16]


class Router:
    def __init__(self, node_urls, unhealthy_after_misses: int = 3):
        self.nodes = {u: NodeState(u) for u in node_urls}
        self.unhealthy_after_misses = unhealthy_after_misses
        self.sessions: dict = {}          # session id -> node url
        self.migrations: list = []
        self.routed = {"affinity": 0, "prefix": 0, "least_loaded": 0}

    # -- health ---------------------------------------------------------------------------------
    def record_poll(self, url: str, status: dict | None):
        n = self.nodes[url]
        if status is None:
            n.misses += 1
            if n.misses >= self.unhealthy_after_misses and n.healthy:
                n.healthy = False
                self._migrate_sessions(url, "node missed %d status polls" % n.misses)
            return
        n.misses, n.healthy, n.last_seen = 0, True, time.time()
        n.kv_usage = float(status.get("kv_usage", 0.0))
        n.queue_depth = int(status.get("queue_depth", 0))
        n.tokens_per_second = float(status.get("tokens_per_second", 0.0))
        n.prefix_hashes = set(status.get("prefix_hashes") or [])

    def drain(self, url: str, on: bool = True):
        self.nodes[url].draining = on

    def _candidates(self):
        return [n for n in self.nodes.values() if n.healthy and not n.draining]

    def _migrate_sessions(self, url, reason):
        for sid, node in list(self.sessions.items()):
            if node == url:
                target = self._least_loaded()
                if target is None:
                    del self.sessions[sid]
                    continue
                self.sessions[sid] = target.url
                self.migrations.append(MigrationEvent(sid, url, target.url, reason, time.time()))

    def _least_loaded(self):
        c = self._candidates()
        return min(c, key=lambda n: (round(n.kv_usage, 2), n.queue_depth, n.url)) if c else None

    # -- routing --------------------------------------------------------------------------------
    def pick(self, session_id: str | None = None, prompt_text: str | None = None) -> NodeState:
        if session_id and session_id in self.sessions:
            n = self.nodes.get(self.sessions[session_id])
            if n is not None and n.healthy:      # a draining node still serves its existing sessions
                self.routed["affinity"] += 1
                return n
        cands = self._candidates()
        if not cands:
            raise RuntimeError("no healthy node is available; every node is down or draining")
        chosen = None
        if prompt_text:
            h = prefix_hash(prompt_text)
            holders = [n for n in cands if h in n.prefix_hashes]
            if holders:
                chosen = min(holders, key=lambda n: (n.queue_depth, n.url))
                self.routed["prefix"] += 1
        if chosen is None:
            chosen = self._least_loaded()
            self.routed["least_loaded"] += 1
        if session_id:
            self.sessions[session_id] = chosen.url
        return chosen

    def metrics_text(self) -> str:
        lines = ["# TYPE onnx_genai_router_routed_total counter"]
        for k, v in self.routed.items():
            lines.append(f'onnx_genai_router_routed_total{{policy="{k}"}} {v}')
        lines += ["# TYPE onnx_genai_router_nodes_healthy gauge",
                  f"onnx_genai_router_nodes_healthy {sum(n.healthy for n in self.nodes.values())}",
                  "# TYPE onnx_genai_router_migrations_total counter", f"onnx_genai_router_migrations_total {len(self.migrations)}"]
        return "\n".join(lines) + "\n"


def create_router_app(router: Router, poll_interval: float = 1.0):
    """aiohttp application: reverse proxy for /v1/* plus /router/{nodes,sessions,migrations,drain,metrics}."""
    import aiohttp
    from aiohttp import web

    async def poller(app):
        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=2)) as sess:
            while True:
                for url in list(router.nodes):
                    try:
                        async with sess.get(url + "/v1/status") as r:
                            router.record_poll(url, await r.json() if r.status == 200 else None)
                    except Exception:
                        router.record_poll(url, None)
                await asyncio.sleep(poll_interval)

    async def start(app):
        app["poller"] = asyncio.create_task(poller(app))

    async def stop(app):
        app["poller"].cancel()

    async def proxy(request: web.Request):
        body = await request.read()
        text = None
        try:
            obj = json.loads(body) if body else {}
            text = obj.get("prompt") if isinstance(obj.get("prompt"), str) else json.dumps(obj.get("messages", ""))[:512]
        except Exception:
            pass
        try:
            node = router.pick(request.headers.get("X-Session-Id"), text)
        except RuntimeError as exc:
            return web.json_response({"error": {"message": str(exc)}}, status=503)
        async with aiohttp.ClientSession() as sess:
            async with sess.request(request.method, node.url + request.rel_url.path_qs, data=body,
                                    headers={k: v for k, v in request.headers.items() if k.lower() not in ("host", "content-length")}) as up:
                resp = web.StreamResponse(status=up.status, headers={"Content-Type": up.headers.get("Content-Type", "application/json")})
                await resp.prepare(request)
                async for chunk in up.content.iter_any():
                    await resp.write(chunk)
                await resp.write_eof()
                return resp

    async def nodes(request):
        return web.json_response([{**n.__dict__, "prefix_hashes": sorted(n.prefix_hashes)} for n in router.nodes.values()])

    async def sessions(request):
        return web.json_response(router.sessions)

    async def migrations(request):
        return web.json_response([m.__dict__ for m in router.migrations])

    async def drain(request):
        data = await request.json()
        router.drain(data["url"], bool(data.get("drain", True)))
        return web.json_response({"ok": True})

    async def metrics(request):
        return web.Response(text=router.metrics_text(), content_type="text/plain")

    app = web.Application(client_max_size=25 * 1024 * 1024)
    app.on_startup.append(start)
    app.on_cleanup.append(stop)
    app.router.add_get("/router/nodes", nodes)
    app.router.add_get("/router/sessions", sessions)
    app.router.add_get("/router/migrations", migrations)
    app.router.add_post("/router/drain", drain)
    app.router.add_get("/router/metrics", metrics)
    app.router.add_route("*", "/{tail:.*}", proxy)
    return app
