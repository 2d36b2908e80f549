"""Several models behind one endpoint: a registry that loads on demand and evicts the least recently used.

``ModelRegistry`` maps model names to model directories.  A request names its model in the JSON body
(``"model"``); the registry loads it on first use (one :func:`create_app` sub-application and one engine driver
per loaded model), keeps at most ``max_loaded`` models resident and, when a new one must come in, shuts down the
least recently used model that has no request in flight.  ``warmup`` loads a list of models at start.  This is
the role of the reference server's ``--models-dir / --models-config / --max-loaded-models`` options
(crates/onnx-genai-server/src/cli.rs:27-145).

``RegistryApp`` is the ASGI front: it answers ``/v1/models`` and ``/health`` itself, reads the body of every other
request to find the model, and forwards the request unchanged to that model's sub-application.
"""
from __future__ import annotations

import asyncio
import json
import os
import threading
import time
from collections import OrderedDict

from ..engine.api import Engine
from .app import create_app


class ModelRegistry:
    def __init__(self, models: dict, max_loaded: int = 1, loader=None, **app_kw):
        if not models:
            raise ValueError("the model registry needs at least one model (name -> directory)")
        self.models = dict(models)
        self.max_loaded = max(1, int(max_loaded))
        self.loader = loader or (lambda path: Engine.from_dir(path))
        self.app_kw = app_kw
        self.loaded: OrderedDict = OrderedDict()   # name -> {"app", "engine", "inflight", "loaded_at"}
        self.lock = threading.Lock()
        self.loads = 0
        self.evictions = 0

    @classmethod
    def from_dir(cls, models_dir: str, **kw):
        """Every sub-directory that holds a model (inference metadata, a manifest or an .onnx file) is one model."""
        found = {}
        for name in sorted(os.listdir(models_dir)):
            path = os.path.join(models_dir, name)
            if os.path.isdir(path) and any(f.endswith((".onnx", ".yaml", ".yml")) or f == "manifest.json" for f in os.listdir(path)):
                found[name] = path
        return cls(found, **kw)

    @property
    def default(self) -> str:
        return next(iter(self.models))

    def names(self):
        return list(self.models)

    def acquire(self, name: str | None):
        """The loaded entry for ``name`` (loading and evicting as needed); marks one request in flight."""
        name = name or self.default
        if name not in self.models:
            raise KeyError(f"model {name!r} is not served here; available: {', '.join(self.models)}")
        with self.lock:
            entry = self.loaded.get(name)
            if entry is None:
                while len(self.loaded) >= self.max_loaded:
                    victim = next((n for n, e in self.loaded.items() if e["inflight"] == 0), None)
                    if victim is None:
                        raise RuntimeError(f"cannot load {name!r}: all {self.max_loaded} resident model(s) have requests in "
                                           "flight; retry later or raise --max-loaded-models")
                    self._evict(victim)
                engine = self.loader(self.models[name])
                app = create_app(engine, model_name=name, **self.app_kw)
                entry = {"app": app, "engine": engine, "inflight": 0, "loaded_at": time.time()}
                self.loaded[name] = entry
                self.loads += 1
            self.loaded.move_to_end(name)
            entry["inflight"] += 1
            return entry

    def release(self, entry) -> None:
        with self.lock:
            entry["inflight"] = max(0, entry["inflight"] - 1)

    def _evict(self, name: str) -> None:
        entry = self.loaded.pop(name)
        entry["app"].state.driver.shutdown()
        entry["app"] = entry["engine"] = None
        self.evictions += 1
        try:
            import torch

            if torch.cuda.is_available():
                torch.cuda.empty_cache()
        except Exception:
            pass

    def warmup(self, names=None) -> None:
        for n in (names or [self.default])[: self.max_loaded]:
            self.release(self.acquire(n))

    def shutdown(self) -> None:
        with self.lock:
            for n in list(self.loaded):
                self._evict(n)


class RegistryApp:
    """ASGI application that routes each request to the sub-application of the model it names."""

    def __init__(self, registry: ModelRegistry, enable_admin_endpoints: bool = False):
        self.registry = registry
        self.admin = enable_admin_endpoints

    async def _admin(self, scope, send):
        """GET /v1/admin/models, POST /v1/admin/models/{id}/load | warmup, DELETE /v1/admin/models/{id}."""
        reg, path, method = self.registry, scope["path"], scope["method"]
        parts = [p for p in path.split("/") if p][3:]            # after v1/admin/models
        loop = asyncio.get_running_loop()
        if not parts and method == "GET":
            with reg.lock:
                data = [{"id": n, "path": reg.models[n], "loaded": n in reg.loaded,
                         "inflight": reg.loaded[n]["inflight"] if n in reg.loaded else 0} for n in reg.names()]
            return await self._json(send, 200, {"models": data, "max_loaded": reg.max_loaded, "loads": reg.loads, "evictions": reg.evictions})
        if not parts:
            return await self._json(send, 405, {"error": {"message": "use GET on /v1/admin/models"}})
        name = parts[0]
        if name not in reg.models:
            return await self._json(send, 404, {"error": {"message": f"model {name!r} is not served here; available: {', '.join(reg.models)}"}})
        action = parts[1] if len(parts) > 1 else None
        try:
            if method == "POST" and action in ("load", "warmup"):
                entry = await loop.run_in_executor(None, reg.acquire, name)
                try:
                    if action == "warmup":           # one short generation so kernels, graphs and caches are primed
                        from ..engine.api import GenerateOptions

                        await loop.run_in_executor(None, lambda: entry["engine"].llm.generate([[1, 2, 3]], max_new_tokens=2))
                finally:
                    reg.release(entry)
                return await self._json(send, 200, {"id": name, "loaded": True, "action": action})
            if method == "DELETE" and action is None:
                with reg.lock:
                    entry = reg.loaded.get(name)
                    if entry is None:
                        return await self._json(send, 200, {"id": name, "loaded": False})
                    if entry["inflight"]:
                        return await self._json(send, 409, {"error": {"message": f"model {name!r} has {entry['inflight']} request(s) in flight; retry when idle"}})
                    reg._evict(name)
                return await self._json(send, 200, {"id": name, "loaded": False})
        except RuntimeError as exc:
            return await self._json(send, 503, {"error": {"message": str(exc), "type": "overloaded"}})
        return await self._json(send, 405, {"error": {"message": "use POST .../load, POST .../warmup or DELETE /v1/admin/models/{id}"}})

    async def __call__(self, scope, receive, send):
        if scope["type"] == "lifespan":
            while True:
                msg = await receive()
                if msg["type"] == "lifespan.startup":
                    await send({"type": "lifespan.startup.complete"})
                elif msg["type"] == "lifespan.shutdown":
                    self.registry.shutdown()
                    await send({"type": "lifespan.shutdown.complete"})
                    return
        if scope["type"] != "http":
            return
        path = scope["path"]
        if path == "/health":
            return await self._json(send, 200, {"status": "ok", "loaded": list(self.registry.loaded)})
        if path.startswith("/v1/admin/"):
            if not self.admin:
                return await self._json(send, 404, {"error": {"message": "admin endpoints are disabled; start the server with --enable-admin-endpoints"}})
            if path.startswith("/v1/admin/models"):
                return await self._admin(scope, send)
            return await self._json(send, 404, {"error": {"message": f"no admin route {path}"}})
        if path == "/v1/models" and scope["method"] == "GET":
            return await self._json(send, 200, {"object": "list", "data": [
                {"id": n, "object": "model", "owned_by": "onnx-genai-b200", "loaded": n in self.registry.loaded} for n in self.registry.names()]})
        body = b""
        more = True
        while more:
            msg = await receive()
            if msg["type"] == "http.disconnect":
                return
            body += msg.get("body", b"")
            more = msg.get("more_body", False)
        model = None
        if body:
            try:
                parsed = json.loads(body)
                if isinstance(parsed, dict):
                    model = parsed.get("model")
            except ValueError:
                pass
        if model is None:      # GET routes may name the model in the query string
            for part in scope.get("query_string", b"").decode().split("&"):
                k, _, v = part.partition("=")
                if k == "model" and v:
                    model = v
        try:
            entry = await asyncio.get_running_loop().run_in_executor(None, self.registry.acquire, model)
        except KeyError as exc:
            return await self._json(send, 404, {"error": {"message": str(exc.args[0]), "type": "model_not_found"}})
        except RuntimeError as exc:
            return await self._json(send, 503, {"error": {"message": str(exc), "type": "overloaded"}})
        sent = False

        async def replay():
            nonlocal sent
            if not sent:
                sent = True
                return {"type": "http.request", "body": body, "more_body": False}
            return await receive()

        try:
            await entry["app"](scope, replay, send)
        finally:
            self.registry.release(entry)

    @staticmethod
    async def _json(send, status: int, obj) -> None:
        data = json.dumps(obj).encode()
        await send({"type": "http.response.start", "status": status,
                    "headers": [(b"content-type", b"application/json"), (b"content-length", str(len(data)).encode())]})
        await send({"type": "http.response.body", "body": data})
