"""Image generation endpoints over a text-to-image workflow package.

``POST /v1/images/generations`` (OpenAI shape: ``prompt``, ``n``, ``response_format: b64_json``) and
``POST /sdapi/v1/txt2img`` (the A1111 shape many front ends speak: ``prompt``, ``negative_prompt``, ``seed``, ``steps``,
``cfg_scale``, ``batch_size``) run the package's workflow -- tokenize, text encoder, denoising loop, VAE -- on the
workflow runtime and return PNG images.  ``POST /sdapi/v1/img2img`` adds one base64 ``init_images`` entry and a
``denoising_strength`` for workflows that declare an image input, and ``GET /sdapi/v1/sd-models | samplers | options``
answer the questions A1111 front ends ask before they let a user generate.  The reference serves the same routes from
its workflow packages (crates/onnx-genai-server/src/lib.rs:76-90, routes/images.rs:377-395,985-1027).

The package is found by shape, not by name: the workflow input whose role is ``prompt_tokens`` (or whose name ends in
``input_ids``) takes the prompt, an input with ``negative`` in its name takes the negative prompt, ``seed``,
``guidance_scale`` and ``max_iterations`` inputs take the matching request fields, and the output named ``image`` (or with
role ``image``) is returned.  Requests run one at a time on a worker thread; the event loop stays free.
"""
from __future__ import annotations

import asyncio
import base64
import os
import threading
import time

import numpy as np
from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse

from ..engine.workflow_runtime import WorkflowRuntimeError, WorkflowSession
from ..utils.png import encode_png


class ImagePipeline:
    def __init__(self, package_dir: str, device: str = "cpu"):
        self.session = WorkflowSession.from_package(package_dir, device=device)
        self.lock = threading.Lock()
        tok_path = os.path.join(package_dir, "tokenizer.json")
        self.tokenizer = None
        if os.path.exists(tok_path):
            from tokenizers import Tokenizer

            self.tokenizer = Tokenizer.from_file(tok_path)
        wf = self.session.wf
        names = list(wf.inputs)

        def find(pred):
            return next((n for n in names if pred(n, wf.inputs[n])), None)

        self.negative_in = find(lambda n, s: "negative" in n and s["contract"].dtype.startswith("int"))
        self.prompt_in = find(lambda n, s: n != self.negative_in and (s["role"] == "prompt_tokens" or n.endswith(("input_ids", "positive_ids"))))
        self.seed_in = find(lambda n, s: n.endswith("seed"))
        self.guidance_in = find(lambda n, s: n.endswith("guidance_scale"))
        self.steps_in = find(lambda n, s: n.endswith("max_iterations"))
        self.init_in = find(lambda n, s: s["role"] in ("image", "init_image", "media") or "init_image" in n)
        self.strength_in = find(lambda n, s: n.endswith(("denoising_strength", "strength")))
        self.samplers = list((wf.serving or {}).get("samplers") or ["Euler"])
        self.image_out = "image" if "image" in wf.outputs else next(iter(wf.outputs), None)
        if self.prompt_in is None or self.image_out is None:
            raise WorkflowRuntimeError(f"{package_dir} does not look like a text-to-image package: it needs a prompt-token input and an "
                                       f"image output (inputs: {names}, outputs: {list(wf.outputs)})")
        self.generated = 0

    def _ids(self, text: str) -> list:
        if self.tokenizer is None:
            raise HTTPException(500, "the package has no tokenizer.json, so prompts cannot be tokenized")
        return self.tokenizer.encode(text or "").ids or [0]

    def generate(self, prompt: str, negative: str = "", n: int = 1, seed: int | None = None, steps: int | None = None,
                 guidance: float | None = None, init_image=None, strength: float | None = None) -> list:
        """``n`` images as [C, H, W] float arrays.  ``init_image`` ([3, H, W] floats in 0..255) feeds the workflow's image
        input: as [n, 3, H, W] in 0..1 when that input is a float tensor, as [n, H, W, 3] bytes when it is uint8."""
        pos, neg = self._ids(prompt), self._ids(negative)
        width = max(len(pos), len(neg))
        pad = lambda ids: ids + [0] * (width - len(ids))
        feeds = {self.prompt_in: np.asarray([pad(pos)] * n, dtype=np.int64)}
        if self.negative_in:
            feeds[self.negative_in] = np.asarray([pad(neg)] * n, dtype=np.int64)
        if self.seed_in and seed is not None:
            feeds[self.seed_in] = np.asarray([int(seed) + i for i in range(n)], dtype=np.int64)       # one seed per image
        if self.guidance_in and guidance is not None:
            feeds[self.guidance_in] = np.full((n,), float(guidance), dtype=np.float32)
        if self.steps_in and steps is not None:
            feeds[self.steps_in] = np.asarray([int(steps)], dtype=np.int64)
        if init_image is not None:
            if self.init_in is None:
                raise HTTPException(400, "the loaded workflow declares no image input, so img2img is unavailable")
            img = np.asarray(init_image, dtype=np.float32)
            if self.session.wf.inputs[self.init_in]["contract"].dtype == "uint8":
                feeds[self.init_in] = np.repeat(np.clip(img, 0, 255).astype(np.uint8).transpose(1, 2, 0)[None], n, axis=0)
            else:
                feeds[self.init_in] = np.repeat((img / 255.0)[None], n, axis=0)
            if self.strength_in and strength is not None:
                feeds[self.strength_in] = np.full((n,), float(strength), dtype=np.float32)
        with self.lock:
            out = self.session.run(feeds)
        img = out[self.image_out]
        img = img[-1] if isinstance(img, list) else img
        arr = np.asarray(img.detach().cpu() if hasattr(img, "detach") else img, dtype=np.float32)
        if arr.ndim != 4 or arr.shape[1] not in (1, 3):
            raise HTTPException(500, f"the workflow's image output has shape {list(arr.shape)}; [n, 1 or 3, height, width] is needed")
        self.generated += arr.shape[0]
        return [arr[i] for i in range(arr.shape[0])]


def add_image_routes(app: FastAPI, pipeline: ImagePipeline, model_name: str = "image-model") -> None:
    async def _json(request: Request) -> dict:
        try:
            body = await request.json()
        except Exception:
            raise HTTPException(400, "the request body is not valid JSON")
        if not isinstance(body, dict):
            raise HTTPException(400, "the request body must be a JSON object")
        return body

    async def _run(**kw):
        loop = asyncio.get_running_loop()
        try:
            return await loop.run_in_executor(None, lambda: pipeline.generate(**kw))
        except WorkflowRuntimeError as e:
            raise HTTPException(500, str(e))

    @app.post("/v1/images/generations")
    async def openai_images(request: Request):
        body = await _json(request)
        prompt = body.get("prompt")
        if not isinstance(prompt, str) or not prompt:
            raise HTTPException(400, "prompt must be a non-empty string")
        n = body.get("n", 1)
        if not isinstance(n, int) or isinstance(n, bool) or not 1 <= n <= 8:
            raise HTTPException(400, f"n must be an integer between 1 and 8, not {n!r}")
        if body.get("response_format", "b64_json") != "b64_json":
            raise HTTPException(400, "only response_format 'b64_json' is available: this server does not host image URLs")
        images = await _run(prompt=prompt, negative=str(body.get("negative_prompt") or ""), n=n, seed=body.get("seed"),
                            steps=body.get("steps"), guidance=body.get("guidance_scale"))
        return JSONResponse({"created": int(time.time()), "model": model_name,
                             "data": [{"b64_json": base64.b64encode(encode_png(img)).decode()} for img in images]})

    @app.get("/sdapi/v1/sd-models")
    async def a1111_models():
        return [{"title": model_name, "model_name": model_name, "hash": None, "sha256": None, "filename": model_name, "config": None}]

    @app.get("/sdapi/v1/samplers")
    async def a1111_samplers():
        return [{"name": name, "aliases": [], "options": {}} for name in pipeline.samplers]

    @app.get("/sdapi/v1/options")
    async def a1111_options():
        return {"sd_model_checkpoint": model_name, "samples_format": "png", "save_images": False,
                "sampler_name": pipeline.samplers[0] if pipeline.samplers else None}

    @app.post("/sdapi/v1/txt2img")
    async def a1111_txt2img(request: Request):
        return await _a1111(await _json(request), img2img=False)

    @app.post("/sdapi/v1/img2img")
    async def a1111_img2img(request: Request):
        return await _a1111(await _json(request), img2img=True)

    async def _a1111(body: dict, img2img: bool):
        extra = {}
        if img2img:
            if pipeline.init_in is None:
                raise HTTPException(400, "the loaded workflow declares no image input, so img2img is unavailable")
            inits = body.get("init_images")
            if not isinstance(inits, list) or len(inits) != 1 or not isinstance(inits[0], str):
                raise HTTPException(400, "img2img requires exactly one base64 entry in `init_images`")
            text = inits[0].split(",", 1)[1] if inits[0].startswith("data:") else inits[0]
            try:
                from ..preprocess import PreprocessError, decode_rgb

                extra["init_image"] = decode_rgb(base64.b64decode(text, validate=True)).numpy()
            except (ValueError, PreprocessError) as e:
                raise HTTPException(400, f"`init_images[0]` is not a base64-encoded image: {e}")
            strength = body.get("denoising_strength", 0.75)
            if not isinstance(strength, (int, float)) or isinstance(strength, bool) or not 0.0 <= float(strength) <= 1.0:
                raise HTTPException(400, f"denoising_strength must lie in 0..1, not {strength!r}")
            extra["strength"] = float(strength)
        sampler = body.get("sampler_name")
        if sampler is not None and sampler not in pipeline.samplers:
            raise HTTPException(400, f"sampler {sampler!r} is not one of {pipeline.samplers}")
        n = int(body.get("batch_size", 1) or 1) * int(body.get("n_iter", 1) or 1)
        if not 1 <= n <= 8:
            raise HTTPException(400, f"batch_size x n_iter must be between 1 and 8, got {n}")
        seed = body.get("seed", -1)
        seed = int(time.time_ns() % (1 << 31)) if seed in (None, -1) else int(seed)
        images = await _run(prompt=str(body.get("prompt") or ""), negative=str(body.get("negative_prompt") or ""), n=n, seed=seed,
                            steps=body.get("steps"), guidance=body.get("cfg_scale"), **extra)
        params = {k: body.get(k) for k in ("prompt", "negative_prompt", "steps", "cfg_scale", "width", "height", "sampler_name")}
        if img2img:
            params["denoising_strength"] = extra["strength"]
        return JSONResponse({"images": [base64.b64encode(encode_png(img)).decode() for img in images],
                             "parameters": {**params, "seed": seed, "batch_size": n},
                             "info": f'{{"seed": {seed}, "all_seeds": {[seed + i for i in range(n)]}}}'})


def create_image_app(package_dir: str, model_name: str | None = None, device: str = "cpu") -> FastAPI:
    pipeline = ImagePipeline(package_dir, device)
    name = model_name or os.path.basename(os.path.abspath(package_dir))
    app = FastAPI(title="onnx-genai-b200 images")
    app.state.pipeline = pipeline

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": name, "object": "model", "owned_by": "local", "capabilities": ["image_generation"]}]}

    add_image_routes(app, pipeline, name)
    return app
