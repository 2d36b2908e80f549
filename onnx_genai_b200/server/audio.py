"""Speech synthesis endpoint over a text-to-speech workflow package: ``POST /v1/audio/speech``.

The request's ``input`` (and optional ``instructions``) are assembled into one string by the package's text-assembly
specification (ordered segments: request fields with clean-up transforms, and literals), tokenized, and run through the
package's workflow (prompt tokens in, waveform out).  The waveform is resampled from the model's rate to the delivery
rate the metadata declares and returned as a WAV file (16-bit PCM) or raw PCM.  The reference serves the same route
from its speech packages (crates/onnx-genai-server/src/lib.rs ``/v1/audio/speech``; the ``onnx-genai.text-assembly``
adapter and the ``media`` block of the audio output in the inference metadata).
"""
from __future__ import annotations

import asyncio
import json
import os
import re
import threading

import numpy as np
import yaml
from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import Response

from ..engine.workflow_runtime import WorkflowRuntimeError, WorkflowSession
from ..preprocess import resample, write_wav


def _strip_markdown(text: str) -> str:
    text = re.sub(r"```.*?```", " ", text, flags=re.S)                       # fenced code is not read aloud
    text = re.sub(r"!?\[([^\]]*)\]\([^)]*\)", r"\1", text)                   # links and images keep their label
    text = re.sub(r"^\s{0,3}(#{1,6}|>|[-*+]|\d+\.)\s+", "", text, flags=re.M)  # headings, quotes, list markers
    return re.sub(r"[*_`~]+", "", text)


TRANSFORMS = {"strip_markdown": _strip_markdown, "collapse_newlines": lambda t: re.sub(r"\s*\n+\s*", " ", t).strip(),
              "trim": str.strip, "lowercase": str.lower}


def assemble_text(spec: dict, fields: dict) -> str:
    """Concatenate the specification's segments: ``{"field": name, "transforms": [...]}`` or ``{"literal": text}``.  A literal
    between two fields is dropped when the field before it is empty, so an absent ``instructions`` leaves no stray separator."""
    parts, last_empty = [], True
    for seg in spec.get("segments") or []:
        if "literal" in seg:
            if not last_empty:
                parts.append(str(seg["literal"]))
            continue
        text = str(fields.get(seg.get("field"), "") or "")
        for tr in seg.get("transforms") or []:
            fn = TRANSFORMS.get(tr.get("kind"))
            if fn is None:
                raise ValueError(f"text assembly: unknown transform {tr.get('kind')!r}; known: {', '.join(sorted(TRANSFORMS))}")
            text = fn(text)
        last_empty = not text
        if text:
            parts.append(text)
    while parts and not parts[-1].strip():
        parts.pop()
    return "".join(parts)


class SpeechPipeline:
    def __init__(self, package_dir: str, device: str = "cpu"):
        self.session = WorkflowSession.from_package(package_dir, device=device)
        self.lock = threading.Lock()
        with open(os.path.join(package_dir, "inference_metadata.yaml"), encoding="utf-8") as f:
            doc = yaml.safe_load(f)
        wf_doc = doc["pipeline"]["workflow"]
        wf = self.session.wf
        self.prompt_in = next((n for n, s in wf.inputs.items() if s["role"] == "prompt_tokens" or n.endswith(("prompt_tokens", "input_ids"))), None)
        audio = [(n, o) for n, o in (wf_doc.get("outputs") or {}).items() if o.get("role") == "audio" or n in ("audio", "waveform")]
        if self.prompt_in is None or not audio:
            raise WorkflowRuntimeError(f"{package_dir} does not look like a speech package: it needs a prompt-token input and an audio output")
        self.audio_out, out_doc = audio[0]
        media = out_doc.get("media") or {}
        self.rate = int(media.get("sample_rate_hz", 24000))
        self.source_rate = int(media.get("source_sample_rate_hz", self.rate))
        self.assembly = {"segments": [{"field": "input"}]}
        self.max_tokens = None
        for comp in (wf_doc.get("components") or {}).values():
            impl = comp.get("implementation") or {}
            if impl.get("abi") == "onnx-genai.text-assembly" and impl.get("artifact"):
                with open(os.path.join(package_dir, impl["artifact"]), encoding="utf-8") as f:
                    self.assembly = json.load(f)
                self.max_tokens = self.assembly.get("max_input_tokens")
        tok_path = os.path.join(package_dir, "tokenizer.json")
        if not os.path.exists(tok_path):
            raise WorkflowRuntimeError(f"{package_dir} has no tokenizer.json, so text cannot become prompt tokens")
        from tokenizers import Tokenizer

        self.tokenizer = Tokenizer.from_file(tok_path)

    def synthesize(self, text: str, instructions: str = "") -> np.ndarray:
        """[channels, samples] float32 at the delivery rate."""
        prompt = assemble_text(self.assembly, {"input": text, "instructions": instructions})
        ids = self.tokenizer.encode(prompt).ids or [0]
        if self.max_tokens and len(ids) > int(self.max_tokens):
            raise HTTPException(400, f"the input is {len(ids)} tokens after assembly; this voice model takes at most {self.max_tokens}")
        with self.lock:
            out = self.session.run({self.prompt_in: np.asarray([ids], dtype=np.int64)})
        wave = out[self.audio_out]
        wave = wave[-1] if isinstance(wave, list) else wave
        wave = np.asarray(wave.detach().cpu() if hasattr(wave, "detach") else wave, dtype=np.float32)
        wave = wave[0] if wave.ndim == 3 else wave                                  # first (only) request row
        wave = wave[None] if wave.ndim == 1 else wave
        if self.source_rate != self.rate:
            wave = np.stack([resample(ch, self.source_rate, self.rate) for ch in wave])
        return wave


def add_speech_routes(app: FastAPI, pipeline: SpeechPipeline) -> None:
    @app.post("/v1/audio/speech")
    async def speech(request: Request):
        try:
            body = await request.json()
        except Exception:
            raise HTTPException(400, "the request body is not valid JSON")
        text = body.get("input") if isinstance(body, dict) else None
        if not isinstance(text, str) or not text.strip():
            raise HTTPException(400, "input must be a non-empty string")
        fmt = body.get("response_format", "wav")
        if fmt not in ("wav", "pcm"):
            raise HTTPException(400, f"response_format {fmt!r} is not available; use wav or pcm (16-bit little-endian)")
        loop = asyncio.get_running_loop()
        try:
            wave = await loop.run_in_executor(None, lambda: pipeline.synthesize(text, str(body.get("instructions") or "")))
        except (WorkflowRuntimeError, ValueError) as e:
            raise HTTPException(500, str(e))
        data = write_wav(wave, pipeline.rate)
        if fmt == "pcm":
            return Response(data[44:], media_type="audio/pcm", headers={"X-Sample-Rate": str(pipeline.rate), "X-Channels": str(wave.shape[0])})
        return Response(data, media_type="audio/wav")


def create_speech_app(package_dir: str, device: str = "cpu") -> FastAPI:
    app = FastAPI(title="onnx-genai-b200 speech")
    app.state.pipeline = SpeechPipeline(package_dir, device)

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    add_speech_routes(app, app.state.pipeline)
    return app
