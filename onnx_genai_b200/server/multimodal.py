"""Media attachments of chat requests: ``image_url`` and ``input_audio`` content parts.

The reference admits at most one media attachment per chat request and binds it to the typed media input of a
workflow package (crates/onnx-genai-server/src/multimodal.rs:64-88 ``admit_attachments``, ``MultimodalInput``):
an image arrives as a ``data:`` URL and is handed over as its encoded bytes (the package's own preprocessing
program decodes and sizes it), audio arrives as base64 WAV.  This module does the same for a server whose chat route
has a *media chat* mounted -- any object with

    accepts            -> {"image": bool, "audio": bool}
    generate(prompt_ids, image=None, audio=None, max_new_tokens=...) -> list of token ids

:class:`WorkflowMediaChat` is that object over a workflow package run by the generic workflow runtime (the upstream
vision-language package runs from image bytes this way).  Remote URLs are never fetched.
"""
from __future__ import annotations

import base64
import binascii
import re

import numpy as np

MAX_MEDIA_BYTES = 32 << 20


class MediaError(ValueError):
    """A request problem with an HTTP status: 400 for malformed parts, 422 for a package that cannot take the media."""

    def __init__(self, message: str, status: int = 400):
        super().__init__(message)
        self.status = status


def split_content(messages):
    """Chat messages -> (messages with text-only content, image byte strings, audio byte strings).  Text parts are
    joined in order; every media part is decoded and validated for shape (not for what the model accepts)."""
    images, audio, norm = [], [], []
    for m in messages:
        if not isinstance(m, dict):
            raise MediaError("every message must be an object with role and content")
        content = m.get("content")
        if isinstance(content, list):
            texts = []
            for part in content:
                kind = part.get("type") if isinstance(part, dict) else None
                if kind == "text":
                    texts.append(str(part.get("text", "")))
                elif kind == "image_url":
                    ref = part.get("image_url")
                    url = ref.get("url") if isinstance(ref, dict) else ref
                    images.append(_decode_data_url(url))
                elif kind == "input_audio":
                    ref = part.get("input_audio") or {}
                    fmt = str(ref.get("format", "wav")).lower()
                    if fmt != "wav":
                        raise MediaError(f"input_audio format '{fmt}' is not supported; send PCM WAV (format: \"wav\")")
                    audio.append(_b64(ref.get("data"), "input_audio.data"))
                else:
                    raise MediaError(f"content part of type {kind!r} is not supported (text, image_url and input_audio are)")
            content = "".join(texts)
        norm.append({**m, "content": content or ""})
    return norm, images, audio


def _b64(data, what: str) -> bytes:
    if not isinstance(data, str) or not data:
        raise MediaError(f"{what} must be a base64 string")
    try:
        raw = base64.b64decode(data, validate=True)
    except (binascii.Error, ValueError):
        raise MediaError(f"{what} is not valid base64")
    if len(raw) > MAX_MEDIA_BYTES:
        raise MediaError(f"{what} is larger than {MAX_MEDIA_BYTES >> 20} MiB", 413)
    return raw


def _decode_data_url(url) -> bytes:
    if not isinstance(url, str) or not url:
        raise MediaError("image_url needs a url")
    m = re.match(r"^data:([\w.+-]+/[\w.+-]+)?((?:;[\w=.+-]+)*),(.*)$", url, flags=re.S)
    if not m:
        raise MediaError("image_url must be a data: URL with the encoded image (remote URLs are not fetched by this server)")
    if ";base64" not in (m.group(2) or ""):
        raise MediaError("image_url data: URLs must be base64 encoded")
    return _b64(m.group(3), "image_url")


def admit_attachments(media_chat, model: str, images: int, audio: int) -> None:
    """The reference's admission rule: one media attachment per request, and only of a kind the package declares."""
    if images > 1:
        raise MediaError(f"workflow package '{model}' accepts one encoded media tensor per request; bind a multi-image application "
                         "tensor explicitly when the package declares one")
    if audio > 1 or (images > 0 and audio > 0):
        raise MediaError(f"workflow package '{model}' accepts one media attachment per request")
    accepts = getattr(media_chat, "accepts", {}) if media_chat is not None else {}
    if images > 0 and not accepts.get("image"):
        raise MediaError(f"workflow package '{model}' declares no typed image media input", 422)
    if audio > 0 and not accepts.get("audio"):
        raise MediaError(f"workflow package '{model}' declares no typed audio media input", 422)


class WorkflowMediaChat:
    """A workflow package with a typed media input (encoded bytes, role ``media``) and a prompt-token input, behind the
    chat route.  The media input is classed as image or audio by its name; the token-typed output is the answer."""

    def __init__(self, package_dir: str, device: str = "cpu"):
        import threading

        from ..engine.workflow_runtime import WorkflowRuntimeError, WorkflowSession

        self.session = WorkflowSession.from_package(package_dir, device=device)
        self.lock = threading.Lock()
        wf = self.session.wf
        self.prompt_in = next((n for n, s in wf.inputs.items() if s["role"] == "prompt_tokens"), None)
        self.max_in = next((n for n, s in wf.inputs.items() if s["role"] == "max_output_tokens"), None)
        media = [n for n, s in wf.inputs.items() if s["role"] in ("media", "image", "audio", "input_audio")
                 or (s["contract"].dtype == "uint8" and s["contract"].rank == 1)]
        self.image_in = next((n for n in media if "image" in n or "pixel" in n or "vision" in n), None)
        self.audio_in = next((n for n in media if "audio" in n or "wav" in n or "speech" in n), None)
        self.tokens_out = next((n for n, c in wf.outputs.items() if c.dtype.startswith("int")), None)
        if self.prompt_in is None or self.tokens_out is None or not (self.image_in or self.audio_in):
            raise WorkflowRuntimeError(f"{package_dir} is not a media chat package: it needs a prompt-token input, a typed media input "
                                       f"and a token output (inputs: {list(wf.inputs)}, outputs: {list(wf.outputs)})")

    @property
    def accepts(self) -> dict:
        return {"image": self.image_in is not None, "audio": self.audio_in is not None}

    def generate(self, prompt_ids, image: bytes | None = None, audio: bytes | None = None, max_new_tokens: int = 64):
        import torch

        feeds = {self.prompt_in: torch.tensor([list(prompt_ids)], dtype=torch.int64)}
        if self.max_in is not None:
            feeds[self.max_in] = torch.tensor([int(max_new_tokens)], dtype=torch.int64)
        if image is not None:
            feeds[self.image_in] = torch.from_numpy(np.frombuffer(image, dtype=np.uint8).copy())
        if audio is not None:
            feeds[self.audio_in] = torch.from_numpy(np.frombuffer(audio, dtype=np.uint8).copy())
        for name, spec in self.session.wf.inputs.items():      # other request inputs without a default: neutral values
            if name not in feeds and spec["source"] in ("request", "application") and spec.get("default") is None:
                c = spec["contract"]
                shape = [s if isinstance(s, int) else 1 for s in c.shape] or [1]
                feeds[name] = torch.zeros(shape) if c.dtype.startswith("float") else torch.ones(shape, dtype=torch.int64)
        with self.lock:
            out = self.session.run(feeds)
        toks = out[self.tokens_out]
        flat: list = []
        for item in (toks if isinstance(toks, list) else [toks]):
            row = torch.as_tensor(item)
            flat += [int(v) for v in (row[0] if row.dim() > 1 else row).reshape(-1).tolist()]
        return flat
