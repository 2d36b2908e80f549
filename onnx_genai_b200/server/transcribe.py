"""Audio transcription endpoint: ``POST /v1/audio/transcriptions`` (the OpenAI shape).

The request is a ``multipart/form-data`` body with a ``file`` part (a PCM WAV file) and optional ``model``,
``language`` and ``response_format`` (``json`` or ``text``) parts.  The file is decoded to mono float samples and
handed to a transcriber -- any object with ``sample_rate`` (the rate it wants; the samples are resampled to it) and
``transcribe(samples, language) -> str``.  The reference serves the same route from packages with an audio encoder
(crates/onnx-genai-server/src/routes/multimodal.rs:3-115): same parts, same two response formats, the same refusal
of MP3 uploads.

The multipart body is parsed here (boundary split, part headers, ``name`` / ``filename`` parameters): the form
parser FastAPI would use is a separate package that this environment does not have.
"""
from __future__ import annotations

import asyncio
import re
import struct

import numpy as np
from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, PlainTextResponse

from ..preprocess import resample

MAX_UPLOAD_BYTES = 64 << 20


class MultipartError(ValueError):
    pass


def parse_multipart(content_type: str, body: bytes) -> dict:
    """``multipart/form-data`` -> ``{name: {"filename": str | None, "content_type": str | None, "data": bytes}}``."""
    m = re.search(r'boundary="?([^";]+)"?', content_type or "", flags=re.I)
    if not (content_type or "").lower().startswith("multipart/form-data") or not m:
        raise MultipartError("the request must be multipart/form-data with a boundary")
    delim = b"--" + m.group(1).encode("latin-1")
    chunks = body.split(delim)
    if len(chunks) < 3 or not chunks[-1].lstrip().startswith(b"--"):
        raise MultipartError("the multipart body does not end with its closing boundary")
    parts: dict = {}
    for chunk in chunks[1:-1]:
        chunk = chunk[2:] if chunk.startswith(b"\r\n") else chunk.lstrip(b"\n")
        head, sep, data = chunk.partition(b"\r\n\r\n")
        if not sep:
            head, sep, data = chunk.partition(b"\n\n")
        if not sep:
            raise MultipartError("a multipart part has no blank line after its headers")
        data = data[:-2] if data.endswith(b"\r\n") else data[:-1] if data.endswith(b"\n") else data
        headers = {}
        for line in head.decode("utf-8", errors="replace").splitlines():
            key, _, value = line.partition(":")
            headers[key.strip().lower()] = value.strip()
        disp = headers.get("content-disposition", "")
        name = re.search(r'\bname="([^"]*)"', disp)
        if not disp.lower().startswith("form-data") or not name:
            raise MultipartError("a multipart part lacks `Content-Disposition: form-data; name=...`")
        filename = re.search(r'\bfilename="([^"]*)"', disp)
        parts[name.group(1)] = {"filename": filename.group(1) if filename else None, "content_type": headers.get("content-type"), "data": data}
    return parts


def read_wav(data: bytes):
    """RIFF/WAVE bytes -> (mono float32 samples in [-1, 1], sample rate).  PCM of 8, 16, 24 or 32 bits and 32-bit float
    are read; channels are averaged."""
    if len(data) < 12 or data[:4] != b"RIFF" or data[8:12] != b"WAVE":
        raise ValueError("not a RIFF/WAVE file")
    pos, fmt, pcm = 12, None, None
    while pos + 8 <= len(data):
        tag, size = data[pos:pos + 4], struct.unpack("<I", data[pos + 4:pos + 8])[0]
        payload = data[pos + 8:pos + 8 + size]
        if tag == b"fmt ":
            if len(payload) < 16:
                raise ValueError("the fmt chunk is shorter than 16 bytes")
            fmt = struct.unpack("<HHIIHH", payload[:16])
            if fmt[0] == 0xFFFE and len(payload) >= 26:                          # extensible: the real code sits in the sub-format
                fmt = (struct.unpack("<H", payload[24:26])[0],) + fmt[1:]
        elif tag == b"data":
            pcm = payload
        pos += 8 + size + (size & 1)
    if fmt is None or pcm is None:
        raise ValueError("the file lacks a fmt or a data chunk")
    code, channels, rate, _, _, bits = fmt
    if channels < 1 or rate < 1:
        raise ValueError(f"{channels} channels at {rate} Hz is not audio")
    if code == 1 and bits == 16:
        x = np.frombuffer(pcm[: len(pcm) // 2 * 2], dtype="<i2").astype(np.float32) / 32768.0
    elif code == 1 and bits == 8:
        x = (np.frombuffer(pcm, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
    elif code == 1 and bits == 24:
        b = np.frombuffer(pcm[: len(pcm) // 3 * 3], dtype=np.uint8).reshape(-1, 3).astype(np.int32)
        v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
        x = np.where(v >= 1 << 23, v - (1 << 24), v).astype(np.float32) / float(1 << 23)
    elif code == 1 and bits == 32:
        x = np.frombuffer(pcm[: len(pcm) // 4 * 4], dtype="<i4").astype(np.float32) / float(1 << 31)
    elif code == 3 and bits == 32:
        x = np.frombuffer(pcm[: len(pcm) // 4 * 4], dtype="<f4").astype(np.float32)
    else:
        raise ValueError(f"WAV format code {code} with {bits} bits per sample is not read (PCM 8/16/24/32 and float 32 are)")
    frames = len(x) // channels
    return x[: frames * channels].reshape(frames, channels).mean(axis=1).astype(np.float32), int(rate)


def add_transcription_routes(app: FastAPI, transcriber, model_name: str = "speech-model") -> None:
    @app.post("/v1/audio/transcriptions")
    async def audio_transcriptions(request: Request):
        declared = request.headers.get("content-length")
        if declared and declared.isdigit() and int(declared) > MAX_UPLOAD_BYTES:
            raise HTTPException(413, f"the upload is larger than {MAX_UPLOAD_BYTES >> 20} MiB")
        body = await request.body()
        if len(body) > MAX_UPLOAD_BYTES:
            raise HTTPException(413, f"the upload is larger than {MAX_UPLOAD_BYTES >> 20} MiB")
        try:
            parts = parse_multipart(request.headers.get("content-type", ""), body)
        except MultipartError as e:
            raise HTTPException(400, f"invalid multipart form: {e}")
        if "file" not in parts:
            raise HTTPException(400, "multipart field 'file' is required")
        text_of = lambda key, default: parts[key]["data"].decode("utf-8", errors="replace").strip() if key in parts else default
        fmt = text_of("response_format", "json")
        if fmt not in ("json", "text"):
            raise HTTPException(400, f"unsupported response_format '{fmt}'; expected 'json' or 'text'")
        wanted = text_of("model", "")
        if wanted and wanted != model_name:
            raise HTTPException(404, f"model '{wanted}' is not served here; this server hosts '{model_name}'")
        if (parts["file"]["filename"] or "").lower().endswith(".mp3"):
            raise HTTPException(400, "MP3 audio is not supported yet; provide a PCM WAV file")
        try:
            samples, rate = read_wav(parts["file"]["data"])
        except ValueError as e:
            raise HTTPException(400, f"invalid audio input: {e}")
        if len(samples) == 0:
            raise HTTPException(400, "invalid audio input: the file holds no samples")
        want_rate = int(getattr(transcriber, "sample_rate", rate) or rate)
        language = text_of("language", None) or None

        def work():
            x = resample(samples, rate, want_rate) if rate != want_rate else samples
            return str(transcriber.transcribe(np.asarray(x, dtype=np.float32), language))

        text = await asyncio.get_running_loop().run_in_executor(None, work)
        return JSONResponse({"text": text}) if fmt == "json" else PlainTextResponse(text)


class WorkflowTranscriber:
    """A speech-to-text workflow package behind the route: the workflow input that takes the waveform (role ``audio`` /
    ``waveform``, or a float input with one of those words in its name) gets ``[1, samples]`` mono floats at the rate
    the package's ``serving.audio.sample_rate`` declares (16 kHz when silent); the token-typed output is decoded with
    the package tokenizer."""

    def __init__(self, package_dir: str, device: str = "cpu"):
        import os
        import threading

        from ..engine.workflow_runtime import WorkflowRuntimeError, WorkflowSession

        self.session = WorkflowSession.from_package(package_dir, device=device)
        self.lock = threading.Lock()
        wf = self.session.wf
        words = ("waveform", "audio")
        self.audio_in = next((n for n, s in wf.inputs.items() if s["role"] in words + ("input_audio",)), None) or next(
            (n for n, s in wf.inputs.items() if s["contract"].dtype.startswith("float") and any(w in n for w in words)), None)
        self.tokens_out = next((n for n, c in wf.outputs.items() if c.dtype.startswith("int")), None)
        if self.audio_in is None or self.tokens_out is None:
            raise WorkflowRuntimeError(f"{package_dir} does not look like a speech-to-text package: it needs a waveform input and a token "
                                       f"output (inputs: {list(wf.inputs)}, outputs: {list(wf.outputs)})")
        self.sample_rate = int(((wf.serving or {}).get("audio") or {}).get("sample_rate") or 16000)
        tok_path = os.path.join(package_dir, "tokenizer.json")
        if not os.path.exists(tok_path):
            raise WorkflowRuntimeError(f"{package_dir} has no tokenizer.json, so tokens cannot become text")
        from tokenizers import Tokenizer

        self.tokenizer = Tokenizer.from_file(tok_path)

    def transcribe(self, samples, language=None) -> str:
        import torch

        with self.lock:
            out = self.session.run({self.audio_in: np.asarray(samples, dtype=np.float32)[None]})
        toks = out[self.tokens_out]
        flat: list = []
        for item in (toks if isinstance(toks, list) else [toks]):
            flat += [int(v) for v in torch.as_tensor(item).reshape(-1).tolist()]
        return self.tokenizer.decode(flat, skip_special_tokens=True).strip()
