"""Speech synthesis route over a text-to-speech workflow package; text assembly; WAV writing."""
import os
import struct

import numpy as np
import pytest
from fastapi.testclient import TestClient

from onnx_genai_b200.preprocess import read_wav, write_wav
from onnx_genai_b200.server.audio import assemble_text

REF = os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))
PKG = os.path.join(REF, "tests", "fixtures", "onnx_genai_workflows", "speech_wav")


def test_wav_round_trip_and_channel_interleaving():
    t = np.linspace(0, 1, 480, endpoint=False, dtype=np.float32)
    stereo = np.stack([np.sin(2 * np.pi * 5 * t) * 0.5, np.full_like(t, 0.25)])
    data = write_wav(stereo, 24000)
    assert data[:4] == b"RIFF" and struct.unpack("<HHI", data[20:28]) == (1, 2, 24000) and len(data) == 44 + 480 * 2 * 2
    frames = np.frombuffer(data[44:], dtype="<i2").reshape(-1, 2)
    assert abs(frames[7, 1] / 32767 - 0.25) < 1e-4 and abs(frames[24, 0] / 32767 - stereo[0, 24]) < 1e-4
    mono, rate = read_wav(data)                                   # the reader folds channels to mono
    assert rate == 24000 and np.allclose(mono, stereo.mean(0), atol=1e-4)
    assert len(write_wav(np.array([2.0, -2.0]), 8000)) == 48      # clipped, mono


def test_text_assembly_segments_transforms_and_separators():
    spec = {"segments": [{"field": "instructions", "transforms": [{"kind": "strip_markdown"}, {"kind": "collapse_newlines"}]},
                         {"literal": " "}, {"field": "input", "transforms": [{"kind": "collapse_newlines"}]}]}
    out = assemble_text(spec, {"instructions": "# Calm\n\nSpeak **slowly**, see [notes](http://x)", "input": "Hello\nworld"})
    assert out == "Calm Speak slowly, see notes Hello world"
    assert assemble_text(spec, {"input": "Hello"}) == "Hello"      # no stray separator without instructions
    with pytest.raises(ValueError, match="unknown transform 'shout'"):
        assemble_text({"segments": [{"field": "input", "transforms": [{"kind": "shout"}]}]}, {"input": "x"})


@pytest.mark.skipif(not os.path.exists(os.path.join(PKG, "inference_metadata.yaml")), reason="the upstream speech fixture is not available")
def test_speech_route_returns_wav_at_the_declared_rate():
    from onnx_genai_b200.server.audio import create_speech_app

    with TestClient(create_speech_app(PKG)) as c:
        pipe = c.app.state.pipeline
        assert (pipe.rate, pipe.source_rate) == (24000, 48000) and pipe.max_tokens == 256
        r = c.post("/v1/audio/speech", json={"model": "voice", "input": "hello there", "instructions": "**warm**"})
        assert r.status_code == 200 and r.headers["content-type"] == "audio/wav"
        channels, rate = struct.unpack("<HI", r.content[22:28])
        assert (channels, rate) == (2, 24000)
        n = (len(r.content) - 44) // 4
        assert n == 32                                               # 64 samples at 48 kHz -> 32 at 24 kHz
        pcm = c.post("/v1/audio/speech", json={"input": "hello there", "instructions": "**warm**", "response_format": "pcm"})
        assert pcm.content == r.content[44:] and pcm.headers["x-sample-rate"] == "24000"
        assert c.post("/v1/audio/speech", json={"input": " "}).status_code == 400
        assert c.post("/v1/audio/speech", json={"input": "x", "response_format": "mp3"}).status_code == 400
        assert c.post("/v1/audio/speech", json={"input": "word " * 400}).status_code == 400


@pytest.mark.skipif(not os.path.exists(os.path.join(PKG, "inference_metadata.yaml")), reason="the upstream speech fixture is not available")
def test_serve_mounts_media_packages_without_a_text_model(monkeypatch):
    import uvicorn

    from onnx_genai_b200 import cli

    captured = {}
    monkeypatch.setattr(uvicorn, "run", lambda app, **kw: captured.update(app=app))
    image_pkg = os.path.join(REF, "tests", "fixtures", "comfyui_workflows", "txt2img_sd15")
    assert cli.main(["serve", "--speech-package", PKG, "--image-package", image_pkg, "--device", "cpu", "--addr", "127.0.0.1:0"]) == 0
    with TestClient(captured["app"]) as c:
        assert c.get("/health").json() == {"status": "ok"}
        assert c.post("/v1/audio/speech", json={"input": "hi"}).status_code == 200
        assert c.post("/v1/images/generations", json={"prompt": "fox", "seed": 1}).status_code == 200
