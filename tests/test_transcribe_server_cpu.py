"""The transcription route: multipart parsing, WAV decoding, validation, response formats."""
import struct

import numpy as np
import pytest
from fastapi import FastAPI
from fastapi.testclient import TestClient

from onnx_genai_b200.preprocess import write_wav
from onnx_genai_b200.server.transcribe import MultipartError, add_transcription_routes, parse_multipart, read_wav


def _form(fields: dict, boundary="XbOuNdArY"):
    body = b""
    for name, value in fields.items():
        if isinstance(value, tuple):
            filename, data = value
            body += f'--{boundary}\r\nContent-Disposition: form-data; name="{name}"; filename="{filename}"\r\nContent-Type: audio/wav\r\n\r\n'.encode() + data + b"\r\n"
        else:
            body += f'--{boundary}\r\nContent-Disposition: form-data; name="{name}"\r\n\r\n{value}\r\n'.encode()
    return body + f"--{boundary}--\r\n".encode(), {"content-type": f"multipart/form-data; boundary={boundary}"}


def test_multipart_parts_keep_binary_payloads_intact():
    payload = bytes(range(256)) + b"\r\n--XbOuNdArZ\r\n"                             # line ends and a near-boundary inside the data
    body, headers = _form({"file": ("a.wav", payload), "language": "de"})
    parts = parse_multipart(headers["content-type"], body)
    assert parts["file"]["data"] == payload and parts["file"]["filename"] == "a.wav" and parts["file"]["content_type"] == "audio/wav"
    assert parts["language"]["data"] == b"de" and parts["language"]["filename"] is None
    with pytest.raises(MultipartError, match="boundary"):
        parse_multipart("application/json", body)
    with pytest.raises(MultipartError, match="closing boundary"):
        parse_multipart(headers["content-type"], body[:-12])


def test_wav_decoding_of_the_usual_sample_formats():
    t = np.arange(800) / 8000.0
    tone = 0.5 * np.sin(2 * np.pi * 440 * t).astype(np.float32)
    x, rate = read_wav(write_wav(tone, 8000))
    assert rate == 8000 and np.allclose(x, tone, atol=1e-4)
    stereo, _ = read_wav(write_wav(np.stack([tone, -tone]), 8000))
    assert len(stereo) == 800 and float(np.abs(stereo).max()) < 1e-4                   # the channels cancel in the mono mix

    def wav(code, bits, frames: bytes, channels=1, rate=16000, extra=b""):
        fmt = struct.pack("<HHIIHH", code, channels, rate, rate * channels * bits // 8, channels * bits // 8, bits)
        chunks = b"fmt " + struct.pack("<I", len(fmt)) + fmt + extra + b"data" + struct.pack("<I", len(frames)) + frames
        return b"RIFF" + struct.pack("<I", 4 + len(chunks)) + b"WAVE" + chunks

    f32, _ = read_wav(wav(3, 32, tone.astype("<f4").tobytes()))
    assert np.array_equal(f32, tone)
    u8, _ = read_wav(wav(1, 8, bytes([0, 128, 255])))
    assert np.allclose(u8, [-1.0, 0.0, 127 / 128])
    i24, _ = read_wav(wav(1, 24, bytes([0, 0, 0x40, 0, 0, 0xC0])))
    assert np.allclose(i24, [0.5, -0.5])
    skipped, _ = read_wav(wav(1, 16, struct.pack("<hh", 16384, -16384), extra=b"LIST" + struct.pack("<I", 3) + b"abc\x00"))   # an odd-sized chunk is padded
    assert np.allclose(skipped, [0.5, -0.5])
    for bad, why in ((b"RIFX" + b"\x00" * 20, "RIFF"), (wav(2, 4, b"\x00" * 8), "format code 2"), (b"RIFF\x04\x00\x00\x00WAVE", "fmt or a data")):
        with pytest.raises(ValueError, match=why):
            read_wav(bad)


class _Loudness:
    """Stands in for a model: reports what it was given."""
    sample_rate = 16000

    def transcribe(self, samples, language):
        return f"{len(samples)} samples, peak {float(np.abs(samples).max()):.2f}, language {language}"


@pytest.fixture()
def client():
    app = FastAPI()
    add_transcription_routes(app, _Loudness(), "ear")
    with TestClient(app) as c:
        yield c


def test_route_resamples_and_answers_in_both_formats(client):
    tone = 0.5 * np.sin(2 * np.pi * 200 * np.arange(8000) / 8000.0)
    body, headers = _form({"file": ("clip.wav", write_wav(tone, 8000)), "model": "ear", "language": "en"})
    r = client.post("/v1/audio/transcriptions", content=body, headers=headers)
    assert r.status_code == 200 and r.json() == {"text": "16000 samples, peak 0.50, language en"}          # one second at 8 kHz -> 16 kHz
    body, headers = _form({"file": ("clip.wav", write_wav(tone, 8000)), "response_format": "text"})
    r = client.post("/v1/audio/transcriptions", content=body, headers=headers)
    assert r.status_code == 200 and r.headers["content-type"].startswith("text/plain") and r.text.endswith("language None")


def test_route_refusals(client):
    wav = write_wav(np.zeros(100, dtype=np.float32), 16000)
    cases = [({"language": "en"}, 400, "'file' is required"), ({"file": ("a.wav", wav), "response_format": "srt"}, 400, "unsupported response_format"),
             ({"file": ("a.mp3", wav)}, 400, "MP3"), ({"file": ("a.wav", b"junk")}, 400, "invalid audio input"),
             ({"file": ("a.wav", wav), "model": "other"}, 404, "not served here"),
             ({"file": ("a.wav", write_wav(np.zeros(0, dtype=np.float32), 16000))}, 400, "no samples")]
    for fields, status, why in cases:
        body, headers = _form(fields)
        r = client.post("/v1/audio/transcriptions", content=body, headers=headers)
        assert r.status_code == status and why in r.text, (fields.keys(), r.status_code, r.text)
    assert client.post("/v1/audio/transcriptions", json={"file": "x"}).status_code == 400
