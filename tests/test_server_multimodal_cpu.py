"""Chat requests that carry an image or an audio clip: content-part parsing, the one-attachment admission rule, routing
to a mounted media chat, and the upstream vision-language workflow package behind the route."""
import base64
import io
import json
import os

import numpy as np
import pytest
import torch
from fastapi.testclient import TestClient

from onnx_genai_b200.engine.api import Engine
from onnx_genai_b200.models.config import DecoderConfig
from onnx_genai_b200.models.decoder import random_weights
from onnx_genai_b200.package.export import export_package
from onnx_genai_b200.server import create_app
from onnx_genai_b200.server import multimodal as mm

CFG = DecoderConfig(name="t", num_layers=1, hidden=32, num_heads=2, num_kv_heads=1, head_dim=16, intermediate=64, vocab=300,
                    rope_theta=1e4, tie_embeddings=True, max_position=256)
FIXTURES = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference", "tests", "fixtures",
                        "onnx_genai_workflows")


class EchoMediaChat:
    """Accepts images only; answers with token ids that encode what it was given."""
    accepts = {"image": True, "audio": False}

    def __init__(self):
        self.calls = []

    def generate(self, prompt_ids, image=None, audio=None, max_new_tokens=64):
        self.calls.append((len(prompt_ids), None if image is None else len(image), audio, max_new_tokens))
        return [65, 66, 67][:max_new_tokens]


@pytest.fixture(scope="module")
def engine(tmp_path_factory):
    w = random_weights(CFG, "cpu", seed=5, std=0.3, dtype=torch.float32)
    d = export_package(CFG, w, str(tmp_path_factory.mktemp("pkg")))
    return Engine.from_dir(d, device="cpu", num_pages=64, max_seqs=4, max_tokens_per_step=64)


def _png(n=8):
    from PIL import Image

    buf = io.BytesIO()
    Image.fromarray((np.random.default_rng(0).random((n, n, 3)) * 255).astype(np.uint8)).save(buf, format="PNG")
    return buf.getvalue()


def _img_part(raw):
    return {"type": "image_url", "image_url": {"url": "data:image/png;base64," + base64.b64encode(raw).decode()}}


def test_content_parts_are_split_and_validated():
    raw = _png()
    msgs = [{"role": "user", "content": [{"type": "text", "text": "what is "}, _img_part(raw), {"type": "text", "text": "this?"}]}]
    norm, images, audio = mm.split_content(msgs)
    assert norm == [{"role": "user", "content": "what is this?"}] and images == [raw] and audio == []
    wav = base64.b64encode(b"RIFFxxxxWAVE").decode()
    _, _, audio = mm.split_content([{"role": "user", "content": [{"type": "input_audio", "input_audio": {"data": wav, "format": "wav"}}]}])
    assert audio == [b"RIFFxxxxWAVE"]
    for bad, why in (({"type": "image_url", "image_url": {"url": "https://example.com/a.png"}}, "not fetched"),
                     ({"type": "image_url", "image_url": {"url": "data:image/png,rawbytes"}}, "base64 encoded"),
                     ({"type": "image_url", "image_url": {"url": "data:image/png;base64,@@@"}}, "not valid base64"),
                     ({"type": "input_audio", "input_audio": {"data": wav, "format": "mp3"}}, "not supported"),
                     ({"type": "video", "video": {}}, "not supported")):
        with pytest.raises(mm.MediaError, match=why):
            mm.split_content([{"role": "user", "content": [bad]}])


def test_admission_follows_the_one_attachment_rule():
    chat = EchoMediaChat()
    mm.admit_attachments(chat, "m", 1, 0)
    for images, audio, why in ((2, 0, "one encoded media tensor"), (1, 1, "one media attachment"), (0, 2, "one media attachment"),
                               (0, 1, "no typed audio media input")):
        with pytest.raises(mm.MediaError, match=why):
            mm.admit_attachments(chat, "m", images, audio)
    with pytest.raises(mm.MediaError, match="no typed image media input"):
        mm.admit_attachments(None, "m", 1, 0)


def test_chat_with_an_image_runs_on_the_media_chat(engine):
    chat = EchoMediaChat()
    raw = _png()
    body = {"messages": [{"role": "user", "content": [{"type": "text", "text": "describe"}, _img_part(raw)]}], "max_tokens": 2}
    with TestClient(create_app(engine, model_name="tiny", media_chat=chat)) as c:
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        out = r.json()
        assert out["choices"][0]["message"]["content"] == engine.detokenize([65, 66]) and out["usage"]["completion_tokens"] == 2
        assert chat.calls[-1][1] == len(raw) and chat.calls[-1][3] == 2
        with c.stream("POST", "/v1/chat/completions", json={**body, "stream": True}) as s:
            lines = [l for l in s.iter_lines() if l.startswith("data: ")]
        assert lines[-1] == "data: [DONE]" and json.loads(lines[1][6:])["choices"][0]["delta"]["content"] == engine.detokenize([65, 66])
        # audio on an image-only package, and two images, are refused with the reason
        wav = base64.b64encode(b"RIFF0000WAVE").decode()
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [
            {"type": "input_audio", "input_audio": {"data": wav, "format": "wav"}}]}]})
        assert r.status_code == 422 and "no typed audio media input" in r.text
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [_img_part(raw), _img_part(raw)]}]})
        assert r.status_code == 400 and "one encoded media tensor" in r.text
    # a text-only server says so
    with TestClient(create_app(engine, model_name="tiny")) as c:
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 422 and "declares no typed image media input" in r.text
        ok = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}], "max_tokens": 2})
        assert ok.status_code == 200


@pytest.mark.skipif(not os.path.isdir(os.path.join(FIXTURES, "vlm")), reason="the upstream workflow fixtures are not available on this machine")
def test_upstream_vision_language_package_answers_a_chat_request(engine):
    chat = mm.WorkflowMediaChat(os.path.join(FIXTURES, "vlm"))
    assert chat.accepts == {"image": True, "audio": False}
    with TestClient(create_app(engine, model_name="vlm", media_chat=chat)) as c:
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [{"type": "text", "text": "x"}, _img_part(_png())]}],
                                                   "max_tokens": 3})
        assert r.status_code == 200, r.text
        assert r.json()["usage"]["completion_tokens"] >= 1
        assert chat.session.stats["invocations"]["vision_encoder"] >= 1
        bad = {"type": "image_url", "image_url": {"url": "data:image/png;base64," + base64.b64encode(b"0123456789").decode()}}
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [bad]}], "max_tokens": 3})
        assert r.status_code == 422 and "could not be processed" in r.text
