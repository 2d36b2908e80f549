"""Image generation routes over a text-to-image workflow package."""
import base64
import json
import os
import struct
import zlib

import numpy as np
import pytest
from fastapi.testclient import TestClient

from onnx_genai_b200.server.images import create_image_app

REF = os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))
PKG = os.path.join(REF, "tests", "fixtures", "comfyui_workflows", "txt2img_sd15")
pytestmark = pytest.mark.skipif(not os.path.exists(os.path.join(PKG, "reference.json")), reason="the upstream text-to-image fixture is not available")


def _decode_png(b64: str):
    png = base64.b64decode(b64)
    assert png[:8] == b"\x89PNG\r\n\x1a\n"
    w, h = struct.unpack(">II", png[16:24])
    raw = zlib.decompress(png[png.index(b"IDAT") + 4: png.index(b"IEND") - 8])
    rows = np.frombuffer(raw, dtype=np.uint8).reshape(h, 1 + 3 * w)
    assert not rows[:, 0].any()
    return rows[:, 1:].reshape(h, w, 3)


@pytest.fixture(scope="module")
def client():
    with TestClient(create_image_app(PKG, model_name="sd-tiny")) as c:
        yield c


def test_openai_route_returns_seeded_pngs(client):
    assert client.get("/v1/models").json()["data"][0]["id"] == "sd-tiny"
    body = {"model": "sd-tiny", "prompt": "a photograph of a red fox in snow", "n": 2, "seed": 7}
    r = client.post("/v1/images/generations", json=body)
    assert r.status_code == 200, r.text
    imgs = [_decode_png(d["b64_json"]) for d in r.json()["data"]]
    assert len(imgs) == 2 and imgs[0].shape == (4, 4, 3) and not np.array_equal(imgs[0], imgs[1])       # one seed per image
    again = [_decode_png(d["b64_json"]) for d in client.post("/v1/images/generations", json=body).json()["data"]]
    assert all(np.array_equal(a, b) for a, b in zip(imgs, again))                                        # reproducible
    other = _decode_png(client.post("/v1/images/generations", json={**body, "n": 1, "seed": 8}).json()["data"][0]["b64_json"])
    assert np.array_equal(other, imgs[1])                                                                # image i uses seed + i
    assert client.post("/v1/images/generations", json={"prompt": ""}).status_code == 400
    assert client.post("/v1/images/generations", json={"prompt": "x", "n": 99}).status_code == 400
    assert client.post("/v1/images/generations", json={"prompt": "x", "response_format": "url"}).status_code == 400


def test_a1111_route_maps_steps_and_cfg(client):
    base = {"prompt": "fox", "negative_prompt": "blurry", "seed": 11, "steps": 4, "cfg_scale": 7.5}
    a = client.post("/sdapi/v1/txt2img", json=base).json()
    assert a["parameters"]["seed"] == 11 and json.loads(a["info"])["all_seeds"] == [11]
    img = _decode_png(a["images"][0])
    fewer = _decode_png(client.post("/sdapi/v1/txt2img", json={**base, "steps": 2}).json()["images"][0])
    weaker = _decode_png(client.post("/sdapi/v1/txt2img", json={**base, "cfg_scale": 1.0}).json()["images"][0])
    assert not np.array_equal(img, fewer) and not np.array_equal(img, weaker)
    pipe = client.app.state.pipeline
    assert pipe.session.stats["iterations"] >= 4 + 2 + 4 and pipe.generated >= 3
    assert client.post("/sdapi/v1/txt2img", json={**base, "batch_size": 20}).status_code == 400


def test_text_server_mounts_the_image_routes_next_to_chat(tmp_path):
    import torch

    from onnx_genai_b200.engine.api import Engine
    from onnx_genai_b200.models.config import DecoderConfig
    from onnx_genai_b200.models.decoder import random_weights
    from onnx_genai_b200.package.export import export_package
    from onnx_genai_b200.server.app import create_app
    from onnx_genai_b200.server.images import ImagePipeline

    cfg = DecoderConfig(name="t", num_layers=1, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96, vocab=300,
                        rope_theta=1e4, tie_embeddings=True, max_position=256)
    d = export_package(cfg, random_weights(cfg, "cpu", seed=5, std=0.3, dtype=torch.float32), str(tmp_path / "pkg"))
    eng = Engine.from_dir(d, device="cpu", num_pages=32, max_seqs=2, max_tokens_per_step=64)
    with TestClient(create_app(eng, model_name="tiny", image_pipeline=ImagePipeline(PKG))) as c:
        assert c.post("/v1/completions", json={"model": "tiny", "prompt": "hi", "max_tokens": 2, "temperature": 0}).status_code == 200
        r = c.post("/v1/images/generations", json={"prompt": "fox", "seed": 1})
        assert r.status_code == 200 and _decode_png(r.json()["data"][0]["b64_json"]).shape == (4, 4, 3)
        r = c.post("/sdapi/v1/img2img", json={"prompt": "fox", "init_images": ["AAAA"]})
        assert r.status_code == 400 and "no image input" in r.text
        assert c.post("/v1/audio/speech").status_code == 501 and c.post("/v1/audio/transcriptions").status_code == 501
        assert c.get("/sdapi/v1/sd-models").json()[0]["model_name"] == "tiny"
    with TestClient(create_app(eng, model_name="tiny")) as c:
        assert c.post("/v1/images/generations").status_code == 501


def test_a1111_front_end_questions(client):
    models = client.get("/sdapi/v1/sd-models").json()
    assert models == [{"title": "sd-tiny", "model_name": "sd-tiny", "hash": None, "sha256": None, "filename": "sd-tiny", "config": None}]
    samplers = client.get("/sdapi/v1/samplers").json()
    assert samplers and set(samplers[0]) == {"name", "aliases", "options"}
    options = client.get("/sdapi/v1/options").json()
    assert options["sd_model_checkpoint"] == "sd-tiny" and options["samples_format"] == "png" and options["sampler_name"] == samplers[0]["name"]
    assert client.post("/sdapi/v1/txt2img", json={"prompt": "fox", "sampler_name": "No Such Sampler"}).status_code == 400
    assert client.post("/sdapi/v1/txt2img", json={"prompt": "fox", "sampler_name": samplers[0]["name"], "seed": 3}).status_code == 200


def test_img2img_request_handling_over_a_stand_in_pipeline():
    """The HTTP layer of image-to-image: one base64 image (data URLs accepted) reaches the pipeline decoded, with the
    strength checked; what the pipeline returns comes back as PNGs."""
    from fastapi import FastAPI

    from onnx_genai_b200.server.images import add_image_routes
    from onnx_genai_b200.utils.png import encode_png

    class StandIn:
        samplers = ["Euler"]
        init_in = "init_image"

        def __init__(self):
            self.calls = []

        def generate(self, **kw):
            self.calls.append(kw)
            img = kw["init_image"] / 255.0
            return [img * (1.0 - kw["strength"])] * kw["n"]

    pipe = StandIn()
    app = FastAPI()
    add_image_routes(app, pipe, "stand-in")
    src = np.zeros((3, 2, 2), dtype=np.float32)
    src[0] = 1.0                                                                    # a red 2x2 image
    b64 = base64.b64encode(encode_png(src)).decode()
    with TestClient(app) as c:
        r = c.post("/sdapi/v1/img2img", json={"prompt": "fox", "init_images": ["data:image/png;base64," + b64], "denoising_strength": 0.5,
                                              "batch_size": 2, "seed": 9})
        assert r.status_code == 200, r.text
        body = r.json()
        assert len(body["images"]) == 2 and body["parameters"]["denoising_strength"] == 0.5 and body["parameters"]["seed"] == 9
        px = _decode_png(body["images"][0])
        assert px.shape == (2, 2, 3) and abs(int(px[0, 0, 0]) - 128) <= 1 and px[0, 0, 1] == 0
        call = pipe.calls[0]
        assert call["init_image"].shape == (3, 2, 2) and call["init_image"][0, 0, 0] == 255.0 and call["n"] == 2 and call["seed"] == 9
        for bad in ({"init_images": []}, {"init_images": [b64, b64]}, {"init_images": ["@@not base64@@"]},
                    {"init_images": [base64.b64encode(b"not an image").decode()]}, {"init_images": [b64], "denoising_strength": 1.5}):
            assert c.post("/sdapi/v1/img2img", json={"prompt": "fox", **bad}).status_code == 400, bad
