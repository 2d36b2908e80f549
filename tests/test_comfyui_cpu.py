"""ComfyUI API-format graph -> workflow metadata document."""
import copy
import json

import pytest
import yaml

from onnx_genai_b200.metadata import workflow as wfm
from onnx_genai_b200.package.comfyui import ComfyImportError, import_comfyui

GRAPH = {
    "3": {"class_type": "KSampler", "inputs": {"seed": 5, "steps": 20, "cfg": 8, "sampler_name": "euler", "scheduler": "karras", "denoise": 1,
                                                "model": ["4", 0], "positive": ["6", 0], "negative": ["7", 0], "latent_image": ["5", 0]}},
    "4": {"class_type": "CheckpointLoaderSimple", "inputs": {"ckpt_name": "models/sd15.safetensors"}},
    "5": {"class_type": "EmptyLatentImage", "inputs": {"width": 768, "height": 512, "batch_size": 2}},
    "6": {"class_type": "CLIPTextEncode", "inputs": {"text": "a cat", "clip": ["4", 1]}},
    "7": {"class_type": "CLIPTextEncode", "inputs": {"text": "blurry", "clip": ["4", 1]}},
    "8": {"class_type": "VAEDecode", "inputs": {"samples": ["3", 0], "vae": ["4", 2]}},
    "9": {"class_type": "SaveImage", "inputs": {"images": ["8", 0], "filename_prefix": "out"}},
}


def test_guided_graph_validates_and_carries_parameters():
    doc = import_comfyui(GRAPH)
    wf = wfm.parse(doc["pipeline"]["workflow"])
    assert wfm.validate(wf) == []
    assert {"text_encoder", "denoiser", "vae_decoder", "solver_step", "guidance", "schedule"} <= set(wf.components)
    assert wf.components["denoiser"].artifact == "sd15/unet.onnx"
    assert wf.components["solver_step"].artifact == "policies/solver_euler.onnx"
    assert wf.components["schedule"].artifact == "policies/schedule_karras.onnx"
    d = doc["generation"]["defaults"]
    assert (d["steps"], d["guidance_scale"], d["seed"], d["width"], d["height"], d["batch_size"]) == (20, 8.0, 5, 768, 512, 2)
    assert d["positive_prompt"] == "a cat" and d["negative_prompt"] == "blurry" and d["filename_prefix"] == "out"
    w = doc["pipeline"]["workflow"]
    assert w["inputs"]["request.noise"]["contract"]["shape"] == ["batch", 4, 64, 96]
    assert w["outputs"]["image"]["contract"]["shape"] == ["batch", 3, 512, 768]
    assert w["inputs"]["request.max_iterations"]["default"] == 20
    loop = w["steps"][0]
    assert loop["kind"] == "loop" and [s["component"] for s in loop["steps"]] == ["denoiser", "denoiser", "guidance", "solver_step", "continue_predicate"]
    assert yaml.safe_load(yaml.safe_dump(doc)) == doc


def test_cfg_one_drops_the_negative_pass():
    g = copy.deepcopy(GRAPH)
    g["3"]["inputs"]["cfg"] = 1.0
    doc = import_comfyui(g)
    w = doc["pipeline"]["workflow"]
    assert "guidance" not in w["components"] and "request.negative_ids" not in w["inputs"]
    assert [s["component"] for s in w["steps"][0]["steps"]] == ["denoiser", "solver_step", "continue_predicate"]
    assert wfm.validate(wfm.parse(w)) == []


def test_imported_document_is_checked_not_rubber_stamped():
    w = import_comfyui(GRAPH)["pipeline"]["workflow"]
    w["steps"][1]["inputs"]["latent"] = "nowhere.defined"
    assert wfm.validate(wfm.parse(w))


@pytest.mark.parametrize("mutate, needle", [
    (lambda g: g.update({"10": {"class_type": "LoraLoader", "inputs": {}}}), "LoraLoader"),
    (lambda g: g["3"]["inputs"].update(denoise=0.5), "denoise"),
    (lambda g: g["5"]["inputs"].update(width=500), "multiples of 8"),
    (lambda g: g["8"]["inputs"].update(vae=["4", 1]), "output 2"),
    (lambda g: g["3"]["inputs"].update(positive="a cat"), "link"),
    (lambda g: g.pop("9"), "SaveImage"),
    (lambda g: g["6"].pop("class_type"), "class_type"),
])
def test_unsupported_graphs_are_rejected_with_a_reason(mutate, needle):
    g = copy.deepcopy(GRAPH)
    mutate(g)
    with pytest.raises(ComfyImportError, match=needle):
        import_comfyui(g)


def test_cli_round_trip(tmp_path):
    from onnx_genai_b200.cli import main

    src, out = tmp_path / "g.json", tmp_path / "meta.yaml"
    src.write_text(json.dumps(GRAPH))
    assert main(["import-comfyui", str(src), "-o", str(out)]) == 0
    doc = yaml.safe_load(out.read_text())
    assert wfm.validate(wfm.load_document(doc)) == []
