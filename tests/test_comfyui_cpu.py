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
    (lambda g: g.update({"10": {"class_type": "ControlNetApply", "inputs": {}}}), "ControlNetApply"),
    (lambda g: g["3"]["inputs"].update(denoise=0.5), "needs an image to start from"),
    (lambda g: g["3"]["inputs"].update(model=["6", 0]), "checkpoint / UNET loader"),
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


def test_lora_chain_clip_skip_and_separate_loaders_are_followed():
    g = copy.deepcopy(GRAPH)
    g["10"] = {"class_type": "LoraLoader", "inputs": {"lora_name": "style.safetensors", "strength_model": 0.8, "strength_clip": 0.6,
                                                      "model": ["4", 0], "clip": ["4", 1]}}
    g["11"] = {"class_type": "LoraLoaderModelOnly", "inputs": {"lora_name": "detail.safetensors", "strength_model": 0.5, "model": ["10", 0]}}
    g["12"] = {"class_type": "CLIPSetLastLayer", "inputs": {"stop_at_clip_layer": -2, "clip": ["10", 1]}}
    g["13"] = {"class_type": "VAELoader", "inputs": {"vae_name": "vae-ft-mse.safetensors"}}
    g["3"]["inputs"]["model"] = ["11", 0]
    g["6"]["inputs"]["clip"] = ["12", 0]
    g["7"]["inputs"]["clip"] = ["12", 0]
    g["8"] = {"class_type": "VAEDecodeTiled", "inputs": {"samples": ["3", 0], "vae": ["13", 0], "tile_size": 512}}
    doc = import_comfyui(g)
    d = doc["generation"]["defaults"]
    assert d["loras"] == [{"name": "detail.safetensors", "strength_model": 0.5},
                          {"name": "style.safetensors", "strength_model": 0.8, "strength_clip": 0.6}]
    assert d["clip_skip"] == 1 and d["vae_name"] == "vae-ft-mse.safetensors"
    assert wfm.validate(wfm.parse(doc["pipeline"]["workflow"])) == []
    assert doc["pipeline"]["workflow"]["components"]["denoiser"]["implementation"]["artifact"] == "sd15/unet.onnx"


def test_image_to_image_encodes_noises_and_runs_the_tail_of_the_schedule():
    g = copy.deepcopy(GRAPH)
    g["5"] = {"class_type": "VAEEncode", "inputs": {"pixels": ["14", 0], "vae": ["4", 2]}}
    g["14"] = {"class_type": "LoadImage", "inputs": {"image": "photo.png"}}
    g["3"]["inputs"]["denoise"] = 0.6
    doc = import_comfyui(g)
    w = doc["pipeline"]["workflow"]
    assert wfm.validate(wfm.parse(w)) == []
    assert {"vae_encoder", "add_noise"} <= set(w["components"])
    assert w["inputs"]["request.image"]["contract"]["shape"] == ["batch", 3, "height", "width"]
    assert w["inputs"]["request.noise"]["contract"]["shape"] == ["batch", 4, "latent_height", "latent_width"]
    assert w["inputs"]["package.start_step"]["default"] == 8 and w["inputs"]["package.end_step"]["default"] == 20      # 20 - round(20 * 0.6)
    assert w["inputs"]["request.max_iterations"]["default"] == 12
    loop = w["steps"][0]
    assert [s["component"] for s in loop["setup"]] == ["schedule", "text_encoder", "text_encoder", "vae_encoder", "add_noise"]
    assert loop["setup"][0]["inputs"] == {"start_step": "package.start_step", "end_step": "package.end_step"}
    assert loop["carried"][0]["initial"] == "latent.start"
    d = doc["generation"]["defaults"]
    assert d["source_image"] == "photo.png" and d["denoise"] == 0.6


def test_advanced_sampler_window_and_sd3_latents():
    g = copy.deepcopy(GRAPH)
    g["3"] = {"class_type": "KSamplerAdvanced", "inputs": {"noise_seed": 9, "steps": 30, "cfg": 5, "sampler_name": "dpmpp_2m", "scheduler": "normal",
                                                            "add_noise": "enable", "start_at_step": 0, "end_at_step": 24,
                                                            "return_with_leftover_noise": "disable",
                                                            "model": ["4", 0], "positive": ["6", 0], "negative": ["7", 0], "latent_image": ["5", 0]}}
    g["5"] = {"class_type": "EmptySD3LatentImage", "inputs": {"width": 1024, "height": 1024, "batch_size": 1}}
    doc = import_comfyui(g)
    w = doc["pipeline"]["workflow"]
    assert wfm.validate(wfm.parse(w)) == []
    assert w["inputs"]["request.noise"]["contract"]["shape"] == ["batch", 16, 128, 128]
    assert w["inputs"]["request.max_iterations"]["default"] == 24 and w["inputs"]["package.end_step"]["default"] == 24
    d = doc["generation"]["defaults"]
    assert (d["start_at_step"], d["end_at_step"], d["add_noise"], d["latent_channels"]) == (0, 24, True, 16)
    g["3"]["inputs"]["return_with_leftover_noise"] = "enable"
    with pytest.raises(ComfyImportError, match="leftover"):
        import_comfyui(g)
    g["3"]["inputs"].update(return_with_leftover_noise="disable", start_at_step=24, end_at_step=24)
    with pytest.raises(ComfyImportError, match="no step to run"):
        import_comfyui(g)


def test_cli_round_trip(tmp_path):
    from onnx_genai_b200.cli import main

    src, out = tmp_path / "g.json", tmp_path / "meta.yaml"
    src.write_text(json.dumps(GRAPH))
    assert main(["import-comfyui", str(src), "-o", str(out)]) == 0
    doc = yaml.safe_load(out.read_text())
    assert wfm.validate(wfm.load_document(doc)) == []
