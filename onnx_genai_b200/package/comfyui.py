"""ComfyUI "Save (API Format)" graphs -> the canonical workflow form of the inference metadata.

ComfyUI exports a text-to-image graph as a JSON object of numbered nodes, each with a ``class_type`` and ``inputs``
whose values are literals or ``[node id, output index]`` links.  The reference converts such a graph into a
``pipeline.workflow`` document so its workflow runtime can execute it
(crates/onnx-genai-comfyui-config, README.md:396-415).  This importer does the same for the classic latent-diffusion
graph::

    CheckpointLoaderSimple -> CLIPTextEncode (positive / negative) -> KSampler <- EmptyLatentImage
                                                                        |
                                                                    VAEDecode -> SaveImage | PreviewImage

with its usual variations -- LoRA loaders on the model and CLIP links (recorded with their strengths), ``CLIPSetLastLayer``
(clip skip), separate ``UNETLoader`` / ``CLIPLoader`` / ``VAELoader`` nodes, ``KSamplerAdvanced`` (a window of the schedule),
``VAEDecodeTiled``, 16-channel SD3 latents, and image to image (``LoadImage -> VAEEncode`` as the latent, ``denoise`` < 1) --
and emits a document with one component per model part (``text_encoder``, ``denoiser``, ``vae_decoder``), policy
components for the sampler (``solver_step`` named after ``sampler_name`` / ``scheduler``) and, when ``cfg`` is not 1,
classifier-free guidance (a second denoiser pass on the negative conditioning and a ``guidance`` combine), a
denoising ``loop`` of ``steps`` iterations, the VAE decode and an ``emit`` of the image.  Graph parameters (steps, cfg,
seed, size, sampler) become generation defaults.  Graphs with other node types are rejected with the node id, its
class and the list of supported classes; nothing is guessed.

This build has no diffusion executor: the output is a validated document (see :mod:`onnx_genai_b200.metadata.workflow`)
for tools that consume the standard, not something ``Engine`` can run.
"""
from __future__ import annotations

import os

SUPPORTED = ("CheckpointLoaderSimple", "CheckpointLoader", "UNETLoader", "CLIPLoader", "VAELoader", "LoraLoader", "LoraLoaderModelOnly",
             "CLIPSetLastLayer", "CLIPTextEncode", "EmptyLatentImage", "EmptySD3LatentImage", "LoadImage", "VAEEncode", "KSampler",
             "KSamplerAdvanced", "VAEDecode", "VAEDecodeTiled", "SaveImage", "PreviewImage")


class ComfyImportError(ValueError):
    pass


def _link(value, what, node_id):
    if not (isinstance(value, (list, tuple)) and len(value) == 2 and isinstance(value[1], int)):
        raise ComfyImportError(f"node {node_id}: input '{what}' must be a link [node id, output index], found {value!r}")
    return str(value[0]), int(value[1])


def _contract(dtype, shape):
    return {"dtype": dtype, "rank": len(shape), "shape": list(shape), "batch_layout": {"kind": "request_aligned", "axis": 0}}


def import_comfyui(graph: dict) -> dict:
    """``graph``: the parsed API-format JSON.  Returns an inference-metadata document (a plain dict)."""
    if not isinstance(graph, dict) or not graph:
        raise ComfyImportError("the ComfyUI API export is a JSON object of nodes keyed by id; this is not one")
    nodes = {}
    for nid, node in graph.items():
        if not isinstance(node, dict) or "class_type" not in node:
            raise ComfyImportError(f"node {nid}: every node needs a 'class_type' (is this the API format, not the UI save format?)")
        if node["class_type"] not in SUPPORTED:
            raise ComfyImportError(f"node {nid} is a {node['class_type']!r}; this importer handles {', '.join(SUPPORTED)}")
        nodes[str(nid)] = node

    def of_class(cls):
        return [(nid, n) for nid, n in nodes.items() if n["class_type"] == cls]

    sinks = of_class("SaveImage") + of_class("PreviewImage")
    if len(sinks) != 1:
        raise ComfyImportError(f"expected one SaveImage / PreviewImage node, found {len(sinks)}")
    sink_id, sink = sinks[0]
    dec_id, _ = _link(sink["inputs"].get("images"), "images", sink_id)
    dec = nodes.get(dec_id)
    if dec is None or dec["class_type"] not in ("VAEDecode", "VAEDecodeTiled"):
        raise ComfyImportError(f"node {sink_id}: 'images' must come from a VAEDecode node")
    ks_id, _ = _link(dec["inputs"].get("samples"), "samples", dec_id)
    ks = nodes.get(ks_id)
    if ks is None or ks["class_type"] not in ("KSampler", "KSamplerAdvanced"):
        raise ComfyImportError(f"node {dec_id}: 'samples' must come from a KSampler node")
    ki = ks["inputs"]
    advanced = ks["class_type"] == "KSamplerAdvanced"
    loras: list = []

    def lora_of(nid, n, clip_too):
        e = {"name": str(n["inputs"].get("lora_name", "")), "strength_model": float(n["inputs"].get("strength_model", 1.0))}
        if clip_too:
            e["strength_clip"] = float(n["inputs"].get("strength_clip", 1.0))
        if not e["name"]:
            raise ComfyImportError(f"node {nid}: a LoRA loader needs 'lora_name'")
        if e not in loras:
            loras.append(e)

    def model_source(value, what, from_id):
        """Follow a MODEL link through LoRA loaders back to the loader that owns the denoiser; returns (loader id, node)."""
        nid, out = _link(value, what, from_id)
        for _ in range(64):
            n = nodes.get(nid)
            if n is None:
                raise ComfyImportError(f"node {from_id}: '{what}' points at node {nid}, which does not exist")
            cls = n["class_type"]
            if cls in ("LoraLoader", "LoraLoaderModelOnly") and out == 0:
                lora_of(nid, n, cls == "LoraLoader")
                nid, out = _link(n["inputs"].get("model"), "model", nid)
                continue
            if cls in ("CheckpointLoaderSimple", "CheckpointLoader") and out == 0:
                return nid, n
            if cls == "UNETLoader" and out == 0:
                return nid, n
            raise ComfyImportError(f"node {from_id}: '{what}' must be output 0 of a checkpoint / UNET loader (through LoRA loaders at most); found output {out} of a {cls!r}")
        raise ComfyImportError(f"node {from_id}: the '{what}' chain does not end")

    clip_skip = [0]

    def clip_source(value, from_id):
        """Follow a CLIP link through CLIPSetLastLayer and LoRA loaders to its loader."""
        nid, out = _link(value, "clip", from_id)
        for _ in range(64):
            n = nodes.get(nid)
            if n is None:
                raise ComfyImportError(f"node {from_id}: 'clip' points at node {nid}, which does not exist")
            cls = n["class_type"]
            if cls == "CLIPSetLastLayer":
                clip_skip[0] = -int(n["inputs"].get("stop_at_clip_layer", -1)) - 1        # -1 = the last layer = skip 0
                nid, out = _link(n["inputs"].get("clip"), "clip", nid)
                continue
            if cls == "LoraLoader" and out == 1:
                lora_of(nid, n, True)
                nid, out = _link(n["inputs"].get("clip"), "clip", nid)
                continue
            if cls in ("CheckpointLoaderSimple", "CheckpointLoader") and out == 1:
                return nid, n
            if cls == "CLIPLoader" and out == 0:
                return nid, n
            raise ComfyImportError(f"node {from_id}: 'clip' must be output 1 of the checkpoint loader (node of class {cls!r}, output {out} found)")
        raise ComfyImportError(f"node {from_id}: the 'clip' chain does not end")

    def vae_source(value, from_id):
        nid, out = _link(value, "vae", from_id)
        n = nodes.get(nid)
        if n is not None and n["class_type"] in ("CheckpointLoaderSimple", "CheckpointLoader") and out == 2:
            return nid, n
        if n is not None and n["class_type"] == "VAELoader" and out == 0:
            return nid, n
        raise ComfyImportError(f"node {from_id}: 'vae' must be output 2 of the checkpoint loader or a VAELoader")

    ckpt_id, ckpt = model_source(ki.get("model"), "model", ks_id)
    vae_id, vae_node = vae_source(dec["inputs"].get("vae"), dec_id)
    cond = {}
    clip_node = None
    for side in ("positive", "negative"):
        cid, _ = _link(ki.get(side), side, ks_id)
        c = nodes.get(cid)
        if c is None or c["class_type"] != "CLIPTextEncode":
            raise ComfyImportError(f"node {ks_id}: '{side}' must come from a CLIPTextEncode node")
        _, clip_node = clip_source(c["inputs"].get("clip"), cid)
        cond[side] = str(c["inputs"].get("text", ""))
    lat_id, _ = _link(ki.get("latent_image"), "latent_image", ks_id)
    lat = nodes.get(lat_id)
    source_image = None
    if lat is not None and lat["class_type"] == "VAEEncode":
        # image to image: LoadImage -> VAEEncode -> sampler; the size comes with the request's image
        px_id, _ = _link(lat["inputs"].get("pixels"), "pixels", lat_id)
        px = nodes.get(px_id)
        if px is None or px["class_type"] != "LoadImage":
            raise ComfyImportError(f"node {lat_id}: 'pixels' must come from a LoadImage node")
        vae_source(lat["inputs"].get("vae"), lat_id)
        source_image = str(px["inputs"].get("image", ""))
        width = height = 0
        batch = 1
        latent_channels = 4
    elif lat is not None and lat["class_type"] in ("EmptyLatentImage", "EmptySD3LatentImage"):
        width, height = int(lat["inputs"].get("width", 512)), int(lat["inputs"].get("height", 512))
        batch = int(lat["inputs"].get("batch_size", 1))
        latent_channels = 16 if lat["class_type"] == "EmptySD3LatentImage" else 4
        if width % 8 or height % 8:
            raise ComfyImportError(f"node {lat_id}: width and height must be multiples of 8 (the VAE's stride), got {width}x{height}")
    else:
        raise ComfyImportError(f"node {ks_id}: 'latent_image' must come from an EmptyLatentImage node, or from VAEEncode of a LoadImage (image to image)")
    steps, cfg = int(ki.get("steps", 20)), float(ki.get("cfg", 7.0))
    denoise = float(ki.get("denoise", 1.0))
    start_step, end_step, add_noise = 0, steps, True
    if advanced:
        start_step = int(ki.get("start_at_step", 0))
        end_step = min(int(ki.get("end_at_step", steps)), steps)
        add_noise = str(ki.get("add_noise", "enable")) == "enable"
        if not 0 <= start_step < end_step:
            raise ComfyImportError(f"node {ks_id}: start_at_step={start_step} / end_at_step={end_step} leave no step to run out of {steps}")
        if str(ki.get("return_with_leftover_noise", "disable")) == "enable":
            raise ComfyImportError(f"node {ks_id}: return_with_leftover_noise=enable (a sampler that hands a noisy latent on) is not handled")
    elif not 0.0 < denoise <= 1.0:
        raise ComfyImportError(f"node {ks_id}: denoise={denoise} must lie in (0, 1]")
    elif denoise < 1.0:
        if source_image is None:
            raise ComfyImportError(f"node {ks_id}: denoise={denoise} (partial denoising) needs an image to start from (VAEEncode of a LoadImage)")
        start_step = steps - max(1, int(round(steps * denoise)))     # the last round(steps * denoise) steps of the schedule run
    iterations = end_step - start_step
    sampler, scheduler = str(ki.get("sampler_name", "euler")), str(ki.get("scheduler", "normal"))
    guided = cfg != 1.0
    stem = os.path.splitext(os.path.basename(str(ckpt["inputs"].get("ckpt_name") or ckpt["inputs"].get("unet_name") or "checkpoint")))[0]
    lat_h, lat_w = (height // 8, width // 8) if source_image is None else ("latent_height", "latent_width")
    img_h, img_w = (height, width) if source_image is None else ("height", "width")

    def onnx(part):
        return {"implementation": {"kind": "onnx", "artifact": f"{stem}/{part}.onnx"}}

    inputs = {
        "request.positive_ids": {"contract": _contract("int64", ["batch", "sequence"]), "source": {"kind": "request"}, "required": True,
                                 "role": {"kind": "runtime", "version": "1.0", "role": "prompt_tokens"}},
        "request.noise": {"contract": _contract("float32", ["batch", latent_channels, lat_h, lat_w]), "source": {"kind": "application", "name": "noise"},
                          "required": True, "role": {"kind": "opaque"}},
        "request.max_iterations": {"contract": {"dtype": "int64", "rank": 1, "shape": [1]}, "source": {"kind": "request"}, "required": False,
                                   "default": iterations, "role": {"kind": "runtime", "version": "1.0", "role": "max_output_tokens"}},
        "package.false": {"contract": {"dtype": "bool", "rank": 1, "shape": [1]}, "source": {"kind": "literal"}, "default": False,
                          "role": {"kind": "opaque"}},
        "package.loop_active": {"contract": {"dtype": "bool", "rank": 1, "shape": [1]}, "source": {"kind": "literal"}, "default": True,
                                "role": {"kind": "opaque"}},
    }
    components = {"text_encoder": onnx("text_encoder"), "denoiser": onnx("unet"), "vae_decoder": onnx("vae_decoder"),
                  "schedule": {"implementation": {"kind": "onnx", "artifact": f"policies/schedule_{scheduler}.onnx"}},
                  "solver_step": {"implementation": {"kind": "onnx", "artifact": f"policies/solver_{sampler}.onnx"}},
                  "continue_predicate": {"implementation": {"kind": "onnx", "artifact": "policies/continue.onnx"}}}
    schedule_inputs = {}
    if start_step or end_step != steps:
        # a window of the schedule: the policy lays out `steps` noise levels and hands back those in [start, end)
        for name, val in (("start_step", start_step), ("end_step", end_step)):
            inputs[f"package.{name}"] = {"contract": {"dtype": "int64", "rank": 1, "shape": [1]}, "source": {"kind": "literal"}, "default": val,
                                         "role": {"kind": "opaque"}}
            schedule_inputs[name] = f"package.{name}"
    setup = [{"kind": "invoke", "component": "schedule", "inputs": schedule_inputs, "outputs": {"schedule": "diffusion.schedule"}},
             {"kind": "invoke", "component": "text_encoder", "inputs": {"input_ids": "request.positive_ids"},
              "outputs": {"encoder_hidden_states": "conditioning.positive"}}]
    body = [{"kind": "invoke", "component": "denoiser",
             "inputs": {"sample": "latent_state", "step": "loop.iteration", "schedule": "diffusion.schedule",
                        "encoder_hidden_states": "conditioning.positive"}, "outputs": {"noise_pred": "denoiser.positive"}}]
    estimate = "denoiser.positive"
    if guided:
        inputs["request.negative_ids"] = {"contract": _contract("int64", ["batch", "sequence"]), "source": {"kind": "request"}, "required": True,
                                          "role": {"kind": "runtime", "version": "1.0", "role": "negative_prompt_tokens"}}
        inputs["package.guidance_scale"] = {"contract": {"dtype": "float32", "rank": 1, "shape": [1]}, "source": {"kind": "literal"},
                                            "default": cfg, "role": {"kind": "opaque"}}
        components["guidance"] = {"implementation": {"kind": "onnx", "artifact": "policies/classifier_free_guidance.onnx"}}
        setup.append({"kind": "invoke", "component": "text_encoder", "inputs": {"input_ids": "request.negative_ids"},
                      "outputs": {"encoder_hidden_states": "conditioning.negative"}})
        body.append({"kind": "invoke", "component": "denoiser",
                     "inputs": {"sample": "latent_state", "step": "loop.iteration", "schedule": "diffusion.schedule",
                                "encoder_hidden_states": "conditioning.negative"}, "outputs": {"noise_pred": "denoiser.negative"}})
        body.append({"kind": "invoke", "component": "guidance",
                     "inputs": {"conditional": "denoiser.positive", "unconditional": "denoiser.negative", "scale": "package.guidance_scale"},
                     "outputs": {"guided": "denoiser.guided"}})
        estimate = "denoiser.guided"
    body += [{"kind": "invoke", "component": "solver_step",
              "inputs": {"sample": "latent_state", "step": "loop.iteration", "schedule": "diffusion.schedule", "derivative": estimate},
              "outputs": {"next_state": "latent.body"}},
             {"kind": "invoke", "component": "continue_predicate", "inputs": {"done": "package.false"}, "outputs": {"continue": "loop.continue"}}]
    latent_contract = _contract("float32", ["batch", latent_channels, lat_h, lat_w])
    pre, start_value = [], "request.noise"
    if source_image is not None:
        # image to image: the request's image is encoded and noised up to the first level of the schedule window
        inputs["request.image"] = {"contract": _contract("float32", ["batch", 3, img_h, img_w]), "source": {"kind": "application", "name": "image"},
                                   "required": True, "role": {"kind": "opaque"}}
        components["vae_encoder"] = onnx("vae_encoder")
        setup.append({"kind": "invoke", "component": "vae_encoder", "inputs": {"image": "request.image"}, "outputs": {"latent": "latent.encoded"}})
        start_value = "latent.encoded"
        if add_noise:
            components["add_noise"] = {"implementation": {"kind": "onnx", "artifact": "policies/add_noise.onnx"}}
            setup.append({"kind": "invoke", "component": "add_noise",
                          "inputs": {"latent": "latent.encoded", "noise": "request.noise", "schedule": "diffusion.schedule"},
                          "outputs": {"noised": "latent.start"}})
            start_value = "latent.start"
    workflow = {
        "manifest": {"capabilities": ["workflow_ssa", "typed_emit", "loop_induction_values"]},
        "inputs": inputs,
        "outputs": {"image": {"contract": _contract("float32", ["batch", 3, img_h, img_w]), "role": "image", "stage": "post_adapter"}},
        "components": components,
        "state": {"latent_state": {"contract": latent_contract, "scope": "invocation", "initializer": "request.noise",
                                   "recurrence": {"kind": "invariant"}},
                  "loop_active": {"contract": {"dtype": "bool", "rank": 1, "shape": [1]}, "scope": "invocation", "initializer": "package.loop_active",
                                  "recurrence": {"kind": "invariant"}}},
        "steps": [
            {"kind": "loop", "setup": setup, "steps": body, "continue_when": "loop_active", "max_iterations": "request.max_iterations",
             "carried": [{"cell": "latent_state", "initial": start_value, "next": "latent.body"},
                         {"cell": "loop_active", "next": "loop.continue"}],
             "iteration": {"value": "loop.iteration", "contract": {"dtype": "int64", "rank": 1, "shape": [1]}}},
            {"kind": "invoke", "component": "vae_decoder", "inputs": {"latent": "latent_state"}, "outputs": {"image": "vae.image"}},
            {"kind": "emit", "value": "vae.image", "output": "image", "mode": "replace"},
        ],
    }
    prefix = str(sink["inputs"].get("filename_prefix", "")) if sink["class_type"] == "SaveImage" else ""
    return {
        "schema_version": "1.0",
        "pipeline": {"workflow": workflow},
        "generation": {"defaults": {"steps": steps, "guidance_scale": cfg, "seed": int(ki.get("seed", 0)), "sampler": sampler,
                                    "scheduler": scheduler, "width": width, "height": height, "batch_size": batch,
                                    "positive_prompt": cond["positive"], "negative_prompt": cond["negative"],
                                    **({"filename_prefix": prefix} if prefix else {}),
                                    **({"loras": loras} if loras else {}),
                                    **({"clip_skip": clip_skip[0]} if clip_skip[0] else {}),
                                    **({"source_image": source_image, "denoise": denoise} if source_image is not None else {}),
                                    **({"start_at_step": start_step, "end_at_step": end_step, "add_noise": add_noise} if advanced else {}),
                                    **({"vae_name": str(vae_node["inputs"].get("vae_name", ""))} if vae_node["class_type"] == "VAELoader" else {}),
                                    **({"clip_name": str(clip_node["inputs"].get("clip_name", ""))} if clip_node["class_type"] == "CLIPLoader" else {}),
                                    **({"latent_channels": latent_channels} if latent_channels != 4 else {})}},
    }


def main(argv=None) -> int:
    import argparse
    import json
    import sys

    import yaml

    ap = argparse.ArgumentParser(description="Convert a ComfyUI API-format export into an inference-metadata workflow document")
    ap.add_argument("graph", help="ComfyUI 'Save (API Format)' JSON file")
    ap.add_argument("-o", "--out", default="-", help="output YAML (default: stdout)")
    args = ap.parse_args(argv)
    with open(args.graph, encoding="utf-8") as f:
        doc = import_comfyui(json.load(f))
    text = yaml.safe_dump(doc, sort_keys=False)
    if args.out == "-":
        sys.stdout.write(text)
    else:
        with open(args.out, "w", encoding="utf-8") as f:
            f.write(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
